"""Stand-in for the few `diffusers` building blocks the reference's Qwen-Image transformer imports.
diffusers is not installable offline here; these classes restate the published layer definitions
(sinusoidal timestep projection, two-layer timestep MLP, continuous AdaLayerNorm) in plain PyTorch so
that the reference's own transformer module runs unmodified."""
__version__ = "0.0.shim"
