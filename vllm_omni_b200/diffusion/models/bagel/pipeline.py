"""BAGEL image generation (vllm_omni/diffusion/models/bagel/pipeline_bagel.py:153-724): the
mixture-of-transformers language model denoises 2x2-patched VAE latents by flow matching while
attending to the key/value cache of the prompt.

Two ways to get that context.  (a) The upstream AR stage prefills the prompt and hands its KV cache
over through the KV transfer manager (``sampling_params.past_key_values``); then, as in the reference,
classifier-free guidance is off.  (b) No cache arrives: this stage tokenizes
``<|im_start|> prompt <|im_end|>`` itself, prefills it in understanding mode, prefills the negative
prompt as the text-CFG context, and samples with text guidance ``v = v_neg + s (v - v_neg)`` inside
the guidance interval, rescaled so that its norm does not exceed the conditional velocity's
(``global`` / ``channel`` / ``text_channel`` renormalisation).

Time grid: ``linspace(1, 0, steps)`` warped by ``shift t / (1 + (shift - 1) t)``, Euler updates
``x -= v dt`` over the first steps - 1 points.  Latent tokens are (h, w) row-major with channel order
(p, q, c); decoding un-patches them and runs the FLUX-layout KL decoder.  Reference images for editing
(VAE + vision-tower context) are not built: an edit request is refused with a clear error.
"""
from __future__ import annotations

import os

import torch
from torch import nn

from ...data import DiffusionOutput, OmniDiffusionConfig
from ..vae import build_vae
from .mot import BagelMoT, BagelMoTConfig


def shifted_time_grid(steps: int, shift: float, device=None) -> torch.Tensor:
    t = torch.linspace(1, 0, steps, device=device)
    return shift * t / (1 + (shift - 1) * t)


def guided_velocity(v, v_text=None, v_img=None, text_scale=1.0, img_scale=1.0, renorm_min=0.0, renorm_type="global"):
    """Text (and image) classifier-free guidance with the norm clamp of the reference."""
    if v_text is None or text_scale <= 1.0:
        return v
    if renorm_type == "text_channel":
        vt = v_text + text_scale * (v - v_text)
        scale = (v.norm(dim=-1, keepdim=True) / (vt.norm(dim=-1, keepdim=True) + 1e-8)).clamp(min=renorm_min, max=1.0)
        vt = vt * scale
        return v_img + img_scale * (vt - v_img) if (v_img is not None and img_scale > 1.0) else vt
    vt = v_text + text_scale * (v - v_text)
    out = v_img + img_scale * (vt - v_img) if (v_img is not None and img_scale > 1.0) else vt
    if renorm_type == "global":
        n0, n1 = v.norm(), out.norm()
    elif renorm_type == "channel":
        n0, n1 = v.norm(dim=-1, keepdim=True), out.norm(dim=-1, keepdim=True)
    else:
        raise NotImplementedError(f"{renorm_type} is not supported")
    return out * (n0 / (n1 + 1e-8)).clamp(min=renorm_min, max=1.0)


class BagelPipeline(nn.Module):
    vae_scale_factor = 8

    def __init__(self, od_config: OmniDiffusionConfig | None = None, transformer_config=None, vae_config=None, device=None, **_):
        super().__init__()
        self.od_config = od_config or OmniDiffusionConfig()
        dtype = self.od_config.dtype
        self.device_ = torch.device(device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
        cfg = transformer_config or BagelMoTConfig.from_dict(self.od_config.tf_model_config.to_dict())
        self.transformer = BagelMoT(cfg, dtype=dtype, device=self.device_)
        vc = dict(vae_config or self.od_config.vae_config or {})
        vc.setdefault("latent_channels", cfg.z_channels)
        self.vae = build_vae(vc, "kl").to(device=self.device_, dtype=dtype)
        self.vae.use_tiling = self.od_config.vae_use_tiling
        self.tokenizer = None
        self.vae_decode = None

    def attach_text_encoder(self, model_path: str) -> bool:
        """The checkpoint's tokenizer, for prompts that this stage prefills itself."""
        if not any(os.path.exists(os.path.join(model_path, f)) for f in ("tokenizer.json", "tokenizer_config.json", "vocab.json")):
            return False
        from transformers import AutoTokenizer
        self.tokenizer = AutoTokenizer.from_pretrained(model_path)
        c = self.transformer.cfg
        for attr, tok in (("bos_token_id", "<|im_start|>"), ("eos_token_id", "<|im_end|>"), ("start_of_image", "<|vision_start|>"),
                          ("end_of_image", "<|vision_end|>")):
            tid = self.tokenizer.convert_tokens_to_ids(tok)
            if isinstance(tid, int) and tid >= 0 and tid != getattr(self.tokenizer, "unk_token_id", None):
                setattr(c, attr, tid)
        return True

    def load_weights(self, weights) -> set:
        tw, vw = [], []
        for n, w in weights:
            m = n[len("vae."):] if n.startswith("vae.") else (n[len("vae_model."):] if n.startswith("vae_model.") else None)
            if m is not None or n.startswith(("encoder.", "decoder.")):
                vw.append((m if m is not None else n, w))
            else:
                tw.append((n[len("transformer."):] if n.startswith("transformer.") else n, w))
        loaded = set(self.transformer.load_weights(tw))
        if vw and hasattr(self.vae, "load_weights"):
            loaded |= {"vae." + n for n in self.vae.load_weights(vw)}
        return loaded

    # ------------------------------------------------------------------ context
    def _prompt_ids(self, text: str) -> torch.Tensor:
        c = self.transformer.cfg
        if self.tokenizer is not None:
            ids = list(self.tokenizer.encode(text, add_special_tokens=False))
        else:                                            # no tokenizer files: bytes of the prompt, a stand-in for tests
            ids = [b % max(1, min(c.vocab_size, 256)) for b in text.encode("utf-8")]
        return torch.tensor([c.bos_token_id] + ids + [c.eos_token_id], dtype=torch.long, device=self.device_)

    def _injected(self, kv):
        """KV handed over by the AR stage -> list of (k, v) [T, Hkv, Dh] per layer."""
        if hasattr(kv, "key_cache"):
            kv = list(zip(kv.key_cache, kv.value_cache))
        L = len(self.transformer.layers)
        out = []
        for li in range(L):
            k, v = kv[li % len(kv)]
            Dh = self.transformer.cfg.head_dim
            out.append((k.to(self.device_).reshape(-1, k.shape[-2], Dh), v.to(self.device_).reshape(-1, v.shape[-2], Dh)))
        return out

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def forward(self, req) -> DiffusionOutput:
        sp = req.sampling_params
        tf = self.transformer
        c = tf.cfg
        extra = sp.extra_args or {}
        first = req.prompts[0]
        if isinstance(first, dict) and (first.get("multi_modal_data") or {}).get("image") is not None and sp.past_key_values is None:
            raise NotImplementedError("BAGEL image editing needs the reference image in the context (VAE + vision-tower "
                                      "prefill); this build generates from text, or from a context handed over as KV")
        prompt = first if isinstance(first, str) else (first.get("prompt") or "")
        max_hw = c.max_latent_size * c.latent_downsample
        H = int(sp.height) if sp.height else max_hw
        W = int(sp.width) if sp.width else max_hw
        if H > max_hw or W > max_hw:
            raise ValueError(f"requested {H}x{W} exceeds the checkpoint's limit {max_hw}x{max_hw}")
        h, w = H // c.latent_downsample, W // c.latent_downsample
        steps = int(sp.num_inference_steps or 50)
        text_scale = float(extra.get("cfg_text_scale", 4.0))
        interval = tuple(extra.get("cfg_interval", (0.4, 1.0)))
        renorm_min, renorm_type = float(extra.get("cfg_renorm_min", 0.0)), extra.get("cfg_renorm_type", "global")
        neg_ctx, neg_pos = None, 0
        if sp.past_key_values is not None:
            ctx = self._injected(sp.past_key_values)
            pos = int(ctx[0][0].shape[0])
            text_scale = 1.0                                 # guidance is off with an injected context
        else:
            ids = self._prompt_ids(prompt)
            ctx, pos = tf.prefill_text(ids), int(ids.shape[0])
            if text_scale > 1.0:
                neg = first.get("negative_prompt") if isinstance(first, dict) else None
                nids = self._prompt_ids(neg if neg is not None else str(extra.get("negative_prompt", "")))
                neg_ctx, neg_pos = tf.prefill_text(nids), int(nids.shape[0])
        gen = sp.generator or (torch.Generator(device="cpu").manual_seed(int(sp.seed)) if sp.seed is not None else None)
        x = torch.randn(1, h * w, c.patch_latent_dim, generator=gen, device=gen.device if gen is not None else self.device_)
        x = x.to(self.device_, torch.float32)
        ts = shifted_time_grid(steps, float(extra.get("timestep_shift", c.timestep_shift)), self.device_)
        for i in range(steps - 1):
            t = ts[i]
            v = tf.flow(x, t.reshape(1), (h, w), ctx, pos).float()
            if text_scale > 1.0 and interval[0] < float(t) <= interval[1]:
                vn = tf.flow(x, t.reshape(1), (h, w), neg_ctx, neg_pos, branch=1).float()
                v = guided_velocity(v, vn, None, text_scale, 1.0, renorm_min, renorm_type)
            x = x - v * (ts[i] - ts[i + 1])
        p = c.latent_patch_size
        z = torch.einsum("nhwpqc->nchpwq", x.reshape(1, h, w, p, p, c.z_channels)).reshape(1, c.z_channels, h * p, w * p)
        if (sp.output_type or self.od_config.output_type) == "latent":
            return DiffusionOutput(output=z)
        img = (self.vae_decode or self.vae.decode)(z)
        return DiffusionOutput(output=img, metrics={"num_steps": steps - 1})
