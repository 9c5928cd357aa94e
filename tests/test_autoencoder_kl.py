"""The 2-D KL autoencoder (FLUX / SD3 / Z-Image checkpoints): structure, names, tiling."""
import torch

from vllm_omni_b200.diffusion.models.vae import build_vae
from vllm_omni_b200.diffusion.models.vae.autoencoder_kl import AutoencoderKL, AutoencoderKLConfig

SMALL = AutoencoderKLConfig(block_out_channels=(8, 16, 16), layers_per_block=1, norm_num_groups=4, latent_channels=4,
                            scaling_factor=0.5, shift_factor=0.1)


def test_full_size_parameter_counts_and_names():
    """The published checkpoints have 83,653,863 (4 latent channels, with quant convs) and 83,819,683
    (16 channels, FLUX) parameters; the counts pin every layer's shape."""
    with torch.device("meta"):
        sd = AutoencoderKL(AutoencoderKLConfig(latent_channels=4, use_quant_conv=True, use_post_quant_conv=True), with_encoder=True)
        fl = AutoencoderKL(AutoencoderKLConfig(), with_encoder=True)
    assert sum(p.numel() for p in sd.parameters()) == 83_653_863
    assert sum(p.numel() for p in fl.parameters()) == 83_819_683
    names = set(dict(fl.named_parameters()))
    for k in ("decoder.conv_in.weight", "decoder.mid_block.resnets.1.norm2.bias", "decoder.mid_block.attentions.0.to_q.weight",
              "decoder.mid_block.attentions.0.to_out.0.bias", "decoder.mid_block.attentions.0.group_norm.weight",
              "decoder.up_blocks.0.resnets.2.conv2.weight", "decoder.up_blocks.2.resnets.0.conv_shortcut.weight",
              "decoder.up_blocks.2.upsamplers.0.conv.bias", "decoder.conv_norm_out.weight", "decoder.conv_out.bias",
              "encoder.down_blocks.0.downsamplers.0.conv.weight", "encoder.down_blocks.1.resnets.0.conv_shortcut.weight",
              "encoder.conv_out.weight"):
        assert k in names, k
    assert "decoder.up_blocks.3.upsamplers.0.conv.weight" not in names       # the last block does not up-sample


def test_decode_encode_shapes_and_latent_scaling():
    torch.manual_seed(0)
    vae = AutoencoderKL(SMALL, with_encoder=True).float()
    z = torch.randn(2, 4, 6, 5)
    img = vae.decode(z)
    assert img.shape == (2, 3, 24, 20) and img.abs().max() <= 1
    assert torch.allclose(vae.decode(z[:, :, None]), img)                    # [B, C, 1, h, w] accepted
    raw = vae.decode((z / 0.5) + 0.1, denormalize=False)
    assert torch.allclose(raw, img, atol=1e-6)
    lat = vae.encode(img)
    assert lat.shape == z.shape
    assert torch.allclose(vae.normalize(vae.denormalize(z)), z, atol=1e-6)


def test_tiled_decode_close_to_plain_decode():
    torch.manual_seed(1)
    vae = AutoencoderKL(SMALL).float()
    z = torch.randn(1, 4, 40, 24)
    plain = vae.decode(z)
    vae.use_tiling, vae.tile_latent, vae.tile_overlap = True, 24, 8
    tiled = vae.decode(z)
    assert tiled.shape == plain.shape
    # group-norm statistics and the mid-block attention see one tile instead of the whole image, so the
    # two decodes agree only approximately; the seams are cross-faded
    assert (tiled - plain).abs().mean().item() < 0.05
    vae.tile_latent = 64                                            # one tile covers everything: identical
    assert torch.equal(vae.decode(z), plain)


def test_load_weights_accepts_old_attention_names_and_build_vae_picks_class():
    torch.manual_seed(2)
    a, b = AutoencoderKL(SMALL).float(), AutoencoderKL(SMALL).float()
    sd = {}
    for k, v in a.state_dict().items():
        for new, old in (("to_q", "query"), ("to_k", "key"), ("to_v", "value"), ("to_out.0", "proj_attn")):
            k = k.replace(f".attentions.0.{new}.", f".attentions.0.{old}.")
        sd[k] = v[..., None, None] if ("attentions" in k and k.endswith("weight") and "group_norm" not in k) else v
    assert b.load_weights(sd.items()) == set(sd)
    z = torch.randn(1, 4, 4, 4)
    assert torch.equal(a.decode(z), b.decode(z))
    assert type(build_vae({"_class_name": "AutoencoderKL", "latent_channels": 4, "block_out_channels": [8, 8],
                           "norm_num_groups": 4}, "qwen")).__name__ == "AutoencoderKL"
    assert type(build_vae(None, "qwen")).__name__ == "AutoencoderKLQwenImage2d"


def test_channels_last_video_decoder_equals_the_module_for_every_chunking():
    """The causal 3-D decoder restated on the channels-last ops (temporal taps as accumulated 2-D convolutions,
    frame caches per convolution) against the PyTorch module, on the ops' CPU paths in fp32."""
    import torch
    from vllm_omni_b200.diffusion.models.vae.autoencoder_kl_qwenimage import QwenImageVAEConfig
    from vllm_omni_b200.diffusion.models.vae.autoencoder_kl_wan import AutoencoderKLWan
    from vllm_omni_b200.diffusion.models.vae.nhwc_video_decoder import NHWCVideoDecoder
    torch.manual_seed(0)
    cfg = QwenImageVAEConfig(base_dim=8, num_res_blocks=1)
    vae = AutoencoderKLWan(cfg).float()
    for p in vae.parameters():
        if p.dim() > 1:
            p.data.normal_(0, (1.0 / p[0].numel()) ** 0.5)
        else:
            p.data.uniform_(0.5, 1.5)
    z = torch.randn(2, cfg.z_dim, 3, 6, 8)
    ref = vae.decode(z, chunk_frames=1)
    dec = NHWCVideoDecoder(vae.decoder, vae.post_quant_conv, torch.float32)
    for chunk in (1, 0, 2):
        out = dec(vae.denormalize(z.float()), chunk_frames=chunk)
        assert out.shape == ref.shape == (2, 3, 9, 48, 64)
        assert (out - ref).abs().max().item() < 1e-4, chunk


def test_channels_last_kl_decoder_equals_the_module():
    """The GroupNorm decoder restated on the channels-last ops (CPU paths, fp32), incl. the post-quant convolution
    and the attention projections as 1x1 convolutions."""
    import torch
    from vllm_omni_b200.diffusion.models.vae.autoencoder_kl import AutoencoderKL, AutoencoderKLConfig
    from vllm_omni_b200.diffusion.models.vae.nhwc_decoder_kl import NHWCDecoderKL
    torch.manual_seed(0)
    cfg = AutoencoderKLConfig(block_out_channels=(32, 64, 64, 64), layers_per_block=1, norm_num_groups=8, use_post_quant_conv=True)
    vae = AutoencoderKL(cfg).float()
    for p in vae.parameters():
        if p.dim() > 1:
            p.data.normal_(0, (1.0 / p[0].numel()) ** 0.5)
        else:
            p.data.uniform_(0.5, 1.5)
    z = torch.randn(2, 16, 6, 10)
    ref = vae.decode(z)
    assert NHWCDecoderKL.supported(vae.decoder)
    out = NHWCDecoderKL(vae.decoder, vae.post_quant_conv, torch.float32)(vae.denormalize(z))
    assert out.shape == ref.shape and (out - ref).abs().max().item() < 1e-4
    odd = AutoencoderKL(AutoencoderKLConfig(block_out_channels=(24, 48, 48, 48), layers_per_block=1, norm_num_groups=4))
    assert not NHWCDecoderKL.supported(odd.decoder)          # 24 channels: the native GroupNorm does not take them
