"""Fused Qwen-Image-style MMDiT forward vs its straight-line fp32 restatement."""
import pytest
import torch

from vllm_omni_b200.diffusion.models.qwen_image.transformer import (
    QwenImageTransformer2DModel, QwenImageTransformerConfig, reference_forward)


def _tiny(dtype, device, head_dim=32, heads=4, layers=2):
    axes = {32: (8, 12, 12), 128: (16, 56, 56)}[head_dim]
    cfg = QwenImageTransformerConfig(num_layers=layers, attention_head_dim=head_dim, num_attention_heads=heads,
                                     joint_attention_dim=64, in_channels=16, out_channels=4, axes_dims_rope=axes)
    torch.manual_seed(0)
    m = QwenImageTransformer2DModel(cfg, dtype=dtype, device=device)
    for p in m.parameters():
        if p.dim() == 1:
            p.normal_(0, 0.5)
    return m


def test_forward_matches_reference_cpu():
    m = _tiny(torch.float32, "cpu")
    B, h, w, St = 2, 6, 4, 5
    x = torch.randn(B, h * w, 16)
    e = torch.randn(B, St, 64)
    t = torch.tensor([0.7, 0.7])
    y = m(x, e, t, (1, h, w), txt_seq_lens=[5, 3])
    ref = reference_forward(m, x, e, t, (1, h, w), txt_seq_lens=[5, 3])
    assert y.shape == (B, h * w, 16)
    assert torch.allclose(y, ref, atol=2e-4, rtol=1e-3), (y - ref).abs().max()


def test_checkpoint_name_map_roundtrip():
    m = _tiny(torch.float32, "cpu")
    nmap = m.checkpoint_name_map()
    params = dict(m.named_parameters())
    ckpt = {}
    for name, (pn, sl) in nmap.items():
        p = params[pn]
        ckpt[name] = torch.randn_like(p if sl is None else p[sl[0]:sl[1]])
    loaded = m.load_weights(ckpt.items())
    assert loaded == set(ckpt)
    # every parameter element is covered by exactly the checkpoint tensors
    covered = {pn: 0 for pn in params}
    for name, (pn, sl) in nmap.items():
        covered[pn] += ckpt[name].numel()
    for pn, p in params.items():
        assert covered[pn] == p.numel(), pn
    w = ckpt["transformer_blocks.1.attn.add_k_proj.weight"]
    HD = m.cfg.inner_dim
    assert torch.equal(m.blocks[1].txt.to_qkv.weight[HD:2 * HD], w)


@pytest.mark.gpu
def test_forward_matches_reference_gpu():
    dev = torch.device("cuda")
    m = _tiny(torch.bfloat16, dev, head_dim=128, heads=2, layers=2)
    B, h, w, St = 2, 16, 12, 40
    x = torch.randn(B, h * w, 16, device=dev)
    e = torch.randn(B, St, 64, device=dev)
    t = torch.tensor([0.3, 0.3], device=dev)
    y = m(x, e, t, (1, h, w), txt_seq_lens=[40, 17]).float()
    ref = reference_forward(m, x.bfloat16().float(), e.bfloat16().float(), t, (1, h, w), txt_seq_lens=[40, 17])
    err = (y - ref).abs().max().item()
    assert err < 0.08 * max(1.0, ref.abs().max().item()), err


def test_loop_fast_path_matches_forward_cpu():
    m = _tiny(torch.float32, "cpu")
    B, h, w, St = 2, 6, 4, 5
    x = torch.randn(B, h * w, 16)
    e = torch.randn(B, St, 64)
    st = m.prepare_loop(e, [0.9, 0.4], (1, h, w), h * w, txt_seq_lens=[5, 4])
    st.lat_in.copy_(x)
    for i, sig in enumerate([0.9, 0.4]):
        y = m.forward_step(st, i).clone()
        ref = m(x, e, torch.tensor([sig, sig]), (1, h, w), txt_seq_lens=[5, 4])
        assert torch.allclose(y, ref, atol=1e-5, rtol=1e-4), (i, (y - ref).abs().max())


@pytest.mark.gpu
def test_loop_graph_replay_matches_eager_gpu():
    dev = torch.device("cuda")
    m = _tiny(torch.bfloat16, dev, head_dim=128, heads=2, layers=2)
    B, h, w, St = 2, 16, 12, 40
    x = torch.randn(B, h * w, 16, device=dev)
    e = torch.randn(B, St, 64, device=dev)
    sig = [0.9, 0.7, 0.5, 0.3]
    st_e = m.prepare_loop(e, sig, (1, h, w), h * w, txt_seq_lens=[40, 17], use_graph=False)
    st_g = m.prepare_loop(e, sig, (1, h, w), h * w, txt_seq_lens=[40, 17], use_graph=True)
    st_e.lat_in.copy_(x)
    st_g.lat_in.copy_(x)
    for i in range(len(sig)):
        a = m.forward_step(st_e, i).float().clone()
        b = m.forward_step(st_g, i).float().clone()
        assert torch.equal(a, b), (i, (a - b).abs().max().item())
    assert st_g.graph is not None
