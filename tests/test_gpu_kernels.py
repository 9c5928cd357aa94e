"""Numerics of the sm_100a kernels against plain PyTorch fp32 restatements."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda")


def _status_ok(dev):
    from vllm_omni_b200.ops import _native as nv
    torch.cuda.synchronize()
    assert int(nv.status_word(dev).item()) == 0


@pytest.mark.parametrize("bn", [0, 576, 448, 384, 256, 192, 128])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (300, 264, 136), (1024, 3072, 1024)])
def test_gemm_plain(dev, M, N, K, bn):
    from vllm_omni_b200.ops import gemm
    torch.manual_seed(0)
    x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05
    y = gemm.linear(x, w, force_bn=bn).float()
    ref = x.float() @ w.float().t()
    _status_ok(dev)
    assert (y - ref).abs().max().item() <= 0.02 * ref.abs().max().item() + 1e-3


def test_gemm_pair_kernel_many_tiles(dev):
    """CTA-pair kernel over more tiles than CTA pairs (both accumulators and the whole ring wrap),
    ragged M and N, full epilogue."""
    from vllm_omni_b200.ops import gemm
    torch.manual_seed(2)
    B, S, K, N = 2, 2003, 640, 2568
    x = torch.randn(B, S, K, device=dev, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device=dev, dtype=torch.bfloat16)
    res = torch.randn(B, S, N, device=dev, dtype=torch.bfloat16)
    gate = torch.randn(B, N, device=dev, dtype=torch.bfloat16)
    y = gemm.linear(x, w, bias, "gelu_tanh", res, gate, force_bn=gemm.PAIR_BN).float()
    ref = gemm.linear_reference(x, w, bias, "gelu_tanh", res, gate).float()
    _status_ok(dev)
    assert (y - ref).abs().max().item() <= 0.02 * ref.abs().max().item() + 1e-2


@pytest.mark.parametrize("act", [None, "gelu_tanh", "silu"])
def test_gemm_epilogue(dev, act):
    from vllm_omni_b200.ops import gemm
    torch.manual_seed(1)
    B, S, K, N = 2, 520, 512, 768
    x = torch.randn(B, S, K, device=dev, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device=dev, dtype=torch.bfloat16)
    res = torch.randn(B, S, N, device=dev, dtype=torch.bfloat16)
    mod = torch.randn(B, 3 * N, device=dev, dtype=torch.bfloat16)
    gate = mod[:, N:2 * N]
    y = gemm.linear(x, w, bias, act, res, gate).float()
    ref = gemm.linear_reference(x, w, bias, act, res, gate).float()
    _status_ok(dev)
    assert (y - ref).abs().max().item() <= 0.02 * ref.abs().max().item() + 1e-2


def test_gemm_batched_output_rows(dev):
    from vllm_omni_b200.ops import gemm
    torch.manual_seed(2)
    B, S1, S2, K, N = 2, 200, 56, 256, 384
    x = torch.randn(B, S1, K, device=dev, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05
    joint = torch.zeros(B, S1 + S2, N, device=dev, dtype=torch.bfloat16)
    gemm.linear(x, w, out=joint[:, :S1], out_rows_per_batch=S1, out_batch_stride=(S1 + S2) * N)
    ref = (x.float() @ w.float().t())
    _status_ok(dev)
    assert (joint[:, :S1].float() - ref).abs().max().item() < 0.05
    assert joint[:, S1:].abs().max().item() == 0


@pytest.mark.parametrize("B,S,H,Hkv,kvl", [(1, 128, 1, 1, None), (1, 384, 2, 1, None), (2, 600, 4, 4, [600, 333]),
                                           (1, 2100, 3, 3, None)])
def test_attention(dev, B, S, H, Hkv, kvl):
    from vllm_omni_b200.ops import attention as A
    torch.manual_seed(3)
    qkv = torch.randn(B, S, H + 2 * Hkv, 128, device=dev, dtype=torch.bfloat16)
    q, k, v = qkv[:, :, :H], qkv[:, :, H:H + Hkv], qkv[:, :, H + Hkv:]
    kl = torch.tensor(kvl, dtype=torch.int32, device=dev) if kvl else None
    o, lse = A.attention(q, k, v, kv_lens=kl, return_lse=True)
    ref, rl = A.attention_reference(q, k, v, kv_lens=kl, return_lse=True)
    _status_ok(dev)
    assert (o.float() - ref.float()).abs().max().item() < 0.02
    assert (lse - rl).abs().max().item() < 1e-3


def test_attention_split_outputs(dev):
    from vllm_omni_b200.ops import attention as A
    torch.manual_seed(4)
    B, S, H, split = 2, 300, 2, 260
    q, k, v = (torch.randn(B, S, H, 128, device=dev, dtype=torch.bfloat16) for _ in range(3))
    o1 = torch.empty(B, split, H, 128, device=dev, dtype=torch.bfloat16)
    o2 = torch.empty(B, S - split, H, 128, device=dev, dtype=torch.bfloat16)
    A.attention(q, k, v, out=o1, out2=o2, split=split)
    ref = A.attention_reference(q, k, v)
    _status_ok(dev)
    assert (o1.float() - ref[:, :split].float()).abs().max().item() < 0.02
    assert (o2.float() - ref[:, split:].float()).abs().max().item() < 0.02


def test_norm_modulate(dev):
    from vllm_omni_b200.ops import fused
    torch.manual_seed(5)
    B, S, D = 2, 333, 3072
    x = torch.randn(B, S, D, device=dev, dtype=torch.bfloat16)
    mod = torch.randn(B, 6 * D, device=dev, dtype=torch.bfloat16) * 0.3
    y = fused.norm_modulate(x, shift=mod[:, :D], scale=mod[:, D:2 * D])
    ref = fused.norm_modulate_reference(x, shift=mod[:, :D], scale=mod[:, D:2 * D])
    assert (y.float() - ref.float()).abs().max().item() < 0.05
    w = torch.randn(D, device=dev, dtype=torch.bfloat16)
    y = fused.norm_modulate(x, weight=w, rms=True)
    ref = fused.norm_modulate_reference(x, weight=w, rms=True)
    assert (y.float() - ref.float()).abs().max().item() < 0.05


@pytest.mark.parametrize("interleaved", [True, False])
def test_qk_norm_rope(dev, interleaved):
    from vllm_omni_b200.ops import fused
    torch.manual_seed(6)
    B, S, H, Dh, s_alt = 2, 300, 6, 128, 263
    qkv = torch.randn(B, S, 3 * H * Dh, device=dev, dtype=torch.bfloat16)
    ws = [torch.randn(Dh, device=dev, dtype=torch.bfloat16) for _ in range(4)]
    ang = torch.randn(S, Dh // 2, device=dev)
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    ref = fused.qk_norm_rope_reference(qkv.clone(), H, H, Dh, *ws, s_alt, cos, sin, interleaved, 1e-6)
    out = fused.qk_norm_rope_(qkv.clone(), H, H, Dh, *ws, s_alt=s_alt, cos=cos, sin=sin, interleaved=interleaved)
    assert (out.float() - ref.float()).abs().max().item() < 0.05


def test_cfg_euler_and_rel_l1(dev):
    from vllm_omni_b200.ops import fused
    torch.manual_seed(7)
    pos = torch.randn(2, 4096, 64, device=dev, dtype=torch.bfloat16)
    neg = torch.randn_like(pos)
    lat = torch.randn(2, 4096, 64, device=dev)
    ref = fused.cfg_euler_step_reference(pos, neg, lat.clone(), 4.0, -0.02, True)
    lb = torch.empty_like(pos)
    out = fused.cfg_euler_step_(pos, neg, lat.clone(), 4.0, -0.02, True, lb)
    assert (out - ref).abs().max().item() < 1e-4
    assert (lb.float() - ref).abs().max().item() < 0.03
    a = torch.randn(2, 1000, 3072, device=dev, dtype=torch.bfloat16)
    b = a + 0.1 * torch.randn_like(a)
    st = fused.RelL1State(dev, [2.0, 0.5], 10.0)
    fused.rel_l1_update(a, b, st)
    rel = float(fused.rel_l1_reference(a, b))
    got = st.state.tolist()
    assert abs(got[1] - rel) < 1e-3 * rel and abs(got[0] - (2.0 * rel + 0.5)) < 1e-3 and got[2] == 1.0


@pytest.mark.parametrize("Sq,Skv,off", [(300, 300, 0), (128, 700, 572), (513, 513, 0), (40, 1000, 960)])
def test_attention_causal(dev, Sq, Skv, off):
    from vllm_omni_b200.ops import attention as A
    torch.manual_seed(8)
    q = torch.randn(1, Sq, 8, 128, device=dev, dtype=torch.bfloat16)
    k = torch.randn(1, Skv, 2, 128, device=dev, dtype=torch.bfloat16)
    v = torch.randn(1, Skv, 2, 128, device=dev, dtype=torch.bfloat16)
    o = A.attention(q, k, v, causal=True, q_offset=off)
    ref = A.attention_reference(q, k, v, causal=True, q_offset=off)
    _status_ok(dev)
    assert (o.float() - ref.float()).abs().max().item() < 0.03


@pytest.mark.parametrize("impl", ["tc", "simt"])
@pytest.mark.parametrize("H,Hkv,splits", [(32, 4, 4), (8, 8, 1), (16, 4, 3)])
def test_paged_decode(dev, H, Hkv, splits, impl):
    from vllm_omni_b200.ops import kv_cache as KC
    from vllm_omni_b200.ops import attention as A
    torch.manual_seed(9)
    bs, nblk, D = 16, 64, 128
    lens = [37, 200, 1, 129]
    kc = torch.zeros(nblk, bs, Hkv, D, device=dev, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    perm = torch.randperm(nblk).tolist()
    tables, ks, vs = [], [], []
    for L in lens:
        nb = (L + bs - 1) // bs
        ids = [perm.pop() for _ in range(nb)]
        tables.append(ids)
        k = torch.randn(L, Hkv, D, device=dev, dtype=torch.bfloat16)
        v = torch.randn(L, Hkv, D, device=dev, dtype=torch.bfloat16)
        slots = torch.tensor([ids[t // bs] * bs + t % bs for t in range(L)], dtype=torch.int32, device=dev)
        KC.kv_write(k, v, kc, vc, slots)
        ks.append(k); vs.append(v)
    maxb = max(len(t) for t in tables)
    bt = torch.tensor([t + [0] * (maxb - len(t)) for t in tables], dtype=torch.int32, device=dev)
    sl = torch.tensor(lens, dtype=torch.int32, device=dev)
    q = torch.randn(len(lens), H, D, device=dev, dtype=torch.bfloat16)
    out = KC.paged_decode(q, kc, vc, bt, sl, num_splits=splits, impl=impl)
    for i, L in enumerate(lens):
        ref = A.attention_reference(q[i:i + 1, None].reshape(1, 1, H, D), ks[i][None], vs[i][None])
        assert (out[i].float() - ref[0, 0].float()).abs().max().item() < 0.03, i
        gk, gv = KC.kv_gather(kc, vc, bt[i], L)
        assert torch.equal(gk, ks[i]) and torch.equal(gv, vs[i])


@pytest.mark.parametrize("M,N,K,act", [(300, 384, 512, None), (1024, 3072, 1024, "gelu_tanh"), (64, 136, 256, None)])
def test_fp8_block_scaled_gemm(dev, M, N, K, act):
    from vllm_omni_b200.diffusion.quantization import fp8
    torch.manual_seed(4)
    x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device=dev, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=dev, dtype=torch.bfloat16)
    w8, sw = fp8.quantize_weight_blockwise(w)
    y = fp8.fp8_linear(x, (w8, sw), bias=bias, act=act, residual=res)
    _status_ok(dev)
    # oracle 1: the same quantised operands, dequantised and multiplied in fp32
    ref = fp8.fp8_linear_reference(x.cpu(), w8.cpu(), sw.cpu(), bias.cpu(), act, res.cpu())
    err = (y.float().cpu() - ref).abs().max().item()
    assert err < 0.02 * max(1.0, ref.abs().max().item()), err
    # oracle 2: the unquantised product; e4m3 with 128-wide scales stays within a few percent
    full = fp8._epi(x.float().cpu() @ w.float().cpu().t(), bias.cpu(), act, res.cpu(), None)
    rel = (y.float().cpu() - full).norm() / full.norm()
    assert rel < 0.05, rel


@pytest.mark.parametrize("T,L", [(150, 150), (140, 290), (1, 77), (300, 1000)])
def test_paged_prefill_chunk(dev, T, L):
    """Causal attention of the last T tokens of an L-token sequence straight from the pages."""
    from vllm_omni_b200.ops import kv_cache as KC
    from vllm_omni_b200.ops import attention as A
    torch.manual_seed(11)
    bs, nblk, H, Hkv, D = 16, 80, 8, 2, 128
    kc = torch.zeros(nblk, bs, Hkv, D, device=dev, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    ids = torch.randperm(nblk)[: (L + bs - 1) // bs].tolist()
    k = torch.randn(L, Hkv, D, device=dev, dtype=torch.bfloat16)
    v = torch.randn(L, Hkv, D, device=dev, dtype=torch.bfloat16)
    slots = torch.tensor([ids[t // bs] * bs + t % bs for t in range(L)], dtype=torch.int32, device=dev)
    KC.kv_write(k, v, kc, vc, slots)
    bt = torch.tensor(ids, dtype=torch.int32, device=dev)
    q = torch.randn(T, H, D, device=dev, dtype=torch.bfloat16)
    out = KC.paged_prefill(q, kc, vc, bt, L)
    ref = A.attention_reference(q[None], k[None], v[None], causal=True, q_offset=L - T)[0]
    _status_ok(dev)
    assert (out.float() - ref.float()).abs().max().item() < 0.03


@pytest.mark.parametrize("N,H,W,cin,cout,k", [(1, 16, 16, 16, 96, 3), (2, 13, 21, 96, 192, 3), (1, 40, 24, 384, 384, 3),
                                            (1, 9, 7, 96, 8, 3), (2, 10, 33, 192, 96, 1)])
def test_conv2d_nhwc_implicit_gemm(dev, N, H, W, cin, cout, k):
    from vllm_omni_b200.ops import conv as C
    torch.manual_seed(5)
    w = torch.randn(cout, cin, k, k, device=dev) * (1.0 / (cin * k * k) ** 0.5)
    b = torch.randn(cout, device=dev) * 0.1
    wp, bp = C.pack_conv_weight(w, b)
    x = torch.randn(N, H, W, cin, device=dev, dtype=torch.bfloat16)
    res = torch.randn(N, H, W, wp.shape[0], device=dev, dtype=torch.bfloat16)
    y = C.conv2d_nhwc(x, wp, bp, k, cin, act="silu", residual=res)
    ref = C.conv2d_nhwc_reference(x, wp, bp, k, cin, act="silu", residual=res)
    _status_ok(dev)
    assert (y.float() - ref).abs().max().item() < 0.03 * max(1.0, ref.abs().max().item())


def test_vae_elementwise_nhwc(dev):
    from vllm_omni_b200.ops import conv as C
    torch.manual_seed(6)
    x = torch.randn(2, 9, 11, 96, device=dev, dtype=torch.bfloat16) * 3
    g = (torch.rand(96, device=dev) + 0.5).bfloat16()
    for silu in (True, False):
        y = C.rmsnorm_silu_nhwc(x, g, silu=silu)
        ref = C.rmsnorm_silu_nhwc(x.cpu(), g.cpu(), silu=silu)
        assert (y.cpu().float() - ref.float()).abs().max().item() < 0.03
    assert torch.equal(C.upsample2x_nhwc(x).cpu(), C.upsample2x_nhwc(x.cpu()))
    z = torch.randn(2, 5, 7, 6, device=dev)
    assert torch.equal(C.nchw_to_nhwc(z).cpu(), C.nchw_to_nhwc(z.cpu()))
    img = torch.randn(2, 6, 5, 8, device=dev, dtype=torch.bfloat16)
    assert torch.equal(C.nhwc_to_image(img).cpu(), C.nhwc_to_image(img.cpu()))
    d = (C.nhwc_to_image(img, uint8=True).cpu().int() - C.nhwc_to_image(img.cpu(), uint8=True).int()).abs().max()
    assert int(d) <= 1


def test_vae_decoder_nhwc_matches_torch(dev):
    from vllm_omni_b200.diffusion.models.vae.autoencoder_kl_qwenimage import AutoencoderKLQwenImage2d, QwenImageVAEConfig
    torch.manual_seed(7)
    vae = AutoencoderKLQwenImage2d(QwenImageVAEConfig()).to(dev).bfloat16()
    for p in vae.parameters():
        if p.dim() > 1:
            p.data.normal_(0, (1.0 / p[0].numel()) ** 0.5)
    z = torch.randn(1, 16, 24, 20, device=dev)
    vae.decoder_impl = "torch"
    ref = vae.decode(z).float()
    vae.decoder_impl = "nhwc"
    out = vae.decode(z).float()
    _status_ok(dev)
    assert out.shape == ref.shape == (1, 3, 192, 160)
    assert (out - ref).abs().mean().item() < 0.02 and (out - ref).abs().max().item() < 0.25


@pytest.mark.parametrize("N,H,W,ch,G", [(2, 17, 23, 128, 32), (1, 64, 64, 512, 32), (3, 5, 7, 32, 8), (1, 40, 40, 256, 32)])
def test_groupnorm_nhwc(dev, N, H, W, ch, G):
    """Channels-last GroupNorm (+ SiLU) against torch's GroupNorm in fp32; bit-identical between two runs."""
    import torch.nn.functional as F
    from vllm_omni_b200.ops import conv as C
    torch.manual_seed(13)
    x = (torch.randn(N, H, W, ch, device=dev) * 2 + 0.7).to(torch.bfloat16)
    gamma, beta = torch.rand(ch, device=dev) + 0.5, torch.randn(ch, device=dev) * 0.2
    for silu in (True, False):
        y = C.groupnorm_nhwc(x, gamma, beta, G, 1e-6, silu=silu)
        _status_ok(dev)
        ref = F.group_norm(x.float().permute(0, 3, 1, 2), G, gamma, beta, 1e-6)
        ref = (F.silu(ref) if silu else ref).permute(0, 2, 3, 1)
        assert (y.float() - ref).abs().max().item() < 0.04, (silu, (y.float() - ref).abs().max().item())
        assert torch.equal(y, C.groupnorm_nhwc(x, gamma, beta, G, 1e-6, silu=silu))


def test_kl_vae_decoder_nhwc_matches_torch(dev):
    """The FLUX-family AutoencoderKL decoder on the channels-last kernels against the cuDNN module, full width."""
    from vllm_omni_b200.diffusion.models.vae.autoencoder_kl import AutoencoderKL
    torch.manual_seed(12)
    vae = AutoencoderKL().to(dev).bfloat16()
    for p in vae.parameters():
        if p.dim() > 1:
            p.data.normal_(0, (1.0 / p[0].numel()) ** 0.5)
    z = torch.randn(1, 16, 24, 20, device=dev)
    vae.decoder_impl = "torch"
    ref = vae.decode(z).float()
    vae.decoder_impl = "nhwc"
    out = vae.decode(z).float()
    _status_ok(dev)
    assert vae._nhwc, "the channels-last decoder was not used"
    assert out.shape == ref.shape == (1, 3, 192, 160)
    assert (out - ref).abs().mean().item() < 0.02 and (out - ref).abs().max().item() < 0.3


def test_video_vae_decoder_nhwc_matches_torch(dev):
    """Causal 3-D decoder on the channels-last kernels (temporal taps accumulated through the residual operand,
    per-convolution frame caches across chunks) against the cuDNN module, full-width channels."""
    from vllm_omni_b200.diffusion.models.vae.autoencoder_kl_wan import AutoencoderKLWan
    torch.manual_seed(11)
    vae = AutoencoderKLWan().to(dev).bfloat16()
    for p in vae.parameters():
        if p.dim() > 1:
            p.data.normal_(0, (1.0 / p[0].numel()) ** 0.5)
    z = torch.randn(1, 16, 3, 12, 16, device=dev)
    vae.decoder_impl = "torch"
    ref = vae.decode(z).float()
    vae.decoder_impl = "nhwc"
    for chunk in (1, 0):
        out = vae.decode(z, chunk_frames=chunk).float()
        _status_ok(dev)
        assert out.shape == ref.shape == (1, 3, 9, 96, 128)
        assert (out - ref).abs().mean().item() < 0.02 and (out - ref).abs().max().item() < 0.3, chunk


def test_wide_head_attention_gemm_softmax_gemm(dev):
    """The VAE's one-head attention: two GEMM launches around the row-softmax kernel, queries in chunks."""
    import torch.nn.functional as F

    from vllm_omni_b200.ops import conv as C
    torch.manual_seed(9)
    B, N, ch = 2, 1000, 384
    t = torch.randn(B, N, 3, ch, device=dev, dtype=torch.bfloat16)
    q, k, v = t[:, :, 0], t[:, :, 1], t[:, :, 2]
    ref = F.scaled_dot_product_attention(q.float()[:, None], k.float()[:, None], v.float()[:, None])[:, 0]
    for rows in (4096, 384):
        out = C.wide_head_attention(q, k, v, chunk_rows=rows)
        _status_ok(dev)
        assert (out.float() - ref).abs().max().item() < 0.03, rows
    x = torch.randn(37, 4096, device=dev, dtype=torch.bfloat16) * 4
    keep = x.clone()
    want = torch.softmax(x.float()[:, :2056] * 0.3, dim=-1)
    got = C.softmax_rows_(x[:, :2056], 0.3)                # a pitched view: row stride 4096, 2056 columns
    assert (got.float() - want).abs().max().item() < 4e-3 and abs(got.float().sum(-1) - 1).max().item() < 2e-2
    assert torch.equal(x[:, 2056:], keep[:, 2056:])        # columns past the view are untouched


def test_gemm_two_problems_one_launch(dev):
    """Image-stream and text-stream linears of one layer through a single CTA-pair launch."""
    from vllm_omni_b200.ops import gemm
    torch.manual_seed(8)
    B, S1, S2, K, N = 2, 2100, 260, 512, 1544
    mk = lambda *s: torch.randn(*s, device=dev, dtype=torch.bfloat16)
    x1, x2 = mk(B, S1, K), mk(B, S2, K)
    w1, w2 = mk(N, K) * 0.05, mk(N, K) * 0.05
    b1, b2 = mk(N), mk(N)
    r1, r2 = mk(B, S1, N), mk(B, S2, N)
    g1, g2 = mk(B, N), mk(B, N)
    o1, o2 = torch.empty_like(r1), torch.empty_like(r2)
    gemm.linear_pair(dict(x=x1, w=w1, bias=b1, act="gelu_tanh", residual=r1, gate=g1, out=o1),
                     dict(x=x2, w=w2, bias=b2, residual=r2, gate=g2, out=o2))
    _status_ok(dev)
    ref1 = gemm.linear_reference(x1, w1, b1, "gelu_tanh", r1, g1).float()
    ref2 = gemm.linear_reference(x2, w2, b2, None, r2, g2).float()
    assert (o1.float() - ref1).abs().max().item() <= 0.02 * ref1.abs().max().item() + 1e-2
    assert (o2.float() - ref2).abs().max().item() <= 0.02 * ref2.abs().max().item() + 1e-2
    # joint [B, S1 + S2, N] output buffer, rows of each stream written in place (the QKV layout)
    joint = torch.zeros(B, S1 + S2, N, device=dev, dtype=torch.bfloat16)
    gemm.linear_pair(dict(x=x1, w=w1, bias=b1, out=joint[:, :S1], out_rows_per_batch=S1, out_batch_stride=(S1 + S2) * N),
                     dict(x=x2, w=w2, bias=b2, out=joint[:, S1:], out_rows_per_batch=S2, out_batch_stride=(S1 + S2) * N))
    _status_ok(dev)
    refj = torch.cat([gemm.linear_reference(x1, w1, b1).float(), gemm.linear_reference(x2, w2, b2).float()], 1)
    assert (joint.float() - refj).abs().max().item() <= 0.02 * refj.abs().max().item() + 1e-2


@pytest.mark.parametrize("S1,S2,N,K", [(1024, 64, 3072, 512), (1024, 64, 1536, 256), (300, 40, 9216, 128), (64, 8, 3080, 64)])
def test_gemm_two_small_problems_share_a_one_cta_launch(dev, S1, S2, N, K):
    """Row counts of a sequence-parallel rank: too few 256-row tiles for a wave, so the launcher takes
    128-row tiles and runs the text rows' tiles beside the image rows' (epilogue variants and the
    joint-buffer output included); forcing the CTA-pair kernel gives the same numbers."""
    from vllm_omni_b200.ops import gemm
    torch.manual_seed(S1 + N)
    B = 1
    mk = lambda *s: torch.randn(*s, device=dev, dtype=torch.bfloat16)
    x1, x2 = mk(B, S1, K), mk(B, S2, K)
    w1, w2 = mk(N, K) * 0.05, mk(N, K) * 0.05
    b1, b2 = mk(N), mk(N)
    r1, r2 = mk(B, S1, N), mk(B, S2, N)
    g1, g2 = mk(B, N), mk(B, N)
    ref1 = gemm.linear_reference(x1, w1, b1, "gelu_tanh", r1, g1).float()
    ref2 = gemm.linear_reference(x2, w2, b2, None, r2, g2).float()
    for force in (False, True):
        o1, o2 = torch.empty_like(r1), torch.empty_like(r2)
        gemm.linear_pair(dict(x=x1, w=w1, bias=b1, act="gelu_tanh", residual=r1, gate=g1, out=o1),
                         dict(x=x2, w=w2, bias=b2, residual=r2, gate=g2, out=o2), force_pair=force)
        _status_ok(dev)
        assert (o1.float() - ref1).abs().max().item() <= 0.02 * ref1.abs().max().item() + 1e-2
        assert (o2.float() - ref2).abs().max().item() <= 0.02 * ref2.abs().max().item() + 1e-2
    joint = torch.zeros(B, S1 + S2, N, device=dev, dtype=torch.bfloat16)
    gemm.linear_pair(dict(x=x1, w=w1, bias=b1, out=joint[:, :S1], out_rows_per_batch=S1, out_batch_stride=(S1 + S2) * N),
                     dict(x=x2, w=w2, bias=b2, out=joint[:, S1:], out_rows_per_batch=S2, out_batch_stride=(S1 + S2) * N))
    _status_ok(dev)
    refj = torch.cat([gemm.linear_reference(x1, w1, b1).float(), gemm.linear_reference(x2, w2, b2).float()], 1)
    assert (joint.float() - refj).abs().max().item() <= 0.02 * refj.abs().max().item() + 1e-2
    # the scatter epilogue through local "peer" pointers: two column groups into two buffers
    if N % 128 == 0:
        G = N // 2
        bufs = [torch.zeros(B, S1 + S2, G, device=dev, dtype=torch.bfloat16) for _ in range(2)]
        es = 2
        sc1 = (2, G, [b_.data_ptr() for b_ in bufs], G)
        sc2 = (2, G, [b_.data_ptr() + S1 * G * es for b_ in bufs], G)
        gemm.linear_pair(dict(x=x1, w=w1, bias=b1, scatter=sc1, out_rows_per_batch=S1, out_batch_stride=(S1 + S2) * G),
                         dict(x=x2, w=w2, bias=b2, scatter=sc2, out_rows_per_batch=S2, out_batch_stride=(S1 + S2) * G))
        _status_ok(dev)
        for r in range(2):
            want = refj[:, :, r * G:(r + 1) * G]
            assert (bufs[r].float() - want).abs().max().item() <= 0.02 * want.abs().max().item() + 1e-2


@pytest.mark.parametrize("B,S,H,Hkv,kvl,causal", [(1, 128, 1, 1, None, False), (2, 600, 4, 2, [600, 333], False),
                                                  (1, 2100, 3, 3, None, False), (1, 700, 2, 2, None, True)])
def test_attention_head_dim_64(dev, B, S, H, Hkv, kvl, causal):
    """Head size 64 (SD3, Stable Audio, audio / vision towers): one 64-wide TMA box per tile, N = 64
    for P*V, 4-deep K/V rings; same checks as the 128 case, plus split outputs."""
    from vllm_omni_b200.ops import attention as A
    torch.manual_seed(5)
    qkv = torch.randn(B, S, H + 2 * Hkv, 64, device=dev, dtype=torch.bfloat16)
    q, k, v = qkv[:, :, :H], qkv[:, :, H:H + Hkv], qkv[:, :, H + Hkv:]
    kl = torch.tensor(kvl, dtype=torch.int32, device=dev) if kvl else None
    o, lse = A.attention(q, k, v, kv_lens=kl, return_lse=True, causal=causal)
    ref, rl = A.attention_reference(q, k, v, kv_lens=kl, return_lse=True, causal=causal)
    _status_ok(dev)
    assert (o.float() - ref.float()).abs().max().item() < 0.02
    assert (lse - rl).abs().max().item() < 1e-3
    if kvl is None and not causal:
        split = S - 60
        o1 = torch.empty(B, split, H, 64, device=dev, dtype=torch.bfloat16)
        o2 = torch.empty(B, S - split, H, 64, device=dev, dtype=torch.bfloat16)
        A.attention(q, k, v, out=o1, out2=o2, split=split)
        _status_ok(dev)
        assert (o1.float() - ref[:, :split].float()).abs().max().item() < 0.02
        assert (o2.float() - ref[:, split:].float()).abs().max().item() < 0.02


def test_kernels_launch_on_every_device_of_the_process():
    """One process driving two GPUs (stages of a pipeline as threads): the large-shared-memory kernels
    are prepared per device, so the second device launches as well as the first."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from vllm_omni_b200.ops import gemm
    from vllm_omni_b200.ops.attention import attention, attention_reference
    prev = torch.cuda.current_device()
    try:
        for d in (0, 1, 0):
            torch.cuda.set_device(d)
            dv = torch.device("cuda", d)
            torch.manual_seed(d)
            x = torch.randn(300, 256, device=dv, dtype=torch.bfloat16)
            w = torch.randn(512, 256, device=dv, dtype=torch.bfloat16) * 0.05
            for bn in (0, 128, 384):
                y = gemm.linear(x, w, force_bn=bn).float()
                ref = x.float() @ w.float().t()
                assert (y - ref).abs().max().item() <= 0.02 * ref.abs().max().item() + 1e-3
            q, k, v = (torch.randn(1, 200, 2, 128, device=dv, dtype=torch.bfloat16) for _ in range(3))
            o = attention(q, k, v).float()
            assert (o - attention_reference(q.float(), k.float(), v.float())).abs().max().item() < 0.03
            _status_ok(dv)
    finally:
        torch.cuda.set_device(prev)


@pytest.mark.parametrize("D", [128, 64])
def test_attention_continuation_merges_two_key_sets(dev, D):
    """A launch over keys B with ``merge_prev`` = the result over keys A equals attention over A + B;
    an empty second key set leaves the first result untouched; in-place (prev is out) is allowed."""
    from vllm_omni_b200.ops.attention import attention, attention_reference
    torch.manual_seed(5)
    B, Sq, H, Hkv = 2, 300, 4, 2
    q = torch.randn(B, Sq, H, D, device=dev, dtype=torch.bfloat16)
    ka, va = (torch.randn(B, 200, Hkv, D, device=dev, dtype=torch.bfloat16) for _ in range(2))
    kb, vb = (torch.randn(B, 333, Hkv, D, device=dev, dtype=torch.bfloat16) for _ in range(2))
    lens_b = torch.tensor([333, 150], dtype=torch.int32, device=dev)
    o, lse = attention(q, ka, va, return_lse=True)
    o2, lse2 = attention(q, kb, vb, kv_lens=lens_b, merge_prev=(o, lse), out=o, return_lse=True)
    assert o2.data_ptr() == o.data_ptr()
    for b in range(B):
        n = int(lens_b[b])
        k_all, v_all = torch.cat([ka[b:b + 1], kb[b:b + 1, :n]], 1), torch.cat([va[b:b + 1], vb[b:b + 1, :n]], 1)
        ref, ref_lse = attention_reference(q[b:b + 1].float(), k_all.float(), v_all.float(), return_lse=True)
        assert (o2[b:b + 1].float() - ref).abs().max().item() < 0.03
        assert (lse2[b:b + 1] - ref_lse).abs().max().item() < 0.02
    # no valid key in the continuation: the earlier rows and LSE come back unchanged
    o3, lse3 = attention(q, ka, va, return_lse=True)
    keep = o3.clone()
    zero = torch.zeros(B, dtype=torch.int32, device=dev)
    o4, lse4 = attention(q, kb, vb, kv_lens=zero, merge_prev=(o3, lse3), out=o3, return_lse=True)
    assert torch.equal(o4, keep) and torch.equal(lse4, lse3)
    _status_ok(dev)
