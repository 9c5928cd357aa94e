"""Channels-last vocoder path (K15): the 1-D implicit-GEMM convolution, transposed convolution as one
stride-1 convolution on phase-stacked weights, depthwise convolution and the fused snake activation
against PyTorch's NCT modules; code2wav end to end in both layouts.  GPU twins at the end."""
import pytest
import torch
import torch.nn.functional as F

from vllm_omni_b200.ops import conv as C


def _conv_case(dev, dtype, B, T, Cin, Cout, k, dil, pad, with_res):
    torch.manual_seed(k * 100 + dil)
    x = torch.randn(B, T, Cin, device=dev).to(dtype)
    w = (torch.randn(Cout, Cin, k, device=dev) * (1.0 / (Cin * k) ** 0.5)).to(dtype)
    b = torch.randn(Cout, device=dev).to(dtype)
    pw, pb = C.pack_conv1d_weight(w, b, dtype)
    res = torch.randn(B, T, pw.shape[0], device=dev).to(dtype) if with_res else None
    y = C.conv1d_nlc(x, pw, pb, k, Cin, dil, pad, residual=res).float()[..., :Cout]
    right = max(0, (k - 1) * dil - pad)
    ref = F.conv1d(F.pad(x.float().transpose(1, 2), (pad, right)), w.float(), b.float(), dilation=dil)[..., :T].transpose(1, 2)
    if with_res:
        ref = ref + res.float()[..., :Cout]
    return y, ref


@pytest.mark.parametrize("k,dil,causal", [(7, 1, True), (7, 9, True), (1, 1, True), (3, 5, False), (11, 3, False)])
def test_conv1d_nlc_matches_conv1d(k, dil, causal):
    pad = (k - 1) * dil if causal else (k - 1) * dil // 2
    y, ref = _conv_case("cpu", torch.float32, 2, 41, 12, 20, k, dil, pad, with_res=(k == 1))
    assert (y - ref).abs().max() < 1e-5


@pytest.mark.parametrize("k,r,p,trim", [(8, 4, 4, 4), (16, 8, 8, 8), (11, 5, 3, 3), (3, 3, 0, 0), (7, 3, 2, 2), (4, 2, 0, 2)])
def test_transposed_conv_as_one_phase_stacked_convolution(k, r, p, trim):
    torch.manual_seed(k)
    B, T, Cin, Cout = 2, 23, 10, 6
    x = torch.randn(B, T, Cin)
    w, b = torch.randn(Cin, Cout, k) * 0.2, torch.randn(Cout)
    full = F.conv_transpose1d(x.transpose(1, 2), w, b, stride=r)
    ref = full[..., p:full.shape[-1] - trim].transpose(1, 2)
    packed = C.pack_conv_transpose1d_weight(w, b, r, p, torch.float32)
    y = C.conv_transpose1d_nlc(x, packed, Cin, r, ref.shape[1])
    assert y.shape[1] == ref.shape[1] and (y[..., :Cout] - ref).abs().max() < 1e-5
    assert packed[2] <= -(-k // r) + 1            # taps of the stacked kernel: at most ceil(k / r) + 1


def test_depthwise_and_snake():
    torch.manual_seed(0)
    x = torch.randn(2, 19, 16)
    w, b = torch.randn(16, 1, 7), torch.randn(16)
    ref = F.conv1d(F.pad(x.transpose(1, 2), (6, 0)), w, b, groups=16).transpose(1, 2)
    assert (C.dwconv1d_nlc(x, w[:, 0].t().contiguous(), b, 7, 1, 6) - ref).abs().max() < 1e-5
    a, ib = torch.rand(16) + 0.5, torch.rand(16) + 0.5
    assert torch.allclose(C.snake_nlc(x, a, ib), x + ib * torch.sin(x * a) ** 2, atol=1e-6)


def _code2wav(dev, dtype):
    from vllm_omni_b200.models.qwen3_omni.code2wav import Qwen3OmniCode2Wav
    from vllm_omni_b200.models.qwen3_omni.config import Qwen3OmniConfig
    torch.manual_seed(0)
    cfg = Qwen3OmniConfig.tiny()
    m = Qwen3OmniCode2Wav(cfg, dtype, dev)
    for p in m.parameters():
        if p.dim() >= 1:
            p.data.normal_(0, 0.1)
    c = cfg.code2wav
    codes = torch.randint(0, c.codebook_size, (2, c.num_quantizers, 9), device=dev)
    return m, codes


def test_code2wav_channels_last_equals_channels_first():
    m, codes = _code2wav("cpu", torch.float32)
    m.vocoder_layout = "nct"
    a = m.decode(codes)
    m.vocoder_layout = "nlc"
    b = m.decode(codes)
    assert a.shape == b.shape and (a - b).abs().max() < 1e-3
    assert (a.abs() < 1.0).any()                  # not everything is clamped


# ------------------------------------------------------------------ GPU
@pytest.mark.gpu
@pytest.mark.parametrize("Cin,Cout,k,dil,causal,res", [(96, 96, 7, 9, True, False), (768, 768, 7, 3, True, False),
                                                         (192, 192, 1, 1, True, True), (96, 1, 7, 1, True, False),
                                                         (512, 1536, 7, 1, True, False), (64, 64, 11, 5, False, False)])
def test_conv1d_nlc_gpu(Cin, Cout, k, dil, causal, res):
    pad = (k - 1) * dil if causal else (k - 1) * dil // 2
    y, ref = _conv_case("cuda", torch.bfloat16, 2, 1000, Cin, Cout, k, dil, pad, res)
    assert (y - ref).abs().max().item() <= 0.03 * ref.abs().max().item() + 0.02


@pytest.mark.gpu
@pytest.mark.parametrize("k,r,p,trim", [(16, 8, 8, 8), (10, 5, 5, 5), (2, 2, 0, 0), (11, 5, 3, 3)])
def test_transposed_conv_gpu(k, r, p, trim):
    torch.manual_seed(k)
    B, T, Cin, Cout = 2, 300, 384, 192
    x = torch.randn(B, T, Cin, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(Cin, Cout, k, device="cuda") * 0.05).bfloat16()
    b = torch.randn(Cout, device="cuda").bfloat16()
    full = F.conv_transpose1d(x.float().transpose(1, 2), w.float(), b.float(), stride=r)
    ref = full[..., p:full.shape[-1] - trim].transpose(1, 2)
    packed = C.pack_conv_transpose1d_weight(w, b, r, p, torch.bfloat16)
    y = C.conv_transpose1d_nlc(x, packed, Cin, r, ref.shape[1]).float()
    assert y.shape[1] == ref.shape[1] and (y[..., :Cout] - ref).abs().max().item() <= 0.03 * ref.abs().max().item() + 0.02


@pytest.mark.gpu
def test_depthwise_snake_and_code2wav_gpu():
    torch.manual_seed(0)
    x = torch.randn(2, 500, 64, device="cuda", dtype=torch.bfloat16)
    w, b = torch.randn(64, 1, 7, device="cuda"), torch.randn(64, device="cuda")
    ref = F.conv1d(F.pad(x.float().transpose(1, 2), (6, 0)), w, b, groups=64).transpose(1, 2)
    assert (C.dwconv1d_nlc(x, w[:, 0].t().contiguous(), b, 7, 1, 6).float() - ref).abs().max().item() < 0.05
    a, ib = torch.rand(64, device="cuda") + 0.5, torch.rand(64, device="cuda") + 0.5
    xf = x.float()
    assert (C.snake_nlc(x, a, ib).float() - (xf + ib * torch.sin(xf * a) ** 2)).abs().max().item() < 0.03
    m, codes = _code2wav("cuda", torch.bfloat16)
    m.vocoder_layout = "nct"
    want = m.decode(codes)
    m.vocoder_layout = None                        # the default on a GPU is the channels-last path
    got = m.decode(codes)
    assert got.shape == want.shape and (got - want).abs().max().item() < 0.08
    from vllm_omni_b200.ops import _native as nv
    torch.cuda.synchronize()
    assert int(nv.status_word(torch.device("cuda")).item()) == 0


def test_tts_tokenizer_decoder_channels_last_equals_channels_first():
    """The Qwen3-TTS 12 Hz decoder (transposed convolutions trimmed on the right only) in both layouts."""
    from vllm_omni_b200.models.qwen3_tts.tokenizer_12hz import Qwen3TTSTokenizerDecoder, TokenizerDecoderConfig
    torch.manual_seed(0)
    cfg = TokenizerDecoderConfig(codebook_size=32, num_quantizers=4, hidden_size=32, num_hidden_layers=1, num_attention_heads=2,
                                 num_key_value_heads=2, intermediate_size=48, sliding_window=8, head_dim=16, decoder_dim=64,
                                 upsample_rates=(4, 2), upsampling_ratios=(2,), codebook_dim=16, latent_dim=32)
    m = Qwen3TTSTokenizerDecoder(cfg, torch.float32, "cpu")
    for p in m.parameters():
        if p.dim() >= 1:
            p.data.normal_(0, 0.1)
    codes = torch.randint(0, 32, (2, 4, 11))
    m.vocoder_layout = "nct"
    a = m.decode(codes)
    m.vocoder_layout = "nlc"
    b = m.decode(codes)
    assert a.shape == b.shape == (2, 11 * 2 * 4 * 2) and (a - b).abs().max() < 1e-3


def _bigvgan(dev, dtype):
    from vllm_omni_b200.models.qwen2_5_omni.config import BigVGANConfig
    from vllm_omni_b200.models.qwen2_5_omni.token2wav import BigVGAN
    torch.manual_seed(0)
    cfg = BigVGANConfig(mel_dim=16, upsample_initial_channel=64, upsample_rates=(5, 2), upsample_kernel_sizes=(11, 4),
                        resblock_kernel_sizes=(3, 7), resblock_dilation_sizes=((1, 3), (1, 5)))
    m = BigVGAN(cfg).to(dev, dtype)
    for p in m.parameters():
        p.data.normal_(0, 0.15)
    mel = torch.randn(2, 16, 13, device=dev)
    return m, mel


def test_anti_aliased_snake_and_bigvgan_channels_last():
    from vllm_omni_b200.models.qwen2_5_omni.token2wav import FilteredActivation
    torch.manual_seed(1)
    fa = FilteredActivation(8)
    fa.act.alpha.data.normal_(0, 0.3)
    fa.act.beta.data.normal_(0, 0.3)
    x = torch.randn(2, 8, 11)
    want = fa(x).transpose(1, 2)
    got = C.aa_snake_nlc(x.transpose(1, 2).contiguous(), fa.act.alpha.exp(), 1.0 / (fa.act.beta.exp() + 1e-9),
                         fa.up_filter.flatten(), fa.down_filter.flatten())
    assert (got - want).abs().max() < 1e-5
    m, mel = _bigvgan("cpu", torch.float32)
    m.vocoder_layout = "nct"
    a = m(mel)
    m.vocoder_layout = "nlc"
    b = m(mel)
    assert a.shape == b.shape == (2, 130) and (a - b).abs().max() < 1e-3 and (a.abs() < 1).any()


@pytest.mark.gpu
def test_anti_aliased_snake_and_bigvgan_gpu():
    from vllm_omni_b200.models.qwen2_5_omni.token2wav import FilteredActivation
    torch.manual_seed(1)
    fa = FilteredActivation(64).cuda()
    fa.act.alpha.data.normal_(0, 0.3)
    fa.act.beta.data.normal_(0, 0.3)
    for T in (1, 3, 1001):                                   # ends of the signal are replicate-padded twice
        x = torch.randn(2, 64, T, device="cuda").bfloat16()
        want = fa(x.float()).transpose(1, 2)
        got = C.aa_snake_nlc(x.transpose(1, 2).contiguous(), fa.act.alpha.exp().contiguous(),
                             (1.0 / (fa.act.beta.exp() + 1e-9)).contiguous(), fa.up_filter.flatten().contiguous(),
                             fa.down_filter.flatten().contiguous()).float()
        assert (got - want).abs().max().item() < 0.05, T
    m, mel = _bigvgan("cuda", torch.bfloat16)
    m.vocoder_layout = "nct"
    want = m(mel.bfloat16())
    m.vocoder_layout = None
    assert m.use_nlc(mel)
    got = m(mel.bfloat16())
    assert got.shape == want.shape and (got - want).abs().max().item() < 0.1


def test_wide_head_attention_and_softmax_cpu_fallback():
    from vllm_omni_b200.ops import conv as C
    torch.manual_seed(0)
    t = torch.randn(1, 40, 3, 16)
    o = C.wide_head_attention(t[:, :, 0], t[:, :, 1], t[:, :, 2])
    want = torch.softmax(t[0, :, 0] @ t[0, :, 1].T / 4.0, -1) @ t[0, :, 2]
    assert torch.allclose(o[0], want, atol=1e-5)
    x = torch.randn(5, 16)
    w = torch.softmax(x * 0.5, -1)
    assert torch.allclose(C.softmax_rows_(x, 0.5), w)
