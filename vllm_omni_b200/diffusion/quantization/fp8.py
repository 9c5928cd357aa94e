"""FP8 (e4m3) W8A8 linear layers with 128-element block scales.

Weights are quantised once after loading (per 128 x 128 block), activations dynamically per
row and 128-wide K block right before the GEMM; the contraction runs on the block-scaled
tcgen05 kernel (csrc/gemm_fp8_sm100.cu).  Configuration mirrors the reference's
``DiffusionFp8Config`` (vllm_omni/diffusion/quantization/fp8.py -> vLLM ``Fp8Config`` with
``is_checkpoint_fp8_serialized=False``, ``activation_scheme='dynamic'``,
``weight_block_size=[128, 128]``, ``ignored_layers``); its documentation advises keeping the
image-stream MLP of Qwen-Image in bf16, which ``ignored_layers`` expresses.
"""
from __future__ import annotations

import ctypes
import fnmatch
from dataclasses import dataclass, field

import torch

from ...ops import _native as nv
from ...ops import gemm

FP8_MAX = 448.0


@dataclass
class DiffusionFp8Config:
    activation_scheme: str = "dynamic"
    weight_block_size: tuple = (128, 128)
    ignored_layers: list[str] = field(default_factory=list)     # glob patterns on module names
    min_features: int = 1024                                    # small layers stay in bf16

    @classmethod
    def from_dict(cls, d: dict | None) -> "DiffusionFp8Config":
        d = dict(d or {})
        names = set(cls.__dataclass_fields__)
        c = cls(**{k: v for k, v in d.items() if k in names})
        if tuple(c.weight_block_size) != (128, 128):
            raise ValueError("only weight_block_size=[128, 128] is supported")
        if c.activation_scheme != "dynamic":
            raise ValueError("only activation_scheme='dynamic' is supported")
        return c


def quantize_weight_blockwise(w: torch.Tensor):
    """w [N, K] -> (w8 [N, K] float8_e4m3fn, scales [ceil(N/128), K/128] fp32)."""
    N, K = w.shape
    assert K % 128 == 0, "K must be a multiple of 128 for block-scaled fp8"
    Np = (N + 127) // 128 * 128
    wf = torch.zeros(Np, K, dtype=torch.float32, device=w.device)
    wf[:N] = w.float()
    blocks = wf.view(Np // 128, 128, K // 128, 128)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-8)
    scale = amax / FP8_MAX
    q = (blocks / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).view(Np, K)[:N]
    return q.to(torch.float8_e4m3fn).contiguous(), scale.contiguous()


def quantize_rows_reference(x: torch.Tensor):
    """x [M, K] -> (x8, scales [M, K/128]) with the kernel's rounding rules."""
    M, K = x.shape
    b = x.float().view(M, K // 128, 128)
    scale = b.abs().amax(-1).clamp_min(1e-8) / FP8_MAX
    q = (b / scale[..., None]).clamp(-FP8_MAX, FP8_MAX).view(M, K).to(torch.float8_e4m3fn)
    return q, scale


def fp8_linear_reference(x, w8, sw, bias=None, act=None, residual=None, gate=None):
    """Dequantise-and-matmul restatement (fp32) of the block-scaled GEMM."""
    K = x.shape[-1]
    x2 = x.reshape(-1, K)
    q, sa = quantize_rows_reference(x2)
    xd = (q.float().view(x2.shape[0], K // 128, 128) * sa[..., None]).view_as(x2)
    N = w8.shape[0]
    wd = w8.float().view(N, K // 128, 128) * sw.repeat_interleave(128, 0)[:N, :, None]
    y = xd @ wd.view(N, K).t()
    y = y.reshape(*x.shape[:-1], N)
    return _epi(y, bias, act, residual, gate)


def _epi(y, bias, act, residual, gate):
    import torch.nn.functional as F
    if bias is not None:
        y = y + bias.float()
    if act == "gelu_tanh":
        y = F.gelu(y, approximate="tanh")
    elif act == "silu":
        y = F.silu(y)
    if gate is not None:
        shp = y.shape
        y = (y.reshape(gate.shape[0], -1, shp[-1]) * gate.float().unsqueeze(1)).reshape(shp)
    if residual is not None:
        y = y + residual.float()
    return y


def fp8_linear(x, fp8_state, bias=None, act=None, residual=None, gate=None, out=None, **_):
    w8, sw = fp8_state
    K, N = x.shape[-1], w8.shape[0]
    if not x.is_cuda:
        y = fp8_linear_reference(x, w8, sw, bias, act, residual, gate).to(x.dtype)
        if out is not None:
            out.copy_(y.reshape(out.shape))
            return out
        return y
    x2 = x.reshape(-1, K)
    M = x2.shape[0]
    lib = nv.lib("gemm_fp8_sm100")
    xq = torch.empty(M, K, dtype=torch.uint8, device=x.device)
    sa = torch.empty(M, K // 128, dtype=torch.float32, device=x.device)
    nv.check_rc(lib.omni_quant_fp8_rows(nv.ptr(x2), ctypes.c_long(x2.stride(0)), nv.ptr(xq), ctypes.c_long(K), nv.ptr(sa),
                                        ctypes.c_int(K // 128), ctypes.c_int(M), ctypes.c_int(K), nv.stream_ptr()),
                "omni_quant_fp8_rows")
    if out is None:
        out = torch.empty(*x.shape[:-1], N, dtype=x.dtype, device=x.device)
    o2 = out.view(-1, N)
    res2 = residual.reshape(-1, N) if residual is not None else None
    gs, rpb = 0, 0
    if gate is not None:
        rpb = M // gate.shape[0]
        gs = gate.stride(0) if gate.shape[0] > 1 else N
    st = nv.status_word(x.device)
    rc = lib.omni_gemm_fp8(nv.ptr(xq), ctypes.c_long(K), nv.ptr(sa), ctypes.c_int(K // 128), nv.ptr(w8), ctypes.c_long(K),
                           nv.ptr(sw), ctypes.c_int(sw.shape[1]), nv.ptr(o2), ctypes.c_int(o2.stride(0)), ctypes.c_int(M),
                           ctypes.c_int(N), ctypes.c_int(K), nv.ptr(bias), nv.ptr(res2),
                           ctypes.c_int(res2.stride(0) if res2 is not None else 0), nv.ptr(gate), ctypes.c_int(gs),
                           ctypes.c_int(rpb), ctypes.c_int(gemm.ACT[act]), nv.ptr(st), nv.stream_ptr())
    nv.check_rc(rc, "omni_gemm_fp8")
    return out


def quantize_pipeline(pipe, od_config) -> int:
    """Quantise every eligible ``FusedLinear`` of the pipeline's transformer in place; returns
    the number of layers converted."""
    from ..layers.linear import FusedLinear
    qc = od_config.quantization_config
    cfg = qc if isinstance(qc, DiffusionFp8Config) else DiffusionFp8Config.from_dict(qc if isinstance(qc, dict) else None)
    if od_config.quantization not in ("fp8",):
        raise ValueError(f"unsupported quantization {od_config.quantization!r}")
    n = 0
    for name, m in pipe.transformer.named_modules():
        if not isinstance(m, FusedLinear):
            continue
        if m.in_features % 128 or min(m.in_features, m.out_features) < cfg.min_features:
            continue
        if any(fnmatch.fnmatch(name, pat) for pat in cfg.ignored_layers):
            continue
        if name in ("mod", "norm_out", "proj_out", "img_in", "txt_in") or name.startswith("time_embed"):
            continue
        w8, sw = quantize_weight_blockwise(m.weight.data)
        m.fp8 = (w8.view(torch.uint8) if w8.is_cuda else w8, sw)
        m.weight.data = torch.empty(0, dtype=m.weight.dtype, device=m.weight.device)
        n += 1
    return n
