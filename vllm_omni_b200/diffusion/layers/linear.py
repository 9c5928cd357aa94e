"""Linear layer whose forward is the tcgen05 GEMM with a fused epilogue.

The layer keeps the HF/diffusers parameter names (``weight`` [out, in], ``bias`` [out]) so
checkpoints load unchanged.  Optional LoRA deltas (``y += scale * (x A^T) B^T``, the
semantics of vllm_omni/diffusion/lora/layers/base_linear.py) and fp8 block-scaled weights
attach to the same object.
"""
from __future__ import annotations

import torch
from torch import nn

from ...ops import gemm


class FusedLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, dtype=torch.bfloat16,
                 device=None, init_std: float = 0.02):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device),
                                   requires_grad=False)
        self.bias = nn.Parameter(torch.empty(out_features, dtype=dtype, device=device),
                                 requires_grad=False) if bias else None
        self.init_std = init_std
        self.lora = None      # set by the LoRA manager: list of (A [r, in], B [out, r], scale)
        self.fp8 = None       # set by the fp8 quantiser: (w_fp8, w_scale) block-scaled weights
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self, generator=None):
        if self.weight.device.type == "meta":
            return
        self.weight.normal_(0.0, self.init_std, generator=generator)
        if self.bias is not None:
            self.bias.zero_()

    def forward(self, x, act=None, residual=None, gate=None, out=None, **kw):
        if self.fp8 is not None:
            from ..quantization.fp8 import fp8_linear
            y = fp8_linear(x, self.fp8, self.bias, act=act, residual=residual, gate=gate, out=out, **kw)
        elif self.lora:
            # the LoRA delta enters before the activation / gate, so apply the epilogue last
            y = gemm.linear(x, self.weight, self.bias)
            for (A, B, scale) in self.lora:
                y = y + scale * gemm.linear(gemm.linear(x, A), B)
            y = _epilogue(y, act, residual, gate, out)
        else:
            y = gemm.linear(x, self.weight, self.bias, act=act, residual=residual, gate=gate, out=out, **kw)
        return y

    def extra_repr(self):
        return f"in={self.in_features}, out={self.out_features}, bias={self.bias is not None}"


def _epilogue(y, act, residual, gate, out):
    import torch.nn.functional as F
    if act == "gelu_tanh":
        y = F.gelu(y.float(), approximate="tanh").to(y.dtype)
    elif act == "silu":
        y = F.silu(y)
    if gate is not None:
        B = gate.shape[0]
        y = (y.reshape(B, -1, y.shape[-1]) * gate.unsqueeze(1)).reshape(y.shape)
    if residual is not None:
        y = y + residual
    if out is not None:
        out.copy_(y.reshape(out.shape))
        return out
    return y
