"""K16 — batched token sampling on the device (csrc/sampler.cu) with a PyTorch restatement
for CPU runs.  ``sample`` takes one ``RowParams`` per sequence."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field

import torch

from . import _native as nv


class _Row(ctypes.Structure):
    _fields_ = [("temperature", ctypes.c_float), ("top_p", ctypes.c_float), ("min_p", ctypes.c_float),
                ("top_k", ctypes.c_int), ("rep_penalty", ctypes.c_float), ("presence_penalty", ctypes.c_float),
                ("frequency_penalty", ctypes.c_float), ("seed", ctypes.c_ulonglong), ("step", ctypes.c_int),
                ("hist_off", ctypes.c_int), ("hist_len", ctypes.c_int), ("gen_off", ctypes.c_int),
                ("sup_off", ctypes.c_int), ("sup_len", ctypes.c_int), ("range_lo", ctypes.c_int),
                ("range_hi", ctypes.c_int)]


@dataclass
class RowParams:
    temperature: float = 1.0
    top_p: float = 1.0
    min_p: float = 0.0
    top_k: int = 0
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    seed: int = 0
    step: int = 0
    history: list = field(default_factory=list)      # prompt + generated token ids
    num_prompt_tokens: int = 0
    suppressed: list = field(default_factory=list)
    allowed_range: tuple | None = None                # (lo, hi) of admissible token ids


def _uniform(seed: int, step: int) -> float:
    def sm(x):
        x = (x + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
        x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
        x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
        return x ^ (x >> 31)
    h = sm((seed & 0xFFFFFFFFFFFFFFFF) ^ sm(step))
    return ((h >> 40) + 0.5) / 16777216.0


def sample_reference(logits: torch.Tensor, rows: list[RowParams]):
    """Same pipeline in PyTorch: returns (ids int64 [B], logprobs [B])."""
    ids, lps = [], []
    for r, p in enumerate(rows):
        w = logits[r].float().clone()
        V = w.numel()
        if p.allowed_range is not None:
            lo, hi = p.allowed_range
            m = torch.ones(V, dtype=torch.bool)
            m[lo:hi] = False
            w[m] = float("-inf")
        for t in p.suppressed:
            if 0 <= t < V:
                w[t] = float("-inf")
        if p.repetition_penalty != 1.0 or p.presence_penalty or p.frequency_penalty:
            hist = torch.tensor(p.history, dtype=torch.long)
            if hist.numel():
                uniq = torch.unique(hist[(hist >= 0) & (hist < V)])
                x = w[uniq]
                if p.repetition_penalty != 1.0:
                    x = torch.where(x > 0, x / p.repetition_penalty, x * p.repetition_penalty)
                gen = hist[p.num_prompt_tokens:]
                cnt = torch.bincount(gen[(gen >= 0) & (gen < V)], minlength=V)[uniq].float()
                x = x - (cnt > 0).float() * p.presence_penalty - cnt * p.frequency_penalty
                w[uniq] = x
        if p.temperature <= 0:
            i = int(torch.argmax(w))
            ids.append(i)
            lps.append(float(torch.log_softmax(w, 0)[i]))
            continue
        w = w / p.temperature
        lp = torch.log_softmax(w, 0)
        mx = w.max()
        cut = torch.tensor(float("-inf"))
        if p.min_p > 0:
            cut = torch.maximum(cut, mx + torch.log(torch.tensor(p.min_p)))
        if 0 < p.top_k < V:
            cut = torch.maximum(cut, torch.topk(w, p.top_k).values[-1])
        keep = w >= cut
        if p.top_p < 1.0:
            pr = torch.where(keep, torch.exp(w - mx), torch.zeros(()))
            srt, order = torch.sort(pr, descending=True)
            cum = torch.cumsum(srt, 0)
            n = int((cum < p.top_p * pr.sum()).sum()) + 1       # mass of what survived min-p / top-k
            k2 = torch.zeros(V, dtype=torch.bool)
            k2[order[:n]] = True
            keep &= k2
        pr = torch.where(keep, torch.exp(w - mx), torch.zeros(()))
        u = _uniform(p.seed, p.step) * float(pr.sum())
        cum = torch.cumsum(pr, 0)
        i = int(torch.searchsorted(cum, torch.tensor(u), right=True).clamp(max=V - 1))
        while pr[i] == 0 and i > 0:
            i -= 1
        ids.append(i)
        lps.append(float(lp[i]))
    return torch.tensor(ids, dtype=torch.long), torch.tensor(lps)


_work: dict = {}


def pack_rows(rows: list[RowParams]) -> torch.Tensor:
    """Row parameters as the byte tensor the kernel reads (host memory).  Rows that use penalties or
    suppression lists are not supported here (their side tables vary in size): plain temperature /
    top-k / top-p / min-p / seed / step rows only, which is what a captured sampling step needs."""
    arr = (_Row * len(rows))()
    for r, p in enumerate(rows):
        a = arr[r]
        if p.repetition_penalty != 1.0 or p.presence_penalty or p.frequency_penalty or p.suppressed:
            raise ValueError("pack_rows: penalties and suppression lists need sample()")
        a.temperature, a.top_p, a.min_p, a.top_k = p.temperature, p.top_p, p.min_p, int(p.top_k or 0)
        a.rep_penalty, a.presence_penalty, a.frequency_penalty = 1.0, 0.0, 0.0
        a.seed, a.step = int(p.seed) & 0xFFFFFFFFFFFFFFFF, int(p.step)
        a.range_lo, a.range_hi = p.allowed_range if p.allowed_range is not None else (0, 0)
    return torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8)


def row_bytes() -> int:
    return ctypes.sizeof(_Row)


def sample_packed(logits: torch.Tensor, rows_dev: torch.Tensor, out: torch.Tensor, work: torch.Tensor,
                  logprob: torch.Tensor | None = None) -> torch.Tensor:
    """Sampling on rows already packed on the device (``pack_rows(...).to(device)``): no host work and
    no allocation, so the call can be captured in a CUDA graph and the rows refreshed between replays.
    ``work``: fp32 [B, V] scratch; ``out``: int32 [B]."""
    B, V = logits.shape
    assert logits.is_cuda and logits.stride(1) == 1 and rows_dev.numel() >= B * row_bytes()
    rc = nv.lib("sampler").omni_sample(nv.ptr(logits), ctypes.c_int(1 if logits.dtype == torch.bfloat16 else 0),
                                       ctypes.c_long(logits.stride(0)), ctypes.c_int(V), ctypes.c_int(B), nv.ptr(rows_dev),
                                       nv.ptr(None), nv.ptr(None), nv.ptr(work), nv.ptr(None), nv.ptr(out),
                                       nv.ptr(logprob), nv.stream_ptr())
    nv.check_rc(rc, "omni_sample")
    return out


def sample(logits: torch.Tensor, rows: list[RowParams]):
    """logits [B, V] (fp32 or bf16).  Returns (ids int32 [B] on the logits' device, logprobs)."""
    if not logits.is_cuda:
        i, lp = sample_reference(logits, rows)
        return i.to(torch.int32), lp
    B, V = logits.shape
    assert logits.stride(1) == 1 and len(rows) == B
    arr = (_Row * B)()
    hist, sup = [], []
    need_cnt = False
    for r, p in enumerate(rows):
        a = arr[r]
        a.temperature, a.top_p, a.min_p, a.top_k = p.temperature, p.top_p, p.min_p, int(p.top_k or 0)
        a.rep_penalty, a.presence_penalty, a.frequency_penalty = p.repetition_penalty, p.presence_penalty, p.frequency_penalty
        a.seed, a.step = int(p.seed) & 0xFFFFFFFFFFFFFFFF, int(p.step)
        pen = p.repetition_penalty != 1.0 or p.presence_penalty != 0.0 or p.frequency_penalty != 0.0
        need_cnt |= pen
        a.hist_off, a.hist_len, a.gen_off = len(hist), (len(p.history) if pen else 0), p.num_prompt_tokens
        if pen:
            hist.extend(p.history)
        a.sup_off, a.sup_len = len(sup), len(p.suppressed)
        sup.extend(p.suppressed)
        a.range_lo, a.range_hi = p.allowed_range if p.allowed_range is not None else (0, 0)
    dev = logits.device
    rows_t = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8).to(dev)
    hist_t = torch.tensor(hist or [0], dtype=torch.int32, device=dev)
    sup_t = torch.tensor(sup or [0], dtype=torch.int32, device=dev)
    key = (dev.index, B, V)
    wk = _work.get(key)
    if wk is None:
        wk = [torch.empty(B, V, dtype=torch.float32, device=dev), None]
        _work[key] = wk
    if need_cnt and wk[1] is None:
        wk[1] = torch.empty(B, V, dtype=torch.int32, device=dev)
    out = torch.empty(B, dtype=torch.int32, device=dev)
    lp = torch.empty(B, dtype=torch.float32, device=dev)
    rc = nv.lib("sampler").omni_sample(nv.ptr(logits), ctypes.c_int(1 if logits.dtype == torch.bfloat16 else 0),
                                       ctypes.c_long(logits.stride(0)), ctypes.c_int(V), ctypes.c_int(B), nv.ptr(rows_t),
                                       nv.ptr(hist_t), nv.ptr(sup_t), nv.ptr(wk[0]), nv.ptr(wk[1] if need_cnt else None),
                                       nv.ptr(out), nv.ptr(lp), nv.stream_ptr())
    nv.check_rc(rc, "omni_sample")
    return out, lp
