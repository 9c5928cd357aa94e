"""CUDA-graph replay of a denoiser's forward for every model that has no step loop of its own.

The reference gets launch-overhead relief from regional ``torch.compile``
(vllm_omni/diffusion/compile.py, ``enforce_eager`` in vllm_omni/diffusion/data.py); here a forward
that is called with the same signature at every denoising step (tensor shapes, dtypes and strides,
plus the plain values of the other arguments) is captured into a CUDA graph on its second use and
replayed afterwards: inputs are copied into the static tensors the capture ran on, the output is the
capture's static output (valid until the next call with the same signature).

A model opts in with the class attribute ``graph_safe_forward = True`` (its forward keeps no state
between calls of one signature).  Only forwards whose arguments are tensors, ``None``, numbers, strings, or (nested) tuples / lists of
those are graphed; anything else runs eagerly.  Small host tensors among the arguments (position ids) count
by value.  Qwen-Image keeps its own captured loop
(``prepare_loop`` / ``forward_step``).
"""
from __future__ import annotations

import logging
import os

import torch

log = logging.getLogger(__name__)
total_replays = 0                 # over all wrappers of the process (tests, statistics)
_SIMPLE = (type(None), bool, int, float, str)


_CONSTS: dict = {}


def device_constant(values, dtype, device) -> torch.Tensor:
    """A small device tensor holding ``values`` (a flat sequence of numbers), created once per
    (values, dtype, device) and kept for the life of the process.  A forward that builds such tensors from
    Python numbers at every call (key lengths, position offsets) copies host memory to the device, which a
    stream capture refuses; taking them from here makes the eager warm-up call create them and the captured
    call reuse them.  Entries are never dropped (a captured graph may read them); past 512 entries new ones
    are built uncached."""
    key = (tuple(values), dtype, str(device))
    t = _CONSTS.get(key)
    if t is None:
        t = torch.tensor(list(values), dtype=dtype, device=device)
        if len(_CONSTS) < 512:
            _CONSTS[key] = t
    return t


def _sig(x):
    if isinstance(x, torch.Tensor):
        if x.is_cuda:
            return ("T", tuple(x.shape), x.dtype, tuple(x.stride()), str(x.device))
        if x.numel() > (1 << 20):
            raise TypeError("large host tensor")
        # host tensors (position ids, small tables) are part of the signature by VALUE: the captured call saw
        # these exact numbers, so a call with other numbers is another entry
        raw = x.detach().contiguous().reshape(-1).view(torch.uint8).numpy().tobytes()
        return ("C", tuple(x.shape), x.dtype, hash(raw))
    if isinstance(x, _SIMPLE):
        return ("V", x)
    if isinstance(x, (tuple, list)):
        return ("L", type(x).__name__, tuple(_sig(v) for v in x))
    if isinstance(x, dict):
        return ("D", tuple((k, _sig(v)) for k, v in sorted(x.items())))
    raise TypeError(type(x).__name__)


def _map(x, fn):
    if isinstance(x, torch.Tensor):
        return fn(x)
    if isinstance(x, (tuple, list)):
        return type(x)(_map(v, fn) for v in x)
    if isinstance(x, dict):
        return {k: _map(v, fn) for k, v in x.items()}
    return x


def _copy_in(dst, src):
    if isinstance(dst, torch.Tensor):
        if dst.is_cuda:
            dst.copy_(src)
    elif isinstance(dst, (tuple, list)):
        for d, s in zip(dst, src):
            _copy_in(d, s)
    elif isinstance(dst, dict):
        for k in dst:
            _copy_in(dst[k], src[k])


class _Entry:
    __slots__ = ("calls", "graph", "args", "kwargs", "out")

    def __init__(self):
        self.calls, self.graph, self.args, self.kwargs, self.out = 0, None, None, None, None


class GraphedForward:
    def __init__(self, fn, warmup: int = 1, max_entries: int = 8, enabled=lambda: True):
        self.fn, self.warmup, self.max_entries, self.enabled = fn, warmup, max_entries, enabled
        self.entries: dict = {}
        self.replays = 0
        self.broken = False

    def _eager(self, args, kwargs):
        return self.fn(*args, **kwargs)

    @torch.no_grad()
    def __call__(self, *args, **kwargs):
        if self.broken or not self.enabled():
            return self._eager(args, kwargs)
        try:
            key = (_sig(args), _sig(kwargs))
        except TypeError:
            return self._eager(args, kwargs)
        tens = [t for t in _flatten((args, kwargs)) if isinstance(t, torch.Tensor)]
        if not any(t.is_cuda for t in tens):
            return self._eager(args, kwargs)
        ent = self.entries.get(key)
        if ent is None:
            if len(self.entries) >= self.max_entries:
                return self._eager(args, kwargs)
            ent = self.entries[key] = _Entry()
        if ent.graph is None:
            if ent.calls < self.warmup:
                ent.calls += 1
                return self._eager(args, kwargs)       # eager first: lazy tables, workspaces, function attributes
            own = lambda t: t.clone() if t.is_cuda else t          # host tensors are fixed by the signature
            ent.args, ent.kwargs = _map(args, own), _map(kwargs, own)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            try:
                with torch.cuda.graph(g, capture_error_mode="thread_local"):
                    ent.out = self.fn(*ent.args, **ent.kwargs)
            except Exception as e:   # noqa: BLE001  (a forward that cannot be captured keeps running eagerly)
                log.warning("forward not capturable (%s); running it eagerly", e)
                self.broken = True
                torch.cuda.synchronize()
                return self._eager(args, kwargs)
            ent.graph = g
        else:
            _copy_in(ent.args, args)
            _copy_in(ent.kwargs, kwargs)
        global total_replays
        ent.graph.replay()
        self.replays += 1
        total_replays += 1
        return ent.out


def _flatten(x):
    if isinstance(x, (tuple, list)):
        for v in x:
            yield from _flatten(v)
    elif isinstance(x, dict):
        for v in x.values():
            yield from _flatten(v)
    else:
        yield x


def maybe_graph_transformer(pipe, od_config) -> bool:
    """Wrap ``pipe.transformer.forward`` when the step is safe to capture: a GPU run without
    ``enforce_eager``, no cache hook that decides on the host, no sequence / tensor parallel exchange
    made of library calls.  ``OMNI_DIT_CUDA_GRAPH=0`` switches it off."""
    tr = getattr(pipe, "transformer", None)
    if tr is None or getattr(od_config, "enforce_eager", False) or os.environ.get("OMNI_DIT_CUDA_GRAPH", "1") == "0":
        return False
    if not getattr(tr, "graph_safe_forward", False):
        return False                                  # forwards that keep state between calls (condition-image K/V caches ...)
    if hasattr(pipe, "_loop_state") or isinstance(getattr(tr, "forward", None), GraphedForward):
        return False                                  # the pipeline drives a captured loop of its own / already wrapped
    try:
        dev = next(tr.parameters()).device
    except StopIteration:
        return False
    if dev.type != "cuda":
        return False

    def enabled():
        return (getattr(tr, "sp", None) is None and getattr(tr, "tp_group", None) is None
                and not getattr(tr, "tp_heads", 0) and getattr(tr, "stack_hook", None) is None
                and getattr(tr, "block_hook", None) is None and not getattr(tr, "_lora_active", False))
    tr.forward = GraphedForward(tr.forward, enabled=enabled)
    return True
