"""CUDA-graph replay of the AR decode step.

A decode-only engine step (one new token per running request) is launch-bound: a 48-layer MoE
decoder issues several hundred small kernels per step.  ``DecodeGraphRunner`` keeps, per batch-size
bucket, a set of STATIC input tensors (token ids / embedding overlay, positions, slot mapping,
block tables, sequence lengths), copies each step's values into them, and replays one captured
graph of ``decoder.forward`` on them.  Rows beyond the live batch repeat row 0 with slot -1 (the
KV write skips them), so a bucket never computes on undefined data.

The reference gets the same effect from vLLM's CUDA-graph runner plus dedicated buffers for the
talker's multi-token step (vllm_omni/worker/gpu_model_runner.py:71-89, 1085-1112).

Off the GPU (or with ``use_graph=False``) the runner executes the same static-buffer step eagerly,
which is how the host-side logic is tested.  On a GPU the runner is on by default
(``OMNI_AR_CUDA_GRAPH=0`` switches it off).
"""
from __future__ import annotations

import torch

from ..models.qwen_decoder import ModelBatch

DEFAULT_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)


class _Bucket:
    def __init__(self, n, D, max_blocks, mrope, dtype, device):
        z = lambda *s, dt=torch.long: torch.zeros(*s, dtype=dt, device=device)
        self.n = n
        self.ids = z(n)
        self.pos = z(3, n) if mrope else z(n)
        self.slots = torch.full((n,), -1, dtype=torch.int32, device=device)
        self.tables = z(n, max_blocks, dt=torch.int32)
        self.lens = torch.ones(n, dtype=torch.int32, device=device)
        self.embeds = z(n, D, dt=dtype)
        self.emask = z(n, dt=torch.bool)
        self.rows = torch.arange(n, dtype=torch.long, device=device)
        self.graph = None
        self.hidden = None
        self.captured: dict = {}
        self.warm = False

    def batch(self) -> ModelBatch:
        return ModelBatch(self.ids, self.pos, self.slots, [], decode_rows=self.rows, decode_block_tables=self.tables,
                          decode_seq_lens=self.lens, input_embeds=self.embeds, embeds_mask=self.emask)


class DecodeGraphRunner:
    def __init__(self, decoder, kv_caches, max_blocks: int, capture_layers=(), buckets=DEFAULT_BUCKETS,
                 use_graph: bool | None = None):
        self.decoder, self.kv_caches, self.max_blocks = decoder, kv_caches, max_blocks
        self.capture_layers = tuple(capture_layers)
        self.buckets = tuple(sorted(buckets))
        dev = decoder.embed_tokens.device
        self.device, self.dtype = dev, decoder.embed_tokens.dtype
        self.use_graph = (dev.type == "cuda") if use_graph is None else bool(use_graph and dev.type == "cuda")
        self._state: dict[int, _Bucket] = {}
        self.replays = 0

    def supports(self, batch: ModelBatch) -> bool:
        """Decode-only batches whose block tables fit the static width."""
        if batch.prefills or batch.decode_rows is None:
            return False
        n = int(batch.decode_rows.numel())
        return (n == batch.input_ids.shape[0] and 0 < n <= self.buckets[-1]
                and batch.decode_block_tables.shape[1] <= self.max_blocks)

    def _bucket(self, n: int) -> _Bucket:
        size = next(b for b in self.buckets if b >= n)
        st = self._state.get(size)
        if st is None:
            cfg = self.decoder.cfg
            st = _Bucket(size, cfg.hidden_size, self.max_blocks, cfg.mrope_section is not None, self.dtype, self.device)
            self._state[size] = st
        return st

    def _fill(self, st: _Bucket, b: ModelBatch) -> int:
        n = int(b.decode_rows.numel())
        order = b.decode_rows                      # rows of the step's batch in decode order (identity here)
        pad = st.n - n

        def put(dst, src, dim=0):
            src = src.index_select(dim, order) if order is not None else src
            if dim == 0:
                dst[:n].copy_(src)
                if pad:
                    dst[n:].copy_(src[:1].expand(pad, *src.shape[1:]))
            else:
                dst[:, :n].copy_(src)
                if pad:
                    dst[:, n:].copy_(src[:, :1].expand(-1, pad))
        put(st.ids, b.input_ids)
        pos = b.positions
        if st.pos.dim() == 2 and pos.dim() == 1:
            pos = pos[None].expand(3, -1)
        put(st.pos, pos, dim=pos.dim() - 1)
        st.slots[:n].copy_(b.slot_mapping.index_select(0, order))
        if pad:
            st.slots[n:].fill_(-1)                 # padding rows never write the cache
        w = b.decode_block_tables.shape[1]
        st.tables.zero_()
        st.tables[:n, :w].copy_(b.decode_block_tables)
        st.lens[:n].copy_(b.decode_seq_lens)
        if pad:
            st.tables[n:].copy_(st.tables[:1].expand(pad, -1))
            st.lens[n:].copy_(st.lens[:1].expand(pad))
        if b.input_embeds is not None:
            put(st.embeds, b.input_embeds.to(st.embeds.dtype))
            put(st.emask, b.embeds_mask if b.embeds_mask is not None else torch.ones_like(order, dtype=torch.bool))
        else:
            st.emask.zero_()
        return n

    def _step(self, st: _Bucket):
        st.hidden, st.captured = self.decoder(st.batch(), self.kv_caches, capture_layers=self.capture_layers)

    @torch.no_grad()
    def run(self, batch: ModelBatch):
        """Returns (hidden [n, D], captured layers) for a batch that ``supports`` accepted."""
        st = self._bucket(int(batch.decode_rows.numel()))
        n = self._fill(st, batch)
        if not self.use_graph:
            self._step(st)
        elif st.graph is None:
            if not st.warm:                        # first use: allocate scratch / workspaces outside the capture
                self._step(st)
                st.warm = True
                torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            try:
                with torch.cuda.graph(g, capture_error_mode="thread_local"):   # other stages' threads keep issuing CUDA calls
                    self._step(st)
            except Exception as e:   # noqa: BLE001  (a step that cannot be captured runs eagerly from here on)
                import logging
                logging.getLogger(__name__).warning("decode step not capturable (%s); running it eagerly", e)
                self.use_graph = False
                torch.cuda.synchronize(self.device)
                self._step(st)
            else:
                st.graph = g
                g.replay()
        else:
            st.graph.replay()
        self.replays += 1
        return st.hidden[:n], {k: v[:n] for k, v in st.captured.items()}
