"""Process groups for DiT parallelism: TP x SP(ulysses x ring) x PP x CFG x DP.

Rank layout follows the reference's order string "tp-sp-pp-cfg-dp"
(vllm_omni/diffusion/distributed/parallel_state.py:62-237, :624-775): tensor-parallel ranks
are adjacent, then sequence-parallel, pipeline, CFG and data-parallel.  Inside the SP
dimension Ulysses owns the contiguous (fast) sub-dimension and ring the strided one
(parallel_state.py:477-621).

One process per GPU.  Every group has an NCCL (device) communicator and a Gloo (CPU) twin
for object exchange and barriers; on CPU-only runs both are Gloo.  The fused kernels attach
their peer-memory windows to these groups (see ``peer_memory.py``).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from datetime import timedelta

import torch
import torch.distributed as dist

from .group_coordinator import GroupCoordinator, PipelineGroupCoordinator, SequenceParallelGroupCoordinator

ORDER = "tp-sp-pp-cfg-dp"


def generate_masked_orthogonal_rank_groups(world_size: int, parallel_size: list[int], mask: list[bool]):
    """All rank groups obtained by varying the masked dimensions and fixing the others.

    ``parallel_size`` lists the extent of every dimension, fastest-varying first.
    """
    def prefix_product(a, init=1):
        r = [init]
        for v in a:
            init *= v
            r.append(init)
        return r

    def decompose(index, shape):
        strides = prefix_product(shape)
        return [(index // s) % d for s, d in zip(strides, shape)]

    masked = [s for s, m in zip(parallel_size, mask) if m]
    unmasked = [s for s, m in zip(parallel_size, mask) if not m]
    global_stride = prefix_product(parallel_size)
    masked_stride = [d for d, m in zip(global_stride, mask) if m]
    unmasked_stride = [d for d, m in zip(global_stride, mask) if not m]
    group_size = prefix_product(masked)[-1]
    num_groups = world_size // group_size
    ranks = []
    for g in range(num_groups):
        gidx = decompose(g, unmasked)
        rank = []
        for r in range(group_size):
            ridx = decompose(r, masked)
            rank.append(sum(a * b for a, b in zip(ridx, masked_stride)) +
                        sum(a * b for a, b in zip(gidx, unmasked_stride)))
        ranks.append(rank)
    return ranks


class RankGenerator:
    def __init__(self, tp: int, sp: int, pp: int, cfg: int, dp: int, order: str = ORDER, rank_offset: int = 0):
        self.sizes = {"tp": tp, "sp": sp, "pp": pp, "cfg": cfg, "dp": dp}
        self.order = order.split("-")
        assert sorted(self.order) == sorted(self.sizes), f"bad order {order}"
        self.world_size = tp * sp * pp * cfg * dp
        self.ordered_size = [self.sizes[n] for n in self.order]
        self.rank_offset = rank_offset

    def get_ranks(self, token: str) -> list[list[int]]:
        """token: dash-joined dimension names, e.g. "sp" or "tp-sp"."""
        names = token.split("-")
        mask = [n in names for n in self.order]
        groups = generate_masked_orthogonal_rank_groups(self.world_size, self.ordered_size, mask)
        return [[r + self.rank_offset for r in g] for g in groups]


@dataclass
class _State:
    world: GroupCoordinator | None = None
    tp: GroupCoordinator | None = None
    sp: SequenceParallelGroupCoordinator | None = None
    pp: PipelineGroupCoordinator | None = None
    cfg: GroupCoordinator | None = None
    dp: GroupCoordinator | None = None
    vae: GroupCoordinator | None = None


_S = _State()


def init_distributed_environment(world_size: int = -1, rank: int = -1, distributed_init_method: str = "env://",
                                 local_rank: int = -1, backend: str | None = None, timeout_s: int | None = None):
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if not dist.is_initialized():
        kw = {}
        if timeout_s:
            kw["timeout"] = timedelta(seconds=timeout_s)
        if backend == "nccl" and local_rank >= 0:
            kw["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend=backend, init_method=distributed_init_method, world_size=world_size,
                                rank=rank, **kw)
    if local_rank < 0:
        local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if _S.world is None:
        ranks = list(range(dist.get_world_size()))
        _S.world = GroupCoordinator([ranks], local_rank, backend, name="world")
    return _S.world


def sp_subgroup_ranks(sp_ranks: list[int], ulysses: int, ring: int):
    """Split one SP group into its Ulysses groups (contiguous) and ring groups (strided)."""
    assert len(sp_ranks) == ulysses * ring
    uly = [sp_ranks[i * ulysses:(i + 1) * ulysses] for i in range(ring)]
    rng = [sp_ranks[i::ulysses] for i in range(ulysses)]
    return uly, rng


def initialize_model_parallel(data_parallel_size: int = 1, cfg_parallel_size: int = 1,
                              sequence_parallel_size: int | None = None, ulysses_degree: int = 1,
                              ring_degree: int = 1, tensor_parallel_size: int = 1, pipeline_parallel_size: int = 1,
                              vae_patch_parallel_size: int = 1, backend: str | None = None):
    assert dist.is_initialized(), "call init_distributed_environment first"
    world_size = dist.get_world_size()
    if sequence_parallel_size is None:
        sequence_parallel_size = ulysses_degree * ring_degree
    if sequence_parallel_size != ulysses_degree * ring_degree:
        raise ValueError("sequence_parallel_size must equal ulysses_degree * ring_degree")
    need = (data_parallel_size * cfg_parallel_size * sequence_parallel_size * tensor_parallel_size *
            pipeline_parallel_size)
    if world_size != need:
        raise RuntimeError(f"world_size ({world_size}) != dp {data_parallel_size} x cfg {cfg_parallel_size} x sp "
                           f"{sequence_parallel_size} x tp {tensor_parallel_size} x pp {pipeline_parallel_size}")
    backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
    local_rank = _S.world.local_rank if _S.world is not None else int(os.environ.get("LOCAL_RANK", "0"))
    rg = RankGenerator(tensor_parallel_size, sequence_parallel_size, pipeline_parallel_size, cfg_parallel_size,
                       data_parallel_size)
    _S.dp = GroupCoordinator(rg.get_ranks("dp"), local_rank, backend, name="dp")
    _S.cfg = GroupCoordinator(rg.get_ranks("cfg"), local_rank, backend, name="cfg")
    _S.pp = PipelineGroupCoordinator(rg.get_ranks("pp"), local_rank, backend, name="pp")
    _S.tp = GroupCoordinator(rg.get_ranks("tp"), local_rank, backend, name="tp")
    sp_groups = rg.get_ranks("sp")
    uly_all, ring_all = [], []
    for g in sp_groups:
        u, r = sp_subgroup_ranks(g, ulysses_degree, ring_degree)
        uly_all += u
        ring_all += r
    _S.sp = SequenceParallelGroupCoordinator(sp_groups, local_rank, backend, ulysses_groups=uly_all,
                                             ring_groups=ring_all, name="sp")
    # VAE patch parallelism reuses the first `vae_patch_parallel_size` ranks of the world
    vsz = max(1, min(vae_patch_parallel_size, world_size))
    vgroups = [list(range(i, i + vsz)) for i in range(0, world_size - world_size % vsz, vsz)]
    if world_size % vsz:
        vgroups.append(list(range(world_size - world_size % vsz, world_size)))
    _S.vae = GroupCoordinator(vgroups, local_rank, backend, name="vae")


def model_parallel_is_initialized() -> bool:
    return _S.tp is not None


def destroy_model_parallel():
    for n in ("tp", "sp", "pp", "cfg", "dp", "vae"):
        g = getattr(_S, n)
        if g is not None:
            g.destroy()
        setattr(_S, n, None)


def destroy_distributed_environment():
    destroy_model_parallel()
    if _S.world is not None:
        _S.world.destroy()
        _S.world = None
    if dist.is_initialized():
        dist.destroy_process_group()


def _get(name):
    g = getattr(_S, name)
    assert g is not None, f"{name} group is not initialized"
    return g


def get_world_group(): return _get("world")
def get_tp_group(): return _get("tp")
def get_sp_group(): return _get("sp")
def get_pp_group(): return _get("pp")
def get_cfg_group(): return _get("cfg")
def get_dp_group(): return _get("dp")
def get_vae_parallel_group(): return _get("vae")


def _ws(name): return getattr(_S, name).world_size if getattr(_S, name) is not None else 1
def _rk(name): return getattr(_S, name).rank_in_group if getattr(_S, name) is not None else 0


def get_tensor_model_parallel_world_size(): return _ws("tp")
def get_tensor_model_parallel_rank(): return _rk("tp")
def get_sequence_parallel_world_size(): return _ws("sp")
def get_sequence_parallel_rank(): return _rk("sp")
def get_ulysses_parallel_world_size(): return _S.sp.ulysses_world_size if _S.sp is not None else 1
def get_ulysses_parallel_rank(): return _S.sp.ulysses_rank if _S.sp is not None else 0
def get_ring_parallel_world_size(): return _S.sp.ring_world_size if _S.sp is not None else 1
def get_ring_parallel_rank(): return _S.sp.ring_rank if _S.sp is not None else 0
def get_classifier_free_guidance_world_size(): return _ws("cfg")
def get_classifier_free_guidance_rank(): return _rk("cfg")
def get_pipeline_parallel_world_size(): return _ws("pp")
def get_pipeline_parallel_rank(): return _rk("pp")
def get_data_parallel_world_size(): return _ws("dp")
def get_data_parallel_rank(): return _rk("dp")
