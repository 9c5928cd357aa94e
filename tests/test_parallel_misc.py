"""Rank-group construction, SP plan hooks, VAE tile planning/blending, TP sharding (CPU)."""
import pytest
import torch
from torch import nn

from vllm_omni_b200.parallel.parallel_state import RankGenerator, sp_subgroup_ranks
from vllm_omni_b200.parallel.sp_plan import (SequenceParallelInput, SequenceParallelOutput, apply_sp_plan, sp_gather,
                                             sp_shard, validate_sp_plan)
from vllm_omni_b200.parallel.tensor_parallel import shard_cols, shard_rows
from vllm_omni_b200.parallel.vae_patch_parallel import blend_tiles, plan_tiles


def test_rank_groups_cover_world_once():
    rg = RankGenerator(tp=2, sp=2, pp=1, cfg=2, dp=1)
    for tok in ("tp", "sp", "cfg", "dp", "pp"):
        flat = sorted(r for g in rg.get_ranks(tok) for r in g)
        assert flat == list(range(8)), tok
    assert rg.get_ranks("tp")[0] == [0, 1] and rg.get_ranks("sp")[0] == [0, 2] and rg.get_ranks("cfg")[0] == [0, 4]
    for rank in range(8):       # every rank sits in exactly one Ulysses and one ring group
        sp = next(g for g in RankGenerator(1, 8, 1, 1, 1).get_ranks("sp") if rank in g)
        uly, ring = sp_subgroup_ranks(sp, 4, 2)
        assert sum(rank in g for g in uly) == 1 and sum(rank in g for g in ring) == 1
    uly, ring = sp_subgroup_ranks(list(range(8)), 4, 2)
    assert uly == [[0, 1, 2, 3], [4, 5, 6, 7]] and ring == [[0, 4], [1, 5], [2, 6], [3, 7]]


def test_sp_plan_shard_pad_gather_simulated():
    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.proj_out = nn.Identity()

        def forward(self, hidden_states=None):
            return self.proj_out(hidden_states * 2)
    plan = {"": {"hidden_states": SequenceParallelInput(split_dim=1, expected_dims=3, auto_pad=True)},
            "proj_out": SequenceParallelOutput(gather_dim=1)}
    validate_sp_plan(plan)
    x = torch.randn(2, 10, 4)
    world = 4
    shards = []
    for r in range(world):
        net = Net()
        reg = apply_sp_plan(net, plan, group=None, rank=r, world=world)
        shards.append(net(hidden_states=x))
        assert reg.state["pad"] == 2 and shards[-1].shape == (2, 3, 4)
        reg.remove()
    full = torch.cat(shards, dim=1)[:, :10]
    assert torch.allclose(full, x * 2)
    with pytest.raises(ValueError):
        sp_shard(x, 1, 0, 4, auto_pad=False)
    with pytest.raises(TypeError):
        validate_sp_plan({"a": 3})
    assert sp_gather(x, 1, None).shape == x.shape


def test_tiles_cover_and_blend_is_identity_for_constant_tiles():
    tiles = plan_tiles(100, 70, 32, 8)
    cover = torch.zeros(100, 70)
    for t in tiles:
        cover[t.y0:t.y1, t.x0:t.x1] += 1
        assert t.y1 - t.y0 <= 32 and t.x1 - t.x0 <= 32
    assert (cover > 0).all()
    dec = [(t, torch.full((1, 3, (t.y1 - t.y0) * 2, (t.x1 - t.x0) * 2), 0.25)) for t in tiles]
    img = blend_tiles(dec, 200, 140, 2, 16)
    assert torch.allclose(img, torch.full_like(img, 0.25), atol=1e-6)


def test_tp_shards_recompose():
    w = torch.arange(24 * 8, dtype=torch.float32).view(24, 8)
    parts = [shard_rows(w, r, 2, groups=3) for r in range(2)]
    # q|k|v each split in two: rank 0 gets the first half of every part
    assert torch.equal(parts[0], torch.cat([w[0:4], w[8:12], w[16:20]]))
    x = torch.randn(5, 8)
    cols = [shard_cols(w, r, 2) for r in range(2)]
    y = sum(x[:, r * 4:(r + 1) * 4] @ cols[r].t() for r in range(2))
    assert torch.allclose(y, x @ w.t(), atol=1e-4)
