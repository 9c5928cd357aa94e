"""The declarative sequence-parallel plan installed at load (``parallel/apply.install_sp_plan``):
a transformer that does not shard rows itself (``sp_hooks = True``, the custom-pipeline case) gets
split / gather hooks and an SP attention object; two Gloo ranks reproduce the single-rank output.
Malformed plans are refused at load."""
import pytest
import torch
from torch import nn

from dist_utils import run_distributed


class _Cfg:
    num_attention_heads, attention_head_dim = 4, 16


class HookedTransformer(nn.Module):
    """Rows in, rows out; attention through ``self.sp`` when the sequence is sharded."""
    from vllm_omni_b200.parallel.sp_plan import SequenceParallelInput, SequenceParallelOutput
    sp_style, sp_hooks = "attention", True
    _sp_plan = {"": {"hidden_states": SequenceParallelInput(split_dim=1, expected_dims=3, auto_pad=False)},
                "proj_out": SequenceParallelOutput(gather_dim=1, expected_dims=3)}

    def __init__(self):
        super().__init__()
        self.cfg = _Cfg()
        torch.manual_seed(0)
        self.qkv = nn.Linear(64, 192)
        self.proj_out = nn.Linear(64, 8)
        self.sp = None

    def forward(self, hidden_states):
        from vllm_omni_b200.ops.attention import attention
        B, S, _ = hidden_states.shape
        q5 = self.qkv(hidden_states).view(B, S, 3, 4, 16)
        if self.sp is not None:
            o = self.sp(q5)
        else:
            o = attention(q5[:, :, 0], q5[:, :, 1], q5[:, :, 2])
        return self.proj_out(o.reshape(B, S, 64) + hidden_states)


class _Pipe:
    def __init__(self):
        self.transformer = HookedTransformer()
        self.cfg_exchange = None


def _worker(rank, world):
    from vllm_omni_b200.diffusion.data import DiffusionParallelConfig, OmniDiffusionConfig
    from vllm_omni_b200.parallel import parallel_state as ps
    from vllm_omni_b200.parallel.apply import apply_parallelism
    ps.init_distributed_environment(world, rank, local_rank=rank, backend="gloo")
    ps.initialize_model_parallel(sequence_parallel_size=world, ulysses_degree=world, backend="gloo")
    pipe = _Pipe()
    x = torch.randn(2, 12, 64, generator=torch.Generator().manual_seed(3))
    torch.set_grad_enabled(False)                         # inference, as the workers run
    ref = pipe.transformer(hidden_states=x)
    od = OmniDiffusionConfig(parallel_config=DiffusionParallelConfig(ulysses_degree=world))
    apply_parallelism(pipe, od)
    assert pipe.transformer._sp_hook_registry is not None and pipe.transformer.sp is not None
    got = pipe.transformer(hidden_states=x)               # full rows in: the hooks split and gather
    assert got.shape == ref.shape
    assert torch.allclose(got, ref, atol=1e-5), (got - ref).abs().max()


def test_hooked_transformer_two_ranks_matches_single():
    run_distributed(_worker, 2, "gloo")


def test_malformed_plan_is_refused_at_load():
    from vllm_omni_b200.parallel.apply import install_sp_plan

    class Bad(nn.Module):
        _sp_plan = {"hidden_states": {"split_dim": 1}}
    with pytest.raises(TypeError):
        install_sp_plan(Bad(), None)


def test_builtin_plans_validate():
    from vllm_omni_b200.diffusion.models.qwen_image.transformer import QwenImageTransformer2DModel
    from vllm_omni_b200.diffusion.models.z_image.transformer import ZImageTransformer2DModel
    from vllm_omni_b200.parallel.sp_plan import validate_sp_plan
    validate_sp_plan(QwenImageTransformer2DModel._sp_plan)
    validate_sp_plan(ZImageTransformer2DModel._sp_plan)
