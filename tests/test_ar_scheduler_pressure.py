"""AR scheduler under KV-page pressure: recompute preemption and KV hand-off page accounting.

Preemption drops a request's pages and puts it back at the head of the queue; when it is admitted
again every token it owns (prompt and the ones already generated) is fed again and the next token
is sampled only after the last of them, so greedy output equals a run with plenty of pages."""
import pytest
import torch

from vllm_omni_b200.engine.kv_cache_manager import KVCacheManager
from vllm_omni_b200.engine.request import Request, RequestStatus
from vllm_omni_b200.engine.scheduler import OmniARScheduler
from vllm_omni_b200.inputs import SamplingParams


def _req(i, n_prompt, max_tokens):
    return Request(f"r{i}", list(range(10 + i, 10 + i + n_prompt)),
                   SamplingParams(temperature=0.0, max_tokens=max_tokens, detokenize=False, ignore_eos=True))


def _check_step(sched_out, kv, block_size):
    """Every scheduled entry owns the pages of the positions it writes; nobody shares a page; no duplicates."""
    ids = [s.request.request_id for s in sched_out.scheduled]
    assert len(ids) == len(set(ids)), f"request scheduled twice in one step: {ids}"
    owner = {}
    for s in sched_out.scheduled:
        r = s.request
        assert r.status == RequestStatus.RUNNING
        need = (s.start + s.num_new_tokens + block_size - 1) // block_size
        assert len(r.block_ids) >= need, (r.request_id, s.start, s.num_new_tokens, r.block_ids)
        kv.slot_mapping(r, s.start, s.num_new_tokens)          # raises if a page is missing
        for b in r.block_ids:
            assert owner.setdefault(b, r.request_id) == r.request_id, f"page {b} shared"


def _drive(num_blocks, block_size, n_req=3, n_prompt=6, max_tokens=8):
    """Runs the scheduler with a fake model (next token = f(all tokens so far)) and returns outputs."""
    kv = KVCacheManager(num_blocks, block_size)
    sch = OmniARScheduler(kv, max_num_seqs=8, max_num_batched_tokens=64)
    reqs = [_req(i, n_prompt, max_tokens) for i in range(n_req)]
    for r in reqs:
        sch.add_request(r)
    waiting_twice = False
    for _ in range(400):
        if not sch.has_unfinished():
            break
        out = sch.schedule()
        _check_step(out, kv, block_size)
        waiting_twice |= len({id(r) for r in sch.waiting}) != len(sch.waiting)
        sampled = {}
        for s in out.scheduled:
            if s.samples:
                toks = s.request.all_token_ids[: s.start + s.num_new_tokens]
                assert len(toks) == s.request.num_tokens, "sampling before every owned token is in the cache"
                sampled[s.request.request_id] = (sum(toks) * 31 + len(toks)) % 997
        sch.update_from_output(out, sampled)
    assert not sch.has_unfinished()
    assert not waiting_twice
    assert kv.pool.num_free == num_blocks
    return [list(r.output_token_ids) for r in reqs]


def test_preemption_under_page_pressure_keeps_pages_exclusive_and_output_unchanged():
    relaxed = _drive(num_blocks=64, block_size=4)
    tight = _drive(num_blocks=6, block_size=4)
    assert tight == relaxed
    assert all(len(o) == 8 for o in tight)


@pytest.mark.parametrize("blocks", [5, 7, 9])
def test_preemption_other_pool_sizes(blocks):
    assert _drive(num_blocks=blocks, block_size=4, n_req=4, n_prompt=5, max_tokens=6) == \
        _drive(num_blocks=64, block_size=4, n_req=4, n_prompt=5, max_tokens=6)


def test_engine_greedy_tokens_survive_preemption():
    """Through the real model runner: a pool that forces preemption gives the same greedy tokens."""
    from vllm_omni_b200.entrypoints.omni_llm import OmniLLM
    prompts = [{"prompt_token_ids": [506, 509, 11, 12, 507, 506, 510, 13]},
               {"prompt_token_ids": [506, 509, 20, 507, 506, 510]},
               {"prompt_token_ids": [506, 509, 33, 34, 35, 507, 506, 510]}]
    sp = SamplingParams(temperature=0.0, max_tokens=10, detokenize=False, ignore_eos=True)

    def run(nblk):
        torch.manual_seed(0)
        llm = OmniLLM(None, model_arch="Qwen3ForCausalLM", device="cpu", num_gpu_blocks=nblk, block_size=4,
                      model_overrides={"tiny": True})
        outs = llm.generate(prompts, sp)
        assert llm.engine.kv.pool.num_free == nblk
        return [list(o.outputs[0].token_ids) for o in outs]
    assert run(9) == run(128)


def test_prefill_finished_handoff_frees_pages_when_request_ends_later():
    kv = KVCacheManager(8, 4)
    sch = OmniARScheduler(kv, kv_transfer_criteria={"type": "prefill_finished"})
    r = _req(0, 6, 5)
    sch.add_request(r)
    handed = False
    for _ in range(40):
        if not sch.has_unfinished():
            break
        out = sch.schedule()
        sampled = {s.request.request_id: 7 for s in out.scheduled if s.samples}
        sch.update_from_output(out, sampled)
        if out.kv_transfer_ids:
            handed = True
            assert not r.is_finished()                    # still decoding when the KV goes out
            sch.update_from_output(type(out)(), {}, list(out.kv_transfer_ids))
    assert handed and r.is_finished()
    assert not sch.waiting_for_kv_extract
    assert kv.pool.num_free == 8
