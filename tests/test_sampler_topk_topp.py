"""top-p combined with top-k / min-p: the nucleus is measured on the renormalised survivors
(top-k first, then top-p on what is left), as vLLM's sampler does."""
import pytest
import torch

from vllm_omni_b200.ops.sampler import RowParams, sample_reference


def _kept_set(logits, top_k, top_p, min_p=0.0):
    """Straight restatement: min-p mask, top-k mask, softmax over the survivors, sorted nucleus."""
    w = logits.clone().float()
    if min_p > 0:
        pr = torch.softmax(w, 0)
        w[pr < min_p * pr.max()] = float("-inf")
    if top_k:
        kth = torch.topk(w, top_k).values[-1]
        w[w < kth] = float("-inf")
    pr = torch.softmax(w, 0)
    srt, order = torch.sort(pr, descending=True)
    cum = torch.cumsum(srt, 0)
    n = int((cum < top_p).sum()) + 1
    return set(order[:n].tolist())


def test_top_p_is_measured_on_the_top_k_survivors_cpu():
    # 3 heavy tokens hold 60 % of the mass, a long flat tail the rest: with top_k=3 and top_p=0.5 the
    # nucleus must be cut inside the three survivors (the full-distribution reading keeps all three)
    logits = torch.cat([torch.tensor([3.0, 2.6, 2.2]), torch.full((200,), -1.1)])
    want = _kept_set(logits, 3, 0.5)
    assert want == {0, 1}
    seen = set()
    for step in range(300):
        ids, _ = sample_reference(logits[None], [RowParams(temperature=1.0, top_k=3, top_p=0.5, seed=9, step=step)])
        seen.add(int(ids[0]))
    assert seen == want


@pytest.mark.gpu
def test_top_k_top_p_min_p_kernel_matches_oracle():
    from vllm_omni_b200.ops.sampler import sample
    dev = torch.device("cuda")
    torch.manual_seed(3)
    V = 4096
    base = torch.randn(V) * 2.5
    cases = [(3, 0.5, 0.0), (20, 0.7, 0.0), (0, 0.8, 0.05), (50, 0.9, 0.02)]
    for top_k, top_p, min_p in cases:
        want = _kept_set(base, top_k, top_p, min_p)
        n = 400
        rows = [RowParams(temperature=1.0, top_k=top_k, top_p=top_p, min_p=min_p, seed=21, step=i) for i in range(n)]
        ids, _ = sample(base.to(dev)[None].repeat(n, 1), rows)
        ref_ids, _ = sample_reference(base[None].repeat(n, 1), rows)
        got = set(ids.tolist())
        assert got <= want, (top_k, top_p, min_p, sorted(got - want))
        assert (ids.cpu() == ref_ids).float().mean().item() > 0.97      # same draws up to fp rounding at the cut
