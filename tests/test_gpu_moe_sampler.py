"""MoE (route / plan / dispatch / grouped GEMM / combine) and the sampler kernel vs PyTorch."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("padded", ["0", "1"])
@pytest.mark.parametrize("T,E,k", [(37, 16, 4), (700, 8, 2), (5, 16, 2)])
def test_moe_forward_matches_reference(monkeypatch, padded, T, E, k):
    """Both row layouts (experts' rows back to back: the default; padded to 128 per expert), experts with
    more than one M tile of rows, and batches smaller than the number of experts."""
    from vllm_omni_b200.ops.moe import MoEWorkspace, moe_forward
    from vllm_omni_b200.ops import gemm, _native as nv
    monkeypatch.setenv("OMNI_MOE_PADDED", padded)
    dev = torch.device("cuda")
    torch.manual_seed(0)
    D, Fd = 256, 128
    x = torch.randn(T, D, device=dev, dtype=torch.bfloat16)
    rw = torch.randn(E, D, device=dev, dtype=torch.bfloat16) * 0.1
    w13 = torch.randn(E, 2 * Fd, D, device=dev, dtype=torch.bfloat16) * 0.05
    w2 = torch.randn(E, D, Fd, device=dev, dtype=torch.bfloat16) * 0.05
    logits = gemm.linear(x, rw)
    ws = MoEWorkspace()
    y = moe_forward(x, logits, w13, w2, k, ws=ws).float()
    torch.cuda.synchronize()
    assert int(nv.status_word(dev).item()) == 0
    # routing: the picked probabilities are the k largest (the choice among exactly tied bf16
    # logits is free, so compare values, not ids) and the weights are renormalised
    import torch.nn.functional as F
    ids, w = ws.ids.cpu().long(), ws.weights.cpu()
    p = torch.softmax(logits.cpu().float(), -1)
    ref_w, _ = torch.topk(p, k, -1)
    got = torch.gather(p, 1, ids)
    assert (got.sort(-1, descending=True).values - ref_w).abs().max().item() < 1e-5
    assert (w - got / got.sum(-1, keepdim=True)).abs().max().item() < 1e-4
    assert all(len(set(r.tolist())) == k for r in ids)
    # expert compute and combine against a dense fp32 restatement on the SAME routing
    xc, w13c, w2c = x.cpu().float(), w13.cpu().float(), w2.cpu().float()
    ref = torch.zeros(T, D)
    for t in range(T):
        for j in range(k):
            e = int(ids[t, j])
            h = F.linear(xc[t], w13c[e])
            h = (F.silu(h[:Fd]) * h[Fd:]).bfloat16().float()
            ref[t] += w[t, j] * F.linear(h, w2c[e])
    err = (y.cpu() - ref).abs().max().item()
    assert err < 0.05 * max(1.0, ref.abs().max().item()), f"moe max abs err {err} (ref max {ref.abs().max().item()})"
    # expert-parallel halves sum to the whole
    h = E // 2
    a = moe_forward(x, logits, w13[:h].contiguous(), w2[:h].contiguous(), k, e_lo=0, e_hi=h).float()
    b = moe_forward(x, logits, w13[h:].contiguous(), w2[h:].contiguous(), k, e_lo=h, e_hi=E).float()
    assert ((a + b) - y).abs().max().item() < 0.05
    torch.cuda.synchronize()
    assert int(nv.status_word(dev).item()) == 0


def test_sampler_greedy_topk_topp_and_masks():
    from vllm_omni_b200.ops.sampler import RowParams, sample
    dev = torch.device("cuda")
    torch.manual_seed(1)
    B, V = 6, 151936
    logits = torch.randn(B, V, device=dev) * 3
    rows = [RowParams(temperature=0.0),
            RowParams(temperature=0.0, suppressed=[int(logits[1].argmax())]),
            RowParams(temperature=0.0, allowed_range=(1000, 2000)),
            RowParams(temperature=1.0, top_k=1, seed=3),
            RowParams(temperature=0.8, top_k=50, top_p=0.9, seed=5, step=2),
            RowParams(temperature=0.0, repetition_penalty=1e4, history=[int(logits[5].argmax())], num_prompt_tokens=0)]
    ids, lp = sample(logits, rows)
    ids = ids.tolist()
    assert ids[0] == int(logits[0].argmax())
    l1 = logits[1].clone(); l1[int(logits[1].argmax())] = float("-inf")
    assert ids[1] == int(l1.argmax())
    assert 1000 <= ids[2] < 2000 and ids[2] == 1000 + int(logits[2, 1000:2000].argmax())
    assert ids[3] == int(logits[3].argmax())
    top50 = set(torch.topk(logits[4], 50).indices.tolist())
    assert ids[4] in top50
    assert ids[5] != int(logits[5].argmax())            # the repeated token was pushed down
    assert torch.isfinite(lp).all()
    # sampling frequencies follow the distribution (top-k=4 -> 4 outcomes)
    small = torch.tensor([[2.0, 1.0, 0.0, -1.0] + [-30.0] * 60], device=dev).repeat(2000, 1)
    ids, _ = sample(small, [RowParams(temperature=1.0, top_k=4, seed=11, step=i) for i in range(2000)])
    freq = torch.bincount(ids.long().cpu(), minlength=4)[:4].float() / 2000
    ref = torch.softmax(torch.tensor([2.0, 1.0, 0.0, -1.0]), 0)
    assert (freq - ref).abs().max().item() < 0.05
