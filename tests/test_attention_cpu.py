"""CPU restatement of the attention continuation (``merge_prev``): two key sets combined by their
log-sum-exps equal one attention over both; key sets that contribute nothing drop out."""
import torch

from vllm_omni_b200.ops.attention import attention, attention_reference, merge_partials


def test_merge_prev_equals_attention_over_both_key_sets():
    torch.manual_seed(0)
    B, Sq, H, Hkv, D = 2, 7, 4, 2, 16
    q = torch.randn(B, Sq, H, D)
    ka, va, kb, vb = (torch.randn(B, n, Hkv, D) for n in (5, 5, 9, 9))
    lens_b = torch.tensor([9, 4], dtype=torch.int32)
    o, lse = attention(q, ka, va, return_lse=True)
    o2, lse2 = attention(q, kb, vb, kv_lens=lens_b, merge_prev=(o, lse), return_lse=True)
    for b in range(B):
        n = int(lens_b[b])
        ref, ref_lse = attention_reference(q[b:b + 1], torch.cat([ka[b:b + 1], kb[b:b + 1, :n]], 1),
                                           torch.cat([va[b:b + 1], vb[b:b + 1, :n]], 1), return_lse=True)
        assert torch.allclose(o2[b:b + 1], ref, atol=1e-5) and torch.allclose(lse2[b:b + 1], ref_lse, atol=1e-5)


def test_empty_partials_drop_out():
    o_a, o_b = torch.randn(1, 3, 2, 4), torch.randn(1, 3, 2, 4)
    lse = torch.randn(1, 2, 3)
    ninf = torch.full((1, 2, 3), float("-inf"))
    o, l = merge_partials(o_a, lse, o_b, ninf)
    assert torch.equal(o, o_a) and torch.equal(l, lse)
    o, l = merge_partials(o_a, ninf, o_b, lse)
    assert torch.equal(o, o_b) and torch.equal(l, lse)
    o, l = merge_partials(o_a, ninf, o_b, ninf)
    assert torch.isfinite(o).all() and torch.isinf(l).all()
