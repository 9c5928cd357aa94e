"""The allocation-free rel-L1 entry point against the general one.

Some users of the library cannot allocate device memory when they need the TeaCache
metric (no PyTorch allocator in a plain C host, or a memory budget that is already fully
committed), so ``omni_rel_l1_noalloc`` keeps its partial sums in a static device array.
This test calls it through its exported C symbol, twice in a row on different data, and
checks each result against ``omni_rel_l1`` given caller-owned scratch.  It is collected
last so that a failure here cannot hide the outcome of any other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _raw_lib():
    from vllm_omni_b200.build import lib_path
    lib = ctypes.CDLL(str(lib_path("elementwise")))
    lib.omni_rel_l1_noalloc.restype = ctypes.c_int
    lib.omni_rel_l1_noalloc_max_elems.restype = ctypes.c_long
    lib.omni_rel_l1_noalloc_strerror.restype = ctypes.c_char_p
    lib.omni_rel_l1.restype = ctypes.c_int
    lib.omni_rel_l1_parts.restype = ctypes.c_int
    return lib


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def test_noalloc_matches_general_entry_point_twice():
    lib = _raw_lib()
    dev = torch.device("cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    torch.manual_seed(11)
    for call, shape in enumerate([(2, 4096, 3072), (1, 1000, 3072)]):
        a = torch.randn(*shape, device=dev, dtype=torch.bfloat16)
        b = a + (0.05 + 0.1 * call) * torch.randn_like(a)
        n = a.numel()
        parts = lib.omni_rel_l1_parts(ctypes.c_long(n))
        scratch = torch.empty(2 * parts, device=dev, dtype=torch.float32)
        ref = torch.zeros(2, device=dev, dtype=torch.float32)
        got = torch.zeros(2, device=dev, dtype=torch.float32)
        rc = lib.omni_rel_l1(_p(a), _p(b), ctypes.c_long(n), _p(scratch), _p(None), _p(None), ctypes.c_int(0),
                             ctypes.c_float(0.0), ctypes.c_int(0), _p(ref), stream)
        assert rc == 0
        rc = lib.omni_rel_l1_noalloc(_p(a), _p(b), ctypes.c_long(n), _p(got), _p(None), _p(None), ctypes.c_int(0),
                                     ctypes.c_float(0.0), ctypes.c_int(0), stream)
        assert rc == 0, lib.omni_rel_l1_noalloc_strerror(rc)
        torch.cuda.synchronize()
        assert torch.allclose(got, ref, rtol=1e-5, atol=1e-3), (call, got.tolist(), ref.tolist())
        exact = torch.stack([(a.float() - b.float()).abs().sum(), b.float().abs().sum()])
        assert torch.allclose(got, exact, rtol=1e-3), (call, got.tolist(), exact.tolist())


def test_noalloc_rejects_oversize_and_bad_arguments():
    lib = _raw_lib()
    dev = torch.device("cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    a = torch.zeros(64, device=dev, dtype=torch.bfloat16)
    out = torch.zeros(2, device=dev, dtype=torch.float32)
    too_big = lib.omni_rel_l1_noalloc_max_elems() + 8
    rc = lib.omni_rel_l1_noalloc(_p(a), _p(a), ctypes.c_long(too_big), _p(out), _p(None), _p(None), ctypes.c_int(0),
                                 ctypes.c_float(0.0), ctypes.c_int(0), stream)
    assert rc < 0 and b"exceeds" in lib.omni_rel_l1_noalloc_strerror(rc)
    rc = lib.omni_rel_l1_noalloc(_p(a), _p(a), ctypes.c_long(60), _p(out), _p(None), _p(None), ctypes.c_int(0),
                                 ctypes.c_float(0.0), ctypes.c_int(0), stream)
    assert rc < 0 and b"multiple of 8" in lib.omni_rel_l1_noalloc_strerror(rc)
    torch.cuda.synchronize()


def test_noalloc_state_path_matches_general_entry_point_and_small_after_large():
    """The TeaCache bookkeeping (`state`, `coef`) through the allocation-free entry point equals the
    general one, also when a small input (fewer partial sums) follows a large one in the shared array."""
    lib = _raw_lib()
    dev = torch.device("cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    torch.manual_seed(5)
    coef = torch.tensor([2.0, -1.5, 0.9, -0.02], device=dev, dtype=torch.float32)     # dips below 0 at small rel
    st_ref = torch.zeros(4, device=dev, dtype=torch.float32)
    st_got = torch.zeros(4, device=dev, dtype=torch.float32)
    for call, (shape, noise) in enumerate([((2, 4096, 3072), 0.004), ((8 * 256 * 3,), 0.3), ((1, 512, 3072), 0.01)]):
        a = torch.randn(*shape, device=dev, dtype=torch.bfloat16)
        b = a + noise * torch.randn_like(a)
        n = a.numel()
        parts = lib.omni_rel_l1_parts(ctypes.c_long(n))
        scratch = torch.empty(2 * parts, device=dev, dtype=torch.float32)
        rc = lib.omni_rel_l1(_p(a), _p(b), ctypes.c_long(n), _p(scratch), _p(st_ref), _p(coef), ctypes.c_int(4),
                             ctypes.c_float(0.5), ctypes.c_int(0), _p(None), stream)
        assert rc == 0
        rc = lib.omni_rel_l1_noalloc(_p(a), _p(b), ctypes.c_long(n), _p(None), _p(st_got), _p(coef), ctypes.c_int(4),
                                     ctypes.c_float(0.5), ctypes.c_int(0), stream)
        assert rc == 0, lib.omni_rel_l1_noalloc_strerror(rc)
        torch.cuda.synchronize()
        assert torch.allclose(st_got, st_ref, rtol=1e-5, atol=1e-6), (call, st_got.tolist(), st_ref.tolist())
        assert st_got[0].item() >= 0.0                      # |rescale(rel)| never pulls the accumulator down


def test_noalloc_refuses_missing_coefficients():
    lib = _raw_lib()
    dev = torch.device("cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    a = torch.zeros(64, device=dev, dtype=torch.bfloat16)
    st = torch.zeros(4, device=dev, dtype=torch.float32)
    rc = lib.omni_rel_l1_noalloc(_p(a), _p(a), ctypes.c_long(64), _p(None), _p(st), _p(None), ctypes.c_int(3),
                                 ctypes.c_float(0.1), ctypes.c_int(0), stream)
    assert rc < 0
    rc = lib.omni_rel_l1_noalloc(_p(a), _p(a), ctypes.c_long(64), _p(None), _p(st), _p(None), ctypes.c_int(-1),
                                 ctypes.c_float(0.1), ctypes.c_int(0), stream)
    assert rc < 0
    torch.cuda.synchronize()
