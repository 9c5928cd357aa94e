"""Checked build (-DOMNI_BOUNDS_CHECK): a slot or page id outside the cache is recorded in the status
word and the access is skipped.  The test runs in a child process (the checked library is chosen at
load time) and the "bad" indices point past the DECLARED cache but inside the allocation, so that no
variant of the library can touch memory it does not own."""
import os
import subprocess
import sys

import pytest

CHILD = r"""
import ctypes, torch
from vllm_omni_b200.ops import _native as nv
from vllm_omni_b200.ops import kv_cache as KC
lib = nv.lib("kv_cache")
assert lib._cdll.omni_kv_bounds_check_enabled() == 1, "checked twin not loaded"
dev = torch.device("cuda")
big_k = torch.zeros(8, 16, 2, 128, device=dev, dtype=torch.bfloat16)      # the allocation: 8 pages
big_v = torch.zeros_like(big_k)
kc, vc = big_k[:4], big_v[:4]                                             # the cache the kernels are told about: 4 pages
k = torch.randn(3, 2, 128, device=dev, dtype=torch.bfloat16)
v = torch.randn_like(k)
st = nv.status_word(dev)
# in range: written, no report
KC.kv_write(k, v, kc, vc, torch.tensor([0, 17, 63], dtype=torch.int32, device=dev))
torch.cuda.synchronize()
assert int(st.item()) == 0 and torch.equal(kc.view(-1, 2, 128)[17], k[1])
# slot 70 lies in page 4: outside the declared cache -> reported (kernel id 1), skipped
KC.kv_write(k, v, kc, vc, torch.tensor([1, 70, 2], dtype=torch.int32, device=dev))
torch.cuda.synchronize()
code = int(st.item())
assert code & 0xff == 9 and (code >> 8) & 0xff == 1, hex(code)
assert float(big_k.view(-1, 2, 128)[70].abs().sum()) == 0.0               # nothing was written there
assert torch.equal(kc.view(-1, 2, 128)[1], k[0]) and torch.equal(kc.view(-1, 2, 128)[2], k[2])
st.zero_()
# a block table that names page 6 of a 4-page cache -> reported by the gather kernel (kernel id 2)
outk, outv = KC.kv_gather(kc, vc, torch.tensor([0, 6], dtype=torch.int32, device=dev), 32)
torch.cuda.synchronize()
code = int(st.item())
assert code & 0xff == 9 and (code >> 8) & 0xff == 2, hex(code)
st.zero_()
print("BOUNDS-OK")
"""


MOE_CHILD = r"""
import ctypes, torch
from vllm_omni_b200.ops import _native as nv
lib = nv.lib("moe")
assert lib._cdll.omni_moe_bounds_check_enabled() == 1, "checked twin not loaded"
c_int, c_long = ctypes.c_int, ctypes.c_long
dev = torch.device("cuda")
st = nv.status_word(dev)
T, k, D, E = 4, 2, 64, 8
x = torch.randn(T, D, device=dev, dtype=torch.bfloat16)
big = torch.zeros(32, D, device=dev, dtype=torch.bfloat16)            # the allocation: 32 rows
lib.omni_moe_set_bounds(c_long(16), nv.ptr(st))                       # the buffer the kernels are told about: 16 rows
rows = torch.tensor([0, 1, 2, 3, 20, 5, -1, 7], dtype=torch.int32, device=dev)     # pair 4 -> row 20: outside
nv.check_rc(lib.omni_moe_dispatch(nv.ptr(x), c_long(D), nv.ptr(rows), c_int(T * k), c_int(k), c_int(D), nv.ptr(big),
                                  nv.stream_ptr()), "dispatch")
torch.cuda.synchronize()
code = int(st.item())
assert code & 0xff == 9 and (code >> 8) & 0xff == 4, hex(code)
assert float(big[20].abs().sum()) == 0.0 and torch.equal(big[5], x[2]) and torch.equal(big[0], x[0])
st.zero_()
# combine reading a row past the declared buffer: reported (kernel id 5), that pair contributes nothing
w = torch.ones(T * k, device=dev)
out = torch.empty(T, D, device=dev, dtype=torch.bfloat16)
big[20] = 100.0
nv.check_rc(lib.omni_moe_combine(nv.ptr(big), nv.ptr(rows), nv.ptr(w), c_int(T), c_int(k), c_int(D), None, c_long(0),
                                 nv.ptr(out), c_long(D), nv.stream_ptr()), "combine")
torch.cuda.synchronize()
code = int(st.item())
assert code & 0xff == 9 and (code >> 8) & 0xff == 5, hex(code)
assert torch.equal(out[2], big[5])                                     # token 2 = pairs (4 -> skipped, 5)
st.zero_()
# an expert id outside [0, E) in the plan: reported (kernel id 3), the pair gets no row
ids = torch.tensor([0, 1, 2, 9, 3, 3, 7, 0], dtype=torch.int32, device=dev)
rop = torch.empty(8, dtype=torch.int32, device=dev)
te, t0, tr = (torch.empty(16, dtype=torch.int32, device=dev) for _ in range(3))
nr = torch.zeros(1, dtype=torch.int32, device=dev)
nv.check_rc(lib.omni_moe_plan_compact(nv.ptr(ids), c_int(8), c_int(E), c_int(0), c_int(E), c_int(16), nv.ptr(rop),
                                      nv.ptr(te), nv.ptr(t0), nv.ptr(tr), nv.ptr(nr), nv.stream_ptr()), "plan")
torch.cuda.synchronize()
code = int(st.item())
assert code & 0xff == 9 and (code >> 8) & 0xff == 3, hex(code)
assert int(nr.item()) == 7 and int(rop[3].item()) == -1
st.zero_()
print("BOUNDS-OK")
"""


@pytest.mark.gpu
def test_checked_moe_kernels_report_and_skip():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    env = dict(os.environ, OMNI_BOUNDS_CHECK="1")
    r = subprocess.run([sys.executable, "-c", MOE_CHILD], env=env, capture_output=True, text=True, timeout=300,
                       cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0 and "BOUNDS-OK" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_checked_kv_kernels_report_and_skip():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    env = dict(os.environ, OMNI_BOUNDS_CHECK="1")
    r = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=300,
                       cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0 and "BOUNDS-OK" in r.stdout, r.stdout + r.stderr


def test_release_build_compiles_the_check_out():
    """The macro is a constant in release builds (no kernel carries the test)."""
    src = open(os.path.join(os.path.dirname(__file__), "..", "vllm_omni_b200", "csrc", "ptx_sm100.cuh")).read()
    assert "#define OMNI_IN_BOUNDS(ok, status, kernel_id) (true)" in src
