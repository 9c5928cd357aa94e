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
