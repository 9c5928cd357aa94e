"""C++ safetensors reader (``csrc/io_host.cpp``): header parsing, threaded bulk reads into one
buffer, row slices for tensor-parallel loading, error reporting; NVTX range wrapper."""
import json
import struct

import pytest
import torch

from vllm_omni_b200.utils.safetensors_reader import NativeSafetensorsFile, NvtxRange, open_safetensors, save_safetensors


@pytest.fixture()
def shard(tmp_path):
    torch.manual_seed(0)
    t = {"model.layers.0.w": torch.randn(64, 48).to(torch.bfloat16), "b": torch.randn(7), "ids": torch.arange(12).reshape(3, 4),
         "empty": torch.zeros(0, 5), "big": torch.randn(3_000_000), "weird \"name\"\\x": torch.ones(2, dtype=torch.float16)}
    p = tmp_path / "m.safetensors"
    save_safetensors(t, str(p), metadata={"format": "pt", "note": "a \"quoted\" value"})
    return p, t


def test_matches_python_reader_and_original_tensors(shard):
    p, t = shard
    f = NativeSafetensorsFile(str(p), threads=4)
    py = open_safetensors(str(p))
    assert set(f.keys()) == set(t) == set(py.keys())
    assert f.metadata == {"format": "pt", "note": "a \"quoted\" value"}
    got = f.read()
    for k, v in t.items():
        assert got[k].dtype == v.dtype and got[k].shape == v.shape and torch.equal(got[k], v), k
        assert f.header[k] == py.header[k]
    # one backing allocation for the whole read
    bases = {g.untyped_storage().data_ptr() for g in got.values() if g.numel()}
    assert len(bases) == 1
    assert torch.equal(f.get_tensor("ids"), t["ids"])
    f.close()


def test_row_slices_for_tensor_parallel_loading(shard):
    p, t = shard
    f = NativeSafetensorsFile(str(p))
    w = t["model.layers.0.w"]
    for rank in range(4):
        assert torch.equal(f.read_rows("model.layers.0.w", rank * 16, (rank + 1) * 16), w[rank * 16:(rank + 1) * 16])
    assert torch.equal(f.read_rows("ids", 1, 99), t["ids"][1:])


def test_safetensors_written_by_the_reference_package_are_read(tmp_path):
    st = pytest.importorskip("safetensors.torch")
    t = {"a": torch.randn(5, 3), "b.c": torch.randint(0, 9, (4,), dtype=torch.int32), "h": torch.randn(2, 2).half()}
    p = tmp_path / "x.safetensors"
    st.save_file(t, str(p), metadata={"k": "v"})
    f = NativeSafetensorsFile(str(p))
    got = f.read(pin=False)
    assert f.metadata == {"k": "v"} and all(torch.equal(got[k], v) for k, v in t.items())


def test_corrupt_files_are_refused(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(ValueError, match="header length"):
        NativeSafetensorsFile(str(p))
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)          # data section too short
    with pytest.raises(ValueError, match="outside the file"):
        NativeSafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 5) + b"{oops")
    with pytest.raises(ValueError, match="malformed"):
        NativeSafetensorsFile(str(p))
    with pytest.raises(ValueError, match="cannot open"):
        NativeSafetensorsFile(str(tmp_path / "missing.safetensors"))


def test_nvtx_ranges_are_harmless_without_a_profiler():
    with NvtxRange("outer"):
        with NvtxRange("inner"):
            pass
