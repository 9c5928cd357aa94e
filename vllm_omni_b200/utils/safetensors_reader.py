"""safetensors reader/writer on a memory map.

File layout: 8-byte little-endian header length, JSON header {name: {dtype, shape,
data_offsets}}, raw tensor bytes.  Tensors are zero-copy views of the mapping
(``torch.frombuffer``), so loading to the GPU is one H2D copy per tensor with no
intermediate host allocation.
"""
from __future__ import annotations

import json
import mmap
import struct

import torch

_DTYPES = {"F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
           "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
           "BOOL": torch.bool, "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_COPY)
        (n,) = struct.unpack("<Q", self._mm[:8])
        self.header = json.loads(self._mm[8:8 + n].decode("utf-8"))
        self.metadata = self.header.pop("__metadata__", {})
        self._base = 8 + n

    def keys(self):
        return list(self.header.keys())

    def get_tensor(self, name: str) -> torch.Tensor:
        info = self.header[name]
        b, e = info["data_offsets"]
        dt = _DTYPES[info["dtype"]]
        if e == b:
            return torch.empty(info["shape"], dtype=dt)
        t = torch.frombuffer(self._mm, dtype=dt, count=(e - b) // dt.itemsize, offset=self._base + b)
        return t.reshape(info["shape"])

    def close(self):
        try:
            self._mm.close()
        except BufferError:   # tensors still alias the mapping
            pass
        self._f.close()


def open_safetensors(path: str) -> SafetensorsFile:
    return SafetensorsFile(path)


def save_safetensors(tensors: dict[str, torch.Tensor], path: str, metadata: dict | None = None) -> None:
    header, off, blobs = {}, 0, []
    for name, t in tensors.items():
        t = t.detach().contiguous().cpu()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    if metadata:
        header["__metadata__"] = {k: str(v) for k, v in metadata.items()}
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
