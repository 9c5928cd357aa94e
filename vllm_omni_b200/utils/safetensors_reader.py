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


class NativeSafetensorsFile:
    """The same file behind the C++ reader (``csrc/io_host.cpp``): the header is parsed natively and
    tensors are copied out of the mapping by a thread pool, straight into caller-owned buffers.

    ``read(names, pin=True)`` returns ``{name: tensor}`` backed by ONE host allocation (pinned when
    a GPU is present), so a whole shard becomes a single asynchronous host-to-device copy.
    ``read_rows(name, r0, r1)`` pulls only rows [r0, r1) of a tensor: what a tensor-parallel rank
    needs of a column-parallel weight, without touching the other ranks' bytes.
    """

    def __init__(self, path: str, threads: int = 8):
        import ctypes
        from ..build import build_one, lib_path
        if not lib_path("io_host").exists():
            build_one("io_host")
        L = self._L = ctypes.CDLL(str(lib_path("io_host")))
        L.omni_st_open.restype = ctypes.c_void_p
        L.omni_st_open.argtypes = [ctypes.c_char_p]
        L.omni_st_error.restype = ctypes.c_char_p
        L.omni_st_error.argtypes = [ctypes.c_void_p]
        L.omni_st_metadata.restype = ctypes.c_char_p
        L.omni_st_metadata.argtypes = [ctypes.c_void_p]
        L.omni_st_count.argtypes = [ctypes.c_void_p]
        L.omni_st_info.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(ctypes.c_char_p),
                                   ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64)]
        L.omni_st_read.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64),
                                   ctypes.POINTER(ctypes.c_void_p), ctypes.c_int]
        L.omni_st_close.argtypes = [ctypes.c_void_p]
        self.path, self.threads = path, threads
        self._h = L.omni_st_open(path.encode())
        err = L.omni_st_error(self._h).decode()
        if err:
            L.omni_st_close(self._h)
            self._h = None
            raise ValueError(f"{path}: {err}")
        self.header = {}
        name, dtype = ctypes.c_char_p(), ctypes.c_char_p()
        shape = (ctypes.c_int64 * 8)()
        b, e = ctypes.c_uint64(), ctypes.c_uint64()
        for i in range(L.omni_st_count(self._h)):
            nd = L.omni_st_info(self._h, i, ctypes.byref(name), ctypes.byref(dtype), shape, ctypes.byref(b), ctypes.byref(e))
            self.header[name.value.decode()] = {"dtype": dtype.value.decode(), "shape": [int(shape[d]) for d in range(nd)],
                                                "data_offsets": [int(b.value), int(e.value)]}
        md = L.omni_st_metadata(self._h).decode()
        self.metadata = json.loads(md) if md else {}

    def keys(self):
        return list(self.header.keys())

    def _read_ranges(self, ranges, pin):
        """ranges: [(offset, nbytes)] -> one uint8 buffer holding them back to back (64-byte aligned starts)."""
        import ctypes
        starts, total = [], 0
        for _, n in ranges:
            starts.append(total)
            total += (n + 63) // 64 * 64
        buf = torch.empty(max(total, 1), dtype=torch.uint8, pin_memory=bool(pin and torch.cuda.is_available()))
        n = len(ranges)
        if n:
            offs = (ctypes.c_uint64 * n)(*[r[0] for r in ranges])
            sizes = (ctypes.c_uint64 * n)(*[r[1] for r in ranges])
            dsts = (ctypes.c_void_p * n)(*[buf.data_ptr() + s for s in starts])
            if self._L.omni_st_read(self._h, n, offs, sizes, dsts, self.threads) != 0:
                raise ValueError(f"{self.path}: byte range outside the file")
        return buf, starts

    def read(self, names=None, pin: bool = True) -> dict[str, torch.Tensor]:
        names = list(self.header) if names is None else list(names)
        infos = [self.header[n] for n in names]
        buf, starts = self._read_ranges([(i["data_offsets"][0], i["data_offsets"][1] - i["data_offsets"][0]) for i in infos], pin)
        out = {}
        for n, i, s in zip(names, infos, starts):
            dt = _DTYPES[i["dtype"]]
            nb = i["data_offsets"][1] - i["data_offsets"][0]
            out[n] = buf[s:s + nb].view(dt).reshape(i["shape"]) if nb else torch.empty(i["shape"], dtype=dt)
        return out

    def get_tensor(self, name: str) -> torch.Tensor:
        return self.read([name], pin=False)[name]

    def read_rows(self, name: str, r0: int, r1: int, pin: bool = False) -> torch.Tensor:
        i = self.header[name]
        dt = _DTYPES[i["dtype"]]
        shape = i["shape"]
        row = dt.itemsize
        for d in shape[1:]:
            row *= d
        r0, r1 = max(0, r0), min(shape[0], r1)
        buf, _ = self._read_ranges([(i["data_offsets"][0] + r0 * row, (r1 - r0) * row)], pin)
        return buf[:(r1 - r0) * row].view(dt).reshape([r1 - r0] + shape[1:])

    def close(self):
        if self._h is not None:
            self._L.omni_st_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass


class NvtxRange:
    """``with NvtxRange("denoise step 3"):`` — NVTX push/pop through the C++ runtime (no-op without a
    profiler attached or when the library is not built)."""
    _L = None

    @classmethod
    def _lib(cls):
        if cls._L is None:
            import ctypes
            from ..build import lib_path
            p = lib_path("io_host")
            cls._L = ctypes.CDLL(str(p)) if p.exists() else False
            if cls._L:
                cls._L.omni_nvtx_push.argtypes = [ctypes.c_char_p]
                cls._L.omni_nvtx_mark.argtypes = [ctypes.c_char_p]
        return cls._L

    def __init__(self, name: str):
        self.name = name.encode()

    def __enter__(self):
        L = self._lib()
        if L:
            L.omni_nvtx_push(self.name)
        return self

    def __exit__(self, *a):
        L = self._lib()
        if L:
            L.omni_nvtx_pop()
        return False
