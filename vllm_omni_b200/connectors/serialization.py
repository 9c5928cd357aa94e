"""msgpack serialisation of stage payloads: tensors, ndarrays, PIL images, dataclasses and
nested containers (vllm_omni/distributed/omni_connectors/utils/serialization.py).  Tensor
bytes are written once into the msgpack stream as ``bin`` objects; decoding rebuilds
tensors with ``torch.frombuffer`` on the received buffer (no second copy)."""
from __future__ import annotations

import dataclasses
import importlib
import io
from typing import Any

import msgpack
import numpy as np
import torch

_T2N = {torch.bfloat16: "bfloat16", torch.float16: "float16", torch.float32: "float32", torch.float64: "float64",
        torch.int64: "int64", torch.int32: "int32", torch.int16: "int16", torch.int8: "int8", torch.uint8: "uint8",
        torch.bool: "bool"}
_N2T = {v: k for k, v in _T2N.items()}


class OmniSerializer:
    @staticmethod
    def _enc(o: Any):
        if isinstance(o, torch.Tensor):
            t = o.detach()
            if t.is_cuda:
                t = t.cpu()
            t = t.contiguous()
            raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
            return {"__t__": _T2N[t.dtype], "s": list(t.shape), "b": raw}
        if isinstance(o, np.ndarray):
            return {"__n__": str(o.dtype), "s": list(o.shape), "b": np.ascontiguousarray(o).tobytes()}
        if isinstance(o, (np.integer,)):
            return int(o)
        if isinstance(o, (np.floating,)):
            return float(o)
        if hasattr(o, "save") and hasattr(o, "size") and hasattr(o, "mode"):      # PIL image
            buf = io.BytesIO()
            o.save(buf, format="PNG")
            return {"__pil__": buf.getvalue()}
        if dataclasses.is_dataclass(o) and not isinstance(o, type):
            return {"__dc__": f"{type(o).__module__}:{type(o).__qualname__}",
                    "f": {f.name: getattr(o, f.name) for f in dataclasses.fields(o)}}
        if isinstance(o, (set, frozenset, tuple)):
            return {"__seq__": type(o).__name__, "v": list(o)}
        if isinstance(o, bytes):
            return o
        raise TypeError(f"cannot serialise {type(o)!r}")

    @staticmethod
    def _dec(d: dict):
        if "__t__" in d:
            dt = _N2T[d["__t__"]]
            if not d["b"]:
                return torch.empty(d["s"], dtype=dt)
            return torch.frombuffer(bytearray(d["b"]), dtype=dt).reshape(d["s"])
        if "__n__" in d:
            return np.frombuffer(d["b"], dtype=np.dtype(d["__n__"])).reshape(d["s"]).copy()
        if "__pil__" in d:
            from PIL import Image
            return Image.open(io.BytesIO(d["__pil__"])).copy()
        if "__dc__" in d:
            mod, _, qn = d["__dc__"].partition(":")
            cls = importlib.import_module(mod)
            for part in qn.split("."):
                cls = getattr(cls, part)
            names = {f.name for f in dataclasses.fields(cls) if f.init}
            obj = cls(**{k: v for k, v in d["f"].items() if k in names})
            for k, v in d["f"].items():
                if k not in names:
                    try:
                        setattr(obj, k, v)
                    except Exception:
                        pass
            return obj
        if "__seq__" in d:
            return {"set": set, "frozenset": frozenset, "tuple": tuple}[d["__seq__"]](d["v"])
        return d

    @classmethod
    def serialize(cls, obj: Any) -> bytes:
        return msgpack.packb(obj, default=cls._enc, use_bin_type=True, strict_types=True)

    @classmethod
    def deserialize(cls, data: bytes) -> Any:
        return msgpack.unpackb(data, object_hook=cls._dec, raw=False, strict_map_key=False)
