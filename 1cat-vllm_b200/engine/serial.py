"""Wire codec of the engine-core protocol: msgpack with out-of-band tensor / ndarray buffers
(reference: vllm/v1/serial_utils.py ``MsgpackEncoder``/``MsgpackDecoder``; frame layout of v1/engine/core.py:1598-1744).

A message is a list of ZMQ frames: frame 0 is the msgpack body; tensors and arrays larger than ``INLINE_LIMIT`` are
replaced in the body by ``{"__buf__": i, dtype, shape}`` and their bytes travel as frame ``i`` without a copy."""
from __future__ import annotations

from typing import Any

import msgpack
import numpy as np
import torch

INLINE_LIMIT = 256

REQ_ADD, REQ_ABORT, REQ_START_DP_WAVE, REQ_UTILITY = b"\x00", b"\x01", b"\x02", b"\x03"

_NP = {"float32": np.float32, "float16": np.float16, "int64": np.int64, "int32": np.int32, "uint8": np.uint8, "bool": np.bool_,
       "float64": np.float64, "int16": np.int16, "int8": np.int8}


def encode(obj: Any) -> list:
    bufs: list = []

    def default(o):
        if isinstance(o, torch.Tensor):
            t = o.detach().cpu().contiguous()
            if t.dtype == torch.bfloat16:
                arr, dt = t.view(torch.int16).numpy(), "bfloat16"
            else:
                arr, dt = t.numpy(), str(t.dtype).replace("torch.", "")
            return _arr(arr, dt, "T")
        if isinstance(o, np.ndarray):
            return _arr(np.ascontiguousarray(o), str(o.dtype), "A")
        if isinstance(o, (set, frozenset)):
            return {"__set__": sorted(o)}
        if isinstance(o, np.generic):
            return o.item()
        if hasattr(o, "to_wire"):
            return o.to_wire()
        if hasattr(o, "__dict__"):
            return {"__obj__": type(o).__name__, **{k: v for k, v in o.__dict__.items() if not k.startswith("_")}}
        raise TypeError(f"cannot serialise {type(o)}")

    def _arr(arr, dt, kind):
        raw = arr.tobytes() if arr.nbytes <= INLINE_LIMIT else None
        if raw is not None:
            return {"__arr__": kind, "dtype": dt, "shape": list(arr.shape), "data": raw}
        bufs.append(memoryview(arr).cast("B"))
        return {"__arr__": kind, "dtype": dt, "shape": list(arr.shape), "__buf__": len(bufs)}

    body = msgpack.packb(obj, default=default, use_bin_type=True)
    return [body] + bufs


def decode(frames: list) -> Any:
    def hook(d):
        if "__arr__" in d:
            raw = d["data"] if "data" in d else bytes(frames[d["__buf__"]])
            dt = d["dtype"]
            if dt == "bfloat16":
                return torch.frombuffer(bytearray(raw), dtype=torch.int16).view(torch.bfloat16).reshape(d["shape"])
            arr = np.frombuffer(raw, dtype=_NP[dt]).reshape(d["shape"])
            return torch.from_numpy(arr.copy()) if d["__arr__"] == "T" else arr
        if "__set__" in d:
            return set(d["__set__"])
        return d

    return msgpack.unpackb(bytes(frames[0]), object_hook=hook, raw=False, strict_map_key=False)
