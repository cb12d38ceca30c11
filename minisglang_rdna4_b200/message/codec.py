"""msgpack (de)serialisation of message dataclasses. 1-D tensors travel as raw bytes plus a
dtype tag (the fast path of python/minisgl/message/utils.py:101-170); nested dataclasses and
lists of messages are handled recursively."""
from __future__ import annotations

import dataclasses
from typing import Any, Dict

import msgpack
import numpy as np
import torch

from ..core import SamplingParams
from . import types as T

_CLASSES: Dict[str, type] = {
    cls.__name__: cls
    for cls in (
        T.TokenizeMsg, T.AbortMsg, T.UserMsg, T.AbortBackendMsg, T.ExitMsg, T.BatchMsg,
        T.DetokenizeMsg, T.StatsMsg, T.UserReply, SamplingParams,
    )
}
_NP = {"int32": np.int32, "int64": np.int64, "float32": np.float32, "uint8": np.uint8}


def _pack(obj: Any) -> Any:
    if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        body = {f.name: _pack(getattr(obj, f.name)) for f in dataclasses.fields(obj)}
        return {"__dc__": type(obj).__name__, "f": body}
    if isinstance(obj, torch.Tensor):
        arr = obj.detach().cpu().contiguous().numpy()
        return {"__t__": str(arr.dtype), "s": list(arr.shape), "b": arr.tobytes()}
    if isinstance(obj, (list, tuple)):
        return [_pack(v) for v in obj]
    if isinstance(obj, dict):
        return {k: _pack(v) for k, v in obj.items()}
    return obj


def _unpack(obj: Any) -> Any:
    if isinstance(obj, dict):
        if "__dc__" in obj:
            cls = _CLASSES[obj["__dc__"]]
            return cls(**{k: _unpack(v) for k, v in obj["f"].items()})
        if "__t__" in obj:
            arr = np.frombuffer(obj["b"], dtype=_NP[obj["__t__"]]).reshape(obj["s"])
            return torch.from_numpy(arr.copy())
        return {k: _unpack(v) for k, v in obj.items()}
    if isinstance(obj, list):
        return [_unpack(v) for v in obj]
    return obj


def encode_msg(msg: Any) -> bytes:
    return msgpack.packb(_pack(msg), use_bin_type=True)


def decode_msg(data: bytes) -> Any:
    return _unpack(msgpack.unpackb(data, raw=False, strict_map_key=False))
