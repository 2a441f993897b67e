"""msgpack with numpy arrays as an extension type: ``{dtype, shape, raw bytes}`` (reference:
loongforge/embodied/eval/transport/msgpack_numpy.py)."""
from __future__ import annotations

import msgpack
import numpy as np

_EXT_NDARRAY = 42


def _default(obj):
    if isinstance(obj, np.ndarray):
        if obj.dtype.kind in ("O", "V"):
            raise TypeError(f"unsupported array dtype {obj.dtype}")
        header = msgpack.packb((obj.dtype.str, list(obj.shape)), use_bin_type=True)
        body = np.ascontiguousarray(obj).tobytes()
        return msgpack.ExtType(_EXT_NDARRAY, len(header).to_bytes(4, "little") + header + body)
    if isinstance(obj, np.generic):
        return obj.item()
    raise TypeError(f"cannot serialise {type(obj)}")


def _ext_hook(code, data):
    if code != _EXT_NDARRAY:
        return msgpack.ExtType(code, data)
    n = int.from_bytes(data[:4], "little")
    dtype, shape = msgpack.unpackb(data[4:4 + n], raw=False)
    return np.frombuffer(data[4 + n:], dtype=np.dtype(dtype)).reshape(shape).copy()


def packb(obj) -> bytes:
    return msgpack.packb(obj, default=_default, use_bin_type=True)


def unpackb(data: bytes):
    return msgpack.unpackb(data, ext_hook=_ext_hook, raw=False, strict_map_key=False)
