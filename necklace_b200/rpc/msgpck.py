"""Message (de)serialisation: msgpack with explicit numpy / torch tensor support,
plus pickle-inside-msgpack and raw pickle helpers.

``packb`` / ``unpackb`` carry every RPC request and reply, so they never pickle: an object
they cannot describe raises ``TypeError`` on the sending side and an unknown extension
record is returned as an opaque ``ExtType`` on the receiving side.  (Unpickling bytes that
arrive on a socket would let anyone who can reach the port run code in this process.)
Pickle is only used by the explicit helpers ``pkpackb`` / ``unpkpackb`` / ``pkl_*``, as in
the reference, for payloads a caller has decided to trust.  ``ALLOW_PICKLE_FALLBACK = True``
restores the implicit fallback for closed, trusted networks.

The reference relies on the ``msgpack_numpy`` monkey patch
(necklace/rpc/msgpck.py:14-45); here arrays travel as msgpack ``ExtType`` records
(dtype, shape, raw bytes), torch tensors are sent as CPU arrays and come back as
tensors, and tuples survive a round trip as tuples.
"""
from __future__ import annotations

import pickle

import msgpack
import numpy as np

_EXT_NDARRAY, _EXT_TENSOR, _EXT_TUPLE, _EXT_PICKLE = 1, 2, 3, 4
ALLOW_PICKLE_FALLBACK = False


def _default(obj):
    try:
        import torch
        if isinstance(obj, torch.Tensor):
            arr = obj.detach().cpu()
            if arr.dtype == torch.bfloat16:
                body = (b"bfloat16", list(arr.shape), arr.view(torch.int16).numpy().tobytes())
            else:
                a = arr.numpy()
                body = (a.dtype.str.encode(), list(a.shape), a.tobytes())
            return msgpack.ExtType(_EXT_TENSOR, msgpack.packb(body, use_bin_type=True))
    except ImportError:
        pass
    if isinstance(obj, np.ndarray):
        a = np.ascontiguousarray(obj)
        return msgpack.ExtType(_EXT_NDARRAY, msgpack.packb(
            (a.dtype.str.encode(), list(a.shape), a.tobytes()), use_bin_type=True))
    if isinstance(obj, np.generic):
        return obj.item()
    if isinstance(obj, tuple):
        return msgpack.ExtType(_EXT_TUPLE, packb(list(obj)))
    if isinstance(obj, (set, frozenset)):
        return sorted(obj)
    if isinstance(obj, range):           # a list on arrival (what Python 2 scripts meant)
        return list(obj)
    if ALLOW_PICKLE_FALLBACK:
        return msgpack.ExtType(_EXT_PICKLE, pickle.dumps(obj, protocol=4))
    raise TypeError(f"cannot serialise {type(obj).__name__} for RPC; send plain data, arrays or "
                    f"tensors, or use pkpackb() explicitly")


def _ext_hook(code, data):
    if code in (_EXT_NDARRAY, _EXT_TENSOR):
        dt, shape, raw = msgpack.unpackb(data, raw=False)
        if isinstance(dt, str):
            dt = dt.encode()
        if code == _EXT_TENSOR:
            import torch
            if dt == b"bfloat16":
                a = np.frombuffer(raw, dtype=np.int16).reshape(shape).copy()
                return torch.from_numpy(a).view(torch.bfloat16)
            return torch.from_numpy(np.frombuffer(raw, dtype=np.dtype(dt.decode()))
                                    .reshape(shape).copy())
        return np.frombuffer(raw, dtype=np.dtype(dt.decode())).reshape(shape).copy()
    if code == _EXT_TUPLE:
        return tuple(unpackb(data))
    if code == _EXT_PICKLE and ALLOW_PICKLE_FALLBACK:
        return pickle.loads(data)
    return msgpack.ExtType(code, data)


def packb(obj) -> bytes:
    return msgpack.packb(obj, default=_default, use_bin_type=True, strict_types=True)


def unpackb(data: bytes):
    return msgpack.unpackb(data, ext_hook=_ext_hook, raw=False, strict_map_key=False)


def pkpackb(obj) -> bytes:
    """pickle first, then wrap in msgpack (for objects msgpack cannot describe)."""
    return msgpack.packb(pickle.dumps(obj, protocol=4), use_bin_type=True)


def unpkpackb(data: bytes):
    return pickle.loads(msgpack.unpackb(data, raw=False))


def pkl_dumps(obj) -> bytes:
    return pickle.dumps(obj, protocol=4)


def pkl_loads(data: bytes):
    return pickle.loads(data)
