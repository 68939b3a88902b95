"""``encode`` / ``decode`` hooks for msgpack that carry numpy arrays and scalars
(the two functions of msgpack_numpy the reference uses: ``default=m.encode``,
``object_hook=m.decode``)."""
import numpy as np


def encode(obj, chain=None):
    if isinstance(obj, np.ndarray):
        a = np.ascontiguousarray(obj)
        return {"__nd__": True, "dtype": a.dtype.str, "shape": list(a.shape), "data": a.tobytes()}
    if isinstance(obj, (np.bool_, np.number)):
        return {"__npscalar__": True, "dtype": obj.dtype.str, "data": obj.tobytes()}
    if isinstance(obj, complex):
        return {"__complex__": True, "data": repr(obj)}
    try:
        import torch
        if isinstance(obj, torch.Size):
            return list(obj)
    except ImportError:
        pass
    return obj if chain is None else chain(obj)


def decode(obj, chain=None):
    if isinstance(obj, dict):
        if obj.get("__nd__") or obj.get(b"__nd__"):
            g = lambda k: obj.get(k, obj.get(k.encode()))
            dt = g("dtype")
            dt = dt.decode() if isinstance(dt, bytes) else dt
            return np.frombuffer(g("data"), dtype=np.dtype(dt)).reshape(g("shape")).copy()
        if obj.get("__npscalar__") or obj.get(b"__npscalar__"):
            g = lambda k: obj.get(k, obj.get(k.encode()))
            dt = g("dtype")
            dt = dt.decode() if isinstance(dt, bytes) else dt
            return np.frombuffer(g("data"), dtype=np.dtype(dt))[0]
        if obj.get("__complex__"):
            return complex(obj["data"])
    return obj if chain is None else chain(obj)


def patch():
    pass
