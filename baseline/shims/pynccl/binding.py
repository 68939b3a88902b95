"""ctypes binding of libnccl (the copy PyTorch's wheel depends on) and libcudart.

Only what the reference's call sites need: unique id, communicator init / destroy, group
start / end, all-reduce, broadcast, reduce, all-gather, reduce-scatter, send, recv."""
import ctypes
import glob
import os
from ctypes import POINTER, Structure, byref, c_char, c_int, c_size_t, c_void_p

# ncclDataType_t
ncclInt8 = ncclChar = 0
ncclUint8 = 1
ncclInt32 = ncclInt = 2
ncclUint32 = 3
ncclInt64 = 4
ncclUint64 = 5
ncclFloat16 = ncclHalf = 6
ncclFloat32 = ncclFloat = 7
ncclFloat64 = ncclDouble = 8
ncclBfloat16 = 9
# ncclRedOp_t
ncclSum, ncclProd, ncclMax, ncclMin, ncclAvg = 0, 1, 2, 3, 4
ncclNumOps = 4      # the value the reference's table names (NCCL 2.x before ncclAvg)
ncclNumTypes = 9

NCCL_UNIQUE_ID_BYTES = 128


class ncclUniqueId(Structure):
    _fields_ = [("internal", c_char * NCCL_UNIQUE_ID_BYTES)]

    def __reduce__(self):
        return (_uid_from_bytes, (bytes(bytearray(self)),))


def _uid_from_bytes(b):
    u = ncclUniqueId()
    ctypes.memmove(byref(u), b, NCCL_UNIQUE_ID_BYTES)
    return u


ncclComm_t = c_void_p
cudaStream_t = c_void_p


def _find(name_glob, env=None):
    cands = []
    if env and os.environ.get(env):
        cands.append(os.environ[env])
    try:
        import torch
        base = os.path.dirname(os.path.dirname(torch.__file__))
        cands += glob.glob(os.path.join(base, "nvidia", "*", "lib", name_glob))
        cands += glob.glob(os.path.join(os.path.dirname(torch.__file__), "lib", name_glob))
    except ImportError:
        pass
    cands += glob.glob(os.path.join("/usr/local/cuda/lib64", name_glob))
    cands += glob.glob(os.path.join("/usr/lib/x86_64-linux-gnu", name_glob))
    for c in cands:
        if os.path.isfile(c):
            return c
    return name_glob.replace("*", "")


_nccl = None
_cudart = None


def libnccl():
    global _nccl
    if _nccl is None:
        import torch  # noqa: F401  (loads its own libnccl first; dlopen then returns that copy)
        _nccl = ctypes.CDLL(_find("libnccl.so.2", "PYNCCL_LIB"), mode=ctypes.RTLD_GLOBAL)
        L = _nccl
        L.ncclGetErrorString.restype = ctypes.c_char_p
        L.ncclGetErrorString.argtypes = [c_int]
        L.ncclGetUniqueId.argtypes = [POINTER(ncclUniqueId)]
        L.ncclCommInitRank.argtypes = [POINTER(ncclComm_t), c_int, ncclUniqueId, c_int]
        L.ncclCommDestroy.argtypes = [ncclComm_t]
        L.ncclAllReduce.argtypes = [c_void_p, c_void_p, c_size_t, c_int, c_int, ncclComm_t,
                                    cudaStream_t]
        L.ncclBroadcast.argtypes = [c_void_p, c_void_p, c_size_t, c_int, c_int, ncclComm_t,
                                    cudaStream_t]
        L.ncclReduce.argtypes = [c_void_p, c_void_p, c_size_t, c_int, c_int, c_int, ncclComm_t,
                                 cudaStream_t]
        L.ncclAllGather.argtypes = [c_void_p, c_void_p, c_size_t, c_int, ncclComm_t, cudaStream_t]
        L.ncclReduceScatter.argtypes = [c_void_p, c_void_p, c_size_t, c_int, c_int, ncclComm_t,
                                        cudaStream_t]
        L.ncclSend.argtypes = [c_void_p, c_size_t, c_int, c_int, ncclComm_t, cudaStream_t]
        L.ncclRecv.argtypes = [c_void_p, c_size_t, c_int, c_int, ncclComm_t, cudaStream_t]
    return _nccl


def libcudart():
    global _cudart
    if _cudart is None:
        import torch  # noqa: F401
        _cudart = ctypes.CDLL(_find("libcudart.so.1*", "PYNCCL_CUDART"))
        _cudart.cudaStreamCreateWithFlags.argtypes = [POINTER(cudaStream_t), ctypes.c_uint]
        _cudart.cudaStreamSynchronize.argtypes = [cudaStream_t]
        _cudart.cudaSetDevice.argtypes = [c_int]
    return _cudart


class NcclError(RuntimeError):
    pass


def check(rc, what):
    if rc != 0:
        raise NcclError(f"{what} failed: {libnccl().ncclGetErrorString(rc).decode()} ({rc})")
    return rc
