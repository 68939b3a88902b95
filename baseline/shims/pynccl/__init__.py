"""The part of the ``pynccl`` package the reference uses: ``Nccl`` (thin object over the
NCCL C API plus one CUDA stream), ``NcclWrp`` (one communicator for the whole job, with
``do_*`` convenience calls) and the ``binding`` constants."""
from ctypes import byref, c_void_p

from . import binding
from .binding import check, libcudart, libnccl, ncclComm_t, ncclUniqueId

__version__ = "0.0-shim"


def _p(x):
    """Device pointer argument: int, numpy integer, ctypes pointer or None."""
    if x is None:
        return None
    if isinstance(x, c_void_p):
        return x
    if hasattr(x, "value") and not isinstance(x, (int, float)):
        return c_void_p(x.value)
    return c_void_p(int(x))


class _Stream:
    """A blocking CUDA stream (flags 0), which is what a numba stream is: it orders against
    work that PyTorch enqueues on the legacy default stream."""

    def __init__(self):
        self.handle = c_void_p()
        rc = libcudart().cudaStreamCreateWithFlags(byref(self.handle), 0)
        if rc != 0:
            raise RuntimeError(f"cudaStreamCreateWithFlags failed: {rc}")

    def synchronize(self):
        rc = libcudart().cudaStreamSynchronize(self.handle)
        if rc != 0:
            raise RuntimeError(f"cudaStreamSynchronize failed: {rc}")


class Nccl:
    def __init__(self):
        self.lib = libnccl()
        self._stream = None

    def get_unique_id(self):
        uid = ncclUniqueId()
        check(self.lib.ncclGetUniqueId(byref(uid)), "ncclGetUniqueId")
        return uid

    def get_comm(self):
        return ncclComm_t()

    def get_stream(self):
        if self._stream is None:
            self._stream = _Stream()
        return self._stream

    def comm_init_rank(self, comm_ref, world_size, nuid, rank):
        return check(self.lib.ncclCommInitRank(comm_ref, int(world_size), nuid, int(rank)),
                     "ncclCommInitRank")

    def comm_destroy(self, comm):
        if comm is not None and getattr(comm, "value", None):
            return self.lib.ncclCommDestroy(comm)
        return 0

    def group_start(self):
        return check(self.lib.ncclGroupStart(), "ncclGroupStart")

    def group_end(self):
        return check(self.lib.ncclGroupEnd(), "ncclGroupEnd")

    def all_reduce(self, send, recv, count, datatype, op, comm, stream):
        return check(self.lib.ncclAllReduce(_p(send), _p(recv), int(count), int(datatype),
                                            int(op), comm, stream), "ncclAllReduce")

    def broadcast(self, send, recv, count, datatype, root, comm, stream):
        return check(self.lib.ncclBroadcast(_p(send), _p(recv), int(count), int(datatype),
                                            int(root), comm, stream), "ncclBroadcast")

    def reduce(self, send, recv, count, datatype, op, root, comm, stream):
        return check(self.lib.ncclReduce(_p(send), _p(recv), int(count), int(datatype), int(op),
                                         int(root), comm, stream), "ncclReduce")

    def all_gather(self, send, recv, count, datatype, comm, stream):
        return check(self.lib.ncclAllGather(_p(send), _p(recv), int(count), int(datatype), comm,
                                            stream), "ncclAllGather")

    def reduce_scatter(self, send, recv, count, datatype, op, comm, stream):
        return check(self.lib.ncclReduceScatter(_p(send), _p(recv), int(count), int(datatype),
                                                int(op), comm, stream), "ncclReduceScatter")

    def send(self, buf, count, datatype, peer, comm, stream):
        return check(self.lib.ncclSend(_p(buf), int(count), int(datatype), int(peer), comm,
                                       stream), "ncclSend")

    def recv(self, buf, count, datatype, peer, comm, stream):
        return check(self.lib.ncclRecv(_p(buf), int(count), int(datatype), int(peer), comm,
                                       stream), "ncclRecv")


class NcclWrp:
    """``NcclWrp(kn, rank, gpu_i)``: world size, this process's rank, local GPU index."""

    def __init__(self, kn, rank, gpu_i=0):
        self.kn, self.rank, self.gpu_i = int(kn), int(rank), int(gpu_i)
        libcudart().cudaSetDevice(self.gpu_i)
        self.nk = Nccl()
        self.comm_i = self.nk.get_comm()
        self.nuid = None

    # bring-up -------------------------------------------------------------------
    def get_nuid(self):
        self.nuid = self.nk.get_unique_id()
        return self.nuid

    def set_nuid(self, nuid):
        self.nuid = nuid

    def init_comm(self):
        self.nk.comm_init_rank(byref(self.comm_i), self.kn, self.nuid, self.rank)

    def del_comm(self):
        self.nk.comm_destroy(self.comm_i)
        self.comm_i = self.nk.get_comm()

    def stream_sync(self):
        self.nk.get_stream().synchronize()

    # collectives on the job-wide communicator ----------------------------------------
    def _h(self):
        return self.nk.get_stream().handle

    def do_all_reduce(self, send, recv, count, datatype=binding.ncclFloat, op=binding.ncclSum):
        self.nk.group_start()
        self.nk.all_reduce(send, recv, count, datatype, op, self.comm_i, self._h())
        self.nk.group_end()

    def do_bcast(self, buf, count, root=0, datatype=binding.ncclFloat):
        self.nk.group_start()
        self.nk.broadcast(buf, buf, count, datatype, root, self.comm_i, self._h())
        self.nk.group_end()

    def do_reduce(self, send, recv, count, root=0, datatype=binding.ncclFloat,
                  op=binding.ncclSum):
        self.nk.group_start()
        self.nk.reduce(send, recv, count, datatype, op, root, self.comm_i, self._h())
        self.nk.group_end()

    def do_all_gather(self, send, recv, count, datatype=binding.ncclFloat):
        self.nk.group_start()
        self.nk.all_gather(send, recv, count, datatype, self.comm_i, self._h())
        self.nk.group_end()

    def do_reduce_scatter(self, send, recv, count, datatype=binding.ncclFloat,
                          op=binding.ncclSum):
        self.nk.group_start()
        self.nk.reduce_scatter(send, recv, count, datatype, op, self.comm_i, self._h())
        self.nk.group_end()

    def do_pp_send_recv(self, send, recv, count, rank_send, rank_recv,
                        datatype=binding.ncclFloat):
        """The rank that holds ``send`` sends to ``rank_recv``; the rank that holds ``recv``
        receives from ``rank_send``."""
        self.nk.group_start()
        if send is not None and self.rank == rank_send:
            self.nk.send(send, count, datatype, rank_recv, self.comm_i, self._h())
        if recv is not None and self.rank == rank_recv:
            self.nk.recv(recv, count, datatype, rank_send, self.comm_i, self._h())
        self.nk.group_end()
