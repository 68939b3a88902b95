"""``comm.fns`` sends tensors that live in the symmetric heap to the peer-memory kernels and
everything else to ``torch.distributed`` (reference call shapes: necklace/cuda/ncclfns.py:32-260).
The peer group and the process group are stand-ins that record their calls."""
import torch
import torch.distributed as dist

from necklace_b200.comm import fns
from necklace_b200.comm.groups import GroupInfo


class FakePeer:
    def __init__(self):
        self.calls = []

    def all_reduce(self, t):
        self.calls.append(("all_reduce", t.data_ptr()))

    def all_gather(self, full):
        self.calls.append(("all_gather", full.data_ptr()))

    def broadcast(self, t, root):
        self.calls.append(("broadcast", t.data_ptr(), root))

    def reduce_scatter(self, full, out):
        self.calls.append(("reduce_scatter", full.numel(), out.numel()))


def _group(rank=1, world=2):
    g = GroupInfo(rank, list(range(world)), "dp")
    assert g.rank == rank and g.world_size == world
    return g


def test_heap_tensors_take_the_peer_kernels(monkeypatch):
    peer = FakePeer()
    monkeypatch.setattr(fns, "_peer", lambda group, t: peer)
    g = _group()
    t = torch.arange(1024, dtype=torch.float32)
    fns.broadcast(t, 1, g)
    out = torch.zeros(2048)
    fns.all_gather(out, t, g)
    assert torch.equal(out[1024:], t) and out[:1024].abs().sum() == 0   # own slice, rank 1
    fns.all_gather(out, out[1024:], g)                                  # already in place
    rs_out = torch.zeros(512)
    fns.reduce_scatter(rs_out, t, group=g)
    fns.all_reduce(t, group=g)
    kinds = [c[0] for c in peer.calls]
    assert kinds == ["broadcast", "all_gather", "all_gather", "reduce_scatter", "all_reduce"]
    assert peer.calls[0][2] == 1 and peer.calls[3][1:] == (1024, 512)


def test_other_tensors_and_odd_sizes_take_torch_distributed(monkeypatch):
    peer = FakePeer()
    seen = []
    monkeypatch.setattr(fns, "_peer", lambda group, t: peer)
    monkeypatch.setattr(dist, "reduce_scatter_tensor", lambda o, i, **k: seen.append("rs"))
    monkeypatch.setattr(dist, "broadcast", lambda t, **k: seen.append(("bc", k["src"])))
    monkeypatch.setattr(dist, "all_gather_into_tensor", lambda o, i, **k: seen.append("ag"))
    g = _group(rank=0)
    fns.reduce_scatter(torch.zeros(5), torch.zeros(10), group=g)        # 10 % 512 != 0
    fns.reduce_scatter(torch.zeros(512), torch.zeros(1024), op="max", group=g)
    fns.broadcast(torch.zeros(3), 1, g)                                 # 12 bytes
    fns.all_gather(torch.zeros(6), torch.zeros(3), g)                   # 24 bytes, 2 ranks
    assert seen == ["rs", "rs", ("bc", 1), "ag"] and peer.calls == []
    monkeypatch.setattr(fns, "_peer", lambda group, t: None)            # not in the heap
    fns.broadcast(torch.zeros(1024), 0, g)
    assert seen[-1] == ("bc", 0) and peer.calls == []


def test_non_members_and_single_rank_groups_return_at_once():
    g = GroupInfo(5, [0, 1], "dp")          # rank 5 is not in the group
    t = torch.ones(4)
    assert fns.all_reduce(t, group=g) is t and fns.broadcast(t, 0, g) is t
    one = GroupInfo(0, [0], "dp")
    out = torch.zeros(4)
    fns.all_gather(out, t, one)
    assert torch.equal(out, t)


def test_reference_argument_order_of_the_compat_module(monkeypatch):
    """``cuda.ncclfns`` keeps the reference's positional order (datatype before op / group;
    broadcast's root defaults to the caller's own group rank) and maps operator codes."""
    from necklace_b200.cuda import ncclfns, ncclwrp
    seen = []
    monkeypatch.setattr(fns, "_peer", lambda group, t: None)
    monkeypatch.setattr(dist, "all_reduce", lambda t, **k: seen.append(("ar", k["op"])))
    monkeypatch.setattr(dist, "broadcast", lambda t, **k: seen.append(("bc", k["src"])))
    monkeypatch.setattr(dist, "reduce", lambda t, **k: seen.append(("rd", k["dst"], k["op"])))
    monkeypatch.setattr(dist, "all_gather_into_tensor", lambda o, i, **k: seen.append("ag"))
    g = _group(rank=1)
    t = torch.zeros(4)
    ncclfns.all_reduce(t, ncclwrp.ncclFloat, ncclwrp.ncclMax, g)
    ncclfns.all_reduce(t, group=g)
    ncclfns.broadcast(t, None, None, g)                       # root = my group rank = 1
    ncclfns.broadcast(t, 0, group=g)
    ncclfns.reduce(t, 0, None, "sum", g)
    ncclfns.all_gather(torch.zeros(8), t, None, g)
    send = torch.arange(4.0)
    ncclfns.pg_all_reduce(send, t, 4, None, None, g)
    assert torch.equal(t, send)                               # copied into the receive tensor
    assert seen == [("ar", dist.ReduceOp.MAX), ("ar", dist.ReduceOp.SUM), ("bc", 1), ("bc", 0),
                    ("rd", 0, dist.ReduceOp.SUM), "ag", ("ar", dist.ReduceOp.SUM)]
    import pytest
    with pytest.raises(TypeError):
        ncclfns.pg_all_reduce(1234, 5678, 4, group=g)
