"""Group layout math and the OneRPC control plane (CPU only)."""
import threading
import time

import numpy as np
import pytest
import torch

from necklace_b200.comm import groups as G
from necklace_b200.rpc import msgpck, svctmp, zrpc


@pytest.fixture(autouse=True)
def _fresh_groups():
    G.reset_nccl_groups_map()
    yield
    G.reset_nccl_groups_map()


# layouts the reference computes for world = 8 (necklace/cuda/ncclgrp.py:584-767)
LAYOUTS = [
    ("dp", {}, {"dp_group": [[0, 1, 2, 3, 4, 5, 6, 7]]}),
    ("dp+mp", {"dp_size": 4, "mp_size": 2},
     {"dp_group": [[0, 2, 4, 6], [1, 3, 5, 7]], "mp_group": [[0, 1], [2, 3], [4, 5], [6, 7]]}),
    ("dp+pp", {"dp_size": 2, "pp_size": 4},
     {"dp_group": [[0, 4], [1, 5], [2, 6], [3, 7]], "pp_group": [[0, 1, 2, 3], [4, 5, 6, 7]]}),
    ("dp+pp+mp", {"dp_size": 2, "pp_size": 2, "mp_size": 2},
     {"dp_group": [[0, 4], [1, 5], [2, 6], [3, 7]], "pp_group": [[0, 2], [1, 3], [4, 6], [5, 7]],
      "mp_group": [[0, 1], [2, 3], [4, 5], [6, 7]]}),
    ("dp+zr", {"dp_size": 1, "zr_size": 8},
     {"dp_group": [[i] for i in range(8)], "zr_group": [[0, 1, 2, 3, 4, 5, 6, 7]]}),
    ("dp+zr+mp", {"dp_size": 1, "zr_size": 2, "mp_size": 4},
     {"dp_group": [[i] for i in range(8)], "zr_group": [[0, 4], [1, 5], [2, 6], [3, 7]],
      "mp_group": [[0, 1, 2, 3], [4, 5, 6, 7]]}),
    ("dp+zr+mp", {"dp_size": 2, "zr_size": 2, "mp_size": 2},
     {"dp_group": [[0, 4], [1, 5], [2, 6], [3, 7]], "zr_group": [[0, 2], [1, 3], [4, 6], [5, 7]],
      "mp_group": [[0, 1], [2, 3], [4, 5], [6, 7]]}),
]


@pytest.mark.parametrize("tmode,sizes,expect", LAYOUTS)
def test_group_layouts_match_reference_tables(tmode, sizes, expect):
    pgs, _ = G.build_nccl_pgs_map(tmode, {"world_size": 8, "my_rank": 0, **sizes})
    assert pgs == expect


@pytest.mark.parametrize("world,kinds,szs", [(8, ["dp", "mp"], [4, 2]), (12, ["dp", "pp", "mp"], [2, 3, 2]),
                                             (16, ["dp", "zr", "pp", "mp"], [2, 2, 2, 2]),
                                             (6, ["zr", "mp"], [3, 2])])
def test_groups_partition_world(world, kinds, szs):
    groups = G.calc_groups(world, kinds, dict(zip(kinds, szs)))
    for k, s in zip(kinds, szs):
        gl = groups[k + "_group"]
        assert all(len(g) == s for g in gl)
        assert sorted(r for g in gl for r in g) == list(range(world))  # a partition
    # two ranks share at most one group kind unless identical
    inner = groups[kinds[-1] + "_group"]
    assert all(g == list(range(g[0], g[0] + szs[-1])) for g in inner)  # innermost is contiguous


def test_registry_getters_and_fallbacks():
    G.init_nccl_groups_map("dp+mp", {"world_size": 8, "my_rank": 5, "dp_size": 4, "mp_size": 2})
    assert G.get_nccl_group_dp().pg_ranks == [1, 3, 5, 7] and G.get_nccl_group_dp().rank == 2
    assert G.get_nccl_group_mp().pg_ranks == [4, 5] and G.get_rank(G.get_nccl_group_mp()) == 1
    assert G.get_nccl_group_pp() is None and G.get_nccl_group_pp_or_main().world_size == 8
    assert G.get_world_size() == 8 and G.get_rank() == 5
    cfg = G.get_nccl_groups_map_cfg_dict()
    assert cfg["mp_group"] == {"pg_rank": 5, "pg_ranks": [4, 5], "rank": 1, "ranks": [0, 1],
                               "world_size": 2}
    assert G.get_nccl_groups_map_grp_dict()["dp_group"][1] == [1, 3, 5, 7]
    assert G.get_nccl_group_main_grp_list() == list(range(8))
    # idempotent: a second call with other arguments changes nothing
    G.init_nccl_groups_map("dp", {"world_size": 2, "my_rank": 0})
    assert G.get_world_size() == 8


def test_bad_modes_rejected():
    with pytest.raises(ValueError):
        G.build_nccl_pgs_map("dp+xx", {"world_size": 4, "my_rank": 0})
    with pytest.raises(ValueError):
        G.build_nccl_pgs_map("dp+mp", {"world_size": 8, "my_rank": 0, "dp_size": 3, "mp_size": 2})
    pgs, _ = G.build_nccl_pgs_map("dp+mp", {"world_size": 8, "my_rank": 0, "mp_size": 2})
    assert len(pgs["dp_group"][0]) == 4  # missing size inferred


def test_msgpack_roundtrip_arrays_tensors_tuples():
    msg = {"fn": "x", "rank": 3, "msg": {"a": np.arange(6, dtype=np.float32).reshape(2, 3),
                                         "t": torch.arange(4).bfloat16(), "shp": (2, 3),
                                         "nested": [1, (2, 3), {"k": None}], "b": b"\x00\x01"}}
    out = msgpck.unpackb(msgpck.packb(msg))
    assert np.array_equal(out["msg"]["a"], msg["msg"]["a"])
    assert torch.equal(out["msg"]["t"], msg["msg"]["t"]) and out["msg"]["t"].dtype == torch.bfloat16
    assert out["msg"]["shp"] == (2, 3) and out["msg"]["nested"] == [1, (2, 3), {"k": None}]
    assert out["msg"]["b"] == b"\x00\x01"
    assert msgpck.unpkpackb(msgpck.pkpackb({"x": {1, 2}})) == {"x": {1, 2}}
    assert msgpck.pkl_loads(msgpck.pkl_dumps((1, "a"))) == (1, "a")


def test_rpc_serialiser_never_pickles_implicitly():
    import pickle
    import msgpack

    class Thing:
        pass

    with pytest.raises(TypeError):
        msgpck.packb({"x": Thing()})
    # a forged pickle extension record is handed back opaque, not executed
    evil = msgpack.packb(msgpack.ExtType(4, pickle.dumps(print)), use_bin_type=True)
    out = msgpck.unpackb(evil)
    assert isinstance(out, msgpack.ExtType)


class _Echo(svctmp.TmplServer):
    def fn_echo(self, msg):
        m = self.msg_unpck(msg)
        self.q_put_state(7, m["msg"], m["rank"])
        return self.msg_pck(self.mk_rpc_ret("fn_echo", "ok", got=m["msg"]))

    def fn_boom(self):
        raise ValueError("nope")


def test_rpc_envelope_state_queue_errors_and_timeout(tmp_path):
    url = f"ipc://{tmp_path}/svr.ipc"
    dropped = []
    svr = _Echo({"url": url, "rank": 0, "role": "scheduler",
                 "drop_filter": lambda n, a, k: n == "fn_lost" and not dropped.append(n)})
    svr.start()
    try:
        caller = svctmp.TmplServer({"url": f"ipc://{tmp_path}/w.ipc", "rank": 2, "role": "worker"})
        cli = caller.mk_rpc_cli(url, zc_hb_timeout=5)
        rep = caller.do_rpc_call(cli, "fn_echo", x=1, arr=np.ones(3))
        assert rep["ret"] == "ok" and rep["role"] == "scheduler" and rep["ndid"] == "svr-0"
        assert rep["msg"]["got"]["x"] == 1
        state, args, kwargs = svr.q.get(timeout=1)
        assert state == 7 and args[1] == 2  # sender's rank travelled in the envelope
        assert cli.add(2, 3) == 5 and cli.alive()
        with pytest.raises(zrpc.RpcRemoteError):
            cli.fn_boom()
        t0 = time.time()
        with pytest.raises(zrpc.RpcTimeout):
            cli.call("fn_lost", timeout=0.3)
        assert time.time() - t0 < 2 and dropped == ["fn_lost"]
        assert cli.add(1, 1) == 2  # the connection survives a lost message
        cli.close()
        caller.stop()
    finally:
        svr.stop()


def test_node_timers_and_stop():
    hits = []

    class N(zrpc.Node):
        def check_state(self, *a, **k):
            hits.append(time.time())
            if len(hits) >= 3:
                self.stop()

    n = N({})
    th = threading.Thread(target=n.loop)
    th.start()
    th.join(timeout=5)
    assert not th.is_alive() and len(hits) >= 3


def test_groups_assembled_by_hand_with_the_builder_entry_points():
    """The reference's lower-level calls (necklace/cuda/ncclgrp.py:62-121, :429-500): explicit
    rank lists instead of a trainer mode."""
    from necklace_b200.comm import groups as G
    G.reset_nccl_groups_map()
    try:
        G.init_nccl_group_main(4, 3)
        G.init_nccl_group_pgs(4, 3, {"dp_group": [[0, 2], [1, 3]], "mp_group": [[0, 1], [2, 3]]},
                              {"dp_group": 2, "mp_group": 2}, True)
        assert G.get_nccl_group_dp().pg_ranks == [1, 3] and G.get_nccl_group_dp().rank == 1
        assert G.get_nccl_group_mp().pg_ranks == [2, 3] and G.get_nccl_group_mp().kind == "mp"
        assert G.get_nccl_groups_map_grp_dict()["dp_group"] == [[0, 2], [1, 3]]
        assert G.build_pg_cfg(3, [1, 3]) == {"pg_rank": 3, "pg_ranks": [1, 3]}
        g = G.make_pg_by_nc("comm", 1, [3, 1])
        assert g.comm == "comm" and g.pg_ranks == [1, 3] and g.rank == 0
        G.set_nccl_group_main_world_size(8)
        G.set_nccl_group_main_rank(5)
        assert G.get_nccl_group_main_world_size() == 8 and G.get_nccl_group_main_rank() == 5

        class Nc:
            rank = 2
        main = G.set_nccl_group_main_by_nc(Nc(), 4)
        assert main.rank == 2 and isinstance(G.get_nccl_main_nk(), Nc)
        G.set_nccl_groups_map({"zr_group": g})
        assert G.get_nccl_group_zr() is g
    finally:
        G.reset_nccl_groups_map()


def test_input_broadcast_helpers_accept_both_call_shapes(monkeypatch):
    import torch
    from necklace_b200.comm import fns
    from necklace_b200.comm.groups import GroupInfo
    from necklace_b200.data import dtdist
    seen = []
    monkeypatch.setattr(fns, "broadcast", lambda t, root, group: seen.append(("bc", root, group)))
    monkeypatch.setattr(fns, "all_reduce", lambda t, group=None: seen.append(("ar", group)))
    g, t = GroupInfo(0, [0, 1], "mp"), torch.zeros(2)
    dtdist.dt_shape_do_nccl_broadcast(t, 1, g)
    dtdist.dt_shape_do_nccl_broadcast(g, t)                 # reference order
    dtdist.dt_input_do_nccl_broadcast(g, t, "float32")      # reference order
    dtdist.dt_sampler_do_nccl_bcast(g, 2, 1, t)             # reference order: nc, kn, root, buf
    dtdist.dt_sampler_do_nccl_bcast(t, 0, g)
    dtdist.dt_sampler_do_nccl_allreduce(g, 2, 0, t)
    assert seen == [("bc", 1, g), ("bc", 0, g), ("bc", 0, g), ("bc", 1, g), ("bc", 0, g), ("ar", g)]


def test_range_travels_as_a_list_and_servers_can_sleep():
    from necklace_b200.rpc import msgpck, zrpc
    assert msgpck.unpackb(msgpck.packb({"data": range(4)})) == {"data": [0, 1, 2, 3]}
    assert hasattr(zrpc.Server, "g_sleep") and hasattr(zrpc.Node, "g_sleep")
