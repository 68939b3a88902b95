"""The small modules kept for scripts written against the reference's tree: the numpy
shared-memory array (necklace/data/shmmx.py), the host-buffer averaging helpers
(necklace/frmwrk/pytorch/ptmpi.py:107-174) on two gloo ranks, the data exchanger stub and the
Gluon operator placeholder."""
import os
import pickle
import socket

import numpy as np
import pytest
import torch


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _attach_and_write(sk, q):
    from necklace_b200.data.shmmx import SharedMemArray
    a = SharedMemArray.create_from_shmem_key(sk)
    a[2] = np.full(3, 7.0, dtype=np.float32)
    q.put(a[1].tolist())
    a.unlink()


def test_shared_array_is_visible_across_processes():
    import multiprocessing as mp
    from necklace_b200.data.shmmx import SharedMemArray
    a = SharedMemArray(obj_shape=(4, 3), dtype=np.float32)
    try:
        a[1] = np.arange(3, dtype=np.float32)
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        p = ctx.Process(target=_attach_and_write, args=(pickle.loads(pickle.dumps(a.sk)), q))
        p.start()
        assert q.get(timeout=60) == [0.0, 1.0, 2.0]
        p.join(60)
        assert a[2].tolist() == [7.0, 7.0, 7.0]
        view = SharedMemArray.ndarray_from_shmem_key(a.sk)
        assert view.shape == (4, 3) and view[2, 0] == 7.0
    finally:
        a.unlink()
    with pytest.raises(Exception):
        SharedMemArray.create_from_shmem_key(None)


def _avg_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from necklace_b200.comm import backend
    from necklace_b200.frmwrk.pytorch import ptmpi
    backend.init_backend("dp", {"world_size": world, "my_rank": rank, "dp_size": world},
                         comm_type="gloo", master_port=port)
    torch.manual_seed(rank)
    net = torch.nn.Linear(3, 2)
    opt = torch.optim.SGD(net.parameters(), lr=0.1)
    net(torch.ones(1, 3) * (rank + 1)).sum().backward()
    before = (net.weight.detach().clone().numpy(), net.weight.grad.clone().numpy())
    ptmpi.params_do_mpi_allreduce(None, world, net, ptmpi.init_params_recvs(net))
    ptmpi.opt_grads_do_mpi_allreduce(None, world, opt)
    q.put((rank, before, net.weight.detach().numpy().copy(), net.weight.grad.numpy().copy()))
    backend.shutdown_backend()


@pytest.mark.timeout(300)
def test_host_buffer_averaging_on_two_gloo_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q, port = ctx.Queue(), _free_port()
    procs = [ctx.Process(target=_avg_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted((q.get(timeout=240) for _ in procs), key=lambda r: r[0])
    for p in procs:
        p.join(60)
    w_mean = (res[0][1][0] + res[1][1][0]) / 2
    g_mean = (res[0][1][1] + res[1][1][1]) / 2
    for _, _, w, g in res:
        assert np.allclose(w, w_mean, atol=1e-6) and np.allclose(g, g_mean, atol=1e-6)


def test_exchanger_dataloader_wrapper_and_gluon_placeholder():
    from necklace_b200.data.dtexchg import DataExchanger
    from necklace_b200.data.ptdlspn import spawn_dataloader
    from necklace_b200.frmwrk.pytorch.dtwrp import DataLoaderIterWrp, DataLoaderWrp
    from necklace_b200.trainer.tnopmx import TrainerOPGluon
    assert DataExchanger().exchange(1) is None
    assert DataExchanger(exchange_fn=lambda a, b=0: a + b).exchange(2, b=3) == 5
    ds = torch.utils.data.TensorDataset(torch.arange(10.0))
    assert sum(len(b[0]) for b in DataLoaderIterWrp(DataLoaderWrp(ds, batch_size=4))) == 10
    assert len(list(spawn_dataloader(ds, batch_size=5))) == 2
    try:
        import mxnet  # noqa: F401
    except ImportError:
        with pytest.raises(RuntimeError):
            TrainerOPGluon({})


def _mpu_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.nn.functional as F
    from necklace_b200.comm import backend
    from necklace_b200.frmwrk.pytorch import mpnn
    backend.init_backend("mp", {"world_size": world, "my_rank": rank, "mp_size": world},
                         comm_type="gloo", master_port=port)
    g = torch.Generator().manual_seed(5)
    full = torch.randn(6, 10, generator=g)
    target = torch.randint(0, 10, (6,), generator=g)
    per = 10 // world
    mine = full[:, rank * per:(rank + 1) * per].clone().requires_grad_(True)
    loss = mpnn.vocab_parallel_cross_entropy(mine, target)
    loss.sum().backward()
    ref_in = full.clone().requires_grad_(True)
    ref = F.cross_entropy(ref_in, target, reduction="none")
    ref.sum().backward()
    ok_ce = torch.allclose(loss, ref, atol=1e-5) and \
        torch.allclose(mine.grad, ref_in.grad[:, rank * per:(rank + 1) * per], atol=1e-5)
    data = {"text": torch.arange(12).view(3, 4) * (7 if rank == 0 else 0)}
    got = mpnn.broadcast_data(["text"], data, torch.int64)
    ok_bc = torch.equal(got["text"], torch.arange(12).view(3, 4) * 7)
    shard = torch.nn.Parameter(torch.zeros(4))
    shard.model_parallel = True
    shard.grad = torch.full((4,), float(rank + 1))
    repl = torch.nn.Parameter(torch.zeros(3))
    repl.grad = torch.full((3,), 2.0)
    total = mpnn.clip_grad_norm([shard, repl], max_norm=1.0)
    want = (sum(4 * (r + 1) ** 2 for r in range(world)) + 3 * 4.0) ** 0.5
    ok_clip = abs(total - want) < 1e-5 and \
        torch.allclose(repl.grad, torch.full((3,), 2.0 / (want + 1e-6)), atol=1e-6)
    q.put((rank, ok_ce, ok_bc, ok_clip, total))
    backend.shutdown_backend()


@pytest.mark.timeout(300)
def test_model_parallel_cross_entropy_data_broadcast_and_clipping_on_two_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q, port = ctx.Queue(), _free_port()
    procs = [ctx.Process(target=_mpu_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(60)
    assert all(r[1] and r[2] and r[3] for r in res), res


def test_matrix_codec_wrappers_take_the_reference_call_shape():
    """``cu_fn_matrix_quantize_e(A, C, R, thrd)`` / ``cu_fn_matrix_dequantize_e(A, C, R, thrd)``
    work in place on tensors and on numpy arrays; decoded value + residual = input (error
    feedback), 16 fp32 values per 32-bit word."""
    from necklace_b200.cuda import quantize as q
    assert q.CMP_RATIO == 16
    A = torch.randn(40, 6)
    C = torch.zeros(3, 6, dtype=torch.int32)
    R = torch.zeros(40, 6)
    q.cu_fn_matrix_quantize_e(A, C, R, 0.5)
    B = torch.ones(40, 6)
    q.cu_fn_matrix_dequantize_e(B, C, R, 0.5)
    assert torch.allclose(B + R, A, atol=1e-6)
    assert set(B.unique().tolist()) <= {-0.5, 0.0, 0.5}
    An = np.random.RandomState(0).randn(32, 4).astype(np.float32)
    Cn, Rn, Bn = np.zeros((2, 4), dtype=np.uint32), np.zeros_like(An), np.zeros_like(An)
    q.cu_knl_matrix_quantize_e(An, Cn, Rn, 0.3)
    q.cu_knl_matrix_dequantize_e(Bn, Cn, Rn, 0.3)
    assert np.allclose(Bn + Rn, An, atol=1e-6) and Cn.any()


def test_small_data_helpers_and_dataset_wrappers():
    from necklace_b200.data import dtwrp
    assert dtwrp.is_generator(x for x in []) and not dtwrp.is_generator([])
    assert dtwrp.is_iterator([]) and not dtwrp.is_iterator(3)
    assert dtwrp.get_len([1, 2]) == 2
    with pytest.raises(Exception):
        dtwrp.get_len(3)
    a = np.ones(2)
    assert dtwrp.np_array(a) is a and dtwrp.np_is_ndarray(dtwrp.np_array([1, 2]))
    assert dtwrp.label_to_onehot([1, 0], (2, 3)).tolist() == [[0, 1, 0], [1, 0, 0]]
    ds = dtwrp.DatasetWrp([[10, 20, 30], ["a", "b", "c"]])
    assert len(ds) == 3 and ds[2] == [30, "c"]

    class Direct(dtwrp.DataLoaderBase):
        def get_batch_by_dbi(self, dbi, dbf=None):
            return ("direct", list(dbi))
    w = dtwrp.DataLoaderWrp(Direct(), list(range(8)), rank=1, batch_size=2, kn=2)
    assert w.get_data_batch_index(1, 1) == [6, 7]             # i*b*k + r*b = 1*2*2 + 1*2
    assert w.get_data_batch([6, 7]) == ("direct", [6, 7])
    plain = dtwrp.DataLoaderWrp(None, list(range(8)), rank=0, batch_size=2, kn=2)
    assert plain.get_data_batch([0, 1], dbf=sum) == 1


def test_launcher_environment_gives_rank_and_size():
    from necklace_b200.pympi import api
    assert api.rank_size_from_env({}) == (0, 1, None, None)
    w = api.MpiWrp({"OMPI_COMM_WORLD_RANK": "3", "OMPI_COMM_WORLD_SIZE": "8",
                    "OMPI_COMM_WORLD_LOCAL_RANK": "1"})
    assert (w.rank, w.world_size, w.local_rank, w.launcher) == (3, 8, 1, "OMPI_COMM_WORLD_RANK")
    assert api.rank_size_from_env({"SLURM_PROCID": "2", "SLURM_NTASKS": "4"})[:3] == (2, 4, None)
    assert api.rank_size_from_env({"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"})[:3] == (1, 2, 1)
    a = np.ones(3, dtype=np.float32)
    assert api.MpiWrp({}).do_all_reduce(a, np.zeros(3, dtype=np.float32)).tolist() == [1, 1, 1]
