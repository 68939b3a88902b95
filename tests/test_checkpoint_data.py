"""Checkpoint round trips (incl. re-sharding over gloo ranks), data loaders, samplers,
flat-memory manager, activation checkpointing, hooks (CPU)."""
import os
import socket

import pytest
import torch
import torch.nn as nn


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tiny():
    from necklace_b200.models.gpt2 import GPT2, GPT2Config
    torch.manual_seed(0)
    return GPT2(GPT2Config(n_layer=1, d_model=32, n_head=2, d_ff=64, vocab=50, max_seq=16,
                           dtype=torch.float32))


def test_engine_checkpoint_resume_is_bit_identical(tmp_path):
    from necklace_b200 import checkpoint as ck
    from necklace_b200.parallel.engine import OptimConfig, TrainEngine
    tok = torch.randint(0, 50, (4, 17), generator=torch.Generator().manual_seed(1))
    x, y = tok[:, :-1], tok[:, 1:]
    a = TrainEngine(_tiny(), optim=OptimConfig("adam", lr=1e-2))
    for _ in range(3):
        a.step(x, y)
    ck.save(ck.engine_state(a, epoch=2), str(tmp_path / "c.pt"))
    la = [float(a.step(x, y)) for _ in range(2)]
    b = TrainEngine(_tiny(), optim=OptimConfig("adam", lr=1e-2))
    meta = ck.load_engine_state(b, ck.load(str(tmp_path / "c.pt")))
    assert meta["epoch"] == 2 and b.step_count == 3
    lb = [float(b.step(x, y)) for _ in range(2)]
    assert la == lb
    # the state dict loads into a plain module
    plain = _tiny()
    plain.load_state_dict(ck.load(str(tmp_path / "c.pt"))["state_dict"], strict=False)


def _reshard_worker(rank, world, port, path, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from necklace_b200 import checkpoint as ck
    from necklace_b200.comm.symm import TorchGroup
    from necklace_b200.parallel.engine import OptimConfig, TrainEngine
    eng = TrainEngine(_tiny(), mode="zero", group=TorchGroup(), optim=OptimConfig("adam", lr=1e-2))
    ck.load_engine_state(eng, ck.load(path))
    tok = torch.randint(0, 50, (4, 17), generator=torch.Generator().manual_seed(1))
    mine = tok[rank * 2:(rank + 1) * 2]
    eng.step(mine[:, :-1], mine[:, 1:])
    st = ck.engine_state(eng)
    if rank == 0:
        q.put({k: v.clone() for k, v in st["state_dict"].items()})
    dist.barrier()
    dist.destroy_process_group()


def test_checkpoint_reshards_from_1_to_2_zero_ranks(tmp_path):
    import torch.multiprocessing as mp
    from necklace_b200 import checkpoint as ck
    from necklace_b200.parallel.engine import OptimConfig, TrainEngine
    tok = torch.randint(0, 50, (4, 17), generator=torch.Generator().manual_seed(1))
    a = TrainEngine(_tiny(), optim=OptimConfig("adam", lr=1e-2))
    a.step(tok[:, :-1], tok[:, 1:])
    path = str(tmp_path / "c.pt")
    ck.save(ck.engine_state(a), path)
    a.step(tok[:, :-1], tok[:, 1:])  # single-process continuation on the global batch
    ref = ck.engine_state(a)["state_dict"]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_reshard_worker, args=(r, 2, port, path, q)) for r in range(2)]
    for p in ps:
        p.start()
    got = q.get(timeout=120)
    for p in ps:
        p.join(timeout=60)
    for k in ref:
        assert torch.allclose(got[k], ref[k], atol=1e-5), k


def test_samplers_and_slices():
    from necklace_b200.data.sampler import (BatchSampler, SequentialSampler, SliceBatchSampler,
                                            SliceSampler)
    assert list(BatchSampler(SequentialSampler(7), 3, "keep")) == [[0, 1, 2], [3, 4, 5], [6]]
    assert list(BatchSampler(SequentialSampler(7), 3, "discard")) == [[0, 1, 2], [3, 4, 5]]
    bs = BatchSampler(SequentialSampler(7), 3, "rollover")
    assert list(bs) == [[0, 1, 2], [3, 4, 5]] and list(bs)[0] == [6, 0, 1]
    s = SliceSampler(10)
    assert list(s[2:5]) == [2, 3, 4] and len(s[5:]) == 5
    s2 = SliceSampler(100, shuffle=True, seed=3)
    assert sorted(s2) == list(range(100)) and list(s2) != list(range(100))
    sb = SliceBatchSampler(SliceSampler(12), 4, "keep")
    assert list(sb[1:]) == [[4, 5, 6, 7], [8, 9, 10, 11]]


@pytest.mark.timeout(180)
@pytest.mark.parametrize("kind", ["queue", "ring"])
def test_multiprocess_loaders_deliver_every_batch_in_order(kind):
    from necklace_b200.data.dtset import SyntheticDataset
    from necklace_b200.data.loaders import QueueDataLoader, ShmRingDataLoader
    ds = SyntheticDataset(50, (3, 4), classes=5, seed=2)
    cls = QueueDataLoader if kind == "queue" else ShmRingDataLoader
    dl = cls(ds, batch_size=8, num_workers=2, part_num=2, last_batch="keep")
    try:
        for _ in range(2):  # two epochs on the same workers
            got = list(dl)
            assert len(got) == 7 and sum(b[0].shape[0] for b in got) == 50
            x0 = torch.stack([ds[i][0] for i in range(8)])
            assert torch.equal(got[0][0], x0)
            x5 = torch.stack([ds[i][0] for i in range(40, 48)])
            assert torch.equal(got[5][0], x5)
            assert got[6][0].shape[0] == 2
    finally:
        dl.clear()


def test_flat_memory_manager_roundtrip():
    from necklace_b200.frmwrk.pytorch.tsmem import PtCudaFltnMemManager
    a, b = nn.Linear(4, 3), nn.Linear(3, 5)
    wa = a.weight.detach().clone()
    mm = PtCudaFltnMemManager(32, 32, "cpu")
    mm.register(a)
    mm.register(b)
    mm.md_to_gpu(a)
    assert torch.equal(a.weight, wa) and a.weight.data_ptr() == mm.gpu_weig.data_ptr()
    a(torch.randn(2, 4)).sum().backward()
    ga = a.weight.grad.clone()
    assert ga.abs().sum() > 0
    mm.md_to_gpu(b)          # implicitly parks `a`, keeping its gradients
    mm.md_to_cpu(b)
    mm.md_to_gpu(a)
    assert torch.equal(a.weight.grad, ga) and torch.equal(a.weight, wa)


def test_activation_checkpoint_matches_plain_backward():
    from necklace_b200.frmwrk.pytorch.mpnn.checkpointing import (checkpoint,
                                                                 model_parallel_cuda_manual_seed)
    model_parallel_cuda_manual_seed(123)
    net = nn.Sequential(nn.Linear(8, 16), nn.Dropout(0.5), nn.Tanh(), nn.Linear(16, 4))
    x = torch.randn(5, 8, requires_grad=True)
    st = torch.get_rng_state()
    y = checkpoint(net, x)
    y.pow(2).sum().backward()
    g1, gw1 = x.grad.clone(), net[0].weight.grad.clone()
    x.grad = None
    net.zero_grad()
    torch.set_rng_state(st)
    net(x).pow(2).sum().backward()
    assert torch.allclose(g1, x.grad, atol=1e-6) and torch.allclose(gw1, net[0].weight.grad, atol=1e-6)


def test_hook_order_and_return_override():
    from necklace_b200.trainer.tnopbs import ModelWrapperHooks
    calls = []

    class T(ModelWrapperHooks):
        def _one_step(self, rank=0):
            calls.append("step")
            return "one_step"

    t = T({})
    t.register_hook_before_batch(lambda trnr: calls.append("b1"))
    t.register_hook_before_batch(lambda trnr: calls.append("b2"))
    t.register_hook_after_batch(lambda trnr, r: calls.append(("a1", r)))
    assert t.one_step() == "one_step" and calls == ["b1", "b2", "step", ("a1", "one_step")]
    t.register_hook_after_batch(lambda trnr, r: "overridden")
    assert t.one_step() == "overridden"
    for ev in ("train", "epoch", "data_batch", "batch", "do_a_batch_grads", "do_a_train_step"):
        assert hasattr(t, f"register_hook_before_{ev}") and hasattr(t, f"register_hook_after_{ev}")


def test_posix_shared_memory_object_lists():
    from necklace_b200.data.shmem import SharedMemArray, SharedMemList
    lst = SharedMemList(obj_size=256, obj_cnt=4)
    lst[2] = {"a": [1, 2, 3]}
    other = SharedMemList(lst.name, 256, 4)
    assert other[2] == {"a": [1, 2, 3]}
    other.close()
    lst.close()
    lst.unlink()
    arr = SharedMemArray(obj_size=512, obj_cnt=3)
    arr[0] = "x" * 100
    arr[1] = (1, 2.5, None)
    att = SharedMemArray(arr.name, 512, 3)
    assert att[0] == "x" * 100 and att[1] == (1, 2.5, None) and att[2] is None
    with pytest.raises(ValueError):
        arr[2] = "y" * 1000
    att.close()
    arr.close()
    arr.unlink()


class _RaggedDataset:
    def __len__(self):
        return 10

    def __getitem__(self, i):
        return {"idx": i, "tokens": list(range(i % 4 + 1))}


def test_object_ring_loader_yields_arbitrary_batches_in_order():
    from necklace_b200.data.dtmem import DataLoaderSharedMemory
    from necklace_b200.cuda.ncclwrp import PYNCCL_DTYPE_MAP, torch_dtype
    dl = DataLoaderSharedMemory(_RaggedDataset(), 3, num_workers=2, part_num=2, last_batch="keep")
    try:
        for _ in range(2):
            got = [b for b in dl]
            assert [s["idx"] for b in got for s in b] == list(range(10))
            assert got[1][0]["tokens"] == [0, 1, 2, 3]
    finally:
        dl.clear()
    assert PYNCCL_DTYPE_MAP["float"] == 7 and torch_dtype("half") == torch.float16


def test_trainer_epoch_checkpoints_keep_the_newest_common_epoch(tmp_path):
    """Per-rank epoch files: the resume point is the newest epoch every rank has; a rank that
    owns several units with one optimizer each (the ZeRO flavours) gets them all back."""
    import torch.nn as nn
    from necklace_b200.trainer import resume

    class T:                      # the attributes the helpers read from an operator
        def __init__(self, ti, seed):
            torch.manual_seed(seed)
            self.ti, self.e = ti, 0
            self.nets = [nn.Linear(3, 3), nn.Linear(3, 2)]
            self.opts = {i: torch.optim.SGD(m.parameters(), lr=0.1, momentum=0.9)
                         for i, m in enumerate(self.nets)}

        def step(self):
            for i, m in enumerate(self.nets):
                self.opts[i].zero_grad()
                m(torch.ones(1, 3)).sum().backward()
                self.opts[i].step()

    d = str(tmp_path)
    a, b = T(0, 1), T(1, 2)
    for e in (1, 2, 3):
        a.step()
        resume.save_trainer(a, d, e, keep=2)
        if e < 3:                                 # rank 1 died before finishing epoch 3
            b.step()
            resume.save_trainer(b, d, e, keep=2)
    assert resume.epochs_of_rank(d, 0) == [2, 3] and resume.epochs_of_rank(d, 1) == [1, 2]
    assert resume.resume_epoch(d, 2) == 2 and resume.resume_epoch(d, 3) == 0
    assert resume.resume_epoch(str(tmp_path / "none"), 2) == 0
    want = [p.detach().clone() for m in b.nets for p in m.parameters()]
    mom = b.opts[0].state_dict()["state"][0]["momentum_buffer"].clone()
    fresh = T(1, 99)
    resume.load_trainer(fresh, d, 2)
    got = [p.detach() for m in fresh.nets for p in m.parameters()]
    assert fresh.e == 2 and all(torch.equal(x, y) for x, y in zip(want, got))
    assert torch.equal(fresh.opts[0].state_dict()["state"][0]["momentum_buffer"], mom)


def test_shared_tensor_array_in_the_reference_call_shape():
    """``SharedMemArray(name=None, obj_shape=..., dtype='torch.float')`` creates,
    ``create_from_shmem_key(sk)`` attaches (necklace/data/shmpt.py:209-295)."""
    import pickle
    from necklace_b200.data import shmpt
    a = shmpt.SharedMemArray(name=None, obj_shape=(3, 2), dtype="torch.float")
    try:
        a[1] = [5.0, 6.0]
        b = shmpt.SharedMemArray.create_from_shmem_key(pickle.loads(pickle.dumps(a.sk)))
        assert b.buf.shape == (3, 2) and b[1].tolist() == [5.0, 6.0]
        c = shmpt.SharedMemArray(sk=a.sk)
        c[0] = torch.tensor([1.0, 2.0])
        assert a.buf[0].tolist() == [1.0, 2.0]
        b.unlink()
        c.unlink()
        assert shmpt.dtype_to_tensor("torch.long") is torch.LongTensor
        old = shmpt.SharedMemArray((2,), torch.int64)          # this framework's call shape
        assert shmpt.SharedMemArray.attach(*old.key).tensor.dtype == torch.int64
        old.close()
    finally:
        a.unlink()


def test_loaders_take_the_reference_constructor_arguments():
    """``DataLoaderSharedMemory(dataset, batch_size=..., data_shape=..., shuffle=..., last_batch=...,
    batchify_fn=..., inter_batchify_fn=..., part_num=..., num_workers=0)`` as in the reference's
    examples/dp/mnist/pytorch/train_ngn_mnist_2_dtpt.py:113-122."""
    from necklace_b200.data import batchify, dtmptv, dtqpto
    from necklace_b200.data.dtset import SyntheticDataset
    ds = SyntheticDataset(24, (1, 4, 4), classes=10, seed=0)
    for mod in (dtqpto, dtmptv):
        ld = mod.DataLoaderSharedMemory(ds, batch_size=8, data_shape=(1, 4, 4), shuffle=False,
                                        last_batch="discard", batchify_fn=batchify.flt2int_bchfn,
                                        inter_batchify_fn=batchify.pt_batchify_fn, part_num=4,
                                        num_workers=0)
        try:
            batches = list(ld)
            assert len(batches) == 3 and batches[0][0].shape == (8, 1, 4, 4)
            assert ld.num_workers == 1 and ld.data_shape == (1, 4, 4)
        finally:
            ld.clear()
