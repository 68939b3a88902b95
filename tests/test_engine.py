"""TrainEngine: gradient accumulation, clipping, bucketed ZeRO state layout (CPU / gloo) and,
on a GPU, independence of the result from how far the host runs ahead of the device."""
import os
import socket

import pytest
import torch


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tiny(dtype=torch.float32, device=None, n_layer=2):
    from necklace_b200.models.gpt2 import GPT2, GPT2Config
    torch.manual_seed(0)
    return GPT2(GPT2Config(n_layer=n_layer, d_model=32, n_head=2, d_ff=64, vocab=50, max_seq=16,
                           dtype=dtype), device=device)


def _tiny_gpu():
    from necklace_b200.models.gpt2 import GPT2, GPT2Config
    torch.manual_seed(0)
    return GPT2(GPT2Config(n_layer=2, d_model=128, n_head=2, d_ff=512, vocab=512, max_seq=128),
                device="cuda")


def _tok_gpu(n=4):
    tok = torch.randint(0, 512, (n, 129), generator=torch.Generator().manual_seed(1)).cuda()
    return tok[:, :-1].contiguous(), tok[:, 1:].contiguous()


def _tok(n=8):
    tok = torch.randint(0, 50, (n, 17), generator=torch.Generator().manual_seed(1))
    return tok[:, :-1].contiguous(), tok[:, 1:].contiguous()


def test_micro_batches_equal_one_big_batch():
    from necklace_b200.parallel.engine import OptimConfig, TrainEngine
    x, y = _tok(8)
    a = TrainEngine(_tiny(), optim=OptimConfig("adam", lr=1e-2))
    b = TrainEngine(_tiny(), optim=OptimConfig("adam", lr=1e-2), micro_batches=4)
    for _ in range(3):
        la, lb = a.step(x, y), b.step(x, y)
    assert abs(float(la) - float(lb)) < 1e-4
    assert torch.allclose(a.master, b.master, atol=2e-5)


def test_clip_grad_norm_matches_torch():
    from necklace_b200.parallel.engine import OptimConfig, TrainEngine
    x, y = _tok(4)
    eng = TrainEngine(_tiny(), optim=OptimConfig("sgd", lr=0.1, beta1=0.0), clip_grad_norm=0.05)
    ref = _tiny()
    opt = torch.optim.SGD(ref.parameters(), lr=0.1)
    for _ in range(2):
        eng.step(x, y)
        opt.zero_grad()
        ref(x, y).backward()
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.05)
        opt.step()
    assert float(eng.hyper[4]) < 1.0            # the clip was active
    for p, q in zip(eng.flat.params, ref.parameters()):
        assert torch.allclose(p, q, atol=1e-5)


def test_set_lr_and_device_step_counter():
    from necklace_b200.parallel.engine import OptimConfig, TrainEngine
    x, y = _tok(4)
    eng = TrainEngine(_tiny(), optim=OptimConfig("adam", lr=1e-2, beta2=0.95))
    for _ in range(5):
        eng.step(x, y)
    assert float(eng.hyper[3]) == 5.0
    assert abs(float(eng.hyper[2]) - 1.0 / (1.0 - 0.95 ** 5)) < 1e-4
    eng.set_lr(0.0)
    before = eng.master.clone()
    eng.step(x, y)
    assert torch.equal(before, eng.master)


def _bucket_worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from necklace_b200.comm.symm import TorchGroup
    from necklace_b200.parallel.engine import OptimConfig, TrainEngine
    x, y = _tok(4)
    mine = slice(rank * 2, rank * 2 + 2)
    outs = []
    for kw in ({}, {"bucket_mb": 0.004}, {"bucket_mb": 0.004, "clip_grad_norm": 0.5}):
        eng = TrainEngine(_tiny(), mode="zero", group=TorchGroup(),
                          optim=OptimConfig("adam", lr=1e-2), **kw)
        for _ in range(3):
            eng.step(x[mine], y[mine])
        outs.append((len(eng.buckets), eng.full_master()))
    if rank == 0:
        q.put([(n, m.clone()) for n, m in outs])
    dist.barrier()
    dist.destroy_process_group()


def test_bucketed_zero_state_layout_matches_single_bucket():
    """Cutting the flat buffer into buckets changes which elements a rank owns, not the result."""
    import torch.multiprocessing as mp
    from necklace_b200.parallel.engine import OptimConfig, TrainEngine
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_bucket_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    outs = q.get(timeout=120)
    for p in procs:
        p.join(60)
    (n1, m1), (n2, m2), (n3, m3) = outs
    assert n1 == 1 and n2 > 1
    assert torch.allclose(m1, m2, atol=1e-6)
    x, y = _tok(4)
    ref = TrainEngine(_tiny(), optim=OptimConfig("adam", lr=1e-2))
    refc = TrainEngine(_tiny(), optim=OptimConfig("adam", lr=1e-2), clip_grad_norm=0.5)
    for _ in range(3):
        ref.step(x, y)
        refc.step(x, y)
    n = ref.master.numel()
    # Adam divides by sqrt(v): elements with near-zero gradients amplify summation-order
    # noise, so compare in norm
    rel = lambda a, b: float((a - b).norm() / b.norm())
    assert rel(m1[:n], ref.master) < 2e-3
    assert rel(m3[:n], refc.master) < 2e-3


@pytest.mark.gpu
@pytest.mark.parametrize("graph", [False, True])
def test_steps_enqueued_without_sync_match_synced_steps(graph):
    """The Adam bias corrections come from a device step counter: a host that enqueues many
    steps ahead (or replays a graph) must give the same weights as one that waits every step.
    fp32 atomics in the bias-gradient sums make the last bits run-dependent and Adam's
    normalised update amplifies them, so the yardstick is the difference between two runs that
    both wait after every step; scalars of another step (beta2 = 0.95: 1 / (1 - beta2^t) is
    4.4 at t = 5 and 1.4 at t = 25) would change the early updates by a factor 1.8."""
    from necklace_b200.parallel.engine import OptimConfig, TrainEngine
    x, y = _tok_gpu()
    opt = OptimConfig("adam", lr=1e-3, beta1=0.9, beta2=0.95)
    res = []
    for sync in (True, True, False):
        eng = TrainEngine(_tiny_gpu(), optim=opt, use_cuda_graph=graph)
        w0 = eng.master.clone()
        for _ in range(12):
            eng.step(x, y)
            if sync:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
        eng.check()
        res.append(eng.master - w0)
        assert float(eng.hyper[3]) == 12.0
        assert abs(float(eng.hyper[2]) - 1.0 / (1.0 - 0.95 ** 12)) < 1e-3
    rel = lambda a, b: float((a - b).norm() / a.norm())
    noise = rel(res[0], res[1])
    assert rel(res[0], res[2]) < max(4 * noise, 2e-3), (noise, rel(res[0], res[2]))
    assert noise < 0.2


@pytest.mark.gpu
def test_overlapped_buckets_match_plain_step_single_gpu():
    """Side-stream buckets (learned delivery order, graph capture of both streams)."""
    from necklace_b200.parallel.engine import OptimConfig, TrainEngine
    x, y = _tok_gpu()
    opt = OptimConfig("adam", lr=1e-2, beta1=0.9, beta2=0.95)
    a = TrainEngine(_tiny_gpu(), optim=opt)
    b = TrainEngine(_tiny_gpu(), optim=opt, bucket_mb=0.25, use_cuda_graph=True)
    assert len(b.buckets) > 1
    for _ in range(6):
        a.step(x, y)
        b.step(x, y)
    torch.cuda.synchronize()
    b.check()
    assert float((a.master - b.master).norm() / a.master.norm()) < 3e-2
