"""Peer-memory collectives against NCCL results on the same inputs (needs >= 2 GPUs).

Ranks run as child processes, one GPU each.  NCCL is used for bootstrap and as the
oracle; NVLS is switched off (plain peer loads/stores everywhere)."""
import os
import socket

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class Checks:
    """Deferred assertions: a rank that fails a numeric check keeps issuing the same
    collectives as its peers (so nobody is left waiting inside one) and raises at the end."""

    def __init__(self):
        self.failed = []

    def __call__(self, cond, *info):
        if not cond:
            self.failed.append(info)

    def finish(self):
        assert not self.failed, self.failed[:5]


def _worker(rank, world, rdv, fn_name, q):
    os.environ.update(NCCL_NVLS_ENABLE="0", RANK=str(rank), WORLD_SIZE=str(world))
    import datetime
    import torch.distributed as dist
    try:
        torch.cuda.set_device(rank)
        # rendezvous through a file: a TCP store on a port picked in the parent can lose the
        # port to another process between the pick and the bind
        dist.init_process_group("nccl", init_method=f"file://{rdv}", rank=rank, world_size=world,
                                device_id=torch.device("cuda", rank),
                                timeout=datetime.timedelta(seconds=60))
        from necklace_b200.comm.symm import SymmetricHeap
        from necklace_b200.ops import check_status
        heap = SymmetricHeap(256 << 20)
        grp = heap.peer_group()
        chk = Checks()
        globals()[fn_name](rank, world, heap, grp, chk)
        torch.cuda.synchronize()
        dist.barrier()
        check_status()
        chk.finish()
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, "ERR " + traceback.format_exc()[-1500:]))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def _run(fn_name, world=None):
    import torch.multiprocessing as mp
    world = world or min(torch.cuda.device_count(), 8)
    import tempfile
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    rdv = os.path.join(tempfile.mkdtemp(prefix="nkb_rdv_"), "store")
    procs = [ctx.Process(target=_worker, args=(r, world, rdv, fn_name, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = []
    try:
        for _ in procs:
            res.append(q.get(timeout=150))
    except Exception:  # noqa: BLE001
        res.append((-1, "ERR a rank did not report within 150 s"))
    for p in procs:
        p.join(timeout=30)
    for p in procs:
        if p.is_alive():
            p.kill()  # exactly the child started above
    bad = [r for r in res if r[1] != "ok"]
    assert not bad, bad


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def case_allreduce_allgather(rank, world, heap, grp, chk):
    import torch.distributed as dist
    for dtype, n in [(torch.float32, 1 << 20), (torch.bfloat16, (1 << 22) + 8 * world),
                     (torch.float32, 1000)]:
        t = heap.alloc(n, dtype)
        for it in range(3):
            torch.manual_seed(100 * it + rank)
            src = torch.randn(n, device="cuda").to(dtype)
            t.copy_(src)
            ref = src.float().clone()
            dist.all_reduce(ref)
            grp.barrier()
            grp.all_reduce(t, scale=0.5)
            tol = 1e-5 if dtype == torch.float32 else 2e-2
            chk(_rel(t, ref * 0.5) < tol, (dtype, n, it))
    shard = 1 << 18
    full = heap.alloc(shard * world, torch.bfloat16)
    for it in range(2):
        full.zero_()
        mine = torch.full((shard,), float(rank + 1 + it), device="cuda").bfloat16()
        full.view(world, shard)[rank].copy_(mine)
        grp.all_gather(full)
        exp = torch.arange(1 + it, world + 1 + it, device="cuda").float()[:, None].expand(world, shard)
        chk(torch.equal(full.view(world, shard).float(), exp))


def case_dp_quant(rank, world, heap, grp, chk):
    import torch.distributed as dist
    from necklace_b200.ops.quant import quantize_flat, dequantize_flat
    n = 3_000_001
    nw = (n + 15) // 16
    codes = heap.alloc(nw, torch.int32)
    counts = heap.alloc(nw * 16, torch.int8)
    residual = torch.zeros(n, device="cuda")
    res_ref = torch.zeros(n, device="cuda")
    thr = 0.4
    for it in range(3):
        torch.manual_seed(7 * it + rank)
        g = torch.randn(n, device="cuda")
        out = torch.empty(n, device="cuda")
        grp.dp_quant_allreduce(g, residual, codes, counts, out, thr, 1.0 / world)
        # oracle: separate codec kernels + NCCL sum of the decoded ternary values
        c = quantize_flat(g, res_ref, thr)
        tern = torch.empty(n, device="cuda")
        dequantize_flat(c, tern, thr)
        dist.all_reduce(tern)
        chk(torch.allclose(out, tern / world, atol=1e-6), it)
        chk(torch.equal(residual, res_ref), it)


def case_rs_opt_ag(rank, world, heap, grp, chk):
    import torch.distributed as dist
    from necklace_b200.ops import adam_step
    n = 8 * world * 64 * 1000
    grads = heap.alloc(n, torch.bfloat16)
    params = heap.alloc(n, torch.bfloat16)
    torch.manual_seed(1)
    p0 = torch.randn(n, device="cuda").bfloat16()
    params.copy_(p0)
    shard = n // world
    master = p0[rank * shard:(rank + 1) * shard].float()
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    ref_master, ref_m, ref_v = p0.float(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    for step in (1, 2, 3):
        torch.manual_seed(50 * step + rank)
        g = torch.randn(n, device="cuda").bfloat16()
        grads.copy_(g)
        gsum = g.float().clone()
        dist.all_reduce(gsum)
        grp.rs_opt_ag(grads, params, master, m, v, adam=True, lr=1e-2, beta1=0.9, beta2=0.95,
                      eps=1e-8, weight_decay=0.1, step=step, grad_scale=1.0 / world)
        adam_step(ref_master, ref_m, ref_v, gsum, None, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8,
                  weight_decay=0.1, step=step, grad_scale=1.0 / world)
        torch.cuda.synchronize()
        chk(torch.allclose(master, ref_master[rank * shard:(rank + 1) * shard], atol=1e-5,
                           rtol=1e-4), step)
        chk(_rel(params, ref_master) < 1e-2, step)


def case_engine_zero_matches_single(rank, world, heap, grp, chk):
    """dp+zr training of a small GPT-2 equals a single-process run on the global batch."""
    from necklace_b200.models.gpt2 import GPT2, GPT2Config
    from necklace_b200.parallel.engine import OptimConfig, TrainEngine
    cfg = GPT2Config(n_layer=2, d_model=128, n_head=2, d_ff=512, vocab=512, max_seq=128)
    torch.manual_seed(0)
    model = GPT2(cfg, device="cuda")
    torch.manual_seed(0)
    ref_model = GPT2(cfg, device="cuda")
    opt = OptimConfig("adam", lr=1e-3, beta1=0.9, beta2=0.95)
    eng = TrainEngine(model, mode="zero", group=grp, heap=heap, optim=opt)
    ref = TrainEngine(ref_model, mode="local", optim=opt)
    g = torch.Generator().manual_seed(3)
    tok = torch.randint(0, cfg.vocab, (world * 2, 129), generator=g).cuda()
    for _ in range(3):
        mine = tok[rank * 2:(rank + 1) * 2]
        l1 = eng.step(mine[:, :-1].contiguous(), mine[:, 1:].contiguous())
        l2 = ref.step(tok[:, :-1].contiguous(), tok[:, 1:].contiguous())
    chk(_rel(eng.flat.flat[:eng.flat.numel_used], ref.flat.flat[:ref.flat.numel_used]) < 2e-2)


def case_ag_gemm(rank, world, heap, grp, chk):
    """all-gather -> GEMM in one kernel vs NCCL all-gather + fp32 matmul."""
    import torch.distributed as dist
    for (R, K, N, bn) in [(256, 512, 768, 0), (1024, 1024, 4096, 0), (128, 256, 384, 256),
                          (512, 1024, 1024, 512)]:
        x_full = heap.alloc(world * R * K, torch.bfloat16).view(world * R, K)
        for it in range(3):
            torch.manual_seed(10 * it + rank)
            mine = torch.randn(R, K, device="cuda").bfloat16()
            torch.manual_seed(999)
            w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
            x_full.zero_()
            x_full[rank * R:(rank + 1) * R].copy_(mine)
            gathered = torch.empty(world * R, K, device="cuda", dtype=torch.bfloat16)
            dist.all_gather_into_tensor(gathered, mine)
            out = grp.ag_gemm(x_full, w, bn=bn)
            ref = gathered.float() @ w.float().t()
            chk(_rel(out, ref) < 1e-2, (R, K, N, it))
            chk(torch.equal(x_full, gathered))
            grp.barrier()


def case_gemm_rs(rank, world, heap, grp, chk):
    """GEMM -> reduce-scatter in one kernel vs fp32 matmul + NCCL reduce_scatter."""
    import torch.distributed as dist
    for (R, K, N, bn) in [(128, 256, 256, 256), (256, 512, 768, 0), (512, 1024, 4096, 0),
                          (384, 320, 520, 256)]:
        M = R * world
        for it in range(3):
            torch.manual_seed(10 * it + rank)
            x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
            w = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
            torch.manual_seed(5)
            bias = torch.randn(N, device="cuda").bfloat16()
            res = torch.randn(R, N, device="cuda").bfloat16()
            part = x.float() @ w.float().t()
            ref = torch.empty(R, N, device="cuda")
            dist.reduce_scatter_tensor(ref, part)
            ref = ref + bias.float() + res.float()
            out = grp.gemm_rs(x, w, bias=bias, res=res, bn=bn)
            chk(_rel(out, ref) < 1.5e-2, (R, K, N, it, _rel(out, ref)))
            grp.barrier()


def case_sp_tp_mlp(rank, world, heap, grp, chk):
    """Sequence-parallel tensor-parallel MLP (fused AG->GEMM, GEMM->RS, both directions)
    against the unsharded fp32 computation."""
    import torch.distributed as dist
    import torch.nn.functional as F
    from necklace_b200.parallel.tensor import SPColumnParallelLinear, SPRowParallelLinear
    C, Fh, R = 256, 1024, 256
    M = R * world
    up = SPColumnParallelLinear(C, Fh, grp, device="cuda", seed=11, std=0.05)
    down = SPRowParallelLinear(Fh, C, grp, device="cuda", seed=12, std=0.05)
    torch.manual_seed(3)
    x_full = torch.randn(M, C, device="cuda").bfloat16()
    dy_full = torch.randn(M, C, device="cuda").bfloat16()
    xs = x_full[rank * R:(rank + 1) * R].clone().requires_grad_(True)
    y = down(F.gelu(up(xs), approximate="tanh"), residual=xs)
    y.backward(dy_full[rank * R:(rank + 1) * R])
    # reference with the full weights
    g1, g2 = torch.Generator().manual_seed(11), torch.Generator().manual_seed(12)
    w1 = (torch.randn(Fh, C, generator=g1) * 0.05).bfloat16().float().cuda().requires_grad_(True)
    w2 = (torch.randn(C, Fh, generator=g2) * 0.05).bfloat16().float().cuda().requires_grad_(True)
    xr = x_full.float().requires_grad_(True)
    yr = F.linear(F.gelu(F.linear(xr, w1), approximate="tanh"), w2) + xr
    yr.backward(dy_full.float())
    sl = slice(rank * R, (rank + 1) * R)
    chk(_rel(y, yr[sl]) < 2e-2)
    chk(_rel(xs.grad, xr.grad[sl]) < 3e-2)
    chk(_rel(up.weight.grad, w1.grad.chunk(world, 0)[rank]) < 3e-2)
    chk(_rel(down.weight.grad, w2.grad.chunk(world, 1)[rank]) < 3e-2)


def case_reduce_scatter_broadcast(rank, world, heap, grp, chk):
    """Peer-memory reduce-scatter and broadcast kernels against NCCL."""
    import torch.distributed as dist
    for dtype, rows, cols in [(torch.bfloat16, 256 * world, 384), (torch.float32, 64 * world, 256)]:
        full = heap.alloc(rows * cols, dtype).view(rows, cols)
        for it in range(3):
            torch.manual_seed(7 * it + rank)
            src = torch.randn(rows, cols, device="cuda").to(dtype)
            full.copy_(src)
            ref = src.float().clone()
            dist.all_reduce(ref)
            grp.barrier()
            out = grp.reduce_scatter(full, scale=0.5)
            per = rows // world
            tol = 1e-5 if dtype == torch.float32 else 2e-2
            chk(_rel(out, ref[rank * per:(rank + 1) * per] * 0.5) < tol, ("rs", dtype, it))
            chk(torch.equal(full, src), "reduce_scatter must not modify its input")
            grp.barrier()
    buf = heap.alloc(4096, torch.int64)
    for root in range(world):
        buf.fill_(rank + 100 * root)
        grp.barrier()
        grp.broadcast(buf, root)
        chk(bool((buf == root + 100 * root).all()), ("bcast", root))
        grp.barrier()


def case_llama_tp_fused(rank, world, heap, grp, chk):
    """Llama on the fused tensor-parallel kernels (sequence-parallel layout, vocabulary-parallel
    embedding and cross-entropy) against the same model on one GPU: loss and gradients."""
    from necklace_b200 import checkpoint as ck
    from necklace_b200.models.llama import Llama, LlamaConfig
    for hd, seq in ((64, 128), (128, 256)):
        nh = max(4, world)                   # every rank needs at least one head
        kw = dict(n_layer=2, d_model=nh * hd, n_head=nh, d_ff=1024, vocab=1000, max_seq=seq)
        tp = Llama(LlamaConfig(tp_group=grp, **kw), device="cuda")
        ref = Llama(LlamaConfig(**kw), device="cuda")
        nb = max(2, world * 128 // seq)      # the fused kernels want 128-row blocks per rank
        tok = torch.randint(0, 1000, (nb, seq + 1),
                            generator=torch.Generator().manual_seed(3)).cuda()
        x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
        for step in range(2):          # twice: buffers and flags are reused
            for m in (tp, ref):
                m.zero_grad(set_to_none=True)
            l_tp = tp(x, y)
            l_tp.backward()
            l_ref = ref(x, y)
            l_ref.backward()
            chk(abs(float(l_tp) - float(l_ref)) < 2e-2, ("loss", hd, step, float(l_tp), float(l_ref)))
            rp = dict(ref.named_parameters())
            for name, p in tp.named_parameters():
                sharded, dim, stride = ck._tp_attrs(p)
                full = rp[name].grad
                if sharded:
                    want = ck.tp_split(full, world, rank, dim, stride)
                    chk(_rel(p.grad, want) < 4e-2, (name, hd, step, _rel(p.grad, want)))
                else:
                    # replicated norm weights: every rank holds the gradient of its rows only
                    import torch.distributed as dist
                    g = p.grad.float().clone()
                    dist.all_reduce(g)
                    chk(_rel(g, full) < 4e-2, (name, hd, step, _rel(g, full)))
            grp.barrier()


def case_heap_grad_reducer(rank, world, heap, grp, chk):
    """Trainer-API data parallelism on the fused kernels: gradients of an ordinary module in
    the heap, reduced bucket by bucket under backward, plain and 2-bit compressed, against
    the unfused codec + NCCL path (bit-equal residuals) and an NCCL all-reduce."""
    import torch.distributed as dist
    import torch.nn as nn
    from necklace_b200.frmwrk.pytorch import ptprms
    from necklace_b200.ops.quant import dequantize_flat, quantize_flat
    from necklace_b200.parallel.flat import HeapGradReducer

    def make():
        torch.manual_seed(0)
        return nn.Sequential(nn.Linear(300, 700), nn.ReLU(), nn.Linear(700, 700), nn.ReLU(),
                             nn.Linear(700, 10)).cuda()

    for comp in (None, {"grad_comp_threshold": 0.002, "grad_size_threshold": 0}):
        net, ref = make(), make()
        red = HeapGradReducer(net, grp, heap, comp, bucket_mb=0.5, overlap=True)
        chk(len(red.buckets) > 1, "want several buckets")
        ref_res = torch.zeros(red.flat.numel, device="cuda")
        for step in range(3):
            torch.manual_seed(100 * step + rank)
            x = torch.randn(64, 300, device="cuda")
            for m in (net, ref):
                for p in m.parameters():
                    if p.grad is not None:
                        p.grad.zero_()
            net(x).square().mean().backward()
            red.finish()
            ref(x).square().mean().backward()
            flat_ref = torch.zeros(red.flat.numel, device="cuda")
            for p, o in zip(ref.parameters(), red.flat.offsets):
                flat_ref[o:o + p.numel()] = p.grad.reshape(-1)
            if comp is None:
                dist.all_reduce(flat_ref)
                flat_ref /= world
                chk(_rel(red.flat.grad, flat_ref) < 1e-5, ("plain", step))
            else:
                thr = comp["grad_comp_threshold"]
                codes = quantize_flat(flat_ref, ref_res, thr)
                allc = torch.empty(world, codes.numel(), dtype=codes.dtype, device="cuda")
                dist.all_gather_into_tensor(allc, codes)
                out = torch.zeros_like(flat_ref)
                for r in range(world):
                    dequantize_flat(allc[r].contiguous(), out, thr, accumulate=True)
                out /= world
                chk(torch.equal(red.residual, ref_res), ("residual", step))
                chk(_rel(red.flat.grad, out) < 1e-6, ("quant", step, _rel(red.flat.grad, out)))
            torch.cuda.synchronize()
            grp.barrier()


def test_heap_grad_reducer():
    _run("case_heap_grad_reducer")


def test_llama_tp_fused():
    _run("case_llama_tp_fused")


def test_reduce_scatter_broadcast():
    _run("case_reduce_scatter_broadcast")


def test_sp_tp_mlp():
    _run("case_sp_tp_mlp")


def test_gemm_rs():
    _run("case_gemm_rs")


def test_ag_gemm():
    _run("case_ag_gemm")


def test_allreduce_allgather():
    _run("case_allreduce_allgather")


def test_dp_quant_allreduce():
    _run("case_dp_quant")


def test_rs_opt_ag():
    _run("case_rs_opt_ag")


def test_engine_zero_matches_single():
    _run("case_engine_zero_matches_single")
