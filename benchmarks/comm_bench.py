"""CUDA-event timings of the peer-memory collectives and of the fused GEMM + collective
kernels, against NCCL on the same buffers and against their rooflines.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29600 benchmarks/comm_bench.py [--max-mb 1024] [--gemm]

Every number is the max over ranks of the mean of ``--iters`` launches after warm-up, with a
barrier + synchronize on both sides of the timed region.  Bus bandwidth follows the usual
convention: all-reduce ``2 (N-1)/N * bytes / t``, all-gather and reduce-scatter
``(N-1)/N * bytes / t``.  For the fused kernels the floor is the slower of FLOPs over the
measured sustained bf16 GEMM rate and the bytes that must cross NVLink per direction over the
measured 770 GB/s peer-copy bandwidth.  Rank 0 prints markdown tables.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def timed(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mb", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--gemm", action="store_true", help="also time ag_gemm / gemm_rs")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from necklace_b200.comm.symm import SymmetricHeap
    from necklace_b200.ops import check_status
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:  # noqa: BLE001
        pass
    gemm_peak = peaks.get("bf16_tflops_sustained", 1401.1) * 1e12
    heap = SymmetricHeap((args.max_mb << 20) * 3 + (1 << 30))
    grp = heap.peer_group()
    out = []
    p = lambda *a: out.append(" ".join(str(x) for x in a))
    W = world
    p(f"## Peer-memory collectives, {W} x B200 (bf16 payloads, ms = max over ranks)\n")
    p("| size MB | all-reduce ms | busbw GB/s | NCCL ms | all-gather ms | busbw | NCCL ms | "
      "reduce-scatter ms | busbw | NCCL ms | rs_opt_ag (ZeRO Adam) ms | dp_quant_allreduce ms |")
    p("|---|---|---|---|---|---|---|---|---|---|---|---|")
    sizes = [1, 4, 16, 64, 256, 1024]
    big = heap.alloc((args.max_mb << 20) // 2, torch.bfloat16)
    params = heap.alloc((args.max_mb << 20) // 2, torch.bfloat16)
    codes_all = heap.alloc((args.max_mb << 20) // 2 // 16, torch.int32)
    counts_all = heap.alloc((args.max_mb << 20) // 2, torch.int8)
    for mb in [s for s in sizes if s <= args.max_mb]:
        n = (mb << 20) // 2 // (512 * W) * (512 * W)
        t = big[:n]
        t.normal_()
        nbytes = n * 2
        ar = timed(lambda: grp.all_reduce(t, scale=1.0), args.iters)
        ref = torch.empty(n, dtype=torch.bfloat16, device="cuda").normal_()
        ar_n = timed(lambda: dist.all_reduce(ref), args.iters)
        ag = timed(lambda: grp.all_gather(t), args.iters)
        shard = ref[:n // W].clone()
        ag_n = timed(lambda: dist.all_gather_into_tensor(ref, shard), args.iters)
        rs_out = torch.empty(n // W, dtype=torch.bfloat16, device="cuda")
        rs = timed(lambda: grp.reduce_scatter(t.view(W, -1), rs_out.view(1, -1)), args.iters)
        rs_n = timed(lambda: dist.reduce_scatter_tensor(rs_out, ref), args.iters)
        master = torch.zeros(n // W, device="cuda")
        m, v = torch.zeros_like(master), torch.zeros_like(master)
        zo = timed(lambda: grp.rs_opt_ag(t, params[:n], master, m, v, adam=True, lr=1e-4,
                                         step=3, grad_scale=1.0 / W), args.iters)
        res = torch.zeros(n, device="cuda")
        codes, counts = codes_all[:n // 16], counts_all[:n]
        dq = timed(lambda: grp.dp_quant_allreduce(t, res, codes, counts, t, 0.01, 1.0 / W),
                   args.iters)
        bw = lambda f, ms: f * nbytes / (ms * 1e-3) / 1e9
        p(f"| {mb} | {ar:.3f} | {bw(2 * (W - 1) / W, ar):.0f} | {ar_n:.3f} | {ag:.3f} | "
          f"{bw((W - 1) / W, ag):.0f} | {ag_n:.3f} | {rs:.3f} | {bw((W - 1) / W, rs):.0f} | "
          f"{rs_n:.3f} | {zo:.3f} | {dq:.3f} |")
    check_status()
    if args.gemm:
        p(f"\n## Fused GEMM + collective kernels, {W} x B200 (bf16)\n")
        p("| kernel | M (all ranks) | N | K | ms | TFLOP/s per GPU | NVLink MB per dir | "
          "compute floor ms | link floor ms | achieved / roofline | unfused (NCCL + own GEMM) ms |")
        p("|---|---|---|---|---|---|---|---|---|---|---|")
        from necklace_b200.ops.gemm import gemm

        def timed_pair(f1, f2, iters, warmup=3):
            """Two kernels that alternate as in a transformer block (all-gather -> GEMM, then
            GEMM -> reduce-scatter): each is timed by its own pair of events."""
            for _ in range(warmup):
                f1()
                f2()
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(iters)]
            for e in evs:
                e[0].record()
                f1()
                e[1].record()
                f2()
                e[2].record()
            torch.cuda.synchronize()
            t = torch.tensor([sum(e[0].elapsed_time(e[1]) for e in evs) / iters,
                              sum(e[1].elapsed_time(e[2]) for e in evs) / iters],
                             dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t[0]), float(t[1])

        r8 = lambda v: v // 8 * 8
        pairs = [("llama-7B attention", 4096, 4096, r8(3 * 4096 // W), r8(4096 // W)),
                 ("llama-7B mlp", 4096, 4096, r8(2 * 11008 // W), r8(11008 // W)),
                 ("llama-13B attention", 4096, 5120, r8(3 * 5120 // W), r8(5120 // W)),
                 ("llama-13B mlp", 4096, 5120, r8(2 * 13824 // W), r8(13824 // W))]
        for name, M, C, N1, K2 in pairs:
            R = M // W
            xf = heap.alloc(M * C, torch.bfloat16).view(M, C)
            xf.normal_()
            w1 = (torch.randn(N1, C, device="cuda") * 0.02).bfloat16()
            x2 = (torch.randn(M, K2, device="cuda") * 0.5).bfloat16()
            w2 = (torch.randn(C, K2, device="cuda") * 0.02).bfloat16()
            t_ag, t_rs = timed_pair(lambda: grp.ag_gemm(xf, w1), lambda: grp.gemm_rs(x2, w2),
                                    args.iters)
            g = torch.empty(M, C, dtype=torch.bfloat16, device="cuda")
            sh = xf[:R].clone()
            part = torch.empty(M, C, dtype=torch.bfloat16, device="cuda")
            o = torch.empty(R, C, dtype=torch.bfloat16, device="cuda")
            u_ag, u_rs = timed_pair(
                lambda: (dist.all_gather_into_tensor(g, sh), gemm(g, w1)),
                lambda: (gemm(x2, w2, out=part), dist.reduce_scatter_tensor(o, part)), args.iters)
            for kern, ms, un, fl, link, n, k in (
                    ("ag_gemm", t_ag, u_ag, 2.0 * M * N1 * C, (W - 1) / W * M * C * 2, N1, C),
                    ("gemm_rs", t_rs, u_rs, 2.0 * M * C * K2, (W - 1) / W * M * C * 2, C, K2)):
                cf, lf = fl / gemm_peak * 1e3, link / 770e9 * 1e3
                p(f"| {kern} {name} | {M} | {n} | {k} | {ms:.3f} | {fl / ms / 1e9:.0f} | "
                  f"{link / 1e6:.1f} | {cf:.3f} | {lf:.3f} | {max(cf, lf) / ms:.2f} | {un:.3f} |")
        check_status()
    if rank == 0:
        print("\n".join(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
