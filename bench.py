"""Headline benchmark: samples/sec of a full training step (forward, backward,
gradient collective, optimizer) of GPT-2 medium in trainer mode ``dp+zr`` (ZeRO over
all ranks), bf16 compute with fp32 master weights and Adam, micro-batch 8 x 1024
tokens per GPU, synthetic token data, random-init weights.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5

``--impl torch`` runs the stock torch.distributed / cuBLAS / SDPA implementation of the
same step (the baseline this framework is compared with); ``--impl reference`` tries the
unmodified reference package from ``baseline/_ref``.

Rank 0 prints one JSON line.  ``value`` is device-timed (CUDA events around exactly
``--steps`` steps, max over ranks) with inputs already on the device; ``e2e`` repeats the
measurement through the public ``TrainEngine.step`` call with a pinned-host -> device copy
of each step's batch and a device -> host read of each step's loss inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "samples/sec whole job (device-timed, max over ranks)"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch"])
    ap.add_argument("--config", type=int, default=3, choices=[1, 2, 3, 4, 5],
                    help="which named configuration: 1 LeNet on the CPU through one scheduler "
                         "and one worker (plumbing; no GPU), 2 dp + 2-bit ResNet-50, 3 dp+zr GPT-2 "
                         "medium (the headline), 4 dp+pp+mp Llama-7B-like, 5 dp+zr+mp "
                         "Llama-13B-like")
    ap.add_argument("--model", default="gpt2-medium", choices=["gpt2-medium", "gpt2-tiny"])
    ap.add_argument("--micro-batch", type=int, default=0, help="0 = the configuration's value")
    ap.add_argument("--seq", type=int, default=0, help="0 = the configuration's value")
    ap.add_argument("--layers", type=int, default=0,
                    help="cut the model to this many layers (smoke runs only; the JSON line "
                         "is then marked reduced and is not a benchmark number)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--bucket-mb", type=float, default=0.0,
                    help="> 0: cut the gradient buffer into buckets of this size and overlap "
                         "their collectives with backward")
    ap.add_argument("--no-baseline", action="store_true",
                    help="skip the stock-torch arm that is timed after ours for vs_baseline")
    ap.add_argument("--tp-impl", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--grad-comp-threshold", type=float, default=1e-3)
    ap.add_argument("--launcher", default="torchrun", choices=["torchrun", "necklace"],
                    help="necklace: run config 3 through the framework's own scheduler + "
                         "worker processes (examples/gpt2/train_gpt2_necklace.py)")
    return ap.parse_args()


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed
    region runs (read-only queries)."""

    def __init__(self, index: int, period: float = 0.1):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001
                pass
            self._stop_evt.wait(self.period)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def reference_arm(args):
    """Runs the unmodified reference package (``baseline/_ref``) through its own scheduler /
    worker services and ZeRO trainer on the same model and batch (``baseline/ref_gpt2_zero.py``),
    with stand-ins for the third-party modules it imports and this image lacks
    (``baseline/shims``).  Every rank of the launch starts one reference worker as a child
    process; rank 0 also starts the reference scheduler.  The reference has no device-resident
    input path (its trainer copies each batch host -> device and its loss wrapper reads the
    loss back every step), so the device-timed value and the end-to-end value are the same
    measurement."""
    import subprocess
    import tempfile
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    tag = os.environ.get("MASTER_PORT", str(os.getpid())) if world > 1 else str(os.getpid())
    work = os.path.join(tempfile.gettempdir(), f"nkref-{tag}")
    os.makedirs(work, exist_ok=True)
    ref_pkg = os.path.join(ROOT, "baseline", "_ref", "necklace", "trainer", "zroppt.py")

    def unavailable(why):
        if rank == 0:
            print(json.dumps({"impl": "reference",
                              "unavailable": str(why).replace("\n", " ")[:300]}), flush=True)
        return 0

    if not os.path.exists(ref_pkg) or not os.path.exists(
            os.path.join(ROOT, "baseline", "_ref", "necklace", "frmwrk", "pytorch", "ptprms.py")):
        return unavailable("baseline/_ref does not hold an installed reference package")
    warmup = max(args.warmup, 3)
    if args.config != 3:
        return unavailable(f"the reference arm covers config 3 only (asked for {args.config})")
    B, S = args.micro_batch or 8, args.seq or 1024
    driver = os.path.join(ROOT, "baseline", "ref_gpt2_zero.py")
    common = ["--world", str(world), "--steps", str(args.steps), "--warmup", str(warmup),
              "--model", args.model, "--micro-batch", str(B), "--seq", str(S),
              "--server-url", f"ipc://{work}/svr.ipc"]
    env = dict(os.environ, NCCL_DEBUG=os.environ.get("NCCL_DEBUG", "WARN"))
    for k in list(env):    # the reference has its own bring-up (unique id relayed over RPC)
        if k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT") or \
                k.startswith("TORCHELASTIC_"):
            env.pop(k)
    procs = []
    if rank == 0:
        procs.append(subprocess.Popen(
            [sys.executable, driver, "--role", "scheduler", *common],
            stdout=open(os.path.join(work, "sched.log"), "w"), stderr=subprocess.STDOUT, env=env))
    out = os.path.join(work, f"rank{rank}.json")
    sampler = ClockSampler(local_rank)
    sampler.start()
    procs.append(subprocess.Popen(
        [sys.executable, driver, "--role", "worker", "--rank", str(rank), "--gpu",
         str(local_rank), "--url", f"ipc://{work}/w{rank}.ipc", "--out", out, *common],
        stdout=open(os.path.join(work, f"w{rank}.log"), "w"), stderr=subprocess.STDOUT, env=env))
    deadline = time.time() + float(os.environ.get("NKB_REF_TIMEOUT", "900"))
    failed = None
    worker = procs[-1]
    sched = procs[0] if rank == 0 else None

    def tail(name, n=300):
        try:
            return open(os.path.join(work, name)).read()[-n:]
        except OSError:
            return ""

    while worker.poll() is None:
        if time.time() > deadline:
            failed = f"reference run exceeded its time limit: {tail(f'w{rank}.log')}"
            break
        if sched is not None and sched.poll() is not None:
            failed = f"reference scheduler ended early: {tail('sched.log')}"
            break
        time.sleep(0.5)
    clocks = sampler.stop()
    if failed is None and not os.path.exists(out):
        failed = f"reference worker {rank} ended without a result: {tail(f'w{rank}.log', 400)}"
    if rank == 0 and failed is None:
        # the scheduler is only needed until every worker has written its result
        t_end = time.time() + 120
        while time.time() < t_end and not all(
                os.path.exists(os.path.join(work, f"rank{r}.json")) for r in range(world)):
            time.sleep(0.2)
    for p in procs:                       # exactly the children started above
        if p.poll() is None:
            p.kill()
    keep = os.environ.get("NKB_REF_LOGDIR")
    if keep:
        import shutil
        os.makedirs(keep, exist_ok=True)
        for name in os.listdir(work):
            if name.endswith(".log"):
                shutil.copy(os.path.join(work, name), os.path.join(keep, f"n{world}_{name}"))
    if rank != 0:
        return 0
    if failed is not None:
        return unavailable(failed)
    res = []
    t_end = time.time() + 120
    for r in range(world):
        f = os.path.join(work, f"rank{r}.json")
        while not os.path.exists(f) and time.time() < t_end:
            time.sleep(0.2)
        if not os.path.exists(f):
            return unavailable(f"reference worker {r} wrote no result")
        res.append(json.load(open(f)))
    if any(r["ms"] is None for r in res):
        return unavailable("reference workers saw fewer steps than requested")
    ms = max(r["ms"] for r in res)
    value = B * world * args.steps / (ms / 1e3)
    line = {
        "metric": METRIC, "value": round(value, 3), "unit": "samples/s", "n_gpus": world,
        "steps": args.steps, "warmup": warmup, "ms_per_step": round(ms / args.steps, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "impl": "reference",
        "config": {"model": args.model, "global_batch": B * world, "seq_len": S,
                   "parallelism": f"zr (zr={world}, dp=1): necklace.trainer.tndszr + zroppt, "
                                  f"{world} net_map sub-modules",
                   "optimizer": "torch AdamW on fp32 parameters, bf16 autocast",
                   "note": "third-party imports (pynccl, zerorpc, gevent, msgpack_numpy) served "
                           "by baseline/shims; output projection untied from the embedding when "
                           "the model is split over more than one owner",
                   "l2": "working set exceeds L2; no explicit flush"},
        "clocks": clocks,
        "e2e": {"value": round(value, 3), "unit": "samples/s",
                "ms_per_step": round(ms / args.steps, 3),
                "h2d_bytes_per_step": int(B * S * 8 * 2), "d2h_bytes_per_step": 4,
                "note": "same run: the reference's step always copies its batch from pinned "
                        "host memory and reads the loss back"},
        "loss_first": res[0]["loss_first"], "loss_last": res[0]["loss_last"],
    }
    print(json.dumps(line), flush=True)
    return 0


# ======================================================================== workloads
class Workload:
    """What the timing harness needs from a configuration."""
    samples_per_step = 0          # whole job
    h2d_bytes_per_step = 0
    config: dict = {}
    engine = None

    def step_dev(self, i):        # inputs already on the device
        raise NotImplementedError

    def step_e2e(self, i):        # inputs copied from pinned host memory inside the call
        raise NotImplementedError

    def finish(self):
        if self.engine is not None:
            self.engine.check()


def _token_pool(vocab, B, S, rank, dev, pool=8):
    import torch
    g = torch.Generator().manual_seed(100 + rank)
    tok = [torch.randint(0, vocab, (B, S + 1), generator=g) for _ in range(pool)]
    hx = [t[:, :-1].contiguous().pin_memory() for t in tok]
    hy = [t[:, 1:].contiguous().pin_memory() for t in tok]
    return hx, hy, [t.to(dev) for t in hx], [t.to(dev) for t in hy]


class GPT2Zero(Workload):
    """Config 3: dp+zr, GPT-2 medium, bf16 + fp32 master Adam, micro-batch 8 x 1024 per GPU."""

    def __init__(self, args, world, rank, dev, impl, mode=None):
        import torch
        self.impl = impl
        B, S = args.micro_batch or 8, args.seq or 1024
        torch.manual_seed(1234)
        if impl == "ours":
            from necklace_b200.comm.symm import SymmetricHeap
            from necklace_b200.models.gpt2 import GPT2, GPT2Config
            from necklace_b200.parallel.engine import OptimConfig, TrainEngine
            cfg = GPT2Config.medium() if args.model == "gpt2-medium" else GPT2Config.tiny()
            if args.layers:
                cfg.n_layer = args.layers
            S = min(S, cfg.max_seq)
            model = GPT2(cfg, device=dev)
            heap = group = None
            mode = mode or ("zero" if world > 1 else "local")
            if world > 1 and mode != "local":
                heap = SymmetricHeap(int(model.num_params() * 2 * 2 * 1.02) + (64 << 20))
                group = heap.peer_group()
            self.engine = TrainEngine(
                model, mode=mode, group=group, heap=heap,
                optim=OptimConfig("adam", lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8,
                                  weight_decay=0.1),
                use_cuda_graph=not args.no_graph,
                bucket_mb=args.bucket_mb if (args.bucket_mb > 0 and mode != "local") else None)
            self._step = self.engine.step
            vocab = cfg.vocab
        else:
            sys.path.insert(0, os.path.join(ROOT, "baseline"))
            from torch_gpt2 import TorchZeroTrainer
            tr = TorchZeroTrainer(args.model, dev, world, rank)
            self._step, vocab, S = tr.step, tr.vocab, min(S, tr.max_seq)
            self._xbuf = self._ybuf = None
        self.hx, self.hy, self.dx, self.dy = _token_pool(vocab, B, S, rank, dev)
        self.samples_per_step = B * world
        self.h2d_bytes_per_step = B * S * 8 * 2
        self.config = {"model": args.model, "global_batch": B * world, "seq_len": S,
                       "parallelism": f"dp+zr (zr={world})", "optimizer": "adam fp32 master",
                       "l2": "per-step working set (0.7 GB bf16 weights + activations) exceeds "
                             "the 126 MB L2; no explicit flush",
                       "cuda_graph": impl == "ours" and not args.no_graph,
                       "bucket_mb": args.bucket_mb}
        if getattr(self, "which", 0) == 4:
            self.config["pipeline"] = self.pipeline
        if args.layers:
            self.config["reduced"] = f"{args.layers} layers: smoke run, not a benchmark number"

    def step_dev(self, i):
        n = len(self.dx)
        return self._step(self.dx[i % n], self.dy[i % n])

    def step_e2e(self, i):
        import torch
        n = len(self.hx)
        if self.impl == "ours":     # the engine copies into its static input buffers
            return self._step(self.hx[i % n], self.hy[i % n])
        if self._xbuf is None:
            self._xbuf, self._ybuf = torch.empty_like(self.dx[0]), torch.empty_like(self.dy[0])
        self._xbuf.copy_(self.hx[i % n], non_blocking=True)
        self._ybuf.copy_(self.hy[i % n], non_blocking=True)
        return self._step(self._xbuf, self._ybuf)


class LlamaHybrid(Workload):
    """Config 4 (dp+pp+mp, Llama 32 L / d 4096 / seq 2048, 8 micro-batches x 2 sequences per
    pipeline step, mp=2, pp=2, dp=world/4) and config 5 (dp+zr+mp, Llama 40 L / d 5120 /
    seq 4096, mp=4, zr=world/4, micro-batch 1 with 8-fold gradient accumulation), both on the
    fused tensor-parallel kernels with Adam on fp32 master weights."""

    def __init__(self, args, world, rank, dev, which):
        import torch
        import torch.nn as nn
        from necklace_b200.comm import backend
        from necklace_b200.comm import groups as G
        from necklace_b200.models.llama import Llama, LlamaConfig
        from necklace_b200.parallel.engine import OptimConfig, TrainEngine
        from necklace_b200.parallel.pipe_engine import PipelineEngine
        self.which = which
        opt = OptimConfig("adam", lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1)
        if which == 4:
            mp, pp = 2, 2
            assert world % 4 == 0, "config 4 needs 4 (dp=1) or 8 (dp=2) GPUs"
            dp = world // 4
            tmode, gcfg = "dp+pp+mp", {"dp_size": dp, "pp_size": pp, "mp_size": mp}
            cfgm = LlamaConfig.llama7b()
            S, mb_seqs, n_mb = args.seq or 2048, args.micro_batch or 2, 8
        else:
            mp = 4
            assert world % 4 == 0, "config 5 needs 4 (zr=1) or 8 (zr=2) GPUs"
            zr = world // 4
            tmode, gcfg = "dp+zr+mp", {"dp_size": 1, "zr_size": zr, "mp_size": mp}
            cfgm = LlamaConfig.llama13b()
            S, mb_seqs, n_mb = args.seq or 4096, args.micro_batch or 1, 8
        if args.layers:
            cfgm.n_layer = args.layers
        gcfg.update(world_size=world, my_rank=rank)
        # heap: bf16 parameters + gradients of this rank's model slice (when they are reduced
        # over peers) plus the gather / staging buffers of the fused kernels
        per_layer = 4 * cfgm.d_model ** 2 + 3 * cfgm.d_model * cfgm.d_ff
        n_local = (cfgm.n_layer * per_layer // (pp if which == 4 else 1) +
                   2 * 32768 * cfgm.d_model) // mp
        heap_bytes = int(n_local * 4 * 1.05) + (3 << 30)
        fused = args.tp_impl == "fused"
        heap = backend.init_backend(tmode, gcfg, comm_type="peer", device=dev,
                                    heap_bytes=heap_bytes)
        mpg = G.get_nccl_group_mp()
        mp_peer = mpg.comm.peer
        cfgm.tp_group = mp_peer if fused else None
        cfgm.mp, cfgm.mp_rank = mpg.world_size, mpg.rank
        self.mp_rank = mpg.rank
        B = mb_seqs * n_mb
        if which == 4:
            ppg = G.get_nccl_group_pp()
            stage, n_stage = ppg.rank, ppg.world_size
            per = cfgm.n_layer // n_stage
            layers = range(stage * per, (stage + 1) * per if stage < n_stage - 1 else cfgm.n_layer)
            net = Llama(cfgm, device=dev, layers=layers, with_embed=stage == 0,
                        with_head=stage == n_stage - 1)

            class Stage(nn.Module):
                def __init__(s):
                    super().__init__()
                    s.net = net

                def forward(s, x, targets=None):
                    return s.net(x, targets, batch=mb_seqs)

            dpg = G.get_nccl_group_dp()
            self.engine = PipelineEngine(
                Stage(), stage=stage, pp_ranks=ppg.pg_ranks, micro_batches=n_mb,
                group=dpg.comm.peer if dpg.world_size > 1 else None, heap=heap, mp_group=mp_peer,
                optim=opt, bucket_mb=args.bucket_mb if args.bucket_mb > 0 else None,
                grad_sync=net.make_grad_sync())
            self.has_data = stage == 0
            replicas = dpg.world_size
            par = f"dp={replicas} pp={pp} mp={mp}"
            # share of a 1F1B step in which a stage waits for the pipeline to fill and drain
            self.pipeline = {"stages": n_stage, "micro_batches": n_mb, "schedule": "1F1B",
                             "bubble_fraction": round((n_stage - 1) / (n_mb + n_stage - 1), 4)}
        else:
            net = Llama(cfgm, device=dev)
            zrg = G.get_nccl_group_zr()
            self.engine = TrainEngine(
                net, mode="zero" if zrg.world_size > 1 else "local",
                group=zrg.comm.peer if zrg.world_size > 1 else None, heap=heap, optim=opt,
                micro_batches=n_mb, use_cuda_graph=False,
                bucket_mb=args.bucket_mb if args.bucket_mb > 0 else None,
                grad_sync=net.make_grad_sync())
            self.has_data = True
            replicas = zrg.world_size
            par = f"dp=1 zr={replicas} mp={mp}"
        self.mp_peer = mp_peer
        self.fused = fused
        self.shape = {"rows": mb_seqs * S, "d_model": cfgm.d_model, "d_ff": cfgm.d_ff, "mp": mp}
        # model FLOPs of one step (forward + backward): 6 per weight of the GEMMs and of the
        # vocabulary projection per token, plus causal attention (6 * S * d_model per token
        # and layer)
        self.flops_per_step = float(B * replicas * S) * (
            6.0 * (cfgm.n_layer * per_layer + cfgm.vocab * cfgm.d_model) +
            6.0 * cfgm.n_layer * S * cfgm.d_model)
        # the replica's batch is drawn on tensor-parallel rank 0 and broadcast over the group
        seed_rank = rank - self.mp_rank
        self.hx, self.hy, self.dx, self.dy = _token_pool(cfgm.vocab, B, S, seed_rank, dev, pool=4)
        self.samples_per_step = B * replicas
        self.h2d_bytes_per_step = B * S * 8 * 2
        self.config = {"model": f"llama {cfgm.n_layer}L d{cfgm.d_model} ff{cfgm.d_ff} "
                                f"h{cfgm.n_head} vocab{cfgm.vocab}",
                       "global_batch": B * replicas, "seq_len": S, "parallelism": par,
                       "micro_batches": n_mb, "optimizer": "adam fp32 master",
                       "tp": "fused all-gather->GEMM / GEMM->reduce-scatter over peer memory"
                       if fused else "NCCL all-reduce",
                       "l2": "working set exceeds L2; no explicit flush", "cuda_graph": False,
                       "bucket_mb": args.bucket_mb}
        if getattr(self, "which", 0) == 4:
            self.config["pipeline"] = self.pipeline
        if args.layers:
            self.config["reduced"] = f"{args.layers} layers: smoke run, not a benchmark number"

    def _bcast(self, x, y):
        if self.which == 4:
            return self.engine.broadcast_inputs(x, y)
        if self.mp_peer.world == 1:
            return x, y
        if not hasattr(self, "_bb"):
            self._bb = [self.mp_peer.heap.alloc(x.numel(), x.dtype).view(x.shape)
                        for _ in range(2)]
        for buf, t in zip(self._bb, (x, y)):
            if self.mp_peer.rank == 0:
                buf.copy_(t, non_blocking=True)
            self.mp_peer.broadcast(buf, 0)
        return self._bb[0], self._bb[1]

    def _run(self, x, y):
        if not self.has_data:
            return self.engine.step()
        x, y = self._bcast(x, y)
        return self.engine.step(x, y)

    def step_dev(self, i):
        n = len(self.dx)
        return self._run(self.dx[i % n], self.dy[i % n])

    def step_e2e(self, i):
        n = len(self.hx)
        if not self.has_data:
            return self.engine.step()
        if self.mp_rank == 0:       # pinned host -> device on the rank that owns the batch
            return self._run(self.hx[i % n].to(self.dx[0].device, non_blocking=True),
                             self.hy[i % n].to(self.dx[0].device, non_blocking=True))
        return self._run(self.dx[0], self.dy[0])   # placeholders: overwritten by the broadcast


class ResNetDP(Workload):
    """Config 2: dp with 2-bit gradient quantisation (error feedback), ResNet-50, bf16,
    3 x 224 x 224 inputs, batch 256 per GPU, SGD momentum 0.9.  The host batch is bf16
    channels-last (what the loader hands over); labels int64."""

    def __init__(self, args, world, rank, dev, impl):
        import torch
        self.impl = impl
        B, HW = args.micro_batch or 256, args.seq or 224
        layers = (3, 4, 6, 3) if not args.layers else (1,) * 4
        torch.manual_seed(1234)
        if impl == "ours":
            from necklace_b200.comm.symm import SymmetricHeap
            from necklace_b200.models.resnet import ResNet
            from necklace_b200.parallel.engine import GradCompConfig, OptimConfig, TrainEngine
            net = ResNet(1000, layers, 64, device=dev)
            nparam = sum(p.numel() for p in net.parameters())
            heap = SymmetricHeap(int(nparam * (2 + 2 + 0.25 + 1) * 1.05) + (64 << 20))
            self.engine = TrainEngine(
                net, mode="dp", group=heap.peer_group(), heap=heap,
                optim=OptimConfig("sgd", lr=0.1, beta1=0.9),
                grad_comp=GradCompConfig(grad_comp_threshold=args.grad_comp_threshold),
                use_cuda_graph=not args.no_graph,
                bucket_mb=args.bucket_mb if args.bucket_mb > 0 else None)
            self._step = self.engine.step
        else:
            sys.path.insert(0, os.path.join(ROOT, "baseline"))
            from torch_resnet import TorchDDPTrainer
            self._step = TorchDDPTrainer(dev, world, rank, layers).step
        g = torch.Generator().manual_seed(100 + rank)
        pool = 3
        self.hx = [torch.randn(B, HW, HW, 3, generator=g).bfloat16().pin_memory()
                   for _ in range(pool)]
        self.hy = [torch.randint(0, 1000, (B,), generator=g).pin_memory() for _ in range(pool)]
        self.dx, self.dy = [t.to(dev) for t in self.hx], [t.to(dev) for t in self.hy]
        self._xb, self._yb = torch.empty_like(self.dx[0]), torch.empty_like(self.dy[0])
        self.samples_per_step = B * world
        self.h2d_bytes_per_step = B * HW * HW * 3 * 2 + B * 8
        self.config = {"model": "resnet50" if not args.layers else "resnet [1,1,1,1]",
                       "global_batch": B * world, "image": f"3x{HW}x{HW}", "seq_len": 0,
                       "parallelism": f"dp={world}",
                       "grad_compression": f"2-bit, threshold {args.grad_comp_threshold}, error "
                                           "feedback" if impl == "ours" else "none (DDP)",
                       "optimizer": "sgd momentum 0.9, fp32 master",
                       "l2": "activations exceed L2; no explicit flush",
                       "cuda_graph": impl == "ours" and not args.no_graph,
                       "bucket_mb": args.bucket_mb}
        if args.layers:
            self.config["reduced"] = "one block per stage: smoke run, not a benchmark number"

    def step_dev(self, i):
        n = len(self.dx)
        return self._step(self.dx[i % n], self.dy[i % n])

    def step_e2e(self, i):
        n = len(self.hx)
        if self.impl == "ours" and self.engine.use_cuda_graph:
            return self._step(self.hx[i % n], self.hy[i % n])   # copied into the static inputs
        self._xb.copy_(self.hx[i % n], non_blocking=True)
        self._yb.copy_(self.hy[i % n], non_blocking=True)
        return self._step(self._xb, self._yb)


def build_workload(args, world, rank, dev, impl):
    if args.config == 3:
        return GPT2Zero(args, world, rank, dev, impl)
    if args.config == 2:
        return ResNetDP(args, world, rank, dev, impl)
    if impl != "ours":
        raise SystemExit(f"--impl {impl} has no arm for config {args.config}")
    return LlamaHybrid(args, world, rank, dev, args.config)


def timed_regions(wl, args, world, dev, clocks=True):
    """Warm-up, the device-timed region (CUDA events around exactly K steps, barrier +
    synchronize on both sides) and the end-to-end region; returns (dev_ms, e2e_ms, clocks,
    first_loss, last_loss), both times as the max over ranks."""
    import torch
    import torch.distributed as dist

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    W = max(args.warmup, 3)
    for i in range(W):
        loss = wl.step_dev(i)
    sync_all()
    first_loss = float(loss.float().item())
    sampler = ClockSampler(dev.index) if clocks else None
    if sampler:
        sampler.start()
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        loss = wl.step_dev(i)
    e1.record()
    sync_all()
    dev_ms = e0.elapsed_time(e1)

    # end to end: every step copies its batch from pinned host memory and its loss is copied
    # to pinned host memory; the host reads the loss of step i once its copy has finished,
    # while step i+1 is already enqueued (deferred logging, as a training loop does)
    sync_all()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    loss_pin = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(2)]
    loss_ev = [torch.cuda.Event() for _ in range(2)]
    last_loss = first_loss
    f0.record()
    for i in range(args.steps):
        loss = wl.step_e2e(i)
        loss_pin[i & 1].copy_(loss.float().reshape(1), non_blocking=True)
        loss_ev[i & 1].record()
        if i > 0:
            loss_ev[(i - 1) & 1].synchronize()
            last_loss = float(loss_pin[(i - 1) & 1][0])
    loss_ev[(args.steps - 1) & 1].synchronize()
    last_loss = float(loss_pin[(args.steps - 1) & 1][0])
    f1.record()
    sync_all()
    e2e_ms = f0.elapsed_time(f1)
    ck = sampler.stop() if sampler else None
    # pipeline stages other than the last one have no loss (they report 0): the maximum over
    # ranks is the loss of a rank that computed one
    t = torch.tensor([dev_ms, e2e_ms, first_loss, last_loss], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0]), float(t[1]), ck, float(t[2]), float(t[3])


def comm_roofline(wl, world, dev, peaks):
    """Standalone CUDA-event timing of the fused reduce-scatter + Adam + all-gather kernel on
    the engine's own buffers against its floor: the slower of its NVLink bytes per direction
    over the measured 770 GB/s peer bandwidth and its HBM bytes over the measured copy
    bandwidth.  (The kernel updates the weights; it runs after all timed regions.)"""
    import torch
    import torch.distributed as dist
    eng = wl.engine
    if eng is None or not getattr(eng, "sharded", False):
        return None
    f, o = eng.flat, eng.optim
    n, W = f.numel, world
    reps = 5

    def run():
        for b in range(len(eng.buckets)):
            eng._fired.discard(b)
            eng._launch_bucket(b, side=False)

    eng._fired = set()
    run()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / reps], dtype=torch.float64, device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms[0])
    link_bytes = (W - 1) / W * n * 2                 # per direction: gradients in, parameters out
    hbm_bytes = n * 2 / W * (W + 1) + n / W * 4 * 6 + n * 2   # grads read, fp32 state r/w, params
    floor_ms = max(link_bytes / 770e9, hbm_bytes / (peaks.get("hbm_gbs", 6550.0) * 1e9)) * 1e3
    return {"rs_opt_ag": {"ms": round(ms, 4), "nvlink_bytes_per_dir": int(link_bytes),
                          "hbm_bytes": int(hbm_bytes), "floor_ms": round(floor_ms, 4),
                          "frac_of_measured_roofline": round(floor_ms / ms, 3)}}


def tp_roofline(wl, world, dev, peaks):
    """CUDA-event time of the fused all-gather -> GEMM and GEMM -> reduce-scatter kernels on
    the layer shapes of the tensor-parallel group (attention and MLP pair, one micro-batch of
    rows), run as they alternate in a block, against their floors: the slower of FLOPs over
    the measured sustained bf16 GEMM rate and the bytes that cross NVLink per direction over
    the measured 770 GB/s peer bandwidth.  Max over all ranks (every group runs at once)."""
    import torch
    import torch.distributed as dist
    grp, sh = wl.mp_peer, wl.shape
    if not wl.fused or grp is None or grp.world == 1:
        return None
    W, M, C, F = grp.world, sh["rows"], sh["d_model"], sh["d_ff"]
    r8 = lambda v: v // 8 * 8
    gemm_peak = peaks.get("bf16_tflops_sustained", 1401.1) * 1e12
    out, iters = {}, 5
    for name, n1, k2 in (("attention", r8(3 * C // W), r8(C // W)), ("mlp", r8(2 * F // W), r8(F // W))):
        xf = grp.heap.alloc(M * C, torch.bfloat16).view(M, C)
        xf.normal_()
        w1 = (torch.randn(n1, C, device=dev) * 0.02).bfloat16()
        x2 = (torch.randn(M, k2, device=dev) * 0.5).bfloat16()
        w2 = (torch.randn(C, k2, device=dev) * 0.02).bfloat16()
        for _ in range(2):
            grp.ag_gemm(xf, w1)
            grp.gemm_rs(x2, w2)
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(iters)]
        for e in evs:
            e[0].record()
            grp.ag_gemm(xf, w1)
            e[1].record()
            grp.gemm_rs(x2, w2)
            e[2].record()
        torch.cuda.synchronize()
        t = torch.tensor([sum(e[0].elapsed_time(e[1]) for e in evs) / iters,
                          sum(e[1].elapsed_time(e[2]) for e in evs) / iters],
                         dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        link = (W - 1) / W * M * C * 2
        for kern, ms, fl in (("ag_gemm", float(t[0]), 2.0 * M * n1 * C),
                             ("gemm_rs", float(t[1]), 2.0 * M * C * k2)):
            floor = max(fl / gemm_peak, link / 770e9) * 1e3
            out[f"{kern}_{name}"] = {"ms": round(ms, 4), "flops": fl, "nvlink_bytes_per_dir": int(link),
                                     "floor_ms": round(floor, 4),
                                     "frac_of_measured_roofline": round(floor / ms, 3)}
    return out


def cpu_plumbing_arm(args):
    """Config 1: trainer mode ``no`` on the CPU, LeNet, batch 100, SGD 0.01, 3 epochs of 600
    steps, one scheduler and one worker over ZeroMQ ipc (``examples/dp/train_mnist_dp.py``),
    against a plain single-process PyTorch loop on the same host.  Host wall-clock: there is no
    device.  The first epoch is warm-up, the other two are timed."""
    import subprocess
    import tempfile
    import torch
    work = tempfile.mkdtemp(prefix="nkb-c1-")
    script = os.path.join(ROOT, "examples", "dp", "train_mnist_dp.py")
    svr, out = f"ipc://{work}/s.ipc", os.path.join(work, "o.json")
    procs = [subprocess.Popen([sys.executable, script, "-r", "scheduler", "-w", "1", "-u", svr,
                               "-e", "3"], stdout=subprocess.DEVNULL, stderr=subprocess.STDOUT),
             subprocess.Popen([sys.executable, script, "-r", "worker", "-w", "1", "-k", "0", "-u",
                               f"ipc://{work}/w.ipc", "-s", svr, "-t", "no", "-e", "3", "--no-cuda",
                               "--log-interval", "0", "--out", out],
                              stdout=subprocess.DEVNULL, stderr=subprocess.STDOUT)]
    codes = []
    for p in procs:
        try:
            codes.append(p.wait(timeout=900))
        except subprocess.TimeoutExpired:
            p.kill()
            codes.append(-9)
    if codes != [0, 0]:
        print(json.dumps({"impl": "ours", "config": 1, "error": f"exit codes {codes}"}))
        return 1
    r = json.load(open(out))
    secs, steps = sum(r["epoch_seconds"][1:]), sum(r["epoch_steps"][1:])
    value = 100.0 * steps / secs
    # the stock loop: same network, batch, optimizer, and the same synthetic dataset and
    # in-process loader, so that the difference is the scheduler / worker / hook plumbing
    import torch.nn.functional as F
    from necklace_b200.data.dtldngn import DataLoaderNgnBase
    from necklace_b200.data.dtset import SyntheticDataset
    from necklace_b200.models.lenet import LeNet
    torch.manual_seed(1)
    net = LeNet()
    opt = torch.optim.SGD(net.parameters(), lr=0.01)
    loader = DataLoaderNgnBase(SyntheticDataset(60000, (1, 28, 28), classes=10, seed=1),
                               batch_size=100, last_batch="discard")

    def epoch(n):
        k = 0
        for x, y in loader:
            opt.zero_grad()
            loss = F.cross_entropy(net(x), y)
            loss.backward()
            opt.step()
            loss.item()
            k += 1
            if k == n:
                break
    epoch(50)
    t0 = time.time()
    epoch(600)
    base = 600 * 100.0 / (time.time() - t0)
    print(json.dumps({
        "metric": "samples/sec (host wall-clock; CPU plumbing configuration)",
        "value": round(value, 1), "unit": "samples/s", "n_gpus": 0, "steps": steps, "warmup": 600,
        "ms_per_step": round(secs / steps * 1e3, 3), "higher_is_better": True,
        "vs_baseline": round(value / base, 3), "dtype": "fp32", "data": "synthetic",
        "impl": "ours",
        "config": {"model": "lenet", "global_batch": 100, "parallelism": "no (1 scheduler + 1 "
                   "worker over ZeroMQ ipc)", "optimizer": "sgd 0.01", "epochs": 3,
                   "host_threads": torch.get_num_threads()},
        "baseline": {"impl": "single-process PyTorch loop over the same dataset and loader, same "
                             "host", "value": round(base, 1)},
        "loss_last": r["epoch_loss"][-1]}), flush=True)
    return 0


def necklace_launcher_arm(args):
    """Config 3 through the framework's own process model: every rank of the launch starts
    one worker of ``examples/gpt2/train_gpt2_necklace.py`` (scheduler / worker services over
    ZeroMQ, ZeRO trainer with the native engine, peer-memory communicator), rank 0 also the
    scheduler.  The workers time K steps with CUDA events from a trainer hook; every step
    copies its batch from pinned host memory, so the number is an end-to-end one."""
    import subprocess
    import tempfile
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    tag = os.environ.get("MASTER_PORT", str(os.getpid())) if world > 1 else str(os.getpid())
    work = os.path.join(tempfile.gettempdir(), f"nkb-launch-{tag}")
    os.makedirs(work, exist_ok=True)
    script = os.path.join(ROOT, "examples", "gpt2", "train_gpt2_necklace.py")
    W, K = max(args.warmup, 3), args.steps
    B = args.micro_batch or 8
    env = dict(os.environ)
    for k in list(env):           # the workers rendezvous through the scheduler, not torchrun
        if k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT", "GROUP_RANK",
                 "ROLE_RANK", "LOCAL_WORLD_SIZE", "ROLE_WORLD_SIZE", "GROUP_WORLD_SIZE") or \
                k.startswith("TORCHELASTIC_"):
            env.pop(k)
    svr = f"ipc://{work}/svr.ipc"
    procs = []
    if rank == 0:
        procs.append(subprocess.Popen(
            [sys.executable, script, "-r", "scheduler", "-w", str(world), "-u", svr, "-e", "1",
             "--model", "medium" if args.model == "gpt2-medium" else "tiny"],
            stdout=open(os.path.join(work, "sched.log"), "w"), stderr=subprocess.STDOUT, env=env))
    out = os.path.join(work, f"rank{rank}.json")
    cmd = [sys.executable, script, "-r", "worker", "-w", str(world), "-k", str(rank), "-g",
           str(local_rank), "-u", f"ipc://{work}/w{rank}.ipc", "-s", svr, "-x", "peer",
           "--model", "medium" if args.model == "gpt2-medium" else "tiny", "--micro-batch", str(B),
           "--time-steps", str(K), "--time-warmup", str(W), "--out", out]
    if world > 1:
        cmd += ["-t", "dp+zr", "-dpsz", "1", "-zrsz", str(world)]
    if not args.no_graph:
        cmd.append("--graph")
    sampler = ClockSampler(local_rank)
    sampler.start()
    procs.append(subprocess.Popen(cmd, stdout=open(os.path.join(work, f"w{rank}.log"), "w"),
                                  stderr=subprocess.STDOUT, env=env))
    try:
        procs[-1].wait(timeout=600)
    except subprocess.TimeoutExpired:
        pass
    clocks = sampler.stop()
    for p in procs:                 # exactly the children started above
        if p.poll() is None:
            try:
                p.wait(timeout=30)
            except subprocess.TimeoutExpired:
                p.kill()
    if rank != 0:
        return 0
    res = []
    for r in range(world):
        f = os.path.join(work, f"rank{r}.json")
        t_end = time.time() + 60
        while not os.path.exists(f) and time.time() < t_end:
            time.sleep(0.2)
        if not os.path.exists(f):
            tail = open(os.path.join(work, f"w{r if r == 0 else 0}.log")).read()[-300:]
            print(json.dumps({"impl": "ours", "launcher": "necklace",
                              "error": f"worker {r} wrote no result: {tail}"}))
            return 1
        res.append(json.load(open(f)))
    ms = max(r["ms"] for r in res)
    S = 1024 if args.model == "gpt2-medium" else 128
    value = B * world * K / (ms / 1e3)
    print(json.dumps({
        "metric": METRIC, "value": round(value, 2), "unit": "samples/s", "n_gpus": world,
        "steps": K, "warmup": W, "ms_per_step": round(ms / K, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours", "launcher": "necklace",
        "config": {"model": args.model, "global_batch": B * world, "seq_len": S,
                   "parallelism": f"dp+zr (zr={world})", "optimizer": "adam fp32 master",
                   "process_model": "scheduler + one worker per GPU over ZeroMQ, "
                                    "trainer zroppd.TrainerMPOPPytorch(engine='native'), "
                                    "comm_type peer", "cuda_graph": not args.no_graph,
                   "l2": "working set exceeds L2; no explicit flush"},
        "clocks": clocks,
        "e2e": {"value": round(value, 2), "unit": "samples/s", "ms_per_step": round(ms / K, 3),
                "h2d_bytes_per_step": B * S * 8 * 2, "d2h_bytes_per_step": 0,
                "note": "same run: the trainer copies every batch from pinned host memory"},
        "loss_last": res[0]["loss"]}), flush=True)
    return 0


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)
    if args.config == 1:
        return cpu_plumbing_arm(args)
    if args.launcher == "necklace":
        return necklace_launcher_arm(args)

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:  # noqa: BLE001
        pass

    from necklace_b200 import _lib
    wl = build_workload(args, world, rank, dev, args.impl)
    dev_ms, e2e_ms, clocks, first_loss, last_loss = timed_regions(wl, args, world, dev)
    wl.finish()
    W = max(args.warmup, 3)
    value = wl.samples_per_step * args.steps / (dev_ms / 1e3)
    e2e_value = wl.samples_per_step * args.steps / (e2e_ms / 1e3)
    cfg = dict(wl.config)
    cfg["tokens_per_s"] = round(value * cfg.get("seq_len", 0), 1)
    out = {
        "metric": METRIC, "value": round(value, 2), "unit": "samples/s", "n_gpus": world,
        "steps": args.steps, "warmup": W, "ms_per_step": round(dev_ms / args.steps, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "impl": args.impl, "config": cfg, "clocks": clocks,
        "e2e": {"value": round(e2e_value, 2), "unit": "samples/s",
                "ms_per_step": round(e2e_ms / args.steps, 3),
                "h2d_bytes_per_step": int(wl.h2d_bytes_per_step), "d2h_bytes_per_step": 4},
        "loss_first": round(first_loss, 4), "loss_last": round(last_loss, 4),
    }
    if args.impl == "ours":
        per_step = getattr(wl.engine, "launches_per_step", None)
        if per_step is None:                      # eager engine: count one more step
            torch.cuda.synchronize()
            l0 = _lib.launch_count
            wl.step_dev(0)
            torch.cuda.synchronize()
            per_step = _lib.launch_count - l0
        out["gpu_launches"] = int(per_step * args.steps)

    # ---- the other half of the metric and the comparison, measured in this invocation ----
    if args.impl == "ours" and args.config == 2 and not args.no_baseline:
        try:
            base = ResNetDP(args, world, rank, dev, "torch")
            b_ms, b_e2e, _, _, _ = timed_regions(base, args, world, dev, clocks=False)
            b_val = base.samples_per_step * args.steps / (b_ms / 1e3)
            out["vs_baseline"] = round(value / b_val, 3)
            out["baseline"] = {"impl": "stock torch DistributedDataParallel (NCCL, cuDNN, bf16 "
                                       "autocast, channels-last, uncompressed gradients), same "
                                       "box, same invocation",
                               "value": round(b_val, 2), "ms_per_step": round(b_ms / args.steps, 3),
                               "e2e_value": round(base.samples_per_step * args.steps /
                                                  (b_e2e / 1e3), 2)}
        except Exception as e:  # noqa: BLE001
            out["baseline"] = {"error": repr(e)[:300]}
    if args.impl == "ours" and args.config == 3:
        if world > 1 and not args.layers:
            try:
                # step time of the same model with no collective at all (every rank updates
                # all parameters locally): what is left is the communication that backward
                # and the optimizer do not hide
                local = GPT2Zero(args, world, rank, dev, "ours", mode="local")
                l_ms, _, _, _, _ = timed_regions(local, args, world, dev, clocks=False)
                out["exposed_comm_ms"] = round((dev_ms - l_ms) / args.steps, 3)
                out["no_comm_ms_per_step"] = round(l_ms / args.steps, 3)
                del local
            except Exception as e:  # noqa: BLE001
                out["exposed_comm_ms"] = None
                out["exposed_comm_error"] = repr(e)[:200]
            try:
                out["roofline"] = comm_roofline(wl, world, dev, peaks)
            except Exception as e:  # noqa: BLE001
                out["roofline"] = {"error": repr(e)[:200]}
        elif world == 1:
            out["exposed_comm_ms"] = 0.0
        flops = None
        if args.model == "gpt2-medium" and not args.layers:
            flops = 18.8e12 * (cfg["global_batch"] / world) / 8     # matmul + causal attention
            out["roofline_compute"] = {
                "tflops_per_gpu": round(flops / (dev_ms / args.steps / 1e3) / 1e12, 1),
                "frac_of_measured_sustained_bf16": round(
                    flops / (dev_ms / args.steps / 1e3) / 1e12 /
                    peaks.get("bf16_tflops_sustained", 1401.1), 3)}
        if not args.no_baseline:
            try:
                base = GPT2Zero(args, world, rank, dev, "torch")
                b_ms, b_e2e, _, _, _ = timed_regions(base, args, world, dev, clocks=False)
                b_val = base.samples_per_step * args.steps / (b_ms / 1e3)
                out["vs_baseline"] = round(value / b_val, 3)
                out["baseline"] = {"impl": "stock torch.distributed (NCCL reduce-scatter / "
                                           "all-gather, cuBLAS, SDPA, fused AdamW), same box, "
                                           "same invocation",
                                   "value": round(b_val, 2),
                                   "ms_per_step": round(b_ms / args.steps, 3),
                                   "e2e_value": round(base.samples_per_step * args.steps /
                                                      (b_e2e / 1e3), 2)}
            except Exception as e:  # noqa: BLE001
                out["baseline"] = {"error": repr(e)[:200]}
    if args.impl == "ours" and args.config in (4, 5):
        step_s = dev_ms / args.steps / 1e3
        out["roofline_compute"] = {
            "model_tflop_per_step": round(wl.flops_per_step / 1e12, 1),
            "tflops_per_gpu": round(wl.flops_per_step / step_s / world / 1e12, 1),
            "frac_of_measured_sustained_bf16": round(
                wl.flops_per_step / step_s / world / 1e12 /
                peaks.get("bf16_tflops_sustained", 1401.1), 3)}
        try:
            out["roofline"] = tp_roofline(wl, world, dev, peaks)
        except Exception as e:  # noqa: BLE001
            out["roofline"] = {"error": repr(e)[:200]}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
