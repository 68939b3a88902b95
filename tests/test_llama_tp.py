"""Tensor-parallel Llama in the sequence-parallel layout (all-gather -> GEMM, GEMM ->
reduce-scatter, vocabulary-parallel embedding and cross-entropy) against the unsharded model:
two gloo ranks on CPU with the unfused stand-in group, and the tensor-parallel checkpoint
round trip (save at mp=2, load at mp=1 and mp=4)."""
import os
import socket

import pytest
import torch


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cfg(**kw):
    from necklace_b200.models.llama import LlamaConfig
    return LlamaConfig(n_layer=2, d_model=64, n_head=4, d_ff=128, vocab=200, max_seq=32,
                       dtype=torch.float32, **kw)


def _tokens():
    tok = torch.randint(0, 200, (2, 33), generator=torch.Generator().manual_seed(3))
    return tok[:, :-1].contiguous(), tok[:, 1:].contiguous()


def _tp_worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from necklace_b200.comm.symm import TorchGroup
    from necklace_b200.models.llama import Llama
    grp = TorchGroup()
    model = Llama(_cfg(tp_group=grp))
    x, y = _tokens()
    loss = model(x, y)
    loss.backward()
    # numpy arrays: tensors would travel as shared-memory handles that die with this process
    out = {"loss": float(loss.detach()),
           "grads": {n: p.grad.numpy().copy() for n, p in model.named_parameters()},
           "sd": {n: p.detach().numpy().copy() for n, p in model.named_parameters()}}
    q.put((rank, out))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_sequence_parallel_llama_matches_unsharded():
    import torch.multiprocessing as mp
    from necklace_b200 import checkpoint as ck
    from necklace_b200.models.llama import Llama
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    world = 2
    procs = [ctx.Process(target=_tp_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=200) for _ in procs)
    for p in procs:
        p.join(60)
    for r in res.values():
        r["grads"] = {k: torch.from_numpy(v) for k, v in r["grads"].items()}
        r["sd"] = {k: torch.from_numpy(v) for k, v in r["sd"].items()}
    ref = Llama(_cfg())
    x, y = _tokens()
    loss = ref(x, y)
    loss.backward()
    assert abs(res[0]["loss"] - float(loss)) < 1e-4 and abs(res[1]["loss"] - float(loss)) < 1e-4
    for name, p in ref.named_parameters():
        tp = dict(Llama(_cfg(mp=2, mp_rank=0)).named_parameters())[name]
        sharded, dim, stride = ck._tp_attrs(tp)
        if sharded or name in ("embed.wte", "head.w_out"):
            dim = dim if sharded else 0
            full = ck.tp_concat([res[r]["grads"][name] for r in range(world)], dim, stride)
            wfull = ck.tp_concat([res[r]["sd"][name] for r in range(world)], dim, stride)
            assert torch.equal(wfull, p.detach()), name
        else:  # replicated parameters (norm weights): each rank holds the gradient of its rows
            full = res[0]["grads"][name] + res[1]["grads"][name]
        assert torch.allclose(full, p.grad, atol=2e-5, rtol=1e-4), name


def test_tp_checkpoint_reshards_between_mp_sizes():
    """Shards built at mp=2 assemble into exactly the mp=1 weights (packed q/k/v and gate/up
    blocks de-interleaved) and re-split into exactly the mp=4 shards."""
    from necklace_b200 import checkpoint as ck
    from necklace_b200.models.llama import Llama

    class G:
        def __init__(self, world, rank):
            self.world, self.rank = world, rank

    def build(mp, r):
        cfg = _cfg(tp_group=G(mp, r))
        cfg.vocab = 512          # a multiple of 128 * 4: the same padding at every mp size
        return Llama(cfg)

    shards = [build(2, r) for r in range(2)]
    full = {}
    for name, p in shards[0].named_parameters():
        sharded, dim, stride = ck._tp_attrs(p)
        parts = [dict(s.named_parameters())[name].detach() for s in shards]
        full[name] = ck.tp_concat(parts, dim, stride) if sharded else parts[0]
    one = build(1, 0)
    for name, p in one.named_parameters():
        assert torch.equal(full[name], p.detach()), name
    for r in range(4):
        want = build(4, r)
        got = build(4, r)
        with torch.no_grad():
            for p in got.parameters():
                p.zero_()
        ck.load_tp_state_dict(got, full, ws=4, rank=r)
        for (n, a), (_, b) in zip(got.named_parameters(), want.named_parameters()):
            assert torch.equal(a, b), (n, r)


def _zr_mp_worker(rank, world, port, q):
    """dp+zr+mp with zr=2 (outer), mp=2 (inner): mp groups [0,1] [2,3], zr groups [0,2] [1,3]."""
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from necklace_b200.comm.symm import TorchGroup
    from necklace_b200.models.llama import Llama
    from necklace_b200.parallel.engine import OptimConfig, TrainEngine
    mp_groups, zr_groups = [[0, 1], [2, 3]], [[0, 2], [1, 3]]
    mp_pg = [dist.new_group(g) for g in mp_groups]
    zr_pg = [dist.new_group(g) for g in zr_groups]
    tp = TorchGroup(mp_pg[rank // 2], ranks=mp_groups[rank // 2])
    zr = TorchGroup(zr_pg[rank % 2], ranks=zr_groups[rank % 2])
    net = Llama(_cfg(tp_group=tp))
    eng = TrainEngine(net, mode="zero", group=zr, optim=OptimConfig("adam", lr=1e-2),
                      micro_batches=2, grad_sync=net.make_grad_sync())
    tok = torch.randint(0, 200, (8, 33), generator=torch.Generator().manual_seed(9))
    mine = tok[(rank // 2) * 4:(rank // 2) * 4 + 4]      # each zr rank is a data-parallel replica
    losses = [float(eng.step(mine[:, :-1].contiguous(), mine[:, 1:].contiguous())) for _ in range(2)]
    q.put((rank, losses, {n: p.detach().numpy().copy() for n, p in net.named_parameters()}))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_zero_over_tensor_parallel_llama_with_accumulation_matches_single_process():
    import torch.multiprocessing as mp
    from necklace_b200 import checkpoint as ck
    from necklace_b200.models.llama import Llama
    from necklace_b200.parallel.engine import OptimConfig, TrainEngine
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_zr_mp_worker, args=(r, 4, port, q)) for r in range(4)]
    for p in procs:
        p.start()
    res = {r: (l, sd) for r, l, sd in (q.get(timeout=250) for _ in procs)}
    for p in procs:
        p.join(60)
    ref_net = Llama(_cfg())
    ref = TrainEngine(ref_net, optim=OptimConfig("adam", lr=1e-2), micro_batches=4)
    tok = torch.randint(0, 200, (8, 33), generator=torch.Generator().manual_seed(9))
    # global batch = 2 replicas x 2 micro-batches of 2 sequences; same order of micro-batches
    for _ in range(2):
        ref.step(tok[:, :-1].contiguous(), tok[:, 1:].contiguous())
    tp_model = Llama(_cfg(mp=2, mp_rank=0))
    rel = lambda a, b: float((a - b).norm() / (b.norm() + 1e-12))
    for name, want in ref_net.named_parameters():
        sharded, dim, stride = ck._tp_attrs(dict(tp_model.named_parameters())[name])
        if name in ("embed.wte", "head.w_out"):
            sharded, dim, stride = True, 0, 1
        shards = [torch.from_numpy(res[m][1][name]) for m in range(2)]
        got = ck.tp_concat(shards, dim, stride) if sharded else shards[0]
        assert rel(got, want.detach()) < 2e-3, (name, rel(got, want.detach()))
        other = [torch.from_numpy(res[2 + m][1][name]) for m in range(2)]
        assert torch.equal(shards[0], other[0]), name      # the two zr ranks agree
