"""PipelineEngine (1F1B, shapes negotiated once, posted receives) against a single-process
run: two and three gloo ranks on CPU."""
import os
import socket

import pytest
import torch
import torch.nn as nn


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _parts(n_stage):
    torch.manual_seed(0)
    dims = [12, 16, 16, 16, 5][: n_stage] + [5]
    dims = [12] + [16] * (n_stage - 1) + [5]
    return [nn.Linear(dims[i], dims[i + 1]) for i in range(n_stage)]


class _First(nn.Module):
    def __init__(self, lin):
        super().__init__()
        self.lin = lin

    def forward(self, x):
        return torch.tanh(self.lin(x))


class _Last(nn.Module):
    def __init__(self, lin):
        super().__init__()
        self.lin = lin

    def forward(self, h, y):
        return ((self.lin(h) - y) ** 2).mean()


class _Whole(nn.Module):
    def __init__(self, parts):
        super().__init__()
        self.parts = nn.ModuleList(parts)

    def forward(self, x, y):
        for p in self.parts[:-1]:
            x = torch.tanh(p(x))
        return ((self.parts[-1](x) - y) ** 2).mean()


def _data(m=4):
    g = torch.Generator().manual_seed(2)
    return torch.randn(m * 3, 12, generator=g), torch.randn(m * 3, 5, generator=g)


def _worker(rank, world, port, q, prepost):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from necklace_b200.parallel import pipeline as P
    from necklace_b200.parallel.engine import OptimConfig
    from necklace_b200.parallel.pipe_engine import PipelineEngine
    P.create_channels([list(range(world))])
    parts = _parts(world)
    lin = parts[rank]
    net = _First(lin) if rank < world - 1 else _Last(lin)
    eng = PipelineEngine(net, stage=rank, pp_ranks=list(range(world)), micro_batches=4,
                         optim=OptimConfig("sgd", lr=0.1, beta1=0.0), prepost=prepost)
    x, y = _data()
    losses = []
    for _ in range(3):
        l = eng.step(x, y) if rank == 0 else eng.step()
        losses.append(float(l))
    q.put((rank, [p.detach().numpy().copy() for p in lin.parameters()], losses))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("world,prepost", [(2, True), (3, True), (2, False)])
def test_pipeline_engine_matches_single_process(world, prepost):
    import torch.multiprocessing as mp
    from necklace_b200.parallel.engine import OptimConfig, TrainEngine
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, prepost)) for r in range(world)]
    for p in procs:
        p.start()
    res = {r: (w, l) for r, w, l in (q.get(timeout=200) for _ in procs)}
    for p in procs:
        p.join(60)
    parts = _parts(world)
    ref = TrainEngine(_Whole(parts), optim=OptimConfig("sgd", lr=0.1, beta1=0.0), micro_batches=4)
    x, y = _data()
    ref_losses = [float(ref.step(x, y)) for _ in range(3)]
    for r in range(world):
        for a, b in zip(res[r][0], parts[r].parameters()):
            assert torch.allclose(torch.from_numpy(a), b.detach(), atol=1e-5), r
    assert all(abs(a - b) < 1e-5 for a, b in zip(res[world - 1][1], ref_losses))


# ------------------------------------------------------------ Llama, pp=2 x mp=2 on 4 gloo ranks
def _llama_cfg(**kw):
    from necklace_b200.models.llama import LlamaConfig
    return LlamaConfig(n_layer=4, d_model=64, n_head=4, d_ff=128, vocab=256, max_seq=32,
                       dtype=torch.float32, **kw)


def _llama_tokens(n=4):
    tok = torch.randint(0, 256, (n, 33), generator=torch.Generator().manual_seed(5))
    return tok[:, :-1].contiguous(), tok[:, 1:].contiguous()


def _hybrid_worker(rank, world, port, q):
    """dp+pp+mp with dp=1, pp=2, mp=2: ranks (stage, mp) = (0,0) (0,1) (1,0) (1,1)."""
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from necklace_b200.comm.symm import TorchGroup
    from necklace_b200.models.llama import Llama
    from necklace_b200.parallel import pipeline as P
    from necklace_b200.parallel.engine import OptimConfig
    from necklace_b200.parallel.pipe_engine import PipelineEngine
    mp_groups = [[0, 1], [2, 3]]
    pp_groups = [[0, 2], [1, 3]]
    mp_pg = [dist.new_group(g) for g in mp_groups]
    P.create_channels(pp_groups)
    stage, mpr = rank // 2, rank % 2
    tp = TorchGroup(mp_pg[stage], ranks=mp_groups[stage])
    cfg = _llama_cfg(tp_group=tp)
    net = Llama(cfg, layers=range(stage * 2, stage * 2 + 2), with_embed=stage == 0,
                with_head=stage == 1)

    class Stage(nn.Module):
        def __init__(s):
            super().__init__()
            s.net = net

        def forward(s, x, targets=None):
            return s.net(x, targets, batch=2)

    eng = PipelineEngine(Stage(), stage=stage, pp_ranks=pp_groups[mpr], micro_batches=2,
                         optim=OptimConfig("sgd", lr=0.05, beta1=0.0),
                         grad_sync=net.make_grad_sync())
    x, y = _llama_tokens()
    losses = []
    for _ in range(2):
        l = eng.step(x, y) if stage == 0 else eng.step()
        losses.append(float(l))
    q.put((rank, losses, {n: p.detach().numpy().copy() for n, p in net.named_parameters()}))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(400)
def test_llama_pipeline_with_tensor_parallel_stages_matches_single_process():
    import torch.multiprocessing as mp
    from necklace_b200 import checkpoint as ck
    from necklace_b200.models.llama import Llama
    from necklace_b200.parallel.engine import OptimConfig, TrainEngine
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_hybrid_worker, args=(r, 4, port, q)) for r in range(4)]
    for p in procs:
        p.start()
    res = {r: (l, sd) for r, l, sd in (q.get(timeout=300) for _ in procs)}
    for p in procs:
        p.join(60)
    ref_net = Llama(_llama_cfg())
    ref = TrainEngine(ref_net, optim=OptimConfig("sgd", lr=0.05, beta1=0.0), micro_batches=2)
    x, y = _llama_tokens()
    ref_losses = [float(ref.step(x, y)) for _ in range(2)]
    assert all(abs(a - b) < 1e-4 for a, b in zip(res[2][0], ref_losses)), (res[2][0], ref_losses)
    full = dict(ref_net.named_parameters())
    for stage in range(2):
        names = res[2 * stage][1].keys()
        for name in names:
            shards = [torch.from_numpy(res[2 * stage + m][1][name]) for m in range(2)]
            gname = name
            if name.startswith("blocks."):
                i = int(name.split(".")[1])
                gname = "blocks.%d.%s" % (i + 2 * stage, name.split(".", 2)[2])
            want = full[gname].detach()
            if shards[0].shape != want.shape:
                tp_model = Llama(_llama_cfg(mp=2, mp_rank=0))
                _, dim, stride = ck._tp_attrs(dict(tp_model.named_parameters())[gname])
                if gname in ("embed.wte", "head.w_out"):
                    dim, stride = 0, 1
                got = ck.tp_concat(shards, dim, stride)
            else:
                got = shards[0]
            assert torch.allclose(got, want, atol=2e-5), gname
