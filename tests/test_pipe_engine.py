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
