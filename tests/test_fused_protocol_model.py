"""CPU model of the flag protocols of the two GEMM kernels that are fused with a collective
(``csrc/gemm_sm100.cu``): ranks are threads, peer memory is shared lists, every access goes
through the same steps as the kernels.

All-gather in front (push): a rank enters the call (start barrier), raises the flags of its
own row blocks, stores its blocks into every peer's gather buffer and raises the block's flag
*there*; the consumer walks the blocks starting with its own and waits on each flag.  There
is no barrier at the end.  Checked: a consumer never sees a block of an earlier or later
call although ranks are skewed and the buffers are reused by every call.

Reduce-scatter behind: one warp opens the gate once every rank has entered the call; tiles
of other ranks' rows are stored into the owner's staging slab (after the gate) and flagged;
own tiles come last in the walk, wait for the peers' flags and add the slabs.  Checked: sums
are those of the current call for skewed ranks with reused staging, nothing deadlocks with
the own-rows-last walk, and an absent rank ends in a timeout status on the others.
"""
import random
import threading
import time

TIMEOUT = 5.0


class Shared:
    def __init__(self, world, blocks, nb):
        self.bar = [[0] * world for _ in range(world)]            # [owner][from]
        self.gather = [[None] * (world * blocks) for _ in range(world)]
        self.ag_flags = [[0] * (world * blocks) for _ in range(world)]
        self.stage = [[[None] * (blocks * nb) for _ in range(world)] for _ in range(world)]
        self.t_flags = [[[0] * (blocks * nb) for _ in range(world)] for _ in range(world)]
        self.go = [0] * world
        self.errors = []


def _wait(pred, status, who):
    t0 = time.time()
    while not pred():
        if time.time() - t0 > TIMEOUT:
            status[who] = 5
            return False
        time.sleep(0)
    return True


def _barrier(sh, r, world, value, status):
    for p in range(world):
        sh.bar[p][r] = max(sh.bar[p][r], value)
    return all(_wait(lambda p=p: sh.bar[r][p] >= value, status, r) for p in range(world))


def _rank(sh, r, world, blocks, nb, calls, status, absent, seed):
    rng = random.Random(seed * 100 + r)
    nap = lambda: time.sleep(rng.random() * 0.002) if rng.random() < 0.3 else None
    epoch = 0
    for k in range(calls):
        if absent == (r, k):
            return
        # ---------------- all-gather -> GEMM, call number e
        epoch += 1
        e = epoch
        for b in range(blocks):                       # the layer before wrote my shard
            sh.gather[r][r * blocks + b] = ("ag", k, r, b)
        nap()
        if not _barrier(sh, r, world, 2 * e - 1, status):
            return
        for b in range(blocks):
            sh.ag_flags[r][r * blocks + b] = e

        def push():
            for j in range(world - 1):                # peers below me first
                q = (r + world - 1 - j) % world
                for b in range(blocks):
                    sh.gather[q][r * blocks + b] = sh.gather[r][r * blocks + b]
                    nap()
                    sh.ag_flags[q][r * blocks + b] = e
        copier = threading.Thread(target=push, daemon=True)
        copier.start()
        for i in range(world * blocks):               # the GEMM: own rows first
            blk = (r * blocks + i) % (world * blocks)
            if not _wait(lambda: sh.ag_flags[r][blk] >= e, status, r):
                return
            want = ("ag", k, blk // blocks, blk % blocks)
            if sh.gather[r][blk] != want:
                sh.errors.append((r, k, "ag", blk, sh.gather[r][blk]))
            nap()
        copier.join()
        # ---------------- GEMM -> reduce-scatter, call number e
        epoch += 1
        e = epoch

        def gate():
            if _barrier(sh, r, world, 2 * e - 1, status):
                sh.go[r] = e
        g = threading.Thread(target=gate, daemon=True)
        g.start()
        for i in range(world):                        # owners: next rank first, myself last
            o = (r + 1 + i) % world
            for t in range(blocks * nb):
                part = (k + 1) * 1000 + r * 10 + t
                if o != r:
                    if not _wait(lambda: sh.go[r] >= e, status, r):
                        return
                    sh.stage[o][r][t] = part
                    nap()
                    sh.t_flags[o][r][t] = e
                else:
                    total = part
                    for src in range(world):
                        if src == r:
                            continue
                        if not _wait(lambda: sh.t_flags[r][src][t] >= e, status, r):
                            return
                        total += sh.stage[r][src][t]
                    want = sum((k + 1) * 1000 + s * 10 + t for s in range(world))
                    if total != want:
                        sh.errors.append((r, k, "rs", t, total, want))
        g.join()


def _run(world, blocks=2, nb=3, calls=6, absent=None, seed=0):
    sh = Shared(world, blocks, nb)
    status = [0] * world
    th = [threading.Thread(target=_rank, args=(sh, r, world, blocks, nb, calls, status, absent,
                                               seed), daemon=True) for r in range(world)]
    for t in th:
        t.start()
    for t in th:
        t.join(TIMEOUT * 6)
    assert not any(t.is_alive() for t in th), "a rank did not finish (deadlock)"
    return sh, status


def test_skewed_ranks_see_only_the_current_call():
    for world, seed in ((2, 1), (3, 2), (4, 3), (8, 4)):
        sh, status = _run(world, seed=seed)
        assert status == [0] * world
        assert sh.errors == []


def test_absent_rank_gives_timeout_status_not_a_hang():
    global TIMEOUT
    old, TIMEOUT = TIMEOUT, 0.3
    try:
        sh, status = _run(3, calls=4, absent=(1, 2))
    finally:
        TIMEOUT = old
    assert status[0] == 5 and status[2] == 5
    assert sh.errors == []


def test_accuracy_of_bf16_staged_partial_sums_at_mp4_k13824():
    """GEMM -> reduce-scatter stores the partial sums of the other ranks' rows as bf16 and
    keeps the own partial sum in fp32.  Emulated on the CPU for the widest case asked for
    (4 ranks, K = 13824 split four ways, bf16 operands): the root-mean-square error is less
    than twice that of rounding the exact sum once to bf16, and every element is within
    2^-8 * (sum of the |staged partial sums| + |result|) of the exact sum."""
    import torch
    torch.manual_seed(0)
    W, K, M, N = 4, 13824, 64, 96
    x = (torch.randn(M, K) * 0.5).bfloat16().double()
    w = (torch.randn(N, K) * 0.02).bfloat16().double()
    kp = K // W
    parts = [x[:, r * kp:(r + 1) * kp] @ w[:, r * kp:(r + 1) * kp].t() for r in range(W)]
    exact = sum(parts)
    once = exact.float().bfloat16().double()                     # unfused: fp32 sum, one rounding
    own = 2                                                      # any rank: its partial stays fp32
    fused = sum(p.float().double() if r == own else p.float().bfloat16().double()
                for r, p in enumerate(parts)).float().bfloat16().double()
    scale = exact.abs().mean()
    err_once = ((once - exact).pow(2).mean().sqrt() / scale).item()
    err_fused = ((fused - exact).pow(2).mean().sqrt() / scale).item()
    assert err_fused < 2.0 * err_once, (err_fused, err_once)
    # element-wise: every rounding is within the bf16 unit round-off (2^-8) of what it rounds
    u = 2.0 ** -8
    bound = u * (sum(p.abs() for r, p in enumerate(parts) if r != own) + exact.abs()) * 1.02
    assert bool(((fused - exact).abs() <= bound + 1e-12).all())
