"""CPU model of the epoch-flag protocol used by the peer-memory collectives.

Ranks are threads, "peer memory" is a shared list per rank, and every access goes through
the same steps as the kernels (write my epoch into every peer's slot, wait until every
peer's epoch shows up in mine, epochs only grow).  The model checks the properties the
kernels rely on: no rank passes barrier k before all ranks entered it, data written before
the barrier is visible after it, skewed ranks cannot be confused by flags of a later call,
and a missing peer produces a timeout instead of a hang."""
import random
import threading
import time


class Rank(threading.Thread):
    def __init__(self, r, world, mem, flags, calls, log, absent=None, timeout=2.0):
        super().__init__(daemon=True)
        self.r, self.world, self.mem, self.flags = r, world, mem, flags
        self.calls, self.log, self.absent, self.timeout = calls, log, absent, timeout
        self.status = 0
        self.epoch = 0

    def barrier(self, value):
        for p in range(self.world):
            self.flags[p][self.r] = max(self.flags[p][self.r], value)   # st.release.sys
        t0 = time.time()
        for p in range(self.world):
            while self.flags[self.r][p] < value:                           # ld.acquire.sys
                if time.time() - t0 > self.timeout:
                    self.status = 5
                    return False
                time.sleep(0)
        return True

    def run(self):
        rng = random.Random(self.r)
        for k in range(self.calls):
            if self.absent == (self.r, k):
                return  # this rank dies between calls
            e = self.epoch + 1
            self.mem[self.r] = (k, self.r * 1000 + k)          # produce my data for call k
            time.sleep(rng.random() * 0.002)
            if not self.barrier(2 * e - 1):
                return
            # every peer's data of call k must be visible now
            for p in range(self.world):
                got = self.mem[p]
                self.log.append((self.r, k, p, got[0] >= k))
            if not self.barrier(2 * e):
                return
            self.epoch = e


def _run(world, calls, absent=None, timeout=2.0):
    mem = [None] * world
    flags = [[0] * world for _ in range(world)]
    log = []
    ranks = [Rank(r, world, mem, flags, calls, log, absent, timeout) for r in range(world)]
    for t in ranks:
        t.start()
    for t in ranks:
        t.join(timeout=30)
    return ranks, log


def test_barrier_orders_data_for_skewed_ranks():
    ranks, log = _run(4, 50)
    assert all(t.status == 0 and t.epoch == 50 for t in ranks)
    assert len(log) == 4 * 50 * 4 and all(ok for *_, ok in log)


def test_missing_peer_times_out_instead_of_hanging():
    t0 = time.time()
    ranks, _ = _run(3, 10, absent=(1, 4), timeout=0.3)
    assert time.time() - t0 < 10
    survivors = [t for t in ranks if t.r != 1]
    assert all(t.status == 5 for t in survivors)        # reported, not hung
    assert all(t.epoch in (4, 5) for t in survivors)     # nobody ran past the broken call
