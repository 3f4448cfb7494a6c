"""Host-thread model of the flag protocol of the fused GEMM -> reduce-scatter kernel (csrc/gemm_comm.cu):
same state machine, ranks = threads, device memory = numpy arrays, random delays.  Checks that the
schedule has no circular wait (every run terminates), that epochs make the flags reset-free across calls,
and that double buffering + one barrier per call is enough to keep a rank from overwriting a partial tile
a slower peer is still reading.  A rank that never starts must turn into a timeout status, not a hang."""
import random
import threading
import time

import numpy as np
import pytest


class Model:
    def __init__(self, world, mbps, tiles_n, seed):
        self.world, self.mbps, self.tiles_n = world, mbps, tiles_n
        self.rng = random.Random(seed)
        nt = world * mbps * tiles_n
        self.partial = [[np.zeros(nt), np.zeros(nt)] for _ in range(world)]       # double buffered, per rank
        self.flags = [[np.zeros(nt, dtype=np.int64), np.zeros(nt, dtype=np.int64)] for _ in range(world)]
        self.out = [np.zeros(mbps * tiles_n) for _ in range(world)]
        self.barrier = threading.Barrier(world)
        self.status = [0] * world

    def wait(self, arr, idx, epoch, budget):
        t0 = time.time()
        while arr[idx] < epoch:
            if time.time() - t0 > budget:
                return False
            time.sleep(0)
        return True

    def call(self, rank, call_idx, value_of, budget=5.0, use_barrier=True):
        """One fused op on one rank.  ``value_of(rank, tile)`` is that rank's partial product of a tile."""
        w, mbps, tn = self.world, self.mbps, self.tiles_n
        epoch, buf = call_idx + 1, call_idx & 1
        if use_barrier:
            self.barrier.wait(timeout=30)
        sum_flags = np.zeros(mbps * tn, dtype=np.int64)
        peer_sum = np.zeros(mbps * tn)
        ok = [True]

        def reducer():          # runs beside the "GEMM": pulls peers' partials of this rank's rows
            for u in range(mbps * tn):
                acc = 0.0
                for d in range(1, w):
                    peer = (rank + d) % w
                    idx = rank * mbps * tn + u
                    if not self.wait(self.flags[peer][buf], idx, epoch, budget):
                        self.status[rank] = 640 + peer
                        ok[0] = False
                        return
                    acc += self.partial[peer][buf][idx]
                peer_sum[u] = acc
                sum_flags[u] = epoch

        t = threading.Thread(target=reducer)
        t.start()
        # tile schedule: the other ranks' row blocks first (rank+1, rank+2, ...), the own ones last
        for s in range(w):
            owner = (rank + 1 + s) % w
            for u in range(mbps * tn):
                if self.rng.random() < 0.3:
                    time.sleep(self.rng.random() * 1e-3)
                idx = owner * mbps * tn + u
                if owner != rank:
                    self.partial[rank][buf][idx] = value_of(rank, idx) + 1000.0 * epoch
                    self.flags[rank][buf][idx] = epoch                      # release after the data
                else:
                    if not self.wait(sum_flags, u, epoch, budget):
                        self.status[rank] = self.status[rank] or 635
                        t.join()
                        return False
                    self.out[rank][u] = value_of(rank, idx) + 1000.0 * epoch + peer_sum[u]
        t.join()
        return ok[0]


def _value(rank, idx):
    return float(rank + 1) * 0.5 + idx * 0.01


@pytest.mark.parametrize("world,seed", [(2, 0), (4, 1), (8, 2)])
def test_protocol_terminates_and_sums_over_several_calls(world, seed):
    m = Model(world, mbps=3, tiles_n=2, seed=seed)
    calls = 4
    results = [[] for _ in range(world)]

    def run(rank):
        for c in range(calls):
            assert m.call(rank, c, _value)
            results[rank].append(m.out[rank].copy())

    threads = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
        assert not t.is_alive(), "the protocol deadlocked"
    for rank in range(world):
        for c in range(calls):
            for u in range(6):
                idx = rank * 6 + u
                want = sum(_value(r, idx) + 1000.0 * (c + 1) for r in range(world))
                assert results[rank][c][u] == pytest.approx(want)
    assert m.status == [0] * world


def test_absent_peer_becomes_a_status_not_a_hang():
    m = Model(2, mbps=2, tiles_n=2, seed=3)
    t0 = time.time()
    assert m.call(0, 0, _value, budget=0.3, use_barrier=False) is False      # rank 1 never runs
    assert time.time() - t0 < 5.0
    assert m.status[0] in (641, 635)


def test_magic_number_division_is_exact_for_step_indices():
    """csrc/attn_bwd.cu FastDiv: n / d == (n * (0xffffffff // d + 1)) >> 32 for 1 < d < 65536 and 0 <= n < 65536
    (the kernel takes the plain division outside that range)."""
    import random
    rng = random.Random(0)
    cases = [(n, d) for d in (2, 3, 5, 7, 63, 64, 65, 130, 131, 260, 1024, 4097, 65535) for n in (0, 1, d - 1, d, d + 1, 65535)]
    cases += [(rng.randrange(65536), rng.randrange(2, 65536)) for _ in range(20000)]
    for n, d in cases:
        magic = (0xFFFFFFFF // d + 1) & 0xFFFFFFFF
        assert (n * magic) >> 32 == n // d, (n, d)
