"""Thread-based models of the flag protocols the peer-memory kernels use
(ops/csrc/comm_kernels.cu): monotonically increasing epochs, one flag slot per
(owner, writer), bounded waits.  The models run the same steps in the same
order as the kernels, with random delays to provoke every interleaving the
two-half staging scheme and the double-buffered receive slots must survive."""
import random
import threading
import time


class Pads:
    """pads[owner][writer]: last epoch `writer` announced to `owner`."""

    def __init__(self, world):
        self.v = [[0] * world for _ in range(world)]

    def signal_all(self, rank, epoch):
        for peer in range(len(self.v)):
            self.v[peer][rank] = epoch                   # st.release.sys to every peer's pad

    def wait_all(self, rank, epoch, timeout_s=5.0):
        t0 = time.time()
        while any(x < epoch for x in self.v[rank]):      # ld.acquire.sys on the own pad
            if time.time() - t0 > timeout_s:
                return False                             # the kernel would set status = 3
            time.sleep(0)
        return True


def test_small_allreduce_two_halves_are_enough():
    world, calls = 4, 60
    pads = Pads(world)
    stage = [[None, None] for _ in range(world)]         # two halves per rank
    results = [[None] * calls for _ in range(world)]
    errors = []

    def rank_main(rank):
        rng = random.Random(rank)
        for k in range(1, calls + 1):
            if rng.random() < 0.3:
                time.sleep(rng.random() * 0.002)         # skew between ranks
            stage[rank][k & 1] = (rank + 1) * k          # copy the input into the own half
            pads.signal_all(rank, k)
            if not pads.wait_all(rank, k):
                errors.append(("timeout", rank, k))
                return
            results[rank][k - 1] = sum(stage[r][k & 1] for r in range(world))   # rank order
    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(world)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    assert not errors, errors
    for k in range(1, calls + 1):
        want = sum((r + 1) * k for r in range(world))
        assert all(results[r][k - 1] == want for r in range(world)), k


def test_missing_peer_times_out_instead_of_hanging():
    pads = Pads(2)
    pads.signal_all(0, 1)                                # rank 1 never arrives
    t0 = time.time()
    assert pads.wait_all(0, 1, timeout_s=0.05) is False
    assert time.time() - t0 < 1.0


def test_double_buffered_receive_slots_are_never_overwritten_early():
    """Reduce-scatter as the fused path does it: every rank stores its partial
    row block into its slot of the owner's receive buffer, barrier, the owner
    sums its slots.  Buffers alternate; a fast rank may already be storing
    op k+1 (other buffer) while a slow one still sums op k, but it cannot reach
    op k+2 (same buffer) before the slow rank has passed the barrier of op k+1."""
    world, ops = 3, 50
    pads = Pads(world)
    recv = [[[None] * world for _ in range(2)] for _ in range(world)]   # recv[owner][buf][writer]
    errors = []

    def rank_main(rank):
        rng = random.Random(100 + rank)
        for k in range(1, ops + 1):
            buf = k & 1
            for owner in [(rank + 1 + i) % world for i in range(world)]:  # rotated owner order
                recv[owner][buf][rank] = (k, rank, owner)
            pads.signal_all(rank, k)
            if not pads.wait_all(rank, k):
                errors.append(("timeout", rank, k))
                return
            if rng.random() < 0.4:
                time.sleep(rng.random() * 0.002)          # slow consumer
            got = list(recv[rank][buf])                   # the owner sums its slots
            if got != [(k, w, rank) for w in range(world)]:
                errors.append(("overwritten", rank, k, got))
                return
    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(world)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    assert not errors, errors[:3]
