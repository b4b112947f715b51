"""The hand-over protocol of the peer-memory transport (palimpsa_b200.parallel.chain_peer) on the CPU.

Ranks are threads; the peer-mapped buffers and 64-bit flags are shared Python objects; the library's two stream
operations are stand-ins with the same meaning (``peer_wait`` blocks until the flag has reached the value,
``peer_signal`` stores it), executed at once, which is what an in-order stream does.  Checked over many
back-to-back calls with random delays in every rank: each rank reads exactly the state its predecessor produced for
THAT call (the ``ack`` flag keeps a fast producer from overwriting a buffer that has not been read), the chain's
result equals the sequential recurrence in both directions, ranks in the middle take the relay path, and nothing
deadlocks (a wait that does not complete within its limit fails the test instead of hanging it)."""
import random
import threading
import time

import pytest
import torch

from palimpsa_b200 import parallel


class _Shared:
    def __init__(self, world, n):
        self.cv = threading.Condition()
        self.flags = {}
        self.inbox = {(r, d): torch.zeros(n, dtype=torch.float64) for r in range(world) for d in (0, 1)}
        self.waits = 0


class _Lib:
    """Stand-in for the two C-ABI calls chain_peer makes."""

    def __init__(self, shared):
        self.s = shared

    def palimpsa_peer_wait(self, flag, value, timeout_ms, poison, stream):
        with self.s.cv:
            self.s.waits += 1
            ok = self.s.cv.wait_for(lambda: self.s.flags.get(flag, 0) >= value, timeout=timeout_ms / 1000.0)
        assert ok, f"wait on {flag} for {value} ran out: the protocol deadlocked"
        return 0

    def palimpsa_peer_signal(self, flag, value, stream):
        with self.s.cv:
            assert value >= self.s.flags.get(flag, 0), "sequence numbers only grow"
            self.s.flags[flag] = value
            self.s.cv.notify_all()
        return 0


class _Link:
    def __init__(self, shared, rank):
        self.s, self.rank, self.epoch, self.timeout_ms = shared, rank, [0, 0], 20000

    def inbox(self, d):
        return self.s.inbox[(self.rank, d)]

    def inbox_ptr(self, rank, d):
        return (rank, d)

    def flag_ptr(self, rank, d, ack):
        return ("flag", rank, d, ack)


@pytest.mark.parametrize("world", [2, 4])
def test_chain_peer_hands_every_state_over_exactly_once(world, monkeypatch):
    n = 8
    # forward-only calls (nothing but the ack flag stops rank 0 from running ahead), then forward + backward pairs,
    # then a run in the other direction alone
    plan = [(0,)] * 15 + [(0, 1)] * 10 + [(1,)] * 15
    calls = len(plan)
    shared = _Shared(world, n)
    monkeypatch.setattr(parallel.L, "lib", lambda: _Lib(shared))
    decay = [0.5 + 0.1 * r for r in range(world)]
    seen = {(r, d, c): None for r in range(world) for d in (0, 1) for c in range(calls)}
    relays = [0] * world
    errors = []

    def total(r, d, c):                       # what rank r adds in call c, direction d
        return torch.full((n,), float(1 + r + 10 * c + 100 * d), dtype=torch.float64)

    def rank_main(r):
        rng = random.Random(r)
        link = _Link(shared, r)
        try:
            for c in range(calls):
                for d in plan[c]:
                    def local(inc, out_ptr, want_out, d=d, c=c):
                        time.sleep(rng.random() * 0.002)           # a slow consumer: the producer must not run ahead
                        seen[(r, d, c)] = None if inc is None else inc.clone()
                        if want_out:
                            x = torch.zeros(n, dtype=torch.float64) if inc is None else inc
                            shared.inbox[out_ptr].copy_(decay[r] * x + total(r, d, c))

                    def relay(inc, tot, out_ptr):
                        relays[r] += 1
                        shared.inbox[out_ptr].copy_(decay[r] * inc + tot)

                    parallel.chain_peer(link, d, r, world, local, None, prepare=lambda d=d, c=c: total(r, d, c),
                                        relay=relay)
                    time.sleep(rng.random() * 0.001)
        except BaseException as e:            # noqa: BLE001  (reported by the main thread)
            errors.append((r, repr(e)))

    threads = [threading.Thread(target=rank_main, args=(r,), daemon=True) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(120)
    assert not errors, errors
    assert not any(t.is_alive() for t in threads)
    for c in range(calls):
        for d in plan[c]:
            order = list(range(world)) if d == 0 else list(range(world - 1, -1, -1))
            state = None
            for r in order:                   # the sequential recurrence along the chain
                got = seen[(r, d, c)]
                if state is None:
                    assert got is None
                    state = decay[r] * torch.zeros(n, dtype=torch.float64) + total(r, d, c)
                else:
                    assert got is not None and torch.equal(got, state), (c, d, r, got, state)
                    state = decay[r] * state + total(r, d, c)
    middle = [r for r in range(world) if 0 < r < world - 1]
    hops = sum(len(p) for p in plan)
    assert all(relays[r] == hops for r in middle) and all(relays[r] == 0 for r in (0, world - 1))
