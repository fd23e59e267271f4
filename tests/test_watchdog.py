"""Host watchdog of an expert-parallel group: heartbeats through the rendezvous store and events of the exchanges.

Every failure is made on the host: a heartbeat that stops, an event that never reports completion, a rank that leaves
between steps.  No GPU is involved.
"""
import os
import socket
import time
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe_oracle as O
from oracle.ep_standins import OracleKernels
from torchair_b200 import ep
from torchair_b200.watchdog import EpGroupFailed, EpWatchdog


class FakeStore:
    def __init__(self):
        self.kv = {}

    def set(self, k, v):
        self.kv[k] = v.encode() if isinstance(v, str) else v

    def get(self, k):
        return self.kv[k]

    def check(self, keys):
        return all(k in self.kv for k in keys)


class FakeClock:
    def __init__(self):
        self.t = 100.0

    def __call__(self):
        return self.t


class FakeEvent:
    def __init__(self, done=False):
        self.done = done

    def query(self):
        return self.done


def _pair(timeout=2.0):
    store, clock = FakeStore(), FakeClock()
    a = EpWatchdog("g", store, 0, 2, interval_s=0.5, timeout_s=timeout, clock=clock)
    b = EpWatchdog("g", store, 1, 2, interval_s=0.5, timeout_s=timeout, clock=clock)
    for w in (a, b):        # what start() does, without the thread
        w._seen = {r: (None, clock()) for r in range(2) if r != w.rank}
    return store, clock, a, b


def test_heartbeats_that_move_keep_the_group_alive():
    _, clock, a, b = _pair()
    for _ in range(20):
        clock.t += 0.5
        a.poll_once()
        b.poll_once()
    a.check()
    b.check()
    assert a.failure is None and b.failure is None


def test_a_silent_rank_is_reported_after_the_timeout_and_not_before():
    _, clock, a, b = _pair(timeout=2.0)
    for _ in range(4):
        clock.t += 0.5
        b.poll_once()
        a.poll_once()
    for _ in range(4):              # rank 1 stops beating; 2.0 s of silence is still within the limit
        clock.t += 0.5
        a.poll_once()
    a.check()
    clock.t += 0.5
    a.poll_once()
    with pytest.raises(EpGroupFailed, match="rank 1 has not been heard from"):
        a.check()


def test_a_rank_that_never_wrote_a_heartbeat_is_reported_too():
    _, clock, a, _ = _pair(timeout=1.0)
    for _ in range(3):
        clock.t += 0.5
        a.poll_once()
    with pytest.raises(EpGroupFailed, match="rank 1"):
        a.check()


def test_an_exchange_that_does_not_finish_aborts_the_communicator_once():
    store, clock, a, b = _pair(timeout=2.0)
    calls = []
    a._abort = lambda: calls.append(1)
    done, stuck = FakeEvent(done=True), FakeEvent(done=False)
    a.watch(done, "the dispatch exchange")
    a.watch(stuck, "the combine exchange")
    for _ in range(4):
        clock.t += 0.5
        a.poll_once()
        b.poll_once()
    assert a.failure is None and len(a._pending) == 1          # the finished event was dropped, the other is still followed
    clock.t += 0.5
    b.poll_once()
    a.poll_once()
    with pytest.raises(EpGroupFailed, match="the combine exchange was enqueued 2.5 s ago"):
        a.check()
    a.poll_once()
    assert calls == [1] and a.aborted


def test_constructor_rejects_inconsistent_limits():
    with pytest.raises(ValueError):
        EpWatchdog("g", FakeStore(), 2, 2)
    with pytest.raises(ValueError):
        EpWatchdog("g", FakeStore(), 0, 2, interval_s=1.0, timeout_s=0.5)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        ep.register_ep_group("ep_wd", dist.group.WORLD, watchdog={"interval_s": 0.1, "timeout_s": 1.0})
        cfg = O.CONFIGS["cfg0"]
        x, ids, wt = O.make_tokens(cfg, 0, rank)
        outs = ep.dispatch(OracleKernels, x, ids, "ep_wd", world, rank, cfg.E, 2, 1)     # a step with everybody present
        assert ep.watchdog_of("ep_wd").failure is None
        dist.barrier()
        if rank == 1:                       # leaves between steps: no collective of its own is in flight
            ep.watchdog_of("ep_wd").stop()
            q.put((rank, "left"))
            return
        deadline = time.time() + 20.0
        while ep.watchdog_of("ep_wd").failure is None and time.time() < deadline:
            time.sleep(0.05)
        t0 = time.time()
        try:
            ep.dispatch(OracleKernels, x, ids, "ep_wd", world, rank, cfg.E, 2, 1)
            q.put((rank, "error", "the dispatch after the peer left did not raise"))
        except EpGroupFailed as exc:
            q.put((rank, "raised", str(exc), time.time() - t0, outs[0].shape[0]))
    except Exception:
        q.put((rank, "error", traceback.format_exc()))


def test_a_rank_that_leaves_between_steps_is_reported_before_the_next_exchange():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(2):
        item = q.get(timeout=120)
        got[item[0]] = item
    for p in procs:
        p.join(timeout=30)
    assert got[1][1] == "left", got[1]
    assert got[0][1] == "raised", got[0]
    assert "rank 1 has not been heard from" in got[0][2]
    assert got[0][3] < 0.5          # raised on the host, without waiting for a collective to time out
