"""Failure detection without touching a GPU: host heartbeats (in process and over a TCPStore between processes,
one of which exits), and the bounded-wait contract of the device mailbox on its executable model."""
import os
import socket
import time

import pytest
import torch.multiprocessing as mp

from jetspec_b200.parallel.health import OK, TIMEOUT, DictStore, Heartbeat, MailboxModel, PeerFailure


class FakeClock:
    def __init__(self):
        self.t = 0.0

    def __call__(self):
        return self.t


def test_heartbeat_detects_stall_error_and_absence():
    store, clock = DictStore(), FakeClock()
    a = Heartbeat(store, 0, 3, timeout=5.0, clock=clock)
    b = Heartbeat(store, 1, 3, timeout=5.0, clock=clock)
    a.check()                                    # rank 2 has not reported yet, but the grace period is not over
    clock.t = 4.0
    b.beat()
    a.check()
    clock.t = 6.0
    with pytest.raises(PeerFailure) as e:        # rank 2 never showed up
        a.check()
    assert e.value.rank == 2
    c = Heartbeat(store, 2, 3, timeout=5.0, clock=clock)
    a2 = Heartbeat(store, 0, 3, timeout=5.0, clock=clock)
    a2.check()
    clock.t = 10.0
    b.beat(); c.beat()
    a2.check()
    clock.t = 14.0
    c.beat()
    a2.check()
    clock.t = 16.5                                # rank 1 stuck since t = 10
    with pytest.raises(PeerFailure) as e:
        a2.check()
    assert e.value.rank == 1 and "no progress" in e.value.why
    b.fail("CUDA error in step 7")
    with pytest.raises(PeerFailure) as e:
        Heartbeat(store, 0, 3, timeout=5.0, clock=clock).check()
    assert "CUDA error" in e.value.why


def test_mailbox_bounded_wait_reports_lost_and_late_flags():
    mb = MailboxModel()
    mb.push([3, 42, 0])
    assert mb.wait(limit=10) == (OK, [3, 42, 0])
    mb.delay_polls = 5                            # the flag store arrives late: still delivered within the limit
    mb.push([1, 7, 0])
    assert mb.wait(limit=10) == (OK, [1, 7, 0])
    mb.drop_flag = True                           # the flag store is lost: the wait gives up with a status
    mb.push([9, 9, 9])
    status, payload = mb.wait(limit=50)
    assert status == TIMEOUT and payload is None
    mb.drop_flag = False                          # the protocol stays usable afterwards (round numbers stay aligned)
    mb.push([2, 5, 1])
    assert mb.wait(limit=10) == (OK, [2, 5, 1])


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _hb_worker(rank: int, world: int, port: int, result_path: str):
    from torch.distributed import TCPStore
    store = TCPStore("127.0.0.1", port, world, rank == 0, timeout=__import__("datetime").timedelta(seconds=30))
    hb = Heartbeat(store, rank, world, timeout=1.5)
    if rank == 1:
        for _ in range(3):                        # three healthy steps, then this rank goes away without a word
            time.sleep(0.1)
            hb.beat()
        time.sleep(4.0)                           # (keeps the store connection open while rank 0 finds out)
        return
    deadline, failure = time.time() + 20, None
    while time.time() < deadline:                 # rank 0: between steps, look at the peers before the next launch
        time.sleep(0.1)
        hb.beat()
        try:
            hb.check()
        except PeerFailure as e:
            failure = (e.rank, e.why)
            break
    with open(result_path, "w") as f:
        f.write(repr(failure))


def test_a_rank_that_stops_is_noticed_between_steps(tmp_path):
    path = str(tmp_path / "hb.txt")
    mp.spawn(_hb_worker, args=(2, _free_port(), path), nprocs=2, join=True)
    rank, why = eval(open(path).read())
    assert rank == 1 and "no progress" in why
