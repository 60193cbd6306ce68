"""Properties of the flag-barrier state machine, on the host model (threads stand in for GPUs)."""

import random
import threading
import time

from templar_b200.parallel.flag_protocol import ST_OK, ST_WAIT_TIMEOUT, FlagBarrierModel


def _run(n, body):
    errs = []

    def wrap(r):
        try:
            body(r)
        except Exception as e:  # noqa: BLE001
            errs.append((r, repr(e)))

    ts = [threading.Thread(target=wrap, args=(r,)) for r in range(n)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(30)
    assert not errs and not any(t.is_alive() for t in ts), errs


def test_no_rank_leaves_an_epoch_before_all_arrived_and_writes_are_visible():
    n, epochs = 4, 40
    bar = FlagBarrierModel(n)
    data = [[0] * n for _ in range(n)]                     # data[owner][writer]: a peer store made before arriving
    arrived = [[False] * n for _ in range(epochs + 1)]

    def body(r):
        rng = random.Random(r)
        for e in range(1, epochs + 1):
            time.sleep(rng.random() * 1e-3)
            for peer in range(n):
                data[peer][r] = e                          # "push" into every peer's buffer
            arrived[e][r] = True
            assert bar.barrier(r, e) == ST_OK
            assert all(arrived[e]), (r, e)                 # nobody is released early
            assert all(v >= e for v in data[r]), (r, e)    # every peer's store is visible after the wait
            # a fast rank may already have pushed epoch e + 1 data: values only grow

    _run(n, body)
    assert bar.status == [ST_OK] * n


def test_missing_rank_gives_a_status_not_a_hang_and_a_late_arrival_heals():
    n = 3
    bar = FlagBarrierModel(n)
    out = {}

    def body(r):
        if r == 2:
            time.sleep(0.15)                               # skips epoch 1 (host-side failure injection) ...
            out[r] = bar.barrier(r, 2, timeout_s=2.0)      # ... and arrives at epoch 2 directly
            return
        t0 = time.monotonic()
        st = bar.barrier(r, 1, timeout_s=0.05)
        assert st & ST_WAIT_TIMEOUT and time.monotonic() - t0 < 1.0
        out[r] = bar.barrier(r, 2, timeout_s=2.0)          # epochs only grow: the late arrival satisfies epoch 2

    _run(n, body)
    assert out == {0: ST_OK, 1: ST_OK, 2: ST_OK}
    assert bar.status[2] == ST_OK and bar.status[0] & ST_WAIT_TIMEOUT


def test_repeated_and_out_of_date_arrivals_are_harmless():
    bar = FlagBarrierModel(2)
    bar.arrive(0, 3)
    bar.arrive(1, 3)
    assert bar.wait(0, 3, 0.01) == ST_OK and bar.wait(0, 2, 0.01) == ST_OK      # an older epoch is already satisfied
    bar.arrive(1, 3)                                                             # arriving twice changes nothing
    assert bar.wait(0, 3, 0.01) == ST_OK
    assert bar.wait(0, 4, 0.01) & ST_WAIT_TIMEOUT                                # the next epoch is not
