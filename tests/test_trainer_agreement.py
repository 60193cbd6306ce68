"""Step boundaries of ``Trainer.inner_steps`` are agreed between the ranks (gloo, 2 ranks).

The optimizer step contains collectives, so a rank must never enter it (or leave the loop) on a signal that
only it has seen.  One rank's window clock (or stop request) flips in the middle of an accumulation group; both
ranks finish that group, agree there, and leave together."""

from test_distributed_cpu import launch


def test_ranks_leave_the_window_together_when_one_sees_the_change_early():
    res = launch(2, [], worker="_gloo_trainer_worker.py", port=29647, timeout=300)
    assert len(res) == 2
    for mode in ("window", "stop"):
        a, b = res[0][mode], res[1][mode]
        assert a == b, (mode, a, b)
        # the flip came during the second group of 3 micro-batches: two optimizer steps, six micro-batches per rank
        assert a["inner_steps"] == 2 and a["adam_step"] == 2 and a["batch_count"] == 12, (mode, a)
