"""A validator, two miners and an evaluator as four separate processes on one machine, offline: nothing is wired by
hand (no fixed peers), the nodes find each other through the shared static chain and the directory store."""

from templar_b200 import localnet


def test_three_node_network_finds_its_peers_gathers_scores_and_is_evaluated(tmp_path):
    res = localnet.launch(tmp_path / "net", miners=2, windows=8, block_time=1.5, device="cpu", evaluator=True)
    tails = {k: open(v).read()[-1500:] for k, v in res["logs"].items()}
    assert all(rc == 0 for rc in res["returncodes"].values()), (res["returncodes"], tails)
    s = res["summary"]
    # the miners got the validator's peer list without --peers and gathered each other's gradients
    for uid, m in s["miners"].items():
        assert m["windows"] >= 5 and m["windows_with_gather"] >= 2 and m["global_step"] >= 2, (uid, m, tails[f"miner{uid}"])
    # the validator found both miners active, gathered both and scored them
    v = s["validator"]
    assert v["windows"] >= 4 and v["max_gathered"] == 2 and v["windows_with_scores"] >= 2, (v, tails["validator"])
    assert set(v["last_sync"]) <= {"2", "3"} and v["last_sync"]
    # the evaluator followed the published checkpoints (or, before the first one, took the baseline)
    assert s["evaluator"]["evaluations"] >= 1 and s["evaluator"]["last"]["perplexity"] > 1
