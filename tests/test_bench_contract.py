"""The benchmark's command line and the workload labels that both arms print (so that their `config` objects are the
same for the same arguments), checked without a GPU."""

import sys

import bench
from templar_b200.models.llama import PRESETS


def _args(argv):
    old = sys.argv
    sys.argv = ["bench.py", *argv]
    try:
        return bench.parse()
    finally:
        sys.argv = old


def test_defaults_are_the_headline_configuration():
    a = _args([])
    assert (a.gpus, a.impl, a.model, a.micro_batch, a.seq_len, a.accum, a.peers, a.topk) == (1, "ours", "1B", 8, 2048, 4, 8, 32)
    assert a.steps >= 1 and a.warmup >= 3 and a.values == "uint8" and a.outer_update == "sgd"
    assert not a.shard_params and a.replicas == 1


def test_both_arms_label_the_same_workload_identically():
    for argv, world in (([], 1), (["--gpus", "8"], 8), (["--model", "150M", "--micro-batch", "2", "--accum", "1"], 2)):
        ours = bench.config_labels(_args(argv), world)
        ref = bench.config_labels(_args([*argv, "--impl", "reference"]), world)
        assert ours == ref
        assert ours["global_batch"] == ours["micro_batch"] * ours["accum"] * world
        assert ("single GPU" in ours["parallelism"]) == (world == 1)
        # what differs between the arms (sharding mechanics, kernels) must not leak into the workload labels
        assert "shard" not in ours["model"] and "impl" not in ours


def test_label_shapes_match_the_presets():
    for name, text in bench.MODEL_DIMS.items():
        p = PRESETS[name]
        assert f"d{p.dim} " in text + " " and f"L{p.n_layers} " in text + " " and f"H{p.n_heads} " in text + " "
        assert f"F{p.ffn_hidden}" in text and f"V{p.vocab_size}" in text
        if p.kv_heads != p.n_heads:
            assert f"KV{p.kv_heads}" in text
