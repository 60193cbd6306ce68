"""The replicate dimension of the engine (dp_replicate of the reference's parallel dims, torchtitan's HSDP and DDP,
src/tplr/model_factory.py:122-176) on 4 gloo ranks: 2 replicas x 2 shards and 4 replicas x 1 rank take the same
steps as one sharded group of four."""

from test_distributed_cpu import launch


def test_hybrid_and_replicated_layouts_equal_the_fully_sharded_one():
    res = launch(4, [], worker="_gloo_hsdp_worker.py", port=29671, timeout=1500)
    assert len(res) == 4
    for r in res:
        for tag in ("adamw", "muon"):
            assert r[tag + "_moved"] > 1e-4, r
            for name in ("hybrid", "hybrid_sharded_params", "replicated"):
                d = r[f"{tag}_{name}"]
                # the same sums in another order (fp32): agreement to rounding, far below the change of the weights.
                # Newton-Schulz multiplies the small singular directions of a gradient by several hundred, rounding
                # differences included, and a changed coefficient can change the top-k selection: Muon gets a
                # looser bound on the weights and none on the payload.
                if tag == "adamw":
                    assert d["loss"] < 1e-5 and d["weights"] < 0.01 * r[tag + "_moved"] and d["payload"] < 1e-6, (tag, name, d)
                else:
                    assert d["loss"] < 1e-4 and d["weights"] < 0.1 * r[tag + "_moved"], (tag, name, d)
        # the neurons' path: torchtitan.dp_replicate -> engine topology, inner steps, public outer step with the
        # gathered payloads handed from the master rank to the leader of every copy
        assert r["trainer_moved"] > 1e-3, r
        for replicas in (2, 4):
            d = r[f"trainer_{replicas}"]
            assert d["steps"] == [2, 2] and d["weights"] < 1e-6, d
            assert d["topology"][1:3] == [4 // replicas, replicas], d
    assert sorted(tuple(r["trainer_2"]["topology"]) for r in res) == [(0, 2, 2, 0), (0, 2, 2, 1), (1, 2, 2, 0), (1, 2, 2, 1)]
