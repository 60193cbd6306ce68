"""Worker for test_distributed_cpu.py: sharded engine with 8-bit payload values on CPU (gloo, 2 ranks) against the
unsharded engine on the same state."""

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from templar_b200.models.llama import ModelArgs, build_model  # noqa: E402
from templar_b200.parallel.window_engine import EngineConfig, WindowEngine  # noqa: E402


def _fill(eng, name_seed):
    """Deterministic error feedback and weight change, addressed by parameter name (layouts may differ in padding)."""
    st = eng.store
    eng.snapshot()
    for s in eng.layout.specs:
        g = torch.Generator().manual_seed(name_seed + s.index)
        ef = torch.randn(s.numel, generator=g) * 1e-3
        dw = torch.randn(s.numel, generator=g) * 1e-3
        a, b = max(s.offset, st.lo), min(s.offset + s.numel, st.hi)
        if a < b:
            eng.ef[a - st.lo: b - st.lo].copy_(ef[a - s.offset: b - s.offset])
            st.master_shard[a - st.lo: b - st.lo].add_(dw[a - s.offset: b - s.offset])


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    args = ModelArgs(dim=128, n_layers=1, n_heads=2, vocab_size=256, intermediate_size=256, max_seq_len=32)
    cfg = EngineConfig(topk=8, quantize=True, quant_bins=16)
    eng = WindowEngine(build_model(args, seed=2), cfg, rank=rank, world_size=world)
    one = WindowEngine(build_model(args, seed=2), cfg)
    for e in (eng, one):
        _fill(e, 40)
        e.compress()
    eng.merge_own_payload()                       # already merged inside compress(): must not sum twice
    out = {"val": 0.0, "ef": 0.0, "codes_equal": 1.0, "table": 0.0, "ef_scale": float(one.ef.abs().max())}
    st = eng.store
    for s in eng.layout.specs:
        r = one.layout.by_name[s.name]
        _, v = eng.layout.payload_views(eng.own_idx, eng.own_val, s.name)
        _, w = one.layout.payload_views(one.own_idx, one.own_val, s.name)
        i1, _ = eng.layout.payload_views(eng.own_idx, eng.own_val, s.name)
        i0, _ = one.layout.payload_views(one.own_idx, one.own_val, s.name)
        assert torch.equal(i0, i1), s.name
        out["val"] = max(out["val"], float((v - w).abs().max()))
        _, c1 = eng.layout.payload_views(eng.own_idx, eng._q_codes, s.name)
        _, c0 = one.layout.payload_views(one.own_idx, one._q_codes, s.name)
        out["codes_equal"] = min(out["codes_equal"], float((c0 == c1).float().mean()))
        out["table"] = max(out["table"], float((eng._q_table[s.index] - one._q_table[r.index]).abs().max()))
        a, b = max(s.offset, st.lo), min(s.offset + s.numel, st.hi)
        if a < b:
            mine = eng.ef[a - st.lo: b - st.lo]
            ref = one.ef[r.offset + (a - s.offset): r.offset + (b - s.offset)]
            out["ef"] = max(out["ef"], float((mine - ref).abs().max()))
    res = [None] * world
    dist.all_gather_object(res, out)
    if rank == 0:
        print("RESULT " + json.dumps(res))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
