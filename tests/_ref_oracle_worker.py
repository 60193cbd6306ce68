"""Worker for test_reference_oracle.py: runs the UNMODIFIED reference (installed under baseline/_ref, imported as
``tplr``) and this framework (``templar_b200``) side by side on CPU tensors and prints the largest differences."""

import copy
import json
import os
import sys
from types import SimpleNamespace

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import templar_b200 as ours  # noqa: E402
from baseline import ref_env  # noqa: E402

ref_env.prepare()
import tplr as ref  # noqa: E402  (the reference, from baseline/_ref)

assert os.path.realpath(ref.__file__).startswith(os.path.realpath(os.path.join(ROOT, "baseline", "_ref"))), ref.__file__


class Net(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.a = torch.nn.Linear(192, 128, bias=False)      # chunk grid 2 x 3 of 64 x 64
        self.b = torch.nn.Linear(128, 96, bias=False)       # rows 96: chunk edge 48
        self.n = torch.nn.LayerNorm(128)                    # 1-D tensors


def diff(a, b):
    return float((a.float() - b.float()).abs().max())


def main():
    out = {}
    torch.manual_seed(0)
    # 1. 12-bit packing
    idx = torch.randint(0, 4096, (7, 5, 32))
    pr, po = ref.compress.pack_12bit_indices(idx), ours.compress.pack_12bit_indices(idx)
    out["pack_equal"] = bool(torch.equal(pr, po))
    out["unpack_equal"] = bool(torch.equal(ref.compress.unpack_12bit_indices(pr, idx.shape),
                                           ours.compress.unpack_12bit_indices(po, idx.shape)))
    # 2. chunking + DCT, top-k, decompress, batch_decompress, with and without quantisation
    net = Net()
    worst = 0.0
    bytes_equal = True
    for use_dct in (False, True):
        for quant in (False, True):
            tr_r, tr_o = ref.compress.ChunkingTransformer(net, 64), ours.compress.ChunkingTransformer(net, 64)
            kw = dict(use_quantization=quant, quantization_bins=16, quantization_range=6)
            c_r, c_o = ref.compress.TopKCompressor(**kw), ours.compress.TopKCompressor(**kw)
            for name, p in net.named_parameters():
                x = torch.randn_like(p) * 1e-2
                e_r, e_o = tr_r.encode(x, use_dct=use_dct), tr_o.encode(x, use_dct=use_dct)
                worst = max(worst, diff(e_r, e_o))
                o_r, o_o = c_r.compress(e_r, 8), c_o.compress(e_o, 8)
                bytes_equal &= bool(torch.equal(o_r[0], o_o[0])) and tuple(o_r[2]) == tuple(o_o[2]) and o_r[3] == o_o[3]
                worst = max(worst, diff(o_r[1], o_o[1]))
                qp_r, qp_o = (o_r[4], o_o[4]) if quant else (None, None)
                d_r = c_r.decompress(p, o_r[0], o_r[1], o_r[2], o_r[3], qp_r)
                d_o = c_o.decompress(p, o_o[0], o_o[1], o_o[2], o_o[3], qp_o)
                worst = max(worst, diff(d_r, d_o), diff(tr_r.decode(d_r, use_dct=use_dct), tr_o.decode(d_o, use_dct=use_dct)))
                # three "peers": the same indices with scaled values, so contributor counts above one occur
                idxs, scales = [o_r[0]] * 3, (1.0, 3.0, 0.2)
                if quant:
                    vals_r = c_r.maybe_dequantize_values([o_r[1]] * 3, [qp_r] * 3, "cpu")
                    vals_o = c_o.maybe_dequantize_values([o_o[1]] * 3, [qp_o] * 3, "cpu")
                else:
                    vals_r, vals_o = [o_r[1]] * 3, [o_o[1]] * 3
                vals_r = [v * s for v, s in zip(vals_r, scales)]
                vals_o = [v * s for v, s in zip(vals_o, scales)]
                for clip in (False, True):
                    b_r = c_r.batch_decompress(p, idxs, vals_r, o_r[2], o_r[3], clip_norm=clip)
                    b_o = c_o.batch_decompress(p, idxs, vals_o, o_o[2], o_o[3], clip_norm=clip)
                    worst = max(worst, diff(b_r, b_o))
    out["compress_max_diff"], out["index_bytes_equal"] = worst, bytes_equal
    # 3. prepare_gradient_dict + outer_step on two copies of one model
    def miner(mod, lib, use_dct):
        m = SimpleNamespace(model=mod, hparams=SimpleNamespace(use_dct=use_dct, topk_compression=8, momentum_decay=0.9),
                            transformer=lib.compress.ChunkingTransformer(mod, 64),
                            compressor=lib.compress.TopKCompressor(use_quantization=True, quantization_bins=256,
                                                                   quantization_range=6))
        m.owned_params = {n for n, _ in mod.named_parameters()}
        m.error_feedback = {n: torch.zeros_like(p) for n, p in mod.named_parameters()}
        m.error_feedback_cpu_buffers = {n: torch.zeros_like(p) for n, p in mod.named_parameters()}
        return m

    worst_g = worst_ef = worst_w = 0.0
    for use_dct in (False, True):
        base = Net()
        mods = [copy.deepcopy(base), copy.deepcopy(base)]
        grads = {n: torch.randn_like(p) * 1e-2 for n, p in base.named_parameters()}
        results = []
        for mod, lib in zip(mods, (ref, ours)):
            m = miner(mod, lib, use_dct)
            for rnd in range(2):                              # second round: a non-zero error feedback goes in
                for n, p in mod.named_parameters():
                    p.grad = grads[n].clone() * (rnd + 1)
                g, xs, tk = lib.prepare_gradient_dict(m, step_window=5 + rnd, null_round=False)
            results.append((g, xs, tk, m))
        (g_r, xs_r, tk_r, m_r), (g_o, xs_o, tk_o, m_o) = results
        for k in g_r:
            if k.endswith("idxs"):
                assert torch.equal(g_r[k].cpu(), g_o[k].cpu()), k
            elif k.endswith("vals"):
                worst_g = max(worst_g, diff(g_r[k].cpu(), g_o[k].cpu()))
        for n in m_r.error_feedback:
            worst_ef = max(worst_ef, diff(m_r.error_feedback[n].cpu(), m_o.error_feedback[n].cpu()))
        # outer step: two peers (the payload and a scaled copy)
        for mod, lib, g, xs, tk, m in ((mods[0], ref, g_r, xs_r, tk_r, m_r), (mods[1], ours, g_o, xs_o, tk_o, m_o)):
            sd = {}
            for k, v in g.items():
                if k == "metadata":
                    continue
                sd[k] = [v, copy.deepcopy(v)]
            gather = SimpleNamespace(state_dict=SimpleNamespace(**sd), uids=[1, 2], skipped_uids=[], success_rate=1.0)
            opt = torch.optim.SGD(mod.parameters(), lr=0.4)
            lib.neurons.outer_step(mod, opt, gather_result=gather, transformer=m.transformer, compressor=m.compressor,
                                   xshapes=xs, totalks=tk, device="cpu", is_master=True, world_size=1, use_dct=use_dct)
        for (n, p), (_, q) in zip(mods[0].named_parameters(), mods[1].named_parameters()):
            worst_w = max(worst_w, diff(p.detach(), q.detach()))
        out[f"moved_dct{int(use_dct)}"] = max(diff(p.detach(), b.detach()) for (_, p), (_, b) in
                                              zip(mods[0].named_parameters(), base.named_parameters()))
    out["gradient_vals_max_diff"], out["error_feedback_max_diff"], out["outer_step_max_diff"] = worst_g, worst_ef, worst_w
    print("RESULT " + json.dumps(out))


if __name__ == "__main__":
    main()
