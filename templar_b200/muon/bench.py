"""Newton-Schulz orthogonalisation timings: this package's tcgen05 path (full products and one-triangle products)
against cuBLAS and against the reference's Triton kernels.

    python -m templar_b200.muon.bench [--shapes 2048x2048 2048x8192 8192x2048] [--reference]

Timed with CUDA events after warm-up, median of ``--iters``; the L2 is flushed between iterations.  ``--reference``
also times ``tplr.muon.newton_schulz_triton`` of the unmodified reference install (Triton ``ns_line_1`` /
``ns_line_2`` kernels + cuBLAS for line 3, under its own ``torch.compile`` wrapper;
src/tplr/muon/newton_schulz_triton.py:305-374).  The library arm (``zeropower_via_newtonschulz5`` on cuBLAS) is the
reference's non-Triton fallback.
"""

from __future__ import annotations

import argparse
import json

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", nargs="+", default=["2048x2048", "2048x8192", "8192x2048", "8192x8192"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--reference", action="store_true")
    a = ap.parse_args()

    import importlib

    from ..ops.microbench import time_ms

    ns = importlib.import_module("templar_b200.muon.newton_schulz")     # the module (the package re-exports the function)

    ref_fn = None
    if a.reference:
        import sys
        from pathlib import Path

        sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
        from baseline import ref_env

        ref_env.prepare()
        from tplr.muon.newton_schulz_triton import newton_schulz_triton as ref_fn   # the reference's own kernels

    for shape in a.shapes:
        r, c = (int(v) for v in shape.split("x"))
        g = torch.randn(r, c, device="cuda", generator=torch.Generator(device="cuda").manual_seed(0))
        rec = {"case": "newton_schulz", "shape": [r, c]}
        ns.SYMMETRIC_PRODUCTS = True
        sym = ns.newton_schulz(g)
        rec["own_one_triangle_ms"] = time_ms(lambda: ns.newton_schulz(g), a.iters)[0]
        ns.SYMMETRIC_PRODUCTS = False
        full = ns.newton_schulz(g)
        rec["own_full_products_ms"] = time_ms(lambda: ns.newton_schulz(g), a.iters)[0]
        ns.SYMMETRIC_PRODUCTS = True
        lib = ns.zeropower_via_newtonschulz5(g)
        rec["cublas_ms"] = time_ms(lambda: ns.zeropower_via_newtonschulz5(g), a.iters)[0]
        rec["one_triangle_vs_full_max_diff"] = float((sym.float() - full.float()).abs().max())
        # quality of the orthogonalisation: singular values of the result should sit near 1
        sv = torch.linalg.svdvals(sym.float())
        rec["singular_values_min_max"] = [float(sv.min()), float(sv.max())]
        if ref_fn is not None:
            out = ref_fn(g)
            rec["reference_triton_ms"] = time_ms(lambda: ref_fn(g), a.iters)[0]
            rec["vs_reference_max_diff"] = float((sym.float() - out.float()).abs().max())
            rec["speedup_vs_reference"] = rec["reference_triton_ms"] / rec["own_one_triangle_ms"]
        print(json.dumps(rec))


if __name__ == "__main__":
    main()
