"""The reference's own code as the oracle: ``tplr.compress`` (pack / unpack, chunking + DCT, top-k, quantisation,
decompress, batch_decompress), ``tplr.prepare_gradient_dict`` and ``tplr.neurons.outer_step`` of the unmodified
reference install, run on CPU next to this framework's implementations of the same API.

The reference is imported in a child process (it is installed under ``baseline/_ref`` with ``--no-deps``; absent
third-party packages get stand-in modules, none of which is on the compared path).  Skipped when the install is
not there."""

import json
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(os.path.dirname(HERE), "baseline", "_ref", "tplr")


@pytest.mark.skipif(not os.path.isdir(REF), reason="the reference is not installed under baseline/_ref")
def test_compress_gradient_dict_and_outer_step_match_the_reference():
    r = subprocess.run([sys.executable, os.path.join(HERE, "_ref_oracle_worker.py")], capture_output=True, text=True,
                       timeout=600, env=dict(os.environ, TPLR_LOG_LEVEL="WARNING"))
    lines = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")]
    assert r.returncode == 0 and lines, r.stdout[-2000:] + r.stderr[-4000:]
    res = json.loads(lines[-1][7:])
    assert res["pack_equal"] and res["unpack_equal"] and res["index_bytes_equal"], res
    assert res["compress_max_diff"] < 1e-6, res                  # the reference's own tolerance for its DCT round trip
    assert res["gradient_vals_max_diff"] < 1e-6 and res["error_feedback_max_diff"] < 1e-6, res
    assert res["outer_step_max_diff"] < 1e-6, res
    assert res["moved_dct0"] > 1e-3 and res["moved_dct1"] > 1e-3, res    # the outer step did move the weights
