"""Numerical parity with the unmodified reference model: its single-GPU model class (``src/models/model.py``) with its own
vendored Triton kernels, run on the CPU by Triton's interpreter, against this framework's model loaded with the converted
weights: same tokens, same logits. Covers the whole stack: embedding, every KDA layer (projections, short convolution,
gates, delta-rule recurrence, gated per-head norm), SwiGLU, the block attention residual with non-zero queries, the final
norm and the tied head. Needs the copy of the reference tree under ``baseline/_ref`` (skipped without it)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "src")), reason="no copy of the reference tree")
@pytest.mark.parametrize("kw", [
    {},                                                                     # plain gate, no convolution
    {"use_short_conv": True, "safe_gate": True, "lower_bound": -5.0},       # the reference's production switches
    {"allow_neg_eigval": True, "use_short_conv": True, "kda_mode": "fused_recurrent", "num_layers": 6, "num_blocks": 3},
])
def test_logits_match_the_unmodified_reference_model(kw, tmp_path):
    worker = os.path.join(ROOT, "tests", "reference_parity_worker.py")
    r = subprocess.run([sys.executable, worker, REF, ROOT, json.dumps(kw), "0"], capture_output=True, text=True,
                       timeout=900, cwd=str(tmp_path), env=dict(os.environ, PARITY_TOKENS="40"))
    lines = [l for l in r.stdout.splitlines() if l.startswith("PARITY ")]
    if r.returncode != 0 and "InterpreterError" in r.stderr:
        pytest.skip("Triton's interpreter cannot run one of the reference's kernels here: " + r.stderr.strip().splitlines()[-1])
    assert r.returncode == 0 and lines, r.stdout[-1000:] + r.stderr[-3000:]
    out = json.loads(lines[-1][len("PARITY "):])
    assert out["max_abs_ref"] > 1.0                                         # the comparison is not between two zero tensors
    assert out["max_abs_diff"] < 1e-4 * max(1.0, out["max_abs_ref"]), out
