"""The KDA operator against the reference's own token-recurrent kernel (its oracle, run on the CPU by Triton's
interpreter): packed documents of ragged lengths (one-token documents, documents longer than a chunk), initial and final
states, L2 normalisation and gate activation (plain and lower-bounded) inside the kernel. All three CPU implementations
here (token recurrence, chunked form, chunked form with anchored decay) must reproduce its outputs and final states.
Needs the copy of the reference tree under ``baseline/_ref`` (skipped without it)."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "src")), reason="no copy of the reference tree")
def test_kda_matches_the_reference_recurrent_kernel(tmp_path):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from reference_kda_worker import inputs
    from hippolm_b200.ref import kda as rk
    out = str(tmp_path / "ref.pt")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "reference_kda_worker.py"), REF, out],
                       capture_output=True, text=True, timeout=900, cwd=str(tmp_path))
    if r.returncode != 0 and "InterpreterError" in r.stderr:
        pytest.skip("Triton's interpreter cannot run the reference kernel here: " + r.stderr.strip().splitlines()[-1])
    assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-3000:]
    ref = torch.load(out)
    for case, (o_ref, ht_ref) in enumerate(ref):
        d = inputs(case)
        H, K = d["q"].shape[2], d["q"].shape[3]
        q, k, v, beta = d["q"][0], d["k"][0], d["v"][0], d["beta"][0]
        lb = d["lower_bound"]
        g = rk.kda_gate(d["x_g"][0], d["A_log"], d["dt_bias"].view(H, K), lb is not None, lb if lb is not None else -5.0)
        for name, fn in (("recurrent", rk.kda_recurrent), ("chunked", rk.kda_chunked), ("anchored", rk.kda_chunked_anchored)):
            o, ht = fn(q, k, v, g, beta, None, d["h0"], d["cu"].int(), True)
            assert (o.float() - o_ref[0]).abs().max() < 2e-4 * max(1.0, o_ref.abs().max()), (case, name)
            assert (ht.float() - ht_ref).abs().max() < 2e-4 * max(1.0, ht_ref.abs().max()), (case, name)
