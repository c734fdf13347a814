"""Model and precision configuration classes against the reference's own (run from the unmodified tree in a child process):
same derived fields (block size, packing chunk rounded up to 64, key / value widths), same accepted and refused inputs, same
autocast properties. Needs the copy of the reference tree under ``baseline/_ref`` (skipped without it)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "src")), reason="no copy of the reference tree")
def test_config_classes_behave_like_the_reference(tmp_path):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from reference_config_worker import model_cases, precision_cases
    from hippolm_b200.config import HippoConfig, PrecisionConfig
    out = str(tmp_path / "ref.json")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "reference_config_worker.py"), REF, out],
                       capture_output=True, text=True, timeout=600, cwd=str(tmp_path))
    assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-3000:]
    ref = json.load(open(out))
    for kw, want in zip(model_cases(), ref["model"]):
        try:
            c = HippoConfig(**kw)
            got = {"ok": True, "block_size": c.block_size, "pack_chunk_size": c.pack_chunk_size}
        except Exception:                                           # noqa: BLE001
            got = {"ok": False}
        if kw.get("ffn_nvfp4_no_bf16_master") and not kw.get("ffn_nvfp4"):
            assert not got["ok"]                                    # refused here; whatever the reference does with it
            continue
        assert got["ok"] == want["ok"], (kw, got, want)
        if got["ok"]:
            assert got["block_size"] == want["block_size"] and got["pack_chunk_size"] == want["pack_chunk_size"], (kw, got, want)
            if want.get("key_dim") is not None:
                assert (c.key_dim, c.value_dim) == (want["key_dim"], want["value_dim"]), kw
    for d, want in zip(precision_cases(), ref["precision"]):
        try:
            p = PrecisionConfig.from_dict(d)
            got = {"ok": True, "autocast": bool(p.autocast_enabled), "autocast_dtype": str(p.autocast_dtype), "dict": p.to_dict()}
        except Exception:                                           # noqa: BLE001
            got = {"ok": False}
        if d and "nonsense" in d:
            assert want["ok"] and not got["ok"]                     # an unknown tensor class is ignored there, an error here
            continue
        assert got["ok"] == want["ok"], (d, got, want)
        if got["ok"]:
            assert got["autocast"] == want["autocast"], d
            if got["autocast"]:
                assert got["autocast_dtype"] == want["autocast_dtype"], d
            assert got["dict"] == want["dict"], (d, got["dict"], want["dict"])
