"""The kernel library built with checked data-dependent indices (``HIPPO_DEBUG_BOUNDS=1``): an out-of-range token id or
target id is recorded in the device status word (code 8, detail = which check) and the access is skipped; nothing
faults, the results stay finite, and clean inputs leave the status word clean."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_CHILD = r'''
import ctypes as C, os, sys, torch
sys.path.insert(0, os.environ["HIPPO_ROOT"])
from hippolm_b200.ops import _ext, embed_cuda
from hippolm_b200 import ops
assert _ext.lib_path().endswith("libhippo_kernels_dbg.so")
dev = "cuda"
V, D = 64, 128
w = torch.randn(V, D, device=dev).bfloat16()
ids = torch.tensor([0, 5, 63, 7], device=dev)
out = embed_cuda.gather(ids, [w.data_ptr()], V, D)
torch.cuda.synchronize()
assert _ext.device_status()[0] == 0 and torch.equal(out[1], w[5])
bad = torch.tensor([0, 5, 64 + 1000, 7], device=dev)               # one id beyond the vocabulary
out = embed_cuda.gather(bad, [w.data_ptr()], V, D)
torch.cuda.synchronize()
st = _ext.device_status()
assert st[0] == 8 and st[1] == 1, st
assert float(out[2].abs().max()) == 0.0 and torch.equal(out[3], w[7])
_ext.clear_device_status()
x = torch.randn(6, 64, device=dev).bfloat16()
wv = torch.randn(56, 64, device=dev).bfloat16()
tgt = torch.tensor([1, 2, 3, -100, 55, 77], device=dev)            # -100: ignored row; 77 >= 56: bad target
z, mx, se, tz = ops.lce_chunk_stats(x, wv, tgt)
torch.cuda.synchronize()
st = _ext.device_status()
assert st[0] == 8 and st[1] == 3, st
assert torch.isfinite(tz).all() and float(tz[5]) == 0.0 and float(tz[3]) == 0.0
assert abs(float(tz[4]) - float(z[4, 55])) < 1e-6
print("BOUNDS_OK")
'''


def test_bad_indices_are_recorded_and_skipped(tmp_path):
    from hippolm_b200.ops import _ext
    dbg = os.path.join(os.path.dirname(_ext.lib_path()), "libhippo_kernels_dbg.so")
    if not os.path.exists(dbg):
        pytest.skip("debug-bounds library not built (HIPPO_DEBUG_BOUNDS=1 python -m hippolm_b200.csrc.build)")
    script = tmp_path / "child.py"
    script.write_text(_CHILD)
    r = subprocess.run([sys.executable, str(script)], env=dict(os.environ, HIPPO_ROOT=ROOT, HIPPO_DEBUG_BOUNDS="1"),
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "BOUNDS_OK" in r.stdout, r.stdout[-1500:] + r.stderr[-3000:]
