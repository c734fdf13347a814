"""Differential tests against the reference's own host-side functions (called from the unmodified tree in a child
process): the WSD schedule, ``cu_seqlens`` slicing and the chunk-aligned first-fit-decreasing packer give the same results
here on seeded random inputs. Needs the copy of the reference tree under ``baseline/_ref`` (skipped without it)."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "src")), reason="no copy of the reference tree")
def test_schedule_slicing_and_packer_equal_the_reference(tmp_path):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from reference_functions_worker import cases, ns_inputs
    from hippolm_b200.optim.schedule import wsd_lr
    from hippolm_b200.data.packing import pack_chunk_aligned, slice_cu_seqlens
    out = str(tmp_path / "ref.pt")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "reference_functions_worker.py"), REF, out],
                       capture_output=True, text=True, timeout=600, cwd=str(tmp_path))
    assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-3000:]
    ref = torch.load(out, weights_only=False)
    wsd, slices, packs = cases()
    for c, want in zip(wsd, ref["wsd"]):
        assert wsd_lr(*c) == pytest.approx(want, rel=1e-12, abs=1e-15), c
    for (cu, a, b), want in zip(slices, ref["slices"]):
        if b < a:
            a, b = b, a
        assert slice_cu_seqlens(torch.tensor(cu), a, b).tolist() == want, (cu, a, b)
    n_docs = 0
    for (docs, seq_len, chunk, batch, pad, eos), (ids_r, labels_r, cu_r) in zip(packs, ref["packs"]):
        ids, labels, cu = pack_chunk_aligned(docs, seq_len, chunk, batch, pad_id=pad, eos_id=eos)
        assert torch.equal(ids, ids_r), (seq_len, chunk, batch, eos)
        # One deliberate difference. The reference means to mask the label of the first token after a document boundary, but
        # writes that -100 one position past the previous document and then overwrites it with the next document's own
        # labels (``src/training/data/collate.py:186-193``), so there every document start keeps its label and the last
        # position of the previous document's chunk is trained to predict it. Here the first token of every document is
        # masked, which is what its docstring describes.
        diff = (labels != labels_r).nonzero().tolist()
        starts = set(cu.tolist())
        for b, t in diff:
            assert labels[b, t] == -100 and labels_r[b, t] == ids_r[b, t] and b * seq_len + t in starts, (b, t)
        assert cu.tolist() == cu_r.tolist(), (cu.tolist(), cu_r.tolist())
        n_docs += len(docs)
    assert n_docs > 300
    # Newton-Schulz: same polynomial, same normalisation; the reference iterates in fp16, the oracle here in fp32
    from hippolm_b200.ref.ops import newton_schulz5
    for x, want in zip(ns_inputs(), ref["ns"]):
        got = newton_schulz5(x, 5)
        assert got.shape == want.shape
        assert (got - want).abs().max() < 2e-2 and torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0) > 0.9995
