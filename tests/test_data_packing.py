"""FFD chunk-aligned packer, synthetic packed batches, cu_seqlens slicing, loss weighting."""
import pytest
import torch

from hippolm_b200.data.packing import pack_chunk_aligned, synthetic_packed_batch, slice_cu_seqlens


def test_cu_seqlens_ends_and_alignment():
    docs = [list(range(1, 101)), list(range(1, 31)), list(range(1, 201))]
    ids, labels, cu = pack_chunk_aligned(docs, seq_len=512, chunk_size=64, batch_size=2)
    assert ids.shape == (2, 512) and labels.shape == (2, 512)
    assert cu[0] == 0 and cu[-1] == 2 * 512
    assert torch.all(cu[1:] > cu[:-1])
    assert all(int(c) % 64 == 0 for c in cu)


def test_empty_samples_all_pad():
    ids, labels, cu = pack_chunk_aligned([], seq_len=128, chunk_size=64, batch_size=3, pad_id=9)
    assert (ids == 9).all() and (labels == -100).all()
    assert cu.tolist() == [0, 128, 256, 384]


def test_eos_forced_not_duplicated_and_cross_doc_mask():
    ids, labels, cu = pack_chunk_aligned([[5, 6, 7], [8, 9, 2]], seq_len=128, chunk_size=64, batch_size=1, eos_id=2)
    row = ids[0].tolist()
    assert row[:4] == [5, 6, 7, 2] and row[64:67] == [8, 9, 2] and row[67] == 0
    assert labels[0, 0] == -100 and labels[0, 64] == -100       # first token of each document is never a target
    assert labels[0, 1:4].tolist() == [6, 7, 2] and labels[0, 4] == -100
    assert cu.tolist() == [0, 64, 128]


def test_doc_filling_pack_and_tail_pad_boundary():
    ids, labels, cu = pack_chunk_aligned([list(range(1, 129))], seq_len=128, chunk_size=64, batch_size=1)
    assert cu.tolist() == [0, 128]
    ids, labels, cu = pack_chunk_aligned([list(range(1, 60))], seq_len=256, chunk_size=64, batch_size=1)
    assert cu.tolist() == [0, 64, 256]


def test_packer_errors_and_drop():
    with pytest.raises(ValueError):
        pack_chunk_aligned([[1]], seq_len=100, chunk_size=64, batch_size=1)
    with pytest.raises(ValueError):
        pack_chunk_aligned([[1]], seq_len=128, chunk_size=64, batch_size=0)
    ids, _, _ = pack_chunk_aligned([list(range(300))], seq_len=128, chunk_size=64, batch_size=1)
    assert (ids == 0).all()


def test_synthetic_batch_is_seeded_and_bounded():
    a = synthetic_packed_batch(2048, 1000, 3, 64, 256, row_len=512)
    b = synthetic_packed_batch(2048, 1000, 3, 64, 256, row_len=512)
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    ids, labels, cu = a
    assert cu[0] == 0 and cu[-1] == 2048 and set(range(0, 2049, 512)) <= set(cu.tolist())
    lens = (cu[1:] - cu[:-1])
    assert lens.max() <= 256 and lens.min() >= 1
    assert (labels[cu[:-1].long()] == -100).all()


def test_slice_cu_seqlens():
    cu = torch.tensor([0, 10, 25, 40])
    assert slice_cu_seqlens(cu, 0, 40).tolist() == [0, 10, 25, 40]
    assert slice_cu_seqlens(cu, 5, 30).tolist() == [0, 5, 20, 25]
    assert slice_cu_seqlens(cu, 10, 25).tolist() == [0, 15]
    assert slice_cu_seqlens(cu, 12, 20).tolist() == [0, 8]
    assert slice_cu_seqlens(cu, 7, 7).tolist() == [0]


def test_micro_batch_loss_weighting_equals_full_mean():
    torch.manual_seed(0)
    logits = torch.randn(64, 50)
    labels = torch.randint(0, 50, (64,)); labels[::5] = -100
    full = torch.nn.functional.cross_entropy(logits, labels, ignore_index=-100)
    total = (labels != -100).sum()
    acc = 0.0
    for s in range(0, 64, 16):
        l = labels[s:s + 16]
        n = (l != -100).sum()
        acc = acc + torch.nn.functional.cross_entropy(logits[s:s + 16], l, ignore_index=-100) * n / total
    assert torch.allclose(acc, full, atol=1e-6)


def test_lce_head_matches_cross_entropy_and_epilogue_flag_is_inert_on_cpu():
    """The chunked linear + cross-entropy head against F.cross_entropy; `lce_epilogue_stats` selects a CUDA-only
    kernel path, so on CPU tensors it must not change the result."""
    from hippolm_b200.models.model import _VocabParallelLCE
    torch.manual_seed(0)
    T, D, V = 50, 16, 40
    x = torch.randn(T, D)
    w = 0.3 * torch.randn(V, D)
    tg = torch.randint(0, V, (T,))
    tg[::6] = -100
    nv = int((tg >= 0).sum())
    outs = []
    for epi in (False, True):
        xi, wi = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        loss = _VocabParallelLCE.apply(xi, wi, tg, 0, 3, nv, epi)
        loss.backward()
        outs.append((loss.detach(), xi.grad, wi.grad))
    xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(xr @ wr.t(), tg, ignore_index=-100)
    ref.backward()
    for loss, dx, dw in outs:
        assert torch.allclose(loss, ref, atol=1e-5)
        assert torch.allclose(dx, xr.grad, atol=1e-5) and torch.allclose(dw, wr.grad, atol=1e-5)
