"""Batch sources for the training loop.

``dummy_dataloader`` is the reference's random-token loader (``src/training/data/dummy.py:8-29``);
``synthetic_loader`` yields the benchmark batches (seeded tokens, uniform random document lengths,
``cu_seqlens`` packing). Every batch is a dict of *pinned host* tensors
``{input_ids[T], labels[T], cu_seqlens[int32], row_len}`` for one DP rank.
"""
from __future__ import annotations

from typing import Dict, Iterator, Optional, Tuple

import torch

from .packing import synthetic_packed_batch, pack_chunk_aligned


def _pin(t: torch.Tensor) -> torch.Tensor:
    if torch.cuda.is_available():
        try:
            return t.pin_memory()
        except Exception:
            return t
    return t


def dummy_dataloader(batch_size: int, seq_len: int, vocab_size: int, seed: int = 0, start_step: int = 0
                     ) -> Iterator[Dict]:
    """Batch ``i`` depends on ``(seed, i)`` only, so a resumed run continues the stream at ``start_step``."""
    step = start_step
    while True:
        g = torch.Generator().manual_seed(seed * 1000003 + step)
        step += 1
        ids = torch.randint(0, vocab_size, (batch_size * seq_len,), generator=g)
        labels = ids.clone()
        cu = torch.arange(0, batch_size * seq_len + 1, seq_len, dtype=torch.int32)
        labels[cu[:-1].long()] = -100
        yield {"input_ids": _pin(ids), "labels": _pin(labels), "cu_seqlens": cu, "row_len": seq_len}


def synthetic_loader(batch_size: int, seq_len: int, vocab_size: int, seed: int, doc_len_min: int,
                     doc_len_max: int, align: int = 1, fixed: bool = False, start_step: int = 0) -> Iterator[Dict]:
    step = start_step
    cached = None
    while True:
        if fixed and cached is not None:
            yield cached
            continue
        ids, labels, cu = synthetic_packed_batch(batch_size * seq_len, vocab_size, seed * 100003 + step,
                                                 doc_len_min, doc_len_max, row_len=seq_len, align=align)
        cached = {"input_ids": _pin(ids), "labels": _pin(labels), "cu_seqlens": cu, "row_len": seq_len}
        yield cached
        step += 1


def build_data_iterator(args, cfg, mesh, start_step: int = 0) -> Tuple[Iterator, Optional[object]]:
    """Per-DP-rank batch iterator. TP ranks of one DP replica draw the same stream (same seed);
    real-data runs broadcast from the owner rank through :class:`PrefetchBatcher`. ``start_step`` batches have
    already been consumed by the run being resumed: synthetic streams jump there, real-data streams are fast-forwarded."""
    gb = int(getattr(args, "batch_size", 1))
    assert gb % mesh.dp == 0, f"batch_size {gb} must be divisible by dp {mesh.dp}"
    lb = gb // mesh.dp
    seq = int(getattr(args, "seq_len", 512))
    seed = int(getattr(args, "seed", 0)) * 131 + mesh.dp_rank
    if getattr(args, "use_dummy_data", False) and not getattr(args, "doc_len_max", 0):
        return dummy_dataloader(lb, seq, cfg.vocab_size, seed, start_step), None
    if getattr(args, "use_dummy_data", False) or getattr(args, "synthetic_data", False):
        return synthetic_loader(lb, seq, cfg.vocab_size, seed, int(getattr(args, "doc_len_min", 64)),
                                int(getattr(args, "doc_len_max", 256)),
                                int(getattr(args, "doc_align", 1)),
                                bool(getattr(args, "fixed_batch", False)), start_step), None
    from .streaming import build_streaming_iterator
    it, pre = build_streaming_iterator(args, cfg, mesh, lb, seq)
    # Fast-forward a resumed run. A finite source may end while skipping: the run it resumes had re-opened it for its next
    # epoch at that point, so do the same here and go on skipping; the number of whole passes is handed to the caller.
    left, in_pass, passes = int(start_step), 0, 0
    while left > 0:
        try:
            next(it)
            left -= 1
            in_pass += 1
        except StopIteration:
            if in_pass == 0:
                break                                   # an empty source: nothing to skip through
            if pre is not None:
                pre.close()
            passes += 1
            in_pass = 0
            if passes >= int(getattr(args, "epochs", 1) or 1):
                break                                   # the resumed run had used up its epochs
            it, pre = build_streaming_iterator(args, cfg, mesh, lb, seq)
    try:
        it.epochs_skipped = passes
    except AttributeError:
        pass
    return it, pre
