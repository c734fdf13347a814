"""Packing of variable-length documents into fixed token budgets with ``cu_seqlens``.

* :func:`pack_chunk_aligned` -- first-fit-decreasing packer whose document boundaries fall on
  ``chunk_size`` multiples (same contract as the reference's ``src/training/data/collate.py:42-268``).
* :func:`synthetic_packed_batch` -- seeded uniform-random tokens cut into documents of uniform
  random length, packed back to back (the benchmark data of every throughput config).
* :func:`slice_cu_seqlens` -- boundaries of a token window (``src/training/loop/support.py:92-148``).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


def pack_chunk_aligned(samples: Sequence[Sequence[int]], seq_len: int, chunk_size: int, batch_size: int,
                       pad_id: int = 0, eos_id: Optional[int] = None, return_placed: bool = False):
    """Returns ``(input_ids[B,S], labels[B,S], cu_seqlens)``; with ``return_placed`` also the indices (into ``samples``)
    of the documents that were placed, so that a caller can carry the others over to its next batch.

    Documents are sorted by chunk count (descending) and placed first-fit into exactly
    ``batch_size`` rows; each document starts on a ``chunk_size`` multiple and is padded up to the
    next one. ``labels`` are -100 on padding and on the first token of every document (its
    "previous token" belongs to another document). ``cu_seqlens`` runs over the flattened
    ``[B*S]`` stream: every document's chunk-rounded end, the start of each row's tail padding and
    every row end, deduplicated, starting at 0 and ending at ``B*S``. Documents longer than
    ``seq_len`` and documents that fit in no row are dropped.
    """
    if batch_size < 1:
        raise ValueError("batch_size must be >= 1")
    chunk_size = _round_up(max(chunk_size, 1), 64)
    if seq_len % chunk_size != 0:
        raise ValueError(f"seq_len ({seq_len}) must be a multiple of chunk_size ({chunk_size})")
    docs: List[List[int]] = []
    src: List[int] = []                                   # index of every kept document in ``samples``
    for si, s in enumerate(samples):
        d = list(s)
        if eos_id is not None and (len(d) == 0 or d[-1] != eos_id):
            d.append(eos_id)
        if 0 < len(d) <= seq_len:
            docs.append(d)
            src.append(si)
    order = sorted(range(len(docs)), key=lambda i: -_round_up(len(docs[i]), chunk_size))
    used = [0] * batch_size
    rows: List[List[Tuple[int, List[int]]]] = [[] for _ in range(batch_size)]
    placed: List[int] = []
    for i in order:
        need = _round_up(len(docs[i]), chunk_size)
        for b in range(batch_size):
            if used[b] + need <= seq_len:
                rows[b].append((used[b], docs[i]))
                used[b] += need
                placed.append(src[i])
                break
    ids = torch.full((batch_size, seq_len), pad_id, dtype=torch.long)
    labels = torch.full((batch_size, seq_len), -100, dtype=torch.long)
    bounds = {0}
    for b in range(batch_size):
        base = b * seq_len
        for off, d in rows[b]:
            n = len(d)
            t = torch.tensor(d, dtype=torch.long)
            ids[b, off:off + n] = t
            labels[b, off + 1:off + n] = t[1:]
            bounds.add(base + off + _round_up(n, chunk_size))
        if 0 < used[b] < seq_len:
            bounds.add(base + used[b])
        bounds.add(base + seq_len)
    cu = torch.tensor(sorted(bounds), dtype=torch.long)
    if return_placed:
        return ids, labels, cu, sorted(placed)
    return ids, labels, cu


def synthetic_packed_batch(n_tokens: int, vocab_size: int, seed: int, doc_len_min: int, doc_len_max: int,
                           row_len: Optional[int] = None, align: int = 1
                           ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Flat ``input_ids[T]``, ``labels[T]``, ``cu_seqlens`` (int32) of seeded uniform-random tokens.

    Document lengths are uniform in ``[doc_len_min, doc_len_max]`` (rounded to ``align``); documents
    are packed back to back and cut at every ``row_len`` multiple (a row is one training sequence).
    """
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, vocab_size, (n_tokens,), generator=g, dtype=torch.long)
    row_len = row_len or n_tokens
    bounds = [0]
    for r0 in range(0, n_tokens, row_len):
        r1 = min(r0 + row_len, n_tokens)
        p = r0
        while p < r1:
            l = int(torch.randint(doc_len_min, doc_len_max + 1, (1,), generator=g))
            l = max(align, _round_up(l, align))
            p = min(p + l, r1)
            bounds.append(p)
    cu = torch.tensor(bounds, dtype=torch.int32)
    labels = ids.clone()
    labels[cu[:-1].long()] = -100
    return ids, labels, cu


def slice_cu_seqlens(cu_seqlens: torch.Tensor, start: int, end: int) -> torch.Tensor:
    """Boundaries that fall inside ``[start, end]``, shifted to the window, with a forced leading 0
    and trailing ``end - start``; an empty window gives ``[0]``."""
    if end <= start:
        return torch.zeros(1, dtype=cu_seqlens.dtype, device=cu_seqlens.device)
    inside = cu_seqlens[(cu_seqlens > start) & (cu_seqlens < end)] - start
    z = torch.zeros(1, dtype=cu_seqlens.dtype, device=cu_seqlens.device)
    e = torch.full((1,), end - start, dtype=cu_seqlens.dtype, device=cu_seqlens.device)
    return torch.cat([z, inside, e])
