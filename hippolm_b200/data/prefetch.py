"""Owner-rank prefetch thread fanning packed batches into per-rank queues
(``src/training/data/prefetch_batcher.py:21-228``).

``QueueIterator`` is the single read path of every rank: it pulls from its queue until a ``None``
sentinel and re-raises any exception object the producer put there, so a failure in the data thread
surfaces on every rank instead of hanging them.
"""
from __future__ import annotations

import threading
from typing import Callable, Iterable, Iterator, List, Optional, Sequence

import torch

from .packing import pack_chunk_aligned


class QueueIterator:
    _SENTINEL = None

    def __init__(self, q, timeout_s: Optional[float] = None):
        self._q, self._timeout = q, timeout_s
        self._done = False
        self.epochs_skipped = 0            # set by a resume that fast-forwarded through whole passes over a finite source

    def __iter__(self):
        return self

    def __next__(self):
        if self._done:                     # the sentinel arrives once: every later call ends at once instead of blocking
            raise StopIteration
        item = self._q.get(timeout=self._timeout) if self._timeout else self._q.get()
        if item is self._SENTINEL:
            self._done = True
            raise StopIteration
        if isinstance(item, BaseException):
            raise item
        return item


def _pin(t: torch.Tensor) -> torch.Tensor:
    if torch.cuda.is_available():
        try:
            return t.pin_memory()
        except Exception:
            return t
    return t


class PrefetchBatcher:
    """Pulls tokenised documents from ``doc_iter``, packs ``batch_size`` rows with the FFD chunk-aligned
    packer from a window of documents (up to ``batch_size * pack_buffer_size`` of them, or twice the batch's token
    capacity) and puts the same batch dict on every queue. Documents of the window that found no room are carried over
    into the next window, so every document (that fits a row at all) is eventually emitted; the reference discards them
    (``src/training/data/prefetch_batcher.py:103-108``). Exceptions and end-of-data are forwarded to all queues."""

    def __init__(self, doc_iter: Iterable[Sequence[int]], queues: List, batch_size: int, seq_len: int,
                 chunk_size: int, pack_buffer_size: int = 2048, pad_id: int = 0, eos_id: Optional[int] = None,
                 collate: Optional[Callable] = None):
        self.doc_iter, self.queues = iter(doc_iter), queues
        self.batch_size, self.seq_len, self.chunk_size = batch_size, seq_len, chunk_size
        self.buffer_docs = max(1, batch_size * pack_buffer_size)
        self.pad_id, self.eos_id = pad_id, eos_id
        self.collate = collate or pack_chunk_aligned
        self._carry: List[Sequence[int]] = []          # documents read but not placed yet
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, name="prefetch-batcher", daemon=True)
        self._thread.start()

    def _next_batch(self):
        budget = self.batch_size * self.seq_len
        while True:
            docs = list(self._carry)
            tokens = sum(len(d) for d in docs)
            fresh = 0
            if tokens < 2 * budget and len(docs) < self.buffer_docs:
                for d in self.doc_iter:
                    docs.append(d)
                    tokens += len(d)
                    fresh += 1
                    if len(docs) >= self.buffer_docs or tokens >= 2 * budget:
                        break
            if not docs:
                return None
            if self.collate is not pack_chunk_aligned:
                ids, labels, cu = self.collate(docs, self.seq_len, self.chunk_size, self.batch_size, self.pad_id, self.eos_id)
                self._carry = []
                break
            ids, labels, cu, placed = pack_chunk_aligned(docs, self.seq_len, self.chunk_size, self.batch_size, self.pad_id,
                                                         self.eos_id, return_placed=True)
            taken = set(placed)
            # a document longer than a row can never be placed: it is dropped here instead of circulating for ever
            self._carry = [d for i, d in enumerate(docs)
                           if i not in taken and 0 < len(d) + (1 if self.eos_id is not None and d[-1] != self.eos_id else 0) <= self.seq_len]
            if placed:
                break
            if fresh == 0 and not self._carry:
                return None                      # the source is exhausted and nothing that is left fits a row
            # a window of over-long documents only: read on
        return {"input_ids": _pin(ids.reshape(-1)), "labels": _pin(labels.reshape(-1)),
                "cu_seqlens": cu.to(torch.int32), "row_len": self.seq_len}

    def _put_all(self, item):
        for q in self.queues:
            while not self._stop.is_set():
                try:
                    q.put(item, timeout=0.1)
                    break
                except Exception:          # queue.Full
                    continue

    def _run(self):
        try:
            while not self._stop.is_set():
                batch = self._next_batch()
                if batch is None:
                    break
                self._put_all(batch)
            self._put_all(None)
        except BaseException as ex:
            self._put_all(ex)

    def close(self):
        self._stop.set()
        self._thread.join(timeout=2.0)
