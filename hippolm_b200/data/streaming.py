"""Streaming text datasets, multi-source phase schedule, rotating parquet shard cache.

Behavioural parity with ``src/training/data/{streaming,rotating,sources,cache,parquet}.py``; every network
touchpoint is an injected callable (``list_parts_fn``, ``download_fn``, ``loaders``) so the pipeline runs
and is tested without a network:

* ``StreamingDataset``            examples -> text (pretrain field or SFT chat template) -> token lists,
                                  tokenised 64 documents per call
* ``MultiSourceStreamingDataset`` phase schedule over several sub-datasets (weights per phase)
* ``RotatingParquetIterable``     iterates the rows of a multi-part parquet dataset while a background
                                  thread downloads the next part at 50 % progress; at most two files on
                                  disk, the finished part is evicted
* ``load_streaming_with_fallback`` tries sources in order, falling through on *network* errors only
"""
from __future__ import annotations

import os
import threading
from pathlib import Path
from typing import Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple


def network_exceptions() -> tuple:
    excs = [ConnectionError, TimeoutError]
    try:
        import requests
        excs += [requests.exceptions.ConnectionError, requests.exceptions.Timeout]
    except Exception:
        pass
    return tuple(excs)


def load_streaming_with_fallback(loaders: Sequence[Tuple[str, Callable[[], Iterable]]], logger=None) -> Iterable:
    """``loaders``: (name, zero-arg callable). Network failures fall through to the next source; any other
    exception propagates (a bad config must not be masked by a fallback)."""
    last = None
    for name, fn in loaders:
        try:
            return fn()
        except network_exceptions() as ex:
            last = ex
            if logger:
                logger.warning(f"data source {name} unreachable ({ex!r}); trying the next one")
    raise ConnectionError(f"all data sources failed; last error: {last!r}")


# ----------------------------------------------------------------------------- cache helpers
def get_cache_dir() -> Path:
    d = os.environ.get("HIPPOLM_CACHE_DIR")
    return Path(d) if d else Path.cwd() / ".cache" / "hippolm" / "datasets"


def cache_path_for_part(name: str, config: Optional[str], part_index: int, root: Optional[Path] = None) -> Path:
    safe = name.replace("/", "__") + (f"__{config}" if config else "")
    return (root or get_cache_dir()) / f"{safe}__part{part_index:05d}.parquet"


def list_cached_parts(name: str, config: Optional[str], root: Optional[Path] = None) -> List[Path]:
    safe = name.replace("/", "__") + (f"__{config}" if config else "")
    base = root or get_cache_dir()
    return sorted(base.glob(f"{safe}__part*.parquet")) if base.exists() else []


def purge_stale_cache(name: str, config: Optional[str], keep: Sequence[Path], root: Optional[Path] = None) -> int:
    n = 0
    keep_set = {Path(k) for k in keep}
    for p in list_cached_parts(name, config, root):
        if p not in keep_set:
            try:
                p.unlink(); n += 1
            except OSError:
                pass
    return n


def iter_parquet_rows(path) -> Iterator[dict]:
    import pyarrow.parquet as pq
    pf = pq.ParquetFile(str(path))
    for batch in pf.iter_batches(batch_size=1024):
        for row in batch.to_pylist():
            yield row


def count_parquet_rows(path) -> int:
    import pyarrow.parquet as pq
    return pq.ParquetFile(str(path)).metadata.num_rows


class RotatingParquetIterable:
    """Rows of parts ``0..n-1`` in order. ``list_parts_fn() -> [part ids]``; ``download_fn(part, dest_path)``
    writes the parquet file. The next part is fetched by a background thread once ``prefetch_fraction`` of the
    current part has been read; the previous part's file is deleted when the reader moves on."""

    def __init__(self, name: str, config: Optional[str], list_parts_fn: Callable[[], Sequence],
                 download_fn: Callable[[object, Path], None], cache_root: Optional[Path] = None,
                 prefetch_fraction: float = 0.5, loop: bool = False):
        self.name, self.config = name, config
        self.list_parts_fn, self.download_fn = list_parts_fn, download_fn
        self.root = Path(cache_root) if cache_root else get_cache_dir()
        self.prefetch_fraction, self.loop = prefetch_fraction, loop
        self.parts: List = []
        self._idx = -1
        self._rows: Optional[Iterator[dict]] = None
        self._read = 0
        self._total = 0
        self._dl_thread: Optional[threading.Thread] = None
        self._dl_error: Optional[BaseException] = None
        self._cur_path: Optional[Path] = None
        self.max_files_seen = 0

    def _path(self, i: int) -> Path:
        return cache_path_for_part(self.name, self.config, i, self.root)

    def _download(self, i: int):
        p = self._path(i)
        if not p.exists():
            tmp = p.with_suffix(".tmp")
            self.download_fn(self.parts[i], tmp)
            os.replace(tmp, p)

    def open(self):
        self.root.mkdir(parents=True, exist_ok=True)
        self.parts = list(self.list_parts_fn())
        if not self.parts:
            raise FileNotFoundError(f"{self.name}: no parquet parts")
        purge_stale_cache(self.name, self.config, [self._path(0)], self.root)
        self._download(0)
        self._open_part(0)

    def _open_part(self, i: int):
        self._idx = i
        self._cur_path = self._path(i)
        self._total = count_parquet_rows(self._cur_path)
        self._rows = iter_parquet_rows(self._cur_path)
        self._read = 0
        self._track()

    def _track(self):
        self.max_files_seen = max(self.max_files_seen, len(list_cached_parts(self.name, self.config, self.root)))

    def _next_index(self) -> Optional[int]:
        n = self._idx + 1
        if n < len(self.parts):
            return n
        return 0 if (self.loop and len(self.parts) > 1) else None

    def _schedule_next(self):
        n = self._next_index()
        if n is None or self._dl_thread is not None:
            return

        def work():
            try:
                self._download(n)
            except BaseException as ex:
                self._dl_error = ex
        self._dl_thread = threading.Thread(target=work, name="parquet-prefetch", daemon=True)
        self._dl_thread.start()

    def _switch(self) -> bool:
        n = self._next_index()
        if n is None:
            return False
        if self._dl_thread is None:
            self._schedule_next()
        self._dl_thread.join()
        self._dl_thread = None
        if self._dl_error is not None:
            err, self._dl_error = self._dl_error, None
            raise err
        self._track()
        old = self._cur_path
        self._open_part(n)
        if old is not None and old != self._cur_path:
            try:
                old.unlink()
            except OSError:
                pass
        return True

    def __iter__(self):
        if self._rows is None:
            self.open()
        return self

    def __next__(self) -> dict:
        while True:
            try:
                row = next(self._rows)
                self._read += 1
                if self._total and self._read >= self.prefetch_fraction * self._total:
                    self._schedule_next()
                return row
            except StopIteration:
                if not self._switch():
                    raise

    def close(self):
        if self._dl_thread is not None:
            self._dl_thread.join(timeout=5.0)


# ----------------------------------------------------------------------------- datasets
class StreamingDataset:
    """Iterable of token lists. ``source`` yields dict examples; ``stage='pretrain'`` reads ``text_field``;
    ``stage='sft'`` renders ``messages`` / (``instruction``, ``output``) through the tokenizer's chat template."""

    TOKENIZE_BATCH = 64

    def __init__(self, source: Iterable[dict], tokenizer, text_field: str = "content", stage: str = "pretrain",
                 max_len: Optional[int] = None, add_eos: bool = True, split_long: bool = False):
        """``max_len``: a longer document is cut to it (the reference's choice: its tokenizer truncates,
        ``src/training/data/streaming.py:157``) or, with ``split_long``, yielded as consecutive pieces of ``max_len``
        tokens so that no text is thrown away (the end-of-text token closes the last piece only)."""
        self.source, self.tok, self.text_field, self.stage = source, tokenizer, text_field, stage
        self.max_len, self.add_eos, self.split_long = max_len, add_eos, split_long

    def _format_sft(self, ex: dict) -> Optional[str]:
        msgs = ex.get("messages") or ex.get("conversations")
        if not msgs and "instruction" in ex:
            msgs = [{"role": "user", "content": ex["instruction"]}, {"role": "assistant", "content": ex.get("output", "")}]
        if not msgs:
            return None
        return self.tok.apply_chat_template(msgs, tokenize=False, add_generation_prompt=False)

    def _text(self, ex: dict) -> Optional[str]:
        if self.stage == "sft":
            return self._format_sft(ex)
        t = ex.get(self.text_field)
        return t if isinstance(t, str) and t else None

    def _flush(self, texts: List[str]) -> Iterator[List[int]]:
        enc = self.tok(texts, add_special_tokens=False)["input_ids"]
        eos = getattr(self.tok, "eos_token_id", None)
        for ids in enc:
            ids = list(ids)
            if self.max_len and self.split_long and len(ids) >= self.max_len:
                if self.add_eos and eos is not None and ids[-1] != eos:
                    ids.append(eos)
                for s0 in range(0, len(ids), self.max_len):
                    piece = ids[s0:s0 + self.max_len]
                    if len(piece) > 1 or s0 == 0:
                        yield piece
                continue
            if self.max_len:
                ids = ids[:self.max_len - (1 if self.add_eos and eos is not None else 0)]
            if self.add_eos and eos is not None and (not ids or ids[-1] != eos):
                ids.append(eos)
            if ids:
                yield ids

    def __iter__(self) -> Iterator[List[int]]:
        batch: List[str] = []
        for ex in self.source:
            t = self._text(ex)
            if t is None:
                continue
            batch.append(t)
            if len(batch) >= self.TOKENIZE_BATCH:
                yield from self._flush(batch)
                batch = []
        if batch:
            yield from self._flush(batch)


class MultiSourceStreamingDataset:
    """``phase_schedule``: list of ``(n_docs, {source_name: weight})``; within a phase sources are drawn
    round-robin in proportion to their integer weights; exhausted sources are skipped."""

    def __init__(self, sub_datasets: Dict[str, Iterable], phase_schedule: Sequence[Tuple[int, Dict[str, int]]]):
        self.subs, self.schedule = sub_datasets, list(phase_schedule)

    def __iter__(self):
        its = {k: iter(v) for k, v in self.subs.items()}
        dead = set()
        for n_docs, weights in self.schedule:
            order = [k for k, w in weights.items() for _ in range(int(w))]
            emitted, i = 0, 0
            while emitted < n_docs and any(k not in dead for k in order):
                k = order[i % len(order)]; i += 1
                if k in dead:
                    continue
                try:
                    yield next(its[k]); emitted += 1
                except StopIteration:
                    dead.add(k)


def build_streaming_iterator(args, cfg, mesh, local_batch: int, seq_len: int):
    """Real-data path: the owner rank of each TP group tokenises + packs; here every rank of a DP replica runs
    the same deterministic pipeline (same source order), so no cross-process queue is needed on one node."""
    import queue
    from .prefetch import PrefetchBatcher, QueueIterator
    from .tokenizer import load_tokenizer
    tok = load_tokenizer(getattr(args, "tokenizer_path", None))
    data_files = getattr(args, "data_files", None)
    if data_files:
        files = list(data_files) if isinstance(data_files, (list, tuple)) else [f for f in str(data_files).split(",") if f]
        if getattr(args, "shuffle", False):
            import random
            files = list(files)
            random.Random(int(getattr(args, "seed", 0))).shuffle(files)

        def file_rows(f):
            import json
            if str(f).endswith(".parquet"):
                yield from iter_parquet_rows(f)
            else:
                with open(f) as fh:
                    for line in fh:
                        if line.strip():
                            yield json.loads(line)

        def rows():
            # every data-parallel replica reads its own part: whole files when there are at least as many files as
            # replicas, else every dp-th row of every file
            by_file = len(files) >= mesh.dp
            n = 0
            for i, f in enumerate(files):
                if by_file and i % mesh.dp != mesh.dp_rank:
                    continue
                for row in file_rows(f):
                    if by_file or n % mesh.dp == mesh.dp_rank:
                        yield row
                    n += 1
        ds = StreamingDataset(rows(), tok, getattr(args, "text_field", "content"), getattr(args, "stage", "pretrain"),
                              max_len=seq_len, split_long=bool(getattr(args, "split_long_documents", False)))
    else:
        # hub datasets named by --pretrain_* / --sft_* (ModelScope first with --use_modelscope, hub as the fallback)
        from .sources import build_hub_dataset
        ds = build_hub_dataset(args, tok, seq_len)
    q = queue.Queue(maxsize=2)
    pb = PrefetchBatcher(ds, [q], local_batch, seq_len, cfg.pack_chunk_size, int(getattr(args, "pack_buffer_size", 2048)),
                         pad_id=getattr(tok, "pad_token_id", 0) or 0, eos_id=getattr(tok, "eos_token_id", None))
    return QueueIterator(q), pb
