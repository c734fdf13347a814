"""Streaming datasets, rotating parquet cache (injected list/download functions, no network), prefetch fan-out."""
import queue

import pyarrow as pa
import pyarrow.parquet as pq
import pytest
import torch

from hippolm_b200.data.prefetch import PrefetchBatcher, QueueIterator
from hippolm_b200.data.streaming import (RotatingParquetIterable, StreamingDataset, MultiSourceStreamingDataset,
                                         load_streaming_with_fallback, list_cached_parts)
from hippolm_b200.data.tokenizer import ByteTokenizer, load_tokenizer


def _make_download(log):
    def download(part, dest):
        log.append(part)
        pq.write_table(pa.table({"content": [f"part{part} row{i}" for i in range(10)]}), str(dest))
    return download


def test_rotating_parquet_prefetch_and_eviction(tmp_path):
    log = []
    it = RotatingParquetIterable("org/ds", "cfg", lambda: [0, 1, 2], _make_download(log), cache_root=tmp_path)
    rows = list(it)
    assert len(rows) == 30 and rows[0]["content"] == "part0 row0" and rows[-1]["content"] == "part2 row9"
    assert log == [0, 1, 2]
    assert it.max_files_seen <= 2                       # never more than the current and the next part on disk
    assert len(list_cached_parts("org/ds", "cfg", tmp_path)) == 1


def test_rotating_parquet_download_error_surfaces(tmp_path):
    def bad(part, dest):
        if part == 1:
            raise ConnectionError("boom")
        pq.write_table(pa.table({"content": ["x"] * 4}), str(dest))
    it = RotatingParquetIterable("d", None, lambda: [0, 1], bad, cache_root=tmp_path)
    with pytest.raises(ConnectionError):
        list(it)


def test_streaming_dataset_pretrain_and_sft():
    tok = ByteTokenizer()
    ds = StreamingDataset([{"content": "ab"}, {"content": ""}, {"other": 1}, {"content": "xyz"}], tok)
    docs = list(ds)
    assert docs == [[97, 98, 256], [120, 121, 122, 256]]
    sft = StreamingDataset([{"instruction": "hi", "output": "yo"}], tok, stage="sft")
    text = tok.decode(list(sft)[0])
    assert "<|im_start|>user\nhi<|im_end|>" in text and "assistant\nyo" in text
    assert isinstance(load_tokenizer(None), ByteTokenizer)


def test_multi_source_schedule():
    a, b = ([f"a{i}"] for i in range(100)), ([f"b{i}"] for i in range(3))
    ms = MultiSourceStreamingDataset({"a": a, "b": b}, [(4, {"a": 1, "b": 1}), (4, {"a": 3, "b": 1})])
    out = [d[0] for d in ms]
    assert out[:4] == ["a0", "b0", "a1", "b1"] and len(out) == 8 and out[4:7] == ["a2", "a3", "a4"]


def test_fallback_only_on_network_errors():
    def down():
        raise ConnectionError("x")
    assert load_streaming_with_fallback([("hf", down), ("ms", lambda: [1, 2])]) == [1, 2]
    def bad():
        raise ValueError("config")
    with pytest.raises(ValueError):
        load_streaming_with_fallback([("hf", bad), ("ms", lambda: [1])])
    with pytest.raises(ConnectionError):
        load_streaming_with_fallback([("hf", down)])


def test_prefetch_fanout_sentinel_and_exception():
    docs = [[1] * 40 for _ in range(12)]
    qs = [queue.Queue(maxsize=8) for _ in range(2)]      # drained one after the other below
    pb = PrefetchBatcher(iter(docs), qs, batch_size=2, seq_len=128, chunk_size=64, pack_buffer_size=2)
    outs = [list(QueueIterator(q, timeout_s=10)) for q in qs]
    pb.close()
    assert len(outs[0]) == len(outs[1]) == 3
    assert torch.equal(outs[0][0]["input_ids"], outs[1][0]["input_ids"]) and outs[0][0]["input_ids"].shape == (256,)
    assert outs[0][0]["cu_seqlens"][-1] == 256

    def broken():
        yield [1, 2, 3]
        raise RuntimeError("tokenizer died")
    q = queue.Queue(maxsize=4)
    pb = PrefetchBatcher(broken(), [q], 1, 64, 64, pack_buffer_size=8)
    with pytest.raises(RuntimeError, match="tokenizer died"):
        list(QueueIterator(q, timeout_s=10))
    pb.close()


def test_prefetch_batcher_emits_every_document_exactly_once():
    """Documents that find no room in a batch are carried into the next one: every document that fits a row at all comes
    out exactly once (the reference discards the overflow of each packing window)."""
    import queue
    import random
    from hippolm_b200.data.prefetch import PrefetchBatcher, QueueIterator
    rng = random.Random(0)
    docs = []
    for i in range(300):
        n = rng.choice([5, 20, 60, 64, 100, 130, 250, 256, 300])           # 300 > seq_len: can never be placed
        docs.append([1000 + i] + [rng.randint(2, 90) for _ in range(n - 1)])
    q = queue.Queue(maxsize=2)
    pb = PrefetchBatcher(iter(docs), [q], batch_size=2, seq_len=256, chunk_size=64, pack_buffer_size=8, pad_id=0, eos_id=None)
    seen = []
    for batch in QueueIterator(q):
        ids, cu = batch["input_ids"], batch["cu_seqlens"].tolist()
        assert ids.numel() == 2 * 256
        for s, e in zip(cu, cu[1:]):
            if int(batch["labels"][s:e].ne(-100).sum()) > 0 or int(ids[s]) >= 1000:
                if int(ids[s]) >= 1000:
                    seen.append(int(ids[s]) - 1000)
    pb.close()
    fits = [i for i, d in enumerate(docs) if len(d) <= 256]
    assert sorted(seen) == fits and len(set(seen)) == len(seen)


def test_local_files_are_split_between_data_parallel_replicas(tmp_path):
    """One file, two replicas: each reads every second row (disjoint, together everything); two files: one file each."""
    import json
    import types
    from hippolm_b200.config import HippoConfig
    from hippolm_b200.data.streaming import build_streaming_iterator
    for nfiles in (1, 2):
        files = []
        for k in range(nfiles):
            p = tmp_path / f"d{nfiles}_{k}.jsonl"
            with open(p, "w") as f:
                for i in range(12):
                    f.write(json.dumps({"content": f"doc{k}x{i} " + "word " * (3 + i)}) + "\n")
            files.append(str(p))
        cfg = HippoConfig(vocab_size=1536, hidden_size=32, num_heads=2, head_dim=16, num_layers=2, num_blocks=1, intermediate_size=64)
        seen = []
        for r in range(2):
            args = types.SimpleNamespace(tokenizer_path="builtin", data_files=",".join(files), text_field="content",
                                         stage="pretrain", pack_buffer_size=8, shuffle=False, seed=0)
            mesh = types.SimpleNamespace(dp=2, dp_rank=r)
            it, pb = build_streaming_iterator(args, cfg, mesh, 2, 128)
            from hippolm_b200.data.tokenizer import load_tokenizer
            tok = load_tokenizer("builtin")
            mine = set()
            for b in it:
                text = tok.decode(b["input_ids"].tolist())
                for k in range(nfiles):
                    for i in range(12):
                        if f"doc{k}x{i} " in text:
                            mine.add((k, i))
            pb.close()
            seen.append(mine)
        assert not (seen[0] & seen[1]) and len(seen[0] | seen[1]) == 12 * nfiles, (nfiles, seen)
        assert len(seen[0]) == len(seen[1]) == 6 * nfiles


def test_long_documents_are_cut_or_split():
    from hippolm_b200.data.streaming import StreamingDataset
    from hippolm_b200.data.tokenizer import ByteTokenizer
    tok = ByteTokenizer()
    rows = [{"content": "a" * 25}, {"content": "bc"}]
    eos = tok.eos_token_id
    cut = list(StreamingDataset(rows, tok, max_len=10))
    assert [len(d) for d in cut] == [10, 3] and cut[0][-1] == eos               # the reference's behaviour: truncated
    split = list(StreamingDataset(rows, tok, max_len=10, split_long=True))
    assert [len(d) for d in split] == [10, 10, 6, 3]                            # 25 tokens + eos in pieces of 10
    flat = [t for d in split[:3] for t in d]
    assert flat[:-1] == tok.encode("a" * 25, add_special_tokens=False) and flat[-1] == eos
    assert all(d[-1] != eos for d in split[:2])


def test_prefetch_batcher_reads_past_a_window_of_over_long_documents():
    import queue
    from hippolm_b200.data.prefetch import PrefetchBatcher, QueueIterator
    docs = [[7] * 500, [7] * 400, [7] * 900, [5] * 30, [6] * 40]           # three documents longer than a row, then two short
    q = queue.Queue(maxsize=2)
    pb = PrefetchBatcher(iter(docs), [q], batch_size=1, seq_len=128, chunk_size=64, pack_buffer_size=4)
    batches = list(QueueIterator(q))
    pb.close()
    assert len(batches) == 1
    ids = batches[0]["input_ids"]
    assert int((ids == 5).sum()) == 30 and int((ids == 6).sum()) == 40 and int((ids == 7).sum()) == 0
