"""CLI flags -> hub data sources (fake adapters, no network): single dataset, SFT, the four-subset two-phase schedule,
ModelScope-first fallback order, part shuffling, and a training run fed through the flags over two epochs."""
import os
from pathlib import Path

import pyarrow as pa
import pyarrow.parquet as pq
import pytest

from hippolm_b200.cli import build_parser
from hippolm_b200.data import sources
from hippolm_b200.data.tokenizer import ByteTokenizer


class FakeHub(sources.HubAdapter):
    def __init__(self, name, datasets, fail=None):
        self.name, self.datasets, self.fail, self.log = name, datasets, fail, []

    def list_parts(self, dataset, config):
        self.log.append(("list", dataset, config))
        if self.fail:
            raise self.fail
        return sorted(p for p in self.datasets.get(dataset, {}) if config is None or f"{config}/" in p)

    def download(self, dataset, part, dest):
        self.log.append(("get", dataset, part))
        pq.write_table(pa.table({"content": self.datasets[dataset][part]}), str(dest))


@pytest.fixture
def hubs():
    data = {"org/web": {"en_multi/p0.parquet": ["EM0", "EM1", "EM2", "EM3"], "zh_multi/p0.parquet": ["ZM0", "ZM1"],
                        "en_qa/p0.parquet": ["EQ0", "EQ1"], "zh_qa/p0.parquet": ["ZQ0"],
                        "plain/p0.parquet": ["A0", "A1"], "plain/p1.parquet": ["B0", "B1"], "plain/p2.parquet": ["C0", "C1"]},
            "org/sft": {"p0.parquet": ["unused"]}}
    ms, hf = FakeHub("modelscope", data), FakeHub("huggingface", data)
    old = [sources.register_adapter("modelscope", ms), sources.register_adapter("huggingface", hf)]
    yield ms, hf
    sources.register_adapter("modelscope", old[0]); sources.register_adapter("huggingface", old[1])


def _texts(ds):
    tok = ByteTokenizer()
    return [tok.decode(d).replace("<|endoftext|>", "").strip("\x00") for d in ds]


def _args(**kw):
    a = build_parser().parse_args([])
    for k, v in kw.items():
        setattr(a, k, v)
    return a


def test_single_dataset_modelscope_first_then_hub_fallback(hubs, tmp_path):
    ms, hf = hubs
    a = _args(pretrain_dataset_hf="org/web", pretrain_dataset_ms="org/web", pretrain_config="plain", use_modelscope=True)
    out = _texts(sources.build_hub_dataset(a, ByteTokenizer(), 64, cache_root=tmp_path))
    assert [t[:2] for t in out] == ["A0", "A1", "B0", "B1", "C0", "C1"]
    assert ms.log[0] == ("list", "org/web", "plain") and not hf.log          # ModelScope answered: the hub is not asked
    ms.fail = ConnectionError("mirror down"); ms.log.clear()
    out = _texts(sources.build_hub_dataset(a, ByteTokenizer(), 64, cache_root=tmp_path / "b"))
    assert len(out) == 6 and hf.log[0][0] == "list"                           # network error -> hub
    a.use_modelscope = False; hf.log.clear(); ms.log.clear()
    sources.build_hub_dataset(a, ByteTokenizer(), 64, cache_root=tmp_path / "c")
    assert not ms.log and hf.log
    hf.fail = ValueError("bad config")                                        # not a network error: must propagate
    with pytest.raises(ValueError):
        sources.build_hub_dataset(a, ByteTokenizer(), 64, cache_root=tmp_path / "d")


def test_shuffle_changes_part_order_deterministically(hubs, tmp_path):
    a = _args(pretrain_dataset_hf="org/web", pretrain_config="plain", shuffle=True, seed=1)
    o1 = _texts(sources.build_hub_dataset(a, ByteTokenizer(), 64, cache_root=tmp_path / "a"))
    o2 = _texts(sources.build_hub_dataset(a, ByteTokenizer(), 64, cache_root=tmp_path / "b"))
    assert o1 == o2 and sorted(o1) == sorted(["A0", "A1", "B0", "B1", "C0", "C1"])
    orders = set()
    for seed in range(6):
        a.seed = seed
        orders.add(tuple(_texts(sources.build_hub_dataset(a, ByteTokenizer(), 64, cache_root=tmp_path / f"s{seed}"))))
    assert len(orders) > 1


def test_multi_source_two_phases_two_to_one(hubs, tmp_path):
    a = _args(pretrain_dataset_hf="org/web", pretrain_multi_source=True, pretrain_en_multi_config="en_multi",
              pretrain_zh_multi_config="zh_multi", pretrain_en_qa_config="en_qa", pretrain_zh_qa_config="zh_qa")
    assert [p[0] for p in sources.dataset_plan(a)] == ["en_multi", "zh_multi", "en_qa", "zh_qa"]
    out = _texts(sources.build_hub_dataset(a, ByteTokenizer(), 64, cache_root=tmp_path))
    assert out[:6] == ["EM0", "EM1", "ZM0", "EM2", "EM3", "ZM1"]              # phase 1: en, en, zh, ...
    assert out[6:] == ["EQ0", "EQ1", "ZQ0"]                                   # phase 2 only after phase 1 is exhausted
    hf = hubs[1]
    first_qa = next(i for i, e in enumerate(hf.log) if e[0] == "list" and e[2] == "en_qa")
    last_multi = max(i for i, e in enumerate(hf.log) if e[0] == "get" and "multi" in e[2])
    assert first_qa > last_multi                                              # the QA subsets are opened lazily


def test_sft_plan():
    a = _args(stage="sft", sft_dataset_hf="org/sft", sft_dataset_ms="ms/sft", sft_config="c")
    assert sources.dataset_plan(a) == [("sft", "org/sft", "ms/sft", "c")]
    with pytest.raises(ValueError):
        sources.open_rows(None, None, None, True)


def test_training_loop_reads_hub_flags_for_two_epochs(hubs, tmp_path, monkeypatch):
    from hippolm_b200.train.loop import setup_worker, run_training_loop
    monkeypatch.setenv("HIPPOLM_CACHE_DIR", str(tmp_path / "cache"))
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(k, raising=False)
    hubs[1].datasets["org/web"]["plain/p0.parquet"] = ["some text " * 30] * 8
    a = _args(pretrain_dataset_hf="org/web", pretrain_config="plain", vocab_size=512, hidden_size=32, num_heads=2,
              head_dim=16, num_layers=2, num_blocks=1, intermediate_size=64, full_attn_interval=0, batch_size=2,
              seq_len=128, max_steps=50, epochs=2, gradient_accumulation_steps=2)
    hubs[1].datasets["org/web"] = {"plain/p0.parquet": hubs[1].datasets["org/web"]["plain/p0.parquet"]}
    res = run_training_loop(setup_worker(a, run_dir=None))
    n_opens = sum(1 for e in hubs[1].log if e[0] == "list")
    assert n_opens == 2 and res["steps"] >= 2 and all(l == l for l in res["losses"])
