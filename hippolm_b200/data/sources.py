"""Hub data sources behind the CLI flags (``--pretrain_dataset_hf/_ms``, ``--pretrain_config``, ``--sft_*``,
``--use_modelscope``, ``--pretrain_multi_source`` and the four ``--pretrain_*_config`` subsets, ``--shuffle``).

What the reference does in ``src/training/loop/setup.py:172-306`` and ``src/training/data/sources.py:68-157``:
pick (hub name, ModelScope name, config) from the stage, build one ``StreamingDataset`` (or four, scheduled in two
phases: multi-style first, then QA, English : Chinese = 2 : 1), and open every dataset through a fallback chain
"ModelScope parquet parts with a rotating local cache -> ModelScope streaming -> hub streaming" in which only
network errors and a missing client library fall through.

Every network touchpoint sits behind a small adapter object so that the whole path runs, and is tested, without a
network: an adapter lists the parquet parts of (dataset, config), downloads one part to a path, or opens a row
stream. The built-in adapters import ``modelscope`` / ``huggingface_hub`` / ``datasets`` lazily; a missing library
counts as "source unavailable" and the chain moves on. ``register_adapter`` replaces an adapter (tests inject fakes).
"""
from __future__ import annotations

import random
import shutil
from pathlib import Path
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

from .streaming import (MultiSourceStreamingDataset, RotatingParquetIterable, StreamingDataset,
                        load_streaming_with_fallback)


class SourceUnavailable(ConnectionError):
    """The client library of a source is not installed, or the source has nothing for this dataset: try the next one."""


class HubAdapter:
    """Interface of a data hub. ``list_parts`` -> ids of the parquet parts of (dataset, config), in order;
    ``download(part, dest)`` writes one part; ``stream`` -> iterable of row dicts (the non-parquet fallback)."""
    name = "hub"

    def list_parts(self, dataset: str, config: Optional[str]) -> List[str]:
        raise SourceUnavailable(f"{self.name}: listing is not supported")

    def download(self, dataset: str, part: str, dest: Path) -> None:
        raise SourceUnavailable(f"{self.name}: download is not supported")

    def stream(self, dataset: str, config: Optional[str], split: str) -> Iterable[dict]:
        raise SourceUnavailable(f"{self.name}: streaming is not supported")


def _parts_of_config(files: Sequence[str], config: Optional[str]) -> List[str]:
    out = [f for f in files if f.endswith(".parquet")]
    if config:
        out = [f for f in out if f"/{config}/" in f"/{f}" or Path(f).name.startswith(config)]
    return sorted(out)


class HuggingFaceAdapter(HubAdapter):
    name = "huggingface"

    def list_parts(self, dataset, config):
        try:
            from huggingface_hub import HfApi
        except ImportError as ex:
            raise SourceUnavailable(f"huggingface_hub is not installed ({ex})")
        return _parts_of_config(HfApi().list_repo_files(dataset, repo_type="dataset"), config)

    def download(self, dataset, part, dest):
        from huggingface_hub import hf_hub_download
        shutil.copyfile(hf_hub_download(dataset, part, repo_type="dataset"), dest)

    def stream(self, dataset, config, split):
        try:
            from datasets import load_dataset
        except ImportError as ex:
            raise SourceUnavailable(f"datasets is not installed ({ex})")
        kw = dict(split=split, streaming=True)
        if config:
            kw["name"] = config
        return load_dataset(dataset, **kw)


class ModelScopeAdapter(HubAdapter):
    name = "modelscope"

    def _api(self):
        try:
            from modelscope.hub.api import HubApi
        except ImportError as ex:
            raise SourceUnavailable(f"modelscope is not installed ({ex})")
        return HubApi()

    def list_parts(self, dataset, config):
        api = self._api()
        owner, _, name = dataset.partition("/")
        files = [f.get("Path") or f.get("Name") for f in api.get_dataset_files(f"{owner}/{name}", recursive=True)]
        return _parts_of_config([f for f in files if f], config)

    def download(self, dataset, part, dest):
        self._api()
        from modelscope.hub.file_download import dataset_file_download
        shutil.copyfile(dataset_file_download(dataset, part), dest)

    def stream(self, dataset, config, split):
        self._api()
        from modelscope.msdatasets import MsDataset
        return MsDataset.load(dataset, subset_name=config, split=split, use_streaming=True)


_ADAPTERS: Dict[str, HubAdapter] = {"modelscope": ModelScopeAdapter(), "huggingface": HuggingFaceAdapter()}


def register_adapter(name: str, adapter: HubAdapter) -> Optional[HubAdapter]:
    """Install ``adapter`` under ``name`` ('modelscope' | 'huggingface'); returns the one it replaced."""
    old = _ADAPTERS.get(name)
    _ADAPTERS[name] = adapter
    return old


def open_rows(hf_name: Optional[str], ms_name: Optional[str], config: Optional[str], use_modelscope: bool,
              shuffle: bool = False, seed: int = 0, split: str = "train", cache_root: Optional[Path] = None,
              logger=None) -> Iterable[dict]:
    """Row stream of one dataset through the fallback chain. With ``shuffle`` the parquet parts are visited in a seeded
    random order (rows inside a part keep their order: a part is read once, front to back, then evicted)."""
    chain: List[Tuple[str, Callable[[], Iterable]]] = []

    def rotating(adapter: HubAdapter, dataset: str):
        def make():
            parts = list(adapter.list_parts(dataset, config))
            if not parts:
                raise SourceUnavailable(f"{adapter.name}: no parquet parts for {dataset} (config={config})")
            if shuffle:
                random.Random(seed).shuffle(parts)
            rot = RotatingParquetIterable(dataset, config, lambda: parts,
                                          lambda part, dest: adapter.download(dataset, part, Path(dest)),
                                          cache_root=cache_root)
            rot.open()                      # synchronous download of the first part: failures surface here
            return rot
        return make

    def streaming(adapter: HubAdapter, dataset: str):
        return lambda: adapter.stream(dataset, config, split)

    if use_modelscope and ms_name:
        ms = _ADAPTERS["modelscope"]
        chain += [(f"modelscope parquet parts of {ms_name}", rotating(ms, ms_name)),
                  (f"modelscope streaming of {ms_name}", streaming(ms, ms_name))]
    if hf_name:
        hf = _ADAPTERS["huggingface"]
        chain += [(f"hub parquet parts of {hf_name}", rotating(hf, hf_name)),
                  (f"hub streaming of {hf_name}", streaming(hf, hf_name))]
    if not chain:
        raise ValueError("no dataset configured: set use_dummy_data / synthetic_data, data_files, or a "
                         "--pretrain_dataset_hf / --pretrain_dataset_ms / --sft_dataset_* name")
    return load_streaming_with_fallback(chain, logger)


def dataset_plan(args) -> List[Tuple[str, Optional[str], Optional[str], Optional[str]]]:
    """(label, hub name, ModelScope name, config) of every sub-dataset the flags ask for."""
    if getattr(args, "stage", "pretrain") == "sft":
        return [("sft", getattr(args, "sft_dataset_hf", None), getattr(args, "sft_dataset_ms", None),
                 getattr(args, "sft_config", None))]
    hf, ms = getattr(args, "pretrain_dataset_hf", None), getattr(args, "pretrain_dataset_ms", None)
    if getattr(args, "pretrain_multi_source", False):
        return [(label, hf, ms, getattr(args, f"pretrain_{label}_config", None))
                for label in ("en_multi", "zh_multi", "en_qa", "zh_qa")]
    return [("pretrain", hf, ms, getattr(args, "pretrain_config", None))]


# two phases: the multi-style subsets first, then the QA subsets; English : Chinese = 2 : 1 inside a phase
MULTI_SOURCE_PHASES = [{"en_multi": 2, "zh_multi": 1}, {"en_qa": 2, "zh_qa": 1}]


def build_hub_dataset(args, tokenizer, seq_len: int, logger=None, cache_root: Optional[Path] = None):
    """Token-list iterable for the hub datasets the CLI flags name (one dataset, or the four-subset two-phase schedule)."""
    stage = getattr(args, "stage", "pretrain")
    plan = dataset_plan(args)
    seed = int(getattr(args, "seed", 0))

    def sub(label, hf, ms, cfg):
        rows = open_rows(hf, ms, cfg, bool(getattr(args, "use_modelscope", False)), bool(getattr(args, "shuffle", False)),
                         seed, cache_root=cache_root, logger=logger)
        return StreamingDataset(rows, tokenizer, getattr(args, "text_field", "content"), stage, max_len=seq_len,
                                split_long=bool(getattr(args, "split_long_documents", False)))

    if len(plan) == 1:
        return sub(*plan[0])

    class _Lazy:
        """Opens its dataset when the schedule first reaches it (a later phase costs nothing until then)."""

        def __init__(self, spec):
            self.spec = spec

        def __iter__(self):
            return iter(sub(*self.spec))

    subs = {spec[0]: _Lazy(spec) for spec in plan}
    # a phase ends when its subsets are exhausted (the per-phase document count is unbounded)
    schedule = [(1 << 62, weights) for weights in MULTI_SOURCE_PHASES]
    return MultiSourceStreamingDataset(subs, schedule)
