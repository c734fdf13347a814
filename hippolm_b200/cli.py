"""Command line + YAML overlay (same surface as the reference's ``scripts/cli.py:34-470``).

* ``--config file.yml``: top-level YAML keys become parser defaults, so explicit flags win.
* ``extends: other.yml`` (relative to the child file): recursive, *shallow* merge, child wins,
  cycles are an error.
* nested ``optimizer: {adamw: {...}, muon: {...}}`` is flattened to ``learning_rate / weight_decay /
  adamw_beta1 / adamw_beta2 / adamw_eps / muon_lr / muon_weight_decay / muon_momentum``; a flat key
  given next to the block wins over the block.
* ``precision:`` passes through as a dict; unknown YAML keys become Namespace attributes.
"""
from __future__ import annotations

import argparse
import os
from typing import Any, Dict, List, Optional

import yaml


def _bool(v) -> bool:
    if isinstance(v, bool):
        return v
    s = str(v).strip().lower()
    if s in ("1", "true", "yes", "y", "on"):
        return True
    if s in ("0", "false", "no", "n", "off"):
        return False
    raise argparse.ArgumentTypeError(f"expected a boolean, got {v!r}")


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="hippolm_b200 training")

    def a(*names, **kw):
        # boolean flags take a value (``--flag false``) or stand alone (``--flag`` = true, the way the reference's
        # store_true flags ``--use_dummy_data`` and ``--tp_sim`` are typed)
        if kw.get("type") is _bool:
            kw.setdefault("nargs", "?")
            kw.setdefault("const", True)
        return p.add_argument(*names, **kw)

    a("--config", type=str, default=None)
    # model
    a("--vocab_size", type=int, default=32000); a("--hidden_size", type=int, default=256)
    a("--tie_word_embeddings", type=_bool, default=False); a("--use_bias", type=_bool, default=False)
    a("--num_heads", type=int, default=4); a("--head_dim", type=int, default=64)
    a("--expand_v", type=float, default=1.0); a("--kda_mode", type=str, default="chunk")
    a("--use_short_conv", type=_bool, default=False); a("--allow_neg_eigval", type=_bool, default=False)
    a("--safe_gate", type=_bool, default=False); a("--lower_bound", type=float, default=-5.0)
    a("--conv_size", type=int, default=4); a("--conv_bias", type=_bool, default=False)
    a("--num_layers", type=int, default=4); a("--num_blocks", type=int, default=1)
    a("--attn_res_heads", type=int, default=0)
    a("--full_attn_interval", type=int, default=4); a("--rope_theta", type=float, default=10000.0)
    a("--intermediate_size", type=int, default=1024); a("--rms_norm_eps", type=float, default=1e-6)
    a("--ffn_nvfp4", type=_bool, default=False); a("--ffn_nvfp4_marlin", type=_bool, default=False)
    a("--ffn_nvfp4_no_bf16_master", type=_bool, default=False); a("--nvfp4_stochastic_rounding", type=_bool, default=True); a("--ffn_nvfp4_backward", type=str, default="bf16")
    a("--gradient_checkpointing", type=_bool, default=False); a("--lce_num_chunks", type=int, default=0)
    a("--lce_epilogue_stats", type=_bool, default=True)
    # training
    a("--batch_size", type=int, default=1); a("--seq_len", type=int, default=512)
    a("--micro_batch_size", type=int, default=0)
    a("--learning_rate", type=float, default=0.004); a("--weight_decay", type=float, default=0.01)
    a("--adamw_beta1", type=float, default=0.9); a("--adamw_beta2", type=float, default=0.95)
    a("--adamw_eps", type=float, default=1e-8); a("--adamw_reference_compat", type=_bool, default=False)
    a("--muon_lr", type=float, default=0.02); a("--muon_weight_decay", type=float, default=0.0)
    a("--muon_momentum", type=float, default=0.95); a("--muon_ns_scope", type=str, default="full"); a("--muon_dp_shard", type=_bool, default=True); a("--muon_ns_row_chunk", type=int, default=None)
    a("--epochs", type=int, default=1); a("--max_steps", type=int, default=1000)
    a("--gradient_accumulation_steps", type=int, default=1)
    a("--lr_warmup_steps", type=int, default=0); a("--lr_decay_steps", type=int, default=0)
    a("--max_grad_norm", type=float, default=1.0); a("--seed", type=int, default=42)
    a("--carry_kda_state", type=_bool, default=False); a("--trainable_regex", type=str, default=None)
    # logging / checkpoints
    a("--log_interval", type=int, default=1); a("--checkpoint_interval", type=int, default=0)
    a("--checkpoint_keep_last_n", type=int, default=3); a("--output_dir", type=str, default="output")
    a("--max_restarts", type=int, default=0)
    a("--init_from", type=str, default=None)
    a("--resume", type=str, default=None); a("--diagnostics", type=_bool, default=False)
    a("--mb_timing", type=int, default=0); a("--vram_phases", type=_bool, default=False); a("--empty_cache_between_mb", type=_bool, default=False)
    a("--peer_timeout_s", type=float, default=0.0); a("--dist_timeout_s", type=float, default=1800.0); a("--watchdog_timeout_s", type=float, default=0.0)
    # data
    a("--stage", type=str, default="pretrain"); a("--use_modelscope", type=_bool, default=False)
    a("--pretrain_dataset_hf", type=str, default=None); a("--pretrain_dataset_ms", type=str, default=None)
    a("--pretrain_config", type=str, default=None); a("--pretrain_multi_source", type=_bool, default=False)
    a("--pretrain_en_multi_config", type=str, default=None); a("--pretrain_zh_multi_config", type=str, default=None)
    a("--pretrain_en_qa_config", type=str, default=None); a("--pretrain_zh_qa_config", type=str, default=None)
    a("--sft_dataset_hf", type=str, default=None); a("--sft_dataset_ms", type=str, default=None)
    a("--sft_config", type=str, default=None); a("--text_field", type=str, default="content")
    a("--split_long_documents", type=_bool, default=False)
    a("--data_files", type=str, default=None)        # local .jsonl / .parquet files, comma separated (or a YAML list)
    a("--tokenizer_path", type=str, default=None); a("--cache_dir", type=str, default=None)
    a("--use_dummy_data", type=_bool, default=False); a("--synthetic_data", type=_bool, default=False)
    a("--doc_len_min", type=int, default=0); a("--doc_len_max", type=int, default=0)
    a("--doc_align", type=int, default=1); a("--fixed_batch", type=_bool, default=False); a("--shuffle", type=_bool, default=False)
    a("--pack_chunk_size", type=int, default=0); a("--pack_buffer_size", type=int, default=2048)
    a("--kda_skip_aqk_akk_saved", type=_bool, default=False)
    # parallel / devices
    a("--min_gpu_memory_mb", type=int, default=10240); a("--tp_sim", type=_bool, default=False)
    a("--tp_size", type=int, default=1); a("--dp_size", type=int, default=0)
    a("--nproc", type=int, default=0); a("--dp_overlap", type=_bool, default=True)
    a("--dp_reduce_to_owner", type=_bool, default=True)
    a("--fused_comm", type=_bool, default=True); a("--fused_wait_ms", type=float, default=0.0)
    a("--offload_optimizer", type=_bool, default=False); a("--offload_grads", type=_bool, default=False)
    a("--precision", type=str, default=None)
    return p


_OPT_MAP = {("adamw", "lr"): "learning_rate", ("adamw", "weight_decay"): "weight_decay",
            ("adamw", "beta1"): "adamw_beta1", ("adamw", "beta2"): "adamw_beta2", ("adamw", "eps"): "adamw_eps",
            ("muon", "lr"): "muon_lr", ("muon", "weight_decay"): "muon_weight_decay",
            ("muon", "momentum"): "muon_momentum"}


def _flatten_optimizer_overrides(cfg: Dict[str, Any]) -> Dict[str, Any]:
    out = dict(cfg)
    block = out.pop("optimizer", None)
    if isinstance(block, dict):
        for sect, d in block.items():
            if not isinstance(d, dict):
                continue
            for k, v in d.items():
                flat = _OPT_MAP.get((sect, k))
                if flat is None:
                    raise ValueError(f"unknown optimizer key optimizer.{sect}.{k}")
                if flat not in cfg:            # a flat key written next to the block wins
                    out[flat] = float(v) if isinstance(v, str) else v
    return out


def _load_yaml_with_extends(path: str, _stack: Optional[List[str]] = None) -> Dict[str, Any]:
    ap = os.path.abspath(path)
    stack = _stack or []
    if ap in stack:
        raise ValueError("circular 'extends' chain: " + " -> ".join(stack + [ap]))
    with open(ap) as f:
        cfg = yaml.safe_load(f) or {}
    if not isinstance(cfg, dict):
        raise ValueError(f"{path}: top level must be a mapping")
    parent = cfg.pop("extends", None)
    if parent:
        pp = parent if os.path.isabs(parent) else os.path.join(os.path.dirname(ap), parent)
        base = _load_yaml_with_extends(pp, stack + [ap])
        base.update(cfg)                        # shallow merge, child wins
        cfg = base
    return cfg


def parse_args(argv: Optional[List[str]] = None) -> argparse.Namespace:
    parser = build_parser()
    pre = argparse.ArgumentParser(add_help=False)
    pre.add_argument("--config", type=str, default=None)
    known, _ = pre.parse_known_args(argv)
    extra: Dict[str, Any] = {}
    if known.config:
        cfg = _flatten_optimizer_overrides(_load_yaml_with_extends(known.config))
        dests = {a.dest for a in parser._actions}
        defaults = {}
        for k, v in cfg.items():
            if k in dests and k != "precision":
                if k in ("adamw_eps", "learning_rate", "muon_lr", "rms_norm_eps", "weight_decay") and isinstance(v, str):
                    v = float(v)
                defaults[k] = v
            else:
                extra[k] = v
        parser.set_defaults(**defaults)
    ns = parser.parse_args(argv)
    for k, v in extra.items():
        if k == "precision":
            ns.precision = v
        elif not hasattr(ns, k):
            setattr(ns, k, v)
    if isinstance(ns.precision, str):
        ns.precision = {c: {"dtype": ns.precision} for c in
                        ("model_weights", "gradients", "activations", "muon_momentum", "adamw_m", "adamw_v")}
    return ns
