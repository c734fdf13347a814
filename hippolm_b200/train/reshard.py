"""Tensor-parallel model shards <-> the plain single-file layout.

A run with TP > 1 writes one model shard per rank. ``merge_tp_state_dicts`` puts the shards of one data-parallel replica
back together into the plain layout (what TP = 1 saves and what the eval server loads); ``split_plain_state_dict`` cuts a
plain state dict into the shard of one TP rank (to start a TP run from a plain checkpoint, a converted checkpoint of the
reference, or shards merged from another TP size). Optimizer state is not resharded: a run started from resharded weights
starts its moments afresh.

How a tensor is sharded follows from its name (the names are those of the saved state dict):

  rows (dim 0)     embed_tokens, lm_head, attn.{b_proj,f_proj1,g_proj1}.weight, g_proj1.bias, A_log, dt_bias, *_conv1d
  columns (dim 1)  attn.o_proj, ffn.down_proj
  sections         attn.qkv_proj: a rank holds [q_r | k_r | v_r]; ffn.gate_up_proj: [gate_r | up_r]; the plain tensor is
                   [q_0 .. q_w-1 | k_0 .. | v_0 ..] resp. [gate_0 .. | up_0 ..]
  replicated       every norm weight, attn.fg_first, attn_res.*

NVFP4 FFN weights without a master copy are stored per rank as packed codes with that rank's own tensor scale; merged files
carry them as their exact dequantised values under ``...weight`` (``NVFP4Linear`` quantises such a tensor when it loads it),
and a split quantises the rank's slice again.
"""
from __future__ import annotations

import os
import re
from typing import Dict, List, Optional

import torch

from ..config import HippoConfig
from . import checkpoint as ckpt

_ROWS = re.compile(r"(embed_tokens\.weight|lm_head\.weight|attn\.(b_proj|f_proj1|g_proj1)\.weight|attn\.g_proj1\.bias|"
                   r"attn\.A_log|attn\.dt_bias|attn\.[qkv]_conv1d\.weight)$")
_COLS = re.compile(r"(attn\.o_proj\.weight|ffn\.down_proj\.weight)$")
_FP4 = ("packed_weight", "scales", "global_scale")


def _qkv_sections(key: str, cfg: HippoConfig, rows_total: int) -> List[int]:
    """Row counts of the q, k, v sections of a full (TP = 1) fused projection."""
    li = int(re.match(r"layers\.(\d+)\.", key).group(1))
    if cfg.layer_types()[li] == "kda":
        secs = [cfg.key_dim, cfg.key_dim, cfg.value_dim]
    else:
        secs = [cfg.num_heads * cfg.head_dim] * 3
    assert sum(secs) == rows_total, (key, secs, rows_total)
    return secs


def _merge_sections(parts: List[torch.Tensor], secs_full: List[int], w: int) -> torch.Tensor:
    out = []
    for si, n in enumerate(secs_full):
        off = sum(secs_full[:si]) // w
        out += [p[off:off + n // w] for p in parts]
    return torch.cat(out, 0)


def _split_sections(full: torch.Tensor, secs_full: List[int], w: int, r: int) -> torch.Tensor:
    out, off = [], 0
    for n in secs_full:
        out.append(full[off + r * (n // w):off + (r + 1) * (n // w)])
        off += n
    return torch.cat(out, 0)


def _dequant_fp4(sd: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    from .. import ops
    return ops.nvfp4_dequantize(sd[prefix + "packed_weight"], sd[prefix + "scales"], sd[prefix + "global_scale"],
                                torch.bfloat16)


def merge_tp_state_dicts(shards: List[Dict[str, torch.Tensor]], cfg: HippoConfig) -> Dict[str, torch.Tensor]:
    """Plain state dict from the model state dicts of TP ranks 0 .. w-1 (one data-parallel replica)."""
    w = len(shards)
    if w == 1:
        return dict(shards[0])
    # NVFP4 modules without a master: exact dequantised values, then merged like any bf16 weight
    shards = [dict(s) for s in shards]
    for s in shards:
        for k in [k for k in s if k.endswith(".packed_weight")]:
            pre = k[:-len("packed_weight")]
            s[pre + "weight"] = _dequant_fp4(s, pre)
            for n in _FP4:
                s.pop(pre + n, None)
    out: Dict[str, torch.Tensor] = {}
    for k, v0 in shards[0].items():
        parts = [s[k] for s in shards]
        if k.endswith("attn.qkv_proj.weight"):
            out[k] = _merge_sections(parts, _qkv_sections(k, cfg, v0.shape[0] * w), w)
        elif k.endswith("ffn.gate_up_proj.weight"):
            out[k] = _merge_sections(parts, [v0.shape[0] * w // 2] * 2, w)
        elif _ROWS.search(k):
            out[k] = torch.cat(parts, 0)
        elif _COLS.search(k):
            out[k] = torch.cat(parts, 1)
        else:
            out[k] = v0                                               # replicated
    return out


def split_plain_state_dict(plain: Dict[str, torch.Tensor], cfg: HippoConfig, tp: int, rank: int,
                           nvfp4_no_master: Optional[bool] = None) -> Dict[str, torch.Tensor]:
    """The shard of TP rank ``rank`` (of ``tp``) from a plain state dict. ``nvfp4_no_master`` (default: the config's
    setting): store the FFN weights as NVFP4 codes with the rank's own tensor scale, as a no-master run keeps them."""
    if nvfp4_no_master is None:
        nvfp4_no_master = bool(cfg.ffn_nvfp4 and cfg.ffn_nvfp4_no_bf16_master)
    plain = dict(plain)
    for k in [k for k in plain if k.endswith(".packed_weight")]:          # a plain NVFP4 file: work on the values
        pre = k[:-len("packed_weight")]
        plain[pre + "weight"] = _dequant_fp4(plain, pre)
        for n in _FP4:
            plain.pop(pre + n, None)
    out: Dict[str, torch.Tensor] = {}
    for k, v in plain.items():
        if tp == 1:
            t = v
        elif k.endswith("attn.qkv_proj.weight"):
            t = _split_sections(v, _qkv_sections(k, cfg, v.shape[0]), tp, rank)
        elif k.endswith("ffn.gate_up_proj.weight"):
            t = _split_sections(v, [v.shape[0] // 2] * 2, tp, rank)
        elif _ROWS.search(k):
            n = v.shape[0] // tp
            t = v[rank * n:(rank + 1) * n]
        elif _COLS.search(k):
            n = v.shape[1] // tp
            t = v[:, rank * n:(rank + 1) * n]
        else:
            t = v
        t = t.contiguous()
        if nvfp4_no_master and re.search(r"ffn\.(gate_up_proj|down_proj)\.weight$", k):
            from .. import ops
            packed, scales, gs = ops.nvfp4_quantize(t.float())
            pre = k[:-len("weight")]
            out[pre + "packed_weight"], out[pre + "scales"], out[pre + "global_scale"] = packed, scales, gs.float()
        else:
            out[k] = t
    return out


def merge_checkpoint(path: str, cfg: HippoConfig, out_path: Optional[str] = None) -> Dict[str, object]:
    """Reads the canonical checkpoint file ``path`` of a multi-rank run (its manifest and per-rank shards beside it), merges
    the model shards of data-parallel replica 0 and, with ``out_path``, writes ``{"step", "model_state_dict", "loss"}``."""
    man = ckpt.read_manifest(path)
    if man is None or int(man.get("tp", 1)) == 1:
        ck = torch.load(path, map_location="cpu", weights_only=False)
        sd, step, loss = ck["model_state_dict"], int(ck.get("step", 0)), ck.get("loss")
    else:
        if not ckpt.is_complete(path):
            raise FileNotFoundError(f"{path}: shards or manifest missing")
        tp = int(man["tp"])
        d = os.path.dirname(os.path.abspath(path))
        cks = [torch.load(os.path.join(d, man["shards"][r]), map_location="cpu", weights_only=False) for r in range(tp)]
        sd = merge_tp_state_dicts([c["model_state_dict"] for c in cks], cfg)
        step, loss = int(cks[0].get("step", 0)), cks[0].get("loss")
    res = {"step": step, "model_state_dict": sd, "loss": loss}
    if out_path:
        torch.save(res, out_path)
    return res
