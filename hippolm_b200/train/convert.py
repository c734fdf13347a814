"""Checkpoints of the reference into this framework's plain ``layers.N.*`` layout.

Two layouts exist on the reference's side:

* its single-GPU model (``src/models/model.py:68-107``, the wrapper around the KDA layer of its vendored library):
  ``layers.N.kda.attn.{q,k,v}_proj``, ``f_proj.0/1``, ``g_proj.0/1``, ``b_proj``, ``A_log``, ``dt_bias``,
  ``{q,k,v}_conv1d`` (weights ``[dim, 1, width]``), ``o_norm``, ``o_proj``; ``layers.N.{attn_norm,mlp_norm}``;
  ``layers.N.ffn.{gate,up,down}_proj``; ``embed_tokens``, ``norm``, ``attn_res.*``, ``lm_head``;
* its tensor-parallel model (``src/models/tp_model/model.py:213-372``), one module set per device:
  ``layers_per_device.D.N.kda.{qkv_proj,fg_first,f_proj1,g_proj1,b_proj,...}``, ``layers_per_device.D.N.ffn.{gate_up_proj,
  down_proj}`` (bf16 ``weight`` or the NVFP4 buffers), ``replicated_per_device.D.{embed_tokens,norm,attn_res}``.

Here the parameter names follow the tensor-parallel model without the per-device level (``layers.N.attn.qkv_proj`` ...),
the FFN norm is ``ffn_norm`` and convolution weights are ``[dim, width]``. A tensor-parallel file of the reference written
with more than one device holds trained values for the saving rank's shards only (it saves from rank 0 alone), so it cannot
be completed from the file and is refused.
"""
from __future__ import annotations

import re
from typing import Dict

import torch


def detect_layout(sd: Dict[str, torch.Tensor]) -> str:
    """``"native"``, ``"reference_single"`` or ``"reference_tp"``."""
    keys = list(sd)
    if any(k.startswith("layers_per_device.") or k.startswith("replicated_per_device.") for k in keys):
        return "reference_tp"
    if any(".kda.attn." in k or k.endswith("mlp_norm.weight") for k in keys):
        return "reference_single"
    return "native"


def _conv(w: torch.Tensor) -> torch.Tensor:
    return w.reshape(w.shape[0], w.shape[-1]) if w.dim() == 3 else w


def _from_single(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    layers = sorted({int(m.group(1)) for k in sd for m in [re.match(r"layers\.(\d+)\.", k)] if m})
    for i in layers:
        src, dst = f"layers.{i}.kda.attn.", f"layers.{i}.attn."
        g = lambda name: sd[src + name]                                  # noqa: E731
        out[dst + "qkv_proj.weight"] = torch.cat([g("q_proj.weight"), g("k_proj.weight"), g("v_proj.weight")], 0)
        # the two low-rank gates share one first projection here: rows [f | g]
        out[dst + "fg_first.weight"] = torch.cat([g("f_proj.0.weight"), g("g_proj.0.weight")], 0)
        out[dst + "f_proj1.weight"] = g("f_proj.1.weight")
        out[dst + "g_proj1.weight"] = g("g_proj.1.weight")
        if src + "g_proj.1.bias" in sd:
            out[dst + "g_proj1.bias"] = g("g_proj.1.bias")
        for name in ("b_proj.weight", "A_log", "dt_bias", "o_norm.weight", "o_proj.weight"):
            out[dst + name] = g(name)
        for c in ("q_conv1d", "k_conv1d", "v_conv1d"):
            if src + c + ".weight" in sd:
                out[dst + c + ".weight"] = _conv(g(c + ".weight"))
        out[f"layers.{i}.attn_norm.weight"] = sd[f"layers.{i}.attn_norm.weight"]
        out[f"layers.{i}.ffn_norm.weight"] = sd[f"layers.{i}.mlp_norm.weight"]
        f = f"layers.{i}.ffn."
        out[f + "gate_up_proj.weight"] = torch.cat([sd[f + "gate_proj.weight"], sd[f + "up_proj.weight"]], 0)
        out[f + "down_proj.weight"] = sd[f + "down_proj.weight"]
    for k in ("embed_tokens.weight", "norm.weight", "attn_res.query", "attn_res.norm.weight"):
        if k in sd:
            out[k] = sd[k]
    if "lm_head.weight" in sd and not _same(sd["lm_head.weight"], sd.get("embed_tokens.weight")):
        out["lm_head.weight"] = sd["lm_head.weight"]                      # untied head
    return out


def _same(a, b) -> bool:
    return b is not None and a.shape == b.shape and (a.data_ptr() == b.data_ptr() or torch.equal(a, b))


def _from_tp(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    devs = sorted({m.group(1) for k in sd for m in [re.match(r"(?:layers|replicated|lm_head|fused_lm_ce)_per_device\.(\d+)\.", k)] if m})
    if len(devs) != 1:
        raise ValueError(f"tensor-parallel checkpoint of the reference with {len(devs)} devices: it was saved from one rank "
                         "and holds trained values for that rank's shards only; re-save it from a TP=1 run")
    d = devs[0]
    out: Dict[str, torch.Tensor] = {}
    for k, v in sd.items():
        m = re.match(rf"layers_per_device\.{d}\.(\d+)\.(.*)", k)
        if m:
            i, rest = m.group(1), m.group(2)
            rest = re.sub(r"^kda\.", "attn.", rest)
            rest = re.sub(r"^mlp_norm\.", "ffn_norm.", rest)
            if re.match(r"attn\.[qkv]_conv1d\.weight$", rest):
                v = _conv(v)
            if rest.split(".")[-1].startswith("_"):
                continue                                                    # derived caches of the NVFP4 modules
            out[f"layers.{i}.{rest}"] = v
            continue
        m = re.match(rf"replicated_per_device\.{d}\.(.*)", k)
        if m:
            out[m.group(1)] = v
    return out


def convert_reference_state_dict(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """A state dict in this framework's plain layout from either layout of the reference (a native one is returned
    unchanged). The result loads into ``HippoModel`` built with ``full_attn_interval=0`` (every layer KDA) and the
    reference's dimensions."""
    layout = detect_layout(sd)
    if layout == "reference_single":
        return _from_single(sd)
    if layout == "reference_tp":
        return _from_tp(sd)
    return dict(sd)


def convert_checkpoint_file(src: str, dst: str) -> Dict[str, object]:
    """Reads a checkpoint file of the reference (or a bare state dict), converts the model weights and writes
    ``{"step", "model_state_dict", "loss"}``; optimizer state is not carried over (its layout is per device there)."""
    ck = torch.load(src, map_location="cpu", weights_only=False)
    sd = ck.get("model_state_dict", ck) if isinstance(ck, dict) else ck
    layout = detect_layout(sd)
    out = {"step": int(ck.get("step", 0)) if isinstance(ck, dict) else 0,
           "model_state_dict": convert_reference_state_dict(sd),
           "loss": ck.get("loss") if isinstance(ck, dict) else None, "converted_from": layout}
    torch.save(out, dst)
    return {"layout": layout, "tensors": len(out["model_state_dict"]), "step": out["step"]}
