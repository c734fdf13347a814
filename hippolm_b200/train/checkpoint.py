"""Checkpoint save / load / prune / resume.

Payload and file name follow the reference (``src/training/checkpoint.py:34-168``):
``checkpoint_step_{N}.pt`` holding ``{step, model_state_dict, optimizer_state_dict:{muon,adamw},
loss, scaler_state_dict}``. The reference saves rank 0 only, which cannot restore a TP>1 run;
here rank 0 writes the canonical file (complete at TP=1) and, at TP>1 or DP>1, every rank also
writes ``checkpoint_step_{N}.rank{r}.pt`` with its own shard plus the CPU and CUDA RNG states and the data
position. Rank 0 writes a small manifest LAST, after a barrier: a step whose manifest is missing, or whose
manifest lists a shard that is not on disk, is incomplete and is never picked by ``find_latest_checkpoint``.
Loading at world > 1 refuses a missing shard and a manifest written by another world / tp / dp layout
(shards of different ranks have identical shapes, so a wrong file would load without an error).
"""
from __future__ import annotations

import glob
import json
import os
import re
from typing import Dict, Optional, Tuple

import torch

_PAT = re.compile(r"checkpoint_step_(\d+)\.pt$")


def checkpoint_path(ckpt_dir: str, step: int, rank: Optional[int] = None) -> str:
    suffix = f".rank{rank}" if rank is not None else ""
    return os.path.join(ckpt_dir, f"checkpoint_step_{step}{suffix}.pt")


def _payload(model, muon, adamw, step, loss, scaler=None, extra=None) -> Dict:
    p = {"step": int(step),
         "model_state_dict": {k: v.detach().cpu() for k, v in model.state_dict().items()},
         "optimizer_state_dict": {"muon": muon.state_dict() if muon is not None else None,
                                  "adamw": adamw.state_dict() if adamw is not None else None},
         "loss": float(loss) if loss is not None else None,
         "scaler_state_dict": scaler.state_dict() if scaler is not None else None}
    if extra:
        p.update(extra)
    return p


def _atomic_save(obj, path: str) -> None:
    tmp = path + ".tmp"
    torch.save(obj, tmp)
    os.replace(tmp, path)


def save_checkpoint(model, muon, adamw, step: int, loss, path: str, scaler=None,
                    rank: int = 0, world_size: int = 1, mesh=None, extra: Optional[Dict] = None) -> str:
    """``path`` is the canonical file. With world_size > 1 each rank also writes its shard file."""
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    extra = dict(extra or {})
    extra.setdefault("rng_state", torch.get_rng_state())
    if torch.cuda.is_available() and torch.cuda.is_initialized():
        extra.setdefault("cuda_rng_state", torch.cuda.get_rng_state())
    extra.setdefault("data_step", int(step) + 1)          # batches consumed so far: the loader resumes from here
    err: Optional[BaseException] = None
    try:
        if world_size > 1:
            _atomic_save(_payload(model, muon, adamw, step, loss, scaler, extra), path[:-3] + f".rank{rank}.pt")
        if rank == 0:
            _atomic_save(_payload(model, muon, adamw, step, loss, scaler, extra), path)
    except Exception as ex:                       # reported after the collective below, so that no rank is left waiting
        err = ex
    if world_size > 1:
        import torch.distributed as dist
        oks = [err is None]
        if dist.is_available() and dist.is_initialized():
            oks = [None] * dist.get_world_size()
            dist.all_gather_object(oks, err is None)  # also the barrier: every shard is on disk before the manifest appears
        if rank == 0 and all(oks):
            man = {"step": int(step), "world_size": world_size,
                   "tp": getattr(mesh, "tp", 1), "dp": getattr(mesh, "dp", 1),
                   "shards": [os.path.basename(path[:-3] + f".rank{r}.pt") for r in range(world_size)]}
            tmp = path[:-3] + ".manifest.json.tmp"
            with open(tmp, "w") as f:
                json.dump(man, f)
            os.replace(tmp, path[:-3] + ".manifest.json")
        if err is None and not all(oks):
            err = RuntimeError(f"checkpoint step {step}: the shard of rank(s) {[r for r, o in enumerate(oks) if not o]} failed")
    if err is not None:
        raise err
    return path


def read_manifest(path: str) -> Optional[Dict]:
    try:
        with open(path[:-3] + ".manifest.json") as f:
            return json.load(f)
    except (FileNotFoundError, json.JSONDecodeError):
        return None


def is_complete(path: str) -> bool:
    """A single-process checkpoint is its canonical file; a multi-rank one also needs its manifest and every shard."""
    if not os.path.exists(path):
        return False
    man = read_manifest(path)
    if man is None:
        return not glob.glob(path[:-3] + ".rank*.pt")       # shards without a manifest: the save was interrupted
    d = os.path.dirname(path)
    return all(os.path.exists(os.path.join(d, s)) for s in man.get("shards", []))


def load_checkpoint(path: str, model, muon=None, adamw=None, scaler=None, rank: int = 0,
                    world_size: int = 1, map_location="cpu", strict: bool = True, mesh=None,
                    info: Optional[Dict] = None) -> Tuple[int, Optional[float]]:
    """Restore model + optimizers; returns ``(step, loss)``. At world_size > 1 this rank's shard file is required, and the
    manifest must describe the same world / tp / dp layout (``mesh`` given)."""
    use = path
    if world_size > 1:
        use = path[:-3] + f".rank{rank}.pt"
        man = read_manifest(path)
        if man is None:
            raise FileNotFoundError(f"{path}: no manifest; a multi-rank resume needs the per-rank shards and their manifest")
        want = {"world_size": world_size}
        if mesh is not None:
            want.update(tp=mesh.tp, dp=mesh.dp)
        bad = {k: (man.get(k), v) for k, v in want.items() if man.get(k) != v}
        if bad:
            raise ValueError(f"{path}: written by another layout (manifest vs this run): {bad}")
        if not os.path.exists(use):
            raise FileNotFoundError(f"{use}: the shard of rank {rank} is missing")
    ck = torch.load(use, map_location=map_location, weights_only=False)
    model.load_state_dict(ck["model_state_dict"], strict=strict)
    osd = ck.get("optimizer_state_dict") or {}
    if muon is not None and osd.get("muon") is not None:
        muon.load_state_dict(osd["muon"])
    if adamw is not None and osd.get("adamw") is not None:
        adamw.load_state_dict(osd["adamw"])
    if scaler is not None and ck.get("scaler_state_dict") is not None:
        scaler.load_state_dict(ck["scaler_state_dict"])
    if ck.get("rng_state") is not None:
        torch.set_rng_state(ck["rng_state"].cpu())
    if ck.get("cuda_rng_state") is not None and torch.cuda.is_available():
        torch.cuda.set_rng_state(ck["cuda_rng_state"].cpu())
    if info is not None:
        info["data_step"] = int(ck.get("data_step", int(ck["step"]) + 1))
    return int(ck["step"]), ck.get("loss")


def list_checkpoints(ckpt_dir: str):
    out = []
    for p in glob.glob(os.path.join(ckpt_dir, "checkpoint_step_*.pt")):
        m = _PAT.search(os.path.basename(p))
        if m:
            out.append((int(m.group(1)), p))
    return sorted(out)


def find_latest_checkpoint(ckpt_dir: str) -> Optional[str]:
    """Newest step that is complete on disk (see :func:`is_complete`)."""
    for _, p in reversed(list_checkpoints(ckpt_dir)):
        if is_complete(p):
            return p
    return None


def prune_old_checkpoints(ckpt_dir: str, keep_last_n: int) -> int:
    """Keep the newest ``keep_last_n`` by step number (``checkpoint.py:89-131``); 0/None keeps all."""
    if not keep_last_n or keep_last_n <= 0:
        return 0
    c = list_checkpoints(ckpt_dir)
    removed = 0
    for step, p in c[:-keep_last_n]:
        for f in [p, p[:-3] + ".manifest.json"] + glob.glob(p[:-3] + ".rank*.pt"):
            try:
                os.remove(f); removed += 1
            except FileNotFoundError:
                pass
    return removed


def is_sharded_state_dict(sd: Dict) -> bool:
    """Plain (TP=1) layout has ``layers.N...`` keys; anything else is treated as foreign
    (the reference's loader sniffs ``layers_per_device.`` prefixes, ``scripts/eval_server.py:94-107``)."""
    return any(k.startswith("layers_per_device.") or k.startswith("replicated_per_device.") for k in sd)
