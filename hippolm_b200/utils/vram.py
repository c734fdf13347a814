"""VRAM tooling (``tools/vram_profile/*.py``): memory-history snapshots and their analysis by allocation site, a
polling thread on ``torch.cuda.mem_get_info``, a saved-tensor size probe and its per-module attribution."""
from __future__ import annotations

import contextlib
import threading
import time
from typing import Dict, List, Optional

import torch


@contextlib.contextmanager
def memory_history(snapshot_path: Optional[str] = None, max_entries: int = 100000):
    """Records allocator history for the block and optionally dumps a snapshot file for pytorch.org/memory_viz."""
    on = torch.cuda.is_available()
    if on:
        torch.cuda.memory._record_memory_history(max_entries=max_entries)
    try:
        yield
    finally:
        if on:
            if snapshot_path:
                torch.cuda.memory._dump_snapshot(snapshot_path)
            torch.cuda.memory._record_memory_history(enabled=None)


class VramPoller:
    """Samples used device memory every ``period_s`` (100 Hz by default) on a daemon thread."""

    def __init__(self, device: int = 0, period_s: float = 0.01):
        self.device, self.period_s = device, period_s
        self.samples: List[float] = []
        self._stop = threading.Event()
        self._t: Optional[threading.Thread] = None

    def start(self):
        def run():
            while not self._stop.wait(self.period_s):
                free, total = torch.cuda.mem_get_info(self.device)
                self.samples.append((total - free) / 2 ** 20)
        self._t = threading.Thread(target=run, name="vram-poller", daemon=True)
        self._t.start()
        return self

    def stop(self) -> Dict[str, float]:
        self._stop.set()
        if self._t:
            self._t.join(timeout=1.0)
        s = self.samples or [0.0]
        return {"peak_mb": max(s), "mean_mb": sum(s) / len(s), "samples": len(s)}


class SavedTensorProbe:
    """Sums the bytes autograd saves for backward inside the block (``saved_tensors_hooks``)."""

    def __init__(self):
        self.bytes = 0
        self.count = 0
        self._seen = set()

    def __enter__(self):
        def pack(t):
            key = (t.data_ptr(), t.numel())
            if key not in self._seen:
                self._seen.add(key)
                self.bytes += t.numel() * t.element_size(); self.count += 1
            return t
        self._ctx = torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t)
        self._ctx.__enter__()
        return self

    def __exit__(self, *a):
        return self._ctx.__exit__(*a)


def vram_line(device) -> str:
    if not torch.cuda.is_available():
        return "vram n/a"
    return (f"vram alloc {torch.cuda.memory_allocated(device) / 2**20:.0f} MiB reserved "
            f"{torch.cuda.memory_reserved(device) / 2**20:.0f} MiB max {torch.cuda.max_memory_allocated(device) / 2**20:.0f} MiB")


def analyze_snapshot(snapshot, top: int = 20, package_hint: str = "hippolm_b200") -> List[Dict]:
    """Live allocations of an allocator snapshot grouped by the code that made them
    (``tools/vram_profile/analyze_snapshot.py`` in the reference).

    ``snapshot``: the dict from ``torch.cuda.memory._snapshot()`` or the path of a pickle written by
    ``torch.cuda.memory._dump_snapshot``. Every active block is attributed to the innermost frame of its stack that
    lies inside ``package_hint`` (else the innermost Python frame). Returns the ``top`` groups, largest first:
    ``{"where": "file:line name", "bytes": .., "blocks": ..}``."""
    if isinstance(snapshot, (str, bytes)):
        import pickle
        with open(snapshot, "rb") as f:
            snapshot = pickle.load(f)
    groups: Dict[str, List[int]] = {}
    for seg in snapshot.get("segments", []):
        for blk in seg.get("blocks", []):
            if blk.get("state") != "active_allocated":
                continue
            frames = blk.get("frames") or []
            pick = None
            for fr in frames:
                fn = fr.get("filename", "")
                if package_hint in fn:
                    pick = fr
                    break
            if pick is None:
                pick = next((fr for fr in frames if fr.get("filename", "").endswith(".py")), None)
            where = f"{pick['filename']}:{pick.get('line', 0)} {pick.get('name', '')}" if pick else "<no stack>"
            g = groups.setdefault(where, [0, 0])
            g[0] += int(blk.get("size", 0)); g[1] += 1
    out = [{"where": k, "bytes": v[0], "blocks": v[1]} for k, v in groups.items()]
    out.sort(key=lambda r: -r["bytes"])
    return out[:top]


def saved_bytes_by_module(model: torch.nn.Module, run, depth: int = 2) -> List[Dict]:
    """Bytes autograd keeps for backward, attributed to the sub-module whose forward saved them (module paths cut at
    ``depth`` components). ``run()`` performs one forward pass of ``model``. Tells which layer type sets the activation
    memory of a micro-batch (``tools/vram_profile/saved_tensor_probe.py`` in the reference)."""
    stack: List[str] = []
    totals: Dict[str, List[int]] = {}
    seen = set()
    handles = []

    def pre(name):
        def hook(mod, args):
            stack.append(name)
        return hook

    def post(name):
        def hook(mod, args, out):
            if stack and stack[-1] == name:
                stack.pop()
        return hook

    for name, mod in model.named_modules():
        if not name:
            continue
        short = ".".join(name.split(".")[:depth])
        handles.append(mod.register_forward_pre_hook(pre(short)))
        handles.append(mod.register_forward_hook(post(short)))

    def pack(t):
        key = (t.data_ptr(), t.numel())
        if key not in seen:
            seen.add(key)
            g = totals.setdefault(stack[-1] if stack else "<top>", [0, 0])
            g[0] += t.numel() * t.element_size(); g[1] += 1
        return t

    try:
        with torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t):
            run()
    finally:
        for h in handles:
            h.remove()
    out = [{"module": k, "bytes": v[0], "tensors": v[1]} for k, v in totals.items()]
    out.sort(key=lambda r: -r["bytes"])
    return out


def _main(argv=None) -> int:
    """``python -m hippolm_b200.utils.vram analyze <snapshot.pickle> [--top N]``: live allocations of a memory snapshot by
    allocation site. ``python -m hippolm_b200.utils.vram probe --config X.yml [--depth 2] [--tokens N]``: bytes autograd
    keeps for backward per sub-module, for one forward pass of the configured model on synthetic tokens (GPU when one is
    visible, else CPU); with ``--snapshot out.pickle`` the allocator history of that pass is dumped as well.
    (``tools/vram_profile/{analyze,saved_tensor_probe,profile}.py`` of the reference.)"""
    import argparse
    import json
    ap = argparse.ArgumentParser(prog="python -m hippolm_b200.utils.vram")
    sub = ap.add_subparsers(dest="cmd", required=True)
    a1 = sub.add_parser("analyze"); a1.add_argument("snapshot"); a1.add_argument("--top", type=int, default=20)
    a2 = sub.add_parser("probe"); a2.add_argument("--config", required=True); a2.add_argument("--depth", type=int, default=2)
    a2.add_argument("--tokens", type=int, default=0); a2.add_argument("--snapshot", default=None)
    a = ap.parse_args(argv)
    if a.cmd == "analyze":
        for r in analyze_snapshot(a.snapshot, a.top):
            print(f"{r['bytes'] / 2 ** 20:10.1f} MiB  {r['blocks']:6d} blocks  {r['where']}")
        return 0
    from ..cli import parse_args
    from ..config import HippoConfig
    from ..models.model import HippoModel
    args = parse_args(["--config", a.config])
    cfg = HippoConfig.from_namespace(args)
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    model = HippoModel(cfg, device=dev, dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32)
    T = a.tokens or min(int(args.seq_len), 4096)
    ids = torch.randint(0, cfg.vocab_size, (T,), device=dev)

    def run():
        model(ids, labels=ids)["loss"]

    with memory_history(a.snapshot):
        rows = saved_bytes_by_module(model, run, depth=a.depth)
    total = sum(r["bytes"] for r in rows)
    for r in rows:
        print(f"{r['bytes'] / 2 ** 20:10.2f} MiB  {r['tensors']:5d} tensors  {r['module']}")
    print(json.dumps({"tokens": T, "saved_mib": round(total / 2 ** 20, 2), "bytes_per_token": round(total / T, 1),
                      "device": str(dev)}))
    return 0


if __name__ == "__main__":
    raise SystemExit(_main())
