"""VRAM tooling (``tools/vram_profile/*.py``): memory-history snapshots, their analysis by allocation site and by component
class, peak memory per phase of the training step, a polling thread on ``torch.cuda.mem_get_info``, a saved-tensor size
probe and its per-module attribution."""
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


# (class, substrings of "filename name" of a stack frame): the first rule that matches any frame of a block, innermost
# frame first, names the block's class. Order: the most specific producers first.
_CLASS_RULES = (
    ("checkpoint.input", ("torch/utils/checkpoint.py",)),
    ("optimizer.state", ("optim/optimizers.py", "optim/offload.py")),
    ("comm.workspace", ("parallel/symm.py", "parallel/fused.py", "parallel/dp.py")),
    ("lce_head", ("_VocabParallelLCE", "LMHeadLoss", "lce_")),
    ("kda.saved", ("ops/kda_cuda.py", "ref/kda.py", "KDAAttention")),
    ("attention.saved", ("ops/attn_cuda.py", "FullAttention", "rope")),
    ("attn_res.saved", ("attn_res", "BlockAttnRes")),
    ("norm.saved", ("rmsnorm", "RMSNorm", "gated_norm", "l2norm")),
    ("ffn", ("nvfp4", "SwiGLU", "swiglu", "fp4_gemm")),
    ("embedding", ("embed_cuda.py", "VocabParallelEmbedding", "embedding")),
    ("model.weight", ("__init__", "reset_parameters", "load_state_dict", "_load_from_state_dict", "convert.py", "reshard.py")),
    ("data", ("hippolm_b200/data/",)),
    ("linear", ("parallel/linear.py", "cuda_ops.py gemm", "matmul", "linear")),
)


def classify_block(frames) -> str:
    """Component class of one allocation from its stack (``tools/vram_profile/classify.py`` in the reference, with this
    package's producers): see ``_CLASS_RULES``; ``other`` when nothing matches, ``<no stack>`` without frames."""
    if not frames:
        return "<no stack>"
    texts = [f"{fr.get('filename', '')} {fr.get('name', '')}" for fr in frames]
    for cls, keys in _CLASS_RULES:
        for t in texts:
            if any(k in t for k in keys):
                return cls
    return "other"


def classify_snapshot(snapshot) -> List[Dict]:
    """Live allocations of an allocator snapshot (dict or pickle path) summed per component class, largest first:
    ``{"class", "bytes", "blocks", "largest": "file:line name" of the biggest block}``."""
    if isinstance(snapshot, (str, bytes)):
        import pickle
        with open(snapshot, "rb") as f:
            snapshot = pickle.load(f)
    groups: Dict[str, list] = {}
    for seg in snapshot.get("segments", []):
        for blk in seg.get("blocks", []):
            if blk.get("state") != "active_allocated":
                continue
            frames = blk.get("frames") or []
            g = groups.setdefault(classify_block(frames), [0, 0, 0, ""])
            size = int(blk.get("size", 0))
            g[0] += size; g[1] += 1
            if size > g[2]:
                fr = next((f for f in frames if "hippolm_b200" in f.get("filename", "")), frames[0] if frames else None)
                g[2], g[3] = size, (f"{fr['filename']}:{fr.get('line', 0)} {fr.get('name', '')}" if fr else "")
    out = [{"class": k, "bytes": v[0], "blocks": v[1], "largest": v[3]} for k, v in groups.items()]
    out.sort(key=lambda r: -r["bytes"])
    return out


class PhaseMemory:
    """Peak device memory per phase of the training step (the per-phase log of ``tools/vram_profile/profile.py`` in the
    reference). ``begin()`` at the start of a phase resets the allocator's peak counter; ``record(name, step)`` at its end
    notes the peak reached inside the phase, what is still allocated and reserved, and the memory in use on the device as
    the driver sees it. ``readers``: ``{"allocated", "reserved", "peak", "reset_peak", "driver_used"}`` callables (bytes);
    default: the ``torch.cuda`` counters of ``device``, zeros without a GPU."""

    def __init__(self, device=None, readers: Optional[Dict] = None):
        if readers is None:
            if device is not None and torch.device(device).type == "cuda":
                d = torch.device(device)
                readers = {"allocated": lambda: torch.cuda.memory_allocated(d), "reserved": lambda: torch.cuda.memory_reserved(d),
                           "peak": lambda: torch.cuda.max_memory_allocated(d),
                           "reset_peak": lambda: torch.cuda.reset_peak_memory_stats(d),
                           "driver_used": lambda: (lambda fr_to: fr_to[1] - fr_to[0])(torch.cuda.mem_get_info(d))}
            else:
                zero = lambda: 0                                            # noqa: E731
                readers = {"allocated": zero, "reserved": zero, "peak": zero, "reset_peak": zero, "driver_used": zero}
        self.r = readers
        self.rows: List[Dict] = []
        self.run_peak = 0                      # the peak counter is reset per phase: the run's own maximum is kept here

    def begin(self) -> None:
        self.run_peak = max(self.run_peak, int(self.r["peak"]()))
        self.r["reset_peak"]()

    def record(self, name: str, step: int = 0) -> Dict:
        peak = int(self.r["peak"]())
        self.run_peak = max(self.run_peak, peak)
        row = {"step": step, "phase": name, "peak": peak, "allocated": int(self.r["allocated"]()),
               "reserved": int(self.r["reserved"]()), "driver_used": int(self.r["driver_used"]())}
        self.rows.append(row)
        return row

    def step_summary(self, step: int) -> Dict[str, float]:
        """Phase -> peak MiB inside the phase (maximum over its occurrences in ``step``)."""
        out: Dict[str, float] = {}
        for r in self.rows:
            if r["step"] == step:
                out[r["phase"]] = max(out.get(r["phase"], 0.0), round(r["peak"] / 2 ** 20, 1))
        return out

    def table(self) -> List[Dict]:
        """Per phase over all recorded steps: the largest peak, and allocated / reserved / driver-level use at the end of
        the occurrence that had it (MiB), in order of first appearance."""
        best: Dict[str, Dict] = {}
        for r in self.rows:
            if r["phase"] not in best or r["peak"] > best[r["phase"]]["peak"]:
                best[r["phase"]] = r
        mib = lambda v: round(v / 2 ** 20, 1)                               # noqa: E731
        return [{"phase": k, "step": r["step"], "peak_mib": mib(r["peak"]), "allocated_mib": mib(r["allocated"]),
                 "reserved_mib": mib(r["reserved"]), "driver_used_mib": mib(r["driver_used"])} for k, r in best.items()]


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
    ``classify <snapshot.pickle>``: the same allocations summed per component class (weights, optimizer state, KDA /
    attention / norm saves, loss head, communication workspace, ...). ``profile --config X.yml [--steps 2] [--out DIR]``:
    runs training steps of the configuration on synthetic data and prints the peak memory of every phase of the step
    (h2d, fwd_bwd, grad_sync, gradnorm, muon, adamw, zero), the maximum a 100 Hz poll of the device saw, and dumps the
    allocator history of the run to ``DIR/vram_snapshot.pickle`` for ``analyze`` / ``classify`` / pytorch.org/memory_viz.
    (``tools/vram_profile/{analyze,classify,saved_tensor_probe,profile,poll_prod}.py`` of the reference.)"""
    import argparse
    import json
    ap = argparse.ArgumentParser(prog="python -m hippolm_b200.utils.vram")
    sub = ap.add_subparsers(dest="cmd", required=True)
    a1 = sub.add_parser("analyze"); a1.add_argument("snapshot"); a1.add_argument("--top", type=int, default=20)
    a2 = sub.add_parser("probe"); a2.add_argument("--config", required=True); a2.add_argument("--depth", type=int, default=2)
    a2.add_argument("--tokens", type=int, default=0); a2.add_argument("--snapshot", default=None)
    a3 = sub.add_parser("classify"); a3.add_argument("snapshot")
    a4 = sub.add_parser("profile"); a4.add_argument("--config", required=True); a4.add_argument("--steps", type=int, default=2)
    a4.add_argument("--out", default="output/vram_profile"); a4.add_argument("--poll_hz", type=float, default=100.0)
    a4.add_argument("overrides", nargs="*", help="further training flags, e.g. --micro_batch_size 8192 (after --)")
    a = ap.parse_args(argv)
    if a.cmd == "analyze":
        for r in analyze_snapshot(a.snapshot, a.top):
            print(f"{r['bytes'] / 2 ** 20:10.1f} MiB  {r['blocks']:6d} blocks  {r['where']}")
        return 0
    if a.cmd == "classify":
        for r in classify_snapshot(a.snapshot):
            print(f"{r['bytes'] / 2 ** 20:10.1f} MiB  {r['blocks']:6d} blocks  {r['class']:18s} largest: {r['largest']}")
        return 0
    if a.cmd == "profile":
        return _profile(a)
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


def _profile(a) -> int:
    import json
    import os
    from ..cli import parse_args
    from ..train.loop import run_training_loop, setup_worker
    os.makedirs(os.path.join(a.out, "logs"), exist_ok=True)
    args = parse_args(["--config", a.config, "--max_steps", str(a.steps), "--mb_timing", "-1", "--vram_phases", "true",
                       "--checkpoint_interval", "0", "--use_dummy_data", "true", "--output_dir", a.out] + list(a.overrides))
    cuda = torch.cuda.is_available()
    poller = VramPoller(0, 1.0 / max(a.poll_hz, 1.0)).start() if cuda else None
    snap = os.path.join(a.out, "vram_snapshot.pickle")
    with memory_history(snap):
        ctx = setup_worker(args, run_dir=a.out)
        run_training_loop(ctx)
    polled = poller.stop() if poller else None
    mem = ctx.extras.get("phase_memory")
    rows = mem.table() if mem is not None else []
    for r in rows:
        print(f"{r['phase']:10s} peak {r['peak_mib']:10.1f} MiB (step {r['step']})  then allocated {r['allocated_mib']:10.1f}  "
              f"reserved {r['reserved_mib']:10.1f}  device in use {r['driver_used_mib']:10.1f}")
    res = {"phases": rows, "run_peak_mib": round(mem.run_peak / 2 ** 20, 1) if mem is not None else None, "polled": polled,
           "snapshot": snap if cuda else None, "steps": a.steps}
    with open(os.path.join(a.out, "vram_profile.json"), "w") as f:
        json.dump(res, f, indent=1)
    print(json.dumps({k: res[k] for k in ("run_peak_mib", "polled", "snapshot")}))
    return 0


if __name__ == "__main__":
    raise SystemExit(_main())
