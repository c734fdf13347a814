"""Reference arm of ``bench.py``: runs the UNMODIFIED reference tree (a plain copy under ``baseline/_ref``) through its
own stock code path and prints the same JSON line as the framework's arm, with ``"impl": "reference"``.

The reference is a script tree, not an installable package (it has neither ``setup.py`` nor ``pyproject.toml``), so its
"install" is ``cp -r <reference> baseline/_ref`` and it is imported by path. Nothing of ``hippolm_b200`` is imported here.

Training arm.  Each rank calls the reference's own per-rank entry points -- ``_setup_worker`` and ``_run_training_loop``
(``src/training/loop/setup.py:62``, ``src/training/loop/run.py:57``; ``_train_worker`` in ``worker.py:23`` is exactly
these two calls) -- with ``use_dummy_data`` and the closest configuration the reference can express to the benchmarked
one.  The only thing placed between the two calls is a pass-through wrapper around the dummy ``DataLoader`` that takes
time stamps at step boundaries (the loop fetches one batch per step), so the timed region contains, per step, the
host-to-device copy of the batch, every micro-batch forward/backward with the D2H gradient stream, the host optimizer,
and the per-chunk ``loss.item()`` read-back: device-timed and end-to-end values coincide for this arm.

What the reference cannot express (listed under ``config.differences`` in the output): full-attention layers and RoPE
(all layers are KDA), sequence parallelism (activations are replicated and all-reduced), untied embeddings, FP4 tensor
cores (its Marlin W4A16 binary is sm_120-only, so on sm_100 the NVFP4 FFN runs as dequantise + cuBLAS with a bf16 master),
a device-resident optimizer (optimizer state and the gradient accumulator live in pinned host memory by design).

Kernel arm.  ``kda_times`` measures the reference's vendored ``chunk_kda`` (``fla/ops/kda/chunk.py:220``) forward and
forward+backward on the standalone-KDA configuration (B=4, T=8192, H=16, K=V=128, 8 documents, bf16) with CUDA events,
warm-up and an L2 flush between iterations.
"""
from __future__ import annotations

import json
import math
import os
import statistics
import sys
import time
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")

MODELS = {
    # all-KDA version of the benchmarked 7B hybrid (the reference has no attention layer)
    "7b": dict(vocab_size=128256, hidden_size=4096, num_heads=32, head_dim=128, num_layers=32, num_blocks=8,
               intermediate_size=14336),
    "1p3b": dict(vocab_size=128256, hidden_size=2048, num_heads=16, head_dim=128, num_layers=24, num_blocks=6,
                 intermediate_size=5632),
    "tiny": dict(vocab_size=8192, hidden_size=512, num_heads=4, head_dim=128, num_layers=4, num_blocks=2,
                 intermediate_size=1024),
}


def _unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
    return 0


def _prepare_imports():
    if not os.path.isdir(os.path.join(REF, "src")):
        raise FileNotFoundError("baseline/_ref is missing: copy the reference tree there (cp -r <reference> baseline/_ref)")
    # the reference's own ``scripts`` and ``src`` packages must win over same-named packages of this repository
    sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") != os.path.dirname(HERE)]
    sys.path.insert(0, REF)
    for m in [m for m in sys.modules if m == "scripts" or m.startswith("scripts.")]:
        del sys.modules[m]


class _TimedLoader:
    """Pass-through iterable over the reference's dummy DataLoader; fetch number ``i`` marks the start of step ``i``."""

    def __init__(self, inner, warmup, steps, args, budget_s, sampler_factory, t_start):
        self.inner, self.W, self.K = inner, warmup, steps
        self.args, self.budget_s, self.t_start = args, budget_s, t_start
        self.sampler_factory = sampler_factory
        self.sampler = None
        self.result = None
        self.h2d = 0

    def _sync(self):
        import torch
        import torch.distributed as dist
        torch.cuda.synchronize()
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def __iter__(self):
        import torch
        import torch.distributed as dist
        e0 = e1 = None
        t0 = None
        t_prev = None
        for i, batch in enumerate(self.inner):
            if 3 <= i < self.W and t_prev is not None:
                # slow steps: start the timed region early rather than spend the whole budget on warm-up (at least three
                # warm-up steps always run: the first one contains the Triton compilation)
                torch.cuda.synchronize()
                per = time.perf_counter() - t_prev
                spent = time.perf_counter() - self.t_start
                cut = torch.tensor([1 if spent + per * (self.W - i + 3) > self.budget_s else 0], device="cuda")
                if dist.is_initialized() and dist.get_world_size() > 1:
                    dist.all_reduce(cut, op=dist.ReduceOp.MAX)
                if int(cut.item()):
                    self.W = i
                    self.args.max_steps = self.W + self.K
            t_prev = time.perf_counter()
            if i == self.W:
                self.h2d = sum(v.numel() * v.element_size() for v in batch.values() if hasattr(v, "numel"))
                self._sync()
                self.sampler = self.sampler_factory()
                if self.sampler is not None:
                    self.sampler.start()
                e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
                t0 = time.perf_counter()
                e0.record()
            elif i == self.W + 1:
                # one timed step has run: shrink the number of timed steps if K of them would not fit in the time budget
                torch.cuda.synchronize()
                per = time.perf_counter() - t0
                left = self.budget_s - (time.perf_counter() - self.t_start) - 30.0
                k_fit = max(1, min(self.K, 1 + int(max(left, 0.0) // max(per, 1e-3))))
                kt = torch.tensor([k_fit], device="cuda", dtype=torch.int64)
                if dist.is_initialized() and dist.get_world_size() > 1:
                    dist.all_reduce(kt, op=dist.ReduceOp.MIN)
                self.K = int(kt.item())
                self.args.max_steps = self.W + self.K
            if i == self.W + self.K and e0 is not None:
                e1.record()
                self._sync()
                wall_ms = (time.perf_counter() - t0) * 1e3
                dev_ms = e0.elapsed_time(e1)
                t = torch.tensor([dev_ms, wall_ms], device="cuda", dtype=torch.float64)
                if dist.is_initialized() and dist.get_world_size() > 1:
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                clocks = self.sampler.stop() if self.sampler is not None else None
                self.result = {"dev_ms": float(t[0]), "wall_ms": float(t[1]), "steps": self.K, "clocks": clocks}
            yield batch


def run_train(a) -> int:
    t_start = time.perf_counter()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    try:
        _prepare_imports()
        import torch
        if not torch.cuda.is_available():
            return _unavailable("no CUDA device in this process (the reference's worker needs one)") if rank == 0 else 0
        import yaml
        from scripts.cli import parse_args as ref_parse_args
        from src.training.env import configure_runtime_environment
        configure_runtime_environment()
        from src.training.loop.setup import _setup_worker
        from src.training.loop.run import _run_training_loop
    except Exception as e:                                            # noqa: BLE001
        return _unavailable(f"import of the reference tree failed: {type(e).__name__}: {e}") if rank == 0 else 0

    m = MODELS[a.model]
    seq = 8192 if a.model != "tiny" else 1024
    mb_tokens = a.micro_batch_tokens if a.micro_batch_tokens > 0 else seq * world
    total_tokens = a.seqs_per_gpu * world * seq            # the reference's "seq_len" is all tokens of one step
    run_dir = os.path.join("/tmp", f"hippo_ref_run_{os.getpid()}")
    os.makedirs(os.path.join(run_dir, "logs"), exist_ok=True)
    cfg = dict(m)
    cfg.update(dict(
        tie_word_embeddings=True, use_bias=False, expand_v=1.0, kda_mode="chunk", use_short_conv=False,
        allow_neg_eigval=False, safe_gate=True, lower_bound=-5.0, rms_norm_eps=1e-6,
        epochs=1, max_steps=a.warmup + a.steps, batch_size=1, seq_len=total_tokens, micro_batch_size=mb_tokens,
        lr_warmup_steps=200, lr_decay_steps=0, pack_chunk_size=64, pack_buffer_size=2048,
        optimizer={"adamw": {"lr": 0.004, "weight_decay": 0.01, "beta1": 0.9, "beta2": 0.95, "eps": 1e-8},
                   "muon": {"lr": 0.02, "weight_decay": 0.0, "momentum": 0.95}},
        max_grad_norm=1.0, seed=0,
        precision={k: {"dtype": "bf16"} for k in ("model_weights", "gradients", "activations", "muon_momentum",
                                                  "adamw_m", "adamw_v")},
        stage="pretrain", use_dummy_data=True, tp_size=world, tp_sim=False,
        ffn_nvfp4=(a.ref_ffn == "nvfp4"), ffn_nvfp4_marlin=False, ffn_nvfp4_no_bf16_master=False,
        empty_cache_between_mb=False,          # the reference's own measured-faster setting (docs/empty_cache_off.md)
        log_interval=1, checkpoint_interval=0, output_dir=run_dir, mb_timing=0,
    ))
    cfg_path = os.path.join(run_dir, "bench_config.yml")
    with open(cfg_path, "w") as f:
        yaml.safe_dump(cfg, f)
    args = ref_parse_args(["--config", cfg_path])

    def sampler_factory():
        if rank != 0:
            return None
        sys.path.append(os.path.join(os.path.dirname(HERE), "bench"))
        try:
            from clocks import ClockSampler
            return ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
        except Exception:                                             # noqa: BLE001
            return None

    # The reference rendezvous is env:// on a port of its own, with rank 0 hosting the store (what its mp.spawn launch
    # gives it). Under torch.distributed.run the launcher's agent already hosts a store on MASTER_PORT and every
    # worker is a client of it (TORCHELASTIC_USE_AGENT_STORE): hand the reference that port, a private one otherwise.
    port = int(os.environ.get("MASTER_PORT", "29500"))
    if os.environ.get("TORCHELASTIC_USE_AGENT_STORE") != "True":
        port += 37
    try:
        ctx = _setup_worker(rank, args, list(range(world)), port, run_dir, None)
        timed = _TimedLoader(ctx["dataloader"], a.warmup, a.steps, args, a.ref_budget_s, sampler_factory, t_start)
        ctx["dataloader"] = timed
        _run_training_loop(ctx)
    except Exception as e:                                            # noqa: BLE001
        tb = traceback.format_exc().strip().splitlines()
        where = next((l.strip() for l in reversed(tb) if l.strip().startswith("File")), "")
        return _unavailable(f"the reference's stock training path raised {type(e).__name__}: {str(e)[:300]} ({where})") \
            if rank == 0 else 0
    r = timed.result
    if r is None:
        return _unavailable("the reference loop ended before the timed region closed") if rank == 0 else 0
    if rank != 0:
        return 0
    import torch
    ms_step = r["dev_ms"] / r["steps"]
    e2e_ms = max(r["wall_ms"], r["dev_ms"]) / r["steps"]
    n_chunks = total_tokens // mb_tokens
    rec = {
        "impl": "reference", "metric": "train tokens/sec (device-timed, max over ranks)",
        "value": total_tokens / (ms_step / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": r["steps"],
        "steps_requested": a.steps, "warmup": timed.W, "warmup_requested": a.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" + (" (FFN weights NVFP4, dequantised to bf16 per call)" if a.ref_ffn == "nvfp4" else ""),
        "data": "synthetic uniform-random tokens (the reference's dummy_dataloader), random-init weights",
        "same_config": False,
        "config": {"model": f"reference all-KDA decoder at the {a.model} dimensions "
                            f"({m['num_layers']}L, d{m['hidden_size']}, {m['num_heads']}x{m['head_dim']}, "
                            f"ffn{m['intermediate_size']}, v{m['vocab_size']}, tied)",
                   "global_batch": a.seqs_per_gpu * world, "seq_len": seq, "parallelism": f"tp{world} (no SP)",
                   "micro_batch_tokens": mb_tokens, "optimizer": "muon+adamw, state and accumulator in pinned host memory",
                   "l2": "inputs larger than L2 (no explicit flush)",
                   "differences": ["all layers KDA (no full-attention layer, no RoPE)", "no sequence parallelism",
                                   "tied embeddings", "NVFP4 FFN as dequantise + cuBLAS with bf16 master "
                                   "(Marlin binary is sm_120 only)" if a.ref_ffn == "nvfp4" else "bf16 FFN",
                                   "host-resident optimizer state and gradient accumulator",
                                   "one packed stream per step (no cu_seqlens resets in KDA)"]},
        "clocks": r["clocks"],
        "e2e": {"value": total_tokens / (e2e_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": timed.h2d,
                "d2h_bytes_per_step": 8 * n_chunks, "ms_per_step": e2e_ms},
        "gpu_launches": None,
        "max_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1),
    }
    if a.kda and world == 1:
        try:
            rec.update(kda_times())
        except Exception as e:                                        # noqa: BLE001
            rec["kda_unavailable"] = f"{type(e).__name__}: {str(e)[:200]}"
    print(json.dumps(rec), flush=True)
    return 0


def kda_times(B=4, T=8192, H=16, D=128, docs=8, iters=10):
    """Forward and forward+backward time of the reference's ``chunk_kda`` at the standalone-KDA configuration."""
    _prepare_imports()
    import torch
    import torch.nn.functional as F
    from src.models.ops._vendored.fla.ops.kda.chunk import chunk_kda
    torch.manual_seed(0)
    dev = "cuda"
    TT = B * T
    q = F.normalize(torch.randn(1, TT, H, D, device=dev), dim=-1).bfloat16().requires_grad_(True)
    k = F.normalize(torch.randn(1, TT, H, D, device=dev), dim=-1).bfloat16().requires_grad_(True)
    v = torch.randn(1, TT, H, D, device=dev).bfloat16().requires_grad_(True)
    g = (-F.softplus(torch.randn(1, TT, H, D, device=dev))).requires_grad_(True)
    beta = torch.sigmoid(torch.randn(1, TT, H, device=dev)).requires_grad_(True)
    h0 = torch.zeros(docs, H, D, D, device=dev)
    cuts = torch.sort(torch.randperm(TT - 1)[:docs - 1] + 1).values
    cu = torch.cat([torch.zeros(1, dtype=torch.long), cuts, torch.tensor([TT])]).to(dev)
    do = torch.randn(1, TT, H, D, device=dev).bfloat16()
    flush = torch.empty(256 * 2 ** 20, dtype=torch.uint8, device=dev)
    kw = dict(scale=1.0 / math.sqrt(D), initial_state=h0, output_final_state=True, cu_seqlens=cu)

    def fwd():
        with torch.no_grad():
            chunk_kda(q=q, k=k, v=v, g=g, beta=beta, **kw)

    def fwd_bwd():
        for t in (q, k, v, g, beta):
            t.grad = None
        o, _ = chunk_kda(q=q, k=k, v=v, g=g, beta=beta, **kw)
        o.backward(do)

    def time_ms(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record(); e1.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)

    return {"kda_fwd_ms": round(time_ms(fwd), 3), "kda_fwd_bwd_ms": round(time_ms(fwd_bwd), 3),
            "kda_config": {"B": B, "T": T, "H": H, "K": D, "V": D, "docs": docs, "dtype": "bf16",
                           "l2": "flushed between iterations", "impl": "reference vendored FLA chunk_kda (Triton)"}}


def run_kda_only() -> int:
    try:
        rec = {"impl": "reference"}
        rec.update(kda_times())
        print(json.dumps(rec), flush=True)
    except Exception as e:                                            # noqa: BLE001
        return _unavailable(f"reference chunk_kda failed: {type(e).__name__}: {str(e)[:300]}")
    return 0
