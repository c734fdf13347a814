"""Worker setup, the training step and the training loop.

Mirrors the phases of the reference loop (``src/training/loop/setup.py:62-512``,
``run.py:57-583``, ``teardown.py:22-57``) with a device-resident gradient / optimizer path:

  batch (pinned host) -> H2D -> micro-batches { forward, loss * n_valid_i / n_valid_total, backward }
  -> DP gradient reduction -> TP replicated-gradient sync -> finite check -> global norm + clip
  -> WSD lr -> Muon.step -> AdamW.step -> zero grads -> log / checkpoint

Steps whose gradients contain inf/nan skip the update *and clear the gradients* (the reference
leaves poisoned accumulators behind, ``run.py:401-483``).
"""
from __future__ import annotations

import json
import logging
import math
import os
import time
from dataclasses import dataclass, field
from typing import Any, Dict, Iterator, List, Optional

import torch
import torch.distributed as dist

from ..config import HippoConfig, PrecisionConfig
from ..data.packing import slice_cu_seqlens
from ..models.model import HippoModel, shift_targets
from ..models.nvfp4_linear import repack_nvfp4_weights
from ..optim.optimizers import build_param_groups, global_grad_norm, clip_coefficient
from ..optim.schedule import wsd_lr
from ..parallel.mesh import Mesh, get_mesh, init_mesh, init_distributed_from_env
from ..utils.timing import PhaseTimer, nvtx_range
from . import checkpoint as ckpt
from .diagnostics import log_pre_step_diag, log_post_opt_diag

_DIAG_STEPS = 3


@dataclass
class TrainContext:
    args: Any
    cfg: HippoConfig
    mesh: Mesh
    device: torch.device
    model: HippoModel
    muon: Any
    adamw: Any
    precision: PrecisionConfig
    logger: logging.Logger
    data_iter: Optional[Iterator] = None
    run_dir: Optional[str] = None
    step: int = 0
    metrics_file: Optional[Any] = None
    grad_reducer: Optional[Any] = None
    liveness: Optional[Any] = None
    offloader: Optional[Any] = None
    prefetcher: Optional[Any] = None
    watchdog: Optional[Any] = None
    closed: bool = False
    extras: Dict[str, Any] = field(default_factory=dict)


def make_logger(rank: int, run_dir: Optional[str]) -> logging.Logger:
    lg = logging.getLogger(f"hippo.r{rank}")
    lg.setLevel(logging.INFO)
    lg.propagate = False
    if not lg.handlers:
        fmt = logging.Formatter("%(asctime)s [r%(rank)s] %(message)s".replace("%(rank)s", str(rank)))
        if rank == 0:
            sh = logging.StreamHandler(); sh.setFormatter(fmt); lg.addHandler(sh)
        if run_dir:
            os.makedirs(os.path.join(run_dir, "logs"), exist_ok=True)
            fh = logging.FileHandler(os.path.join(run_dir, "logs", f"rank{rank}.log"))
            fh.setFormatter(fmt); lg.addHandler(fh)
    return lg


def setup_worker(args, run_dir: Optional[str] = None, data_iter: Optional[Iterator] = None) -> TrainContext:
    """Rendezvous, mesh, model, optimizers, data. ``args`` is the CLI namespace."""
    device = init_distributed_from_env(timeout_s=float(getattr(args, "dist_timeout_s", 1800)))
    tp = int(getattr(args, "tp_size", 1) or 1)
    world = dist.get_world_size() if dist.is_initialized() else 1
    if world == 1:
        tp = 1
    dp = int(getattr(args, "dp_size", 0) or 0) or world // tp
    mesh = init_mesh(tp=tp, dp=dp, device=device)
    logger = make_logger(mesh.rank, run_dir)
    torch.manual_seed(int(getattr(args, "seed", 42)) + mesh.dp_rank)
    if device.type == "cuda":
        torch.set_float32_matmul_precision("high")
    cfg = HippoConfig.from_namespace(args)
    precision = PrecisionConfig.from_dict(getattr(args, "precision", None))
    wdtype = precision.model_weights if device.type == "cuda" or getattr(args, "force_precision", False) \
        else torch.float32
    model = HippoModel(cfg, device=device, dtype=wdtype, seed=int(getattr(args, "seed", 42)))
    if mesh.is_distributed:
        dist.barrier()
        from ..parallel.collectives import broadcast_replicated_params
        broadcast_replicated_params(model.replicated_parameters(), mesh)
    fused_on = False
    if mesh.tp > 1 and device.type == "cuda" and bool(getattr(args, "fused_comm", True)):
        # symmetric workspace for the fused all-gather->GEMM / GEMM->reduce-scatter kernels: the largest
        # gathered / staged tensor is [micro-batch tokens, hidden]
        from ..parallel import fused
        mbt = int(getattr(args, "micro_batch_size", 0) or 0)
        full = int(getattr(args, "batch_size", 1)) // max(1, dp) * int(getattr(args, "seq_len", 512))
        tokens = min(mbt, full) if mbt > 0 else full
        # bound of every device-side wait on a peer, in milliseconds of SM clock (0 = the kernels' default, ~2 s)
        wait_ms = float(getattr(args, "fused_wait_ms", 0) or 0)
        fused_on = (tokens // mesh.tp) % 128 == 0 and fused.setup(mesh, tokens, cfg.hidden_size,
                                                                  wait_cycles=int(wait_ms * 1.9e6))
    rx = getattr(args, "trainable_regex", None)
    if rx:
        # train only the parameters whose name matches (e.g. "ffn" for the feed-forward weights alone)
        import re
        for name, p in model.named_parameters():
            p.requires_grad_(bool(re.search(rx, name)))
    offload = bool(getattr(args, "offload_optimizer", False))
    muon, adamw = build_param_groups(model, args, precision, offload=offload)
    ctx = TrainContext(args=args, cfg=cfg, mesh=mesh, device=device, model=model, muon=muon, adamw=adamw,
                       precision=precision, logger=logger, data_iter=data_iter, run_dir=run_dir)
    ctx.extras["fused_comm"] = fused_on
    peer_timeout = float(getattr(args, "peer_timeout_s", 0) or 0)
    if peer_timeout > 0 and mesh.is_distributed:
        from .liveness import PeerLiveness, default_store
        store = default_store()
        if store is not None:
            ctx.liveness = PeerLiveness(store, mesh.rank, mesh.world_size, peer_timeout)
    if mesh.dp > 1:
        from ..parallel.dp import DPGradReducer
        # With the fused TP kernels active the DP all-reduces run after backward instead of beside it: an NCCL kernel
        # that shares the GPU with a persistent kernel spinning on its TP peers can keep part of that kernel's grid
        # from becoming resident, and the peers would wait for tiles that are never computed.
        # With gradient offload the hooks of the offloader free ``p.grad`` as soon as it is final, so there is nothing
        # to reduce during backward: the reduction then runs on the gradients uploaded by ``drain_to_device``.
        overlap = (bool(getattr(args, "dp_overlap", True)) and not fused_on
                   and not bool(getattr(args, "offload_grads", False)))
        # optional: reduce the Muon gradients to their owning replica only (needs the ownership split of the Muon work)
        owners = None
        if bool(getattr(args, "dp_reduce_to_owner", False)) and muon.dp_shard and (muon.ns_scope != "full" or mesh.tp == 1):
            owners = muon.dp_owner_map(mesh.dp)
        ctx.extras["owner_reduced"] = owners is not None
        ctx.grad_reducer = DPGradReducer(model, mesh, overlap=overlap, owners=owners)
    if bool(getattr(args, "offload_grads", False)):
        from ..optim.offload import GradOffloader
        ctx.offloader = GradOffloader(model, device)
    if mesh.rank == 0:
        n = model.num_parameters()
        logger.info(f"model: {n/1e6:.1f}M local parameters, tp={mesh.tp} dp={mesh.dp}, layers={cfg.layer_types()}")
        logger.info(f"optimizer: muon entries={len(muon.entries)} adamw entries={len(adamw.entries)} "
                    f"offload={offload} fused_comm={fused_on}")
        if run_dir:
            ctx.metrics_file = open(os.path.join(run_dir, "metrics.jsonl"), "a")
    init_from = getattr(args, "init_from", None)
    if init_from and not getattr(args, "resume", None):
        # Model weights from a plain single-file checkpoint (this framework's TP = 1 layout, shards merged by
        # train/reshard.py, or a checkpoint of the reference in either of its layouts): every rank cuts its own tensor-
        # parallel shard out of it. Step, optimizer moments and data position start afresh.
        from .convert import convert_reference_state_dict
        from .reshard import merge_checkpoint, split_plain_state_dict
        sd = convert_reference_state_dict(merge_checkpoint(init_from, cfg)["model_state_dict"])
        model.load_state_dict(split_plain_state_dict(sd, cfg, mesh.tp, mesh.tp_rank), strict=True)
        model.after_optimizer_step()
        logger.info(f"model weights initialised from {init_from} (tp shard {mesh.tp_rank} of {mesh.tp})")
    resume = getattr(args, "resume", None)
    data_step = 0
    if resume:
        path = resume
        if resume in ("latest", "auto") and run_dir:
            path = ckpt.find_latest_checkpoint(os.path.join(run_dir, "checkpoints"))
        if path and os.path.isdir(path):
            path = ckpt.find_latest_checkpoint(path)
        if path:
            info: Dict[str, Any] = {}
            step, loss = ckpt.load_checkpoint(path, model, muon, adamw, rank=mesh.rank, world_size=mesh.world_size,
                                              map_location=device, mesh=mesh, info=info)
            ctx.step = step + 1
            data_step = int(info.get("data_step", step + 1))
            logger.info(f"resumed from {path} at step {step} (loss {loss}); data position {data_step}")
    if data_iter is None:
        from ..data.loaders import build_data_iterator
        # the loader continues after the batches the checkpointed run had consumed instead of replaying them
        ctx.data_iter, ctx.prefetcher = build_data_iterator(args, cfg, mesh, start_step=data_step)
        ctx.extras["own_data_iter"] = True
        ctx.extras["epoch"] = int(getattr(ctx.data_iter, "epochs_skipped", 0) or 0)
    hb = float(getattr(args, "watchdog_timeout_s", 0) or 0)
    if hb > 0:
        from .watchdog import StepWatchdog
        ctx.watchdog = StepWatchdog(hb, run_dir, mesh.rank)
        ctx.watchdog.start()
    return ctx


def _micro_batches(T: int, mbs: int, row_len: Optional[int]):
    if not mbs or mbs <= 0 or mbs >= T:
        return [(0, T)]
    return [(s, min(T, s + mbs)) for s in range(0, T, mbs)]


def train_step(ctx: TrainContext, batch: Dict[str, torch.Tensor], timer: Optional[PhaseTimer] = None
               ) -> Dict[str, Any]:
    """One optimizer step over ``batch`` = {input_ids[T] | [B,S], labels, cu_seqlens}."""
    args, model, mesh, dev = ctx.args, ctx.model, ctx.mesh, ctx.device
    timer = timer or PhaseTimer(enabled=False)
    model.train()
    with timer.phase("h2d"):
        ids = batch["input_ids"].to(dev, non_blocking=True)
        labels = batch["labels"].to(dev, non_blocking=True)
        cu = batch.get("cu_seqlens")
        row_len = ids.shape[1] if ids.dim() == 2 else batch.get("row_len")
        ids, labels = ids.reshape(-1), labels.reshape(-1)
        T = ids.shape[0]
        if cu is None:
            rl = row_len or T
            cu = torch.arange(0, T + 1, rl, dtype=torch.int32)
        cu = cu.to(dev, non_blocking=True)
    targets = shift_targets(labels, row_len)
    mbs = int(getattr(args, "micro_batch_size", 0) or 0)
    gas = int(getattr(args, "gradient_accumulation_steps", 1) or 1)
    if mbs <= 0 and gas > 1:
        # the step's tokens are cut into ``gas`` windows; in the reference the number of chunks per step replaced this
        # knob (``src/training/loop/run.py:92-115``), here it stays as the way to ask for N windows without naming a size
        mbs = -(-T // gas)
    windows = _micro_batches(T, mbs, row_len)
    # valid-target count per window, summed over the data-parallel replicas, read back once per step: every replica
    # then runs (or skips) the same windows and issues the same gradient collectives
    counts_t = torch.stack([(targets[s:e] >= 0).sum() for s, e in windows]).float()
    counts_g = counts_t.clone()
    if mesh.dp > 1:
        dist.all_reduce(counts_g, group=mesh.dp_group)
    counts = counts_g.tolist()
    total_valid_f = max(float(sum(counts)), 1.0)
    carry = bool(getattr(args, "carry_kda_state", False))
    run = [wi for wi in range(len(windows)) if counts[wi] > 0 or carry]
    last_run = run[-1] if run else -1
    kda_states = None
    loss_acc = torch.zeros((), device=dev, dtype=torch.float32)
    with timer.phase("fwd_bwd"):
        for wi in run:
            s, e = windows[wi]
            cu_w = slice_cu_seqlens(cu, s, e).to(torch.int32)
            if ctx.grad_reducer is not None:
                ctx.grad_reducer.set_last_microbatch(wi == last_run)
            with nvtx_range(f"mb{wi}_forward"):
                init = None
                if carry and kda_states is not None:
                    continues = not bool(((cu == s).any()))
                    init = _carry_states(kda_states, cu_w.numel() - 1, continues)
                h, finals = model.hidden(ids[s:e], cu_w, init)
                loss = model.lm_head.loss(h, targets[s:e], total_valid_f)
            with nvtx_range(f"mb{wi}_backward"):
                loss.backward()
            loss_acc += loss.detach().float()
            if carry:
                kda_states = [f.detach() for f in finals]
            if ctx.offloader is not None:
                ctx.offloader.after_microbatch()
            if bool(getattr(args, "empty_cache_between_mb", False)) and dev.type == "cuda":
                torch.cuda.empty_cache()          # trades step time for a lower reserved-memory peak
    if not run:
        # no window of any replica holds a valid target: nothing was computed, nothing to apply
        return {"loss": loss_acc, "grad_norm": 0.0, "found_inf": False, "lr_muon": 0.0, "lr_adamw": 0.0,
                "tokens": T * mesh.dp, "n_valid": 0.0}
    with timer.phase("grad_sync"):
        if ctx.offloader is not None:
            ctx.offloader.drain_to_device()
        if ctx.grad_reducer is not None:
            ctx.grad_reducer.finish()
            dist.all_reduce(loss_acc, group=mesh.dp_group)
        model.sync_replicated_grads()
    with timer.phase("gradnorm"):
        gnorm_t = global_grad_norm(ctx.muon, ctx.adamw, mesh, owner_reduced=bool(ctx.extras.get("owner_reduced", False)))
        gnorm = float(gnorm_t)
        found_inf = not math.isfinite(gnorm)
    if ctx.extras.get("fused_comm", False):
        # the host is in step with the device here (the norm was just read back): a bounded wait on a peer that ran out
        # during this step left unfinished tiles behind, so the gradients must not be applied
        _check_fused_status(ctx)
    max_norm = float(getattr(args, "max_grad_norm", 1.0) or 0.0)
    lr_m = wsd_lr(ctx.step, float(getattr(args, "muon_lr", 0.02)), int(getattr(args, "lr_warmup_steps", 0)),
                  int(getattr(args, "lr_decay_steps", 0)), int(getattr(args, "max_steps", 1 << 30)))
    lr_a = wsd_lr(ctx.step, float(getattr(args, "learning_rate", 0.004)), int(getattr(args, "lr_warmup_steps", 0)),
                  int(getattr(args, "lr_decay_steps", 0)), int(getattr(args, "max_steps", 1 << 30)))
    if ctx.step < _DIAG_STEPS and getattr(args, "diagnostics", False):
        log_pre_step_diag(ctx.logger, ctx.step, [ctx.muon, ctx.adamw], gnorm)
    if not found_inf:
        coef = clip_coefficient(gnorm, max_norm)
        ctx.muon.set_lr(lr_m); ctx.adamw.set_lr(lr_a)
        with timer.phase("muon"):
            ctx.muon.step(grad_scale=coef)
        with timer.phase("adamw"):
            ctx.adamw.step(grad_scale=coef)
    else:
        ctx.logger.warning(f"step {ctx.step}: non-finite gradient norm; skipping the update")
    with timer.phase("zero"):
        ctx.muon.zero_grad(); ctx.adamw.zero_grad()
        repack_nvfp4_weights(model)
        model.after_optimizer_step()
    if ctx.step < _DIAG_STEPS and getattr(args, "diagnostics", False):
        log_post_opt_diag(ctx.logger, ctx.step, [ctx.muon, ctx.adamw])
    return {"loss": loss_acc, "grad_norm": gnorm, "found_inf": found_inf, "lr_muon": lr_m, "lr_adamw": lr_a,
            "tokens": T * mesh.dp, "n_valid": total_valid_f}


class FusedCommTimeout(RuntimeError):
    """A device-side wait on a tensor-parallel peer ran out inside a fused compute + collective kernel."""


def _check_fused_status(ctx: TrainContext) -> None:
    from ..ops import _ext
    st = _ext.device_status()
    if st[0] == 0:
        return
    _ext.clear_device_status()
    ctx.muon.zero_grad(); ctx.adamw.zero_grad()
    msg = (f"step {ctx.step}: a fused collective gave up waiting for a peer (code={st[0]} detail={st[1]} block={st[2]} "
           f"count={st[3]}); the update was not applied and the gradients were cleared")
    ctx.logger.error(msg)
    raise FusedCommTimeout(msg)


def _carry_states(prev: List[torch.Tensor], n_seq: int, continues: bool) -> List[torch.Tensor]:
    """Initial KDA states for the next token window: the previous window's last sequence state for
    the first sequence when the document continues, zeros for every other sequence."""
    out = []
    for p in prev:
        z = torch.zeros((n_seq,) + tuple(p.shape[1:]), dtype=p.dtype, device=p.device)
        if continues and n_seq > 0:
            z[0] = p[-1]
        out.append(z)
    return out


def _save_step_checkpoint(ctx: TrainContext, step: int, loss: float) -> None:
    args, mesh = ctx.args, ctx.mesh
    ctx.muon.sync_dp_state()              # collective: outside the try so that every rank takes part
    try:
        d = os.path.join(ctx.run_dir, "checkpoints")
        ckpt.save_checkpoint(ctx.model, ctx.muon, ctx.adamw, step, loss, ckpt.checkpoint_path(d, step), rank=mesh.rank,
                             world_size=mesh.world_size, mesh=mesh)
        if mesh.rank == 0:
            ckpt.prune_old_checkpoints(d, int(getattr(args, "checkpoint_keep_last_n", 0) or 0))
    except Exception as ex:   # a disk error must not kill training
        ctx.logger.error(f"checkpoint save failed at step {step}: {ex!r}")


def run_training_loop(ctx: TrainContext) -> Dict[str, Any]:
    args, mesh = ctx.args, ctx.mesh
    max_steps = int(getattr(args, "max_steps", 1000))
    log_interval = max(1, int(getattr(args, "log_interval", 1)))
    ck_int = int(getattr(args, "checkpoint_interval", 0) or 0)
    mb_timing = int(getattr(args, "mb_timing", 0) or 0)
    last = {}
    losses = []
    saved_step = -1
    try:
        while ctx.step < max_steps:
            try:
                batch = next(ctx.data_iter)
            except StopIteration:
                batch = None
            if mesh.dp > 1 and ctx.prefetcher is not None and ctx.extras.get("own_data_iter", False):
                # Finite real data: the replicas read different rows and may run out at different steps. They agree here, so
                # that all of them end the pass at the same step (a replica that still has a batch drops it) instead of
                # meeting in mismatched collectives.
                have = torch.tensor([0 if batch is None else 1], device=ctx.device)
                dist.all_reduce(have, op=dist.ReduceOp.MIN, group=mesh.dp_group)
                if int(have) == 0:
                    batch = None
            if batch is None:
                # end of an epoch: a finite dataset is re-opened until --epochs passes have been made
                epoch = ctx.extras.get("epoch", 0) + 1
                if epoch >= int(getattr(args, "epochs", 1) or 1) or not ctx.extras.get("own_data_iter", False):
                    ctx.logger.info("data exhausted")
                    break
                ctx.extras["epoch"] = epoch
                ctx.logger.info(f"epoch {epoch + 1}/{args.epochs}")
                if ctx.prefetcher is not None:
                    ctx.prefetcher.close()
                from ..data.loaders import build_data_iterator
                ctx.data_iter, ctx.prefetcher = build_data_iterator(args, ctx.cfg, mesh)
                continue
            timed = mb_timing < 0 or ctx.step < mb_timing
            # timed steps also leave their phases in a trace file (logs/trace_rank<r>.json, written at the end of the run)
            phase_mem = None
            if timed and getattr(args, "vram_phases", False):
                if "phase_memory" not in ctx.extras:
                    from ..utils.vram import PhaseMemory
                    ctx.extras["phase_memory"] = PhaseMemory(ctx.device)
                phase_mem = ctx.extras["phase_memory"]
            timer = PhaseTimer(enabled=timed, device=ctx.device, step=ctx.step, memory=phase_mem,
                               events=ctx.extras.setdefault("trace_events", []) if timed and ctx.run_dir else None)
            t0 = time.perf_counter()
            ev0 = ev1 = None
            if ctx.device.type == "cuda":
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ev0.record()
            if ctx.liveness is not None:
                # a peer that left (or went silent) is found here, on the host, before this step's first launch
                ctx.liveness.beat(ctx.step)
                ctx.liveness.check()
                try:
                    out = train_step(ctx, batch, timer)
                except Exception as ex:           # e.g. a collective that ran into the process-group timeout
                    raise ctx.liveness.diagnose(ex)
            else:
                out = train_step(ctx, batch, timer)
            if ev1 is not None:
                ev1.record(); ev1.synchronize()
                step_ms = ev0.elapsed_time(ev1)
            else:
                step_ms = (time.perf_counter() - t0) * 1e3
            loss = float(out["loss"])
            losses.append(loss)
            if ctx.watchdog is not None:
                ctx.watchdog.beat(ctx.step)
            if ctx.step % log_interval == 0:
                ms = torch.tensor([step_ms], device=ctx.device)
                if mesh.is_distributed:
                    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
                step_ms_max = float(ms)
                toks = out["tokens"] / (step_ms_max / 1e3)
                rec = {"step": ctx.step, "loss": loss, "lr_muon": out["lr_muon"], "lr_adamw": out["lr_adamw"],
                       "grad_norm": out["grad_norm"], "tokens": out["tokens"], "step_ms": step_ms_max,
                       "tok_per_s": toks, "found_inf": out["found_inf"]}
                if out["tokens"] > 0:
                    # analytic model FLOPs of the step over the device-timed step, per GPU, and its fraction of the measured
                    # (else the fallback) sustained bf16 GEMM peak
                    from ..utils.flops import utilisation
                    from ..utils.timing import load_measured_peaks
                    peaks = ctx.extras.setdefault("peaks", load_measured_peaks())
                    rec.update(utilisation(ctx.cfg, int(args.seq_len), int(out["tokens"]), step_ms_max, mesh.world_size, peaks))
                if timed:
                    rec["phases_ms"] = timer.summary()
                if phase_mem is not None:
                    rec["phases_peak_mb"] = phase_mem.step_summary(ctx.step)
                if ctx.device.type == "cuda":
                    rec["vram_alloc_mb"] = torch.cuda.memory_allocated(ctx.device) / 2 ** 20
                    rec["vram_reserved_mb"] = torch.cuda.memory_reserved(ctx.device) / 2 ** 20
                    rec["vram_max_mb"] = max(torch.cuda.max_memory_allocated(ctx.device),
                                             phase_mem.run_peak if phase_mem is not None else 0) / 2 ** 20
                if mesh.rank == 0:
                    ctx.logger.info(f"step {ctx.step} loss {loss:.4f} lr {out['lr_muon']:.2e}/{out['lr_adamw']:.2e} "
                                    f"gnorm {out['grad_norm']:.3f} tok {out['tokens']} {step_ms_max:.1f} ms "
                                    f"{toks:,.0f} tok/s" + (f" [mb-time] {timer.summary()}" if timed else ""))
                    if ctx.metrics_file is not None:
                        ctx.metrics_file.write(json.dumps(rec) + "\n"); ctx.metrics_file.flush()
            if ck_int > 0 and ctx.run_dir and (ctx.step + 1) % ck_int == 0:
                _save_step_checkpoint(ctx, ctx.step, loss)
                saved_step = ctx.step
            last = out
            ctx.step += 1
        # the run ended between two periodic checkpoints (last step, or a finite dataset ran out): keep its final state
        if ck_int > 0 and ctx.run_dir and losses and saved_step != ctx.step - 1:
            _save_step_checkpoint(ctx, ctx.step - 1, losses[-1])
    except BaseException as ex:
        if ctx.liveness is not None:
            ctx.liveness.mark_exit(repr(ex))
        raise
    finally:
        if ctx.liveness is not None:
            ctx.liveness.mark_exit("finished")
        if ctx.extras.get("trace_events") and ctx.run_dir:
            try:
                from ..utils.timing import write_chrome_trace
                os.makedirs(os.path.join(ctx.run_dir, "logs"), exist_ok=True)
                write_chrome_trace(os.path.join(ctx.run_dir, "logs", f"trace_rank{mesh.rank}.json"),
                                   ctx.extras["trace_events"], mesh.rank)
            except OSError as ex:
                ctx.logger.error(f"trace file not written: {ex!r}")
        teardown_worker(ctx)
    return {"losses": losses, "last": last, "steps": ctx.step}


def teardown_worker(ctx: Optional[TrainContext]) -> None:
    """Idempotent; tolerates a partially built context (``src/training/loop/teardown.py:22-57``)."""
    if ctx is None or getattr(ctx, "closed", False):
        return
    ctx.closed = True
    try:
        from ..parallel import fused as _fused
        _fused.teardown()
    except Exception:
        pass
    for name in ("prefetcher", "watchdog", "offloader"):
        obj = getattr(ctx, name, None)
        if obj is not None:
            try:
                obj.close()
            except Exception:
                pass
    mf = getattr(ctx, "metrics_file", None)
    if mf is not None:
        try:
            mf.close()
        except Exception:
            pass
    try:
        if dist.is_available() and dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass
