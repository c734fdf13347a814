"""Muon (Newton-Schulz) for matrices, AdamW for everything else, global grad-norm clip.

Device-resident by default (B200 has the HBM for it); ``offload=True`` keeps the optimizer state
in pinned host memory and streams it through the GPU per parameter, which is the reference's only
mode (``src/training/param_offload/muon.py:294-499``, ``adamw.py:233-432``).

Formulas (``muon.py:247-287,392-473``):
  M <- beta M + G;  U = G + beta M (nesterov);  W <- W (1 - lr wd) - lr NS5(U)
AdamW here is the standard one (v from g^2, both bias corrections); ``reference_compat=True``
reproduces the reference's variant (v from m^2, no first-moment correction, ``adamw.py:257-302``).
``ns_scope='shard'`` orthogonalises each TP rank's shard (what the reference does); ``'full'`` gathers a
TP-sharded matrix to one owner rank per matrix, orthogonalises the whole matrix there and scatters the
slices back (TP-invariant result).
Differences on purpose: NS runs on the whole (local) matrix, not on 4096-row slices
(``ns_row_chunk`` restores slices); fused projections are orthogonalised per ``muon_segments``.
"""
from __future__ import annotations

import re
import math
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..config import PrecisionConfig
from ..models.nvfp4_linear import NVFP4Linear
from ..parallel.mesh import get_mesh


def _pinned_like(shape, dtype) -> torch.Tensor:
    t = torch.zeros(shape, dtype=dtype)
    if torch.cuda.is_available():
        try:
            t = t.pin_memory()
        except Exception:
            pass
    return t


class _Entry:
    """One optimised tensor: a Parameter, or a no-master NVFP4 module (``param is None``)."""

    def __init__(self, param: Optional[nn.Parameter], module: Optional[NVFP4Linear], name: str):
        self.param, self.module, self.name = param, module, name
        self.step = 0
        self.exp_avg: Optional[torch.Tensor] = None
        self.exp_avg_sq: Optional[torch.Tensor] = None

    @property
    def shape(self):
        return tuple(self.param.shape) if self.param is not None else \
            (self.module.out_features, self.module.in_features)

    @property
    def device(self):
        return self.param.device if self.param is not None else self.module.packed_weight.device

    def grad(self) -> Optional[torch.Tensor]:
        return self.param.grad if self.param is not None else self.module.grad_w

    def clear_grad(self):
        if self.param is not None:
            self.param.grad = None
        else:
            self.module.grad_w = None


class Muon:
    def __init__(self, lr: float = 0.02, momentum: float = 0.95, weight_decay: float = 0.0,
                 nesterov: bool = True, ns_steps: int = 5, momentum_dtype=torch.bfloat16,
                 offload: bool = False, ns_row_chunk: Optional[int] = None, ns_scope: str = "shard",
                 dp_shard: bool = False, stochastic_rounding: bool = True, sr_seed: int = 0):
        self.ns_scope = ns_scope
        # no-master NVFP4 weights are re-quantised with stochastic rounding (expected value = exact update), keyed by
        # (sr_seed, entry, step) so a run is reproducible
        self.stochastic_rounding, self.sr_seed = stochastic_rounding, int(sr_seed)
        # Under data parallelism every matrix has one owner among the DP replicas (greedy by size): only the owner runs
        # momentum + Newton-Schulz + the update, then broadcasts the new weights to its DP peers. Cuts the Muon work per
        # rank by the DP degree; the reference has neither data parallelism nor this split.
        self.dp_shard = dp_shard
        self._owners: Optional[List[int]] = None
        self.lr, self.momentum, self.weight_decay = lr, momentum, weight_decay
        self.nesterov, self.ns_steps = nesterov, ns_steps
        self.momentum_dtype = momentum_dtype
        self.offload = offload
        self.ns_row_chunk = ns_row_chunk
        self.entries: List[_Entry] = []

    def set_lr(self, lr: float):
        self.lr = lr

    def add_param(self, p: nn.Parameter, name: str = ""):
        assert p.ndim == 2, f"Muon takes 2-D weights, got {tuple(p.shape)} for {name}"
        self._alloc(_Entry(p, None, name))

    def register_nvfp4_module(self, mod: NVFP4Linear, name: str = ""):
        self._alloc(_Entry(None, mod, name))

    def _alloc(self, e: _Entry):
        e.idx = len(self.entries)
        if self.offload:
            e.exp_avg = _pinned_like(e.shape, self.momentum_dtype)
        else:
            e.exp_avg = torch.zeros(e.shape, dtype=self.momentum_dtype, device=e.device)
        self.entries.append(e)

    def _segments(self, e: _Entry) -> List[Tuple[int, int]]:
        rows = e.shape[0]
        segs = getattr(e.param, "muon_segments", None) if e.param is not None else None
        segs = segs or [(0, rows)]
        if self.ns_row_chunk:
            out = []
            for a, b in segs:
                out += [(r, min(r + self.ns_row_chunk, b)) for r in range(a, b, self.ns_row_chunk)]
            segs = out
        return segs

    def _shard_dim(self, e: _Entry, seg) -> Optional[int]:
        """TP shard dimension of a segment (None = replicated / unsharded)."""
        if e.param is not None:
            rows = getattr(e.param, "tp_replicated_rows", None)
            if getattr(e.param, "tp_replicated", False) or (rows is not None and seg[0] >= rows[0] and seg[1] <= rows[1]):
                return None
            return getattr(e.param, "tp_shard_dim", None)
        return getattr(e.module, "tp_shard_dim", None)

    def _apply(self, e: _Entry, a: int, b: int, upd: torch.Tensor, wd_factor: float):
        if e.param is not None:
            pw = e.param.data[a:b]
            if wd_factor != 1.0:
                pw.mul_(wd_factor)
            pw.add_(upd.to(pw.dtype), alpha=-self.lr)
        else:
            for r0, r1 in e.module.chunk_ranges():
                lo, hi = max(r0, a), min(r1, b)
                if lo < hi:
                    e.module.decay_and_apply_chunk(lo, hi, upd[lo - a:hi - a], self.lr, wd_factor)

    def _step_cuda(self, e: _Entry, g: torch.Tensor, grad_scale: float, wd_factor: float, full_scope: bool,
                   work: Optional[list] = None) -> bool:
        """Fully fused device path for one entry; returns False when the entry needs the generic path. Segments that are
        tensor-parallel shards of a larger matrix are, under ``ns_scope = full``, only given their momentum update here and
        queued on ``work`` (entry, row0, row1, u) for the gather -> full-matrix Newton-Schulz -> scatter rounds."""
        from ..ops import muon_cuda as mc
        segs = self._segments(e)
        cols = e.shape[1]
        if g.dtype not in (torch.bfloat16, torch.float32) or not g.is_contiguous():
            return False
        for (a, b) in segs:
            if full_scope and b > a and self._shard_dim(e, (a, b)) is not None and (work is None or not mc.supported(b - a, cols)):
                return False
        fp4_segments = []
        for (a, b) in segs:
            if b <= a:
                continue
            if full_scope and self._shard_dim(e, (a, b)) is not None:
                u, _ = mc.momentum_update(g[a:b], e.exp_avg[a:b], self.momentum, grad_scale, self.nesterov)
                work.append((e, a, b, u))
                continue
            if not mc.supported(b - a, cols):
                # tiny / ragged segment (e.g. the H/tp rows of the beta projection): elementwise momentum on the slice,
                # then Newton-Schulz on the tcgen05 path after padding with zero rows (zero rows stay zero through every
                # iteration and do not touch the others, so the real rows get exactly their own result)
                gf = g[a:b].float() * grad_scale
                m = e.exp_avg[a:b].float().mul_(self.momentum).add_(gf)
                e.exp_avg[a:b].copy_(m)
                u = gf.add(m, alpha=self.momentum) if self.nesterov else m
                if cols % 8 == 0 and e.param is not None:
                    rp = (b - a + 7) // 8 * 8
                    up = torch.zeros((rp, cols), dtype=torch.bfloat16, device=u.device)
                    up[:b - a] = u
                    ssq = up.float().pow(2).sum().reshape(1)
                    self._apply(e, a, b, mc.newton_schulz_(up, ssq, self.ns_steps)[:b - a], wd_factor)
                else:
                    self._apply(e, a, b, ops.newton_schulz5(u, self.ns_steps), wd_factor)
                continue
            u, ssq = mc.momentum_update(g[a:b], e.exp_avg[a:b], self.momentum, grad_scale, self.nesterov)
            o = mc.newton_schulz_(u, ssq, self.ns_steps)
            if e.param is not None:
                mc.apply_update(e.param.data[a:b], o, wd_factor, self.lr)
            else:
                fp4_segments.append((a, b, o))
        if fp4_segments:
            # all segments of a no-master NVFP4 tensor share one tensor scale: update them together
            mc.nvfp4_apply_update(e.module, fp4_segments, wd_factor, self.lr,
                                  seed=(self.sr_seed * 1000003 + e.step * 7919 + getattr(e, "idx", 0)) & 0x7FFFFFFF,
                                  stochastic=self.stochastic_rounding)
        e.step += 1
        return True

    def _dp_owners(self, dp: int) -> List[int]:
        """Owner (DP rank) of every entry: largest matrices first, each to the least loaded replica."""
        if self._owners is None or len(self._owners) != len(self.entries):
            load = [0] * dp
            owners = [0] * len(self.entries)
            for idx in sorted(range(len(self.entries)), key=lambda i: -self.entries[i].shape[0] * self.entries[i].shape[1]):
                o = min(range(dp), key=lambda r: load[r])
                owners[idx] = o
                load[o] += self.entries[idx].shape[0] * self.entries[idx].shape[1]
            self._owners = owners
        return self._owners

    def dp_owner_map(self, dp: int) -> Dict[int, int]:
        """id(parameter) / id(NVFP4 module) -> owning DP rank, for a gradient reducer that reduces to the owner only."""
        owners = self._dp_owners(dp)
        return {id(e.param if e.param is not None else e.module): owners[i] for i, e in enumerate(self.entries)}

    def _broadcast_from_owners(self, mesh, owners: List[int]) -> None:
        ranks = mesh.dp_ranks()
        for idx, e in enumerate(self.entries):
            src = ranks[owners[idx]]
            if e.param is not None:
                dist.broadcast(e.param.data, src=src, group=mesh.dp_group)
            else:
                mod = e.module
                for t in (mod.packed_weight, mod.scales, mod.global_scale):
                    # byte view: not every backend carries float8
                    dist.broadcast(t.view(torch.uint8) if t.dtype not in (torch.float32, torch.uint8) else t,
                                   src=src, group=mesh.dp_group)

    @torch.no_grad()
    def sync_dp_state(self) -> None:
        """Momentum of every matrix from its owner to the DP peers (before a checkpoint: only owners keep it current)."""
        mesh = get_mesh()
        if not (self.dp_shard and mesh.dp > 1) or self._owners is None:
            return
        ranks = mesh.dp_ranks()
        for idx, e in enumerate(self.entries):
            if e.exp_avg.is_cuda or dist.get_backend(mesh.dp_group) == "gloo":
                dist.broadcast(e.exp_avg, src=ranks[self._owners[idx]], group=mesh.dp_group)
            else:                                   # pinned host state under an NCCL group: stage through the device
                t = e.exp_avg.to(mesh.device)
                dist.broadcast(t, src=ranks[self._owners[idx]], group=mesh.dp_group)
                e.exp_avg.copy_(t)

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0):
        mesh = get_mesh()
        full_scope = self.ns_scope == "full" and mesh.tp > 1
        wd_factor = 1.0 - self.lr * self.weight_decay
        owners = self._dp_owners(mesh.dp) if (self.dp_shard and mesh.dp > 1 and not full_scope) else None
        work = []                                   # (entry, a, b, u_segment)
        for idx, e in enumerate(self.entries):
            if owners is not None and owners[idx] != mesh.dp_rank:
                e.step += 1                         # the owner updates this matrix; the new weights arrive below
                continue
            g = e.grad()
            if g is None:
                continue
            dev = e.device
            if dev.type == "cuda" and not self.offload and self._step_cuda(e, g, grad_scale, wd_factor, full_scope, work):
                continue
            gf = g.to(torch.float32)
            if grad_scale != 1.0:
                gf = gf * grad_scale
            m = e.exp_avg.to(dev, non_blocking=True).float() if self.offload else e.exp_avg.float()
            m.mul_(self.momentum).add_(gf)
            u = gf.add(m, alpha=self.momentum) if self.nesterov else m
            if self.offload:
                e.exp_avg.copy_(m.to(self.momentum_dtype), non_blocking=True)
            else:
                e.exp_avg.copy_(m)
            e.step += 1
            for (a, b) in self._segments(e):
                if b <= a:
                    continue
                if full_scope and self._shard_dim(e, (a, b)) is not None:
                    work.append((e, a, b, u[a:b].contiguous()))
                else:
                    self._apply(e, a, b, ops.newton_schulz5(u[a:b], self.ns_steps), wd_factor)
        if owners is not None:
            self._broadcast_from_owners(mesh, owners)
        if not work:
            return
        # full-matrix NS for TP-sharded matrices: matrix i is gathered to TP rank i % tp, orthogonalised there
        # (every rank works on a different matrix of the round) and the slices are scattered back.
        tp, r, grp = mesh.tp, mesh.tp_rank, mesh.tp_group
        ranks = mesh.tp_ranks()
        fp4_pending: Dict[int, list] = {}           # id(module) -> [module, [(a, b, o)]]: all segments share one tensor scale
        for r0 in range(0, len(work), tp):
            rnd = work[r0:r0 + tp]
            gathered = [None] * len(rnd)
            for j, (e, a, b, u) in enumerate(rnd):
                lst = [torch.empty_like(u) for _ in range(tp)] if r == j else None
                dist.gather(u, lst, dst=ranks[j], group=grp)
                gathered[j] = lst
            outs = [None] * len(rnd)
            for j, (e, a, b, u) in enumerate(rnd):
                if r == j:
                    dim = self._shard_dim(e, (a, b))
                    full = torch.cat(gathered[j], dim=dim)
                    o = self._ns_full(full)
                    outs[j] = [t.contiguous() for t in o.chunk(tp, dim=dim)]
            for j, (e, a, b, u) in enumerate(rnd):
                mine = torch.empty_like(u)
                dist.scatter(mine, outs[j] if r == j else None, src=ranks[j], group=grp)
                if mine.is_cuda and mine.dtype == torch.bfloat16 and not self.offload:
                    from ..ops import muon_cuda as mc
                    if e.param is not None:
                        mc.apply_update(e.param.data[a:b], mine, wd_factor, self.lr)
                    else:
                        fp4_pending.setdefault(id(e.module), [e, []])[1].append((a, b, mine))
                else:
                    self._apply(e, a, b, mine, wd_factor)
        for e, segs in fp4_pending.values():
            from ..ops import muon_cuda as mc
            mc.nvfp4_apply_update(e.module, sorted(segs, key=lambda t: t[0]), wd_factor, self.lr,
                                  seed=(self.sr_seed * 1000003 + e.step * 7919 + getattr(e, "idx", 0)) & 0x7FFFFFFF,
                                  stochastic=self.stochastic_rounding)

    def _ns_full(self, full: torch.Tensor) -> torch.Tensor:
        """Newton-Schulz of a gathered full matrix: the tcgen05 path for bf16 CUDA matrices, the fp32 oracle otherwise."""
        if full.is_cuda and full.dtype == torch.bfloat16:
            from ..ops import muon_cuda as mc
            if mc.supported(full.shape[0], full.shape[1]):
                full = full.contiguous()
                ssq = full.float().pow(2).sum().reshape(1)
                return mc.newton_schulz_(full, ssq, self.ns_steps)
        return ops.newton_schulz5(full, self.ns_steps)

    def zero_grad(self):
        for e in self.entries:
            e.clear_grad()

    def state_dict(self) -> Dict:
        return {"lr": self.lr, "momentum": self.momentum, "weight_decay": self.weight_decay,
                "nesterov": self.nesterov, "ns_steps": self.ns_steps,
                "state": [{"shape": list(e.shape), "step": e.step,
                           "kind": "nvfp4" if e.param is None else "param", "name": e.name,
                           "grad": None, "exp_avg": e.exp_avg.detach().cpu().clone()} for e in self.entries]}

    def load_state_dict(self, sd: Dict):
        for k in ("lr", "momentum", "weight_decay", "nesterov", "ns_steps"):
            if k in sd:
                setattr(self, k, sd[k])
        st = sd["state"]
        if len(st) != len(self.entries):
            raise ValueError(f"Muon state has {len(st)} entries, optimizer has {len(self.entries)}")
        for e, s in zip(self.entries, st):
            if tuple(s["shape"]) != e.shape:
                raise ValueError(f"shape mismatch for {e.name}: {s['shape']} vs {e.shape}")
            e.step = s["step"]
            e.exp_avg.copy_(s["exp_avg"].to(e.exp_avg.dtype))


class AdamW:
    def __init__(self, lr: float = 0.004, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.01,
                 m_dtype=torch.bfloat16, v_dtype=torch.bfloat16, offload: bool = False,
                 reference_compat: bool = False):
        self.lr, self.betas, self.eps, self.weight_decay = lr, tuple(betas), eps, weight_decay
        self.m_dtype, self.v_dtype, self.offload = m_dtype, v_dtype, offload
        self.reference_compat = reference_compat
        self.entries: List[_Entry] = []

    def set_lr(self, lr: float):
        self.lr = lr

    def add_param(self, p: nn.Parameter, name: str = ""):
        e = _Entry(p, None, name)
        if self.offload:
            e.exp_avg = _pinned_like(e.shape, self.m_dtype)
            e.exp_avg_sq = _pinned_like(e.shape, self.v_dtype)
        else:
            e.exp_avg = torch.zeros(e.shape, dtype=self.m_dtype, device=p.device)
            e.exp_avg_sq = torch.zeros(e.shape, dtype=self.v_dtype, device=p.device)
        self.entries.append(e)

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0):
        b1, b2 = self.betas
        for e in self.entries:
            g = e.grad()
            if g is None:
                continue
            e.step += 1
            p = e.param.data
            if self.offload:
                m = e.exp_avg.to(p.device, non_blocking=True)
                v = e.exp_avg_sq.to(p.device, non_blocking=True)
            else:
                m, v = e.exp_avg, e.exp_avg_sq
            if self.reference_compat:
                gf = g.float() * grad_scale
                mf = m.float().mul_(b1).add_(gf, alpha=1 - b1)
                vf = v.float().mul_(b2).addcmul_(mf, mf, value=1 - b2)
                m.copy_(mf); v.copy_(vf)
                upd = mf / ((vf / (1 - b2 ** e.step)).sqrt() + self.eps)
                p.copy_(p.float().mul_(1 - self.lr * self.weight_decay).add_(upd, alpha=-self.lr))
            else:
                ops.adamw_update(p, g, m, v, self.lr, b1, b2, self.eps, self.weight_decay, e.step, grad_scale)
            if self.offload:
                e.exp_avg.copy_(m, non_blocking=True)
                e.exp_avg_sq.copy_(v, non_blocking=True)

    def zero_grad(self):
        for e in self.entries:
            e.clear_grad()

    def state_dict(self) -> Dict:
        return {"lr": self.lr, "betas": list(self.betas), "eps": self.eps, "weight_decay": self.weight_decay,
                "state": [{"shape": list(e.shape), "step": e.step, "kind": "param", "name": e.name, "grad": None,
                           "exp_avg": e.exp_avg.detach().cpu().clone(),
                           "exp_avg_sq": e.exp_avg_sq.detach().cpu().clone()} for e in self.entries]}

    def load_state_dict(self, sd: Dict):
        for k in ("lr", "eps", "weight_decay"):
            if k in sd:
                setattr(self, k, sd[k])
        if "betas" in sd:
            self.betas = tuple(sd["betas"])
        st = sd["state"]
        if len(st) != len(self.entries):
            raise ValueError(f"AdamW state has {len(st)} entries, optimizer has {len(self.entries)}")
        for e, s in zip(self.entries, st):
            if tuple(s["shape"]) != e.shape:
                raise ValueError(f"shape mismatch for {e.name}: {s['shape']} vs {e.shape}")
            e.step = s["step"]
            e.exp_avg.copy_(s["exp_avg"].to(e.exp_avg.dtype))
            e.exp_avg_sq.copy_(s["exp_avg_sq"].to(e.exp_avg_sq.dtype))


def build_param_groups(model: nn.Module, args=None, precision: Optional[PrecisionConfig] = None,
                       offload: bool = False) -> Tuple[Muon, AdamW]:
    """Route parameters (``src/training/param_offload/param_groups.py:27-153``): embeddings, head,
    norms, biases, conv taps, gate scalars and the AttnRes query -> AdamW; every other 2-D weight
    and every no-master NVFP4 module -> Muon (nesterov, 5 NS steps)."""
    prec = precision or PrecisionConfig()
    g = (lambda k, d: getattr(args, k, d) if args is not None else d)
    muon = Muon(lr=g("muon_lr", 0.02), momentum=g("muon_momentum", 0.95),
                weight_decay=g("muon_weight_decay", 0.0), nesterov=True, ns_steps=5,
                momentum_dtype=prec.muon_momentum, offload=offload,
                ns_row_chunk=g("muon_ns_row_chunk", None), ns_scope=g("muon_ns_scope", "shard"),
                dp_shard=bool(g("muon_dp_shard", True)),
                stochastic_rounding=bool(g("nvfp4_stochastic_rounding", True)), sr_seed=int(g("seed", 0) or 0))
    adamw = AdamW(lr=g("learning_rate", 0.004), betas=(g("adamw_beta1", 0.9), g("adamw_beta2", 0.95)),
                  eps=g("adamw_eps", 1e-8), weight_decay=g("weight_decay", 0.01),
                  m_dtype=prec.adamw_m, v_dtype=prec.adamw_v, offload=offload,
                  reference_compat=bool(g("adamw_reference_compat", False)))
    for name, p in model.named_parameters():
        if not p.requires_grad:
            continue
        kind = getattr(p, "opt_kind", None)
        if kind is None:
            kind = "muon" if (p.ndim == 2 and "embed" not in name and "lm_head" not in name) else "adamw"
        if kind == "muon" and p.ndim == 2:
            muon.add_param(p, name)
        else:
            adamw.add_param(p, name)
    rx = g("trainable_regex", None)
    for name, mod in model.named_modules():
        if isinstance(mod, NVFP4Linear) and mod.no_master:
            if rx and not re.search(rx, name):
                continue                     # frozen: the module keeps its weights, its dW products are dropped
            muon.register_nvfp4_module(mod, name)
    return muon, adamw


@torch.no_grad()
def global_grad_norm(muon: Muon, adamw: AdamW, mesh=None, owner_reduced: bool = False) -> torch.Tensor:
    """||G||_2 over every gradient of the whole model (device-side; the reference reduces a host
    fp64 scalar, ``src/training/loop/grad_norm.py:97-165``). TP-sharded tensors are summed over
    the TP group; replicated ones are counted once. ``owner_reduced``: the Muon gradients were reduced to
    their owning DP replica only, so every matrix is counted by its owner, the all-reduced rest by DP rank 0,
    and the partial sums are added over the DP group."""
    m = mesh or get_mesh()
    owner_reduced = bool(owner_reduced and m.dp > 1 and muon.dp_shard)
    m_owners = muon._dp_owners(m.dp) if owner_reduced else None
    dev = None
    for e in list(muon.entries) + list(adamw.entries):
        g = e.grad()
        if g is not None:
            dev = g.device
            break
    if dev is None:
        return torch.zeros(())
    acc = torch.zeros(2, dtype=torch.float32, device=dev)      # [sharded, replicated]
    items = []                                                 # (gradient segment, slot)
    n_muon = len(muon.entries)
    for idx, e in enumerate(list(muon.entries) + list(adamw.entries)):
        g = e.grad()
        if g is None:
            continue
        if owner_reduced and (m_owners[idx] if idx < n_muon else 0) != m.dp_rank:
            continue
        rows = getattr(e.param, "tp_replicated_rows", None) if e.param is not None else None
        is_repl = e.param is not None and getattr(e.param, "tp_replicated", False)
        if is_repl:
            items.append((g, 1))
        elif rows is not None:
            a, b = rows
            items += [(g[:a], 0), (g[a:b], 1), (g[b:], 0)]
        else:
            items.append((g, 0))
    if dev.type == "cuda" and all(t.is_contiguous() and t.dtype in (torch.bfloat16, torch.float32) for t, _ in items):
        from ..ops.optim_cuda import sumsq_multi
        sumsq_multi(items, acc)                                # one launch for the whole model
    else:
        for t, slot in items:
            acc[slot] += t.float().pow(2).sum()
    if owner_reduced:
        dist.all_reduce(acc, group=m.dp_group)
    sharded, repl = acc[0], acc[1]
    if m.tp > 1:
        sharded = sharded.clone()
        dist.all_reduce(sharded, group=m.tp_group)
    return (sharded + repl).sqrt()


def clip_coefficient(norm: float, max_norm: float) -> float:
    """coef = max_norm/(norm+1e-6) applied only when norm > max_norm (``grad_norm.py:150-165``)."""
    if max_norm is None or max_norm <= 0 or not math.isfinite(norm) or norm <= max_norm:
        return 1.0
    return max_norm / (norm + 1e-6)
