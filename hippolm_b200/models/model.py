"""Hybrid KDA / full-attention decoder with block attention residuals.

One model class covers TP=1 and TP>1 (with Megatron sequence parallelism): between the
tensor-parallel regions activations are ``[T/tp, D]`` token shards; inside them the projections
see all ``T`` tokens and ``H/tp`` heads. The token axis is a packed stream of documents described
by ``cu_seqlens`` (the batch dimension is folded into it).

Parity notes against the reference (paths relative to its tree):
  layer wiring        ``src/models/tp_model/layer.py:50-97``, ``kda.py:207-337``
  block AttnRes       ``src/models/tp_model/model.py:575-727``, ``src/models/ops/attn_res.py:174-295``
  state_dict keys     ``src/models/model.py:68-107`` (plain layout; written by the state-dict hooks below)
Not in the reference: full-attention layers with RoPE, sequence parallelism, untied head,
cu_seqlens-aware KDA under TP, backward collectives and replicated-gradient sync.
"""
from __future__ import annotations

import os
import math
import zlib
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint as _ckpt

from .. import ops
from ..config import HippoConfig
from ..parallel.collectives import gather_seq, reduce_scatter_seq, all_reduce_sum, all_gather_dim0, \
    reduce_scatter_dim0
from ..parallel.linear import column_linear_sp, row_linear_sp, nvfp4_column_linear_sp, nvfp4_row_linear_sp
from ..parallel.mesh import get_mesh
from ..ref.ops import positions_from_cu
from .nvfp4_linear import NVFP4Linear


def _pad_to(n: int, m: int) -> int:
    return (n + m - 1) // m * m


_INIT_DEVICE = [torch.device("cpu")]


def _seeded(name: str, seed: int, device=None) -> torch.Generator:
    g = torch.Generator(device=device if device is not None else "cpu")
    g.manual_seed((zlib.crc32(name.encode()) + seed * 1000003) % (2 ** 31))
    return g


def _xavier(name: str, shape, seed: int) -> torch.Tensor:
    """TP-invariant init: the full matrix is drawn from a per-name stream (on the model's device, so
    a 7B model initialises in seconds), shards are slices of it."""
    fan_out, fan_in = shape
    a = math.sqrt(6.0 / (fan_in + fan_out))
    dev = _INIT_DEVICE[0]
    return (torch.rand(shape, generator=_seeded(name, seed, dev), device=dev) * 2 - 1) * a


def _normal(name: str, shape, seed: int, std: float) -> torch.Tensor:
    dev = _INIT_DEVICE[0]
    return torch.randn(shape, generator=_seeded(name, seed, dev), device=dev) * std


def _shard_rows(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = w.shape[0] // world
    return w[rank * n:(rank + 1) * n]


def _shard_cols(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = w.shape[1] // world
    return w[:, rank * n:(rank + 1) * n]


def _mark(p: nn.Parameter, kind: str, replicated: bool = False, **kw) -> nn.Parameter:
    p.opt_kind = kind
    p.tp_replicated = replicated
    for k, v in kw.items():
        setattr(p, k, v)
    return p


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.weight = _mark(nn.Parameter(torch.ones(dim, device=device, dtype=dtype)), "adamw", True)

    def forward(self, x):
        return ops.rmsnorm(x, self.weight, self.eps)


# =============================================================================================== KDA
class KDAAttention(nn.Module):
    """Kimi delta attention block. Fused column-parallel input projection
    ``[q | k | v | fg_first | b_proj | pad]`` (one all-gather -> GEMM), low-rank gate
    projections, chunked KDA, gated per-head RMSNorm, row-parallel output projection."""

    def __init__(self, cfg: HippoConfig, layer_idx: int, seed: int, device, dtype):
        super().__init__()
        m = get_mesh()
        w, r = m.tp, m.tp_rank
        self.cfg = cfg
        D, H, K, Vd = cfg.hidden_size, cfg.num_heads, cfg.head_dim, cfg.head_v_dim
        assert H % w == 0, "num_heads must be divisible by tp"
        self.Hl = H // w
        self.key_l, self.val_l = self.Hl * K, self.Hl * Vd
        pre = f"layers.{layer_idx}.attn."
        q = _shard_rows(_xavier(pre + "q", (cfg.key_dim, D), seed), r, w)
        k = _shard_rows(_xavier(pre + "k", (cfg.key_dim, D), seed), r, w)
        v = _shard_rows(_xavier(pre + "v", (cfg.value_dim, D), seed), r, w)
        fg = _xavier(pre + "fg_first", (2 * Vd, D), seed)
        b = _shard_rows(_xavier(pre + "b_proj", (H, D), seed), r, w)
        self.sections = [self.key_l, self.key_l, self.val_l, 2 * Vd, self.Hl]
        n_real = sum(self.sections)
        n_pad = _pad_to(n_real, 64)
        fused = torch.zeros(n_pad, D, device=q.device)
        fused[:n_real] = torch.cat([q, k, v, fg, b], 0)
        self.n_real = n_real
        o_fg = 2 * self.key_l + self.val_l
        self.in_proj_weight = _mark(
            nn.Parameter(fused.to(device=device, dtype=dtype)), "muon",
            muon_segments=[(0, 2 * self.key_l + self.val_l), (o_fg, o_fg + 2 * Vd), (o_fg + 2 * Vd, n_real)],
            tp_replicated_rows=(o_fg, o_fg + 2 * Vd), tp_shard_dim=0)
        if cfg.use_short_conv:
            def conv_w(nm, dim_full):
                full = (torch.rand((dim_full, cfg.conv_size), generator=_seeded(pre + nm, seed)) * 2 - 1) \
                    / math.sqrt(cfg.conv_size)
                return _mark(nn.Parameter(_shard_rows(full, r, w).to(device=device, dtype=dtype)), "adamw")
            self.q_conv1d_weight = conv_w("q_conv1d", cfg.key_dim)
            self.k_conv1d_weight = conv_w("k_conv1d", cfg.key_dim)
            self.v_conv1d_weight = conv_w("v_conv1d", cfg.value_dim)
        self.f_proj1_weight = _mark(nn.Parameter(_shard_rows(
            _xavier(pre + "f_proj1", (cfg.key_dim, Vd), seed), r, w).to(device=device, dtype=dtype)), "muon", tp_shard_dim=0)
        self.g_proj1_weight = _mark(nn.Parameter(_shard_rows(
            _xavier(pre + "g_proj1", (cfg.value_dim, Vd), seed), r, w).to(device=device, dtype=dtype)), "muon", tp_shard_dim=0)
        self.g_proj1_bias = _mark(nn.Parameter(torch.zeros(self.val_l, device=device, dtype=dtype)), "adamw")
        gen = _seeded(pre + "gate", seed)
        if cfg.safe_gate:
            A_full = torch.zeros(H)
        else:
            A_full = torch.log(torch.empty(H).uniform_(1, 16, generator=gen))
        dt = torch.exp(torch.rand(cfg.key_dim, generator=gen) * (math.log(0.1) - math.log(0.001))
                       + math.log(0.001)).clamp(min=1e-4)
        dt_bias_full = dt + torch.log(-torch.expm1(-dt))
        self.A_log = _mark(nn.Parameter(_shard_rows(A_full, r, w).to(device=device, dtype=torch.float32)), "adamw")
        self.dt_bias = _mark(nn.Parameter(_shard_rows(dt_bias_full, r, w).to(device=device, dtype=torch.float32)),
                             "adamw")
        self.o_norm_weight = _mark(nn.Parameter(torch.ones(Vd, device=device, dtype=dtype)), "adamw", True)
        self.o_proj_weight = _mark(nn.Parameter(_shard_cols(
            _xavier(pre + "o_proj", (D, cfg.value_dim), seed), r, w).contiguous().to(device=device, dtype=dtype)),
            "muon", tp_shard_dim=1)
        self._register_state_dict_hook(_kda_split_hook)
        self._register_load_state_dict_pre_hook(_kda_fuse_hook, with_module=True)

    def forward(self, h, cu_seqlens, initial_state, cache: Optional[dict] = None):
        """``cache`` (inference with incremental decoding): a per-layer dict. The recurrent states (one per sequence)
        travel through ``initial_state`` / the returned final state as in training; with the short convolution the cache
        also keeps every sequence's last ``conv_size - 1`` pre-convolution rows (``"conv_tail"``) so that a one-token
        step sees the taps of the tokens before it. A step with one token per sequence runs the token-recurrent form."""
        cfg = self.cfg
        K, Vd, Hl = cfg.head_dim, cfg.head_v_dim, self.Hl
        proj = column_linear_sp(h, self.in_proj_weight)                       # [T, n_pad]
        T = proj.shape[0]
        o_fg = 2 * self.key_l + self.val_l
        fg = proj[:, o_fg:o_fg + 2 * Vd]
        beta_mul = 2.0 if cfg.allow_neg_eigval else 1.0
        mode = cfg.kda_mode
        if cache is not None and T == cu_seqlens.numel() - 1:
            mode = "fused_recurrent"                                          # one token per sequence
        if cfg.use_short_conv:
            qkv_in = proj[:, :o_fg]
            cu_conv, pick = cu_seqlens, None
            W1 = cfg.conv_size - 1
            if cache is not None and W1 > 0:
                # Every sequence keeps its last conv_size - 1 pre-convolution rows, zero-filled while it is shorter: taps
                # before the start of a document are zero, so a zero row in front of the window changes nothing.
                N = cu_seqlens.numel() - 1
                tail = cache.get("conv_tail")
                if tail is None:
                    tail = qkv_in.new_zeros(N, W1, o_fg)
                if T == N:
                    # one token per sequence: windows [tail | new row], convolved as N documents of conv_size rows
                    win = torch.cat([tail, qkv_in.unsqueeze(1)], 1)                  # [N, W, o_fg]
                    cache["conv_tail"] = win[:, 1:].clone()
                    qkv_in = win.reshape(N * cfg.conv_size, o_fg)
                    cu_conv = torch.arange(0, N * cfg.conv_size + 1, cfg.conv_size, device=proj.device, dtype=torch.int32)
                    pick = torch.arange(1, N + 1, device=proj.device) * cfg.conv_size - 1
                else:
                    cu_l = cu_seqlens.tolist()
                    new_tail = qkv_in.new_zeros(N, W1, o_fg)
                    for n in range(N):
                        rows = qkv_in[max(cu_l[n], cu_l[n + 1] - W1):cu_l[n + 1]]
                        if rows.shape[0] > 0:
                            new_tail[n, W1 - rows.shape[0]:] = rows
                    cache["conv_tail"] = new_tail
            q, k, v = qkv_in[:, :self.key_l], qkv_in[:, self.key_l:2 * self.key_l], qkv_in[:, 2 * self.key_l:o_fg]
            q = ops.short_conv_silu(q, self.q_conv1d_weight, None, cu_conv)
            k = ops.short_conv_silu(k, self.k_conv1d_weight, None, cu_conv)
            v = ops.short_conv_silu(v, self.v_conv1d_weight, None, cu_conv)
            if pick is not None:
                q, k, v = q[pick], k[pick], v[pick]
            q, k, v = q.reshape(T, Hl, K), k.reshape(T, Hl, K), v.reshape(T, Hl, Vd)
            q = ops.l2norm(q) * (K ** -0.5)
            k = ops.l2norm(k)
            beta = torch.sigmoid(proj[:, o_fg + 2 * Vd:o_fg + 2 * Vd + Hl].float()) * beta_mul
        else:
            q, k, v, beta, fg = ops.kda_prologue(proj, Hl, K, 0, self.key_l, 2 * self.key_l, o_fg + 2 * Vd,
                                                 K ** -0.5, beta_mul, True, o_fg, 2 * Vd)
        g_raw = ops.linear(fg[:, :Vd].contiguous(), self.f_proj1_weight)
        gate = ops.linear(fg[:, Vd:].contiguous(), self.g_proj1_weight, self.g_proj1_bias)
        g = ops.kda_gate(g_raw.view(T, Hl, K), self.A_log, self.dt_bias, cfg.safe_gate, cfg.lower_bound)
        o, final = ops.kda(q, k, v, g, beta, scale=1.0, initial_state=initial_state, cu_seqlens=cu_seqlens,
                           use_qk_l2norm=False, mode=mode, skip_saved=cfg.kda_skip_aqk_akk_saved)
        o = ops.gated_rmsnorm(o, gate.view(T, Hl, Vd), self.o_norm_weight, cfg.rms_norm_eps)
        out = row_linear_sp(o.reshape(T, Hl * Vd), self.o_proj_weight)       # [T/w, D]
        return out, final


def _kda_split_hook(module, state_dict, prefix, local_metadata):
    """Emit the reference's separate keys instead of the fused storage."""
    w = state_dict.pop(prefix + "in_proj_weight")
    s = module.sections
    o = 0
    parts = []
    for n in s:
        parts.append(w[o:o + n]); o += n
    state_dict[prefix + "qkv_proj.weight"] = torch.cat(parts[:3], 0)
    state_dict[prefix + "fg_first.weight"] = parts[3]
    state_dict[prefix + "b_proj.weight"] = parts[4]
    for nm in ("f_proj1", "g_proj1", "o_proj", "o_norm", "q_conv1d", "k_conv1d", "v_conv1d"):
        k = prefix + nm + "_weight"
        if k in state_dict:
            state_dict[prefix + nm + ".weight"] = state_dict.pop(k)
    if prefix + "g_proj1_bias" in state_dict:
        state_dict[prefix + "g_proj1.bias"] = state_dict.pop(prefix + "g_proj1_bias")


def _kda_fuse_hook(module, state_dict, prefix, *args):
    if prefix + "qkv_proj.weight" in state_dict:
        qkv = state_dict.pop(prefix + "qkv_proj.weight")
        fg = state_dict.pop(prefix + "fg_first.weight")
        b = state_dict.pop(prefix + "b_proj.weight")
        n_pad = module.in_proj_weight.shape[0]
        fused = torch.zeros(n_pad, qkv.shape[1], dtype=qkv.dtype, device=qkv.device)
        fused[:module.n_real] = torch.cat([qkv, fg, b], 0)
        state_dict[prefix + "in_proj_weight"] = fused
    for nm in ("f_proj1", "g_proj1", "o_proj", "o_norm", "q_conv1d", "k_conv1d", "v_conv1d"):
        k = prefix + nm + ".weight"
        if k in state_dict:
            state_dict[prefix + nm + "_weight"] = state_dict.pop(k)
    if prefix + "g_proj1.bias" in state_dict:
        state_dict[prefix + "g_proj1_bias"] = state_dict.pop(prefix + "g_proj1.bias")


# =============================================================================================== full attention
class FullAttention(nn.Module):
    """Causal softmax attention with RoPE, head-parallel over the gathered sequence."""

    def __init__(self, cfg: HippoConfig, layer_idx: int, seed: int, device, dtype):
        super().__init__()
        m = get_mesh()
        w, r = m.tp, m.tp_rank
        self.cfg = cfg
        D, H, dh = cfg.hidden_size, cfg.num_heads, cfg.head_dim
        self.Hl = H // w
        pre = f"layers.{layer_idx}.attn."
        parts = [_shard_rows(_xavier(pre + n, (H * dh, D), seed), r, w) for n in ("q", "k", "v")]
        self.qkv_proj_weight = _mark(nn.Parameter(torch.cat(parts, 0).to(device=device, dtype=dtype)), "muon",
                                     tp_shard_dim=0)
        self.o_proj_weight = _mark(nn.Parameter(_shard_cols(
            _xavier(pre + "o_proj", (D, H * dh), seed), r, w).contiguous().to(device=device, dtype=dtype)), "muon",
            tp_shard_dim=1)
        self._register_state_dict_hook(_attn_names_out)
        self._register_load_state_dict_pre_hook(_attn_names_in, with_module=True)

    def forward(self, h, cu_seqlens, positions, cache: Optional[dict] = None):
        """``cache`` (inference with incremental decoding): ``{"k", "v"}`` buffers ``[sequences, capacity, Hl, dh]`` holding
        the rotated keys and the values of the ``cache["lens"][n]`` tokens seen so far of every sequence. The packed
        prompts fill them and run the regular varlen causal kernel; a step with one token per sequence appends each
        key / value and attends over that sequence's rows."""
        cfg = self.cfg
        dh, Hl = cfg.head_dim, self.Hl
        qkv = column_linear_sp(h, self.qkv_proj_weight)
        T = qkv.shape[0]
        q, k, v = (t.reshape(T, Hl, dh) for t in qkv.split(Hl * dh, dim=1))
        q, k = ops.rope(q, k, positions, cfg.rope_theta)
        if cache is not None:
            lens = cache["lens"]                                              # host list: tokens cached per sequence
            N = len(lens)
            if T == N and any(lens):
                # one new token per sequence: append its key / value, attend over the sequence's own rows
                idx = torch.tensor(lens, device=q.device)
                rows = torch.arange(N, device=q.device)
                cache["k"][rows, idx] = k
                cache["v"][rows, idx] = v
                cache["lens"] = [l + 1 for l in lens]
                o = ops.attention_decode(q, cache["k"], cache["v"], dh ** -0.5, lens=cache["lens"])
                return row_linear_sp(o.reshape(T, Hl * dh), self.o_proj_weight)
            assert not any(lens), "the cache takes whole prompts first, then one token per sequence and step"
            cu_l = cu_seqlens.tolist()
            for n in range(N):
                ln = cu_l[n + 1] - cu_l[n]
                cache["k"][n, :ln] = k[cu_l[n]:cu_l[n + 1]]
                cache["v"][n, :ln] = v[cu_l[n]:cu_l[n + 1]]
            cache["lens"] = [cu_l[n + 1] - cu_l[n] for n in range(N)]
        o = ops.causal_attention(q, k, v, cu_seqlens, dh ** -0.5)
        return row_linear_sp(o.reshape(T, Hl * dh), self.o_proj_weight)


def _attn_names_out(module, sd, prefix, local_metadata):
    for nm in ("qkv_proj", "o_proj"):
        sd[prefix + nm + ".weight"] = sd.pop(prefix + nm + "_weight")


def _attn_names_in(module, sd, prefix, *args):
    for nm in ("qkv_proj", "o_proj"):
        if prefix + nm + ".weight" in sd:
            sd[prefix + nm + "_weight"] = sd.pop(prefix + nm + ".weight")


# =============================================================================================== FFN
class SwiGLU(nn.Module):
    """down(silu(gate(x)) * up(x)); gate and up fused as one column-parallel ``[2I/w, D]`` weight
    (first half gate, second half up), row-parallel down (``src/models/tp_model/swiglu.py:33-106``)."""

    def __init__(self, cfg: HippoConfig, layer_idx: int, seed: int, device, dtype):
        super().__init__()
        m = get_mesh()
        w, r = m.tp, m.tp_rank
        D, I = cfg.hidden_size, cfg.intermediate_size
        assert I % w == 0
        pre = f"layers.{layer_idx}.ffn."
        gate = _shard_rows(_xavier(pre + "gate", (I, D), seed), r, w)
        up = _shard_rows(_xavier(pre + "up", (I, D), seed), r, w)
        down = _shard_cols(_xavier(pre + "down", (D, I), seed), r, w).contiguous()
        self.nvfp4 = cfg.ffn_nvfp4
        if self.nvfp4:
            nm = cfg.ffn_nvfp4_no_bf16_master
            self.gate_up_proj = NVFP4Linear(D, 2 * I // w, nm, device, dtype, init_weight=torch.cat([gate, up], 0))
            self.down_proj = NVFP4Linear(I // w, D, nm, device, dtype, init_weight=down)
            self.gate_up_proj.tp_shard_dim, self.down_proj.tp_shard_dim = 0, 1
            self.gate_up_proj.fp4_backward = self.down_proj.fp4_backward = cfg.ffn_nvfp4_backward in ("fp4", "fp4_dx")
            self.gate_up_proj.fp4_backward_dw = self.down_proj.fp4_backward_dw = cfg.ffn_nvfp4_backward == "fp4"
            if not nm:
                self.gate_up_proj.weight.tp_shard_dim, self.down_proj.weight.tp_shard_dim = 0, 1
        else:
            self.gate_up_proj = nn.Module()
            self.gate_up_proj.weight = _mark(nn.Parameter(torch.cat([gate, up], 0).to(device=device, dtype=dtype)),
                                             "muon", tp_shard_dim=0)
            self.down_proj = nn.Module()
            self.down_proj.weight = _mark(nn.Parameter(down.to(device=device, dtype=dtype)), "muon", tp_shard_dim=1)

    def forward(self, h):
        if self.nvfp4:
            gu = nvfp4_column_linear_sp(h, self.gate_up_proj)
            return nvfp4_row_linear_sp(ops.swiglu(gu), self.down_proj)
        gu = column_linear_sp(h, self.gate_up_proj.weight)
        return row_linear_sp(ops.swiglu(gu), self.down_proj.weight)


# =============================================================================================== layer
class HybridLayer(nn.Module):
    def __init__(self, cfg: HippoConfig, layer_idx: int, kind: str, seed: int, device, dtype):
        super().__init__()
        self.kind = kind
        self.attn_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, device, dtype)
        self.attn = (KDAAttention if kind == "kda" else FullAttention)(cfg, layer_idx, seed, device, dtype)
        self.ffn_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, device, dtype)
        self.ffn = SwiGLU(cfg, layer_idx, seed, device, dtype)

    def forward(self, x, cu_seqlens, positions, initial_state, cache: Optional[dict] = None):
        h = self.attn_norm(x)
        if self.kind == "kda":
            o, final = self.attn(h, cu_seqlens, initial_state, cache)
        else:
            o, final = self.attn(h, cu_seqlens, positions, cache), None
        x, h2 = ops.add_rmsnorm(x, o, self.ffn_norm.weight, self.ffn_norm.eps)     # x + o and its norm in one pass
        x = x + self.ffn(h2)
        return x, final


# =============================================================================================== AttnRes
class BlockAttnRes(nn.Module):
    """Softmax mix over all earlier block outputs with a zero-initialised per-head pseudo-query.
    Under sequence parallelism every rank mixes its own tokens over all heads, so the reference's
    head all-gather (``src/models/ops/attn_res.py:115-118``) disappears."""

    def __init__(self, cfg: HippoConfig, device, dtype):
        super().__init__()
        H = cfg.attn_res_heads or cfg.num_heads
        self.query = _mark(nn.Parameter(torch.zeros(H, cfg.hidden_size // H, device=device, dtype=dtype)),
                           "adamw", True)
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, device, dtype)
        self.eps = cfg.rms_norm_eps

    def forward(self, blocks: List[torch.Tensor]) -> torch.Tensor:
        return ops.attn_res(blocks, self.query, self.norm.weight, self.eps)


# =============================================================================================== embed / head
class _VocabParallelEmbed(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight, v0):
        m = get_mesh()
        Vl = weight.shape[0]
        local = ids - v0
        mask = (local >= 0) & (local < Vl)
        rows = weight[local.clamp(0, Vl - 1)] * mask.unsqueeze(-1).to(weight.dtype)
        ctx.save_for_backward(local, mask)
        ctx.Vl = Vl
        return reduce_scatter_dim0(rows, m.tp_group, m.tp)

    @staticmethod
    def backward(ctx, g):
        m = get_mesh()
        local, mask = ctx.saved_tensors
        gg = all_gather_dim0(g.contiguous(), m.tp_group, m.tp)
        dw = torch.zeros(ctx.Vl, gg.shape[1], dtype=torch.float32, device=gg.device)
        sel = mask.nonzero(as_tuple=True)[0]
        dw.index_add_(0, local[sel], gg[sel].float())
        return None, dw.to(g.dtype), None


class _PeerEmbed(torch.autograd.Function):
    """CUDA path: rows of this rank's token shard gathered from the owning ranks' weight mirrors by one kernel
    (``csrc/embed.cu``); the weight gradient pulls the output-gradient rows it needs from the peers' gradient mirrors."""

    @staticmethod
    def forward(ctx, ids, weight, module):
        from ..ops import embed_cuda
        m = get_mesh()
        T = ids.numel()
        n = T // m.tp
        mine = ids[m.tp_rank * n:(m.tp_rank + 1) * n]
        ctx.module, ctx.T = module, T
        ctx.save_for_backward(ids)
        return embed_cuda.gather(mine, module.weight_ptrs(), module.Vl, weight.shape[1])

    @staticmethod
    def backward(ctx, g):
        from ..ops import embed_cuda
        (ids,) = ctx.saved_tensors
        mod, m = ctx.module, get_mesh()
        g = g.to(torch.bfloat16).contiguous()
        dw = embed_cuda.grad(ids, mod.grad_ptrs(g), ctx.T // m.tp, mod.v0, mod.Vl, g.shape[1])
        return None, dw.to(mod.weight.dtype), None


class VocabParallelEmbedding(nn.Module):
    """[V/w, D] shard. CUDA: one gather kernel reads the rows of the rank's own [T/w] token shard from the rank that owns
    each vocabulary row (peer loads from a symmetric mirror of the weight shards, refreshed after every optimizer step);
    CPU / no peer access: lookup of all T tokens, masked, reduce-scattered to the [T/w, D] token shard
    (``src/models/tp_model/embed.py:23-169`` all-reduces instead)."""

    def __init__(self, cfg: HippoConfig, seed: int, device, dtype):
        super().__init__()
        m = get_mesh()
        assert cfg.vocab_size % m.tp == 0, "vocab_size must be divisible by tp"
        self.Vl = cfg.vocab_size // m.tp
        self.v0 = m.tp_rank * self.Vl
        full = _normal("embed_tokens", (cfg.vocab_size, cfg.hidden_size), seed, 0.02)
        self.weight = _mark(nn.Parameter(full[self.v0:self.v0 + self.Vl].to(device=device, dtype=dtype)), "adamw")
        self._mirror = None          # SymmetricMirror of the weight shard (TP > 1 on CUDA)
        self._gmirror = None         # SymmetricMirror (two parities) of the output-gradient shard
        self._dirty = True           # weight changed since the mirror was published
        self._gpar = 0

    def weights_changed(self) -> None:
        """Called after every optimizer step / checkpoint load: the peer-readable mirror is re-published on next use."""
        self._dirty = True

    def _load_from_state_dict(self, *args, **kwargs):
        super()._load_from_state_dict(*args, **kwargs)
        self._dirty = True

    def _peer_path(self, ids) -> bool:
        m = get_mesh()
        return (ids.is_cuda and self.weight.dtype == torch.bfloat16 and self.weight.shape[1] % 8 == 0
                and ids.numel() % m.tp == 0 and os.environ.get("HIPPO_PEER_EMBED", "1") != "0")

    def weight_ptrs(self) -> List[int]:
        m = get_mesh()
        if m.tp == 1:
            return [self.weight.data_ptr()]
        if self._mirror is None:
            from ..parallel.symm import SymmetricMirror
            self._mirror = SymmetricMirror(m, self.weight.numel() * 2)
        if self._dirty:
            self._mirror.publish(self.weight.detach())
            self._dirty = False
        return self._mirror.ptrs()

    def grad_ptrs(self, g: torch.Tensor) -> List[int]:
        m = get_mesh()
        if m.tp == 1:
            return [g.data_ptr()]
        nbytes = g.numel() * 2
        if self._gmirror is None or self._gmirror.nbytes < nbytes:
            from ..parallel.symm import SymmetricMirror
            self._gmirror = SymmetricMirror(m, nbytes, parities=2)
        self._gpar ^= 1
        self._gmirror.publish(g, self._gpar)
        return self._gmirror.ptrs(self._gpar)

    def forward(self, ids):
        if self._peer_path(ids):
            return _PeerEmbed.apply(ids, self.weight, self)
        return _VocabParallelEmbed.apply(ids, self.weight, self.v0)


class _VocabParallelLCE(torch.autograd.Function):
    """Fused linear + cross entropy over a vocab-sharded head. Loss, dx and dW are all produced in
    forward, chunked over tokens so ``[T, V]`` logits never exist
    (``fla/modules/fused_linear_cross_entropy.py:516-679``). x arrives as the SP token shard."""

    @staticmethod
    def forward(ctx, x_shard, weight, targets, v0, num_chunks, n_valid_total, epilogue_stats=False):
        m = get_mesh()
        x = all_gather_dim0(x_shard, m.tp_group, m.tp)                  # [T, D]
        T, D = x.shape
        Vl = weight.shape[0]
        local_t = targets - v0
        own = (local_t >= 0) & (local_t < Vl) & (targets >= 0)
        local_t = torch.where(own, local_t, torch.full_like(local_t, -1))
        valid = targets >= 0
        nv = float(n_valid_total)
        dx = torch.empty_like(x)
        dw = torch.zeros(Vl, D, dtype=torch.float32, device=x.device)
        loss_sum = torch.zeros((), dtype=torch.float32, device=x.device)
        loss_sum_raw = torch.zeros(1, dtype=torch.float32, device=x.device)     # filled by the fused CE kernels
        _cuda_ops = None
        if x.is_cuda:
            from ..ops import cuda_ops as _cuda_ops
        # statistics in the logits GEMM epilogue: bf16 logits, overwritten by their gradient (CUDA, 16-byte aligned rows)
        epi = bool(epilogue_stats) and x.is_cuda and _cuda_ops.lce_epilogue_supported(x, weight)
        def chunk_rows(bytes_per_logit):
            if num_chunks > 0:
                return max(1, (T + num_chunks - 1) // num_chunks)
            # automatic: the largest chunk whose logits tile [cs, V/w] (fp32, or bf16 on the epilogue path) stays near
            # 2 GiB. Bigger chunks mean fewer read-modify-write passes over the fp32 dW accumulator and deeper
            # (K = cs) dW GEMMs.
            return min(max(1024, ((1 << 31) // (bytes_per_logit * Vl)) // 128 * 128), T)

        cs = chunk_rows(2 if epi else 4)
        ws = None
        if m.tp > 1 and x.is_cuda:
            from ..parallel import fused as _fused
            ws = _fused.workspace()
            if ws is not None and min(cs, T) > ws.lce_rows:
                ws = None
        if epi and m.tp > 1 and ws is None:
            # the cross-rank merge of the epilogue path lives in the workspace kernels
            epi, cs = False, chunk_rows(4)
        for s in range(0, T, cs):
            e = min(T, s + cs)
            xc = x[s:e]
            if epi:
                # logits GEMM whose epilogue emits per-tile (max, sum exp) and the target logit; one small merge kernel
                # (which also carries the statistics to the other ranks), then the gradient in place over the logits
                z, part, tz, tg = _cuda_ops.lce_logits_stats(xc, weight, local_t[s:e])
                roww = valid[s:e].float() / nv
                if ws is not None:
                    pz = ws.lce_grad_inplace(ws.lce_part_push(part, tz, tg), z, roww, loss_sum_raw)
                else:
                    pz = _cuda_ops.lce_grad_inplace_local(z, part, tz, tg, roww, loss_sum_raw)
                dx[s:e] = ops.gemm_nn(pz, weight)
                ops.gemm_tn_accumulate(pz, xc, dw)
                continue
            if ws is not None:
                # cross-rank max / sum-exp merge inside the kernels: statistics go to every rank by peer stores,
                # the gradient kernel waits for all sources; no collective call per chunk
                z = _cuda_ops.gemm_nt(xc, weight, out_dtype=torch.float32)
                handle = ws.lce_stats_push(z, local_t[s:e])
                pz = ws.lce_grad_merge(handle, z, valid[s:e].float() / nv, loss_sum_raw)
                dx[s:e] = ops.gemm_nn(pz, weight)
                ops.gemm_tn_accumulate(pz, xc, dw)
                continue
            z, mx, se, tz = ops.lce_chunk_stats(xc, weight, local_t[s:e])
            if m.tp > 1:
                gmx = mx.clone()
                dist.all_reduce(gmx, op=dist.ReduceOp.MAX, group=m.tp_group)
                se = se * (mx - gmx).exp()
                pack = torch.stack([se, tz], 0)
                dist.all_reduce(pack, group=m.tp_group)
                se, tz, mx = pack[0], pack[1], gmx
            lse = mx + se.log()
            vc = valid[s:e]
            loss_sum += torch.where(vc, lse - tz, torch.zeros_like(lse)).sum()
            # dz = (softmax - onehot)/n_valid on valid rows
            lt = local_t[s:e]
            pz = ops.lce_chunk_grad(z, lse, lt, vc.float() / nv).to(x.dtype)
            dx[s:e] = ops.gemm_nn(pz, weight)
            ops.gemm_tn_accumulate(pz, xc, dw)
        dx_shard = reduce_scatter_dim0(dx, m.tp_group, m.tp)
        ctx.save_for_backward(dx_shard, dw.to(weight.dtype))
        return (loss_sum + loss_sum_raw[0]) / nv

    @staticmethod
    def backward(ctx, do):
        dx, dw = ctx.saved_tensors
        return dx * do.to(dx.dtype), dw * do.to(dw.dtype), None, None, None, None, None


class LMHeadLoss(nn.Module):
    def __init__(self, cfg: HippoConfig, embed: VocabParallelEmbedding, seed: int, device, dtype):
        super().__init__()
        m = get_mesh()
        self.cfg = cfg
        self.Vl = cfg.vocab_size // m.tp
        self.v0 = m.tp_rank * self.Vl
        self.tied = cfg.tie_word_embeddings
        if self.tied:
            self._embed = [embed]          # not registered: the tied weight lives on the embedding
        else:
            full = _normal("lm_head", (cfg.vocab_size, cfg.hidden_size), seed, 0.02)
            self.weight = _mark(nn.Parameter(full[self.v0:self.v0 + self.Vl].to(device=device, dtype=dtype)), "adamw")

    def head_weight(self):
        return self._embed[0].weight if self.tied else self.weight

    def loss(self, x_shard, targets, n_valid_total):
        return _VocabParallelLCE.apply(x_shard, self.head_weight(), targets, self.v0,
                                       self.cfg.lce_num_chunks, n_valid_total, self.cfg.lce_epilogue_stats)

    def logits(self, x_shard, rows: Optional[torch.Tensor] = None):
        """Inference: full-vocab logits for the gathered tokens (gathers vocab shards). ``rows``: only these token rows
        of the gathered sequence (decoding needs the last token of every prompt, not ``[tokens, vocab]`` logits)."""
        m = get_mesh()
        x = gather_seq(x_shard)
        if rows is not None:
            x = x[rows]
        z = ops.gemm_nt(x.contiguous(), self.head_weight())
        if m.tp == 1:
            return z
        zs = all_gather_dim0(z.t().contiguous(), m.tp_group, m.tp)       # [V, T]
        return zs.t()


# =============================================================================================== model
def shift_targets(labels: torch.Tensor, row_len: Optional[int] = None) -> torch.Tensor:
    """targets[t] = labels[t+1]; the last token of every row (and of the stream) has no target."""
    t = torch.full_like(labels, -100)
    t[:-1] = labels[1:]
    if row_len is not None and row_len > 0:
        t[row_len - 1::row_len] = -100
    return t


class HippoModel(nn.Module):
    """forward(input_ids[T], labels[T], cu_seqlens[N+1], kda_states) -> {loss | logits, kda_states}.

    ``input_ids`` may also be ``[B, S]``; it is flattened and ``cu_seqlens`` defaults to row ends.
    ``n_valid_total`` lets a caller weight a micro-batch loss by the step's total valid tokens
    (sum over micro-batches then equals the full-step mean, ``loop/run.py:207-263``).
    """

    def __init__(self, cfg: HippoConfig, device=None, dtype=torch.float32, seed: int = 0):
        super().__init__()
        self.cfg = cfg
        self.mesh = get_mesh()
        device = device if device is not None else torch.device("cpu")
        _INIT_DEVICE[0] = torch.device(device)
        self.embed_tokens = VocabParallelEmbedding(cfg, seed, device, dtype)
        kinds = cfg.layer_types()
        self.layers = nn.ModuleList([HybridLayer(cfg, i, kinds[i], seed, device, dtype)
                                     for i in range(cfg.num_layers)])
        self.attn_res = BlockAttnRes(cfg, device, dtype) if cfg.num_blocks > 1 else None
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, device, dtype)
        self.lm_head = LMHeadLoss(cfg, self.embed_tokens, seed, device, dtype)
        self.kda_layer_ids = [i for i, k in enumerate(kinds) if k == "kda"]

    # ---- parameter views used by the optimizers / grad sync
    def after_optimizer_step(self) -> None:
        """Hook for whoever writes the parameters in place (optimizer kernels, weight surgery): derived copies are stale."""
        self.embed_tokens.weights_changed()

    def replicated_parameters(self):
        return [p for p in self.parameters() if getattr(p, "tp_replicated", False)]

    def partially_replicated_parameters(self):
        return [p for p in self.parameters() if getattr(p, "tp_replicated_rows", None) is not None]

    def sync_replicated_grads(self):
        m = self.mesh
        if m.tp == 1:
            return
        grads = [p.grad for p in self.replicated_parameters() if p.grad is not None]
        grads += [p.grad[p.tp_replicated_rows[0]:p.tp_replicated_rows[1]]
                  for p in self.partially_replicated_parameters() if p.grad is not None]
        if not grads:
            return
        flat = torch.cat([g.reshape(-1).float() for g in grads])
        all_reduce_sum(flat, m.tp_group, m.tp)
        off = 0
        for g in grads:
            n = g.numel()
            g.copy_(flat[off:off + n].view_as(g)); off += n

    def num_parameters(self) -> int:
        n = sum(p.numel() for p in self.parameters())
        n += sum(mod.numel_logical() for mod in self.modules()
                 if isinstance(mod, NVFP4Linear) and mod.no_master)
        return n

    def hidden(self, input_ids, cu_seqlens=None, kda_states=None, caches: Optional[List[dict]] = None,
               position_offset: int = 0):
        """``caches`` / ``position_offset``: incremental decoding (see ``generate_batch``): one dict per layer, and the
        number of tokens that came before ``input_ids`` in their sequence (an int, or one value per token)."""
        cfg, m = self.cfg, self.mesh
        if input_ids.dim() == 2:
            B, S = input_ids.shape
            if cu_seqlens is None:
                cu_seqlens = torch.arange(0, (B + 1) * S, S, device=input_ids.device, dtype=torch.int32)
            input_ids = input_ids.reshape(-1)
        T = input_ids.shape[0]
        if cu_seqlens is None:
            cu_seqlens = torch.tensor([0, T], device=input_ids.device, dtype=torch.int32)
        assert T % m.tp == 0, f"token count {T} must be divisible by tp {m.tp}"
        positions = positions_from_cu(cu_seqlens, T, input_ids.device)
        if isinstance(position_offset, torch.Tensor) or position_offset:
            positions = positions + position_offset
        x = self.embed_tokens(input_ids)
        blocks = [x]
        finals: List[Optional[torch.Tensor]] = []
        ki = 0
        for b in range(cfg.num_blocks):
            if b > 0:
                x = self.attn_res(blocks)
            for li in range(b * cfg.block_size, (b + 1) * cfg.block_size):
                layer = self.layers[li]
                init = None
                if layer.kind == "kda":
                    init = kda_states[ki] if kda_states is not None else None
                    ki += 1
                if cfg.gradient_checkpointing and self.training and li != cfg.num_layers - 1:
                    x, fin = _ckpt(layer, x, cu_seqlens, positions, init, use_reentrant=False)
                else:
                    x, fin = layer(x, cu_seqlens, positions, init, caches[li] if caches is not None else None)
                if layer.kind == "kda":
                    finals.append(fin)
            blocks.append(x)
        return self.norm(x), finals

    def forward(self, input_ids, labels=None, cu_seqlens=None, kda_states=None,
                n_valid_total: Optional[float] = None) -> Dict[str, object]:
        row_len = input_ids.shape[1] if input_ids.dim() == 2 else None
        h, finals = self.hidden(input_ids, cu_seqlens, kda_states)
        out: Dict[str, object] = {"kda_states": finals}
        if labels is not None:
            targets = shift_targets(labels.reshape(-1), row_len)
            if n_valid_total is None:
                n_valid_total = float((targets >= 0).sum().clamp(min=1))
            out["loss"] = self.lm_head.loss(h, targets, n_valid_total)
            out["n_valid"] = (targets >= 0).sum()
        else:
            out["logits"] = self.lm_head.logits(h)
        return out

    def _sample(self, logits, temperature: float, top_k: int, top_p: float = 1.0):
        """Greedy for temperature <= 0; else temperature, then top-k, then nucleus (top-p) filtering, then one draw."""
        if temperature <= 0:
            return logits.argmax()
        logits = logits / temperature
        if top_k > 0:
            kth = logits.topk(min(top_k, logits.numel())).values[-1]
            logits = logits.masked_fill(logits < kth, float("-inf"))
        if 0.0 < top_p < 1.0:
            sl, si = logits.sort(descending=True)
            cum = sl.softmax(-1).cumsum(-1)
            drop = cum - sl.softmax(-1) >= top_p                 # tokens that start beyond the nucleus; the first one stays
            logits = logits.masked_fill(torch.zeros_like(drop).scatter(0, si, drop), float("-inf"))
        return torch.multinomial(logits.softmax(-1), 1)[0]

    def new_decode_caches(self, capacity: int, n_seq: int = 1) -> List[dict]:
        """Empty per-layer caches for ``n_seq`` sequences of at most ``capacity`` tokens each (keys / values of the
        full-attention layers, convolution tails of the KDA layers; the KDA states travel outside, in the list that
        ``hidden`` returns)."""
        cfg = self.cfg
        dev, dt = self.norm.weight.device, self.norm.weight.dtype
        caches: List[dict] = []
        for layer in self.layers:
            if layer.kind == "kda":
                caches.append({})
            else:
                Hl = layer.attn.Hl
                caches.append({"k": torch.empty(n_seq, capacity, Hl, cfg.head_dim, device=dev, dtype=dt),
                               "v": torch.empty(n_seq, capacity, Hl, cfg.head_dim, device=dev, dtype=dt),
                               "lens": [0] * n_seq})
        return caches

    @torch.no_grad()
    def generate_batch(self, prompts: List[torch.Tensor], max_new_tokens, temperature=0.0, top_k=0,
                       eos_token_id: Optional[int] = None, top_p=1.0) -> List[torch.Tensor]:
        """Incremental decoding of several sequences at once. The prompts run as one packed varlen stream through the
        chunked kernels and leave, per layer, the KDA state of every sequence, its short-convolution tail and the keys /
        values of the full-attention layers; every further step feeds one token per sequence (token-recurrent KDA on the
        carried states, one query per sequence against its cached keys / values), so a step costs one pass over the
        weights for the whole batch. ``max_new_tokens``, ``temperature``, ``top_k`` and ``top_p`` are one value or one per
        sequence.
        A sequence that is done (its limit, or ``eos_token_id``) keeps its slot until the others finish; its further
        tokens are discarded.

        Under tensor parallelism (every rank of the group calls this with the same arguments) the token count of each
        pass must split evenly into sequence-parallel shards: dummy one-token sequences fill the batch up to a multiple
        of tp and one of them is lengthened so that the packed prompts do too; the sampled tokens are taken from the
        first rank of the group, so all ranks decode the same text."""
        m = self.mesh
        w = m.tp
        n_real = len(prompts)
        if n_real == 0:
            return []
        per = lambda v: list(v) if isinstance(v, (list, tuple)) else [v] * n_real   # noqa: E731
        limits, temps, topks, topps = per(max_new_tokens), per(temperature), per(top_k), per(top_p)
        seqs = [p.reshape(-1).clone() for p in prompts]
        assert all(s.numel() > 0 for s in seqs), "every prompt needs at least one token"
        dev = seqs[0].device
        done = [lim <= 0 for lim in limits]
        if all(done):
            return seqs
        steps = max(limits)
        if w > 1:
            n_dummy = (-n_real) % w
            total = sum(s.numel() for s in seqs)
            if (total + n_dummy) % w and n_dummy == 0:
                n_dummy = w
            for i in range(n_dummy):
                extra = (-(total + n_dummy)) % w if i == 0 else 0
                seqs.append(torch.zeros(1 + extra, dtype=seqs[0].dtype, device=dev))
            limits, temps, topks, done = limits + [0] * n_dummy, temps + [0.0] * n_dummy, topks + [0] * n_dummy, \
                done + [True] * n_dummy
            topps = topps + [1.0] * n_dummy
        N = len(seqs)
        lens = [s.numel() for s in seqs]
        caches = self.new_decode_caches(max(lens) + steps, N)
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0).tolist()), device=dev, dtype=torch.int32)
        h, states = self.hidden(torch.cat(seqs), cu_seqlens=cu, caches=caches)
        logits = self.lm_head.logits(h, rows=(cu[1:] - 1).long()).float()                  # [N, V]
        cu1 = torch.arange(0, N + 1, device=dev, dtype=torch.int32)
        for step in range(steps):
            nxt = torch.stack([self._sample(logits[n], temps[n], topks[n], topps[n]) for n in range(N)])
            if w > 1:
                dist.broadcast(nxt, src=m.tp_ranks()[0], group=m.tp_group)
            picked = nxt.tolist()
            for n in range(N):
                if done[n]:
                    continue
                seqs[n] = torch.cat([seqs[n], nxt[n].reshape(1)])
                if (eos_token_id is not None and picked[n] == eos_token_id) or step + 1 >= limits[n]:
                    done[n] = True
            if all(done):
                break
            pos = torch.tensor([l + step for l in lens], device=dev)
            h, states = self.hidden(nxt, cu_seqlens=cu1, kda_states=states, caches=caches, position_offset=pos)
            logits = self.lm_head.logits(h).float()
        return seqs[:n_real]

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int, temperature: float = 0.0,
                 top_k: int = 0, eos_token_id: Optional[int] = None, use_cache: bool = True,
                 top_p: float = 1.0) -> torch.Tensor:
        """Greedy / top-k sampling.

        ``use_cache`` (default): incremental decoding (``generate_batch`` with one sequence): the prompt runs once, every
        further token is a one-token step on the carried KDA states and the cached keys / values, so a new token costs one
        pass over the weights instead of a pass over the whole sequence. ``use_cache=False`` re-runs the full forward for
        every token as the reference does (``src/models/model.py:180-219``), with the prompt padded to a multiple of tp."""
        ids = input_ids.reshape(-1).clone()
        w = self.mesh.tp
        if use_cache and max_new_tokens > 0 and ids.numel() > 0:
            return self.generate_batch([ids], max_new_tokens, temperature, top_k, eos_token_id, top_p)[0]
        for _ in range(max_new_tokens):
            T = ids.numel()
            Tp = _pad_to(T, w)
            padded = torch.cat([ids, ids.new_zeros(Tp - T)]) if Tp > T else ids
            cu = torch.tensor([0, Tp], device=ids.device, dtype=torch.int32)
            logits = self.forward(padded, cu_seqlens=cu)["logits"][T - 1].float()
            nxt = self._sample(logits, temperature, top_k, top_p)
            if w > 1:
                dist.broadcast(nxt, src=self.mesh.tp_ranks()[0], group=self.mesh.tp_group)
            ids = torch.cat([ids, nxt.reshape(1)])
            if eos_token_id is not None and int(nxt) == eos_token_id:
                break
        return ids
