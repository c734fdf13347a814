"""Device dispatch: CUDA tensors -> sm_100a extension, CPU tensors -> torch oracle."""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.nn.functional as F

from ..ref import kda as _rk
from ..ref import ops as _ro


def _cu():
    from . import cuda_ops
    return cuda_ops


def cuda_ext_loaded() -> bool:
    try:
        from . import _ext
        return _ext.is_loaded()
    except Exception:
        return False


# ----------------------------------------------------------------------------- GEMMs
def gemm_nt(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a[M,K] @ b[N,K]^T -> [M,N]."""
    if a.is_cuda:
        return _cu().gemm_nt(a, b)
    return a @ b.t()


def gemm_nn(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a[M,N] @ b[N,K] -> [M,K]."""
    if a.is_cuda:
        return _cu().gemm_nn(a, b)
    return a @ b


def gemm_tn(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a[M,N]^T @ b[M,K] -> [N,K]."""
    if a.is_cuda:
        return _cu().gemm_tn(a, b)
    return a.t() @ b


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        y = gemm_nt(x, w)
        if bias is not None:
            y = y + bias
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = gemm_nn(dy, w) if ctx.needs_input_grad[0] else None
        dw = gemm_tn(dy, x).to(w.dtype) if ctx.needs_input_grad[1] else None
        db = dy.sum(0) if ctx.has_bias else None
        return dx, dw, db


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x W^T (+ b) on 2-D x."""
    if x.is_cuda:
        return _Linear.apply(x.contiguous(), w, bias)
    return F.linear(x, w, bias)


# ----------------------------------------------------------------------------- row ops
def rmsnorm(x, weight, eps: float):
    if x.is_cuda:
        return _cu().rmsnorm(x, weight, eps)
    return _ro.rmsnorm(x, weight, eps)


def add_rmsnorm(x, res, weight, eps: float):
    """(x + res, rmsnorm(x + res) * weight): the residual add of a pre-norm layer fused into the norm behind it."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        return _cu().add_rmsnorm(x, res, weight, eps)
    s = x + res
    return s, rmsnorm(s, weight, eps)


def swiglu(gate_up):
    if gate_up.is_cuda:
        return _cu().swiglu(gate_up)
    return _ro.swiglu(gate_up)


def silu(x):
    if x.is_cuda:
        return _cu().silu(x)
    return F.silu(x)


def l2norm(x, eps: float = 1e-6):
    return _rk.l2norm(x, eps)


def gated_rmsnorm(o, gate, weight, eps: float):
    if o.is_cuda:
        return _cu().gated_rmsnorm(o, gate, weight, eps)
    return _rk.gated_rmsnorm(o, gate, weight, eps)


def short_conv_silu(x, weight, bias, cu_seqlens):
    if x.is_cuda and bias is None and weight.shape[1] <= 8:
        return _cu().short_conv_silu(x, weight, bias, cu_seqlens)
    return _rk.short_conv_silu(x, weight, bias, cu_seqlens)


# ----------------------------------------------------------------------------- KDA
def kda_prologue(proj, H: int, K: int, off_q: int, off_k: int, off_v: int, off_b: int, scale: float,
                 beta_mul: float = 1.0, apply_silu: bool = True, off_fg: int = 0, fg_w: int = 0):
    """From the fused projection ``[T, n]`` (columns q | k | v | ... | b): q = l2norm(silu(q)) * scale,
    k = l2norm(silu(k)), v = silu(v) as ``[T, H, K]`` and beta = sigmoid(b) * beta_mul as ``[T, H]`` fp32. With
    ``fg_w`` > 0 a fifth result: the ``fg_w`` columns at ``off_fg`` (inputs of the low-rank gate projections)."""
    if proj.is_cuda:
        return _cu().kda_prologue(proj, H, K, off_q, off_k, off_v, off_b, scale, beta_mul, apply_silu, off_fg, fg_w)
    T = proj.shape[0]
    act = F.silu if apply_silu else (lambda t: t)
    q = _rk.l2norm(act(proj[:, off_q:off_q + H * K]).reshape(T, H, K)) * scale
    k = _rk.l2norm(act(proj[:, off_k:off_k + H * K]).reshape(T, H, K))
    v = act(proj[:, off_v:off_v + H * K]).reshape(T, H, K)
    beta = torch.sigmoid(proj[:, off_b:off_b + H].float()) * beta_mul
    if fg_w > 0:
        return q, k, v, beta, proj[:, off_fg:off_fg + fg_w]
    return q, k, v, beta


def kda_gate(x_g, A_log, dt_bias, safe_gate: bool = False, lower_bound: float = -5.0):
    if x_g.is_cuda:
        return _cu().kda_gate(x_g, A_log, dt_bias, safe_gate, lower_bound)
    return _rk.kda_gate(x_g, A_log, dt_bias, safe_gate, lower_bound)


def kda(q, k, v, g, beta, scale=None, initial_state=None, cu_seqlens=None,
        use_qk_l2norm: bool = True, mode: str = "chunk", skip_saved: bool = False
        ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Kimi delta attention over a packed token stream; see :mod:`hippolm_b200.ref.kda`. ``skip_saved`` (CUDA): keep
    fewer activations for backward and recompute the per-chunk matrices there."""
    if q.is_cuda:
        return _cu().kda(q, k, v, g, beta, scale, initial_state, cu_seqlens, use_qk_l2norm, skip_saved, mode)
    if mode == "fused_recurrent":
        return _rk.kda_recurrent(q, k, v, g, beta, scale, initial_state, cu_seqlens, use_qk_l2norm)
    return _rk.kda_chunked(q, k, v, g, beta, scale, initial_state, cu_seqlens, use_qk_l2norm)


# ----------------------------------------------------------------------------- attention
def rope(q, k, positions, theta: float = 10000.0):
    if q.is_cuda:
        return _cu().rope(q, k, positions, theta)
    cos, sin = _ro.rope_tables(positions, q.shape[-1], theta)
    return _ro.apply_rope(q, cos, sin), _ro.apply_rope(k, cos, sin)


def causal_attention(q, k, v, cu_seqlens, scale=None):
    if q.is_cuda:
        return _cu().causal_attention(q, k, v, cu_seqlens, scale)
    return _ro.causal_attention(q, k, v, cu_seqlens, scale)


def attention_decode(q, k_cache, v_cache, scale=None, lens=None):
    """One query token per sequence against cached keys / values (the query's own key and value included).

    One sequence: q [1, H, dh], k_cache / v_cache [L, H, dh] -> [1, H, dh].
    N sequences:  q [N, H, dh], k_cache / v_cache [N, cap, H, dh], lens = valid rows of every sequence (host ints)
                  -> [N, H, dh]; each sequence is evaluated over exactly its own rows.
    Bandwidth-bound row operations in fp32 (a product and a sum per cached element), the same code on every device."""
    dh = q.shape[-1]
    if scale is None:
        scale = dh ** -0.5
    if k_cache.dim() == 4:
        return torch.cat([attention_decode(q[n:n + 1], k_cache[n, :int(lens[n])], v_cache[n, :int(lens[n])], scale)
                          for n in range(q.shape[0])], 0)
    s = (k_cache * q).sum(-1, dtype=torch.float32) * scale                  # [L, H]
    p = torch.softmax(s, dim=0)
    o = (p.unsqueeze(-1) * v_cache).sum(0, dtype=torch.float32)             # [H, dh]
    return o.unsqueeze(0).to(q.dtype)


def attn_res(sources: List[torch.Tensor], query, norm_weight, eps: float):
    """sources: list of [T, D] tensors (oldest first)."""
    if sources[0].is_cuda:
        return _cu().attn_res(sources, query, norm_weight, eps)
    return _ro.attn_res(torch.stack(sources, 0), query, norm_weight, eps)


# ----------------------------------------------------------------------------- NVFP4
def nvfp4_quantize(w, global_scale=None):
    if w.is_cuda:
        return _cu().nvfp4_quantize(w, global_scale)
    return _ro.nvfp4_quantize(w, global_scale)


def nvfp4_dequantize(packed, scales, global_scale, dtype=torch.float32):
    if packed.is_cuda:
        return _cu().nvfp4_dequantize(packed, scales, global_scale, dtype)
    return _ro.nvfp4_dequantize(packed, scales, global_scale, dtype)


def nvfp4_linear(x, packed, scales, global_scale, act_quant: bool = True, act_gs=None):
    """y = Q(x) @ dq(W)^T with block-scaled FP4 operands (fp32 accumulate). ``act_gs`` (CUDA): the tensor scale of ``x``
    if the caller has it already."""
    if x.is_cuda:
        return _cu().nvfp4_gemm_nt(x, packed, scales, global_scale, act_quant, act_gs)
    w = _ro.nvfp4_dequantize(packed, scales, global_scale, torch.float32)
    xf = x.float()
    if act_quant:
        xf = _ro.nvfp4_dequantize(*_ro.nvfp4_quantize(xf), dtype=torch.float32)
    return (xf @ w.t()).to(x.dtype)


# ----------------------------------------------------------------------------- optimizer math
def newton_schulz5(G, steps: int = 5, eps: float = 1e-7):
    if G.is_cuda:
        return _cu().newton_schulz5(G, steps, eps)
    return _ro.newton_schulz5(G, steps, eps)


def adamw_update(p, g, m, v, lr, beta1, beta2, eps, wd, step, grad_scale: float = 1.0):
    """In-place standard AdamW (both bias corrections) on one tensor."""
    if p.is_cuda:
        return _cu().adamw_update(p, g, m, v, lr, beta1, beta2, eps, wd, step, grad_scale)
    gf = g.float() * grad_scale
    mf = m.float().mul_(beta1).add_(gf, alpha=1 - beta1)
    vf = v.float().mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
    m.copy_(mf); v.copy_(vf)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    upd = (mf / bc1) / ((vf / bc2).sqrt() + eps)
    pf = p.float().mul_(1 - lr * wd).add_(upd, alpha=-lr)
    p.copy_(pf)


# ----------------------------------------------------------------------------- LCE building block
def lce_chunk_stats(x, w, targets_local):
    """For one token chunk: logits = x @ w^T (fp32), returns (logits, rowmax, sumexp, target_logit).

    targets_local: index into this rank's vocab shard, or -1 when the target lives elsewhere / ignored.
    """
    if x.is_cuda:
        return _cu().lce_chunk_stats(x, w, targets_local)
    z = x.float() @ w.float().t()
    mx = z.max(-1).values
    se = (z - mx.unsqueeze(-1)).exp().sum(-1)
    tl = targets_local.clamp(min=0)
    tz = z.gather(1, tl.unsqueeze(1)).squeeze(1)
    tz = torch.where(targets_local >= 0, tz, torch.zeros_like(tz))
    return z, mx, se, tz


def lce_chunk_grad(z, lse, targets_local, row_weight):
    """(softmax(z) - onehot(target)) * row_weight, in the GEMM input dtype."""
    if z.is_cuda:
        return _cu().lce_chunk_grad(z, lse, targets_local, row_weight)
    p = (z - lse.unsqueeze(-1)).exp()
    rows = (targets_local >= 0).nonzero(as_tuple=True)[0]
    p[rows, targets_local[rows]] -= 1.0
    return p * row_weight.unsqueeze(-1)


def gemm_tn_accumulate(a, b, out_fp32):
    """out_fp32 += a^T @ b."""
    if a.is_cuda:
        return _cu().gemm_tn_accumulate(a, b, out_fp32)
    out_fp32 += a.float().t() @ b.float()
    return out_fp32
