"""Pure-PyTorch oracles for every non-KDA op (CPU execution path + test references)."""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.nn.functional as F


# ----------------------------------------------------------------------------- norms / act
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w, fp32 math (``fla/modules/layernorm.py:194``)."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(x.dtype)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up, where gate_up = [gate | up] on the last dim (``tp_model/swiglu.py:97-106``)."""
    g, u = gate_up.float().chunk(2, dim=-1)
    return (F.silu(g) * u).to(gate_up.dtype)


# ----------------------------------------------------------------------------- rope + attention
def rope_tables(positions: torch.Tensor, dim: int, theta: float = 10000.0):
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, device=positions.device, dtype=torch.float32) / dim))
    ang = positions.float().unsqueeze(-1) * inv          # [T, dim/2]
    return ang.cos(), ang.sin()


def positions_from_cu(cu_seqlens: Optional[torch.Tensor], T: int, device) -> torch.Tensor:
    """Position of each token inside its document."""
    pos = torch.arange(T, device=device)
    if cu_seqlens is None:
        return pos
    cu = cu_seqlens.to(device)
    seq = torch.bucketize(pos, cu[1:-1], right=True)
    return pos - cu[seq]


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE (NeoX layout). x: [T, H, dh]; cos/sin: [T, dh/2]."""
    xf = x.float()
    d2 = x.shape[-1] // 2
    x1, x2 = xf[..., :d2], xf[..., d2:]
    c, s = cos.unsqueeze(1), sin.unsqueeze(1)
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1).to(x.dtype)


def causal_attention(q, k, v, cu_seqlens: Optional[torch.Tensor], scale: Optional[float] = None):
    """Varlen causal softmax attention, fp32 math. q,k,v: [T, H, dh] -> [T, H, dh]."""
    T, H, dh = q.shape
    if scale is None:
        scale = dh ** -0.5
    pos = torch.arange(T, device=q.device)
    if cu_seqlens is not None:
        seq = torch.bucketize(pos, cu_seqlens.to(q.device)[1:-1], right=True)
    else:
        seq = torch.zeros_like(pos)
    mask = (seq.unsqueeze(1) == seq.unsqueeze(0)) & (pos.unsqueeze(1) >= pos.unsqueeze(0))
    s = torch.einsum("ihd,jhd->hij", q.float(), k.float()) * scale
    s = s.masked_fill(~mask.unsqueeze(0), float("-inf"))
    p = s.softmax(-1)
    return torch.einsum("hij,jhd->ihd", p, v.float()).to(q.dtype)


# ----------------------------------------------------------------------------- block attention residual
def attn_res(sources: torch.Tensor, query: torch.Tensor, norm_weight: torch.Tensor, eps: float
             ) -> torch.Tensor:
    """Block attention residual mix (``src/models/ops/attn_res.py:238-295``).

    sources: [N, T, D]; query: [H, dh] with H*dh == D; norm_weight: [D].
    K_n = RMSNorm_D(V_n) * w; logit[n,h] = <query[h], K_n[h]>; alpha = softmax_n; out[h] = sum_n alpha V_n[h].
    """
    N, T, D = sources.shape
    H, dh = query.shape
    vf = sources.float()
    kn = vf * torch.rsqrt(vf.pow(2).mean(-1, keepdim=True) + eps) * norm_weight.float()
    logit = (kn.view(N, T, H, dh) * query.float().view(1, 1, H, dh)).sum(-1)       # [N,T,H]
    alpha = logit.softmax(0)
    out = (alpha.unsqueeze(-1) * vf.view(N, T, H, dh)).sum(0)
    return out.reshape(T, D).to(sources.dtype)


# ----------------------------------------------------------------------------- linear cross entropy
def linear_cross_entropy(x: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                         ignore_index: int = -100) -> Tuple[torch.Tensor, torch.Tensor]:
    """Mean CE of (x @ W^T) vs labels over non-ignored rows. Returns (loss, n_valid)."""
    logits = x.float() @ weight.float().t()
    n_valid = (labels != ignore_index).sum()
    loss = F.cross_entropy(logits, labels, ignore_index=ignore_index, reduction="sum")
    return loss / n_valid.clamp(min=1), n_valid


# ----------------------------------------------------------------------------- NVFP4
E2M1_LEVELS = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def _round_e2m1_rne(x: torch.Tensor) -> torch.Tensor:
    """Index (0..7) of the nearest E2M1 magnitude with ties-to-even mantissa (hardware cvt.rn)."""
    a = x.abs()
    # midpoints .25 .75 1.25 1.75 2.5 3.5 5 ; even codes are idx 0,2,4,6 -> ties go to the even index
    idx = torch.zeros_like(a, dtype=torch.int32)
    idx += (a > 0.25).int()          # tie .25 -> 0 (even)
    idx += (a >= 0.75).int()         # tie .75 -> 2 (idx1 odd -> up)
    idx += (a > 1.25).int()          # tie 1.25 -> 2 (stay)
    idx += (a >= 1.75).int()         # tie 1.75 -> 4
    idx += (a > 2.5).int()           # tie 2.5 -> 4
    idx += (a >= 3.5).int()          # tie 3.5 -> 6
    idx += (a > 5.0).int()           # tie 5 -> 6
    return idx


def nvfp4_quantize(w: torch.Tensor, global_scale: Optional[torch.Tensor] = None
                   ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Quantise [N, K] to NVFP4: packed u8 [N, K/2], e4m3 scales [N, K/16], fp32 global scale [1].

    Hardware format: 16-element blocks along K, block scale = e4m3(absmax/6/global), element code =
    RN-even E2M1 of x / (decoded_scale * global). global = max|w| / (6*448) unless given.
    Layout follows ``src/models/ops/nvfp4.py:49-140`` (nibble = sign<<3|idx, byte = even | odd<<4).
    """
    N, K = w.shape
    assert K % 16 == 0
    wf = w.float()
    if global_scale is None:
        amax = wf.abs().max()
        global_scale = torch.where(amax > 0, amax / (6.0 * 448.0), torch.ones_like(amax)).reshape(1)
    gs = global_scale.float().reshape(1)
    blk = wf.view(N, K // 16, 16)
    bmax = blk.abs().amax(-1)
    sc = (bmax / 6.0 / gs).clamp(max=448.0).to(torch.float8_e4m3fn)
    scf = sc.float() * gs
    denom = torch.where(scf > 0, scf, torch.ones_like(scf)).unsqueeze(-1)
    xs = blk / denom
    idx = _round_e2m1_rne(xs)
    code = (idx | ((xs < 0).int() << 3)).view(N, K).to(torch.uint8)
    packed = code[:, 0::2] | (code[:, 1::2] << 4)
    return packed.contiguous(), sc.contiguous(), gs


def nvfp4_quantize_stochastic(w: torch.Tensor, global_scale: torch.Tensor, generator: Optional[torch.Generator] = None
                              ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """NVFP4 quantisation for weights that have no master copy: block scales rounded UP to e4m3 (no element exceeds six
    block scales) and E2M1 codes by stochastic rounding, so that E[dequantise(quantise(w))] = w for |w| inside the
    range of ``global_scale``. Same layout as :func:`nvfp4_quantize`."""
    N, K = w.shape
    assert K % 16 == 0
    gs = global_scale.float().reshape(1)
    blk = w.float().view(N, K // 16, 16)
    want = (blk.abs().amax(-1) / 6.0 / gs).clamp(max=448.0)
    sc = want.to(torch.float8_e4m3fn)
    low = sc.float() < want
    bumped = (sc.view(torch.uint8) + low.to(torch.uint8)).clamp(max=0x7E).view(torch.float8_e4m3fn)
    sc = torch.where(low, bumped.float(), sc.float()).to(torch.float8_e4m3fn)
    scf = sc.float() * gs
    denom = torch.where(scf > 0, scf, torch.ones_like(scf)).unsqueeze(-1)
    xs = (blk / denom).clamp(-6.0, 6.0)
    ax = xs.abs()
    levels = torch.tensor(E2M1_LEVELS, dtype=torch.float32, device=w.device)
    idx = (torch.bucketize(ax, levels, right=True) - 1).clamp(0, 7)          # largest level <= |x|
    lo = levels[idx]
    hi = levels[(idx + 1).clamp(max=7)]
    p = torch.where(hi > lo, (ax - lo) / (hi - lo).clamp(min=1e-9), torch.zeros_like(ax))
    u = torch.rand(ax.shape, generator=generator, device=w.device)
    idx = (idx + (u < p).long()).clamp(max=7)
    code = (idx | ((xs < 0).long() << 3)).view(N, K).to(torch.uint8)
    packed = code[:, 0::2] | (code[:, 1::2] << 4)
    return packed.contiguous(), sc.contiguous(), gs


def nvfp4_dequantize(packed: torch.Tensor, scales: torch.Tensor, global_scale: torch.Tensor,
                     dtype=torch.float32) -> torch.Tensor:
    N, K2 = packed.shape
    lut = torch.tensor(E2M1_LEVELS + tuple(-x for x in E2M1_LEVELS), dtype=torch.float32,
                       device=packed.device)
    lo = lut[(packed & 0xF).long()]
    hi = lut[(packed >> 4).long()]
    w = torch.stack([lo, hi], -1).view(N, K2 * 2)
    s = scales.float().repeat_interleave(16, dim=1) * global_scale.float()
    return (w * s).to(dtype)


def newton_schulz5(G: torch.Tensor, steps: int = 5, eps: float = 1e-7,
                   compute_dtype=torch.float32) -> torch.Tensor:
    """Quintic Newton-Schulz orthogonalisation (``param_offload/muon.py:247-287``).

    X = G/(||G||_F+eps); steps x { S = X X^T (smaller side); X <- (aI + bS + cS^2) X }.
    """
    a, b, c = 3.4445, -4.7750, 2.0315
    X = G.to(compute_dtype)
    X = X / (X.float().norm() + eps).to(compute_dtype)
    tall = X.shape[0] > X.shape[1]
    if tall:
        X = X.t()
    for _ in range(steps):
        S = X @ X.t()
        M = b * S + c * (S @ S)
        X = a * X + M @ X
    if tall:
        X = X.t()
    return X
