"""Pure-PyTorch Kimi-Delta-Attention oracles.

Two implementations of the same gated delta rule:

* :func:`kda_recurrent` -- the token-by-token recurrence, the ground truth every
  kernel is checked against (behaviour of the reference's
  ``fla/ops/kda/fused_recurrent.py:145-190``).
* :func:`kda_chunked` -- the chunk-parallel (WY) form with the same maths the
  CUDA kernels implement (behaviour of ``fla/ops/kda/chunk_fwd.py:43-135``).
  It is differentiable through autograd and is the CPU execution path.

Conventions (all token-major, batch folded into the token axis):
  q, k : [T, H, K]     v : [T, H, V]     g : [T, H, K] (log decay, <= 0)
  beta : [T, H]        cu_seqlens : int tensor [N+1] (state resets at every boundary)
  initial_state / final_state : [N, H, K, V] fp32
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """x / sqrt(sum(x^2) + eps) over the last dim (``fla/modules/l2norm.py:25``)."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + eps)).to(x.dtype)


def kda_gate(x_g: torch.Tensor, A_log: torch.Tensor, dt_bias: Optional[torch.Tensor],
             safe_gate: bool = False, lower_bound: float = -5.0) -> torch.Tensor:
    """Gate activation producing the log decay (``fla/ops/kda/gate.py:25-68``).

    x_g: [T, H, K]; A_log: [H]; dt_bias: [H*K] or None.
    plain: g = -exp(A_log) * softplus(x + b);  safe: g = lower_bound * sigmoid(exp(A_log) * (x + b)).
    """
    T, H, K = x_g.shape
    x = x_g.float()
    if dt_bias is not None:
        x = x + dt_bias.float().view(1, H, K)
    a = A_log.float().exp().view(1, H, 1)
    if safe_gate:
        return lower_bound * torch.sigmoid(a * x)
    return -a * F.softplus(x)


def _default_cu(T: int, device) -> torch.Tensor:
    return torch.tensor([0, T], dtype=torch.int64, device=device)


def kda_recurrent(q, k, v, g, beta, scale: Optional[float] = None,
                  initial_state: Optional[torch.Tensor] = None,
                  cu_seqlens: Optional[torch.Tensor] = None,
                  use_qk_l2norm: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Token-by-token oracle. Returns (o [T,H,V] in v.dtype, final_state [N,H,K,V] fp32)."""
    T, H, K = q.shape
    V = v.shape[-1]
    if scale is None:
        scale = K ** -0.5
    if use_qk_l2norm:
        q, k = l2norm(q), l2norm(k)
    cu = _default_cu(T, q.device) if cu_seqlens is None else cu_seqlens
    N = cu.numel() - 1
    qf, kf, vf, gf, bf = (t.float() for t in (q, k, v, g, beta))
    o = torch.zeros(T, H, V, dtype=torch.float32, device=q.device)
    final = torch.zeros(N, H, K, V, dtype=torch.float32, device=q.device)
    cul = cu.tolist()
    for n in range(N):
        h = (initial_state[n].float().clone() if initial_state is not None
             else torch.zeros(H, K, V, dtype=torch.float32, device=q.device))
        for t in range(cul[n], cul[n + 1]):
            h = h * gf[t].exp().unsqueeze(-1)
            vp = bf[t].unsqueeze(-1) * (vf[t] - torch.einsum("hkv,hk->hv", h, kf[t]))
            h = h + kf[t].unsqueeze(-1) * vp.unsqueeze(-2)
            o[t] = torch.einsum("hkv,hk->hv", h, qf[t] * scale)
        final[n] = h
    return o.to(v.dtype), final


def build_chunk_table(cu_seqlens: torch.Tensor, T: int, chunk: int):
    """Chunks never straddle a sequence boundary.

    Returns python lists (seq_id, start, length) per chunk in token order plus the
    per-sequence chunk counts.
    """
    cul = [int(x) for x in cu_seqlens.tolist()]
    seq_id, start, length, per_seq = [], [], [], []
    for n in range(len(cul) - 1):
        s, e = cul[n], cul[n + 1]
        c = 0
        while s < e:
            l = min(chunk, e - s)
            seq_id.append(n); start.append(s); length.append(l)
            s += l; c += 1
        per_seq.append(c)
    return seq_id, start, length, per_seq


def kda_chunked(q, k, v, g, beta, scale: Optional[float] = None,
                initial_state: Optional[torch.Tensor] = None,
                cu_seqlens: Optional[torch.Tensor] = None,
                use_qk_l2norm: bool = False, chunk: int = 64
                ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Chunk-parallel KDA in plain torch (autograd-differentiable).

    Per chunk (C tokens, inclusive local cumsum G of g):
      Akk[i,j] = beta_i * sum_c k_i k_j exp(G_i-G_j)   (j <  i)
      Aqk[i,j] = scale  * sum_c q_i k_j exp(G_i-G_j)   (j <= i)
      u = (I+Akk)^-1 (beta v),  w = (I+Akk)^-1 (beta k exp(G))
      v_new = u - w S;  o = scale (q exp(G)) S + Aqk v_new;  S <- exp(G_last) S + (k exp(G_last-G))^T v_new
    """
    T, H, K = q.shape
    V = v.shape[-1]
    dev = q.device
    if scale is None:
        scale = K ** -0.5
    if use_qk_l2norm:
        q, k = l2norm(q), l2norm(k)
    cu = _default_cu(T, dev) if cu_seqlens is None else cu_seqlens
    N = cu.numel() - 1
    seq_id, start, length, per_seq = build_chunk_table(cu, T, chunk)
    NC = len(start)
    C = chunk
    # gather index [NC, C] with padding -> T (a zero row appended)
    idx = torch.full((NC, C), T, dtype=torch.int64)
    for c, (s, l) in enumerate(zip(start, length)):
        idx[c, :l] = torch.arange(s, s + l)
    idx = idx.to(dev)

    def pad_gather(x):
        xf = x.float()
        z = torch.zeros((1,) + tuple(xf.shape[1:]), dtype=xf.dtype, device=dev)
        return torch.cat([xf, z], 0)[idx]          # [NC, C, ...]

    qc, kc, vc, gc = pad_gather(q), pad_gather(k), pad_gather(v), pad_gather(g)   # [NC,C,H,*]
    bc = pad_gather(beta)                                                          # [NC,C,H]
    G = gc.cumsum(1)                                                               # inclusive
    # pairwise decay, exact: D[i,j,c] = exp(G_i - G_j) for j<=i
    tri_incl = torch.tril(torch.ones(C, C, dtype=torch.bool, device=dev))
    tri_strict = torch.tril(torch.ones(C, C, dtype=torch.bool, device=dev), -1)
    diff = G.unsqueeze(2) - G.unsqueeze(1)                                         # [NC,C,C,H,K]
    diff = diff.masked_fill(~tri_incl.view(1, C, C, 1, 1), 0.0)
    Dm = diff.exp()
    kk = torch.einsum("nihc,njhc,nijhc->nhij", kc, kc, Dm)
    qk = torch.einsum("nihc,njhc,nijhc->nhij", qc, kc, Dm)
    bh = bc.permute(0, 2, 1)                                                       # [NC,H,C]
    Akk = (kk * bh.unsqueeze(-1)).masked_fill(~tri_strict, 0.0)
    Aqk = (qk * scale).masked_fill(~tri_incl, 0.0)
    eye = torch.eye(C, device=dev, dtype=torch.float32)
    Ainv = torch.linalg.solve_triangular(eye + Akk, eye.expand(NC, H, C, C), upper=False)
    eG = G.exp()
    bv = (vc * bc.unsqueeze(-1)).permute(0, 2, 1, 3)                               # [NC,H,C,V]
    bk = (kc * eG * bc.unsqueeze(-1)).permute(0, 2, 1, 3)                          # [NC,H,C,K]
    u = Ainv @ bv
    w = Ainv @ bk
    qg = (qc * eG).permute(0, 2, 1, 3) * scale                                     # [NC,H,C,K]
    Glast = G[:, -1]                                                               # [NC,H,K]  (padding has g=0)
    kg = (kc * (Glast.unsqueeze(1) - G).exp()).permute(0, 2, 1, 3)                 # [NC,H,C,K]
    dlast = Glast.exp()                                                            # [NC,H,K]

    # inter-chunk recurrence, batched over sequences
    o_chunks = [None] * NC
    first = [0]
    for c in per_seq:
        first.append(first[-1] + c)
    S = (initial_state.float() if initial_state is not None
         else torch.zeros(N, H, K, V, dtype=torch.float32, device=dev))
    S_list = [S[n] for n in range(N)]
    max_c = max(per_seq) if per_seq else 0
    for j in range(max_c):
        seqs = [n for n in range(N) if per_seq[n] > j]
        cids = torch.tensor([first[n] + j for n in seqs], device=dev)
        Sj = torch.stack([S_list[n] for n in seqs])                                # [ns,H,K,V]
        vn = u[cids] - w[cids] @ Sj
        oj = qg[cids] @ Sj + Aqk[cids] @ vn
        Sn = Sj * dlast[cids].unsqueeze(-1) + kg[cids].transpose(-1, -2) @ vn
        for ii, n in enumerate(seqs):
            S_list[n] = Sn[ii]
            o_chunks[first[n] + j] = oj[ii]
    final = torch.stack(S_list) if N > 0 else S
    o = torch.zeros(T + 1, H, V, dtype=torch.float32, device=dev)
    if NC > 0:
        oc = torch.stack(o_chunks).permute(0, 2, 1, 3)                             # [NC,C,H,V]
        o = o.index_put((idx.reshape(-1),), oc.reshape(NC * C, H, V), accumulate=True)
    return o[:T].to(v.dtype), final


def short_conv_silu(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                    cu_seqlens: Optional[torch.Tensor]) -> torch.Tensor:
    """Depthwise causal conv (width W) + SiLU with per-document reset.

    x: [T, D]; weight: [D, W]. Behaviour of ``fla/modules/conv/triton/kernels.py:36``.
    y[t] = silu(sum_w weight[:, w] * x[t - (W-1) + w]) with taps before the document start = 0.
    """
    T, D = x.shape
    W = weight.shape[-1]
    xf = x.float()
    pos = torch.arange(T, device=x.device)
    if cu_seqlens is not None:
        seq = torch.bucketize(pos, cu_seqlens[1:-1].to(pos.device), right=True)
        pos_in = pos - cu_seqlens.to(pos.device)[seq]
    else:
        pos_in = pos
    y = torch.zeros_like(xf)
    for wi in range(W):
        shift = W - 1 - wi
        xs = torch.roll(xf, shifts=shift, dims=0) if shift else xf
        valid = (pos_in >= shift).unsqueeze(-1)
        y = y + torch.where(valid, xs, torch.zeros_like(xs)) * weight[:, wi].float().view(1, D)
    if bias is not None:
        y = y + bias.float().view(1, D)
    return F.silu(y).to(x.dtype)


def gated_rmsnorm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Per-head RMSNorm(o) * w * sigmoid(gate) (``fla/modules/fused_norm_gate.py:992-1052``)."""
    of = o.float()
    y = of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    return (y * torch.sigmoid(gate.float())).to(o.dtype)


def kda_chunked_anchored(q, k, v, g, beta, scale: Optional[float] = None,
                         initial_state: Optional[torch.Tensor] = None,
                         cu_seqlens: Optional[torch.Tensor] = None,
                         use_qk_l2norm: bool = False, chunk: int = 64, sub: int = 16,
                         return_aux: bool = False):
    """Chunked KDA with the two-sided sub-chunk anchoring the CUDA kernels use: for a row block I
    and earlier columns j, exp(G_i - G_j) = exp(G_i - G_a) * exp(G_a - G_j) with a = last row before
    block I, so both factors are <= 1 for any decay magnitude; the diagonal 16x16 blocks are formed
    exactly. Memory is O(T*H*K), which makes this the large-shape oracle on the GPU. Differentiable."""
    T, H, K = q.shape
    V = v.shape[-1]
    dev = q.device
    if scale is None:
        scale = K ** -0.5
    if use_qk_l2norm:
        q, k = l2norm(q), l2norm(k)
    cu = _default_cu(T, dev) if cu_seqlens is None else cu_seqlens
    N = cu.numel() - 1
    seq_id, start, length, per_seq = build_chunk_table(cu, T, chunk)
    NC, C, NS = len(start), chunk, chunk // sub
    idx = torch.full((NC, C), T, dtype=torch.int64)
    for c, (s, l) in enumerate(zip(start, length)):
        idx[c, :l] = torch.arange(s, s + l)
    idx = idx.to(dev)

    def pg(x):
        xf = x.float()
        z = torch.zeros((1,) + tuple(xf.shape[1:]), dtype=xf.dtype, device=dev)
        return torch.cat([xf, z], 0)[idx].transpose(1, 2)      # [NC,H,C,...]

    qc, kc, vc, gc = pg(q) * scale, pg(k), pg(v), pg(g)           # [NC,H,C,K|V]
    bc = torch.cat([beta.float(), torch.zeros(1, H, device=dev)], 0)[idx].transpose(1, 2)   # [NC,H,C]
    G = gc.cumsum(2)
    kk = torch.zeros(NC, H, C, C, device=dev)
    qk = torch.zeros(NC, H, C, C, device=dev)
    for I in range(NS):
        r = slice(I * sub, (I + 1) * sub)
        Gi = G[:, :, r]                                           # [NC,H,sub,K]
        # exact diagonal block
        d = (Gi.unsqueeze(3) - Gi.unsqueeze(2))
        msk = torch.tril(torch.ones(sub, sub, dtype=torch.bool, device=dev)).view(1, 1, sub, sub, 1)
        e = torch.where(msk, d, torch.zeros_like(d)).exp() * msk
        kk[:, :, r, r] = torch.einsum("nhic,nhjc,nhijc->nhij", kc[:, :, r], kc[:, :, r], e)
        qk[:, :, r, r] = torch.einsum("nhic,nhjc,nhijc->nhij", qc[:, :, r], kc[:, :, r], e)
        if I > 0:
            Ga = G[:, :, I * sub - 1:I * sub]                     # anchor row
            rowf = (Gi - Ga).exp()
            cs = slice(0, I * sub)
            colk = kc[:, :, cs] * (Ga - G[:, :, cs]).exp()
            kk[:, :, r, cs] = (kc[:, :, r] * rowf) @ colk.transpose(-1, -2)
            qk[:, :, r, cs] = (qc[:, :, r] * rowf) @ colk.transpose(-1, -2)
    tri_s = torch.tril(torch.ones(C, C, dtype=torch.bool, device=dev), -1)
    tri_i = torch.tril(torch.ones(C, C, dtype=torch.bool, device=dev))
    Akk = (kk * bc.unsqueeze(-1)) * tri_s
    Aqk = qk * tri_i
    eye = torch.eye(C, device=dev)
    Ainv = torch.linalg.solve_triangular(eye + Akk, eye.expand(NC, H, C, C), upper=False)
    eG = G.exp()
    u = Ainv @ (vc * bc.unsqueeze(-1))
    w = Ainv @ (kc * eG * bc.unsqueeze(-1))
    qg = qc * eG
    Glast = G[:, :, -1]
    kg = kc * (Glast.unsqueeze(2) - G).exp()
    dlast = Glast.exp()
    first = [0]
    for c in per_seq:
        first.append(first[-1] + c)
    S0 = (initial_state.float() if initial_state is not None
          else torch.zeros(N, H, K, V, dtype=torch.float32, device=dev))
    S_list = [S0[n] for n in range(N)]
    o_chunks = [None] * NC
    for j in range(max(per_seq) if per_seq else 0):
        seqs = [n for n in range(N) if per_seq[n] > j]
        cids = torch.tensor([first[n] + j for n in seqs], device=dev)
        Sj = torch.stack([S_list[n] for n in seqs])
        vn = u[cids] - w[cids] @ Sj
        oj = qg[cids] @ Sj + Aqk[cids] @ vn
        Sn = Sj * dlast[cids].unsqueeze(-1) + kg[cids].transpose(-1, -2) @ vn
        for ii, n in enumerate(seqs):
            S_list[n] = Sn[ii]
            o_chunks[first[n] + j] = oj[ii]
    final = torch.stack(S_list) if N > 0 else S0
    o = torch.zeros(T + 1, H, V, dtype=torch.float32, device=dev)
    if NC > 0:
        oc = torch.stack(o_chunks).transpose(1, 2)
        o = o.index_put((idx.reshape(-1),), oc.reshape(NC * C, H, V), accumulate=True)
    return o[:T].to(v.dtype), final
