"""Analytic FLOP count of one training step of a hybrid KDA / attention decoder (no GPU needed).

Counts matmul FLOPs as 2 per multiply-add: 6 x parameters per token for the linears (forward + dX + dW), causal attention
4 S d H / 2 per token forward and 3.5x that with backward, the chunked KDA products, the LCE head and the Newton-Schulz
iterations of Muon (5 iterations; Gram products counted at half cost when the symmetric kernel applies). Used by
``bench/model_flops.py`` and by the training loop's metrics (model TFLOP/s per GPU and its fraction of the measured GEMM
peak in every logged step)."""
from __future__ import annotations

from typing import Dict


def step_flops(hidden, heads, head_dim, layers, attn_interval, ffn, vocab, seq_len, tokens):
    hd = heads * head_dim
    n_attn = layers // attn_interval if attn_interval > 0 else 0
    n_kda = layers - n_attn
    kda_proj = (3 * hd + 2 * head_dim + heads) * hidden + 2 * head_dim * hd + hd * hidden   # q k v fg b, f/g low rank, o
    att_proj = 3 * hd * hidden + hd * hidden
    ffn_p = 3 * hidden * ffn
    lin = n_kda * (kda_proj + ffn_p) + n_attn * (att_proj + ffn_p)
    lce = vocab * hidden
    per_tok = {"linears": 6.0 * lin, "lce_head": 6.0 * lce}
    per_tok["attention"] = n_attn * 3.5 * 4.0 * (seq_len / 2.0) * head_dim * heads
    # chunked KDA, chunk C = 64, per token and head: intra-chunk A / WY products ~ 8 C d, state products ~ 6 d^2 / ... forward;
    # backward ~ 2.5x forward
    C, d = 64, head_dim
    kda_fwd = 2.0 * (4 * C * d + 3 * d * d)
    per_tok["kda"] = n_kda * heads * 3.5 * kda_fwd
    total_tok = sum(per_tok.values()) * tokens
    # Muon: per matrix [m, n] (m <= n): 5 x (Gram m^2 n [symmetric: half of 2 m^2 n] + m^3 [half of 2 m^3] + 2 m^2 n)
    def ns(m, n):
        m, n = min(m, n), max(m, n)
        return 5.0 * (m * m * n + m ** 3 + 2.0 * m * m * n)
    mats = n_kda * [(hd, hidden)] * 3 + n_attn * [(hd, hidden)] * 3 + layers * [(hd, hidden)] + layers * [(ffn, hidden)] * 3
    muon = sum(ns(a, b) for a, b in mats)
    return per_tok, total_tok, muon


def config_step_flops(cfg, seq_len: int, tokens: int):
    """``step_flops`` for a ``HippoConfig``: (per-token FLOPs by part, model FLOPs of a step of ``tokens`` tokens, Muon FLOPs)."""
    return step_flops(cfg.hidden_size, cfg.num_heads, cfg.head_dim, cfg.num_layers, int(getattr(cfg, "full_attn_interval", 0) or 0),
                      cfg.intermediate_size, cfg.vocab_size, seq_len, tokens)


def utilisation(cfg, seq_len: int, tokens: int, step_ms: float, n_gpus: int, peaks: Dict) -> Dict[str, float]:
    """Model TFLOP/s per GPU of a step that took ``step_ms`` and its fraction of the sustained bf16 GEMM peak in ``peaks``
    (``utils.timing.load_measured_peaks()``); Muon's own FLOPs are not counted as model FLOPs."""
    _, total, _ = config_step_flops(cfg, seq_len, tokens)
    rate = total / max(step_ms, 1e-6) * 1e3 / 1e12 / max(n_gpus, 1)
    peak = float(peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"])
    return {"model_tflops_per_gpu": round(rate, 2), "mfu": round(rate / peak, 4)}
