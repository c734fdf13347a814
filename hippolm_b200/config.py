"""Model / precision configuration.

``HippoConfig`` keeps every field of the reference dataclass (``src/models/config.py:13-145``)
and adds the hybrid-layer pattern (full causal attention every ``full_attn_interval`` layers,
RoPE), the parallel layout (tp / dp / sequence parallel) and the FFN storage format.
"""
from __future__ import annotations

from dataclasses import dataclass, field, fields, asdict
from typing import Any, Dict, List, Optional

import torch

_DTYPES = {"fp32": torch.float32, "float32": torch.float32, "fp16": torch.float16,
           "float16": torch.float16, "bf16": torch.bfloat16, "bfloat16": torch.bfloat16}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    key = str(name).lower()
    if key not in _DTYPES:
        raise ValueError(f"unknown dtype {name!r}; expected one of {sorted(_DTYPES)}")
    return _DTYPES[key]


def dtype_name(dt: torch.dtype) -> str:
    return {torch.float32: "fp32", torch.float16: "fp16", torch.bfloat16: "bf16"}[dt]


@dataclass
class HippoConfig:
    # vocabulary / width
    vocab_size: int = 32000
    hidden_size: int = 256
    tie_word_embeddings: bool = False
    use_bias: bool = False
    # KDA
    num_heads: int = 4
    head_dim: int = 64
    expand_v: float = 1.0
    kda_mode: str = "chunk"                 # chunk | fused_recurrent
    use_short_conv: bool = False
    allow_neg_eigval: bool = False
    safe_gate: bool = False
    lower_bound: float = -5.0
    conv_size: int = 4
    conv_bias: bool = False
    # depth
    num_layers: int = 4
    num_blocks: int = 1
    attn_res_heads: int = 0                 # heads of the block-attn-res pseudo-query; 0 = num_heads
    full_attn_interval: int = 4             # layer i is full attention when (i+1) % interval == 0; 0 = all KDA
    rope_theta: float = 10000.0
    # ffn
    intermediate_size: int = 1024
    rms_norm_eps: float = 1e-6
    # packing
    pack_chunk_size: int = 0
    pack_buffer_size: int = 2048
    kda_skip_aqk_akk_saved: bool = False
    # FFN storage
    ffn_nvfp4: bool = False
    ffn_nvfp4_marlin: bool = False          # accepted for config compatibility; FP4 tensor cores are always used
    # backward of the NVFP4 FFN: "bf16" = dX and dW as bf16 GEMMs on the dequantised weight (the reference's choice,
    # ``src/models/ops/nvfp4_marlin.py:1036-1077``); "fp4_dx" = dX = Q(dY) Q(W^T)^T on the FP4 tensor cores, dW in bf16;
    # "fp4" = dX as above and dW = Q(dY^T) Q(x^T)^T with both operands re-quantised along the token axis
    ffn_nvfp4_backward: str = "bf16"
    ffn_nvfp4_no_bf16_master: bool = False
    # memory policy
    gradient_checkpointing: bool = False
    lce_num_chunks: int = 0                 # token chunks of the fused linear+CE head; 0 = sized automatically
    # CUDA only: the logits GEMM stores bf16 logits and takes the softmax statistics (row max, sum exp, target logit) from
    # its accumulator in the epilogue, the gradient overwrites the logits in place; false = fp32 logits in global memory
    # and a separate statistics pass over them
    lce_epilogue_stats: bool = True
    # derived
    block_size: int = field(init=False, default=0)

    def __post_init__(self):
        if self.num_blocks <= 0:
            raise ValueError("num_blocks must be positive")
        if self.num_layers % self.num_blocks != 0:
            raise ValueError(f"num_layers ({self.num_layers}) must be divisible by num_blocks ({self.num_blocks})")
        self.block_size = self.num_layers // self.num_blocks
        if self.kda_mode not in ("chunk", "fused_recurrent"):
            raise ValueError(f"kda_mode must be chunk|fused_recurrent, got {self.kda_mode!r}")
        if not (-5.0 <= self.lower_bound < 0):
            raise ValueError("lower_bound must be in [-5, 0)")
        if self.pack_chunk_size <= 0:
            self.pack_chunk_size = self.head_dim
        self.pack_chunk_size = ((self.pack_chunk_size + 63) // 64) * 64
        if self.ffn_nvfp4_backward not in ("bf16", "fp4_dx", "fp4"):
            raise ValueError(f"ffn_nvfp4_backward must be bf16|fp4_dx|fp4, got {self.ffn_nvfp4_backward!r}")
        if self.ffn_nvfp4_no_bf16_master and not self.ffn_nvfp4:
            raise ValueError("ffn_nvfp4_no_bf16_master requires ffn_nvfp4")
        if self.hidden_size % self.num_heads != 0:
            raise ValueError("hidden_size must be divisible by num_heads (AttnRes heads)")
        # accepted names whose only supported value is the reference's production setting: refuse the other value
        # instead of silently ignoring it
        if self.use_bias:
            raise ValueError("use_bias=true is not supported: the projections carry no bias term")
        if self.conv_bias:
            raise ValueError("conv_bias=true is not supported: the short-convolution kernels carry no bias term")

    # ---- derived sizes
    @property
    def key_dim(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def head_v_dim(self) -> int:
        return int(self.head_dim * self.expand_v)

    @property
    def value_dim(self) -> int:
        return self.num_heads * self.head_v_dim

    def layer_types(self) -> List[str]:
        iv = self.full_attn_interval
        return ["attn" if (iv > 0 and (i + 1) % iv == 0) else "kda" for i in range(self.num_layers)]

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)

    @classmethod
    def from_namespace(cls, ns) -> "HippoConfig":
        names = {f.name for f in fields(cls) if f.init}
        src = vars(ns) if not isinstance(ns, dict) else ns
        return cls(**{k: v for k, v in src.items() if k in names and v is not None})


# ----------------------------------------------------------------------------- precision
_CLASSES = ("model_weights", "gradients", "activations", "muon_momentum", "adamw_m", "adamw_v")


@dataclass
class PrecisionConfig:
    """Six tensor classes, each ``{dtype: fp32|fp16|bf16}`` (``src/training/precision_config.py:68-216``)."""
    model_weights: torch.dtype = torch.bfloat16
    gradients: torch.dtype = torch.bfloat16
    activations: torch.dtype = torch.bfloat16
    muon_momentum: torch.dtype = torch.bfloat16
    adamw_m: torch.dtype = torch.bfloat16
    adamw_v: torch.dtype = torch.bfloat16

    @classmethod
    def from_dict(cls, d: Optional[Dict[str, Any]]) -> "PrecisionConfig":
        out = cls()
        if not d:
            return out
        for k, v in d.items():
            if k not in _CLASSES:
                raise ValueError(f"unknown precision class {k!r}; expected {_CLASSES}")
            dt = v.get("dtype") if isinstance(v, dict) else v
            setattr(out, k, parse_dtype(dt))
        return out

    @classmethod
    def uniform(cls, dtype) -> "PrecisionConfig":
        dt = parse_dtype(dtype)
        return cls(**{k: dt for k in _CLASSES})

    def to_dict(self) -> Dict[str, Dict[str, str]]:
        return {k: {"dtype": dtype_name(getattr(self, k))} for k in _CLASSES}

    @property
    def autocast_enabled(self) -> bool:
        return self.activations != torch.float32

    @property
    def autocast_dtype(self) -> torch.dtype:
        return self.activations
