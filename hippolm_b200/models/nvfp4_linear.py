"""NVFP4 weight storage for the FFN linears.

Three modes, as in the reference (``src/models/ops/nvfp4_linear.py:245-783``,
``nvfp4_tp.py:341-935``):

  bf16 master + STE   ``weight`` is a bf16 Parameter, re-quantised every forward
  no master           only ``packed_weight`` u8 [N,K/2], ``scales`` e4m3 [N,K/16] and
                      ``global_scale`` f32 [1] exist; the optimizer streams row chunks through
                      ``material_chunk`` / ``commit_chunk`` / ``decay_and_apply_chunk``
  (bf16 only = a plain bf16 weight; handled by the caller)

Differences from the reference, on purpose: the GEMMs run on the FP4 tensor cores with
activations quantised on the fly (the reference is W4A16 through Marlin), the element rounding
is hardware RN-even, and ``global_scale`` is kept per module and recomputed on re-quantisation
instead of being pinned to 1.0.
"""
from __future__ import annotations

from typing import Iterator, List, Optional, Tuple

import torch
import torch.nn as nn

from .. import ops


class _NVFP4MatmulNoMaster(torch.autograd.Function):
    """y = Q(x) dq(W)^T.  dX = dY dq(W);  dW = dY^T x is handed to ``module.grad_sink`` (no leaf)."""

    @staticmethod
    def forward(ctx, x, module, anchor):
        ctx.module = module
        ctx.save_for_backward(x)
        return ops.nvfp4_linear(x, module.packed_weight, module.scales, module.global_scale,
                                act_quant=module.act_quant)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        mod = ctx.module
        dy = dy.contiguous()
        w = ops.nvfp4_dequantize(mod.packed_weight, mod.scales, mod.global_scale, dy.dtype)
        dx = ops.gemm_nn(dy, w)
        mod.accumulate_grad_product(dy, x)
        return dx, None, None


class _NVFP4MatmulSTE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, act_quant):
        packed, scales, gs = ops.nvfp4_quantize(weight.detach())
        ctx.save_for_backward(x, packed, scales, gs)
        ctx.wdtype = weight.dtype
        return ops.nvfp4_linear(x, packed, scales, gs, act_quant=act_quant)

    @staticmethod
    def backward(ctx, dy):
        x, packed, scales, gs = ctx.saved_tensors
        dy = dy.contiguous()
        w = ops.nvfp4_dequantize(packed, scales, gs, dy.dtype)
        return ops.gemm_nn(dy, w), ops.gemm_tn(dy, x).to(ctx.wdtype), None


class NVFP4Linear(nn.Module):
    """[out_features, in_features] linear stored (or trained through) NVFP4. No bias."""

    CHUNK_ROWS = 4096

    def __init__(self, in_features: int, out_features: int, no_master: bool, device=None,
                 dtype=torch.bfloat16, act_quant: bool = True, init_weight: Optional[torch.Tensor] = None):
        super().__init__()
        assert in_features % 16 == 0
        self.in_features, self.out_features = in_features, out_features
        self.no_master = no_master
        self.act_quant = act_quant
        self.compute_dtype = dtype
        self.stochastic_rounding = True          # optimizer updates of the no-master weight round without bias
        # backward on the FP4 tensor cores: dX = Q(dY) Q(W^T)^T needs W quantised along its OTHER axis (16-element blocks
        # along out_features); that second encoding is derived from the stored one and cached until the weight changes
        self.fp4_backward = False
        self.fp4_backward_dw = False              # with fp4_backward: also dW = Q(dY^T) Q(x^T)^T on the FP4 tensor cores
        self._w_version = 0
        self._wt_cache = None                     # (version, packed_t [K, N/2], scales_t [K, N/16], gs_t [1])
        if init_weight is None:
            init_weight = torch.empty(out_features, in_features, device=device, dtype=torch.float32)
            nn.init.xavier_uniform_(init_weight)
        if no_master:
            packed, scales, gs = ops.nvfp4_quantize(init_weight.to(device=device))
            self.register_buffer("packed_weight", packed)
            self.register_buffer("scales", scales)
            self.register_buffer("global_scale", gs.float())
            self.grad_w: Optional[torch.Tensor] = None      # accumulated dW (no autograd leaf exists)
            self.grad_sink = None                            # optional callback(dw) e.g. host offload
            # gives autograd something to hang the Function on when x does not require grad
            self.register_buffer("_anchor", torch.zeros(1, device=device), persistent=False)
        else:
            self.weight = nn.Parameter(init_weight.to(device=device, dtype=dtype))
            self.weight.opt_kind = "muon"

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.no_master:
            return _NVFP4MatmulNoMaster.apply(x, self, self._anchor.requires_grad_(torch.is_grad_enabled()
                                                                                   and not x.requires_grad))
        return _NVFP4MatmulSTE.apply(x, self.weight, self.act_quant)

    def accumulate_grad_product(self, dy: torch.Tensor, x: torch.Tensor, dy_gs: Optional[torch.Tensor] = None) -> None:
        """grad_w += dy^T x. Once the accumulator exists the GEMM epilogue adds into it directly (no dW temporary,
        no separate add pass); the first micro-batch and the host-offload sink take the materialised product."""
        if self.fp4_backward and self.fp4_backward_dw and self.grad_sink is None and dy.is_cuda \
                and dy.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and dy.shape[0] % 256 == 0 \
                and dy.shape[1] % 8 == 0 and x.shape[1] % 8 == 0 and dy.stride(1) == 1 and x.stride(1) == 1:
            # dW += Q(dY^T) Q(x^T)^T on the FP4 tensor cores: both operands re-quantised with their blocks along the tokens
            from ..ops import nvfp4_cuda, fp4_gemm
            ap, asf, ags = nvfp4_cuda.quantize_transposed(dy, dy_gs)   # dy_gs: tensor scale shared with the dX product
            bp, bsf, bgs = nvfp4_cuda.quantize_transposed(x)
            if self.grad_w is None:
                self.grad_w = fp4_gemm.fp4_matmul_tiled(ap, asf, ags, bp, bsf, bgs)
            else:
                fp4_gemm.fp4_matmul_tiled(ap, asf, ags, bp, bsf, bgs, out=self.grad_w, accumulate=True)
        elif self.grad_sink is None and self.grad_w is not None and dy.is_cuda and self.grad_w.dtype == torch.bfloat16 \
                and dy.shape[1] % 8 == 0 and x.shape[1] % 8 == 0:
            ops.gemm_tn_accumulate(dy, x, self.grad_w)
        else:
            self._accumulate_grad(ops.gemm_tn(dy, x))

    def _accumulate_grad(self, dw: torch.Tensor) -> None:
        if self.grad_sink is not None:
            self.grad_sink(self, dw)
        elif self.grad_w is None:
            self.grad_w = dw.clone()
        else:
            self.grad_w.add_(dw)

    def weight_changed(self) -> None:
        """Every writer of the stored weight calls this (optimizer kernels, chunk commits, checkpoint loads)."""
        self._w_version += 1
        from ..ops import fp4_gemm
        fp4_gemm.weights_changed()

    def transposed_operands(self) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """NVFP4 encoding of W^T ([in_features, out_features], blocks along out_features) for the dX product."""
        c = self._wt_cache
        ver = (self._w_version, 0 if self.no_master else self.weight._version)
        if c is not None and c[0] == ver:
            return c[1], c[2], c[3]
        if self.no_master:
            w = ops.nvfp4_dequantize(self.packed_weight, self.scales, self.global_scale, torch.bfloat16)
        else:
            w = self.weight.detach()
        packed, scales, gs = ops.nvfp4_quantize(w.t().contiguous())
        self._wt_cache = (ver, packed, scales, gs)
        return packed, scales, gs

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        if self.no_master and prefix + "weight" in state_dict and prefix + "packed_weight" not in state_dict:
            # plain values for a weight that is kept without a master copy (a merged or converted checkpoint): quantise
            w = state_dict.pop(prefix + "weight")
            packed, scales, gs = ops.nvfp4_quantize(w.to(device=self.packed_weight.device, dtype=torch.float32))
            state_dict[prefix + "packed_weight"], state_dict[prefix + "scales"] = packed, scales
            state_dict[prefix + "global_scale"] = gs.float()
        elif not self.no_master and prefix + "packed_weight" in state_dict and prefix + "weight" not in state_dict:
            # stored codes for a module that trains through a master copy: the master starts from the dequantised values
            state_dict[prefix + "weight"] = ops.nvfp4_dequantize(
                state_dict.pop(prefix + "packed_weight"), state_dict.pop(prefix + "scales"),
                state_dict.pop(prefix + "global_scale"), self.weight.dtype)
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)
        self.weight_changed()

    # ------------------------------------------------------------------ chunk API (optimizer side)
    def chunk_ranges(self, rows: Optional[int] = None) -> Iterator[Tuple[int, int]]:
        rows = rows or self.CHUNK_ROWS
        for r0 in range(0, self.out_features, rows):
            yield r0, min(r0 + rows, self.out_features)

    def material_chunk(self, r0: int, r1: int, dtype=torch.float32) -> torch.Tensor:
        return ops.nvfp4_dequantize(self.packed_weight[r0:r1], self.scales[r0:r1], self.global_scale, dtype)

    def commit_chunk(self, r0: int, r1: int, w: torch.Tensor, stochastic: bool = False) -> None:
        """Re-quantise rows [r0, r1) against the module's tensor scale. If the rows have outgrown that scale (a block
        scale would exceed the e4m3 maximum of 448 and clip), the whole tensor is first re-expressed against a larger
        tensor scale. ``stochastic``: unbiased rounding for optimizer updates of a weight that has no master copy
        (round-to-nearest silently drops every update below half a code step)."""
        need = w.detach().abs().max().float() / (6.0 * 448.0)
        if bool(need > self.global_scale.reshape(()).float()):
            full = self.material_chunk(0, self.out_features, torch.float32)
            full[r0:r1] = w.float()
            self.global_scale.copy_(torch.maximum(need, full.abs().max() / (6.0 * 448.0)).reshape(1))
            packed, scales, _ = ops.nvfp4_quantize(full, self.global_scale)
            self.packed_weight.copy_(packed); self.scales.copy_(scales)
            self.weight_changed()
            if not stochastic:
                return
        if stochastic:
            from ..ref.ops import nvfp4_quantize_stochastic
            self._sr_calls = getattr(self, "_sr_calls", 0) + 1
            gen = torch.Generator(device=w.device).manual_seed(0x5EED + 7919 * self._sr_calls + r0)
            packed, scales, _ = nvfp4_quantize_stochastic(w, self.global_scale, gen)
        else:
            packed, scales, _ = ops.nvfp4_quantize(w, self.global_scale)
        self.packed_weight[r0:r1].copy_(packed)
        self.scales[r0:r1].copy_(scales)
        self.weight_changed()

    def apply_chunk_update(self, r0: int, r1: int, update: torch.Tensor, lr: float) -> None:
        self.decay_and_apply_chunk(r0, r1, update, lr, 1.0)

    def decay_and_apply_chunk(self, r0: int, r1: int, update: torch.Tensor, lr: float,
                              wd_factor: float = 1.0) -> None:
        """W[r0:r1] <- W*wd_factor - lr*update, then re-quantise those rows."""
        w = self.material_chunk(r0, r1, torch.float32)
        w.mul_(wd_factor).add_(update.float(), alpha=-lr)
        self.commit_chunk(r0, r1, w, stochastic=self.stochastic_rounding)

    def material_bf16_view(self) -> torch.Tensor:
        return self.material_chunk(0, self.out_features, torch.bfloat16)

    def commit_bf16_view(self, w: torch.Tensor) -> None:
        """Full re-quantisation; also refreshes the tensor-level scale."""
        packed, scales, gs = ops.nvfp4_quantize(w.float())
        self.packed_weight.copy_(packed); self.scales.copy_(scales); self.global_scale.copy_(gs)
        self.weight_changed()

    def refresh_global_scale(self, headroom: float = 1.0) -> None:
        """Re-derive global_scale from the current contents (keeps e4m3 scales in range as W grows)."""
        self.commit_bf16_view(self.material_chunk(0, self.out_features, torch.float32))

    def numel_logical(self) -> int:
        return self.in_features * self.out_features


def nvfp4_modules(model: nn.Module) -> List[NVFP4Linear]:
    return [m for m in model.modules() if isinstance(m, NVFP4Linear) and m.no_master]


def repack_nvfp4_weights(model: nn.Module) -> int:
    """Kept for API parity with ``nvfp4_linear.py:repack_nvfp4_weights``: the FP4 tensor-core
    layout is the storage layout, so nothing has to be rebuilt after an optimizer step."""
    return len(nvfp4_modules(model))
