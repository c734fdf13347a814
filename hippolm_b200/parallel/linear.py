"""Sequence-parallel tensor-parallel linears.

  column_linear_sp : x[T/w, K] --all-gather--> [T, K] @ W[N/w, K]^T -> [T, N/w]
  row_linear_sp    : x[T, K/w] @ W[N, K/w]^T --reduce-scatter--> [T/w, N]

Backward runs the conjugate collective (reduce-scatter / all-gather), which the reference's
ColumnParallelLinear omits (``src/models/tp_model/_primitives.py:306-309``). On CUDA with a
symmetric-memory workspace the collective is fused into the GEMM kernel
(:mod:`hippolm_b200.parallel.fused`); otherwise NCCL/gloo + the plain GEMM op run back to back.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .. import ops
from .collectives import all_gather_dim0, reduce_scatter_dim0
from .mesh import get_mesh


# Keep the gathered input of a column-parallel linear for its weight-gradient GEMM instead of gathering it a second
# time in the backward pass (memory for NVLink traffic). HIPPO_KEEP_GATHERED=0 restores the re-gather.
KEEP_GATHERED = os.environ.get("HIPPO_KEEP_GATHERED", "1") != "0"


def _fused():
    from . import fused
    return fused if fused.enabled() else None


class _ColumnLinearSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        m = get_mesh()
        f = _fused()
        def unfused():
            g = all_gather_dim0(x, m.tp_group, m.tp)
            return g, ops.gemm_nt(g, weight), False

        def fused_path():
            g, yy = f.allgather_gemm(x, weight, need_gathered=False)
            return g, yy, True
        if f is not None and x.is_cuda and m.tp > 1 and f.fits(x.shape[0], x.shape[0] * m.tp, x.shape[1]) \
                and weight.shape[0] % 8 == 0 and x.dtype == torch.bfloat16:
            xg, y, was_fused = f.tuned(("ag", x.shape[0], x.shape[1], weight.shape[0], 0), fused_path, unfused)
            if was_fused and KEEP_GATHERED:
                # a private copy of the gathered activations for the dW GEMM of the backward pass (the workspace
                # view is recycled two calls later); costs T*K*2 bytes per layer, saves one all-gather per layer
                rows = x.shape[0]
                xg = xg.clone()
                xg[m.tp_rank * rows:(m.tp_rank + 1) * rows].copy_(x)
        else:
            xg, y, _ = unfused()
        if bias is not None:
            y = y + bias
        ctx.kept = bool(KEEP_GATHERED and m.tp > 1)
        ctx.save_for_backward(xg if ctx.kept else x, weight)
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        m = get_mesh()
        dy = dy.contiguous()
        f = _fused()
        dxg = None
        if ctx.needs_input_grad[0]:
            def unfused():
                return reduce_scatter_dim0(ops.gemm_nn(dy, weight), m.tp_group, m.tp)
            if f is not None and dy.is_cuda and m.tp > 1 and dy.dtype == torch.bfloat16 \
                    and f.fits(dy.shape[0] // m.tp, dy.shape[0], weight.shape[1]) and dy.shape[1] % 8 == 0:
                dx = f.tuned(("rs", dy.shape[0], dy.shape[1], weight.shape[1], 1),
                             lambda: f.gemm_reduce_scatter(dy, weight, transpose_w=True), unfused)
            else:
                dx = unfused()
        else:
            dx = None
        xg = x if ctx.kept else all_gather_dim0(x, m.tp_group, m.tp)
        dw = ops.gemm_tn(dy, xg)                                   # [N/w, K]
        db = dy.sum(0) if ctx.has_bias else None
        return dx, dw.to(weight.dtype), db


class _RowLinearSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight):
        m = get_mesh()
        f = _fused()
        def unfused():
            return reduce_scatter_dim0(ops.gemm_nt(x, weight), m.tp_group, m.tp)
        if f is not None and x.is_cuda and m.tp > 1 and x.dtype == torch.bfloat16 \
                and f.fits(x.shape[0] // m.tp, x.shape[0], weight.shape[0]) and x.shape[1] % 8 == 0:
            y = f.tuned(("rs", x.shape[0], x.shape[1], weight.shape[0], 0),
                        lambda: f.gemm_reduce_scatter(x, weight, transpose_w=False), unfused)
        else:
            y = unfused()
        ctx.save_for_backward(x, weight)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        m = get_mesh()
        f = _fused()
        dy = dy.contiguous()
        def unfused():
            g = all_gather_dim0(dy, m.tp_group, m.tp)              # [T, N]
            return g, ops.gemm_nn(g, weight)                       # [T, K/w]
        if f is not None and dy.is_cuda and m.tp > 1 and dy.dtype == torch.bfloat16 \
                and f.fits(dy.shape[0], dy.shape[0] * m.tp, dy.shape[1]) and weight.shape[1] % 8 == 0:
            dyg, dx = f.tuned(("ag", dy.shape[0], dy.shape[1], weight.shape[1], 1),
                              lambda: f.allgather_gemm(dy, weight, transpose_w=True), unfused)
        else:
            dyg, dx = unfused()
        dw = ops.gemm_tn(dyg, x)                                   # [N, K/w]
        return dx, dw.to(weight.dtype)


def _fp4_backward(module, dy: torch.Tensor, contraction: int, out: int) -> bool:
    """dX of an NVFP4 linear on the FP4 tensor cores? Needs the option, a CUDA bf16 gradient and shapes the block-scaled
    GEMM covers (contraction a multiple of 256, output a multiple of 8)."""
    return (bool(getattr(module, "fp4_backward", False)) and dy.is_cuda and dy.dtype == torch.bfloat16
            and contraction % 256 == 0 and out % 8 == 0)


def _tensor_scale(t: torch.Tensor):
    from ..ops import nvfp4_cuda
    return nvfp4_cuda.tensor_scale(t)


def _nvfp4_operands(module, weight):
    """(packed, scales, global_scale) of an NVFP4Linear: its buffers (no master) or the freshly quantised master."""
    if module.no_master:
        return module.packed_weight, module.scales, module.global_scale
    return ops.nvfp4_quantize(weight.detach())


class _NVFP4ColumnSP(torch.autograd.Function):
    """x[T/w, K] --all-gather--> Q(x) dq(W[N/w, K])^T on the FP4 tensor cores. Backward runs in bf16 on the
    dequantised weight (as the reference's NVFP4 backward, ``src/models/ops/nvfp4_tp.py:61-335``):
    dX = reduce-scatter(dY dq(W)) fused into the GEMM, dW = dY^T gather(x). ``weight`` is the bf16 master
    (STE mode) or a dummy anchor (no-master mode, where dW goes to ``module._accumulate_grad``)."""

    @staticmethod
    def forward(ctx, x, weight, module):
        m = get_mesh()
        packed, scales, gs = _nvfp4_operands(module, weight)
        f = _fused()

        def unfused():
            xg = all_gather_dim0(x, m.tp_group, m.tp) if m.tp > 1 else x
            return ops.nvfp4_linear(xg, packed, scales, gs, act_quant=module.act_quant), \
                (xg if KEEP_GATHERED and m.tp > 1 else None)
        if f is not None and x.is_cuda and m.tp > 1 and module.act_quant:
            y, kept = f.tuned(("fp4_ag", x.shape[0], x.shape[1], packed.shape[0]),
                              lambda: f.nvfp4_allgather_gemm(x, packed, scales, gs, keep_gathered=KEEP_GATHERED), unfused)
        else:
            y, kept = unfused()
        ctx.module = module
        # kept: the gathered input, either bf16 [T, K] or the FP4 bytes the GEMM consumed (uint8, dequantised in backward:
        # dW = dY^T Q(x) is the exact weight gradient of the quantised forward)
        ctx.kept_kind = 0 if kept is None else (2 if kept.dtype == torch.uint8 else 1)
        ctx.T, ctx.K = x.shape[0] * m.tp, x.shape[1]
        ctx.save_for_backward(x if kept is None else kept, packed, scales, gs)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, packed, scales, gs = ctx.saved_tensors
        mod, m = ctx.module, get_mesh()
        dy = dy.contiguous()
        f = _fused()
        dx = None
        dy_gs = None
        if _fp4_backward(mod, dy, contraction=dy.shape[1], out=ctx.K):
            # dX = Q(dY) Q(W^T)^T on the FP4 tensor cores (W^T re-encoded along N once per optimizer step)
            pt, st, gt = mod.transposed_operands()
            if m.tp == 1:
                dy_gs = _tensor_scale(dy)            # one absmax pass serves the row-wise and the token-wise encoding of dY
                dx = ops.nvfp4_linear(dy, pt, st, gt, act_quant=True, act_gs=dy_gs)
            elif f is not None:
                dx = f.tuned(("fp4_rs", dy.shape[0], dy.shape[1], pt.shape[0]),
                             lambda: f.nvfp4_gemm_reduce_scatter(dy, pt, st, gt),     # None: shape not covered
                             lambda: reduce_scatter_dim0(ops.nvfp4_linear(dy, pt, st, gt, act_quant=True), m.tp_group, m.tp))
        w = ops.nvfp4_dequantize(packed, scales, gs, dy.dtype) if dx is None else None   # [N/w, K]
        if m.tp == 1:
            if dx is None:
                dx = ops.gemm_nn(dy, w)
            xg = x
        else:
            if dx is not None:
                pass
            elif f is not None and dy.is_cuda and dy.dtype == torch.bfloat16 \
                    and f.fits(dy.shape[0] // m.tp, dy.shape[0], w.shape[1]) and dy.shape[1] % 8 == 0:
                dx = f.tuned(("rs", dy.shape[0], dy.shape[1], w.shape[1], 1),
                             lambda: f.gemm_reduce_scatter(dy, w, transpose_w=True),
                             lambda: reduce_scatter_dim0(ops.gemm_nn(dy, w), m.tp_group, m.tp))
            else:
                dx = reduce_scatter_dim0(ops.gemm_nn(dy, w), m.tp_group, m.tp)
            if ctx.kept_kind == 2:
                xg = f.nvfp4_dequant_gathered(x, ctx.T, ctx.K) if f is not None else None
                assert xg is not None, "the fused workspace was torn down between forward and backward"
            elif ctx.kept_kind == 1:
                xg = x
            else:
                xg = all_gather_dim0(x, m.tp_group, m.tp)
        if mod.no_master:
            mod.accumulate_grad_product(dy, xg, dy_gs)
            return dx, None, None
        return dx, ops.gemm_tn(dy, xg).to(mod.weight.dtype), None


class _NVFP4RowSP(torch.autograd.Function):
    """x[T, K/w] -> reduce-scatter(Q(x) dq(W[N, K/w])^T) [T/w, N]; backward in bf16: dY is all-gathered inside
    the dX GEMM, dW = gather(dY)^T x."""

    @staticmethod
    def forward(ctx, x, weight, module):
        m = get_mesh()
        packed, scales, gs = _nvfp4_operands(module, weight)
        f = _fused()
        def unfused():
            yy = ops.nvfp4_linear(x, packed, scales, gs, act_quant=module.act_quant)
            return reduce_scatter_dim0(yy, m.tp_group, m.tp) if m.tp > 1 else yy
        if f is not None and x.is_cuda and m.tp > 1 and module.act_quant:
            y = f.tuned(("fp4_rs", x.shape[0], x.shape[1], packed.shape[0]),
                        lambda: f.nvfp4_gemm_reduce_scatter(x, packed, scales, gs), unfused)
        else:
            y = unfused()
        ctx.module = module
        ctx.save_for_backward(x, packed, scales, gs)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, packed, scales, gs = ctx.saved_tensors
        mod, m = ctx.module, get_mesh()
        dy = dy.contiguous()
        f = _fused()
        if m.tp == 1 and _fp4_backward(mod, dy, contraction=dy.shape[1], out=x.shape[1]):
            pt, st, gt = mod.transposed_operands()
            dy_gs = _tensor_scale(dy)
            dx = ops.nvfp4_linear(dy, pt, st, gt, act_quant=True, act_gs=dy_gs)   # Q(dY) Q(W^T)^T
            if mod.no_master:
                mod.accumulate_grad_product(dy, x, dy_gs)
                return dx, None, None
            return dx, ops.gemm_tn(dy, x).to(mod.weight.dtype), None
        dx = dyg = None
        if m.tp > 1 and f is not None and _fp4_backward(mod, dy, contraction=dy.shape[1], out=x.shape[1]):
            # the gradient shard is quantised and pushed as FP4 (0.5625 bytes per element on the wire), the dX GEMM runs
            # on the FP4 tensor cores, and the gathered Q(dY) is dequantised once for the dW product
            pt, st, gt = mod.transposed_operands()
            dx, kept = f.nvfp4_allgather_gemm(dy, pt, st, gt, keep_gathered=True)
            if dx is not None:
                dyg = f.nvfp4_dequant_gathered(kept, dy.shape[0] * m.tp, dy.shape[1])
        if dx is None:
            w = ops.nvfp4_dequantize(packed, scales, gs, dy.dtype)           # [N, K/w]
            if m.tp == 1:
                dyg, dx = dy, ops.gemm_nn(dy, w)
            elif f is not None and dy.is_cuda and dy.dtype == torch.bfloat16 \
                    and f.fits(dy.shape[0], dy.shape[0] * m.tp, dy.shape[1]) and w.shape[1] % 8 == 0:
                def unfused():
                    g = all_gather_dim0(dy, m.tp_group, m.tp)
                    return g, ops.gemm_nn(g, w)
                dyg, dx = f.tuned(("ag", dy.shape[0], dy.shape[1], w.shape[1], 1),
                                  lambda: f.allgather_gemm(dy, w, transpose_w=True), unfused)
            else:
                dyg = all_gather_dim0(dy, m.tp_group, m.tp)
                dx = ops.gemm_nn(dyg, w)
        if mod.no_master:
            mod.accumulate_grad_product(dyg, x)
            return dx, None, None
        return dx, ops.gemm_tn(dyg, x).to(mod.weight.dtype), None


def _nvfp4_weight_arg(module, x):
    if not module.no_master:
        return module.weight
    # a no-master module has no autograd leaf: when nothing upstream requires a gradient (everything else frozen) the
    # anchor does, so that backward still reaches this layer and its dW product is formed
    return module._anchor.requires_grad_(torch.is_grad_enabled() and not x.requires_grad)


def nvfp4_column_linear_sp(x: torch.Tensor, module):
    return _NVFP4ColumnSP.apply(x, _nvfp4_weight_arg(module, x), module)


def nvfp4_row_linear_sp(x: torch.Tensor, module):
    return _NVFP4RowSP.apply(x, _nvfp4_weight_arg(module, x), module)


def column_linear_sp(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
    return _ColumnLinearSP.apply(x, weight, bias)


def row_linear_sp(x: torch.Tensor, weight: torch.Tensor):
    return _RowLinearSP.apply(x, weight)
