"""CTA-pair NVFP4 GEMM (``csrc/gemm_fp4_2sm.cu``) against the one-CTA kernel and the fp32 product of the dequantised
operands: full tiles, ragged edges in M and N (TMA zero fill + predicated stores), several tiles per cluster (the single
TMEM accumulator is handed back and reused), long K (the 4-stage ring wraps), and the accumulating epilogue."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6))


def _operands(M, N, K, seed):
    from hippolm_b200 import ops
    from hippolm_b200.ops import fp4_gemm
    torch.manual_seed(seed)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (0.05 * torch.randn(N, K, device="cuda")).bfloat16()
    xp, xs, xg = ops.nvfp4_quantize(x)
    wp, ws, wg = ops.nvfp4_quantize(w)
    sfa, sfb = fp4_gemm.tile_scales(xs, M, K), fp4_gemm.tile_scales(ws, N, K)
    ref = ops.nvfp4_dequantize(xp, xs, xg) @ ops.nvfp4_dequantize(wp, ws, wg).t()
    return xp, sfa, xg, wp, sfb, wg, ref


@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (512, 768, 2048), (300, 264, 768), (1024, 5376, 4096),
                                   (8192, 2048, 1024)])
def test_pair_kernel_matches_oracle_and_one_cta_kernel(M, N, K):
    from hippolm_b200.ops import fp4_gemm, _ext
    xp, sfa, xg, wp, sfb, wg, ref = _operands(M, N, K, M + N + K)
    y1 = fp4_gemm.fp4_matmul_tiled(xp, sfa, xg, wp, sfb, wg)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")     # unwritten tiles stay NaN
    y2 = fp4_gemm.fp4_matmul_pair(xp, sfa, xg, wp, sfb, wg, out=out)
    torch.cuda.synchronize()
    assert _ext.device_status()[0] == 0
    assert not torch.isnan(y2).any()
    assert _rel(y2, ref) < 1e-2
    # both kernels accumulate the same products in fp32 in the same k order; rounding to bf16 happens once in each
    assert _rel(y2, y1) < 4e-3


def test_pair_kernel_accumulates_into_output():
    from hippolm_b200.ops import fp4_gemm, _ext
    M, N, K = 768, 512, 1024
    xp, sfa, xg, wp, sfb, wg, ref = _operands(M, N, K, 7)
    base = torch.randn(M, N, device="cuda").bfloat16()
    out = base.clone()
    fp4_gemm.fp4_matmul_pair(xp, sfa, xg, wp, sfb, wg, out=out, accumulate=True)
    torch.cuda.synchronize()
    assert _ext.device_status()[0] == 0
    assert _rel(out, ref + base.float()) < 1.5e-2


def test_pair_kernel_is_bit_reproducible():
    from hippolm_b200.ops import fp4_gemm
    xp, sfa, xg, wp, sfb, wg, _ = _operands(2048, 1024, 2048, 11)
    a = fp4_gemm.fp4_matmul_pair(xp, sfa, xg, wp, sfb, wg)
    b = fp4_gemm.fp4_matmul_pair(xp, sfa, xg, wp, sfb, wg)
    assert torch.equal(a, b)
