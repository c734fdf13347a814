"""tcgen05 bf16 GEMM vs an fp32 torch reference, all four operand layouts, ragged edges."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b):
    return a.float() @ b.float()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (300, 264, 136), (1024, 1024, 1024),
                                   (4096, 1800, 512), (64, 8, 8)])
def test_gemm_layouts(M, N, K):
    from hippolm_b200.ops import cuda_ops as co
    from hippolm_b200.ops import _ext
    _ext.clear_device_status()
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    b = torch.randn(N, K, device="cuda", generator=g).bfloat16()
    tol = 2e-2 * (K ** 0.5)
    y = co.gemm_nt(a, b)
    assert (y.float() - _ref(a, b.t())).abs().max() < tol
    bt = b.t().contiguous()                      # [K, N]
    y = co.gemm_nn(a, bt)
    assert (y.float() - _ref(a, bt)).abs().max() < tol
    at = a.t().contiguous()                      # [K, M]
    y = co.gemm_tn(at, bt)                       # at^T @ bt = a @ b^T
    assert (y.float() - _ref(a, bt)).abs().max() < tol
    torch.cuda.synchronize()
    assert _ext.device_status()[0] == 0


def test_gemm_fp32_out_and_accumulate():
    from hippolm_b200.ops import cuda_ops as co
    a = torch.randn(512, 384, device="cuda").bfloat16()
    b = torch.randn(256, 384, device="cuda").bfloat16()
    out = torch.ones(512, 256, device="cuda", dtype=torch.float32)
    co._gemm(a, b, 0, 512, 256, 384, out=out, accumulate=True, alpha=0.5)
    ref = 1.0 + 0.5 * (a.float() @ b.float().t())
    assert (out - ref).abs().max() < 1e-2


@pytest.mark.parametrize("kernel", ["1sm", "2sm"])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (384, 520, 200), (1000, 264, 136), (2048, 1024, 1024), (4096, 1800, 512)])
def test_gemm_one_cta_and_cta_pair_kernels(kernel, M, N, K):
    """Both kernels, named explicitly, against the fp32 product: NT, NN and TN operand layouts, ragged M / N / K."""
    from hippolm_b200.ops import cuda_ops as co
    from hippolm_b200.ops import _ext
    _ext.clear_device_status()
    g = torch.Generator(device="cuda").manual_seed(3 * M + N + K)
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    b = torch.randn(N, K, device="cuda", generator=g).bfloat16()
    bt, at = b.t().contiguous(), a.t().contiguous()
    ref = _ref(a, bt)
    tol = 2e-2 * (K ** 0.5)
    y = co._gemm(a, b, 0, M, N, K, kernel=kernel)
    assert (y.float() - ref).abs().max() < tol
    y = co._gemm(a, bt, 1, M, N, K, kernel=kernel)
    assert (y.float() - ref).abs().max() < tol
    y = co._gemm(at, bt, 2, M, N, K, kernel=kernel)
    assert (y.float() - ref).abs().max() < tol
    out = torch.ones(M, N, device="cuda", dtype=torch.float32)
    co._gemm(a, b, 0, M, N, K, out=out, accumulate=True, alpha=0.5, kernel=kernel)
    assert (out - (1.0 + 0.5 * ref)).abs().max() < tol
    torch.cuda.synchronize()
    assert _ext.device_status()[0] == 0


@pytest.mark.parametrize("n,K", [(512, 256), (1000, 328), (2048, 1024)])
def test_symmetric_output_gemm(n, K):
    """X X^T and c S S + b S through the lower-tiles-then-mirror path against the fp32 products."""
    from hippolm_b200.ops import muon_cuda as mc, _ext
    _ext.clear_device_status()
    g = torch.Generator(device="cuda").manual_seed(n + K)
    x = torch.randn(n, K, device="cuda", generator=g).bfloat16()
    S = torch.empty(n, n, device="cuda", dtype=torch.bfloat16)
    mc._gemm_sym(x, x, S, None, n, K, 0, 1.0, 0.0)
    ref = x.float() @ x.float().t()
    assert bool(((S.float() - ref).abs() <= 8e-3 * ref.abs() + 2e-2 * (K ** 0.5)).all())     # bf16 output rounding
    assert torch.equal(S, S.t())
    M = torch.empty_like(S)
    Ss = (S.float() / n).bfloat16()
    Ss = torch.tril(Ss) + torch.tril(Ss, -1).t()
    mc._gemm_sym(Ss, Ss, M, Ss, n, n, 1, 0.5, 2.0)
    ref2 = 0.5 * (Ss.float() @ Ss.float()) + 2.0 * Ss.float()
    assert (M.float() - ref2).abs().max() < 3e-2 * max(1.0, float(ref2.abs().max()))
    assert torch.equal(M, M.t())
    torch.cuda.synchronize()
    assert _ext.device_status()[0] == 0


@pytest.mark.parametrize("M,N,K,layout", [(512, 128, 16384, 2), (1024, 512, 8200, 2), (300, 264, 9000, 0), (1536, 1024, 12288, 1)])
def test_gemm_split_k(M, N, K, layout):
    """Few output tiles and a long contraction: the dispatcher cuts K into slices (work item = tile x slice, fp32
    partial planes, one reduction pass). Same result as the fp32 product, bf16 and fp32 outputs, accumulate included,
    and bit-identical between two runs (the slices are summed in a fixed order)."""
    from hippolm_b200.ops import cuda_ops as co
    from hippolm_b200.ops import _ext
    assert co._splitk_factor(M, N, K) > 1
    _ext.clear_device_status()
    g = torch.Generator(device="cuda").manual_seed(M + K)
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    b = torch.randn(N, K, device="cuda", generator=g).bfloat16()
    ref = a.float() @ b.float().t()
    if layout == 0:
        A, B = a, b
    elif layout == 1:
        A, B = a, b.t().contiguous()
    else:
        A, B = a.t().contiguous(), b.t().contiguous()
    tol = 2e-2 * (K ** 0.5)
    y = co._gemm(A, B, layout, M, N, K)
    assert (y.float() - ref).abs().max() < tol
    y2 = co._gemm(A, B, layout, M, N, K)
    assert torch.equal(y, y2)
    acc = torch.full((M, N), 3.0, device="cuda", dtype=torch.float32)
    co._gemm(A, B, layout, M, N, K, out=acc, accumulate=True, alpha=0.5)
    assert (acc - (3.0 + 0.5 * ref)).abs().max() < 1e-2 * (K ** 0.5) * 0.5 + 1e-2
    accb = torch.ones(M, N, device="cuda", dtype=torch.bfloat16)
    co._gemm(A, B, layout, M, N, K, out=accb, accumulate=True)
    assert (accb.float() - (1.0 + ref)).abs().max() < tol
    torch.cuda.synchronize()
    assert _ext.device_status()[0] == 0
