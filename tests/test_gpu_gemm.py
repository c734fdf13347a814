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
