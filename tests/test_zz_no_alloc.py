"""The allocation-free RMSNorm backward entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory at call time (their host application owns
the memory, or an allocation on the hot path is not acceptable). ``hippo_rmsnorm_bwd_noalloc`` keeps its
only intermediate buffer inside the library image, so its results must equal those of the regular entry
point, which receives that buffer from the caller. Two calls in a row check that the shared built-in
buffer carries nothing over from one call to the next. The file name sorts last so that every other
test has already run if this one fails under ``-x``.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run_pair(T, D, seed):
    from hippolm_b200.ops._ext import lib, ptr, stream_ptr
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(T, D, device="cuda", generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).bfloat16()
    dy = torch.randn(T, D, device="cuda", generator=g).bfloat16()
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
    # regular entry point: the caller allocates the partial-sum buffer
    nb = min(T, 148 * 4)
    dx_ref = torch.empty_like(x); dw_ref = torch.empty(D, device="cuda")
    part = torch.empty(nb, D, device="cuda")
    rc = lib().hippo_rmsnorm_bwd(ptr(x), ptr(w), ptr(dy), ptr(rstd), ptr(dx_ref), ptr(part), ptr(dw_ref),
                                 C.c_longlong(T), D, nb, stream_ptr())
    assert rc == 0
    # allocation-free entry point: outputs only
    dx = torch.empty_like(x); dw = torch.empty(D, device="cuda")
    fn = lib().hippo_rmsnorm_bwd_noalloc
    fn.restype = C.c_int
    rc = fn(ptr(x), ptr(w), ptr(dy), ptr(rstd), ptr(dx), ptr(dw), C.c_longlong(T), D, stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(dx, dx_ref)
    scale = dw_ref.abs().max().item() + 1e-6
    assert (dw - dw_ref).abs().max().item() <= 2e-2 * scale
    # and against the fp32 formula
    xf, dyf, wf = x.float(), dy.float(), w.float()
    xh = xf * rstd[:, None]
    dw_true = (dyf * xh).sum(0)
    assert (dw - dw_true).abs().max().item() <= 2e-2 * (dw_true.abs().max().item() + 1e-6)


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    _run_pair(1000, 4096, 1)
    _run_pair(333, 2048, 2)          # second call: different shape, same built-in buffer


def test_noalloc_rejects_rows_beyond_the_builtin_buffer():
    from hippolm_b200.ops._ext import lib, ptr, stream_ptr
    fn = lib().hippo_rmsnorm_bwd_noalloc
    fn.restype = C.c_int
    t = torch.zeros(8, device="cuda")
    assert fn(ptr(t), ptr(t), ptr(t), ptr(t), ptr(t), ptr(t), C.c_longlong(4), 8200, stream_ptr()) == -22
    assert fn(ptr(t), ptr(t), ptr(t), ptr(t), ptr(t), ptr(t), C.c_longlong(4), 16384, stream_ptr()) == -22
