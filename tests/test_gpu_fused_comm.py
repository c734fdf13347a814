"""Fused all-gather->GEMM and GEMM->reduce-scatter kernels.

* bounded wait: one GPU, a peer that never arrives -> the kernel gives up within its cycle limit, records
  status code 5 and returns; the context stays usable (no trap, no hang).
* 2-GPU numerics: spawned ranks, fused kernels vs NCCL + plain GEMM, and the model-level switch.
"""
import ctypes as C
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_bounded_wait_reports_and_returns():
    from hippolm_b200.ops import _ext
    from hippolm_b200.ops._ext import lib, ptr, stream_ptr
    _ext.clear_device_status()
    rows, K, N = 128, 256, 256
    x = torch.randn(rows, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda").bfloat16()
    xg0 = torch.zeros(2 * rows, K, device="cuda", dtype=torch.bfloat16)      # this rank's gathered buffer
    xg1 = torch.zeros(2 * rows, K, device="cuda", dtype=torch.bfloat16)      # stands in for the absent peer
    f0 = torch.zeros(64, device="cuda", dtype=torch.int32)
    f1 = torch.zeros(64, device="cuda", dtype=torch.int32)
    y = torch.empty(2 * rows, N, device="cuda", dtype=torch.bfloat16)
    xs = (C.c_void_p * 2)(xg0.data_ptr(), xg1.data_ptr())
    fs = (C.c_void_p * 2)(f0.data_ptr(), f1.data_ptr())
    rc = lib().hippo_allgather_gemm_bf16(ptr(x), C.c_longlong(K), xs, fs, 2, 0, rows, ptr(w), C.c_longlong(K), ptr(y),
                                         C.c_longlong(N), N, K, 0, 4, C.c_uint(1), C.c_longlong(2_000_000), stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()                     # returns: the wait on shard 1 ran out after ~1 ms
    st = _ext.device_status()
    assert st[0] == 5 and st[1] == 1, st         # kWaitPeerFlag on row block 1 (first block of the absent source)
    ref = x.float() @ w.float().t()
    assert (y[:rows].float() - ref).abs().max() < 0.05 * ref.abs().max()     # own shard was still computed
    _ext.clear_device_status()
    z = torch.ones(4, device="cuda") * 2         # context still healthy
    assert float(z.sum()) == 8.0


def test_nvfp4_fused_kernels_single_rank():
    """The quantise-and-push kernel, the gathered-input FP4 GEMM and the FP4 GEMM -> reduce-scatter kernel with a
    world of one rank (every push lands in local buffers): layouts and epilogues against the plain FP4 GEMM."""
    from hippolm_b200.ops import _ext, nvfp4_cuda, fp4_gemm
    from hippolm_b200.ops._ext import lib, ptr, stream_ptr, check
    _ext.clear_device_status()
    rows, K, N = 384, 1024, 520
    x = torch.randn(rows, K, device="cuda").bfloat16()
    W = (0.05 * torch.randn(N, K, device="cuda")).bfloat16()
    wp, wsc, wgs = nvfp4_cuda.quantize(W)
    ref = fp4_gemm.gemm_nt(x, wp, wsc, wgs)
    buf = torch.zeros(rows * K * 9 // 16 + 256, device="cuda", dtype=torch.uint8)
    flags = torch.zeros(64, device="cuda", dtype=torch.int32)
    gs = torch.empty(1, device="cuda"); scratch = torch.empty(1, device="cuda")
    check(lib().hippo_nvfp4_tensor_scale(ptr(x), C.c_longlong(x.numel()), 1, ptr(scratch), ptr(gs), stream_ptr()), "scale")
    bufs = (C.c_void_p * 1)(buf.data_ptr()); fl = (C.c_void_p * 1)(flags.data_ptr())
    check(lib().hippo_nvfp4_quant_push(ptr(x), C.c_longlong(K), rows, K, ptr(gs), bufs, fl, 1, 0, stream_ptr()), "push")
    xp, xs, xg = nvfp4_cuda.quantize(x)
    assert torch.equal(buf[:rows * K // 2].view(rows, K // 2), xp)
    assert torch.equal(buf[rows * K // 2: rows * K // 2 + rows * K // 16], fp4_gemm.tile_scales(xs, rows, K))
    assert int(flags[0]) == K // 512 and int(flags[rows // 128 - 1]) == K // 512
    sfb = fp4_gemm.tile_scales(wsc, N, K)
    y = torch.empty(rows, N, device="cuda", dtype=torch.bfloat16)
    check(lib().hippo_allgather_gemm_nvfp4(ptr(buf), ptr(flags), 1, 0, rows, ptr(wp), ptr(sfb), ptr(wgs), ptr(y),
                                           C.c_longlong(N), N, K, C.c_uint(K // 512), C.c_longlong(0), stream_ptr()), "ag")
    assert torch.equal(y, ref)
    stage = torch.zeros(rows, N, device="cuda", dtype=torch.bfloat16)
    rflags = torch.zeros(8, device="cuda", dtype=torch.int32)
    out = torch.empty(rows, N, device="cuda", dtype=torch.bfloat16)
    sfa = fp4_gemm.tile_scales(xs, rows, K)
    st = (C.c_void_p * 1)(stage.data_ptr()); rf = (C.c_void_p * 1)(rflags.data_ptr())
    tiles = (rows // 128) * ((N + 127) // 128)
    check(lib().hippo_gemm_reduce_scatter_nvfp4(ptr(xp), ptr(sfa), ptr(xg), ptr(wp), ptr(sfb), ptr(wgs), st, rf, 1, 0, rows,
                                                ptr(out), N, K, C.c_uint(tiles * 4), C.c_longlong(0), stream_ptr()), "rs")
    torch.cuda.synchronize()
    assert torch.equal(out, ref)
    assert _ext.device_status()[0] == 0


_CHILD = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["HIPPO_ROOT"])
from hippolm_b200.parallel.mesh import init_distributed_from_env, init_mesh
from hippolm_b200.parallel import fused
from hippolm_b200.parallel.collectives import all_gather_dim0, reduce_scatter_dim0
from hippolm_b200.ops import _ext
dev = init_distributed_from_env()
mesh = init_mesh(tp=dist.get_world_size(), device=dev)
w_, r_ = mesh.tp, mesh.tp_rank
assert fused.setup(mesh, 4096, 4096)
ws = fused._STATE["ws"]
torch.manual_seed(1 + r_)
def rel(a, b): return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-9)).item()
for it in range(3):
    rows, K, N = 512, 1024, 768
    x = torch.randn(rows, K, device=dev).bfloat16(); W = (0.05 * torch.randn(N, K, device=dev)).bfloat16()
    xg, y = ws.allgather_gemm(x, W)
    xg_ref = all_gather_dim0(x, mesh.tp_group, w_)
    assert torch.equal(xg, xg_ref), "gathered activations differ"
    assert rel(y, xg_ref.float() @ W.float().t()) < 2e-2
    Wt = W.t().contiguous()
    _, y2 = ws.allgather_gemm(x, Wt, transpose_w=True)
    assert rel(y2, xg_ref.float() @ W.float().t()) < 2e-2
    # 512-row shards take the CTA-pair kernel (256-row pair tiles); 384-row shards take the one-CTA kernel
    x3 = torch.randn(384, K, device=dev).bfloat16()
    xg3, y3 = ws.allgather_gemm(x3, W)
    xg3_ref = all_gather_dim0(x3, mesh.tp_group, w_)
    assert torch.equal(xg3, xg3_ref) and rel(y3, xg3_ref.float() @ W.float().t()) < 2e-2
    T, Kl, N2 = 1024, 512, 1024
    a = torch.randn(T, Kl, device=dev).bfloat16(); W2 = (0.05 * torch.randn(N2, Kl, device=dev)).bfloat16()
    out = ws.gemm_reduce_scatter(a, W2)
    ref = reduce_scatter_dim0((a.float() @ W2.float().t()), mesh.tp_group, w_)
    assert rel(out, ref) < 2e-2, rel(out, ref)
    out2 = ws.gemm_reduce_scatter(a, W2.t().contiguous(), transpose_w=True)
    assert rel(out2, ref) < 2e-2
    # NVFP4: quantise-and-push -> FP4 GEMM, FP4 GEMM -> reduce-scatter, against the unfused FP4 GEMM
    from hippolm_b200.ops import nvfp4_cuda, fp4_gemm
    rows, K, N = 512, 1024, 768
    x = torch.randn(rows, K, device=dev).bfloat16(); W = (0.05 * torch.randn(N, K, device=dev)).bfloat16()
    dist.broadcast(W, 0)
    wp, wsc, wgs = nvfp4_cuda.quantize(W)
    y, kept = ws.nvfp4_allgather_gemm(x, wp, wsc, wgs, keep_gathered=True)
    assert y is not None
    xg_ref = all_gather_dim0(x, mesh.tp_group, w_)
    xq = ws.nvfp4_dequant_gathered(kept, rows * w_, K)
    xq_ref = torch.cat([nvfp4_cuda.dequantize(*nvfp4_cuda.quantize(xg_ref[i * rows:(i + 1) * rows].contiguous()),
                                              dtype=torch.bfloat16) for i in range(w_)], 0)
    assert torch.equal(xq, xq_ref), "kept FP4 activations differ"
    ref = torch.cat([fp4_gemm.gemm_nt(xg_ref[i * rows:(i + 1) * rows].contiguous(), wp, wsc, wgs) for i in range(w_)], 0)
    assert rel(y, ref) < 1e-3, ("fp4 ag", rel(y, ref))
    T, Kl, N2 = 1024, 512, 1024
    a = torch.randn(T, Kl, device=dev).bfloat16(); W2 = (0.05 * torch.randn(N2, Kl, device=dev)).bfloat16()
    w2p, w2s, w2g = nvfp4_cuda.quantize(W2)
    out = ws.nvfp4_gemm_reduce_scatter(a, w2p, w2s, w2g)
    assert out is not None
    ref = reduce_scatter_dim0(fp4_gemm.gemm_nt(a, w2p, w2s, w2g).float(), mesh.tp_group, w_)
    assert rel(out, ref) < 2e-2, ("fp4 rs", rel(out, ref))
    # vocab-parallel cross entropy: statistics pushed to every rank, merged inside the gradient kernel
    Cr, Vl = 256, 1000
    z = 3 * torch.randn(Cr, Vl, device=dev)
    tgt = torch.randint(0, Vl * w_, (Cr,), device=dev); dist.broadcast(tgt, 0)
    tgt[::7] = -100
    local = tgt - r_ * Vl
    own = (local >= 0) & (local < Vl) & (tgt >= 0)
    local_t = torch.where(own, local, torch.full_like(local, -1))
    valid = tgt >= 0
    roww = valid.float() / valid.sum()
    loss_raw = torch.zeros(1, device=dev)
    hd = ws.lce_stats_push(z, local_t)
    dz = ws.lce_grad_merge(hd, z, roww, loss_raw)
    zs = [torch.empty_like(z) for _ in range(w_)]
    dist.all_gather(zs, z, group=mesh.tp_group)
    zfull = torch.cat(zs, 1)
    lse = torch.logsumexp(zfull, 1)
    tz = zfull.gather(1, tgt.clamp(min=0)[:, None])[:, 0]
    ref_loss = ((lse - tz) * valid).sum()
    assert abs(loss_raw.item() - ref_loss.item()) < 2e-3 * abs(ref_loss.item()), (loss_raw.item(), ref_loss.item())
    pr = (zfull - lse[:, None]).exp()
    pr[valid, tgt[valid]] -= 1
    refdz = (pr * roww[:, None])[:, r_ * Vl:(r_ + 1) * Vl]
    assert (dz.float() - refdz).abs().max() < 2e-2 * roww.max(), "fused CE gradient"
torch.cuda.synchronize()
ws.check_status()
dist.barrier()
if r_ == 0: print("FUSED_OK")
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_kernels_two_gpus(tmp_path):
    script = tmp_path / "child.py"
    script.write_text(_CHILD)
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    env = dict(os.environ, HIPPO_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "FUSED_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
