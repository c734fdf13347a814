"""AttnRes, NVFP4 quantiser, AdamW and cross-entropy kernels vs torch references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-9)).item()


@pytest.mark.parametrize("N,T,D,H", [(2, 100, 256, 4), (5, 300, 2048, 16), (9, 64, 4096, 32)])
def test_attn_res(N, T, D, H):
    from hippolm_b200 import ops
    from hippolm_b200.ref import ops as ro
    g = torch.Generator(device="cuda").manual_seed(N * T)
    srcs = [torch.randn(T, D, device="cuda", generator=g).bfloat16().requires_grad_(True) for _ in range(N)]
    q = (0.3 * torch.randn(H, D // H, device="cuda", generator=g)).bfloat16().requires_grad_(True)
    w = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).bfloat16().requires_grad_(True)
    dout = torch.randn(T, D, device="cuda", generator=g).bfloat16()
    out = ops.attn_res(srcs, q, w, 1e-6)
    out.backward(dout)
    s2 = [s.detach().float().requires_grad_(True) for s in srcs]
    q2, w2 = q.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    out2 = ro.attn_res(torch.stack(s2, 0), q2, w2, 1e-6)
    out2.backward(dout.float())
    assert _rel(out, out2) < 1e-2
    for a, b in zip(srcs, s2):
        assert _rel(a.grad, b.grad) < 3e-2
    assert _rel(q.grad, q2.grad) < 3e-2 and _rel(w.grad, w2.grad) < 3e-2


def test_nvfp4_quantize_byte_exact_and_roundtrip():
    from hippolm_b200 import ops
    from hippolm_b200.ref import ops as ro
    torch.manual_seed(0)
    w = torch.randn(256, 512, device="cuda") * 0.05
    w[3, :16] = 0.0
    p, s, gs = ops.nvfp4_quantize(w)
    p2, s2, gs2 = ro.nvfp4_quantize(w.cpu())
    assert torch.equal(gs.cpu(), gs2)
    assert torch.equal(s.view(torch.uint8).cpu(), s2.view(torch.uint8))
    assert torch.equal(p.cpu(), p2)
    d = ops.nvfp4_dequantize(p, s, gs, torch.float32)
    d2 = ro.nvfp4_dequantize(p2, s2, gs2)
    assert torch.equal(d.cpu(), d2)
    assert _rel(d, w) < 0.2
    pb, sb, gb = ops.nvfp4_quantize(w.bfloat16(), gs)
    assert pb.shape == p.shape


def test_adamw_kernel():
    from hippolm_b200 import ops
    torch.manual_seed(0)
    for dt in (torch.float32, torch.bfloat16):
        p = torch.randn(1000, device="cuda").to(dt); g = torch.randn(1000, device="cuda").to(dt)
        m = torch.zeros(1000, device="cuda").to(dt); v = torch.zeros(1000, device="cuda").to(dt)
        pc, gc, mc, vc = (t.cpu().clone() for t in (p, g, m, v))
        for step in (1, 2):
            ops.adamw_update(p, g, m, v, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, 0.5)
            ops.adamw_update(pc, gc, mc, vc, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, 0.5)
        assert _rel(p.cpu(), pc) < (1e-5 if dt == torch.float32 else 2e-2)


def test_lce_kernels():
    from hippolm_b200 import ops
    torch.manual_seed(0)
    C, D, V = 300, 256, 1000
    x = torch.randn(C, D, device="cuda").bfloat16()
    w = (0.05 * torch.randn(V, D, device="cuda")).bfloat16()
    tg = torch.randint(0, V, (C,), device="cuda"); tg[::7] = -1
    z, mx, se, tz = ops.lce_chunk_stats(x, w, tg)
    zr = x.float() @ w.float().t()
    assert _rel(z, zr) < 1e-2
    assert _rel(mx, zr.max(-1).values) < 1e-2
    lse = mx + se.log()
    assert _rel(lse, torch.logsumexp(zr, -1)) < 1e-2
    roww = (tg >= 0).float() / 10.0
    dz = ops.lce_chunk_grad(z, lse, tg, roww)
    ref = torch.softmax(z, -1)
    rows = (tg >= 0).nonzero(as_tuple=True)[0]
    ref[rows, tg[rows]] -= 1
    ref = ref * roww.unsqueeze(-1)
    assert (dz.float() - ref).abs().max() < 1e-3


def test_muon_fused_device_path_matches_reference():
    import torch.nn as nn
    from hippolm_b200.optim.optimizers import Muon
    from hippolm_b200.ref.ops import newton_schulz5
    torch.manual_seed(0)
    for shape in ((256, 512), (768, 256), (1024, 1536), (1536, 640)):     # the last two take the symmetric-tile GEMMs
        p = nn.Parameter(torch.randn(*shape, device="cuda").bfloat16())
        g = (0.1 * torch.randn(*shape, device="cuda")).bfloat16()
        p.grad = g.clone()
        opt = Muon(lr=0.1, momentum=0.9, weight_decay=0.01, momentum_dtype=torch.bfloat16)
        opt.add_param(p, "w")
        w0 = p.detach().float().clone()
        opt.step(grad_scale=0.5)
        m = 0.5 * g.float()
        u = 0.5 * g.float() + 0.9 * m
        ref = w0 * (1 - 0.1 * 0.01) - 0.1 * newton_schulz5(u, 5)
        assert _rel(opt.entries[0].exp_avg, m) < 1e-2
        assert (p.detach().float() - ref).abs().max() < 0.03          # bf16 weights of magnitude ~4


def test_nvfp4_fused_apply_update():
    """Fused dequantise -> update -> re-quantise of a no-master weight (round-to-nearest mode): the stored result is
    the updated tensor up to one FP4 rounding, with the tensor scale following the new absmax."""
    from hippolm_b200.models.nvfp4_linear import NVFP4Linear
    from hippolm_b200.ops import muon_cuda as mc
    torch.manual_seed(0)
    w = torch.randn(128, 256, device="cuda") * 0.05
    lin = NVFP4Linear(256, 128, no_master=True, device="cuda", init_weight=w)
    o = torch.randn(128, 256, device="cuda").bfloat16()
    w0 = lin.material_chunk(0, 128)
    mc.nvfp4_apply_update(lin, [(0, 64, o[:64]), (64, 128, o[64:])], 0.99, 0.01, seed=3, stochastic=False)
    w1 = lin.material_chunk(0, 128)
    target = w0 * 0.99 - 0.01 * o.float()
    assert float((w1 - target).norm() / target.norm()) < 0.12
    assert abs(float(lin.global_scale) - float(target.abs().max()) / (6 * 448)) < 1e-3 * float(lin.global_scale)
    assert float(w1.abs().max()) >= 0.99 * float(target.abs().max())


def test_muon_ragged_segment_stays_on_the_device_kernels():
    """A segment whose row count is not a multiple of 8 (the H/tp rows of the beta projection) is padded with zero rows
    and orthogonalised by the tcgen05 Newton-Schulz path; the result equals the fp32 oracle on the real rows."""
    import torch.nn as nn
    from hippolm_b200.optim.optimizers import Muon
    from hippolm_b200.ref.ops import newton_schulz5
    torch.manual_seed(1)
    p = nn.Parameter(torch.randn(4, 512, device="cuda").bfloat16())
    g = (0.1 * torch.randn(4, 512, device="cuda")).bfloat16()
    p.grad = g.clone()
    opt = Muon(lr=0.1, momentum=0.9, weight_decay=0.0, momentum_dtype=torch.bfloat16)
    opt.add_param(p, "b_proj")
    w0 = p.detach().float().clone()
    opt.step(grad_scale=1.0)
    u = g.float() + 0.9 * g.float()
    ref = w0 - 0.1 * newton_schulz5(u, 5)
    assert (p.detach().float() - ref).abs().max() < 0.03


@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (300, 264, 768), (1024, 512, 2048)])
def test_nvfp4_tensor_core_gemm(M, N, K):
    """Block-scaled FP4 MMA (kind::mxf4nvf4) vs the fp32 product of the dequantised operands."""
    from hippolm_b200 import ops
    from hippolm_b200.ops import fp4_gemm, _ext
    torch.manual_seed(M + K)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (0.05 * torch.randn(N, K, device="cuda")).bfloat16()
    xp, xs, xg = ops.nvfp4_quantize(x)
    wp, ws, wg = ops.nvfp4_quantize(w)
    y = fp4_gemm.fp4_matmul(xp, xs, xg, wp, ws, wg)
    ref = ops.nvfp4_dequantize(xp, xs, xg) @ ops.nvfp4_dequantize(wp, ws, wg).t()
    assert _rel(y, ref) < 1e-2
    y2 = ops.nvfp4_linear(x, wp, ws, wg, act_quant=True)
    assert _rel(y2, ref) < 1e-2
    torch.cuda.synchronize()
    assert _ext.device_status()[0] == 0


def test_sumsq_multi_one_launch():
    """The global gradient norm sums every tensor in one launch: mixed dtypes, ragged sizes, two output slots."""
    from hippolm_b200.ops import optim_cuda, _ext
    torch.manual_seed(0)
    ts = [torch.randn(n, device="cuda").to(dt) for n, dt in ((5, torch.float32), (2048, torch.bfloat16),
                                                             (2049, torch.bfloat16), (100003, torch.float32),
                                                             (4096 * 33, torch.bfloat16))]
    items = [(t, i % 2) for i, t in enumerate(ts)]
    out = torch.zeros(2, device="cuda")
    n0 = _ext.launch_count()
    optim_cuda.sumsq_multi(items, out)
    assert _ext.launch_count() == n0 + 1
    ref = [sum(float(t.float().pow(2).sum()) for t, s in items if s == k) for k in (0, 1)]
    assert abs(float(out[0]) - ref[0]) < 1e-3 * ref[0] and abs(float(out[1]) - ref[1]) < 1e-3 * ref[1]


def test_embed_gather_and_grad_kernels():
    """Embedding kernels against torch indexing: several vocabulary shards (here all in local memory, one pointer per
    shard as the peer path passes them), ids outside the vocabulary, repeated ids in the gradient."""
    from hippolm_b200.ops import embed_cuda
    torch.manual_seed(0)
    world, Vl, D, T = 4, 50, 256, 64
    shards = [torch.randn(Vl, D, device="cuda").bfloat16() for _ in range(world)]
    full = torch.cat(shards, 0)
    ids = torch.randint(0, world * Vl, (T,), device="cuda")
    ids[3] = ids[5] = ids[9]                                             # repeated id
    out = embed_cuda.gather(ids[16:32], [s.data_ptr() for s in shards], Vl, D)    # "rank 1" of 4: tokens 16..31
    assert torch.equal(out, full[ids[16:32]])
    bad = ids[:8].clone(); bad[2] = -1; bad[4] = world * Vl
    outb = embed_cuda.gather(bad, [s.data_ptr() for s in shards], Vl, D)
    assert float(outb[2].abs().max()) == 0 and float(outb[4].abs().max()) == 0 and torch.equal(outb[0], full[bad[0]])
    g = [torch.randn(T // world, D, device="cuda").bfloat16() for _ in range(world)]    # per-rank token shards
    gfull = torch.cat(g, 0).float()
    for r in range(world):
        dw = embed_cuda.grad(ids, [t.data_ptr() for t in g], T // world, r * Vl, Vl, D)
        ref = torch.zeros(Vl, D, device="cuda")
        sel = ((ids >= r * Vl) & (ids < (r + 1) * Vl)).nonzero(as_tuple=True)[0]
        ref.index_add_(0, ids[sel] - r * Vl, gfull[sel])
        assert (dw - ref).abs().max() < 1e-4
