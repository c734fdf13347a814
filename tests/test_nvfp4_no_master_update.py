"""No-master NVFP4 weights must keep learning: updates far below one code step survive in expectation (stochastic
rounding), and a weight that outgrows the tensor scale it was first quantised with is not clipped. CPU tests cover the
torch restatement and the module's chunk API; the GPU tests cover the fused device kernels of the Muon path."""
import pytest
import torch

from hippolm_b200.models.nvfp4_linear import NVFP4Linear
from hippolm_b200.ref import ops as ro


def test_stochastic_quantiser_is_unbiased_and_never_clips():
    torch.manual_seed(0)
    w = torch.randn(64, 256) * 0.05
    _, _, gs = ro.nvfp4_quantize(w)
    g = torch.Generator().manual_seed(1)
    acc = torch.zeros_like(w)
    n = 400
    for _ in range(n):
        p, s, _ = ro.nvfp4_quantize_stochastic(w, gs, g)
        acc += ro.nvfp4_dequantize(p, s, gs)
    mean = acc / n
    # per-element standard error of the mean is ~ step / sqrt(12 n) with step <= absmax / 3
    assert (mean - w).abs().max() < 0.25 * w.abs().max() / 3
    assert abs(float((mean - w).mean())) < 2e-5
    # round-to-nearest of the same tensor has a visible bias per element but none of the noise
    p, s, _ = ro.nvfp4_quantize_stochastic(w, gs, g)
    dq = ro.nvfp4_dequantize(p, s, gs)
    assert float(dq.abs().max()) >= float(w.abs().max()) * 0.999          # block scale rounded up: the maximum survives


def test_tiny_updates_accumulate_through_the_chunk_api():
    torch.manual_seed(0)
    lin = NVFP4Linear(256, 64, no_master=True)
    w0 = lin.material_chunk(0, 64).clone()
    ulp = float(w0.abs().max()) / 6 * 0.5                                 # smallest code step of the largest block
    step = ulp / 8
    upd = torch.ones(64, 256)
    for _ in range(200):
        lin.decay_and_apply_chunk(0, 64, upd, lr=step)                    # w <- w - step
    moved = float((lin.material_chunk(0, 64) - w0).mean())
    assert abs(moved - (-200 * step)) < 0.1 * 200 * step, (moved, -200 * step)
    lin2 = NVFP4Linear(256, 64, no_master=True, init_weight=w0)
    lin2.stochastic_rounding = False
    w20 = lin2.material_chunk(0, 64).clone()
    for _ in range(200):
        lin2.decay_and_apply_chunk(0, 64, upd, lr=step)
    stuck = float((lin2.material_chunk(0, 64) - w20).mean())
    assert abs(stuck) < 0.5 * 200 * step                                  # round-to-nearest loses most of the movement


def test_weight_growing_past_the_initial_scale_is_not_clipped():
    torch.manual_seed(1)
    lin = NVFP4Linear(64, 32, no_master=True)
    w = lin.material_chunk(0, 32).clone()
    big = w * 4.0
    lin.stochastic_rounding = False
    lin.commit_chunk(0, 16, big[:16])                                     # half the rows grow 4x
    out = lin.material_chunk(0, 32)
    assert float(out[:16].abs().max()) > 3.9 * float(w[:16].abs().max())
    assert (out[:16] - big[:16]).abs().max() < 0.3 * big[:16].abs().max() / 6 * 2
    assert (out[16:] - w[16:]).abs().max() < 0.3 * w.abs().max()          # untouched rows survive the rescale


@pytest.mark.gpu
def test_fused_update_kernel_tiny_steps_move_the_mean():
    from hippolm_b200.ops import muon_cuda as mc
    torch.manual_seed(0)
    lin = NVFP4Linear(1024, 256, no_master=True, device="cuda")
    w0 = lin.material_chunk(0, 256).clone()
    step = float(w0.abs().max()) / 6 * 0.5 / 8
    o = torch.ones(256, 1024, device="cuda", dtype=torch.bfloat16)
    for i in range(200):
        mc.nvfp4_apply_update(lin, [(0, 128, o[:128]), (128, 256, o[128:])], 1.0, step, seed=i)
    moved = float((lin.material_chunk(0, 256) - w0).mean())
    assert abs(moved + 200 * step) < 0.1 * 200 * step, (moved, -200 * step)
    # same seed, same result (counter-based random numbers)
    a, b = (NVFP4Linear(1024, 256, no_master=True, device="cuda", init_weight=w0) for _ in range(2))
    for m in (a, b):
        mc.nvfp4_apply_update(m, [(0, 256, o)], 1.0, step, seed=7)
    assert torch.equal(a.packed_weight, b.packed_weight) and torch.equal(a.scales.view(torch.uint8), b.scales.view(torch.uint8))
    # round-to-nearest loses the movement
    c = NVFP4Linear(1024, 256, no_master=True, device="cuda", init_weight=w0)
    c0 = c.material_chunk(0, 256).clone()
    for i in range(200):
        mc.nvfp4_apply_update(c, [(0, 256, o)], 1.0, step, seed=i, stochastic=False)
    assert abs(float((c.material_chunk(0, 256) - c0).mean())) < 0.5 * 200 * step


@pytest.mark.gpu
def test_fused_update_kernel_follows_a_growing_weight():
    from hippolm_b200.ops import muon_cuda as mc
    torch.manual_seed(2)
    lin = NVFP4Linear(512, 128, no_master=True, device="cuda")
    w0 = lin.material_chunk(0, 128).clone()
    gs0 = float(lin.global_scale)
    # w <- w - lr * o with o = -3 w / lr: the weight becomes 4 w, beyond the range of the first tensor scale
    o = (-3.0 * w0).bfloat16()
    mc.nvfp4_apply_update(lin, [(0, 128, o)], 1.0, 1.0, seed=1, stochastic=False)
    out = lin.material_chunk(0, 128)
    assert float(lin.global_scale) > 3.5 * gs0
    assert float(out.abs().max()) > 3.9 * float(w0.abs().max())
    rel = float((out - 4 * w0).norm() / (4 * w0).norm())
    assert rel < 0.15, rel
    # and shrinking back by the same factor restores the resolution
    o = (0.75 * out).bfloat16()
    mc.nvfp4_apply_update(lin, [(0, 128, o)], 1.0, 1.0, seed=2, stochastic=False)
    assert float(lin.global_scale) < 1.2 * gs0


def test_loss_decreases_with_only_the_nvfp4_ffn_trainable():
    """``configs/test/nvfp4.yml`` with every parameter frozen except the no-master FP4 feed-forward weights: the loss on
    a fixed batch must still go down, i.e. the FP4 weights really move under Muon's small steps."""
    import os
    from hippolm_b200.cli import parse_args
    from hippolm_b200.train.loop import setup_worker, train_step, teardown_worker
    from hippolm_b200.data.loaders import synthetic_loader
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        os.environ.pop(k, None)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    a = parse_args(["--config", os.path.join(root, "configs/test/nvfp4.yml"), "--trainable_regex", r"ffn\.",
                    "--max_steps", "1000", "--muon_lr", "0.02"])
    loader = synthetic_loader(a.batch_size, a.seq_len, a.vocab_size, 0, 16, 64, fixed=True)
    ctx = setup_worker(a, run_dir=None, data_iter=loader)
    assert len(ctx.adamw.entries) == 0 and len(ctx.muon.entries) > 0
    assert all(e.param is None for e in ctx.muon.entries)            # only no-master FP4 modules are optimised
    batch = next(loader)
    losses = []
    for _ in range(30):
        losses.append(float(train_step(ctx, batch)["loss"])); ctx.step += 1
    teardown_worker(ctx)
    assert losses[-1] < losses[0] - 0.05, losses


@pytest.mark.gpu
@pytest.mark.parametrize("no_master", [True, False])
def test_fp4_backward_dx_matches_dequantised_oracle(no_master):
    """``ffn_nvfp4_backward: fp4``: dX = Q(dY) Q(W^T)^T on the FP4 tensor cores against dY dq(W) in fp32 (cosine >= 0.99),
    dW unchanged, and the cached transposed encoding follows the weight through an optimizer update."""
    from hippolm_b200.parallel.linear import nvfp4_column_linear_sp, nvfp4_row_linear_sp
    from hippolm_b200.ops import muon_cuda as mc
    from hippolm_b200 import ops
    torch.manual_seed(0)
    T, K, N = 512, 1024, 768
    for fn in (nvfp4_column_linear_sp, nvfp4_row_linear_sp):
        lin = NVFP4Linear(K, N, no_master=no_master, device="cuda", dtype=torch.bfloat16)
        x = torch.randn(T, K, device="cuda").bfloat16()
        dy = torch.randn(T, N, device="cuda").bfloat16()
        grads = {}
        for mode in (False, True):
            lin.fp4_backward = mode
            lin.grad_w = None if no_master else None
            if not no_master:
                lin.weight.grad = None
            xi = x.clone().requires_grad_(True)
            fn(xi, lin).backward(dy)
            grads[mode] = (xi.grad.float(), (lin.grad_w if no_master else lin.weight.grad).float().clone())
        if no_master:
            wdq = ops.nvfp4_dequantize(lin.packed_weight, lin.scales, lin.global_scale, torch.float32)
        else:
            wdq = ops.nvfp4_dequantize(*ops.nvfp4_quantize(lin.weight.detach()), dtype=torch.float32)
        ref = dy.float() @ wdq
        cos = lambda a, b: float((a * b).sum() / (a.norm() * b.norm()))
        assert cos(grads[False][0], ref) > 0.999
        # no-master: W^T is a re-encoding of the stored FP4 weight. With a master the forward and the transposed
        # encoding are two independent roundings of the same bf16 weight, so the distance to dq(Q(W)) is one rounding more
        assert cos(grads[True][0], ref) > (0.99 if no_master else 0.985), cos(grads[True][0], ref)
        assert abs(float(grads[True][0].norm() / ref.norm()) - 1.0) < 0.05
        assert torch.equal(grads[True][1], grads[False][1])                     # dW is not touched by the option
    if no_master:
        p0 = lin.transposed_operands()[0].clone()
        o = torch.randn(N, K, device="cuda").bfloat16()
        mc.nvfp4_apply_update(lin, [(0, N, o)], 1.0, 0.05, seed=1)
        assert not torch.equal(lin.transposed_operands()[0], p0)                # cache invalidated by the update


@pytest.mark.gpu
def test_fp4_backward_dw_matches_fp32_oracle_and_accumulates():
    """``ffn_nvfp4_backward: fp4``: dW = Q(dY^T) Q(x^T)^T with the blocks along the token axis, against dY^T x in fp32
    (cosine >= 0.99), accumulated over micro-batches by the GEMM epilogue; and the transposed quantiser itself against
    the row quantiser applied to the transposed tensor (bit-identical codes and scales)."""
    from hippolm_b200 import ops
    from hippolm_b200.ops import nvfp4_cuda, fp4_gemm
    torch.manual_seed(0)
    T, K, N = 1024, 512, 384
    x = torch.randn(T, K, device="cuda").bfloat16()
    p_t, sf_t, gs_t = nvfp4_cuda.quantize_transposed(x)
    p_r, s_r, gs_r = nvfp4_cuda.quantize(x.t().contiguous())
    assert torch.equal(gs_t, gs_r) and torch.equal(p_t, p_r)
    assert torch.equal(sf_t, fp4_gemm.tile_scales(s_r, K, T))
    lin = NVFP4Linear(K, N, no_master=True, device="cuda", dtype=torch.bfloat16)
    lin.fp4_backward = lin.fp4_backward_dw = True
    ref = torch.zeros(N, K, device="cuda")
    for i in range(3):
        xi = torch.randn(T, K, device="cuda").bfloat16()
        dy = (torch.randn(T, N, device="cuda") * (1 + i)).bfloat16()
        lin.accumulate_grad_product(dy, xi)
        ref += dy.float().t() @ xi.float()
    g = lin.grad_w.float()
    cos = float((g * ref).sum() / (g.norm() * ref.norm()))
    assert cos > 0.99, cos
    assert abs(float(g.norm() / ref.norm()) - 1.0) < 0.05


@pytest.mark.gpu
def test_fp4_backward_loss_curve_tracks_bf16_backward():
    """50 steps on a fixed batch at small width (no-master NVFP4 FFN, everything trainable): the loss with the FFN
    backward on the FP4 tensor cores (dX and dW) follows the bf16-backward run."""
    import os
    from hippolm_b200.cli import build_parser
    from hippolm_b200.train.loop import setup_worker, train_step, teardown_worker
    from hippolm_b200.data.loaders import synthetic_loader
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        os.environ.pop(k, None)
    curves = {}
    for mode in ("bf16", "fp4"):
        a = build_parser().parse_args([])
        a.vocab_size, a.hidden_size, a.num_heads, a.head_dim = 2048, 512, 4, 128
        a.num_layers, a.num_blocks, a.intermediate_size = 4, 2, 1024
        a.ffn_nvfp4 = a.ffn_nvfp4_no_bf16_master = True
        a.ffn_nvfp4_backward = mode
        a.batch_size, a.seq_len, a.max_steps, a.seed = 4, 512, 1000, 1
        loader = synthetic_loader(a.batch_size, a.seq_len, a.vocab_size, 0, 128, 512, fixed=True)
        ctx = setup_worker(a, run_dir=None, data_iter=loader)
        batch = next(loader)
        losses = []
        for _ in range(50):
            losses.append(float(train_step(ctx, batch)["loss"])); ctx.step += 1
        teardown_worker(ctx)
        curves[mode] = losses
    b, f = curves["bf16"], curves["fp4"]
    assert b[-1] < b[0] - 1.0 and f[-1] < f[0] - 1.0, (b[0], b[-1], f[0], f[-1])
    assert abs(f[-1] - b[-1]) < 0.15 * max(b[0] - b[-1], 1e-6), (b[-1], f[-1])
