"""Flash attention and chunked KDA kernels vs fp32 torch oracles (forward + backward)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-9)).item()


@pytest.mark.parametrize("T,H,DH,cu", [(256, 2, 128, [0, 256]), (333, 2, 64, [0, 100, 333]),
                                       (1000, 4, 128, [0, 64, 65, 700, 1000]),
                                       (2048, 2, 128, [0, 300, 1500, 2048])])
def test_causal_attention(T, H, DH, cu):
    from hippolm_b200 import ops
    from hippolm_b200.ref import ops as ro
    g = torch.Generator(device="cuda").manual_seed(T)
    q, k, v = (torch.randn(T, H, DH, device="cuda", generator=g).bfloat16() for _ in range(3))
    do = torch.randn(T, H, DH, device="cuda", generator=g).bfloat16()
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    ins = [t.clone().requires_grad_(True) for t in (q, k, v)]
    o = ops.causal_attention(ins[0], ins[1], ins[2], cu_t)
    o.backward(do)
    ref_in = [t.float().requires_grad_(True) for t in (q, k, v)]
    o2 = ro.causal_attention(ref_in[0], ref_in[1], ref_in[2], cu_t)
    o2.backward(do.float())
    assert _rel(o, o2) < 2e-2
    for a, b in zip(ins, ref_in):
        assert _rel(a.grad, b.grad) < 3e-2


def test_causal_attention_mma_sync_path(monkeypatch):
    """head_dim 128 through the mma.sync kernels (the path head_dim 64 always takes)."""
    from hippolm_b200.ops import attn_cuda
    monkeypatch.setattr(attn_cuda, "_USE_TC", False)
    test_causal_attention(1000, 4, 128, [0, 64, 65, 700, 1000])


@pytest.mark.parametrize("T,H,D,cu,gs", [(128, 2, 128, [0, 128], 1.0), (200, 2, 64, [0, 70, 200], 1.0),
                                         (700, 3, 128, [0, 100, 500, 700], 1.0), (512, 2, 128, [0, 512], 6.0)])
def test_kda_forward_backward(T, H, D, cu, gs):
    from hippolm_b200 import ops
    from hippolm_b200.ops import _ext
    from hippolm_b200.ref.kda import kda_chunked_anchored, l2norm
    torch.manual_seed(T)
    q = l2norm(torch.randn(T, H, D, device="cuda")).bfloat16().float()
    k = l2norm(torch.randn(T, H, D, device="cuda")).bfloat16().float()
    v = torch.randn(T, H, D, device="cuda").bfloat16().float()
    g = -torch.nn.functional.softplus(torch.randn(T, H, D, device="cuda")) * gs
    beta = torch.sigmoid(torch.randn(T, H, device="cuda"))
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    h0 = torch.randn(len(cu) - 1, H, D, D, device="cuda") * 0.1
    do = torch.randn(T, H, D, device="cuda").bfloat16().float()
    df = torch.randn(len(cu) - 1, H, D, D, device="cuda") * 0.1
    grads = []
    outs = []
    for impl in (0, 1):
        ins = [t.clone().requires_grad_(True) for t in (q, k, v, g, beta, h0)]
        if impl == 0:
            o, f = ops.kda(ins[0], ins[1], ins[2], ins[3], ins[4], 1.0, ins[5], cu_t, use_qk_l2norm=False)
        else:
            o, f = kda_chunked_anchored(ins[0], ins[1], ins[2], ins[3], ins[4], 1.0, ins[5], cu_t, False)
        ((o.float() * do).sum() + (f * df).sum()).backward()
        grads.append([t.grad for t in ins]); outs.append((o, f))
    assert _rel(outs[0][0], outs[1][0]) < 2e-2 and _rel(outs[0][1], outs[1][1]) < 2e-2
    for a, b in zip(*grads):
        assert _rel(a, b) < 3e-2
    torch.cuda.synchronize()
    assert _ext.device_status()[0] == 0


def test_kda_matches_token_recurrence():
    """Small case against the token-by-token oracle itself."""
    from hippolm_b200 import ops
    from hippolm_b200.ref.kda import kda_recurrent, l2norm
    torch.manual_seed(1)
    T, H, D = 96, 1, 64
    q = l2norm(torch.randn(T, H, D, device="cuda")).bfloat16().float()
    k = l2norm(torch.randn(T, H, D, device="cuda")).bfloat16().float()
    v = torch.randn(T, H, D, device="cuda").bfloat16().float()
    g = -torch.nn.functional.softplus(torch.randn(T, H, D, device="cuda"))
    beta = torch.sigmoid(torch.randn(T, H, device="cuda"))
    cu = torch.tensor([0, 40, 96], dtype=torch.int32, device="cuda")
    o, f = ops.kda(q, k, v, g, beta, 1.0, None, cu, use_qk_l2norm=False)
    o2, f2 = kda_recurrent(q.cpu(), k.cpu(), v.cpu(), g.cpu(), beta.cpu(), 1.0, None, cu.cpu().long())
    assert _rel(o.cpu(), o2) < 2e-2 and _rel(f.cpu(), f2) < 2e-2


@pytest.mark.parametrize("D", [64, 128])
def test_kda_recurrent_kernel_matches_oracle_and_chunk_kernels(D):
    """``kda_mode: fused_recurrent`` without gradients runs the token-recurrent kernel: same function as the token oracle
    and as the chunk kernels, including initial state, several sequences and the final state."""
    from hippolm_b200 import ops
    from hippolm_b200.ops import _ext
    from hippolm_b200.ref.kda import kda_recurrent, l2norm
    torch.manual_seed(D)
    T, H = 300, 3
    q = l2norm(torch.randn(T, H, D, device="cuda")).bfloat16().float()
    k = l2norm(torch.randn(T, H, D, device="cuda")).bfloat16().float()
    v = torch.randn(T, H, D, device="cuda").bfloat16().float()
    g = -torch.nn.functional.softplus(torch.randn(T, H, D, device="cuda"))
    beta = torch.sigmoid(torch.randn(T, H, device="cuda"))
    cu = torch.tensor([0, 1, 130, 300], dtype=torch.int32, device="cuda")
    h0 = torch.randn(3, H, D, D, device="cuda") * 0.1
    n0 = _ext.launch_count()
    with torch.no_grad():
        o, f = ops.kda(q, k, v, g, beta, 1.0, h0, cu, use_qk_l2norm=False, mode="fused_recurrent")
        assert _ext.launch_count() == n0 + 1                    # one kernel, not the chunk pipeline
        oc, fc = ops.kda(q, k, v, g, beta, 1.0, h0, cu, use_qk_l2norm=False, mode="chunk")
    o2, f2 = kda_recurrent(q.cpu(), k.cpu(), v.cpu(), g.cpu(), beta.cpu(), 1.0, h0.cpu(), cu.cpu().long())
    assert _rel(o.cpu(), o2) < 1e-2 and _rel(f.cpu(), f2) < 1e-3
    assert _rel(o, oc) < 2e-2 and _rel(f, fc) < 2e-2
    # with gradients required the same mode falls back to the differentiable chunk kernels
    qg = q.clone().requires_grad_(True)
    o3, _ = ops.kda(qg, k, v, g, beta, 1.0, h0, cu, use_qk_l2norm=False, mode="fused_recurrent")
    o3.float().sum().backward()
    assert qg.grad is not None and torch.isfinite(qg.grad).all()


def test_kda_skip_saved_recomputes_identical_gradients():
    """``kda_skip_aqk_akk_saved``: fewer saved activations, bit-identical outputs, and the same gradients up to the
    summation order of the backward kernels (their shared-memory float atomics are not ordered)."""
    from hippolm_b200 import ops
    from hippolm_b200.ref.kda import l2norm
    torch.manual_seed(5)
    T, H, D = 700, 3, 128
    q = l2norm(torch.randn(T, H, D, device="cuda")).bfloat16().float()
    k = l2norm(torch.randn(T, H, D, device="cuda")).bfloat16().float()
    v = torch.randn(T, H, D, device="cuda").bfloat16().float()
    g = -torch.nn.functional.softplus(torch.randn(T, H, D, device="cuda"))
    beta = torch.sigmoid(torch.randn(T, H, device="cuda"))
    cu = torch.tensor([0, 100, 500, 700], dtype=torch.int32, device="cuda")
    h0 = torch.randn(3, H, D, D, device="cuda") * 0.1
    do = torch.randn(T, H, D, device="cuda")
    res = []
    for skip in (False, True):
        ins = [t.clone().requires_grad_(True) for t in (q, k, v, g, beta, h0)]
        saved = []
        with torch.autograd.graph.saved_tensors_hooks(lambda t: (saved.append(t.numel() * t.element_size()), t)[1],
                                                      lambda t: t):
            o, f = ops.kda(ins[0], ins[1], ins[2], ins[3], ins[4], 1.0, ins[5], cu, use_qk_l2norm=False, skip_saved=skip)
        ((o.float() * do).sum() + f.sum()).backward()
        res.append((o, f, [t.grad for t in ins], sum(saved)))
    assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][1], res[1][1])
    for a, b in zip(res[0][2], res[1][2]):
        assert _rel(a, b) < 2e-3, _rel(a, b)
    assert res[1][3] < 0.6 * res[0][3], (res[0][3], res[1][3])


@pytest.mark.slow
def test_kda_at_benchmark_length_against_fp32_oracle():
    """The standalone-KDA benchmark layout on a 2-head slice: 32 768 tokens in 8 documents of random lengths, with an
    initial state and a gradient on the final state, forward and backward against the chunked fp32 oracle."""
    from hippolm_b200 import ops
    from hippolm_b200.ref.kda import kda_chunked_anchored, l2norm
    torch.manual_seed(0)
    T, H, D, docs = 32768, 2, 128, 8
    q = l2norm(torch.randn(T, H, D, device="cuda")).bfloat16().float()
    k = l2norm(torch.randn(T, H, D, device="cuda")).bfloat16().float()
    v = torch.randn(T, H, D, device="cuda").bfloat16().float()
    g = -torch.nn.functional.softplus(torch.randn(T, H, D, device="cuda"))
    beta = torch.sigmoid(torch.randn(T, H, device="cuda"))
    cuts = torch.sort(torch.randperm(T - 1)[:docs - 1] + 1).values
    cu = torch.cat([torch.zeros(1, dtype=torch.long), cuts, torch.tensor([T])]).to(torch.int32).cuda()
    h0 = torch.randn(docs, H, D, D, device="cuda") * 0.1
    do = torch.randn(T, H, D, device="cuda").bfloat16().float()
    df = torch.randn(docs, H, D, D, device="cuda") * 0.1
    outs, grads = [], []
    for impl in (0, 1):
        ins = [t.clone().requires_grad_(True) for t in (q, k, v, g, beta, h0)]
        fn = ops.kda if impl == 0 else kda_chunked_anchored
        o, f = fn(ins[0], ins[1], ins[2], ins[3], ins[4], 1.0, ins[5], cu, False) if impl else \
            fn(ins[0], ins[1], ins[2], ins[3], ins[4], 1.0, ins[5], cu, use_qk_l2norm=False)
        ((o.float() * do).sum() + (f * df).sum()).backward()
        outs.append((o, f)); grads.append([t.grad for t in ins])
    assert _rel(outs[0][0], outs[1][0]) < 2e-2 and _rel(outs[0][1], outs[1][1]) < 2e-2
    for a, b in zip(*grads):
        assert _rel(a, b) < 3e-2


def test_causal_attention_long_sequence():
    """One 8192-token sequence next to short ones, 4 heads of 128: forward and backward against the fp32 oracle."""
    test_causal_attention(10240, 4, 128, [0, 8192, 8200, 10240])


def test_kda_backward_is_reproducible():
    """Two backward passes over the same forward agree to rounding (the only unordered sums are shared-memory float
    atomics of the beta gradient) and the forward is bit-identical."""
    from hippolm_b200 import ops
    from hippolm_b200.ref.kda import l2norm
    torch.manual_seed(3)
    T, H, D = 1500, 4, 128
    q = l2norm(torch.randn(T, H, D, device="cuda")).bfloat16().float()
    k = l2norm(torch.randn(T, H, D, device="cuda")).bfloat16().float()
    v = torch.randn(T, H, D, device="cuda").bfloat16().float()
    g = -torch.nn.functional.softplus(torch.randn(T, H, D, device="cuda"))
    beta = torch.sigmoid(torch.randn(T, H, device="cuda"))
    cu = torch.tensor([0, 700, 1500], dtype=torch.int32, device="cuda")
    do = torch.randn(T, H, D, device="cuda")
    res = []
    for _ in range(2):
        ins = [t.clone().requires_grad_(True) for t in (q, k, v, g, beta)]
        o, f = ops.kda(ins[0], ins[1], ins[2], ins[3], ins[4], 1.0, None, cu, use_qk_l2norm=False)
        (o.float() * do).sum().backward()
        res.append((o, [t.grad for t in ins]))
    assert torch.equal(res[0][0], res[1][0])
    for a, b in zip(res[0][1], res[1][1]):
        assert _rel(a, b) < 1e-5                      # unordered sums: shared-memory float atomics (beta gradient)
