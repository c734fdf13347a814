"""Property tests (hypothesis) of the host-side building blocks: the chunk-aligned packer, ``cu_seqlens`` slicing, the
learning-rate schedule, the NVFP4 reference quantiser, the byte-level BPE tokenizer and the sampling filters."""
import math

import torch
from hypothesis import given, settings, strategies as st

from hippolm_b200.data.packing import pack_chunk_aligned, slice_cu_seqlens, synthetic_packed_batch
from hippolm_b200.optim.schedule import wsd_lr

settings.register_profile("repo", max_examples=60, deadline=None, derandomize=True, database=None)
settings.load_profile("repo")


@given(st.lists(st.lists(st.integers(1, 50), min_size=0, max_size=300), min_size=0, max_size=12),
       st.sampled_from([64, 128]), st.integers(1, 4), st.integers(1, 4))
def test_packer_invariants(samples, chunk, rows_of_chunks, batch):
    seq_len = chunk * rows_of_chunks
    eos = 99
    ids, labels, cu = pack_chunk_aligned(samples, seq_len, chunk, batch, pad_id=0, eos_id=eos)
    assert ids.shape == labels.shape == (batch, seq_len)
    c = cu.tolist()
    assert c[0] == 0 and c[-1] == batch * seq_len and all(a < b for a, b in zip(c, c[1:]))
    assert all(b % seq_len == 0 or b % 64 == 0 for b in c)                  # documents end on chunk borders
    flat_i, flat_l = ids.reshape(-1), labels.reshape(-1)
    for s, e in zip(c, c[1:]):
        assert s // seq_len == (e - 1) // seq_len                          # no segment crosses a row
        assert int(flat_l[s]) == -100                                       # first token of a segment has no target
        seg_l = flat_l[s:e]
        keep = seg_l != -100
        # a target is always the token stored at its own position (labels are shifted later, by the model)
        assert torch.equal(seg_l[keep], flat_i[s:e][keep])
    # every placed document ends with EOS and nothing but documents and padding is in the batch
    n_eos_targets = int((flat_l == eos).sum())
    placed = sum(1 for _ in range(len(c) - 1))
    assert n_eos_targets <= placed


@given(st.lists(st.integers(1, 400), min_size=1, max_size=20), st.data())
def test_slice_cu_seqlens_consistency(lengths, data):
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0).tolist()))
    total = int(cu[-1])
    a = data.draw(st.integers(0, total))
    b = data.draw(st.integers(a, total))
    out = slice_cu_seqlens(cu, a, b).tolist()
    if a == b:
        assert out == [0]
        return
    assert out[0] == 0 and out[-1] == b - a and all(x < y for x, y in zip(out, out[1:]))
    inner = [int(x) - a for x in cu.tolist() if a < x < b]
    assert out[1:-1] == inner
    # slicing in two steps equals slicing once
    mid = data.draw(st.integers(a, b))
    left, right = slice_cu_seqlens(cu, a, mid).tolist(), slice_cu_seqlens(cu, mid, b).tolist()
    if a < mid < b:
        merged = sorted(set(left + [x + (mid - a) for x in right]))
        assert set(out) <= set(merged) and set(merged) - set(out) <= {mid - a}


@given(st.integers(1, 400), st.integers(0, 100), st.integers(0, 100), st.floats(1e-5, 1.0), st.floats(0.0, 0.5))
def test_wsd_schedule_shape(max_steps, warmup, decay, peak, min_frac):
    warmup, decay = min(warmup, max_steps), min(decay, max_steps)
    min_lr = peak * min_frac
    vals = [wsd_lr(s, peak, warmup, decay, max_steps, min_lr) for s in range(max_steps)]
    assert wsd_lr(-1, peak, warmup, decay, max_steps, min_lr) == 0.0
    assert wsd_lr(max_steps, peak, warmup, decay, max_steps, min_lr) == 0.0
    assert all(0.0 <= v <= peak * (1 + 1e-9) for v in vals)
    stable = [vals[s] for s in range(warmup, max_steps - decay)]
    assert all(abs(v - peak) < 1e-12 for v in stable)
    if warmup + decay <= max_steps:
        w = vals[:warmup]
        assert all(x <= y + 1e-15 for x, y in zip(w, w[1:]))                 # warm-up rises
        d = vals[max_steps - decay:]
        assert all(x >= y - 1e-15 for x, y in zip(d, d[1:]))                 # decay falls
        if decay >= 2:
            assert abs(d[-1] - min_lr) < 1e-9 * max(1.0, peak)               # and ends on the floor


@given(st.integers(1, 6), st.integers(1, 4), st.floats(1e-3, 1e3), st.integers(0, 2 ** 31 - 1))
def test_nvfp4_reference_roundtrip_error_bound(rows, blocks, scale, seed):
    from hippolm_b200.ref.ops import nvfp4_dequantize, nvfp4_quantize
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(rows, 16 * blocks, generator=g) * scale
    packed, sc, gs = nvfp4_quantize(w)
    assert packed.shape == (rows, 8 * blocks) and sc.shape == (rows, blocks)
    back = nvfp4_dequantize(packed, sc, gs)
    # per block: the error of an element is at most half the widest E2M1 step (2 between 4 and 6) times the stored block
    # scale, plus the rounding of the scale itself (e4m3: 2^-4 relative) applied to the block maximum
    blk, bb = w.view(rows, blocks, 16), back.view(rows, blocks, 16)
    scf = (sc.float() * gs).unsqueeze(-1)
    bound = scf * 1.0 + blk.abs().amax(-1, keepdim=True) * 2 ** -3 + 1e-12
    assert bool(((blk - bb).abs() <= bound).all())
    assert bool((torch.sign(bb) * torch.sign(blk) >= 0).all())                # a value never changes sign
    again = nvfp4_quantize(back, gs)
    assert torch.equal(nvfp4_dequantize(*again), back)                       # representable values are fixed points


@given(st.text(max_size=200))
def test_bpe_round_trip(text):
    from hippolm_b200.data.bpe import load_default
    tok = load_default()
    ids = tok.encode(text)
    assert all(0 <= i < tok.vocab_size for i in ids)
    assert tok.decode(ids, skip_special_tokens=False) == text.encode("utf-8", errors="replace").decode("utf-8", errors="replace") \
        or "<|" in text                                                      # text that spells a special token maps to it


@given(st.lists(st.floats(-8, 8, width=32), min_size=2, max_size=40), st.integers(0, 10), st.floats(0.05, 1.0),
       st.integers(0, 1000))
def test_sampling_filters_only_draw_allowed_tokens(vals, top_k, top_p, seed):
    m = _tiny_model()
    logits = torch.tensor(vals, dtype=torch.float32)
    vals = [v + 0.0 for v in logits.tolist()]                # the values the sampler sees (and -0.0 folded into 0.0)
    torch.manual_seed(seed)
    tok = int(m._sample(logits, 1.0, top_k, top_p))
    order = sorted(range(len(vals)), key=lambda i: -vals[i])
    if top_k > 0:
        kth = sorted(vals, reverse=True)[min(top_k, len(vals)) - 1]
        assert vals[tok] >= kth
    if top_p < 1.0:
        # the token lies inside the smallest prefix of the sorted distribution whose mass reaches top_p (ties aside)
        pool = [i for i in range(len(vals)) if top_k == 0 or vals[i] >= sorted(vals, reverse=True)[min(top_k, len(vals)) - 1]]
        z = sum(math.exp(vals[i]) for i in pool)
        srt = sorted(pool, key=lambda i: -vals[i])
        mass, allowed = 0.0, set()
        for i in srt:
            if mass >= top_p - 1e-6 and allowed:
                break
            allowed.add(i); mass += math.exp(vals[i]) / z
        assert tok in allowed or any(abs(vals[tok] - vals[j]) < 1e-6 for j in allowed)
    assert int(m._sample(logits, 0.0, top_k, top_p)) == order[0] or vals[int(m._sample(logits, 0.0, top_k, top_p))] == vals[order[0]]


_MODEL = []


def _tiny_model():
    if not _MODEL:
        from hippolm_b200.config import HippoConfig
        from hippolm_b200.models.model import HippoModel
        _MODEL.append(HippoModel(HippoConfig(vocab_size=64, hidden_size=32, num_heads=2, head_dim=16, num_layers=2,
                                             num_blocks=1, intermediate_size=64)).eval())
    return _MODEL[0]


@given(st.integers(64, 4096), st.integers(1, 64), st.integers(1, 300), st.integers(0, 10 ** 6))
def test_synthetic_batches_are_seeded_and_well_formed(n_tokens, lo, span, seed):
    hi = lo + span
    a = synthetic_packed_batch(n_tokens, 100, seed, lo, hi, row_len=min(n_tokens, 512))
    b = synthetic_packed_batch(n_tokens, 100, seed, lo, hi, row_len=min(n_tokens, 512))
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    ids, labels, cu = a
    c = cu.tolist()
    assert c[0] == 0 and c[-1] == n_tokens and all(x < y for x, y in zip(c, c[1:]))
    assert bool((labels[cu[:-1].long()] == -100).all())
    assert all(y - x <= hi for x, y in zip(c, c[1:]))
