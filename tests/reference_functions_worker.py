"""Child process of ``test_reference_functions.py``: calls the reference's own host-side functions (learning-rate
schedule, ``cu_seqlens`` slicing, chunk-aligned packer) on seeded random inputs and writes the results to a file; the test
then calls this framework's functions on the same inputs. Runs in its own interpreter because the reference's ``src`` and
``scripts`` packages would shadow same-named packages here."""
import random
import sys

import torch


def cases(seed=0):
    rng = random.Random(seed)
    wsd = []
    for _ in range(300):
        max_steps = rng.randint(1, 300)
        warm, dec = rng.randint(0, 120), rng.randint(0, 120)
        peak, mn = rng.choice([1.0, 0.02, 3e-4]), rng.choice([0.0, 1e-5, 1e-3])
        for step in {-1, 0, warm - 1, warm, warm + 1, max_steps - dec - 1, max_steps - dec, max_steps - 1, max_steps,
                     rng.randint(0, max_steps)}:
            wsd.append((step, peak, warm, dec, max_steps, mn))
    slices = []
    for _ in range(300):
        lens = [rng.randint(1, 200) for _ in range(rng.randint(1, 12))]
        cu = [0]
        for l in lens:
            cu.append(cu[-1] + l)
        a = rng.randint(0, cu[-1]); b = rng.randint(a, cu[-1])
        slices.append((cu, a, b))
        slices.append((cu, rng.choice(cu), rng.choice([c for c in cu if c >= 0])))
    packs = []
    for _ in range(120):
        chunk = rng.choice([64, 128])
        seq_len = chunk * rng.randint(1, 6)
        batch = rng.randint(1, 4)
        # at least one token per document: the reference gives an empty document a whole chunk of padding, here it is dropped
        docs = [[rng.randint(1, 90) for _ in range(rng.randint(1, int(seq_len * 1.3)))] for _ in range(rng.randint(0, 10))]
        packs.append((docs, seq_len, chunk, batch, 0, rng.choice([None, 99])))
    return wsd, slices, packs


def ns_inputs(seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(shape, generator=g) * scale for shape, scale in (((48, 96), 1.0), ((96, 48), 0.01), ((64, 64), 30.0))]


def main():
    ref_root, out = sys.argv[1], sys.argv[2]
    sys.path.insert(0, ref_root)
    from src.training.loop.support import wsd_lr, _slice_cu_seqlens
    from src.training.data.collate import pack_chunk_aligned
    wsd, slices, packs = cases()
    res = {"wsd": [wsd_lr(*c) for c in wsd], "slices": [], "packs": [], "ns": []}
    # Newton-Schulz orthogonalisation of the reference's Muon (fp16 inside), called on its unbound method
    import types
    from src.training.param_offload.muon import CPUMuon
    me = types.SimpleNamespace(_NS_COEFFS=CPUMuon._NS_COEFFS, ns_steps=5)
    for x in ns_inputs():
        res["ns"].append(CPUMuon._newton_schulz(me, x.clone()).float())
    for cu, a, b in slices:
        if b < a:
            a, b = b, a
        res["slices"].append(_slice_cu_seqlens(torch.tensor(cu), a, b).tolist())
    for docs, seq_len, chunk, batch, pad, eos in packs:
        ids, labels, cu = pack_chunk_aligned([list(d) for d in docs], seq_len, chunk, batch, pad_id=pad, eos_id=eos)
        res["packs"].append((ids, labels, cu))
    torch.save(res, out)


if __name__ == "__main__":
    main()
