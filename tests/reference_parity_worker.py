"""Child process of ``test_reference_parity.py``: runs the UNMODIFIED reference model (its single-GPU class, its vendored
Triton kernels executed on the CPU by Triton's interpreter) and this framework's model with the converted weights on
the same tokens, and prints the differences of the logits (and, when asked and where the reference's kernels allow it,
of the parameter gradients) as one JSON line. In evaluation mode with at most 64 tokens the reference's KDA layer takes its
token-recurrent kernel, the one its own tests use as the oracle; its chunked kernels use constructs the interpreter does
not run, so longer sequences and the backward pass are out of reach here.

Three shims make the reference tree run without a GPU, none of which touches its files: ``TRITON_INTERPRET=1``; a
``torch.cpu.device`` context (its kernels enter a device context by index); an autotuner that takes the first
configuration instead of timing them (timing needs a GPU driver)."""
import contextlib
import json
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
import torch  # noqa: E402

torch.cpu.device = lambda index=None: contextlib.nullcontext()
import triton.runtime.autotuner as _autotuner  # noqa: E402


def _run_first_config(self, *args, **kwargs):
    cfg = self.configs[0]
    self.best_config = cfg
    kw = dict(kwargs)
    kw.update(cfg.all_kwargs())
    return self.fn.run(*args, **kw)


_autotuner.Autotuner.run = _run_first_config


def main():
    ref_root, repo_root, kw, with_grad = sys.argv[1], sys.argv[2], json.loads(sys.argv[3]), sys.argv[4] == "1"
    dims = dict(vocab_size=128, hidden_size=64, num_heads=2, head_dim=32, num_layers=4, num_blocks=2, intermediate_size=128,
                tie_word_embeddings=True)
    dims.update(kw)
    n_tok = int(os.environ.get("PARITY_TOKENS", "40"))
    sys.path.insert(0, ref_root)
    from src.models.config import HippoConfig as RefConfig
    from src.models.model import HippoModel as RefModel
    torch.manual_seed(0)
    rm = RefModel(RefConfig(**dims))
    rm.train(with_grad)
    with torch.no_grad():
        for n, p in rm.named_parameters():
            if "attn_res.query" in n:
                p.normal_(0, 0.5)                       # zero-initialised: make the block mix non-trivial
            if "norm" in n and p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
    ids = torch.randint(0, 128, (1, n_tok))
    tgt = torch.randint(0, 128, (n_tok,))
    with torch.set_grad_enabled(with_grad):
        ref_logits = rm(ids)["logits"][0].float()
        if with_grad:
            torch.nn.functional.cross_entropy(ref_logits, tgt).backward()
    sd = {k: v.detach().float().clone() for k, v in rm.state_dict().items()}
    ref_grads = {n: p.grad.detach().float().clone() for n, p in rm.named_parameters() if p.grad is not None}
    # this framework's side: the reference's `src` / `scripts` packages leave the import path first
    sys.path.remove(ref_root)
    for m in [m for m in sys.modules if m in ("src", "scripts") or m.startswith("src.") or m.startswith("scripts.")]:
        del sys.modules[m]
    sys.path.insert(0, repo_root)
    from hippolm_b200.config import HippoConfig
    from hippolm_b200.models.model import HippoModel
    from hippolm_b200.train.convert import convert_reference_state_dict
    om = HippoModel(HippoConfig(full_attn_interval=0, **dims))
    om.train(with_grad)
    om.load_state_dict(convert_reference_state_dict(sd), strict=True)
    with torch.set_grad_enabled(with_grad):
        our_logits = om(ids[0])["logits"].float()
        if with_grad:
            torch.nn.functional.cross_entropy(our_logits, tgt).backward()
    out = {"max_abs_diff": float((our_logits - ref_logits).abs().max()), "max_abs_ref": float(ref_logits.abs().max())}
    if with_grad:
        # gradients through the same renaming as the weights
        conv = convert_reference_state_dict({k: ref_grads.get(k, torch.zeros_like(v)) for k, v in sd.items()
                                             if k != "lm_head.weight"})
        ours = {n: p.grad for n, p in om.state_dict(keep_vars=True).items() if getattr(p, "grad", None) is not None}
        rel = {}
        for k, g in conv.items():
            if k in ours and g.abs().max() > 0:
                rel[k] = float((ours[k].float() - g).norm() / (g.norm() + 1e-12))
        out["grad_rel_err_max"] = max(rel.values())
        out["grad_rel_err_worst"] = max(rel, key=rel.get)
        out["grads_compared"] = len(rel)
    print("PARITY " + json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
