"""Child process of ``test_reference_checkpoint.py``: the reference's own ``save_checkpoint`` / ``prune_old_checkpoints``
(``src/training/checkpoint.py``) from the unmodified tree. ``save``: its single-GPU model with its two optimizers
(page-locking patched out) written to a checkpoint file, next to the logits of that model on fixed tokens (its KDA layer
runs its token-recurrent Triton kernel under Triton's interpreter). ``prune``: pruning of a directory of file names."""
import contextlib
import json
import os
import sys
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"
os.environ["HIPPO_FUSED_FORCE_PYLOOP"] = "1"
import torch  # noqa: E402

torch.cpu.device = lambda index=None: contextlib.nullcontext()
torch.Tensor.pin_memory = lambda self, *a, **k: self
import triton.runtime.autotuner as _autotuner  # noqa: E402


def _run_first_config(self, *args, **kwargs):
    cfg = self.configs[0]
    self.best_config = cfg
    kw = dict(kwargs)
    kw.update(cfg.all_kwargs())
    return self.fn.run(*args, **kw)


_autotuner.Autotuner.run = _run_first_config

DIMS = dict(vocab_size=128, hidden_size=64, num_heads=2, head_dim=32, num_layers=4, num_blocks=2, intermediate_size=128,
            tie_word_embeddings=True, use_short_conv=True)


def main():
    ref_root, mode, where = sys.argv[1], sys.argv[2], sys.argv[3]
    sys.path.insert(0, ref_root)
    from src.training.checkpoint import prune_old_checkpoints, save_checkpoint
    if mode == "prune":
        # where: a directory with one sub-directory per value of keep_last_n, named after it
        print(json.dumps({"removed": {k: prune_old_checkpoints(Path(where) / k, int(k)) for k in sorted(os.listdir(where))}}))
        return
    from src.models.config import HippoConfig
    from src.models.model import HippoModel
    from src.training.param_offload.adamw import CPUAdamW
    from src.training.param_offload.muon import CPUMuon
    torch.manual_seed(11)
    m = HippoModel(HippoConfig(**DIMS)).eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "attn_res.query" in n:
                p.normal_(0, 0.5)
    mats = [p for n, p in m.named_parameters() if p.ndim == 2 and "embed" not in n and "lm_head" not in n]
    rest = [p for n, p in m.named_parameters() if not (p.ndim == 2 and "embed" not in n and "lm_head" not in n)]
    opts = {"muon": CPUMuon(mats, lr=0.02, momentum=0.95, nesterov=True, ns_steps=5, weight_decay=0.0),
            "adamw": CPUAdamW(rest, lr=0.004, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01)}
    path = save_checkpoint(m, opts, None, 7, 2.5, Path(where), keep_last_n=3)
    ids = torch.randint(0, 128, (1, 24), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        logits = m(ids)["logits"][0].float()
    torch.save({"ids": ids[0], "logits": logits}, os.path.join(where, "expected.pt"))
    print(json.dumps({"path": str(path)}))


if __name__ == "__main__":
    main()
