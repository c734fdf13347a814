"""Child process of ``test_reference_optim.py``: the reference's host-offloaded AdamW and Muon classes, run on the CPU from
the unmodified tree (page-locking, its compiled host kernels and the stream synchronisation patched out: none changes the
arithmetic). Takes a file with parameters and per-step gradients, writes the parameters after every step."""
import os
import sys
import types

os.environ["HIPPO_FUSED_FORCE_PYLOOP"] = "1"                      # the reference's own switch: plain PyTorch loops

import torch  # noqa: E402


def _patch():
    torch.Tensor.pin_memory = lambda self, *a, **k: self
    for name in ("empty", "zeros"):
        orig = getattr(torch, name)

        def f(*a, _orig=orig, **k):
            k.pop("pin_memory", None)
            return _orig(*a, **k)
        setattr(torch, name, f)
    torch.cuda.current_stream = lambda *a, **k: types.SimpleNamespace(synchronize=lambda: None)


def main():
    ref_root, inp, out = sys.argv[1], sys.argv[2], sys.argv[3]
    _patch()
    sys.path.insert(0, ref_root)
    from src.training.param_offload.adamw import CPUAdamW
    from src.training.param_offload.muon import CPUMuon
    from src.training.precision_config import PrecisionConfig
    case = torch.load(inp)
    prec = PrecisionConfig.from_dict({k: {"dtype": "fp32"} for k in
                                      ("model_weights", "gradients", "activations", "muon_momentum", "adamw_m", "adamw_v")})
    res = {"adamw": [], "muon": []}
    h = case["hyper"]
    pa = [torch.nn.Parameter(t.clone()) for t in case["adamw_params"]]
    opt = CPUAdamW(pa, lr=h["lr"], betas=(h["b1"], h["b2"]), eps=h["eps"], weight_decay=h["wd"], precision=prec)
    for grads in case["adamw_grads"]:
        for p, g in zip(pa, grads):
            opt.state[id(p)].grad.copy_(g.reshape(-1))
        opt.step()
        res["adamw"].append([p.detach().clone() for p in pa])
    pm = [torch.nn.Parameter(t.clone()) for t in case["muon_params"]]
    mu = CPUMuon(pm, lr=h["muon_lr"], momentum=h["momentum"], nesterov=True, ns_steps=5, weight_decay=h["muon_wd"], precision=prec)
    for grads in case["muon_grads"]:
        for p, g in zip(pm, grads):
            st = mu.state[id(p)]
            st.grad.copy_(g.reshape(st.grad.shape))
        mu.step()
        res["muon"].append([p.detach().clone() for p in pm])
    torch.save(res, out)


if __name__ == "__main__":
    main()
