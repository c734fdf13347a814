"""Checkpoints of the reference into the plain layout: its single-GPU model (built from the unmodified reference tree when
that copy is present), its one-device tensor-parallel layout (restated from its module names), and the refusal of a
multi-device tensor-parallel file."""
import os
import sys

import pytest
import torch

from hippolm_b200.config import HippoConfig
from hippolm_b200.models.model import HippoModel
from hippolm_b200.train.convert import convert_checkpoint_file, convert_reference_state_dict, detect_layout

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
DIMS = dict(vocab_size=128, hidden_size=64, num_heads=2, head_dim=32, num_layers=4, num_blocks=2, intermediate_size=128,
            use_short_conv=True, tie_word_embeddings=True)


def _ours():
    return HippoModel(HippoConfig(full_attn_interval=0, **DIMS), seed=1)


def _reference_single_state_dict():
    """State dict of the reference's own single-GPU model class, in a child interpreter (its package names shadow ours)."""
    import subprocess
    code = (
        "import sys, torch; sys.path.insert(0, sys.argv[1]);"
        "from src.models.config import HippoConfig as C; from src.models.model import HippoModel as M;"
        f"torch.manual_seed(0); m = M(C(**{DIMS!r}));"
        "torch.save({k: v.detach().float().clone() for k, v in m.state_dict().items()}, sys.argv[2])")
    out = os.path.join(os.environ.get("TMPDIR", "/tmp"), f"hippo_ref_sd_{os.getpid()}.pt")
    r = subprocess.run([sys.executable, "-c", code, REF, out], capture_output=True, text=True, timeout=300, cwd="/tmp")
    if r.returncode != 0:
        pytest.skip("the reference tree could not build its model here: " + r.stderr[-300:])
    sd = torch.load(out)
    os.remove(out)
    return sd


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "src")), reason="no copy of the reference tree")
def test_reference_single_gpu_model_loads(tmp_path):
    sd = _reference_single_state_dict()
    assert detect_layout(sd) == "reference_single"
    conv = convert_reference_state_dict(sd)
    m = _ours()
    missing, unexpected = m.load_state_dict(conv, strict=True)
    assert not missing and not unexpected
    back = m.state_dict()
    i = 2
    q, k, v = (sd[f"layers.{i}.kda.attn.{n}_proj.weight"] for n in "qkv")
    assert torch.equal(back[f"layers.{i}.attn.qkv_proj.weight"], torch.cat([q, k, v], 0))
    assert torch.equal(back[f"layers.{i}.attn.fg_first.weight"],
                       torch.cat([sd[f"layers.{i}.kda.attn.f_proj.0.weight"], sd[f"layers.{i}.kda.attn.g_proj.0.weight"]], 0))
    assert torch.equal(back[f"layers.{i}.attn.k_conv1d.weight"], sd[f"layers.{i}.kda.attn.k_conv1d.weight"][:, 0, :])
    assert torch.equal(back[f"layers.{i}.ffn_norm.weight"], sd[f"layers.{i}.mlp_norm.weight"])
    assert torch.equal(back[f"layers.{i}.ffn.gate_up_proj.weight"],
                       torch.cat([sd[f"layers.{i}.ffn.gate_proj.weight"], sd[f"layers.{i}.ffn.up_proj.weight"]], 0))
    assert torch.equal(back["embed_tokens.weight"], sd["embed_tokens.weight"])
    # and through the file interface
    src, dst = tmp_path / "ref.pt", tmp_path / "ours.pt"
    torch.save({"step": 7, "model_state_dict": sd, "loss": 1.5}, src)
    info = convert_checkpoint_file(str(src), str(dst))
    assert info["layout"] == "reference_single" and info["step"] == 7
    ck = torch.load(dst)
    _ours().load_state_dict(ck["model_state_dict"], strict=True)
    with torch.no_grad():
        out = m(torch.randint(0, 128, (24,)))["logits"]
    assert torch.isfinite(out).all()


def _as_reference_tp(sd, device="0"):
    """The plain layout renamed the way the reference's tensor-parallel model names its per-device modules."""
    out = {}
    for k, v in sd.items():
        if k.startswith("layers."):
            _, i, rest = k.split(".", 2)
            rest = rest.replace("attn.", "kda.", 1) if rest.startswith("attn.") else rest
            rest = rest.replace("ffn_norm.", "mlp_norm.", 1)
            if rest.endswith("_conv1d.weight"):
                v = v.unsqueeze(1)
            out[f"layers_per_device.{device}.{i}.{rest}"] = v
        else:
            out[f"replicated_per_device.{device}.{k}"] = v
    return out


def test_reference_tp_layout_one_device_and_refusal_of_several():
    m = _ours()
    sd = m.state_dict()
    tp = _as_reference_tp(sd)
    tp["layers_per_device.0.0.ffn.gate_up_proj._scales_for_kernel"] = torch.zeros(3)        # derived cache: dropped
    assert detect_layout(tp) == "reference_tp"
    conv = convert_reference_state_dict(tp)
    assert set(conv) == set(sd) and all(torch.equal(conv[k], sd[k]) for k in sd)
    HippoModel(HippoConfig(full_attn_interval=0, **DIMS), seed=9).load_state_dict(conv, strict=True)
    two = dict(tp)
    two.update(_as_reference_tp(sd, device="1"))
    with pytest.raises(ValueError, match="one rank"):
        convert_reference_state_dict(two)
    assert detect_layout(sd) == "native" and convert_reference_state_dict(sd).keys() == sd.keys()


def test_eval_server_loads_a_reference_layout_checkpoint(tmp_path):
    from hippolm_b200.serve.eval_server import build_model_and_load
    m = _ours()
    p = tmp_path / "checkpoint_step_3.pt"
    torch.save({"step": 3, "model_state_dict": _as_reference_tp(m.state_dict())}, p)
    loaded = build_model_and_load(str(p), HippoConfig(full_attn_interval=0, **DIMS), torch.device("cpu"))
    for (k, a), (_, b) in zip(m.state_dict().items(), loaded.state_dict().items()):
        assert torch.equal(a, b), k
