"""YAML `extends`, optimizer flattening, CLI-over-YAML, WSD schedule, precision parsing."""
import os

import pytest
import torch

from hippolm_b200.cli import parse_args, _load_yaml_with_extends, _flatten_optimizer_overrides
from hippolm_b200.config import HippoConfig, PrecisionConfig
from hippolm_b200.optim.schedule import wsd_lr


def _w(p, text):
    with open(p, "w") as f:
        f.write(text)
    return str(p)


def test_extends_chain_child_wins_and_relative(tmp_path):
    os.makedirs(tmp_path / "sub")
    _w(tmp_path / "base.yml", "hidden_size: 128\nnum_layers: 8\nseed: 1\n")
    _w(tmp_path / "sub" / "mid.yml", "extends: ../base.yml\nnum_layers: 4\n")
    child = _w(tmp_path / "sub" / "child.yml", "extends: mid.yml\nseed: 7\n")
    cfg = _load_yaml_with_extends(child)
    assert cfg == {"hidden_size": 128, "num_layers": 4, "seed": 7}


def test_extends_cycle_detected(tmp_path):
    _w(tmp_path / "a.yml", "extends: b.yml\n")
    _w(tmp_path / "b.yml", "extends: a.yml\n")
    with pytest.raises(ValueError, match="circular"):
        _load_yaml_with_extends(str(tmp_path / "a.yml"))


def test_extends_is_shallow(tmp_path):
    _w(tmp_path / "base.yml", "optimizer:\n  adamw: {lr: 0.1, eps: 1e-6}\n")
    child = _w(tmp_path / "c.yml", "extends: base.yml\noptimizer:\n  adamw: {lr: 0.2}\n")
    cfg = _load_yaml_with_extends(child)
    assert cfg["optimizer"] == {"adamw": {"lr": 0.2}}


def test_optimizer_flattening_and_flat_key_wins():
    out = _flatten_optimizer_overrides({"optimizer": {"adamw": {"lr": 0.1, "beta2": 0.99}, "muon": {"momentum": 0.9}},
                                        "learning_rate": 0.5})
    assert out["learning_rate"] == 0.5 and out["adamw_beta2"] == 0.99 and out["muon_momentum"] == 0.9
    assert "optimizer" not in out
    with pytest.raises(ValueError):
        _flatten_optimizer_overrides({"optimizer": {"adamw": {"bogus": 1}}})


def test_cli_over_yaml_and_unknown_keys(tmp_path):
    cfg = _w(tmp_path / "c.yml", "hidden_size: 64\nmy_extra_key: hello\nprecision:\n  adamw_m: {dtype: fp32}\n"
                                 "optimizer:\n  muon: {lr: 0.05}\n")
    ns = parse_args(["--config", cfg])
    assert ns.hidden_size == 64 and ns.my_extra_key == "hello" and ns.muon_lr == 0.05
    assert ns.precision == {"adamw_m": {"dtype": "fp32"}}
    ns = parse_args(["--config", cfg, "--hidden_size", "96", "--muon_lr", "0.3"])
    assert ns.hidden_size == 96 and ns.muon_lr == 0.3


def test_repo_configs_parse():
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs")
    import glob
    names = sorted(os.path.relpath(p, root) for p in glob.glob(os.path.join(root, "*.yml")) + glob.glob(os.path.join(root, "test", "*.yml")))
    assert {"base.yml", "cpu_plumbing.yml", "hybrid_7b_tp8.yml", "hippolm_production.yml", "test/quick.yml"} <= set(names)
    for name in names:
        ns = parse_args(["--config", os.path.join(root, name)])
        cfg = HippoConfig.from_namespace(ns)
        assert cfg.num_layers % cfg.num_blocks == 0
    # the reference's production setup carried over: all layers KDA, its dimensions, optimizer and data keys
    ns = parse_args(["--config", os.path.join(root, "hippolm_production.yml")])
    cfg = HippoConfig.from_namespace(ns)
    assert set(cfg.layer_types()) == {"kda"} and (cfg.hidden_size, cfg.num_heads, cfg.head_dim) == (1536, 12, 128)
    assert cfg.tie_word_embeddings and cfg.use_short_conv and cfg.safe_gate and cfg.ffn_nvfp4_no_bf16_master
    assert (ns.muon_lr, ns.learning_rate, ns.seq_len, ns.micro_batch_size, ns.tp_size) == (0.02, 0.004, 262144, 16384, 2)
    assert ns.pretrain_multi_source and ns.use_modelscope and ns.checkpoint_interval == 100
    ns = parse_args(["--config", os.path.join(root, "hybrid_7b_tp8.yml")])
    cfg = HippoConfig.from_namespace(ns)
    assert cfg.layer_types().count("attn") == 8 and cfg.layer_types().count("kda") == 24
    assert cfg.ffn_nvfp4 and cfg.ffn_nvfp4_no_bf16_master and ns.tp_size == 8


def test_wsd_segments_and_endpoints():
    kw = dict(peak_lr=1.0, warmup_steps=10, decay_steps=20, max_steps=100)
    assert wsd_lr(0, **kw) == 0.0 and wsd_lr(5, **kw) == 0.5 and wsd_lr(10, **kw) == 1.0
    assert wsd_lr(79, **kw) == 1.0 and wsd_lr(80, **kw) == 1.0
    assert wsd_lr(99, **kw) == pytest.approx(0.0)
    assert wsd_lr(90, **kw) == pytest.approx(1.0 - 10 / 19)
    assert wsd_lr(-1, **kw) == 0.0 and wsd_lr(100, **kw) == 0.0
    assert wsd_lr(50, 1.0, 0, 0, 100) == 1.0 and wsd_lr(0, 1.0, 0, 0, 100) == 1.0
    assert wsd_lr(99, 1.0, 0, 10, 100, min_lr=0.1) == pytest.approx(0.1)
    assert wsd_lr(5, -1.0, 0, 10, 100) == -1.0


def test_precision_config():
    p = PrecisionConfig.from_dict({"model_weights": {"dtype": "fp32"}, "adamw_v": "bf16"})
    assert p.model_weights == torch.float32 and p.adamw_v == torch.bfloat16
    assert p.autocast_enabled and p.autocast_dtype == torch.bfloat16
    assert PrecisionConfig.from_dict(p.to_dict()) == p
    assert not PrecisionConfig.uniform("fp32").autocast_enabled
    with pytest.raises(ValueError):
        PrecisionConfig.from_dict({"bogus": {"dtype": "fp32"}})
    with pytest.raises(ValueError):
        PrecisionConfig.from_dict({"adamw_m": {"dtype": "int8"}})


def test_hippo_config_validation():
    with pytest.raises(ValueError):
        HippoConfig(num_layers=6, num_blocks=4)
    with pytest.raises(ValueError):
        HippoConfig(kda_mode="nope")
    with pytest.raises(ValueError):
        HippoConfig(ffn_nvfp4=False, ffn_nvfp4_no_bf16_master=True)
    c = HippoConfig(head_dim=100, pack_chunk_size=0)
    assert c.pack_chunk_size == 128 and c.block_size == 4


def test_launch_selects_gpus_and_tp_sim_skips_them():
    """``launch`` goes through ``select_gpus`` (``--min_gpu_memory_mb``); ``--tp_sim`` asks for no GPU."""
    import types
    import pytest
    from hippolm_b200.launch import pick_devices
    a = types.SimpleNamespace(min_gpu_memory_mb=10240, tp_sim=False)
    free = [50000, 1000, 50000, 50000, 100, 50000, 50000, 50000]
    assert pick_devices(a, 2, query=lambda: free, have_cuda=True) == [2, 3]
    assert pick_devices(a, 1, query=lambda: free, have_cuda=True) == [0]
    with pytest.raises(RuntimeError):
        pick_devices(a, 4, query=lambda: free, have_cuda=True)
    assert pick_devices(a, 2, query=lambda: free, have_cuda=False) is None
    a.tp_sim = True
    assert pick_devices(a, 2, query=lambda: free, have_cuda=True) is None


def test_every_flag_is_read_somewhere_and_unsupported_values_are_refused():
    """No parsed-but-ignored flag: each parser destination is read by the package (or the entry scripts), and the
    two switches that only exist for configuration compatibility refuse the unsupported value."""
    import glob
    import re
    import pytest
    from hippolm_b200.cli import build_parser
    from hippolm_b200.config import HippoConfig
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = ""
    for f in glob.glob(os.path.join(root, "hippolm_b200", "**", "*.py"), recursive=True) + \
            glob.glob(os.path.join(root, "scripts", "*.py")):
        if not f.endswith(os.path.join("hippolm_b200", "cli.py")):
            src += open(f).read()
    by_pattern = {"pretrain_en_multi_config", "pretrain_zh_multi_config", "pretrain_en_qa_config", "pretrain_zh_qa_config"}
    assert 'f"pretrain_{label}_config"' in src            # the four subset names are read through this pattern
    unused = [a.dest for a in build_parser()._actions
              if a.dest != "help" and a.dest not in by_pattern and not re.search(r"\b" + a.dest + r"\b", src)]
    assert unused == [], unused
    with pytest.raises(ValueError):
        HippoConfig(use_bias=True)
    with pytest.raises(ValueError):
        HippoConfig(conv_bias=True)
