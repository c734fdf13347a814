"""Child process of ``test_reference_config.py``: the reference's model configuration and precision configuration classes
on a list of inputs; derived fields, autocast properties and accepted / refused inputs go to a JSON file."""
import json
import sys


def model_cases():
    base = dict(vocab_size=1000, hidden_size=256, num_heads=4, head_dim=64, num_layers=8, num_blocks=4, intermediate_size=512)
    out = [dict(base)]
    for kw in (dict(pack_chunk_size=0), dict(pack_chunk_size=1), dict(pack_chunk_size=64), dict(pack_chunk_size=65),
               dict(pack_chunk_size=100), dict(pack_chunk_size=128), dict(head_dim=128, pack_chunk_size=0),
               dict(num_layers=9, num_blocks=4), dict(num_layers=12, num_blocks=12), dict(num_blocks=0),
               dict(kda_mode="fused_recurrent"), dict(kda_mode="other"), dict(expand_v=2.0), dict(expand_v=0.5),
               dict(ffn_nvfp4=True, ffn_nvfp4_no_bf16_master=True), dict(ffn_nvfp4=False, ffn_nvfp4_no_bf16_master=True)):
        c = dict(base); c.update(kw); out.append(c)
    return out


def precision_cases():
    cls = ("model_weights", "gradients", "activations", "muon_momentum", "adamw_m", "adamw_v")
    return [None, {}, {k: {"dtype": "fp32"} for k in cls}, {k: {"dtype": "bf16"} for k in cls}, {"activations": {"dtype": "fp16"}},
            {"activations": {"dtype": "fp32"}, "adamw_v": {"dtype": "fp32"}}, {"model_weights": {"dtype": "float64"}},
            {"nonsense": {"dtype": "bf16"}}]


def main():
    ref_root, out = sys.argv[1], sys.argv[2]
    sys.path.insert(0, ref_root)
    from src.models.config import HippoConfig
    from src.training.precision_config import PrecisionConfig
    res = {"model": [], "precision": []}
    for kw in model_cases():
        try:
            c = HippoConfig(**kw)
            res["model"].append({"ok": True, "block_size": c.block_size, "pack_chunk_size": c.pack_chunk_size,
                                 "key_dim": getattr(c, "key_dim", None), "value_dim": getattr(c, "value_dim", None)})
        except Exception as ex:                                   # noqa: BLE001
            res["model"].append({"ok": False, "error": type(ex).__name__})
    for d in precision_cases():
        try:
            p = PrecisionConfig.from_dict(d)
            res["precision"].append({"ok": True, "autocast": bool(p.autocast_enabled), "autocast_dtype": str(p.autocast_dtype),
                                     "dict": p.to_dict()})
        except Exception as ex:                                   # noqa: BLE001
            res["precision"].append({"ok": False, "error": type(ex).__name__})
    with open(out, "w") as f:
        json.dump(res, f)


if __name__ == "__main__":
    main()
