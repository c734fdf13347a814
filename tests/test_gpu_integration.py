"""Integration runs of scripts/train.py on the test configs (``configs/test/*.yml``), as the reference does
with its smoke configs: no exception, finite decreasing-or-stable loss, a checkpoint with a non-empty
model_state_dict. Multi-GPU configs run only when enough devices are visible."""
import glob
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GPU_DIMS = ["--hidden_size", "256", "--num_heads", "4", "--head_dim", "64", "--intermediate_size", "512",
            "--vocab_size", "1024", "--seq_len", "512", "--batch_size", "4", "--doc_len_min", "64", "--doc_len_max", "400"]


def _run(cfg, extra, tmp_path, nproc=1, timeout=600):
    out = str(tmp_path / "out")
    cmd = [sys.executable, os.path.join(ROOT, "scripts", "train.py"), "--config", os.path.join(ROOT, "configs/test", cfg),
           "--output_dir", out] + GPU_DIMS + extra
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-3000:]
    runs = glob.glob(os.path.join(out, "*"))
    assert runs
    lines = [json.loads(l) for l in open(os.path.join(runs[0], "metrics.jsonl"))]
    assert lines and all(l["loss"] == l["loss"] and not l["found_inf"] for l in lines)
    return runs[0], lines


@pytest.mark.parametrize("cfg,extra", [("quick.yml", []), ("with_short_conv.yml", []), ("nvfp4.yml", []),
                                       ("quick.yml", ["--gradient_checkpointing", "true", "--micro_batch_size", "1024"]),
                                       ("nvfp4.yml", ["--ffn_nvfp4_no_bf16_master", "false"]),
                                       ("quick.yml", ["--offload_grads", "true", "--offload_optimizer", "true"])])
def test_single_gpu_configs(cfg, extra, tmp_path):
    _run(cfg, extra + ["--fixed_batch", "true", "--max_steps", "6"], tmp_path)


def test_checkpoint_config_writes_loadable_checkpoint(tmp_path):
    run, _ = _run("checkpoint.yml", [], tmp_path)
    cks = glob.glob(os.path.join(run, "checkpoints", "checkpoint_step_*.pt"))
    assert len(cks) == 1
    ck = torch.load(cks[0], map_location="cpu", weights_only=False)
    assert ck["model_state_dict"] and "layers.0.attn.qkv_proj.weight" in ck["model_state_dict"]


def test_loss_decreases_on_fixed_batch(tmp_path):
    _, lines = _run("quick.yml", ["--fixed_batch", "true", "--max_steps", "12"], tmp_path)
    assert lines[-1]["loss"] < lines[0]["loss"] - 0.5


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("cfg,extra", [("tp2.yml", []), ("dp2.yml", []), ("nvfp4_tp2.yml", []),
                                       ("dp2.yml", ["--dp_reduce_to_owner", "true"]),
                                       ("nvfp4_tp2.yml", ["--ffn_nvfp4_backward", "fp4"]),
                                       ("tp2.yml", ["--muon_ns_scope", "full"])])
def test_two_gpu_configs(cfg, extra, tmp_path):
    _run(cfg, extra + ["--max_steps", "4"], tmp_path)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_dp2_tp2_with_offload_and_checkpointing(tmp_path):
    _run("quick.yml", ["--tp_size", "2", "--dp_size", "2", "--nproc", "4", "--offload_grads", "true",
                       "--offload_optimizer", "true", "--gradient_checkpointing", "true", "--max_steps", "4"], tmp_path)
