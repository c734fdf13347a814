"""Eval server endpoints against a tiny CPU model, and the saved-tensor probe."""
import json
import urllib.request

import torch

from hippolm_b200.config import HippoConfig
from hippolm_b200.data.tokenizer import ByteTokenizer
from hippolm_b200.models.model import HippoModel
from hippolm_b200.serve.eval_server import EvalService, serve, build_model_and_load
from hippolm_b200.utils.vram import SavedTensorProbe


def _post(url, body):
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=60) as r:
        return json.loads(r.read())


def test_eval_server_roundtrip(tmp_path):
    cfg = HippoConfig(vocab_size=258, hidden_size=32, num_heads=2, head_dim=16, num_layers=2, num_blocks=1,
                      intermediate_size=64, full_attn_interval=2)
    m = HippoModel(cfg)
    p = tmp_path / "checkpoint_step_0.pt"
    torch.save({"step": 0, "model_state_dict": m.state_dict()}, p)
    model = build_model_and_load(str(p), cfg, torch.device("cpu"))
    srv = serve(EvalService(model, ByteTokenizer(), max_new_tokens=4), port=0)
    url = f"http://127.0.0.1:{srv.server_address[1]}"
    try:
        with urllib.request.urlopen(url + "/health", timeout=10) as r:
            assert json.loads(r.read())["status"] == "ok"
        with urllib.request.urlopen(url + "/v1/models", timeout=10) as r:
            assert json.loads(r.read())["data"][0]["id"] == "hippolm-b200"
        out = _post(url + "/v1/completions", {"prompt": "ab", "max_tokens": 3})
        assert out["object"] == "text_completion" and out["usage"]["prompt_tokens"] == 2
        assert 1 <= out["usage"]["completion_tokens"] <= 3
        out = _post(url + "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 2})
        assert out["choices"][0]["message"]["role"] == "assistant"
    finally:
        srv.shutdown()


def test_saved_tensor_probe():
    lin = torch.nn.Linear(8, 8)
    with SavedTensorProbe() as pr:
        lin(torch.randn(4, 8)).relu().sum().backward()
    assert pr.bytes > 0 and pr.count > 0
