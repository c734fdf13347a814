"""Eval server endpoints against a tiny CPU model, and the saved-tensor probe."""
import json
import urllib.request

import pytest
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


@pytest.mark.parametrize("kw", [
    dict(full_attn_interval=2),                                   # KDA + full-attention layers, two blocks
    dict(full_attn_interval=2, use_short_conv=True),              # + short-convolution tails
    dict(full_attn_interval=0, use_short_conv=True, conv_size=3, safe_gate=True),
    dict(full_attn_interval=4, num_layers=8, num_blocks=4, allow_neg_eigval=True),
])
def test_incremental_decoding_matches_full_reforward(kw):
    """generate() with the per-layer caches (KDA state, convolution tail, keys / values) produces the tokens and the
    logits of the full re-forward per token."""
    import torch
    from hippolm_b200.config import HippoConfig
    from hippolm_b200.models.model import HippoModel
    base = dict(vocab_size=96, hidden_size=32, num_heads=2, head_dim=16, num_layers=4, num_blocks=2, intermediate_size=64)
    base.update(kw)
    torch.manual_seed(0)
    m = HippoModel(HippoConfig(**base), seed=3).eval()
    prompt = torch.randint(0, 96, (11,))
    slow = m.generate(prompt, max_new_tokens=9, use_cache=False)
    fast = m.generate(prompt, max_new_tokens=9, use_cache=True)
    assert fast.tolist() == slow.tolist() and fast.numel() == 20
    # logits of every decode step against the full forward over the same prefix
    T0 = prompt.numel()
    with torch.no_grad():
        caches = m.new_decode_caches(T0 + 4)
        cu = torch.tensor([0, T0], dtype=torch.int32)
        h, states = m.hidden(prompt, cu_seqlens=cu, caches=caches)
        ids = prompt.clone()
        for step in range(4):
            full = m(ids, cu_seqlens=torch.tensor([0, ids.numel()], dtype=torch.int32))["logits"][-1]
            inc = m.lm_head.logits(h[-1:])[0]
            assert torch.allclose(inc, full, atol=2e-4, rtol=1e-4), (step, (inc - full).abs().max())
            nxt = full.argmax().reshape(1)
            ids = torch.cat([ids, nxt])
            h, states = m.hidden(nxt, cu_seqlens=torch.tensor([0, 1], dtype=torch.int32), kda_states=states,
                                 caches=caches, position_offset=ids.numel() - 1)
    # sampling path and EOS stop share the cached loop
    torch.manual_seed(1)
    s = m.generate(prompt, max_new_tokens=5, temperature=0.8, top_k=5)
    assert s.numel() <= T0 + 5 and s[:T0].tolist() == prompt.tolist()
    first = int(fast[T0])
    assert m.generate(prompt, max_new_tokens=9, eos_token_id=first).numel() == T0 + 1
