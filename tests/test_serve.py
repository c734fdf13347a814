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
        with urllib.request.urlopen(url + "/metrics", timeout=10) as r:
            text = r.read().decode()
        vals = {l.split()[0]: float(l.split()[1]) for l in text.splitlines() if l and not l.startswith("#")}
        assert vals["hippo_requests_total"] == 2 and vals["hippo_requests_failed_total"] == 0
        assert vals["hippo_prompt_tokens_total"] >= 3 and 2 <= vals["hippo_completion_tokens_total"] <= 5
        assert vals["hippo_decode_passes_total"] == 2 and vals["hippo_request_latency_seconds_sum"] > 0
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


@pytest.mark.parametrize("kw", [dict(full_attn_interval=2), dict(full_attn_interval=2, use_short_conv=True)])
def test_batched_decoding_matches_one_sequence_at_a_time(kw):
    """generate_batch: prompts of different lengths packed into one prefill, one token per sequence and step, per-sequence
    limits and EOS; every sequence comes out as if it had been generated alone."""
    from hippolm_b200.config import HippoConfig
    from hippolm_b200.models.model import HippoModel
    base = dict(vocab_size=96, hidden_size=32, num_heads=2, head_dim=16, num_layers=4, num_blocks=2, intermediate_size=64)
    base.update(kw)
    torch.manual_seed(0)
    m = HippoModel(HippoConfig(**base), seed=4).eval()
    prompts = [torch.randint(0, 96, (n,)) for n in (1, 7, 12, 3)]
    limits = [6, 3, 8, 5]
    alone = [m.generate(p, lim, use_cache=False) for p, lim in zip(prompts, limits)]
    out = m.generate_batch(prompts, limits)
    for a, b in zip(alone, out):
        assert a.tolist() == b.tolist()
    # EOS stops one sequence early, the others run on
    eos = int(alone[2][prompts[2].numel() + 2])
    ref = [m.generate(p, lim, eos_token_id=eos, use_cache=False) for p, lim in zip(prompts, limits)]
    got = m.generate_batch(prompts, limits, eos_token_id=eos)
    for a, b in zip(ref, got):
        assert a.tolist() == b.tolist()
    assert got[2].numel() <= prompts[2].numel() + 3
    # mixed sampling settings: greedy rows are unaffected by a sampled neighbour
    torch.manual_seed(3)
    mixed = m.generate_batch(prompts[:2], 4, temperature=[0.0, 0.9], top_k=[0, 5])
    assert mixed[0].tolist() == m.generate(prompts[0], 4, use_cache=False).tolist()
    assert mixed[1].numel() == prompts[1].numel() + 4
    assert [t.numel() for t in m.generate_batch(prompts, 0)] == [p.numel() for p in prompts]


def test_eval_server_decodes_waiting_requests_together():
    """Requests that queue up while the decoder is busy are served by one batched decoding pass, and every response equals
    the one the request gets alone."""
    import threading
    import time
    cfg = HippoConfig(vocab_size=258, hidden_size=32, num_heads=2, head_dim=16, num_layers=2, num_blocks=1,
                      intermediate_size=64, full_attn_interval=2)
    model = HippoModel(cfg, seed=1).eval()
    svc = EvalService(model, ByteTokenizer(), max_new_tokens=6, max_batch=8)
    bodies = [{"prompt": "abc"[: 1 + i % 3] * (1 + i), "max_tokens": 2 + i % 4} for i in range(6)]
    alone = [svc.complete(b, chat=False)["choices"][0]["text"] for b in bodies]
    assert svc.largest_batch == 1
    results = [None] * len(bodies)

    def post(i):
        results[i] = svc.complete(bodies[i], chat=False)

    svc.lock.acquire()                          # the decoder takes the first request and then waits here
    try:
        threads = [threading.Thread(target=post, args=(i,)) for i in range(len(bodies))]
        threads[0].start()
        deadline = time.time() + 10
        while svc._queue.qsize() != 0 and time.time() < deadline:
            time.sleep(0.01)                    # request 0 has left the queue: it is the decoder's current batch
        for t in threads[1:]:
            t.start()
        while svc._queue.qsize() != len(bodies) - 1 and time.time() < deadline:
            time.sleep(0.01)
    finally:
        svc.lock.release()
    for t in threads:
        t.join(timeout=60)
    assert [r["choices"][0]["text"] for r in results] == alone
    assert svc.largest_batch == len(bodies) - 1
    svc.close()
    assert not svc._worker.is_alive()
    assert model.generate_batch([], 4) == []


def _tp_decode_worker(rank, world, port, out_path, kw):
    import os
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "HIPPO_TP_SIM": "1"})
    torch.set_num_threads(1)
    from hippolm_b200.parallel.mesh import init_distributed_from_env, init_mesh
    init_distributed_from_env(backend="gloo")
    init_mesh(tp=world)
    base = dict(vocab_size=96, hidden_size=32, num_heads=2, head_dim=16, num_layers=4, num_blocks=2, intermediate_size=64,
                full_attn_interval=2)
    base.update(kw)
    m = HippoModel(HippoConfig(**base), seed=4).eval()
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, 96, (n,), generator=g) for n in (5, 2, 8)]       # three sequences, 15 tokens: both odd
    limits = [4, 6, 3]
    batch = m.generate_batch(prompts, limits)
    alone = [m.generate(p, lim, use_cache=False) for p, lim in zip(prompts, limits)]
    one = m.generate(prompts[0], 4)
    torch.manual_seed(100 + rank)                                                 # different sampling streams per rank
    sampled = m.generate_batch(prompts[:2], 5, temperature=0.9, top_k=8)
    torch.save({"batch": [t.tolist() for t in batch], "alone": [t.tolist() for t in alone], "one": one.tolist(),
                "sampled": [t.tolist() for t in sampled]}, out_path + f".{rank}")
    import torch.distributed as dist
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("kw", [dict(), dict(use_short_conv=True)])
def test_incremental_decoding_under_tensor_parallelism(tmp_path, kw):
    """Two tensor-parallel ranks over gloo: the batch is filled up with dummy sequences so that every pass splits into even
    sequence-parallel shards; both ranks produce the tokens of the full re-forward, and sampled tokens come from rank 0."""
    import socket
    import torch.multiprocessing as mp
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    out = str(tmp_path / "tp")
    mp.spawn(_tp_decode_worker, args=(2, port, out, kw), nprocs=2, join=True)
    r0, r1 = torch.load(out + ".0"), torch.load(out + ".1")
    assert r0["batch"] == r0["alone"] == r1["batch"] == r1["alone"]
    assert r0["one"] == r0["alone"][0] == r1["one"]
    assert r0["sampled"] == r1["sampled"] and [len(t) for t in r0["sampled"]] == [10, 7]


def test_sampling_filters_and_stop_strings():
    cfg = HippoConfig(vocab_size=258, hidden_size=32, num_heads=2, head_dim=16, num_layers=2, num_blocks=1,
                      intermediate_size=64, full_attn_interval=2)
    m = HippoModel(cfg, seed=2).eval()
    logits = torch.tensor([4.0, 3.0, 2.0, -1.0, -2.0])
    torch.manual_seed(0)
    # nucleus of 0.6: softmax = [.66, .24, .09, ...] -> only token 0 survives; 0.8 -> tokens 0 and 1
    assert {int(m._sample(logits, 1.0, 0, 0.6)) for _ in range(50)} == {0}
    assert {int(m._sample(logits, 1.0, 0, 0.8)) for _ in range(200)} == {0, 1}
    assert {int(m._sample(logits, 1.0, 2, 1.0)) for _ in range(200)} == {0, 1}
    assert int(m._sample(logits, 0.0, 0, 0.5)) == 0
    svc = EvalService(m, ByteTokenizer(), max_new_tokens=8)
    full = svc.complete({"prompt": "hello", "max_tokens": 8}, chat=False)["choices"][0]
    assert full["finish_reason"] in ("length", "stop") and len(full["text"]) > 0
    if len(full["text"]) >= 3:
        cut = svc.complete({"prompt": "hello", "max_tokens": 8, "stop": [full["text"][2:4]]}, chat=False)["choices"][0]
        assert cut["finish_reason"] == "stop" and cut["text"] == full["text"][:full["text"].find(full["text"][2:4])]
    out = svc.complete({"prompt": "hello", "max_tokens": 4, "temperature": 0.7, "top_p": 0.9, "top_k": 20}, chat=False)
    assert out["usage"]["completion_tokens"] <= 4


def test_offline_perplexity_matches_per_document_cross_entropy(tmp_path):
    import math
    import torch.nn.functional as F
    from hippolm_b200.serve.perplexity import evaluate_perplexity, iter_documents
    cfg = HippoConfig(vocab_size=258, hidden_size=32, num_heads=2, head_dim=16, num_layers=2, num_blocks=1,
                      intermediate_size=64, full_attn_interval=2)
    m = HippoModel(cfg, seed=6).eval()
    tok = ByteTokenizer()
    docs = ["hello world, this is a document.", "x" * 150, "short", "another one with some more text in it " * 3, "ab"]
    (tmp_path / "a.txt").write_text("\n\n".join(docs[:3]))
    (tmp_path / "b.jsonl").write_text("\n".join(json.dumps({"content": d}) for d in docs[3:]))
    got = evaluate_perplexity(m, tok, iter_documents([tmp_path / "a.txt", tmp_path / "b.jsonl"]), seq_len=128, batch_rows=2)
    nll, n = 0.0, 0
    eos = tok.eos_token_id
    with torch.no_grad():
        for d in docs:
            ids = tok.encode(d, add_special_tokens=False) + ([eos] if eos is not None else [])
            for s in range(0, len(ids), 128):
                piece = torch.tensor(ids[s:s + 128])
                if piece.numel() < 2:
                    continue
                logits = m(piece)["logits"].float()
                nll += float(F.cross_entropy(logits[:-1], piece[1:], reduction="sum"))
                n += piece.numel() - 1
    assert got["tokens"] == n and got["documents"] == len(docs)
    assert abs(got["nll"] - nll / n) < 1e-4 and abs(got["perplexity"] - math.exp(nll / n)) < 1e-2 * math.exp(nll / n)


def test_generate_script(capsys):
    import os
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "scripts"))
    import importlib
    gen = importlib.import_module("generate")
    text = gen.main(["--config", os.path.join(root, "configs/test/quick.yml"), "--prompt", "hello", "--max_new_tokens", "5"])
    assert isinstance(text, str) and capsys.readouterr().out.strip() == text.strip()


def test_server_script_takes_the_reference_servers_options(tmp_path):
    """``scripts/eval_server.py`` as a process, started with the option names of the reference's server (``--tokenizer``,
    ``--model-id``, ``--device``, ``--dtype``, size overrides): it answers ``/v1/models`` with the given id and completes a
    prompt with the overridden model size."""
    import os
    import socket
    import subprocess
    import sys
    import time
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cfg = tmp_path / "m.yml"
    cfg.write_text("vocab_size: 1536\nhidden_size: 64\nnum_heads: 2\nhead_dim: 16\nnum_layers: 2\nnum_blocks: 1\n"
                   "intermediate_size: 64\n")
    proc = subprocess.Popen([sys.executable, os.path.join(root, "scripts", "eval_server.py"), "--config", str(cfg),
                             "--port", str(port), "--model-id", "probe-model", "--device", "cpu", "--dtype", "fp32",
                             "--hidden-size", "32", "--intermediate-size", "48", "--tokenizer", "builtin", "--max_new_tokens", "4"],
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    try:
        url = f"http://127.0.0.1:{port}"
        for _ in range(240):
            try:
                models = json.loads(urllib.request.urlopen(url + "/v1/models", timeout=2).read())
                break
            except Exception:                                       # noqa: BLE001
                assert proc.poll() is None, proc.stdout.read()[-3000:]
                time.sleep(0.5)
        else:
            raise AssertionError("the server did not come up")
        assert models["data"][0]["id"] == "probe-model"
        out = _post(url + "/v1/completions", {"prompt": "ab", "max_tokens": 3})
        assert out["usage"]["completion_tokens"] <= 3 and out["model"] == "probe-model"
    finally:
        proc.terminate()
        proc.wait(timeout=30)
