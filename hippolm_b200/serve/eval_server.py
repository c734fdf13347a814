"""OpenAI-compatible evaluation server on the standard library (``scripts/eval_server.py:94-575``).

Endpoints: ``GET /health``, ``GET /v1/models``, ``GET /metrics`` (Prometheus text format: requests, tokens, decoding
passes, latency), ``POST /v1/completions``, ``POST /v1/chat/completions``.
Greedy decoding (temperature 0) or temperature / top-k sampling; chat requests are rendered with the tokenizer's chat
template (ChatML for the byte tokenizer). Requests that arrive while a batch is being decoded wait in a queue; the decoding
thread takes up to ``max_batch`` of them at a time and runs them through ``HippoModel.generate_batch`` together (one packed
prefill, then one token per request and step), each with its own length limit and sampling settings. The reference serves
one request at a time with a full re-forward per token.
"""
from __future__ import annotations

import json
import queue
import threading
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Optional

import torch

from ..config import HippoConfig
from ..models.model import HippoModel
from ..train.checkpoint import is_sharded_state_dict


def build_model_and_load(ckpt_path: Optional[str], cfg: HippoConfig, device: torch.device, dtype=torch.float32) -> HippoModel:
    model = HippoModel(cfg, device=device, dtype=dtype)
    if ckpt_path:
        from ..train import checkpoint as _ckpt
        man = _ckpt.read_manifest(ckpt_path)
        if man is not None and int(man.get("tp", 1)) > 1:
            # written by a tensor-parallel run: put the shards of the ranks back together
            from ..train.reshard import merge_checkpoint
            ck = merge_checkpoint(ckpt_path, cfg)
        else:
            ck = torch.load(ckpt_path, map_location=device, weights_only=False)
        sd = ck.get("model_state_dict", ck)
        from ..train.convert import convert_reference_state_dict, detect_layout
        if detect_layout(sd) != "native":
            # a checkpoint of the reference (single-GPU or one-device tensor-parallel layout): rename / fuse its tensors;
            # a multi-device tensor-parallel file is refused there with the reason
            sd = convert_reference_state_dict(sd)
        elif is_sharded_state_dict(sd):
            raise ValueError("checkpoint uses a per-device key layout; export the plain layers.N.* layout first")
        model.load_state_dict(sd, strict=True)
    return model.eval()


class _Pending:
    __slots__ = ("ids", "max_tokens", "temperature", "top_k", "top_p", "done", "new", "error")

    def __init__(self, ids, max_tokens, temperature, top_k, top_p=1.0):
        self.ids, self.max_tokens, self.temperature, self.top_k, self.top_p = ids, max_tokens, temperature, top_k, top_p
        self.done = threading.Event()
        self.new, self.error = None, None


class EvalService:
    def __init__(self, model: HippoModel, tokenizer, model_name: str = "hippolm-b200", max_new_tokens: int = 256,
                 max_batch: int = 8):
        self.model, self.tok, self.name, self.max_new = model, tokenizer, model_name, max_new_tokens
        self.max_batch = max(1, int(max_batch))
        self.batches_run = 0                 # decoding passes so far, and the largest number of requests one of them served
        self.largest_batch = 0
        self.stats = {"requests": 0, "failed": 0, "prompt_tokens": 0, "completion_tokens": 0, "latency_s": 0.0}
        self._stats_lock = threading.Lock()
        self._queue: "queue.Queue[_Pending]" = queue.Queue()
        self._batched = True
        self.lock = threading.Lock()
        self._worker = threading.Thread(target=self._decode_loop, name="eval-decode", daemon=True)
        self._worker.start()

    def close(self) -> None:
        """Stops the decoding thread (requests still in the queue are answered first)."""
        self._queue.put(None)
        self._worker.join(timeout=5.0)

    def _decode_loop(self):
        stop = False
        while not stop:
            first = self._queue.get()
            if first is None:
                return
            batch = [first]
            while len(batch) < self.max_batch:
                try:
                    nxt = self._queue.get_nowait()
                except queue.Empty:
                    break
                if nxt is None:
                    stop = True
                    break
                batch.append(nxt)
            try:
                dev = next(self.model.parameters()).device
                eos = getattr(self.tok, "eos_token_id", None)
                prompts = [torch.tensor(p.ids, dtype=torch.long, device=dev) for p in batch]
                with self.lock:
                    if self._batched:
                        outs = self.model.generate_batch(prompts, [p.max_tokens for p in batch],
                                                         [p.temperature for p in batch], [p.top_k for p in batch], eos,
                                                         [p.top_p for p in batch])
                    else:
                        outs = [self.model.generate(x, p.max_tokens, temperature=p.temperature, top_k=p.top_k,
                                                    eos_token_id=eos, top_p=p.top_p) for x, p in zip(prompts, batch)]
                self.batches_run += 1
                self.largest_batch = max(self.largest_batch, len(batch))
                for p, o in zip(batch, outs):
                    p.new = o[len(p.ids):].tolist()
            except Exception as ex:                                   # noqa: BLE001
                for p in batch:
                    p.error = ex
            for p in batch:
                p.done.set()

    def _generate(self, prompt_ids, max_tokens: int, temperature: float, top_k: int, top_p: float = 1.0):
        if not prompt_ids:                                            # nothing to condition on: start from the EOS token
            eos0 = getattr(self.tok, "eos_token_id", None)
            prompt_ids = [eos0 if eos0 is not None else 0]
        req = _Pending(list(prompt_ids), max(0, min(max_tokens, self.max_new)), temperature, top_k, top_p)
        self._queue.put(req)
        req.done.wait()
        if req.error is not None:
            raise req.error
        new = req.new
        eos = getattr(self.tok, "eos_token_id", None)
        finish = "stop" if (new and eos is not None and new[-1] == eos) else "length"
        return new, finish

    def metrics_text(self) -> str:
        """Counters of this service in the Prometheus text exposition format."""
        with self._stats_lock:
            st = dict(self.stats)
        rows = [("hippo_requests_total", "counter", st["requests"]), ("hippo_requests_failed_total", "counter", st["failed"]),
                ("hippo_prompt_tokens_total", "counter", st["prompt_tokens"]),
                ("hippo_completion_tokens_total", "counter", st["completion_tokens"]),
                ("hippo_request_latency_seconds_sum", "counter", round(st["latency_s"], 6)),
                ("hippo_decode_passes_total", "counter", self.batches_run),
                ("hippo_decode_largest_batch", "gauge", self.largest_batch),
                ("hippo_queue_depth", "gauge", self._queue.qsize())]
        return "".join(f"# TYPE {n} {t}\n{n} {v}\n" for n, t, v in rows)

    def complete(self, body: dict, chat: bool) -> dict:
        t0 = time.perf_counter()
        try:
            out = self._complete(body, chat)
        except Exception:
            with self._stats_lock:
                self.stats["requests"] += 1; self.stats["failed"] += 1
            raise
        with self._stats_lock:
            self.stats["requests"] += 1
            self.stats["prompt_tokens"] += out["usage"]["prompt_tokens"]
            self.stats["completion_tokens"] += out["usage"]["completion_tokens"]
            self.stats["latency_s"] += time.perf_counter() - t0
        return out

    def _complete(self, body: dict, chat: bool) -> dict:
        if chat:
            prompt = self.tok.apply_chat_template(body.get("messages", []), tokenize=False, add_generation_prompt=True)
        else:
            prompt = body.get("prompt", "")
            if isinstance(prompt, list):
                prompt = prompt[0] if prompt else ""
        ids = self.tok.encode(prompt, add_special_tokens=False)
        new, finish = self._generate(ids, int(body.get("max_tokens", 64)), float(body.get("temperature", 0.0)),
                                     int(body.get("top_k", 0)), float(body.get("top_p", 1.0)))
        text = self.tok.decode(new, skip_special_tokens=True)
        stop = body.get("stop")
        if stop:                                                      # the text ends before the first stop string
            cuts = [text.find(s) for s in ([stop] if isinstance(stop, str) else list(stop)) if s and text.find(s) >= 0]
            if cuts:
                text, finish = text[:min(cuts)], "stop"
        usage = {"prompt_tokens": len(ids), "completion_tokens": len(new), "total_tokens": len(ids) + len(new)}
        base = {"id": f"cmpl-{uuid.uuid4().hex[:12]}", "created": int(time.time()), "model": self.name, "usage": usage}
        if chat:
            base.update(object="chat.completion", choices=[{"index": 0, "finish_reason": finish,
                                                            "message": {"role": "assistant", "content": text}}])
        else:
            base.update(object="text_completion", choices=[{"index": 0, "finish_reason": finish, "text": text}])
        return base


def make_handler(svc: EvalService):
    class Handler(BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def _send(self, code: int, obj: dict):
            data = json.dumps(obj).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

        def do_GET(self):
            if self.path == "/health":
                self._send(200, {"status": "ok"})
            elif self.path == "/v1/models":
                self._send(200, {"object": "list", "data": [{"id": svc.name, "object": "model"}]})
            elif self.path == "/metrics":
                data = svc.metrics_text().encode()
                self.send_response(200)
                self.send_header("Content-Type", "text/plain; version=0.0.4")
                self.send_header("Content-Length", str(len(data)))
                self.end_headers()
                self.wfile.write(data)
            else:
                self._send(404, {"error": "not found"})

        def do_POST(self):
            try:
                n = int(self.headers.get("Content-Length", "0"))
                body = json.loads(self.rfile.read(n) or b"{}")
            except Exception as ex:
                return self._send(400, {"error": f"bad request: {ex}"})
            try:
                if self.path == "/v1/chat/completions":
                    self._send(200, svc.complete(body, chat=True))
                elif self.path == "/v1/completions":
                    self._send(200, svc.complete(body, chat=False))
                else:
                    self._send(404, {"error": "not found"})
            except Exception as ex:
                self._send(500, {"error": repr(ex)})
    return Handler


def serve(svc: EvalService, host: str = "127.0.0.1", port: int = 8000) -> ThreadingHTTPServer:
    srv = ThreadingHTTPServer((host, port), make_handler(svc))
    threading.Thread(target=srv.serve_forever, name="eval-server", daemon=True).start()
    return srv
