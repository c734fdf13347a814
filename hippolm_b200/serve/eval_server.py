"""OpenAI-compatible evaluation server on the standard library (``scripts/eval_server.py:94-575``).

Endpoints: ``GET /health``, ``GET /v1/models``, ``POST /v1/completions``, ``POST /v1/chat/completions``.
Greedy decoding (temperature 0) or temperature / top-k sampling through ``HippoModel.generate``; chat
requests are rendered with the tokenizer's chat template (ChatML for the byte tokenizer).
"""
from __future__ import annotations

import json
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
        ck = torch.load(ckpt_path, map_location=device, weights_only=False)
        sd = ck.get("model_state_dict", ck)
        if is_sharded_state_dict(sd):
            raise ValueError("checkpoint uses a per-device key layout; export the plain layers.N.* layout first")
        model.load_state_dict(sd, strict=True)
    return model.eval()


class EvalService:
    def __init__(self, model: HippoModel, tokenizer, model_name: str = "hippolm-b200", max_new_tokens: int = 256):
        self.model, self.tok, self.name, self.max_new = model, tokenizer, model_name, max_new_tokens
        self.lock = threading.Lock()

    def _generate(self, prompt_ids, max_tokens: int, temperature: float, top_k: int):
        dev = next(self.model.parameters()).device
        ids = torch.tensor(prompt_ids, dtype=torch.long, device=dev)
        with self.lock:
            out = self.model.generate(ids, min(max_tokens, self.max_new), temperature=temperature, top_k=top_k,
                                      eos_token_id=getattr(self.tok, "eos_token_id", None))
        new = out[len(prompt_ids):].tolist()
        eos = getattr(self.tok, "eos_token_id", None)
        finish = "stop" if (new and eos is not None and new[-1] == eos) else "length"
        return new, finish

    def complete(self, body: dict, chat: bool) -> dict:
        if chat:
            prompt = self.tok.apply_chat_template(body.get("messages", []), tokenize=False, add_generation_prompt=True)
        else:
            prompt = body.get("prompt", "")
            if isinstance(prompt, list):
                prompt = prompt[0] if prompt else ""
        ids = self.tok.encode(prompt, add_special_tokens=False)
        new, finish = self._generate(ids, int(body.get("max_tokens", 64)), float(body.get("temperature", 0.0)),
                                     int(body.get("top_k", 0)))
        text = self.tok.decode(new, skip_special_tokens=True)
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
