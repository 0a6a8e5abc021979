"""Serve recipe: OpenAI-compatible HTTP endpoints on top of the KV-cache decoder.

Endpoints and schemas follow optimus_dl/recipe/serve/base.py:47-428 of the reference
(``POST /v1/completions``, ``POST /v1/chat/completions`` with optional server-sent-event
streaming; temperature 0 means greedy; prompts longer than the model's context are cropped from
the left). Differences by design: tokens come from ``recipe.generation`` (one prefill, then
single-token steps on the cached keys / values instead of a full forward per token), ``top_p`` is
accepted, ``usage`` reports real token counts, ``/v1/completions`` can stream too, and
``GET /health`` answers liveness probes. The server handles one request at a time
(``http.server.HTTPServer``), as the reference does.
"""

from __future__ import annotations

import json
import logging
import time
from http.server import BaseHTTPRequestHandler, HTTPServer
from typing import Any, Iterator

import torch

from ...checkpoint import build_checkpoint_manager
from ...core.dtype import str_to_dtype
from ...models import build_model
from ...tokenizer import build_tokenizer
from ..generation import generate_stream, unwrap
from . import models as M

logger = logging.getLogger(__name__)


class RequestHandler(BaseHTTPRequestHandler):
    protocol_version = "HTTP/1.1"

    def log_message(self, fmt: str, *args: Any) -> None:  # route access logs through logging
        logger.debug("%s - %s", self.address_string(), fmt % args)

    # ------------------------------------------------------------------ plumbing
    def _json(self, status: int, payload: str) -> None:
        body = payload.encode("utf-8")
        self.send_response(status)
        self.send_header("Content-Type", "application/json")
        self.send_header("Content-Length", str(len(body)))
        self.end_headers()
        self.wfile.write(body)

    def _error(self, status: int, message: str) -> None:
        self._json(status, json.dumps({"error": message}))

    def _parse(self, schema: type) -> Any | None:
        try:
            n = int(self.headers.get("Content-Length", 0))
            data = json.loads(self.rfile.read(n) or b"{}")
        except (ValueError, json.JSONDecodeError):
            self._error(400, "Invalid JSON")
            return None
        try:
            return schema(**data)
        except Exception as err:  # pydantic.ValidationError
            self._error(422, str(err))
            return None

    def _sse_start(self) -> None:
        self.send_response(200)
        self.send_header("Content-Type", "text/event-stream")
        self.send_header("Cache-Control", "no-cache")
        self.send_header("Connection", "close")
        self.end_headers()
        self.close_connection = True

    def _sse(self, payload: str) -> None:
        self.wfile.write(f"data: {payload}\n\n".encode("utf-8"))
        self.wfile.flush()

    # ------------------------------------------------------------------ routes
    def do_GET(self) -> None:
        if self.path in ("/health", "/v1/health"):
            self._json(200, json.dumps({"status": "ok"}))
        elif self.path == "/v1/models":
            self._json(200, json.dumps({"object": "list", "data": [{"id": M.DEFAULT_MODEL_NAME, "object": "model"}]}))
        else:
            self._error(404, "Not Found")

    def do_POST(self) -> None:
        route = {"/v1/completions": self._completions, "/v1/chat/completions": self._chat}.get(self.path)
        if route is None:
            self._error(404, "Not Found")
            return
        try:
            route()
        except BrokenPipeError:
            logger.info("client went away")
        except Exception as err:
            logger.exception("request failed")
            try:
                self._error(500, str(err))
            except Exception:
                pass

    def _completions(self) -> None:
        req = self._parse(M.CompletionRequest)
        if req is None:
            return
        recipe: ServeRecipe = self.server.recipe
        prompt = req.prompt[0] if isinstance(req.prompt, list) else req.prompt
        now, rid = int(time.time()), f"cmpl-{time.time_ns()}"
        kw = dict(max_new_tokens=req.max_tokens, temperature=req.temperature, top_k=req.top_k, top_p=req.top_p)
        if req.stream:
            self._sse_start()
            for piece in recipe.generate_stream(prompt, **kw):
                chunk = M.CompletionChunk(id=rid, object="text_completion", created=now, model=req.model,
                                          choices=[M.CompletionChunkChoice(index=0, text=piece)])
                self._sse(chunk.model_dump_json())
            last = M.CompletionChunk(id=rid, object="text_completion", created=now, model=req.model,
                                     choices=[M.CompletionChunkChoice(index=0, text="", finish_reason=recipe.last_finish)])
            self._sse(last.model_dump_json())
            self._sse("[DONE]")
            return
        text = recipe.generate(prompt, **kw)
        resp = M.CompletionResponse(id=rid, object="text_completion", created=now, model=req.model,
                                    choices=[M.Choice(index=0, text=text, finish_reason=recipe.last_finish)],
                                    usage=recipe.last_usage)
        self._json(200, resp.model_dump_json())

    def _chat(self) -> None:
        req = self._parse(M.ChatCompletionRequest)
        if req is None:
            return
        recipe: ServeRecipe = self.server.recipe
        now, rid = int(time.time()), f"chatcmpl-{time.time_ns()}"
        kw = dict(max_new_tokens=req.max_tokens, temperature=req.temperature, top_k=req.top_k, top_p=req.top_p)
        if req.stream:
            self._sse_start()
            first = True
            for piece in recipe.generate_stream(req.messages, **kw):
                delta = M.Delta(role="assistant" if first else None, content=piece)
                first = False
                chunk = M.ChatCompletionChunk(id=rid, object="chat.completion.chunk", created=now, model=req.model,
                                              choices=[M.ChatChunkChoice(index=0, delta=delta)])
                self._sse(chunk.model_dump_json())
            done = M.ChatCompletionChunk(id=rid, object="chat.completion.chunk", created=now, model=req.model,
                                         choices=[M.ChatChunkChoice(index=0, delta=M.Delta(),
                                                                    finish_reason=recipe.last_finish)])
            self._sse(done.model_dump_json())
            self._sse("[DONE]")
            return
        text = recipe.generate(req.messages, **kw)
        resp = M.ChatCompletionResponse(
            id=rid, object="chat.completion", created=now, model=req.model,
            choices=[M.ChatChoice(index=0, message=M.ChatMessage(role="assistant", content=text),
                                  finish_reason=recipe.last_finish)], usage=recipe.last_usage)
        self._json(200, resp.model_dump_json())


class ServeRecipe:
    def __init__(self, cfg: Any):
        self.cfg = cfg
        self.model: torch.nn.Module | None = None
        self.tokenizer = None
        self.device: torch.device | None = None
        self.last_finish = "length"
        self.last_usage: dict = {"prompt_tokens": 0, "completion_tokens": 0, "total_tokens": 0}
        self._requests = 0
        self.httpd: HTTPServer | None = None

    # ------------------------------------------------------------------ setup
    def setup(self) -> None:
        c = self.cfg.common
        dev = str(c.get("device", "auto") if hasattr(c, "get") else c.device)
        self.device = torch.device(("cuda" if torch.cuda.is_available() else "cpu") if dev == "auto" else dev)
        ckpt, model_cfg = c.get("checkpoint_path"), c.get("model")
        assert (ckpt is not None) ^ (model_cfg is not None), \
            "Either checkpoint_path or model must be specified, but not both"
        if ckpt is not None:
            logger.info("loading model from checkpoint %s", ckpt)
            manager = build_checkpoint_manager({"_name": "base"}, output_path=str(ckpt))
            self.model, _ = manager.build_model_from_checkpoint(str(ckpt), device=self.device)
        else:
            logger.info("building model from config")
            self.model = build_model(model_cfg).to(self.device)
        dtype = c.get("dtype")
        if dtype is not None:
            self.model = self.model.to(str_to_dtype(dtype))
        elif self.device.type == "cuda":
            self.model = self.model.to(torch.bfloat16)
        self.model.eval()
        self.tokenizer = build_tokenizer(c.tokenizer)
        logger.info("model and tokenizer ready on %s", self.device)

    # ------------------------------------------------------------------ generation
    def _encode(self, prompt_or_messages: str | list) -> list[int]:
        if isinstance(prompt_or_messages, list) and prompt_or_messages and isinstance(prompt_or_messages[0], dict):
            return list(self.tokenizer.apply_chat_template(prompt_or_messages, tokenize=True, add_generation_prompt=True))
        if isinstance(prompt_or_messages, list):
            prompt_or_messages = prompt_or_messages[0] if prompt_or_messages else ""
        return list(self.tokenizer.encode(prompt_or_messages))

    @torch.no_grad()
    def generate_stream(self, prompt_or_messages: str | list, max_new_tokens: int = 50, temperature: float = 1.0,
                        top_k: int | None = None, top_p: float | None = None) -> Iterator[str]:
        """Yield text pieces. The full token list is re-decoded every step and only the new suffix
        is emitted, which is safe across multi-byte / multi-token characters."""
        ids = self._encode(prompt_or_messages)
        root = unwrap(self.model)
        limit = int(getattr(root.config, "sequence_length", None) or getattr(root.config, "block_size", 0) or 0)
        if limit and len(ids) + max_new_tokens > limit:
            room = max(limit - max_new_tokens, 1)
            ids = ids[-room:]
            max_new_tokens = min(max_new_tokens, max(limit - len(ids), 1))
        if not ids:
            ids = [self.tokenizer.bos_token_id or 0]
        x = torch.tensor([ids], dtype=torch.long, device=self.device)
        eos = getattr(self.tokenizer, "eos_token_id", None)
        self._requests += 1
        out: list[int] = []
        emitted = ""
        self.last_finish = "length"
        stream = generate_stream(self.model, x, max_new_tokens, temperature=max(float(temperature), 0.0), top_k=top_k,
                                 top_p=top_p, greedy=temperature <= 0, eos_token_id=None,
                                 use_kv_cache=bool(self.cfg.common.get("use_kv_cache", True)),
                                 seed=int(self.cfg.common.get("seed", 0)) + self._requests)
        for tok in stream:
            t = int(tok[0])
            if eos is not None and t == eos:
                self.last_finish = "stop"
                break
            out.append(t)
            text = self.tokenizer.decode(out)
            if len(text) > len(emitted) and not text.endswith("�"):
                yield text[len(emitted):]
                emitted = text
        text = self.tokenizer.decode(out) if out else ""
        if len(text) > len(emitted):
            yield text[len(emitted):]
        self.last_usage = {"prompt_tokens": len(ids), "completion_tokens": len(out), "total_tokens": len(ids) + len(out)}

    def generate(self, prompt_or_messages: str | list, max_new_tokens: int = 50, temperature: float = 1.0,
                 top_k: int | None = None, top_p: float | None = None) -> str:
        return "".join(self.generate_stream(prompt_or_messages, max_new_tokens, temperature, top_k, top_p))

    # ------------------------------------------------------------------ server
    def make_server(self) -> HTTPServer:
        httpd = HTTPServer((str(self.cfg.serve.host), int(self.cfg.serve.port)), RequestHandler)
        httpd.recipe = self
        self.httpd = httpd
        return httpd

    def run(self) -> None:
        self.setup()
        httpd = self.make_server()
        host, port = httpd.server_address[:2]
        logger.info("serving at http://%s:%s", host, port)
        logger.info("try: curl -s http://%s:%s/v1/completions -d '%s'", host, port,
                    json.dumps({"prompt": "Once upon a time", "max_tokens": 20, "temperature": 0.8}))
        logger.info("try: curl -s http://%s:%s/v1/chat/completions -d '%s'", host, port,
                    json.dumps({"messages": [{"role": "user", "content": "Hello!"}], "max_tokens": 20, "stream": True}))
        try:
            httpd.serve_forever()
        except KeyboardInterrupt:
            logger.info("shutting down")
        finally:
            httpd.server_close()
