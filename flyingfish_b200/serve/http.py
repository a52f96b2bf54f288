"""OpenAI-compatible HTTP front end: ``POST /v1/completions`` and ``POST /v1/chat/completions``.

Behaviour follows the reference server (src/serve/http.rs): bind 127.0.0.1, bodies up to
128 MiB, greedy-only validation (temperature in {absent, 0}, top_p in {absent, 1}, no top_k / n>1 /
logit_bias / non-zero penalties / stop), unknown non-null parameters -> 400, wrong model name ->
404 ``model_not_found``, ``max_tokens`` and ``max_completion_tokens`` must agree (default 256),
chat template rendering failure -> 422, engine errors -> 500, ids ``cmpl-<secs>-<seq>`` /
``chatcmpl-<secs>-<seq>``, SSE streaming with a first role chunk, per-round text deltas, a final
chunk with ``finish_reason`` and ``data: [DONE]``. Too many requests in flight -> 409 (the
reference answers 409 whenever one request is running; here the bound is the scheduler's
in-flight limit). A client that disconnects aborts its request.

``allow_sampling=True`` additionally accepts temperature / top_p / top_k (an extension; off by
default so the validation matrix matches the reference).
"""
from __future__ import annotations

import asyncio
import base64
import itertools
import json
import time
from typing import Any

from aiohttp import web

from ..loaders.tokenizer import Detok
from .backend import Backend, Busy, EngineEvent, Unavailable

MAX_BODY = 128 * 1024 * 1024
TEMPLATE_ROLES = ("system", "user", "assistant", "tool")
COMMON_KEYS = {"temperature", "top_p", "top_k", "n", "logit_bias", "presence_penalty", "frequency_penalty",
               "max_tokens", "max_completion_tokens", "stop", "stream", "model"}


class HttpError(Exception):
    def __init__(self, status: int, message: str, etype: str = "invalid_request_error", code: str | None = None):
        self.status, self.message, self.etype, self.code = status, message, etype, code

    def response(self) -> web.Response:
        err: dict[str, Any] = {"message": self.message, "type": self.etype}
        if self.code:
            err["code"] = self.code
        return web.json_response({"error": err}, status=self.status)


def bad_request(msg: str) -> HttpError:
    return HttpError(400, msg)


def check_greedy(p: dict) -> None:
    t = p.get("temperature")
    if t is not None and t != 0:
        raise bad_request("greedy only: temperature must be 0 or absent")
    if p.get("top_p") is not None and p["top_p"] != 1:
        raise bad_request("greedy only: top_p must be 1 or absent")
    if p.get("top_k") is not None:
        raise bad_request("greedy only: top_k is not supported")
    if p.get("n") is not None and p["n"] != 1:
        raise bad_request("greedy only: n must be 1")
    if p.get("logit_bias") is not None:
        raise bad_request("greedy only: logit_bias is not supported")
    for k in ("presence_penalty", "frequency_penalty"):
        if p.get(k) is not None and p[k] != 0:
            raise bad_request(f"greedy only: {k} must be 0 or absent")
    if p.get("stop") is not None:
        raise bad_request("stop sequences are not supported")


def check_request(body: dict, allowed_extra: set[str], model_name: str) -> None:
    model = body.get("model")
    if model is not None and model != model_name:
        raise HttpError(404, f"model {model!r} is not served; the loaded model is {model_name!r}",
                        code="model_not_found")
    for k, v in body.items():
        if k not in COMMON_KEYS and k not in allowed_extra and v is not None:
            raise bad_request(f"unsupported parameter {k!r}")


def resolve_max_tokens(p: dict) -> int:
    a, b = p.get("max_tokens"), p.get("max_completion_tokens")
    for v in (a, b):
        if v is not None and (not isinstance(v, int) or isinstance(v, bool) or v < 0):
            raise bad_request("max_tokens must be a non-negative integer")
    if a is not None and b is not None and a != b:
        raise bad_request("max_tokens and max_completion_tokens must agree when both present")
    v = a if a is not None else b
    return 256 if v is None else v


class Server:
    def __init__(self, backend: Backend, tokenizer, model_name: str, chat_template: str | None = None,
                 capacity: int = 4096, allow_sampling: bool = False, image_placeholder: str | None = None):
        self.backend, self.tk, self.model_name = backend, tokenizer, model_name
        self.capacity = capacity
        # text of the image placeholder token (vision-language models only); None refuses image parts
        self.image_placeholder = image_placeholder
        self.allow_sampling = allow_sampling
        self._seq = itertools.count()
        self.template = None
        if chat_template:
            # the template comes from the checkpoint directory, i.e. from whoever published the model: render it
            # in the immutable sandbox so it cannot reach Python internals (``__class__``, ``__globals__`` ...)
            import jinja2
            from jinja2.sandbox import ImmutableSandboxedEnvironment
            env = ImmutableSandboxedEnvironment(loader=jinja2.BaseLoader(), trim_blocks=False, lstrip_blocks=False)

            def raise_exception(msg):
                raise jinja2.TemplateError(msg)
            env.globals["raise_exception"] = raise_exception
            self.template = env.from_string(chat_template)

    def app(self) -> web.Application:
        app = web.Application(client_max_size=MAX_BODY)
        app.router.add_post("/v1/completions", self.completions)
        app.router.add_post("/v1/chat/completions", self.chat_completions)
        app.router.add_get("/health", self.health)
        return app

    async def health(self, request: web.Request) -> web.Response:
        return web.json_response({"state": self.backend.state, "served": self.backend.served,
                                  "p50_ttft_ms": self.backend.p50_ttft_ms()})

    # -- parsing -------------------------------------------------------------------------------
    async def _json(self, request: web.Request) -> dict:
        try:
            body = await request.json()
        except Exception:
            raise bad_request("request body is not valid JSON")
        if not isinstance(body, dict):
            raise bad_request("request body must be a JSON object")
        return body

    def _prompt_ids(self, prompt) -> list[int]:
        if isinstance(prompt, str):
            return self.tk.encode(prompt)
        if isinstance(prompt, list) and all(isinstance(t, int) and not isinstance(t, bool) for t in prompt):
            return list(prompt)
        raise bad_request("prompt must be a string or a flat array of token ids")

    def _render_chat(self, messages, options: dict, images: list | None = None) -> str:
        """``images`` collects the decoded images of ``image_url`` parts in prompt order; each leaves the model's
        image placeholder in the text (models without a vision tower refuse image parts)."""
        if not isinstance(messages, list) or not messages:
            raise bad_request("messages must be a non-empty array")
        norm = []
        for m in messages:
            if not isinstance(m, dict) or m.get("role") not in TEMPLATE_ROLES:
                raise bad_request(f"message role must be one of {list(TEMPLATE_ROLES)}")
            content = m.get("content")
            if isinstance(content, list):
                parts = []
                for part in content:
                    if not isinstance(part, dict):
                        raise bad_request("content parts must be objects")
                    if part.get("type") == "text":
                        parts.append(str(part.get("text", "")))
                    elif part.get("type") == "image_url":
                        url = (part.get("image_url") or {}).get("url", "")
                        if not url.startswith("data:image/png;base64,") and not url.startswith("data:image/jpeg;base64,"):
                            raise bad_request("image_url must be a base64 data URL of a PNG or JPEG")
                        try:
                            raw = base64.b64decode(url.split(",", 1)[1], validate=True)
                        except Exception:
                            raise bad_request("image_url is not valid base64")
                        if self.image_placeholder is None or images is None:
                            raise bad_request("this model has no vision tower: image input is not supported")
                        try:
                            from .image import decode_image
                            images.append(decode_image(raw, url[5:].split(";")[0]))
                        except Exception as e:
                            raise bad_request(f"image_url does not decode: {e}")
                        parts.append(self.image_placeholder)
                    else:
                        raise bad_request(f"unsupported content part type {part.get('type')!r}")
                content = "".join(parts)
            elif content is not None and not isinstance(content, str):
                raise bad_request("message content must be a string or an array of parts")
            norm.append({**m, "content": content or ""})
        if self.template is None:
            raise HttpError(422, "the model directory has no chat template", etype="invalid_request_error")
        ctx = {"messages": norm, "add_generation_prompt": True, "bos_token": getattr(self.tk, "bos_token", "") or ""}
        if options.get("enable_thinking") is not None:
            ctx["enable_thinking"] = bool(options["enable_thinking"])
        try:
            return self.template.render(**ctx)
        except Exception as e:
            raise HttpError(422, f"chat template render: {e}")

    def _check_validity(self, ids: list[int], max_tokens: int) -> None:
        if not ids:
            raise bad_request("prompt is empty")
        vocab = getattr(self.tk, "vocab_size", None) or self.backend.engine.spec.vocab
        vocab = min(vocab, self.backend.engine.spec.vocab) if vocab else self.backend.engine.spec.vocab
        if any(t < 0 or t >= self.backend.engine.spec.vocab for t in ids):
            raise bad_request("prompt contains a token id outside the vocabulary")
        if len(ids) + max_tokens > self.capacity:
            raise bad_request(f"prompt ({len(ids)} tokens) + max_tokens ({max_tokens}) exceeds the context capacity "
                              f"{self.capacity}")

    # -- handlers ------------------------------------------------------------------------------
    async def completions(self, request: web.Request) -> web.StreamResponse:
        try:
            body = await self._json(request)
            if not self.allow_sampling:
                check_greedy(body)
            check_request(body, {"prompt"}, self.model_name)
            max_tokens = resolve_max_tokens(body)
            if body.get("prompt") is None:
                raise bad_request("prompt is required")
            ids = self._prompt_ids(body["prompt"])
            self._check_validity(ids, max_tokens)
            return await self._respond(request, ids, max_tokens, bool(body.get("stream")), chat=False)
        except HttpError as e:
            return e.response()

    async def chat_completions(self, request: web.Request) -> web.StreamResponse:
        try:
            body = await self._json(request)
            if not self.allow_sampling:
                check_greedy(body)
            check_request(body, {"messages", "chat_template_kwargs"}, self.model_name)
            max_tokens = resolve_max_tokens(body)
            opts = body.get("chat_template_kwargs") or {}
            if not isinstance(opts, dict) or any(k != "enable_thinking" for k in opts):
                raise bad_request("chat_template_kwargs only accepts enable_thinking")
            images: list = []
            text = self._render_chat(body.get("messages"), opts, images)
            ids = self.tk.encode(text)
            if images:
                token = self.backend.engine.spec.extra.get("image_token_id")
                if sum(1 for t in ids if t == token) != len(images):
                    raise bad_request("the rendered prompt does not hold one image placeholder token per image")
            self._check_validity(ids, max_tokens)
            return await self._respond(request, ids, max_tokens, bool(body.get("stream")), chat=True, images=images)
        except HttpError as e:
            return e.response()

    def _new_id(self, chat: bool) -> str:
        return f"{'chatcmpl' if chat else 'cmpl'}-{int(time.time())}-{next(self._seq)}"

    async def _respond(self, request: web.Request, ids: list[int], max_tokens: int, stream: bool,
                       chat: bool, images: list | None = None) -> web.StreamResponse:
        rid = self._new_id(chat)
        created = int(time.time())
        if max_tokens == 0:
            return web.json_response(self._final_body(rid, created, chat, "", "length", len(ids), 0))
        try:
            req, q = self.backend.add_request(ids, max_tokens, images=images)
        except Busy as e:
            return HttpError(409, str(e), etype="server_busy").response()
        except Unavailable as e:
            return HttpError(500, str(e), etype="server_error").response()
        detok = Detok(self.tk)
        if not stream:
            text, n_out, reason = "", 0, None
            try:
                while True:
                    ev: EngineEvent = await q.get()
                    if ev.kind == "tokens":
                        n_out += len(ev.tokens)
                        text += detok.push(self._strip_eos(ev.tokens))
                    elif ev.kind in ("done", "aborted"):
                        reason = ev.finish_reason
                        break
                    else:
                        return HttpError(500, ev.message or "engine failure", etype="server_error").response()
            except asyncio.CancelledError:
                self.backend.abort(req)
                raise
            text += detok.flush()
            return web.json_response(self._final_body(rid, created, chat, text, reason, len(ids), n_out))
        # ---- SSE ----
        resp = web.StreamResponse(status=200, headers={"Content-Type": "text/event-stream", "Cache-Control": "no-cache"})
        await resp.prepare(request)
        obj = "chat.completion.chunk" if chat else "text_completion"

        async def send(payload: dict | str) -> None:
            data = payload if isinstance(payload, str) else json.dumps(payload)
            await resp.write(f"data: {data}\n\n".encode())

        def chunk(delta_text: str | None, finish: str | None, role: bool = False) -> dict:
            if chat:
                delta: dict[str, Any] = {}
                if role:
                    delta["role"] = "assistant"
                if delta_text:
                    delta["content"] = delta_text
                choice = {"index": 0, "delta": delta, "finish_reason": finish}
            else:
                choice = {"index": 0, "text": delta_text or "", "finish_reason": finish}
            return {"id": rid, "object": obj, "created": created, "model": self.model_name, "choices": [choice]}

        try:
            if chat:
                await send(chunk(None, None, role=True))
            while True:
                ev = await q.get()
                if ev.kind == "tokens":
                    d = detok.push(self._strip_eos(ev.tokens))
                    if d:
                        await send(chunk(d, None))
                elif ev.kind in ("done", "aborted"):
                    tail = detok.flush()
                    if tail:
                        await send(chunk(tail, None))
                    await send(chunk(None, ev.finish_reason))
                    await send("[DONE]")
                    break
                else:
                    await send({"error": {"message": ev.message or "engine failure", "type": "server_error"}})
                    break
        except (ConnectionResetError, asyncio.CancelledError):
            self.backend.abort(req)      # client went away: stop generating for it
            raise
        await resp.write_eof()
        return resp

    def _strip_eos(self, toks: list[int]) -> list[int]:
        eos = set(self.backend.eos_ids)
        return [t for t in toks if t not in eos]

    def _final_body(self, rid: str, created: int, chat: bool, text: str, reason: str | None, n_prompt: int,
                    n_out: int) -> dict:
        usage = {"prompt_tokens": n_prompt, "completion_tokens": n_out, "total_tokens": n_prompt + n_out}
        if chat:
            choice = {"index": 0, "message": {"role": "assistant", "content": text}, "finish_reason": reason}
            obj = "chat.completion"
        else:
            choice = {"index": 0, "text": text, "finish_reason": reason}
            obj = "text_completion"
        return {"id": rid, "object": obj, "created": created, "model": self.model_name, "choices": [choice],
                "usage": usage}


def run(model, port: int = 8080, host: str = "127.0.0.1", allow_sampling: bool = False,
        chat_template: str | None = None, mtp_depth: int = 0, engine=None) -> None:
    """Blocking server entry point (``ff serve``). Ctrl-C shuts down gracefully."""
    eos = tuple(model.spec.extra.get("eos_token_ids", [model.spec.eos_token_id] if model.spec.eos_token_id is not None else []))
    from ..loaders.tokenizer import ByteTokenizer
    tk = model.tokenizer or ByteTokenizer(model.spec.vocab)
    if mtp_depth > 0:
        from .backend import MtpBackend
        backend = MtpBackend(model, mtp_depth, eos_ids=eos)
    else:
        # ``engine``: a stand-in for the model's engine with the same methods (the tensor-parallel leader proxy)
        backend = Backend(engine if engine is not None else model.engine, eos_ids=eos)
    backend.start()
    placeholder = None
    if getattr(model, "vision", None) is not None:
        placeholder = tk.decode([int(model.spec.extra["image_token_id"])])
    server = Server(backend, tk, model.name, chat_template or getattr(tk, "chat_template", None),
                    capacity=model.settings.capacity, allow_sampling=allow_sampling, image_placeholder=placeholder)
    try:
        web.run_app(server.app(), host=host, port=port, print=None)
    finally:
        backend.shutdown()
