"""FastAPI application exposing the reference's inference API.

Routes (specs/openapi/inference/api.yaml:57-688, zig/pkg/inference/src/server/server.zig:4651-4700):
``POST /ai/v1/embed`` = ``/ai/v1/embeddings``, ``POST /ai/v1/rerank``, ``POST /ai/v1/generate`` =
``/ai/v1/chat/completions`` (SSE when ``stream``; terminator ``data: [DONE]``), ``POST /ai/v1/chunk``,
``GET /ai/v1/models``, ``GET /ai/v1/metrics`` and ``/metrics``, ``GET /healthz``, ``GET /readyz``, plus
``POST /ai/v1/search`` for the vector indexes.  Errors are ``{"error", "message"}`` with 400 / 404 / 500 / 503;
a bounded, weighted request queue answers 503 when full (server/request_queue.zig:22-40).
"""
from __future__ import annotations

import asyncio
import base64
import json
import logging
import os
import re
import shutil
import struct
import threading
import time
import uuid
from typing import Dict, List, Optional

import torch
from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, Response, StreamingResponse

from .. import _native as N
from ..index.codec import decode_vectors
from ..pipelines.chunking import chunk_text
from ..pipelines.embedding import INPUT_TYPE_ALIASES
from ..runtime.sampling_params import SamplingParams
from ..runtime.scheduler import QueueFull
from ..utils import logs as L
from . import schemas as S
from .cache import ResultCache
from .metrics import Metrics
from .model_manager import ModelManager, ModelNotFound
from .._native import device_of as N_device_of


class QueueTimeout(QueueFull):
    """The request waited longer than request_timeout for admission (answered 504, not 503)."""


class RequestQueue:
    """Weighted admission: ``max_units`` of work in flight, ``max_waiting`` callers queued behind it."""

    def __init__(self, max_units: int = 64, max_waiting: int = 256):
        # 0 means unlimited for either bound (the configuration file's convention)
        self.max_units = max_units if max_units > 0 else 1 << 30
        self.max_waiting = max_waiting if max_waiting > 0 else 1 << 30
        self.units, self.waiting = 0, 0
        self._cv = threading.Condition()

    def acquire(self, units: int = 1, timeout: float = 300.0) -> None:
        units = min(units, self.max_units)
        with self._cv:
            if self.units + units > self.max_units and self.waiting >= self.max_waiting:
                raise QueueFull("request queue is full")
            self.waiting += 1
            try:
                ok = self._cv.wait_for(lambda: self.units + units <= self.max_units, timeout)
                if not ok:
                    raise QueueTimeout("timed out waiting for a slot")
                self.units += units
            finally:
                self.waiting -= 1

    def release(self, units: int = 1) -> None:
        with self._cv:
            self.units -= min(units, self.max_units)
            self._cv.notify_all()


class _HbcAdapter:
    """HBC tree behind the table's ``add`` / ``search`` calls: the first batch bulk-builds the tree, later ones are
    online inserts."""

    def __init__(self, dim: int, metric: str):
        from ..index.hbc import HBCConfig

        self.cfg = HBCConfig(dim, "l2_squared" if metric in ("l2", "l2_squared", "euclidean") else metric)
        self.idx = None

    def add(self, vectors, ids):
        from ..index.hbc import HBCIndex

        if self.idx is None:
            self.idx = HBCIndex.bulk_build(vectors, self.cfg, ids=ids)
        else:
            self.idx.insert(vectors, ids)

    def search(self, queries, k, effort: float = 0.5):
        from ..index.distance import resolve_search_effort
        from ..index.flat import SearchResult

        if self.idx is None:
            return SearchResult(torch.full((1, k), float("inf")), torch.full((1, k), -1, dtype=torch.int64))
        width, eps = resolve_search_effort(k, effort, self.idx.vectors.shape[0])
        ids, dists = self.idx.search(queries[0], k, search_width=width, epsilon=eps)
        pad = k - len(ids)
        return SearchResult(torch.tensor([list(dists) + [float("inf")] * pad]),
                            torch.tensor([list(ids) + [-1] * pad], dtype=torch.int64))


def _err(status: int, code: str, message: str) -> JSONResponse:
    return JSONResponse(status_code=status, content={"error": code, "message": message})


def create_app(manager: Optional[ModelManager] = None, indexes: Optional[Dict[str, object]] = None,
               max_concurrent_requests: int = 64, max_queue_size: int = 256,
               request_timeout_s: float = 0.0, result_cache_ttl_s: float = 120.0,
               api_key: Optional[str] = None, content_security=None, data_dir: Optional[str] = None) -> FastAPI:
    """``data_dir``: tables are kept under ``<data_dir>/tables/<name>/`` (their definition in ``table.json``, their
    documents and embeddings in a log-structured merge store) and come back when the server starts again; without
    it tables live in memory only.

    ``content_security``: an :class:`antfly_b200.api.content.ContentSecurity` (or its dictionary form) governing
    media links in requests; by default only ``data:`` URLs are accepted."""
    app = FastAPI(title="antfly-b200 inference", version="0.1")
    from .content import ContentFetcher, ContentSecurity

    if isinstance(content_security, dict):
        content_security = ContentSecurity.from_dict(content_security, bool(content_security.get("allow_downloads")))
    fetcher = ContentFetcher(content_security)
    app.state.fetcher = fetcher
    decode_data_url = fetcher.image             # every image reference of a request goes through the policy
    if api_key:
        # shared deployments: every call except the liveness / readiness probes must carry the key
        import hmac

        @app.middleware("http")
        async def _auth(request: Request, call_next):
            if request.url.path not in ("/healthz", "/readyz"):
                got = request.headers.get("authorization", "")
                token = got[7:] if got.lower().startswith("bearer ") else request.headers.get("x-api-key", "")
                if not hmac.compare_digest(token.encode(), api_key.encode()):
                    return _err(401, "unauthorized", "missing or wrong API key")
            return await call_next(request)

    mgr = manager or ModelManager()
    metrics = Metrics()
    queue = RequestQueue(max_concurrent_requests, max_queue_size)
    cache = ResultCache(result_cache_ttl_s)
    log = L.get("server")
    app.state.result_cache = cache
    gpu_lock = threading.Lock()  # one request drives the device at a time; batching happens inside pipelines
    app.state.manager, app.state.metrics, app.state.queue = mgr, metrics, queue
    app.state.indexes = indexes if indexes is not None else {}

    def run_guarded(endpoint: str, units: int, fn):
        t0 = time.perf_counter()
        try:
            queue.acquire(units, timeout=request_timeout_s if request_timeout_s > 0 else 300.0)
        except QueueTimeout as e:
            metrics.queue_rejected.inc()
            metrics.requests.labels(endpoint, "504").inc()
            return _err(504, "timeout", str(e))
        except QueueFull as e:
            metrics.queue_rejected.inc()
            metrics.requests.labels(endpoint, "503").inc()
            r = _err(503, "queue_full", str(e))
            r.headers["Retry-After"] = "1"
            return r
        metrics.queue_depth.set(queue.waiting)
        try:
            # Handlers run on worker threads, whose current CUDA device starts at 0: select the manager's device
            # for the kernel launches inside.
            with gpu_lock, N_device_of(mgr.device):
                out = fn()
            metrics.requests.labels(endpoint, "200").inc()
            return out
        except ModelNotFound as e:
            metrics.requests.labels(endpoint, "404").inc()
            return _err(404, "model_not_found", str(e.args[0]) if e.args else str(e))
        except (ValueError, AssertionError) as e:
            metrics.requests.labels(endpoint, "400").inc()
            return _err(400, "invalid_request", str(e))
        except Exception as e:  # pragma: no cover - defensive
            metrics.requests.labels(endpoint, "500").inc()
            return _err(500, "internal_error", f"{type(e).__name__}: {e}")
        finally:
            queue.release(units)
            dt = time.perf_counter() - t0
            metrics.latency.labels(endpoint).observe(dt)
            if log.isEnabledFor(logging.INFO):
                L.event(log, logging.INFO, "request", endpoint=endpoint, units=units, duration_ms=round(dt * 1e3, 2),
                        queue_waiting=queue.waiting)
            metrics.loaded_models.set(mgr.loaded_count())
            metrics.kernel_launches.set(N.launches())

    async def parse(request: Request, model):
        try:
            return model.model_validate(await request.json()), None
        except Exception as e:
            return None, _err(400, "invalid_request", str(e))

    # ---- embeddings -----------------------------------------------------------------------------------
    async def embed(request: Request):
        req, bad = await parse(request, S.EmbedRequest)
        if bad:
            return bad
        images = {}  # position in the input -> decoded image (content parts of type image_url / image / media)
        audios = {}  # position in the input -> encoded audio bytes (content parts of type audio / media)
        if isinstance(req.input, str):
            texts = [req.input]
        else:
            texts = []
            for i, p in enumerate(req.input):
                if isinstance(p, str):
                    texts.append(p)
                elif p.type == "text":
                    texts.append(p.text or "")
                elif p.type in ("image_url", "image"):
                    extra = p.model_extra or {}
                    url = extra.get("image_url") or extra.get("url") or extra.get("image")
                    if isinstance(url, dict):
                        url = url.get("url")
                    try:
                        images[i] = decode_data_url(url or "")
                    except Exception as e:
                        return _err(400, "invalid_request", f"content part {i}: {e}")
                    texts.append(None)
                elif p.type in ("audio", "input_audio", "audio_url", "media"):
                    # {"type": "media", "mime_type": "audio/wav" | "image/png", "data": base64 or a data: URL}
                    # (zig/pkg/inference/src/server/server.zig:7389 resolveMediaContentPart); "audio" parts carry
                    # the same payload under data / audio / url
                    extra = p.model_extra or {}
                    payload = extra.get("data") or extra.get("audio") or extra.get("input_audio") or extra.get("url") \
                        or extra.get("audio_url")
                    if isinstance(payload, dict):
                        payload = payload.get("data") or payload.get("url")
                    mime = (extra.get("mime_type") or "").split(";")[0].strip().lower()
                    try:
                        import base64 as _b64

                        if not isinstance(payload, str) or not payload:
                            raise ValueError("missing data")
                        if payload.startswith("data:"):
                            head, _, body = payload.partition(",")
                            embedded = head[5:].split(";")[0].strip().lower()
                            if mime and embedded and mime != embedded:
                                raise ValueError(f"mime_type {mime!r} does not match the data URL's {embedded!r}")
                            mime = mime or embedded
                            payload = body
                        raw = _b64.b64decode(payload, validate=True)
                        if p.type == "media" and not mime:
                            raise ValueError("media parts need a mime_type")
                        if mime.startswith("image/"):
                            from ..pipelines.multimodal import decode_image_bytes

                            images[i] = decode_image_bytes(raw)
                        elif mime.startswith("audio/") or (p.type != "media" and not mime):
                            audios[i] = raw
                        else:
                            raise ValueError(f"unsupported media type {mime!r}")
                    except Exception as e:
                        return _err(400, "invalid_request", f"content part {i}: {e}")
                    texts.append(None)
                else:
                    return _err(400, "invalid_request", f"content part type {p.type!r} is not supported")
        if not texts:
            return _err(400, "invalid_request", "input must not be empty")
        task_type = req.task_type or INPUT_TYPE_ALIASES.get(req.input_type or "")

        def work():
            lm = mgr.get(req.model, "embedder")
            if images or audios:
                if images and not hasattr(lm.pipeline, "embed_images"):
                    raise ValueError(f"model {req.model!r} does not embed images")
                if audios and not hasattr(lm.pipeline, "embed_audio"):
                    raise ValueError(f"model {req.model!r} does not embed audio")
                import torch as _torch

                only_text = [t for t in texts if t is not None]
                temb, ntok = lm.pipeline.embed(only_text, task_type, req.dimensions) if only_text else (None, 0)
                media = {}
                if images:
                    order = sorted(images)
                    media.update(zip(order, lm.pipeline.embed_images([images[i] for i in order]).cpu()))
                if audios:
                    order = sorted(audios)
                    media.update(zip(order, lm.pipeline.embed_audio([audios[i] for i in order]).cpu()))
                rows, ti = [], 0
                for i, t in enumerate(texts):
                    if t is None:
                        row = media[i]
                        if req.dimensions:
                            row = _torch.nn.functional.normalize(row[: req.dimensions], dim=-1)
                        rows.append(row)
                    else:
                        rows.append(temb[ti]); ti += 1
                emb = _torch.stack(rows)
            else:
                # per-text result cache: only texts not seen in the last two minutes reach the model
                import torch as _torch

                keys = [cache.key("embed", req.model, task_type, req.dimensions, t) for t in texts]
                got = [cache.get(k) for k in keys]             # (embedding row, prompt tokens of that text)
                todo = [i for i, r in enumerate(got) if r is None]
                if todo:
                    pipe, sub = lm.pipeline, [texts[i] for i in todo]
                    if hasattr(pipe, "tokenize") and hasattr(pipe, "embed_ids"):
                        seqs = pipe.tokenize(sub, task_type)
                        new, counts = pipe.embed_ids(seqs, req.dimensions), [len(q) for q in seqs]
                    else:
                        new, total = pipe.embed(sub, task_type, req.dimensions)
                        counts = [total // len(sub) + (1 if j < total % len(sub) else 0) for j in range(len(sub))]
                    for i, row, c in zip(todo, new, counts):
                        got[i] = (row.clone(), c)
                        cache.put(keys[i], got[i])
                metrics.cache.labels("embed", "hit").inc(len(texts) - len(todo))
                metrics.cache.labels("embed", "miss").inc(len(todo))
                emb = _torch.stack([g[0] for g in got])
                ntok = sum(g[1] for g in got)                  # usage counts every text, cached or not
            metrics.tokens.labels("embed", "prompt").inc(ntok)
            data = [S.EmbeddingObject(embedding=row.tolist(), index=i) for i, row in enumerate(emb)]
            return S.EmbedResponse(data=data, model=req.model,
                                   usage=S.EmbeddingUsage(prompt_tokens=ntok, total_tokens=ntok)).model_dump()

        return await asyncio.to_thread(run_guarded, "embed", len(texts), work)

    # ---- rerank ---------------------------------------------------------------------------------------
    async def rerank(request: Request):
        req, bad = await parse(request, S.RerankRequest)
        if bad:
            return bad
        if not req.prompts:
            return _err(400, "invalid_request", "prompts must not be empty")

        def work():
            lm = mgr.get(req.model, "reranker")
            keys = [cache.key("rerank", req.model, req.query, d) for d in req.prompts]
            got = [cache.get(k) for k in keys]                 # (score, prompt tokens of that pair)
            todo = [i for i, v in enumerate(got) if v is None]
            if todo:
                new, total = lm.pipeline.rerank(req.query, [req.prompts[i] for i in todo])
                for j, (i, v) in enumerate(zip(todo, new)):
                    got[i] = (float(v), total // len(todo) + (1 if j < total % len(todo) else 0))
                    cache.put(keys[i], got[i])
            metrics.cache.labels("rerank", "hit").inc(len(got) - len(todo))
            metrics.cache.labels("rerank", "miss").inc(len(todo))
            scores, ntok = [g[0] for g in got], sum(g[1] for g in got)
            metrics.tokens.labels("rerank", "prompt").inc(ntok)
            return S.RerankResponse(
                data=[S.RerankObject(index=i, score=float(s)) for i, s in enumerate(scores)], model=req.model,
                usage=S.GenerateUsage(prompt_tokens=ntok, completion_tokens=0, total_tokens=ntok)).model_dump()

        return await asyncio.to_thread(run_guarded, "rerank", len(req.prompts), work)

    async def rerank_multimodal(request: Request):
        """Documents made of text and image content parts scored against a text query.  Text-only documents go to
        the cross-encoder named by ``model``; documents with images need a dual-tower (CLIP) model, and a
        document's score is the best cosine similarity between the query and any of its parts."""
        req, bad = await parse(request, S.RerankMultimodalRequest)
        if bad:
            return bad
        if not req.documents:
            return _err(400, "invalid_request", "documents must not be empty")
        docs = []          # per document: (texts, images)
        for i, d in enumerate(req.documents):
            texts, imgs = [], []
            parts = [{"type": "text", "text": d.content}] if isinstance(d.content, str) else d.content
            for p in parts:
                if p.get("type") == "text":
                    texts.append(p.get("text", ""))
                elif p.get("type") in ("image_url", "image"):
                    url = p.get("image_url") or p.get("url") or p.get("image")
                    if isinstance(url, dict):
                        url = url.get("url")
                    try:
                        imgs.append(decode_data_url(url))
                    except Exception as e:
                        return _err(400, "invalid_request", f"document {i}: {e}")
                else:
                    return _err(400, "invalid_request", f"document {i}: content part type {p.get('type')!r} "
                                                        "is not supported")
            if not texts and not imgs:
                return _err(400, "invalid_request", f"document {i} is empty")
            docs.append((texts, imgs))

        def work():
            import torch as _torch

            if not any(imgs for _t, imgs in docs):
                lm = mgr.get(req.model, "reranker")
                scores, ntok = lm.pipeline.rerank(req.query, [" ".join(t) for t, _i in docs])
            else:
                lm = mgr.get(req.model, "embedder")
                pipe = lm.pipeline
                if hasattr(pipe, "rerank_pages"):
                    # late interaction: token vectors of the query against token vectors of each document's parts
                    scores, ntok = pipe.rerank_pages(req.query, docs)
                    metrics.tokens.labels("rerank", "prompt").inc(ntok)
                    return S.RerankResponse(
                        data=[S.RerankObject(index=i, score=float(s)) for i, s in enumerate(scores)], model=req.model,
                        usage=S.GenerateUsage(prompt_tokens=ntok, completion_tokens=0, total_tokens=ntok)).model_dump()
                if not hasattr(pipe, "embed_images"):
                    raise ValueError(f"model {req.model!r} cannot score images")
                qv, ntok = pipe.embed([req.query])
                scores = []
                for texts, imgs in docs:
                    parts = []
                    if texts:
                        tv, n = pipe.embed(texts)
                        ntok += n
                        parts.append(tv)
                    if imgs:
                        parts.append(pipe.embed_images(imgs).cpu().float())
                    scores.append(float((_torch.cat(parts) @ qv[0].float()).max()))
            metrics.tokens.labels("rerank", "prompt").inc(ntok)
            return S.RerankResponse(
                data=[S.RerankObject(index=i, score=float(s)) for i, s in enumerate(scores)], model=req.model,
                usage=S.GenerateUsage(prompt_tokens=ntok, completion_tokens=0, total_tokens=ntok)).model_dump()

        return await asyncio.to_thread(run_guarded, "rerank_multimodal", len(docs), work)

    # ---- generate / chat completions --------------------------------------------------------------------
    def sampling_from(req: S.GenerateRequest, tok) -> SamplingParams:
        stops: List[int] = []
        if req.stop:
            for s in ([req.stop] if isinstance(req.stop, str) else req.stop):
                ids = tok.encode(s)
                if len(ids) == 1:
                    stops.append(ids[0])
        grammar = None
        fmt = (req.response_format or {}).get("type")
        gbnf = req.grammar
        if not gbnf and fmt == "json_schema":
            # structured output: the schema is compiled into a grammar, so a non-conforming token is never sampled
            from ..runtime.json_schema import json_schema_to_gbnf

            js = (req.response_format or {}).get("json_schema") or {}
            gbnf = json_schema_to_gbnf(js.get("schema", js) if isinstance(js, dict) else {})
        if gbnf:
            # a GBNF grammar supplied with the request constrains the whole reply
            from ..runtime.grammar import GbnfGrammar, token_bytes_table

            table = getattr(tok, "_grammar_token_bytes", None)
            if table is None:
                table = token_bytes_table(tok, int(getattr(tok, "vocab_size", 0)) or len(getattr(tok, "vocab", [])))
                try:
                    tok._grammar_token_bytes = table
                except Exception:
                    pass
            grammar = GbnfGrammar(table, gbnf, eos_id=tok.special.eos_id)
        elif fmt in ("json_object", "json"):
            # JSON mode: every sampled token must keep the reply a valid JSON prefix; the byte table of the
            # vocabulary is built once per tokenizer and shared by all requests.
            from ..runtime.grammar import JsonGrammar, token_bytes_table

            table = getattr(tok, "_grammar_token_bytes", None)
            if table is None:
                table = token_bytes_table(tok, int(getattr(tok, "vocab_size", 0)) or len(getattr(tok, "vocab", [])))
                try:
                    tok._grammar_token_bytes = table
                except Exception:
                    pass
            grammar = JsonGrammar(table, eos_id=tok.special.eos_id, root_object_only=fmt == "json_object")
        return SamplingParams(max_tokens=req.max_tokens, temperature=req.temperature, top_k=req.top_k, top_p=req.top_p,
                              min_p=req.min_p, repetition_penalty=req.repetition_penalty,
                              frequency_penalty=req.frequency_penalty, presence_penalty=req.presence_penalty,
                              stop_token_ids=stops, seed=req.seed, grammar=grammar,
                              cache_compaction_ratio=req.cache_compaction_ratio, speculative_k=req.speculative_k)

    async def generate(request: Request):
        req, bad = await parse(request, S.GenerateRequest)
        if bad:
            return bad
        return await generate_from(req)

    async def generate_from(req: S.GenerateRequest, framer=None):
        """Runs one chat / generate request.  ``framer`` (None = the OpenAI-style wire format) turns the result, or
        the stream of deltas, into another API's wire format."""
        if not req.messages:
            return _err(400, "invalid_request", "messages must not be empty")
        if req.max_tokens <= 0:
            return _err(400, "invalid_request", "max_tokens must be positive")
        msgs = [m.model_dump() for m in req.messages]
        rid = "chatcmpl-" + uuid.uuid4().hex[:24]
        created = int(time.time())
        # Tool calling: declare the tools in a system message and parse calls out of the reply.
        tool_fmt = None
        if req.tools:
            from ..pipelines import tool_calls as TC

            try:
                choice = TC.parse_tool_choice(req.tool_choice)
            except ValueError as e:
                return _err(400, "invalid_request", str(e))
            if choice.enabled:
                try:
                    lm0 = mgr.get(req.model, "generator")
                    tool_fmt = TC.detect_format(getattr(lm0.pipeline.template, "source", None))
                except Exception:
                    tool_fmt = "hermes"
                decl = TC.format_tools_prompt(req.tools, tool_fmt, choice)
                if not req.grammar and (req.response_format or {}).get("type") is None:
                    # a forced call is also enforced: the reply can only be a call that fits the function's schema
                    try:
                        forced = TC.forced_call_grammar(req.tools, tool_fmt, choice)
                    except ValueError as e:
                        return _err(400, "invalid_request", str(e))
                    if forced:
                        req = req.model_copy(update={"grammar": forced})
                if msgs and msgs[0].get("role") == "system":
                    msgs[0] = dict(msgs[0], content=(msgs[0].get("content") or "") + "\n\n" + decl)
                else:
                    msgs.insert(0, {"role": "system", "content": decl})
        if req.cache_dtype == "f32" and mgr.device.type == "cuda":
            return _err(400, "invalid_request", "cache_dtype 'f32' is not available on the GPU (the kernels read "
                                                "bf16 or quantised caches); use f16, fp8, int8 or int4")
        if req.grammar or (req.response_format or {}).get("type") == "json_schema":
            try:  # reject a malformed grammar / unsupported schema before any work is queued
                from ..runtime.grammar import GbnfGrammar
                from ..runtime.json_schema import json_schema_to_gbnf

                text = req.grammar
                if not text:
                    js = req.response_format.get("json_schema") or {}
                    if not isinstance(js, dict) or not isinstance(js.get("schema", js), dict):
                        raise ValueError("response_format.json_schema.schema must be an object")
                    text = json_schema_to_gbnf(js.get("schema", js))
                GbnfGrammar([b"a"], text)
            except ValueError as e:
                return _err(400, "invalid_request", str(e))
        if not req.stream:
            def work():
                lm = mgr.get_generator(req.model, req.draft_model, req.cache_dtype)
                out = lm.pipeline.generate(msgs, sampling_from(req, lm.tokenizer))
                metrics.tokens.labels("generate", "prompt").inc(out.prompt_tokens)
                metrics.tokens.labels("generate", "completion").inc(out.completion_tokens)
                message, finish = S.GenerateMessage(content=out.text), out.finish_reason
                if tool_fmt is not None:
                    from ..pipelines import tool_calls as TC

                    content, calls = TC.parse_tool_calls(out.text, tool_fmt)
                    if calls:
                        message, finish = S.GenerateMessage(content=content or None, tool_calls=calls), "tool_calls"
                resp = S.GenerateResponse(
                    id=rid, created=created, model=req.model,
                    choices=[S.GenerateChoice(message=message, finish_reason=finish)],
                    usage=S.GenerateUsage(prompt_tokens=out.prompt_tokens, completion_tokens=out.completion_tokens,
                                          total_tokens=out.prompt_tokens + out.completion_tokens)).model_dump()
                return framer.response(resp) if framer is not None else resp

            return await asyncio.to_thread(run_guarded, "generate", 1, work)

        # Streaming: the generation runs in a worker thread and feeds an asyncio queue.
        loop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()

        def chunk(delta: dict, finish: Optional[str] = None) -> str:
            body = {"id": rid, "object": "chat.completion.chunk", "created": created, "model": req.model,
                    "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}
            return "data: " + json.dumps(body) + "\n\n"

        if framer is not None:
            framer.begin(rid, req.model)

        def emit_start():
            return framer.start() if framer is not None else chunk({"role": "assistant"})

        def emit_text(t: str):
            return framer.text(t) if framer is not None else chunk({"content": t})

        def emit_calls(calls):
            return framer.tool_calls(calls) if framer is not None else chunk(
                {"tool_calls": [dict(c, index=i) for i, c in enumerate(calls)]})

        def emit_finish(reason, out):
            return framer.finish(reason, out.prompt_tokens, out.completion_tokens) if framer is not None else \
                chunk({}, reason)

        def worker():
            def work():
                lm = mgr.get_generator(req.model, req.draft_model, req.cache_dtype)
                loop.call_soon_threadsafe(q.put_nowait, emit_start())
                parser = None
                if tool_fmt is not None:
                    from ..pipelines import tool_calls as TC

                    parser = TC.ToolCallParser(tool_fmt)

                def on_delta(d: str):
                    shown = parser.feed(d) if parser is not None else d
                    if shown:
                        loop.call_soon_threadsafe(q.put_nowait, emit_text(shown))

                out = lm.pipeline.generate(msgs, sampling_from(req, lm.tokenizer), on_delta=on_delta)
                finish = out.finish_reason
                if parser is not None:
                    _, calls = parser.finish()
                    if calls:
                        loop.call_soon_threadsafe(q.put_nowait, emit_calls(calls))
                        finish = "tool_calls"
                loop.call_soon_threadsafe(q.put_nowait, emit_finish(finish, out))
                return None

            res = run_guarded("generate", 1, work)
            if isinstance(res, JSONResponse):
                err = res.body.decode()
                loop.call_soon_threadsafe(q.put_nowait, framer.error(err) if framer is not None
                                          else "data: " + err + "\n\n")
            loop.call_soon_threadsafe(q.put_nowait, None)

        threading.Thread(target=worker, daemon=True).start()

        async def gen():
            while True:
                item = await q.get()
                if item is None:
                    break
                yield item
            if framer is None:
                yield "data: [DONE]\n\n"

        return StreamingResponse(gen(), media_type="text/event-stream")

    # ---- Anthropic Messages and OpenAI path compatibility -----------------------------------------------------
    async def anthropic_messages(request: Request):
        from .compat import AnthropicFramer, anthropic_to_generate

        try:
            body = json.loads(await request.body() or b"{}")
            greq = S.GenerateRequest(**anthropic_to_generate(body))
        except Exception as e:
            return JSONResponse(status_code=400, content={"type": "error", "error": {
                "type": "invalid_request_error", "message": str(e)}})
        res = await generate_from(greq, AnthropicFramer())
        if isinstance(res, JSONResponse) and res.status_code >= 400:
            err = json.loads(res.body)
            kind = {404: "not_found_error", 503: "overloaded_error", 504: "overloaded_error"}.get(
                res.status_code, "invalid_request_error" if res.status_code < 500 else "api_error")
            return JSONResponse(status_code=res.status_code, content={"type": "error", "error": {
                "type": kind, "message": err.get("message", "")}})
        return res

    async def openai_models():
        per_task = mgr.list_models()
        now = int(time.time())
        return {"object": "list", "data": [{"id": n, "object": "model", "created": now, "owned_by": "antfly"}
                                           for t in ("generators", "embedders") for n in per_task.get(t, {})]}

    # ---- chunk ----------------------------------------------------------------------------------------
    async def chunk_ep(request: Request):
        req, bad = await parse(request, S.ChunkRequest)
        if bad:
            return bad
        cfg = dict(req.config or {})
        topt, aopt = dict(cfg.get("text") or {}), dict(cfg.get("audio") or {})
        model = cfg.get("model") or req.model or "fixed"
        max_chunks = int(cfg.get("max_chunks") or req.max_chunks or 0)
        target = int(topt.get("target_tokens") or req.target_tokens or 500)
        overlap = topt.get("overlap_tokens")
        overlap = int(overlap if overlap is not None else (req.overlap_tokens if req.overlap_tokens is not None else 50))
        part = req.input if req.input is not None else req.text
        if part is None:
            return _err(400, "invalid_request", "input is required")
        binary = None
        if isinstance(part, dict):
            if part.get("type") == "text" or "text" in part:
                part = str(part.get("text") or "")
            else:
                import base64

                try:
                    binary = (str(part.get("mime_type") or "application/octet-stream"),
                              base64.b64decode(part.get("data") or "", validate=False))
                except Exception as e:
                    return _err(400, "invalid_request", f"media data is not base64: {e}")

        def usage(n):
            return {"prompt_tokens": n, "completion_tokens": 0, "total_tokens": n}

        def pack(chunks, used, ntok):
            import base64

            data = []
            for i, c in enumerate(chunks):
                o = {"object": "chunk", "index": i, "id": int(c.get("id", i)), "mime_type": c.get("mime_type", "text/plain")}
                for k in ("text", "start_char", "end_char", "start_time_ms", "end_time_ms", "frame_index", "frame_delay_ms"):
                    if k in c:
                        o[k] = c[k]
                if "data" in c:
                    o["data"] = base64.b64encode(c["data"]).decode()
                data.append(o)
            # ``chunks`` is the older response field, kept beside the reference's ``data``
            return {"object": "list", "data": data, "chunks": data, "model": used, "usage": usage(ntok),
                    "cache_hit": False}

        if binary is not None:
            from ..pipelines.chunking import chunk_binary

            try:
                vad = aopt.get("vad")          # present (even empty): voice-activity segmentation with its defaults
                ch = chunk_binary(binary[0], binary[1], int(aopt.get("window_duration_ms") or 30000),
                                  int(aopt.get("overlap_duration_ms") or 0), max_chunks,
                                  dict(vad) if isinstance(vad, dict) else None)
            except Exception as e:
                return _err(400, "invalid_request", str(e))
            metrics.requests.labels("chunk", "200").inc()
            return pack(ch, "fixed", 0)
        text = str(part)
        from ..pipelines.chunking import _tokens

        if model in ("fixed", "", None):
            try:
                chunks = chunk_text(text, target, overlap, max_chunks, str(topt.get("separator") or "\n\n"))
            except ValueError as e:
                return _err(400, "invalid_request", str(e))
            metrics.requests.labels("chunk", "200").inc()
            return pack(chunks, "fixed", len(_tokens(text)))

        def work():
            from ..pipelines.chunking import NeuralChunker

            lm = mgr.get(model, "chunker")
            kw = {"threshold": float(cfg["threshold"])} if cfg.get("threshold") is not None else {}
            ch = NeuralChunker(lm.pipeline, **kw).chunk(text, max_tokens=target, max_chunks=max_chunks)
            return pack(ch, model, len(_tokens(text)))

        return await asyncio.to_thread(run_guarded, "chunk", 1, work)

    # ---- vector search --------------------------------------------------------------------------------
    async def search(request: Request):
        req, bad = await parse(request, S.SearchRequest)
        if bad:
            return bad
        idx = app.state.indexes.get(req.index)
        if idx is None:
            return _err(404, "index_not_found", f"index {req.index!r} is not loaded")

        def work():
            t0 = time.perf_counter()
            if req.embeddings is not None:
                qv = decode_vectors(req.embeddings)
            elif req.semantic_search is not None:
                if not req.embedder:
                    raise ValueError("semantic_search needs an embedder model name")
                qv, _ = mgr.get(req.embedder, "embedder").pipeline.embed([req.semantic_search])
            else:
                raise ValueError("one of embeddings / semantic_search is required")
            res = idx.search(qv.to(idx.device), req.limit, effort=req.search_effort) if hasattr(idx, "search_effort") \
                else idx.search(qv.to(idx.device), req.limit)
            d, ids = res.distances.cpu(), res.ids.cpu()
            hits = []
            for qi in range(d.shape[0]):
                row = []
                for dist, i in zip(d[qi].tolist(), ids[qi].tolist()):
                    if i < 0 or (req.distance_under is not None and dist >= req.distance_under) or \
                            (req.distance_over is not None and dist <= req.distance_over):
                        continue
                    row.append(S.SearchHit(id=int(i), distance=float(dist)))
                hits.append(row)
            return S.SearchResponse(hits=hits, took_ms=(time.perf_counter() - t0) * 1e3, index=req.index).model_dump()

        return await asyncio.to_thread(run_guarded, "search", 1, work)

    # ---- classify / recognize: the per-task forms of what /extract answers by schema ---------------------------
    async def classify(request: Request):
        """``ClassifyRequest`` -> ``ClassifyResponse`` (specs/openapi/inference/api.yaml ClassifyRequest: texts, candidate
        labels for zero-shot models, hypothesis_template, multi_label; the handler the reference keeps as
        ``classifyText``, zig/pkg/inference/src/server/server.zig:3502)."""
        req, bad = await parse(request, S.ClassifyRequest)
        if bad:
            return bad
        if not req.texts:
            return _err(400, "invalid_request", "texts must not be empty")

        def work():
            lm = mgr.get(req.model, "classifier")
            pipe = lm.pipeline
            if hasattr(pipe, "template"):                          # NLI cross-encoder: labels come from the request
                if not req.labels:
                    raise ValueError("this model classifies against candidate labels: labels must not be empty")
                if req.hypothesis_template is not None and "{}" not in req.hypothesis_template:
                    raise ValueError("hypothesis_template needs a {} placeholder")
                keep, pipe.template = pipe.template, req.hypothesis_template or pipe.template
                try:
                    ranked = pipe.classify(req.texts, req.labels, multi_label=req.multi_label)
                finally:
                    pipe.template = keep
            elif hasattr(pipe, "recognize"):                       # zero-shot span model used as a classifier
                if not req.labels:
                    raise ValueError("this model classifies against candidate labels: labels must not be empty")
                ranked = [[{"label": l, "score": float(sc)} for l, sc in
                           pipe.classify(t, req.labels, threshold=0.0, multi_label=req.multi_label)] for t in req.texts]
            else:                                                  # trained head: its own label set
                ranked = pipe.classify(req.texts, top_k=max(len(getattr(pipe, "id2label", {})), 1))
                if req.labels:
                    want = {l.lower() for l in req.labels}
                    ranked = [[r for r in row if r["label"].lower() in want] for row in ranked]
            n_tok = sum(len(t.split()) for t in req.texts)
            return {"object": "list", "model": req.model,
                    "data": [{"object": "classification", "index": i, "classifications": row}
                             for i, row in enumerate(ranked)],
                    "usage": {"prompt_tokens": n_tok, "completion_tokens": 0, "total_tokens": n_tok}}

        return await asyncio.to_thread(run_guarded, "classify", max(1, len(req.texts)), work)

    async def recognize(request: Request):
        """``RecognizeRequest`` -> ``RecognizeResponse``: entities per text (character offsets), relations when
        ``relation_labels`` are given and the model extracts them, and one resolved graph over all texts when a
        ``resolver`` section is present (specs/openapi/inference/api.yaml RecognizeRequest / ResolverConfig; the
        reference's ``recognizeEntities``, zig/pkg/inference/src/server/server.zig:3220)."""
        req, bad = await parse(request, S.RecognizeRequest)
        if bad:
            return bad
        if not req.texts:
            return _err(400, "invalid_request", "texts must not be empty")

        def work():
            lm = mgr.get(req.model, "recognizer")
            pipe = lm.pipeline

            def span(e, text):
                if hasattr(e, "start") and not hasattr(e, "start_token"):      # byte offsets -> character offsets
                    raw = text.encode("utf-8")
                    a = len(raw[: e.start].decode("utf-8", "replace"))
                    return {"text": e.text, "label": e.label, "start": a, "end": a + len(e.text), "score": float(e.score)}
                t = e.text or ""
                at = text.find(t) if t else -1
                if at < 0 and t:
                    at = text.lower().find(t.lower())
                return {"text": t, "label": e.label, "start": max(at, 0), "end": max(at, 0) + len(t),
                        "score": float(e.score)}

            rels = None
            if hasattr(pipe, "recognize"):
                if req.relation_labels and hasattr(pipe, "extract_relations"):
                    ents, rels = pipe.extract_relations(req.texts, req.labels or None, req.relation_labels)
                else:
                    ents = pipe.recognize(req.texts, req.labels or None, threshold=req.threshold)
            elif hasattr(pipe, "entities"):
                ents = pipe.entities(req.texts)
                if req.labels:
                    want = {l.lower() for l in req.labels}
                    ents = [[e for e in row if e.label.lower() in want] for row in ents]
            else:
                raise ValueError(f"model {req.model!r} does not recognise entities")
            data = []
            for i, (text, row) in enumerate(zip(req.texts, ents)):
                rec = {"object": "recognition", "index": i, "entities": [span(e, text) for e in row]}
                if rels is not None:
                    rec["relations"] = [{"head": span(r.head, text), "tail": span(r.tail, text), "label": r.label,
                                         "score": float(r.score)} for r in rels[i]]
                data.append(rec)
            n_tok = sum(len(t.split()) for t in req.texts)
            out = {"object": "list", "model": req.model, "data": data,
                   "usage": {"prompt_tokens": n_tok, "completion_tokens": 0, "total_tokens": n_tok}}
            if req.resolver is not None:
                from ..pipelines.resolver import ResolverConfig, build_knowledge_graph

                cfg = ResolverConfig(**{k: type(getattr(ResolverConfig, k))(v) for k, v in req.resolver.items()
                                        if k in ResolverConfig.__dataclass_fields__})
                kg = build_knowledge_graph(ents, rels, cfg)
                out["knowledge_graph"] = {
                    "entities": [{"id": e.id, "name": e.canonical_name, "label": e.label, "score": e.score,
                                  "mentions": e.mentions, "inputs": e.text_indices} for e in kg.entities],
                    "relations": [{"source": r.head_id, "target": r.tail_id, "type": r.label, "score": r.score,
                                   "inputs": r.text_indices} for r in kg.relations]}
            return out

        return await asyncio.to_thread(run_guarded, "recognize", max(1, len(req.texts)), work)

    # ---- rewrite (encoder-decoder text-to-text) and schema-driven extraction -------------------------------------
    async def rewrite(request: Request):
        req, bad = await parse(request, S.RewriteRequest)
        if bad:
            return bad

        def work():
            lm = mgr.get(req.model, "rewriter")
            data, pt, ct = [], 0, 0
            for i, text in enumerate(req.inputs):
                out = lm.pipeline.generate(text, SamplingParams(max_tokens=req.max_tokens), raw_prompt=True)
                data.append({"object": "rewrite", "index": i, "texts": [out.text]})
                pt += out.prompt_tokens
                ct += out.completion_tokens
            return {"object": "list", "data": data, "model": req.model,
                    "usage": {"prompt_tokens": pt, "completion_tokens": ct, "total_tokens": pt + ct}}

        return await asyncio.to_thread(run_guarded, "rewrite", max(1, len(req.inputs)), work)

    async def transcribe(request: Request):
        req, bad = await parse(request, S.TranscribeRequest)
        if bad:
            return bad
        try:
            audio = base64.b64decode(req.audio, validate=True)
        except Exception:
            return _err(400, "invalid_request", "audio must be base64")

        def work():
            lm = mgr.get(req.model, "transcriber")
            vad = (req.model_extra or {}).get("vad")           # {"vad": {...}}: decode the speech segments only
            out = lm.pipeline.transcribe(audio, language=req.language, task=req.task, max_new_tokens=req.max_tokens,
                                         **({"vad": dict(vad)} if isinstance(vad, dict) else {}))
            metrics.tokens.labels("transcribe", "completion").inc(out.completion_tokens)
            return {"object": "list", "model": req.model,
                    "data": [{"object": "transcription", "index": 0, "text": out.text,
                              **({"language": out.language} if out.language else {}), "segments": [
                        {k: v for k, v in sgm.items() if k != "tokens"} for sgm in out.segments]}],
                    "usage": {"prompt_tokens": out.prompt_tokens, "completion_tokens": out.completion_tokens,
                              "total_tokens": out.prompt_tokens + out.completion_tokens}}

        return await asyncio.to_thread(run_guarded, "transcribe", 1, work)

    async def read(request: Request):
        req, bad = await parse(request, S.ReadRequest)
        if bad:
            return bad
        if not req.images:
            return _err(400, "invalid_request", "images must not be empty")
        imgs = []
        for i, im in enumerate(req.images):
            url = im.get("url") if isinstance(im, dict) else im
            try:
                imgs.append(decode_data_url(url))
            except Exception as e:
                return _err(400, "invalid_request", f"image {i}: {e}")

        extra = req.model_extra or {}

        def work_multistage():
            # whole pages: find the text regions, read each, return them in reading order
            from ..pipelines.ocr_multistage import MultiStageOCR, RegionPostProcessor

            lm = mgr.get(req.model, "reader")
            post = RegionPostProcessor(**{k: extra[k] for k in ("threshold", "box_threshold", "unclip_ratio",
                                                                "min_box_area") if k in extra})
            ocr = MultiStageOCR(lm.pipeline, post=post)
            data = []
            for i, im in enumerate(imgs):
                r = ocr.run(im, req.max_tokens)
                data.append({"object": "read", "index": i, "text": r.full_text, "regions": [
                    {"bbox": [round(v, 1) for v in g.bbox], "confidence": g.confidence, "text": g.text,
                     **({"label": g.label} if g.label else {})} for g in r.regions]})
            return {"object": "list", "model": req.model, "data": data,
                    "usage": {"prompt_tokens": 0, "completion_tokens": 0, "total_tokens": 0}}

        if extra.get("multistage"):
            return await asyncio.to_thread(run_guarded, "read", len(imgs), work_multistage)

        def work():
            lm = mgr.get(req.model, "reader")
            res = lm.pipeline.read(imgs, req.max_tokens, prompt=req.prompt)
            n = sum(len(r.token_ids) for r in res)
            metrics.tokens.labels("read", "completion").inc(n)
            return {"object": "list", "model": req.model,
                    "data": [{"object": "read", "index": i, "text": r.text,
                              **({"regions": r.regions} if getattr(r, "regions", None) else {})}
                             for i, r in enumerate(res)],
                    "usage": {"prompt_tokens": 0, "completion_tokens": n, "total_tokens": n}}

        return await asyncio.to_thread(run_guarded, "read", len(imgs), work)

    async def layout(request: Request):
        """Words with page boxes (from OCR or a PDF text layer), optionally the page image -> a label per word and
        the fields they form, through a layout-aware token classifier."""
        req, bad = await parse(request, S.LayoutRequest)
        if bad:
            return bad
        if not req.pages:
            return _err(400, "invalid_request", "pages must not be empty")
        from ..pipelines.layout import group_entities, normalize_box
        pages = []
        for i, pg in enumerate(req.pages):
            if len(pg.words) != len(pg.boxes) or any(len(b) != 4 for b in pg.boxes):
                return _err(400, "invalid_request", f"page {i}: one [x0, y0, x1, y1] box per word is required")
            if pg.width and pg.height:
                boxes = [normalize_box(b, pg.width, pg.height) for b in pg.boxes]
            else:
                boxes = [tuple(int(v) for v in b) for b in pg.boxes]
                if any(v < 0 or v > 1000 for b in boxes for v in b):
                    return _err(400, "invalid_request", f"page {i}: boxes outside 0..1000 need width and height")
            img = None
            if pg.image is not None:
                try:
                    img = decode_data_url(pg.image.get("url") if isinstance(pg.image, dict) else pg.image)
                except Exception as e:
                    return _err(400, "invalid_request", f"page {i} image: {e}")
            pages.append((pg.words, boxes, img))

        def work():
            lm = mgr.get(req.model, "recognizer")
            if not hasattr(lm.pipeline, "label_words"):
                raise ValueError(f"model {req.model!r} is not a layout model")
            data = []
            for i, (words, boxes, img) in enumerate(pages):
                labels = lm.pipeline.label_words(words, boxes, img)
                rec = {"object": "layout", "index": i, "words": [
                    {"word": l.word, "box": list(l.box), "label": l.label, "score": l.score} for l in labels]}
                if req.group:
                    rec["entities"] = group_entities(labels)
                data.append(rec)
            return {"object": "list", "model": req.model, "data": data}

        return await asyncio.to_thread(run_guarded, "layout", sum(len(p[0]) for p in pages), work)

    async def extract(request: Request):
        req, bad = await parse(request, S.ExtractionRequest)
        if bad:
            return bad

        def text_of(content) -> str:
            if isinstance(content, str):
                return content
            return "".join(p.get("text", "") for p in content if isinstance(p, dict) and p.get("type") == "text")

        def images_of(content):
            if isinstance(content, str):
                return []
            out = []
            for p in content:
                if isinstance(p, dict) and p.get("type") in ("image_url", "image"):
                    url = p.get("image_url") or p.get("url") or p.get("image")
                    out.append(url.get("url") if isinstance(url, dict) else url)
            return out

        def work():
            schema, opts = req.schema_, req.options
            thr = float(opts.get("threshold", 0.0) or 0.0)
            texts = [text_of(i.content) for i in req.inputs]
            pictures = [images_of(i.content) for i in req.inputs]
            if any(pictures):
                # image inputs: a reader turns every image into text first, extraction then runs on that text
                # (zig/pkg/inference/src/server/server.zig extractImages: read document text -> run extraction)
                ropt = opts.get("reader") or {}
                rname = ropt.get("model") if isinstance(ropt, dict) else None
                if not rname:
                    raise ValueError("inputs with images need options.reader.model (a reader model name)")
                reader = mgr.get(str(rname), "reader").pipeline
                for k, urls in enumerate(pictures):
                    if not urls:
                        continue
                    imgs = [decode_data_url(u) for u in urls]
                    read = reader.read(imgs, int(opts.get("max_tokens", 256) or 256), prompt=ropt.get("prompt"))
                    texts[k] = "\n".join([t for t in [texts[k]] + [r.text for r in read] if t])
            want_ents = [str(x) for x in schema.get("entities") or []]
            tasks = schema.get("classifications") or []
            rel_schema = schema.get("relations") or []
            structures = schema.get("structures") or {}
            if not want_ents and not tasks and not rel_schema and not structures:
                raise ValueError("schema needs entities, relations, classifications and / or structures")
            data = [{"id": i.id} if i.id is not None else {} for i in req.inputs]
            ntok = 0
            if structures:
                from ..pipelines import extraction as EX

                span_model = mgr.get(req.model, "recognizer").pipeline
                if not hasattr(span_model, "recognize") or not hasattr(span_model, "classify"):
                    raise ValueError("structures need a zero-shot span model (a GLiNER-style recognizer)")
                cfg = EX.ExtractionConfig(
                    threshold=float(opts["threshold"]) if opts.get("threshold") is not None else 0.3,
                    flat_ner=bool(opts.get("flat_ner", True)), include_confidence=bool(opts.get("include_confidence", False)),
                    include_spans=bool(opts.get("include_spans", False)), cluster_gap=int(opts.get("cluster_gap", 0) or 0))
                canon = EX.canonical_structures(structures)
                for rec, text in zip(data, texts):
                    rec["structures"] = EX.extract_structures(span_model, text, canon, cfg)
            zero_shot = None
            if want_ents or tasks or rel_schema:
                try:
                    cand = mgr.get(req.model, "recognizer").pipeline
                    zero_shot = cand if hasattr(cand, "extract_relations") else None
                except Exception:
                    zero_shot = None
            if zero_shot is not None:
                # a span model that takes its labels from the request answers the whole schema by itself
                rel_types = [str(r.get("type")) for r in rel_schema if isinstance(r, dict) and r.get("type")]
                if want_ents and rel_types:
                    all_e, all_r = zero_shot.extract_relations(texts, want_ents, rel_types)
                elif want_ents:
                    all_e, all_r = zero_shot.recognize(texts, want_ents, threshold=thr or None), [[] for _ in texts]
                else:
                    all_e, all_r = [[] for _ in texts], [[] for _ in texts]
                for rec, text, ents, rels in zip(data, texts, all_e, all_r):
                    raw = text.encode("utf-8")

                    def item(e):
                        d = {"label": e.label, "text": e.text, "score": e.score}
                        if opts.get("include_spans", True):       # character offsets, from the byte offsets
                            d["start"] = len(raw[: e.start].decode("utf-8", "replace"))
                            d["end"] = d["start"] + len(e.text)
                        if not opts.get("include_confidence", True):
                            d.pop("score")
                        return d

                    if want_ents:
                        rec["entities"] = [item(e) for e in ents]
                    if rel_types:
                        pos = {(e.start, e.end, e.label): i for i, e in enumerate(ents)}
                        rec["relations"] = [{
                            "type": r.label, "score": r.score,
                            "source": {**item(r.head), "entity_index": pos.get((r.head.start, r.head.end, r.head.label), -1)},
                            "target": {**item(r.tail), "entity_index": pos.get((r.tail.start, r.tail.end, r.tail.label), -1)},
                        } for r in rels]
                for t in tasks:
                    labels = [str(l) for l in t.get("labels") or []]
                    for rec, text in zip(data, texts):
                        got = zero_shot.classify(text, labels, threshold=thr, multi_label=bool(t.get("multi_label")))
                        rec.setdefault("classifications", [])
                        rec["classifications"] += [{"name": t.get("name", ""), "label": l, "score": sc} for l, sc in got]
                want_ents, rel_schema, tasks = [], [], []
            if want_ents:
                ner = mgr.get(req.model, "recognizer").pipeline
                allowed = {w.lower() for w in want_ents}
                for rec, text, ents in zip(data, texts, ner.entities(texts)):
                    rec["entities"], cursor = [], 0
                    for e in ents:
                        if e.label.lower() not in allowed or e.score < thr:
                            continue
                        item = {"label": e.label, "text": (e.text or "").strip(), "score": e.score}
                        if opts.get("include_spans", True) and item["text"]:
                            at = text.lower().find(item["text"].lower(), cursor)
                            if at < 0:
                                at = text.lower().find(item["text"].lower())
                            if at >= 0:
                                item["start"], item["end"] = at, at + len(item["text"])
                                item["text"] = text[at: at + len(item["text"])]
                                cursor = item["end"]
                        if not opts.get("include_confidence", True):
                            item.pop("score")
                        rec["entities"].append(item)
            if rel_schema:
                # relation extraction: a sequence-to-sequence model writes triplets, which are parsed back
                from ..pipelines.relations import RelationExtractor

                rx = RelationExtractor(mgr.get(req.model, "rewriter").pipeline,
                                       int(opts.get("max_tokens", 256) or 256))
                types = [str(r.get("type")) for r in rel_schema if isinstance(r, dict) and r.get("type")]
                for rec, text in zip(data, texts):
                    ents, rels = rx.extract(text, types or None)
                    base = len(rec.get("entities", []))
                    for r in rels:
                        r["source"]["entity_index"] += base
                        r["target"]["entity_index"] += base
                    rec["entities"] = rec.get("entities", []) + ents
                    rec["relations"] = rels
            if tasks:
                clf = mgr.get(req.model, "classifier").pipeline
                known = {v.lower(): v for v in clf.id2label.values()}
                nli = {"entailment", "contradiction"} <= set(known)
                ranked = clf.classify(texts, top_k=len(clf.id2label))
                for rec in data:
                    rec["classifications"] = []
                for t in tasks:
                    labels = [str(l) for l in t.get("labels") or []]
                    missing = [l for l in labels if l.lower() not in known]
                    if missing and nli:
                        # labels the model was not trained on: zero-shot through entailment
                        from ..pipelines.classification import ZeroShotClassifier

                        zs = ZeroShotClassifier(clf.model, clf.tokenizer, clf.id2label,
                                                opts.get("hypothesis_template", "This example is {}."))
                        for rec, scores in zip(data, zs.classify(texts, labels, bool(t.get("multi_label")))):
                            keep = [s for s in scores if s["score"] >= thr] if t.get("multi_label") else scores[:1]
                            rec["classifications"] += [{"name": t.get("name", ""), **s} for s in keep]
                        continue
                    if missing:
                        raise ValueError(f"classification {t.get('name')!r}: model has no label(s) {missing}")
                    for rec, scores in zip(data, ranked):
                        cand = [s for s in scores if s["label"].lower() in {l.lower() for l in labels}]
                        keep = [s for s in cand if s["score"] >= thr] if t.get("multi_label") else cand[:1]
                        for s in keep:
                            rec["classifications"].append({"name": t.get("name", ""), "label": s["label"],
                                                           "score": s["score"]})
            out = {"object": "extraction", "model": req.model, "data": data, "usage": {"inputs": len(texts)}}
            if opts.get("resolve"):
                # one graph over all inputs: similar mentions of a type become one entity, relations are re-keyed
                from types import SimpleNamespace as _NS

                from ..pipelines.resolver import ResolverConfig, build_knowledge_graph

                mk = lambda e: _NS(text=e.get("text", ""), label=e.get("label", ""), score=float(e.get("score", 1.0)))
                kg = build_knowledge_graph(
                    [[mk(e) for e in rec.get("entities", [])] for rec in data],
                    [[_NS(head=mk(r["source"]), tail=mk(r["target"]), label=r.get("type", ""),
                          score=float(r.get("score", 1.0))) for r in rec.get("relations", [])] for rec in data],
                    ResolverConfig(**{k: type(getattr(ResolverConfig, k))(v) for k, v in
                                      {**opts, **(opts.get("resolver") if isinstance(opts.get("resolver"), dict) else {})
                                       }.items() if k in ResolverConfig.__dataclass_fields__}))
                out["knowledge_graph"] = {
                    "entities": [{"id": e.id, "name": e.canonical_name, "label": e.label, "score": e.score,
                                  "mentions": e.mentions, "inputs": e.text_indices} for e in kg.entities],
                    "relations": [{"source": r.head_id, "target": r.tail_id, "type": r.label, "score": r.score,
                                   "inputs": r.text_indices} for r in kg.relations]}
            return out

        return await asyncio.to_thread(run_guarded, "extract", max(1, len(req.inputs)), work)

    # ---- tables: documents + dense / sparse / full-text indexes, hybrid query ---------------------------------
    app.state.tables = {}

    def table_dir(name: str) -> str:
        if not re.fullmatch(r"[A-Za-z0-9_.-]{1,128}", name) or name in (".", ".."):
            raise ValueError("a durable table's name is 1 to 128 letters, digits, '_', '-' or '.'")
        d = os.path.join(data_dir, "tables", name)
        os.makedirs(d, exist_ok=True)
        return d

    def build_table(table: str, spec: dict) -> dict:
        from ..index.flat import GrowableFlatIndex
        from ..index.table import Table

        embed = rerank = None
        dim = spec.get("dimension")
        embedder, reranker = spec.get("embedder"), spec.get("reranker")
        metric, index_type = spec.get("metric", "cosine"), spec.get("index_type", "flat")
        if embedder:
            if not dim:
                dim = mgr.get(embedder, "embedder").pipeline.dim
            embed = lambda texts: mgr.get(embedder, "embedder").pipeline.embed(list(texts))[0]
        if reranker:
            rerank = lambda q, docs: mgr.get(reranker, "reranker").pipeline.rerank(q, list(docs))[0]
        dense = None
        if dim:
            if index_type == "hbc":
                dense = _HbcAdapter(dim, metric)
            elif index_type == "flat":
                dense = GrowableFlatIndex(dim, metric, device=str(mgr.device))
            elif index_type == "hnsw":
                from ..index.hnsw import HNSWIndex

                dense = HNSWIndex(dim, metric, neighbors=int(spec.get("neighbors", 16)),
                                  ef_construction=int(spec.get("ef_construction", 200)),
                                  ef_search=int(spec.get("ef_search", 64)))
            else:
                raise ValueError(f"unknown index_type {index_type!r}")
        store = None
        if data_dir:
            from ..index.lsm_store import LsmStore

            store = LsmStore(os.path.join(table_dir(table), "store"))
        tbl = Table(table, dense_index=dense, embed=embed, rerank=rerank, text_field=spec.get("text_field", "text"),
                    store=store)
        restored = tbl.recover()
        app.state.tables[table] = tbl
        return {"table": table, "dimension": dim, "metric": metric, "index_type": index_type,
                "durable": bool(data_dir), "restored": restored}

    if data_dir and os.path.isdir(os.path.join(data_dir, "tables")):
        for name in sorted(os.listdir(os.path.join(data_dir, "tables"))):
            spec_path = os.path.join(data_dir, "tables", name, "table.json")
            if os.path.exists(spec_path):
                with open(spec_path, encoding="utf-8") as f:
                    build_table(name, json.load(f))

    async def table_create(table: str, request: Request):
        req, bad = await parse(request, S.TableCreateRequest)
        if bad:
            return bad
        if table in app.state.tables:
            return _err(409, "table_exists", f"table {table!r} already exists")

        def work():
            spec = req.model_dump()
            info = build_table(table, spec)
            if data_dir:
                with open(os.path.join(table_dir(table), "table.json"), "w", encoding="utf-8") as f:
                    json.dump({**spec, "dimension": info["dimension"]}, f)
            return info

        return await asyncio.to_thread(run_guarded, "table_create", 1, work)

    async def table_batch(table: str, request: Request):
        req, bad = await parse(request, S.BatchRequest)
        if bad:
            return bad
        tbl = app.state.tables.get(table)
        if tbl is None:
            return _err(404, "table_not_found", f"table {table!r} does not exist")

        def work():
            emb = None
            if req.embeddings is not None and req.inserts:
                emb = torch.tensor([req.embeddings[k] for k in req.inserts], dtype=torch.float32)
            if req.inserts:
                tbl.upsert(req.inserts, emb)
            deleted = sum(1 for k in req.deletes if tbl.delete(k))
            return {"inserted": len(req.inserts), "deleted": deleted, "count": len(tbl)}

        return await asyncio.to_thread(run_guarded, "table_batch", max(1, len(req.inserts)), work)

    async def table_query(table: str, request: Request):
        req, bad = await parse(request, S.TableQueryRequest)
        if bad:
            return bad
        tbl = app.state.tables.get(table)
        if tbl is None:
            return _err(404, "table_not_found", f"table {table!r} does not exist")

        def work():
            from ..index.fusion import MergeConfig, Pruner
            from ..index.table import TableQuery

            t0 = time.perf_counter()
            ft = req.full_text_search
            if isinstance(ft, dict):
                ft = ft.get("query") or ft.get("match") or ""
            emb = None
            if req.embeddings is not None:
                e = req.embeddings
                if isinstance(e, dict):          # {index name: vector}: the table has one dense index
                    e = next(iter(e.values()))
                emb = decode_vectors(e)[0]
            mc = req.merge_config or {}
            merge = MergeConfig(mc.get("strategy", "rrf"), dict(mc.get("weights") or {}),
                                int(mc.get("window_size", 0) or 0), float(mc.get("rank_constant", 60.0) or 60.0))
            pr = Pruner(**{k: v for k, v in (req.pruner or {}).items() if k in Pruner.__dataclass_fields__}) \
                if req.pruner else None
            rq = None
            if req.reranker is not None:
                rq = req.reranker.get("query") or req.semantic_search or (ft if isinstance(ft, str) else None)
            if req.search_after is not None and (req.offset or not req.order_by):
                raise ValueError("search_after needs order_by and excludes offset")
            if req.order_by and (emb is not None or req.semantic_search):
                raise ValueError("order_by applies to full-text queries; semantic results are ordered by similarity")
            prof = {} if req.profile else None
            want_all = req.count or bool(req.aggregations)      # counting and aggregating look at every match
            q = TableQuery(embedding=emb, semantic_search=req.semantic_search, full_text_search=ft or None,
                           limit=len(tbl) + 1 if want_all else req.limit + req.offset,
                           search_effort=req.search_effort,
                           distance_under=req.distance_under, distance_over=req.distance_over, merge=merge,
                           pruner=pr, rerank_query=rq,
                           rerank_field=(req.reranker or {}).get("field", tbl.text_field),
                           filter_prefix=req.filter_prefix, filter_query=req.filter_query,
                           exclusion_query=req.exclusion_query, order_by=req.order_by,
                           search_after=req.search_after, profile=prof)
            hits = tbl.query(q)
            total = len(hits)
            aggs = None
            if req.aggregations:
                from ..index.aggregations import aggregate

                aggs = aggregate([h.document or {} for h in hits], req.aggregations)
            hits = [] if req.count else hits[req.offset: req.offset + req.limit]
            out = []
            for h in hits:
                src = h.document or {}
                if req.fields is not None:
                    src = {k: v for k, v in src.items() if k in req.fields}
                rec = {"_id": h.id, "_score": h.score, "_index_scores": h.index_scores, "_source": src}
                if h.sort is not None:
                    rec["_sort"] = h.sort
                out.append(rec)
            body = {"hits": {"total": total if want_all else len(out), "hits": out,
                             "max_score": max((x["_score"] for x in out), default=0.0)},
                    "took": int((time.perf_counter() - t0) * 1e3), "status": 200, "table": table}
            if aggs is not None:
                body["aggregations"] = aggs
            if prof is not None:
                body["profile"] = {k: (round(v, 3) if isinstance(v, float) else v) for k, v in prof.items()}
            return {"responses": [body]}

        return await asyncio.to_thread(run_guarded, "table_query", 1, work)

    async def table_drop(table: str):
        tbl = app.state.tables.pop(table, None)
        if tbl is None:
            return _err(404, "table_not_found", f"table {table!r} does not exist")

        def work():
            if tbl.store is not None:
                tbl.store.close()
                shutil.rmtree(table_dir(table), ignore_errors=True)
            return {"table": table, "dropped": True}

        return await asyncio.to_thread(run_guarded, "table_drop", 1, work)

    async def table_list():
        return {"tables": [{"name": n, "count": len(t)} for n, t in app.state.tables.items()]}

    # ---- models / health / metrics ------------------------------------------------------------------------
    async def models():
        per_task = mgr.list_models()
        data = [{"id": n, "object": "model", "owned_by": "antfly-b200", "task": t[:-1]}
                for t in ("generators", "embedders", "rerankers") for n in per_task.get(t, {})]
        body = {"object": "list", "data": data, "allow_downloads": bool(fetcher.policy.allow_downloads),
                "backends": {"default": "b200", "available": ["b200" if torch.cuda.is_available() else "cpu-oracle"]}}
        body.update(per_task)
        return body

    async def metrics_ep():
        for name, sched_owner in list(mgr._models.items()):
            eng = getattr(getattr(sched_owner.pipeline, "engine", None), "sched", None)
            if eng is not None:
                for k, v in eng.stats().items():
                    metrics.sched.labels(k).set(v)
                e = sched_owner.pipeline.engine
                metrics.kv_free_blocks.labels(sched_owner.name).set(e.cache.alloc.free_blocks)
                for k in ("rounds", "drafted", "matched", "rejected", "accepted", "corrections", "bonus"):
                    metrics.spec.labels(k).set(getattr(e.spec, k))
        return Response(metrics.render(), media_type="text/plain; version=0.0.4")

    async def healthz():
        return {"status": "ok"}

    async def readyz():
        return {"status": "ready", "device": str(mgr.device), "loaded_models": mgr.loaded_count()}

    for path in ("/ai/v1/embed", "/ai/v1/embeddings"):
        app.add_api_route(path, embed, methods=["POST"])
    app.add_api_route("/ai/v1/rerank", rerank, methods=["POST"])
    app.add_api_route("/ai/v1/rerank_multimodal", rerank_multimodal, methods=["POST"])
    for path in ("/ai/v1/generate", "/ai/v1/chat/completions"):
        app.add_api_route(path, generate, methods=["POST"])
    app.add_api_route("/openai/v1/chat/completions", generate, methods=["POST"])
    app.add_api_route("/openai/v1/embeddings", embed, methods=["POST"])
    app.add_api_route("/openai/v1/models", openai_models, methods=["GET"])
    app.add_api_route("/anthropic/v1/messages", anthropic_messages, methods=["POST"])
    app.add_api_route("/ai/v1/chunk", chunk_ep, methods=["POST"])
    app.add_api_route("/ai/v1/rewrite", rewrite, methods=["POST"])
    app.add_api_route("/ai/v1/classify", classify, methods=["POST"])
    app.add_api_route("/ai/v1/recognize", recognize, methods=["POST"])
    app.add_api_route("/ai/v1/extract", extract, methods=["POST"])
    app.add_api_route("/ai/v1/transcribe", transcribe, methods=["POST"])
    app.add_api_route("/ai/v1/read", read, methods=["POST"])
    app.add_api_route("/ai/v1/layout", layout, methods=["POST"])
    app.add_api_route("/ai/v1/search", search, methods=["POST"])
    app.add_api_route("/db/v1/tables", table_list, methods=["GET"])
    app.add_api_route("/db/v1/tables/{table}", table_create, methods=["POST", "PUT"])
    app.add_api_route("/db/v1/tables/{table}", table_drop, methods=["DELETE"])
    app.add_api_route("/db/v1/tables/{table}/batch", table_batch, methods=["POST"])
    app.add_api_route("/db/v1/tables/{table}/query", table_query, methods=["POST"])
    app.add_api_route("/ai/v1/models", models, methods=["GET"])
    app.add_api_route("/ai/v1/metrics", metrics_ep, methods=["GET"])
    app.add_api_route("/metrics", metrics_ep, methods=["GET"])
    app.add_api_route("/healthz", healthz, methods=["GET"])
    app.add_api_route("/readyz", readyz, methods=["GET"])
    return app


def serve(host: str = "127.0.0.1", port: int = 11433, **kw) -> None:
    import uvicorn

    uvicorn.run(create_app(**kw), host=host, port=port, timeout_keep_alive=300)
