"""Minimal HTTP client for the inference API (what the reference ships as its Python SDK's inference part,
py/packages/sdk): embeddings, rerank, generate / chat with optional streaming, rewrite, extract, classify,
recognize, chunk, read, transcribe, and the hybrid table calls.  Depends only on ``requests``."""
from __future__ import annotations

import base64
import json
import time
from typing import Any, Dict, Iterator, List, Optional, Sequence, Union

import requests


class ApiError(RuntimeError):
    def __init__(self, status: int, code: str, message: str):
        super().__init__(f"{status} {code}: {message}")
        self.status, self.code, self.message = status, code, message


class Client:
    def __init__(self, base_url: str = "http://127.0.0.1:11433", timeout: float = 300.0,
                 api_key: Optional[str] = None):
        self.base, self.timeout = base_url.rstrip("/"), timeout
        self.s = requests.Session()
        if api_key:
            self.s.headers["Authorization"] = f"Bearer {api_key}"

    # -- plumbing ------------------------------------------------------------------------------------------
    def _post(self, path: str, body: Dict[str, Any]) -> Dict[str, Any]:
        r = self.s.post(self.base + path, json=body, timeout=self.timeout)
        if r.status_code >= 400:
            try:
                e = r.json()
            except ValueError:
                e = {"error": "http_error", "message": r.text}
            raise ApiError(r.status_code, str(e.get("error")), str(e.get("message")))
        return r.json()

    def wait_ready(self, timeout: float = 120.0) -> None:
        t0 = time.time()
        while True:
            try:
                if self.s.get(self.base + "/readyz", timeout=2).status_code == 200:
                    return
            except requests.RequestException:
                pass
            if time.time() - t0 > timeout:
                raise TimeoutError("server did not become ready")
            time.sleep(0.2)

    # -- inference -----------------------------------------------------------------------------------------
    def models(self) -> Dict[str, Any]:
        return self.s.get(self.base + "/ai/v1/models", timeout=self.timeout).json()

    def embed(self, model: str, texts: Union[str, Sequence[str]], dimensions: Optional[int] = None,
              task_type: Optional[str] = None) -> List[List[float]]:
        body: Dict[str, Any] = {"model": model, "input": texts if isinstance(texts, str) else list(texts)}
        if dimensions:
            body["dimensions"] = dimensions
        if task_type:
            body["task_type"] = task_type
        return [d["embedding"] for d in self._post("/ai/v1/embed", body)["data"]]

    def rerank(self, model: str, query: str, documents: Sequence[str]) -> List[float]:
        data = self._post("/ai/v1/rerank", {"model": model, "query": query, "prompts": list(documents)})["data"]
        return [d["score"] for d in sorted(data, key=lambda d: d["index"])]

    def chat(self, model: str, messages: Sequence[Dict[str, Any]], **params) -> Dict[str, Any]:
        return self._post("/ai/v1/chat/completions", {"model": model, "messages": list(messages), **params})

    def generate(self, model: str, prompt: str, **params) -> str:
        out = self.chat(model, [{"role": "user", "content": prompt}], **params)
        return out["choices"][0]["message"]["content"] or ""

    def stream(self, model: str, messages: Sequence[Dict[str, Any]], **params) -> Iterator[str]:
        """Yields text deltas of a streamed chat completion."""
        body = {"model": model, "messages": list(messages), "stream": True, **params}
        with self.s.post(self.base + "/ai/v1/chat/completions", json=body, timeout=self.timeout, stream=True) as r:
            if r.status_code >= 400:
                e = r.json()
                raise ApiError(r.status_code, str(e.get("error")), str(e.get("message")))
            for line in r.iter_lines():
                if not line or not line.startswith(b"data: "):
                    continue
                payload = line[6:]
                if payload == b"[DONE]":
                    return
                chunk = json.loads(payload)
                if "error" in chunk:
                    raise ApiError(500, str(chunk.get("error")), str(chunk.get("message")))
                delta = chunk["choices"][0]["delta"].get("content")
                if delta:
                    yield delta

    def rewrite(self, model: str, inputs: Sequence[str], max_tokens: int = 128) -> List[str]:
        data = self._post("/ai/v1/rewrite", {"model": model, "inputs": list(inputs), "max_tokens": max_tokens})["data"]
        return [d["texts"][0] for d in sorted(data, key=lambda d: d["index"])]

    def extract(self, model: str, texts: Sequence[str], schema: Dict[str, Any], **options) -> List[Dict[str, Any]]:
        return self._post("/ai/v1/extract", {"model": model, "inputs": [{"content": t} for t in texts],
                                             "schema": schema, "options": options})["data"]

    def transcribe(self, model: str, wav_bytes: bytes, language: Optional[str] = None) -> str:
        body: Dict[str, Any] = {"model": model, "audio": base64.b64encode(wav_bytes).decode()}
        if language:
            body["language"] = language
        return self._post("/ai/v1/transcribe", body)["data"][0]["text"]

    def chunk(self, text_or_bytes: Union[str, bytes], mime_type: Optional[str] = None,
              config: Optional[Dict[str, Any]] = None) -> List[Dict[str, Any]]:
        """Chunks of a text, or of a media payload (WAV audio in windows or voice-activity segments, GIF frames)."""
        part: Any = text_or_bytes
        if isinstance(text_or_bytes, (bytes, bytearray)):
            part = {"type": "media", "mime_type": mime_type or "application/octet-stream",
                    "data": base64.b64encode(bytes(text_or_bytes)).decode()}
        body: Dict[str, Any] = {"input": part}
        if config:
            body["config"] = config
        data = self._post("/ai/v1/chunk", body)["data"]
        return data[0]["chunks"] if data and isinstance(data[0], dict) and "chunks" in data[0] else data

    def classify(self, model: str, texts: Sequence[str], labels: Sequence[str] = (), **options) -> List[List[Dict[str, Any]]]:
        body = {"model": model, "texts": list(texts), "labels": list(labels), **options}
        data = self._post("/ai/v1/classify", body)["data"]
        return [d["classifications"] for d in sorted(data, key=lambda d: d["index"])]

    def recognize(self, model: str, texts: Sequence[str], labels: Sequence[str] = (),
                  relation_labels: Sequence[str] = (), resolver: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
        body: Dict[str, Any] = {"model": model, "texts": list(texts), "labels": list(labels),
                                "relation_labels": list(relation_labels)}
        if resolver is not None:
            body["resolver"] = resolver
        return self._post("/ai/v1/recognize", body)

    def read(self, model: str, images: Sequence[bytes], mime_type: str = "image/png", **options) -> Dict[str, Any]:
        urls = [{"url": f"data:{mime_type};base64," + base64.b64encode(b).decode()} for b in images]
        return self._post("/ai/v1/read", {"model": model, "images": urls, **options})

    # -- tables --------------------------------------------------------------------------------------------
    def create_table(self, name: str, **spec) -> Dict[str, Any]:
        return self._post(f"/db/v1/tables/{name}", spec)

    def drop_table(self, name: str) -> Dict[str, Any]:
        r = self.s.delete(self.base + f"/db/v1/tables/{name}", timeout=self.timeout)
        if r.status_code >= 400:
            e = r.json()
            raise ApiError(r.status_code, str(e.get("error")), str(e.get("message")))
        return r.json()

    def upsert(self, table: str, docs: Dict[str, Dict[str, Any]], deletes: Sequence[str] = ()) -> Dict[str, Any]:
        return self._post(f"/db/v1/tables/{table}/batch", {"inserts": docs, "deletes": list(deletes)})

    def query(self, table: str, **q) -> List[Dict[str, Any]]:
        return self._post(f"/db/v1/tables/{table}/query", q)["responses"][0]["hits"]["hits"]
