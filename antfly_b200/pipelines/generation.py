"""Generation pipeline: chat template -> tokenize -> engine -> detokenize, with streaming deltas.

Mirrors the reference's generateWithCallback (zig/pkg/inference/src/pipelines/generation.zig:1288): apply the
model's Jinja chat template (``chat_template.jinja`` or the ``chat_template`` field of tokenizer_config.json, a
plain role-tagged fallback otherwise), add BOS, run prefill + decode through the scheduler, emit decoded text
deltas, and report usage and timing (``generate_timing_ms: prompt_format tokenize prefill decode total``).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

from ..runtime.engine import LLMEngine
from ..runtime.sampling_params import SamplingParams

DEFAULT_TEMPLATE = (
    "{% for m in messages %}<|{{ m['role'] }}|>\n{{ m['content'] }}\n{% endfor %}"
    "{% if add_generation_prompt %}<|assistant|>\n{% endif %}"
)


@dataclass
class GenerationOutput:
    text: str
    token_ids: List[int]
    finish_reason: str
    prompt_tokens: int
    completion_tokens: int
    timing_ms: Dict[str, float] = field(default_factory=dict)

    def timing_line(self) -> str:
        t = self.timing_ms
        return ("generate_timing_ms: prompt_format=%.1f tokenize=%.1f prefill=%.1f decode=%.1f total=%.1f" %
                (t.get("prompt_format", 0), t.get("tokenize", 0), t.get("prefill", 0), t.get("decode", 0),
                 t.get("total", 0)))


class ChatTemplate:
    def __init__(self, source: Optional[str] = None):
        import jinja2

        env = jinja2.Environment(trim_blocks=True, lstrip_blocks=True)
        env.globals["raise_exception"] = lambda m: (_ for _ in ()).throw(ValueError(m))
        self.source = source or DEFAULT_TEMPLATE
        self.template = env.from_string(self.source)

    def apply(self, messages: Sequence[dict], add_generation_prompt: bool = True,
              image_placeholder: Optional[str] = None, **extra) -> str:
        msgs = []
        for m in messages:
            c = m.get("content", "")
            if isinstance(c, list):  # OpenAI content parts: text parts, and a placeholder where an image stands
                c = "".join(
                    p.get("text", "") if p.get("type") == "text" else
                    (image_placeholder or "") if p.get("type") in ("image_url", "image") else ""
                    for p in c if isinstance(p, dict))
            msgs.append({**m, "content": c})
        return self.template.render(messages=msgs, add_generation_prompt=add_generation_prompt, **extra)


class Generator:
    def __init__(self, engine: LLMEngine, tokenizer, chat_template: Optional[str] = None, add_bos: bool = True,
                 vlm=None):
        self.engine, self.tokenizer, self.add_bos = engine, tokenizer, add_bos
        self.vlm = vlm                  # image adapter (pipelines.vlm); None for text-only models
        self.template = ChatTemplate(chat_template)
        if engine.eos is None and tokenizer.special.eos_id is not None:
            engine.eos = tokenizer.special.eos_id

    def generate(self, messages_or_prompt, params: SamplingParams, raw_prompt: bool = False,
                 on_delta: Optional[Callable[[str], None]] = None, images: Optional[Sequence] = None
                 ) -> GenerationOutput:
        """``images`` (or image parts inside chat messages) need a model with an image adapter; in a plain prompt
        each image stands where the adapter's placeholder text is written (appended in front if it is absent)."""
        t0 = time.perf_counter()
        images = list(images or [])
        ph = self.vlm.placeholder if self.vlm is not None else None
        if isinstance(messages_or_prompt, str):
            text = messages_or_prompt
            if images and ph and text.count(ph) < len(images):
                text = ph * (len(images) - text.count(ph)) + text
            prompt = text if raw_prompt else self.template.apply([{"role": "user", "content": text}])
        else:
            if self.vlm is not None:
                from .vlm import split_content

                images = split_content(messages_or_prompt) + images
            prompt = self.template.apply(messages_or_prompt, image_placeholder=ph)
        if images and self.vlm is None:
            raise ValueError("this model does not take images")
        t1 = time.perf_counter()
        ids = self.tokenizer.encode_prompt(prompt, add_bos=self.add_bos)
        soft = None
        if self.vlm is not None:
            ids, soft = self.vlm.expand(ids, images)
        t2 = time.perf_counter()
        emitted = {"n": 0, "text": ""}
        collected: List[int] = []

        def on_token(_rid, tok):
            collected.append(tok)
            if on_delta is not None:
                full = self.tokenizer.decode(collected)
                # Hold back while the tail is an incomplete UTF-8 sequence.
                if not full.endswith("�"):
                    delta = full[len(emitted["text"]):]
                    if delta:
                        emitted["text"] = full
                        on_delta(delta)

        p0, d0 = self.engine.timing["prefill_s"], self.engine.timing["decode_s"]
        res = self.engine.generate([ids], params, on_token=on_token, soft=[soft] if soft is not None else None)[0]
        t3 = time.perf_counter()
        toks = res.token_ids
        eos = self.engine.eos
        text_ids = [t for t in toks if t != eos]
        out = GenerationOutput(self.tokenizer.decode(text_ids), toks, res.finish_reason, len(ids), len(toks), {
            "prompt_format": (t1 - t0) * 1e3, "tokenize": (t2 - t1) * 1e3,
            "prefill": (self.engine.timing["prefill_s"] - p0) * 1e3,
            "decode": (self.engine.timing["decode_s"] - d0) * 1e3, "total": (t3 - t0) * 1e3})
        return out


class StatefulGenerator:
    """Generation pipeline for decoders that carry a per-sequence state of their own instead of block tables in
    the paged-KV engine (hybrid recurrent / attention decoders such as Qwen3.5, and decoders with per-layer cache
    geometries such as Gemma-4): same interface as :class:`Generator`, one request at a time.  The model provides
    ``forward(ids, state) -> (logits [T, vocab], state)``; sampling follows the request's temperature / top-k /
    top-p / min-p on the last position's logits (greedy at temperature <= 0)."""

    def __init__(self, model, tokenizer, chat_template: Optional[str] = None, add_bos: bool = True,
                 eos_token_id: Optional[int] = None, assistant=None):
        self.model, self.tokenizer, self.add_bos = model, tokenizer, add_bos
        self.assistant = assistant          # drafts for greedy requests (``stream(ids, n, k, forward_kwargs)``)
        self.template = ChatTemplate(chat_template)
        self.vlm = None
        self.eos = eos_token_id if eos_token_id is not None else tokenizer.special.eos_id

    def _pick(self, logits, params: SamplingParams, gen) -> int:
        import torch

        if params.greedy:
            return int(logits.argmax())
        lg = logits.float() / params.temperature
        if params.top_k:
            kth = lg.topk(min(params.top_k, lg.numel())).values[-1]
            lg = lg.masked_fill(lg < kth, float("-inf"))
        p = lg.softmax(-1)
        if params.top_p < 1.0:
            sp, si = p.sort(descending=True)
            keep = (sp.cumsum(0) - sp) < params.top_p
            p = torch.zeros_like(p).scatter(0, si[keep], sp[keep])
        if params.min_p > 0.0:
            p = p.masked_fill(p < params.min_p * p.max(), 0.0)
        return int(torch.multinomial(p / p.sum(), 1, generator=gen))

    def generate(self, messages_or_prompt, params: SamplingParams, raw_prompt: bool = False,
                 on_delta: Optional[Callable[[str], None]] = None, images=None) -> GenerationOutput:
        import torch

        if images and not hasattr(self.model, "prepare_images"):
            raise ValueError("this model does not take images")
        t0 = time.perf_counter()
        if isinstance(messages_or_prompt, str):
            prompt = messages_or_prompt if raw_prompt else self.template.apply(
                [{"role": "user", "content": messages_or_prompt}])
        else:
            prompt = self.template.apply(messages_or_prompt)
        t1 = time.perf_counter()
        ids = self.tokenizer.encode_prompt(prompt, add_bos=self.add_bos)
        t2 = time.perf_counter()
        dev = self.model.device
        gen = torch.Generator(device="cpu")
        if params.seed is not None:
            gen.manual_seed(params.seed)
        extra = {}
        if images:
            ids, extra = self.model.prepare_images(ids, images, bos_id=self.tokenizer.special.bos_id)
        k = getattr(params, "speculative_k", None) or 4
        drafting = self.assistant is not None and params.greedy and not images
        marks = {}

        def plain():
            logits, st = self.model.forward(torch.tensor(ids, dtype=torch.int64, device=dev), None, **extra)
            marks["prefill"] = time.perf_counter()
            for _ in range(params.max_tokens):
                tok = self._pick(logits[-1].cpu(), params, gen)
                yield tok
                logits, st = self.model.forward(torch.tensor([tok], dtype=torch.int64, device=dev), st)

        # Drafting serves greedy, text-only requests (the verifier compares argmaxes); others decode token by token.
        source = self.assistant.stream(ids, params.max_tokens, k) if drafting else plain()
        toks: List[int] = []
        shown = ""
        finish = "length"
        for tok in source:
            marks.setdefault("prefill", time.perf_counter())
            toks.append(tok)
            if (not params.ignore_eos and tok == self.eos) or tok in params.stop_token_ids:
                finish = "stop"
                break
            if on_delta is not None:
                full = self.tokenizer.decode(toks)
                if not full.endswith("\ufffd"):
                    if full[len(shown):]:
                        on_delta(full[len(shown):])
                    shown = full
            if len(toks) >= params.max_tokens:
                break
        source.close()
        t3 = marks.get("prefill", time.perf_counter())
        t4 = time.perf_counter()
        text_ids = [t for t in toks if t != self.eos]
        return GenerationOutput(self.tokenizer.decode(text_ids), toks, finish, len(ids), len(toks), {
            "prompt_format": (t1 - t0) * 1e3, "tokenize": (t2 - t1) * 1e3, "prefill": (t3 - t2) * 1e3,
            "decode": (t4 - t3) * 1e3, "total": (t4 - t0) * 1e3})
