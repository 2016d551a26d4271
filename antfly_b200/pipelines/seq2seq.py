"""Text-to-text generation with an encoder-decoder model (T5 / Flan-T5): query rewriting, summarisation,
instruction prompts.  Same call shape as :class:`antfly_b200.pipelines.generation.Generator` so the HTTP handlers
and the CLI can use either; chat messages are flattened to one input text (encoder-decoder checkpoints have no
chat template).  Follows the reference's encoder-decoder pipeline (zig/pkg/inference/src/pipelines/
encoder_decoder.zig, pipelines/rewriting.zig): encode once, greedy-decode with cached keys / values until the
end-of-sequence token or the token limit.
"""
from __future__ import annotations

import time
from typing import Callable, List, Optional

from ..models.t5 import T5Model  # noqa: F401  (the pipeline also drives BartModel: same interface)
from ..runtime.sampling_params import SamplingParams
from .generation import GenerationOutput


def _takes_skip(tokenizer) -> bool:
    import inspect

    try:
        return "skip_special" in inspect.signature(tokenizer.decode).parameters
    except (TypeError, ValueError):
        return False


class Seq2SeqGenerator:
    def __init__(self, model: T5Model, tokenizer, max_input_tokens: int = 512):
        self.model, self.tokenizer, self.max_input_tokens = model, tokenizer, max_input_tokens

    def _encode(self, text: str) -> List[int]:
        ids = list(self.tokenizer.encode(text))
        eos = self.model.cfg.eos_token_id
        ids = [t for t in ids if t != eos][: self.max_input_tokens - 1]
        return ids + [eos]                                     # T5 inputs end with </s>

    def generate(self, messages_or_prompt, params: Optional[SamplingParams] = None, raw_prompt: bool = False,
                 on_delta: Optional[Callable[[str], None]] = None, keep_special: bool = False) -> GenerationOutput:
        """``keep_special`` decodes marker tokens too (relation-extraction checkpoints write their structure with
        added special tokens)."""
        t0 = time.perf_counter()
        if isinstance(messages_or_prompt, str):
            text = messages_or_prompt
        else:
            parts = []
            for m in messages_or_prompt:
                c = m.get("content", "")
                if isinstance(c, list):
                    c = "".join(p.get("text", "") for p in c if isinstance(p, dict) and p.get("type") == "text")
                parts.append(c)
            text = "\n".join(p for p in parts if p)
        ids = self._encode(text)
        t1 = time.perf_counter()
        max_new = params.max_tokens if params is not None else 64
        state = self.model.start_decoding(self.model.encode(ids))
        t2 = time.perf_counter()
        cfg = self.model.cfg
        forced = getattr(cfg, "forced_bos_token_id", -1)
        feed = [cfg.decoder_start_token_id] + ([forced] if forced is not None and forced >= 0 else [])
        out, emitted, reason = [], "", "length"
        dec = (lambda ids: self.tokenizer.decode(ids, skip_special=False)) if keep_special and _takes_skip(
            self.tokenizer) else self.tokenizer.decode
        for _ in range(max_new):
            tok = int(self.model.decode(state, feed)[-1].argmax())
            feed = [tok]
            if tok == self.model.cfg.eos_token_id:
                reason = "stop"
                break
            out.append(tok)
            if on_delta is not None:
                full = dec(out)
                if not full.endswith("�") and len(full) > len(emitted):
                    on_delta(full[len(emitted):])
                    emitted = full
        t3 = time.perf_counter()
        return GenerationOutput(dec(out), out, reason, len(ids), len(out), {
            "prompt_format": 0.0, "tokenize": (t1 - t0) * 1e3, "prefill": (t2 - t1) * 1e3,
            "decode": (t3 - t2) * 1e3, "total": (t3 - t0) * 1e3})
