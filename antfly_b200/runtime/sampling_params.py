"""Per-request sampling parameters (the generate endpoint's knobs)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class SamplingParams:
    max_tokens: int = 256
    temperature: float = 0.0        # <= 0: greedy
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    stop_token_ids: List[int] = field(default_factory=list)
    ignore_eos: bool = False
    seed: Optional[int] = None
    cache_compaction_ratio: Optional[float] = None  # in (0, 1): compact the KV cache to this fraction after prefill
    grammar: Optional[object] = None  # antfly_b200.runtime.grammar.JsonGrammar: constrains every sampled token
    speculative_k: Optional[int] = None  # draft tokens per speculative round (1..16); None: the engine's default

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def needs_penalties(self) -> bool:
        return self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0 or self.presence_penalty != 0.0
