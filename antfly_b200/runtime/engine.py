"""Generation engine: continuous batching over a paged KV cache, CUDA-graph decode, speculative decoding.

The control flow mirrors the reference's NativeGenerationPipeline
(zig/pkg/inference/src/pipelines/generation.zig:1288 generateWithCallback, :1819 executePrefill, :2079
standardDecode, :2889 speculativeDecode, :3228 acceptVerifiedDraftTokens, :3436 runScheduledDecodeBatch): the
scheduler packs a step (decode tokens first, then prefill chunks), one fused forward runs it, the sampler picks
tokens, sequences grow or finish.  On the B200 the whole decode step of a steady batch is one CUDA graph replay
between a pinned-memory H2D copy of the step's integer inputs and a D2H read of the sampled tokens.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
import torch

from ..models.llama import LlamaModel, StepBatch
from ..ops import attention as A
from ..ops import sampling as S
from .kv_cache import KvOutOfBlocks, PagedKvCache
from .prefix_cache import PrefixCache
from .sampling_params import SamplingParams
from .scheduler import SchedulerPolicy, StepItem, StepScheduler


@dataclass
class SpecStats:
    """Counters of the reference's SpeculativeDecodeStats (generation.zig:205-216)."""
    rounds: int = 0
    drafted: int = 0
    matched: int = 0
    rejected: int = 0
    accepted: int = 0
    corrections: int = 0
    bonus: int = 0

    @property
    def acceptance_rate(self) -> float:
        return self.matched / self.drafted if self.drafted else 0.0

    def line(self) -> str:
        return (f"speculative: rounds={self.rounds} drafted={self.drafted} matched={self.matched} "
                f"rejected={self.rejected} accepted={self.accepted} corrections={self.corrections} bonus={self.bonus}")


@dataclass
class Request:
    rid: int
    prompt: List[int]
    params: SamplingParams
    out: List[int] = field(default_factory=list)
    finished: bool = False
    finish_reason: Optional[str] = None
    t_admit: float = 0.0
    t_first: Optional[float] = None
    row: int = -1  # row in the penalty-count table
    kv_removed: int = 0  # tokens dropped from the physical KV cache by compaction (logical positions keep counting)
    # multimodal prompts: prompt positions whose embedding is given (image patches), those embeddings [n, H], the
    # prompt's three rotary position streams [3, len(prompt)], and what to add to a cache index past the prompt
    soft_rows: Optional[List[int]] = None
    soft_vals: Optional[torch.Tensor] = None
    pos3: Optional[torch.Tensor] = None
    rope_delta: int = 0
    bidir_spans: Optional[List[tuple]] = None     # [start, end) prompt ranges that attend in both directions
    draft_attached: bool = False                  # has a sequence in the separate draft model's KV cache

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.out


@dataclass
class GenerationResult:
    token_ids: List[int]
    finish_reason: str
    prompt_tokens: int
    ttft_s: float


class _StaticStep:
    """Static device buffers + captured graph for a decode step of fixed batch size."""

    def __init__(self, B: int, max_blocks: int, device):
        self.B, self.max_blocks = B, max_blocks
        n = 3 * B + B + B + B + B * max_blocks  # ids, positions, slots | q_starts | q_lens | kv_lens | tables
        self.host = torch.empty(n, dtype=torch.int32).pin_memory()
        self.dev = torch.empty(n, dtype=torch.int32, device=device)
        o = 0
        def take(k):
            nonlocal o
            v = (self.host[o:o + k], self.dev[o:o + k])
            o += k
            return v
        (self.h_ids, self.ids), (self.h_pos, self.pos), (self.h_slots, self.slots) = take(B), take(B), take(B)
        (self.h_qs, self.qs), (self.h_ql, self.ql), (self.h_kvl, self.kvl) = take(B), take(B), take(B)
        self.h_tab, tab = take(B * max_blocks)
        self.h_tab = self.h_tab.view(B, max_blocks)
        self.tab = tab.view(B, max_blocks)
        self.h_qs.copy_(torch.arange(B, dtype=torch.int32))
        self.h_ql.fill_(1)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.out_tokens: Optional[torch.Tensor] = None
        self.logits: Optional[torch.Tensor] = None
        self.launches = 0

    def h2d_bytes(self) -> int:
        return self.host.numel() * 4


class LLMEngine:
    def __init__(self, model: LlamaModel, num_blocks: int, page: int = 16, max_batch: int = 64,
                 max_step_tokens: int = 8192, prefill_chunk: int = 2048, kv_dtype: str = "bf16",
                 use_cuda_graph: bool = True, draft_layers: int = 0, spec_k: int = 4, eos_token_id: Optional[int] = None,
                 max_seq_len: int = 8192 + 1024, max_queue: int = 0, prefix_cache: bool = False,
                 prefix_cache_entries: int = 256, draft_model: Optional[LlamaModel] = None,
                 draft_num_blocks: Optional[int] = None):
        """``draft_layers`` > 0: self-speculative draft (the target's first layers, sharing its KV cache).
        ``draft_model``: a separate, smaller model with the same vocabulary as the draft (the reference's
        ``draft_model`` request field, zig/pkg/inference/src/pipelines/generation.zig:1563-1745): it gets a paged KV
        cache and block tables of its own, drafts K <= 16 tokens greedily per round, the target verifies them in
        one pass with each request's sampler, and both caches are truncated to what was accepted."""
        self.model = model
        self.device = model.device
        self.page = page
        self.kv_dtype = kv_dtype
        self.cache = PagedKvCache(model.n_layers, num_blocks, model.Hkv, model.D, page, kv_dtype, self.device)
        self.max_batch = max_batch
        self.max_blocks = (max_seq_len + page - 1) // page
        self.sched = StepScheduler(SchedulerPolicy(max_step_items=max_batch, max_step_query_tokens=max_step_tokens,
                                                   prefill_chunk=prefill_chunk, min_chunk=32, decode_streak=4,
                                                   page=page, max_queue=max_queue))
        # Decode steps are captured in CUDA graphs when nothing in a step depends on the data; the integer codecs
        # encode new rows with tensor ops (and turbo3 builds its sign table on first use), so they run eagerly.
        self.use_graph = (use_cuda_graph and self.device.type == "cuda" and getattr(model, "graph_safe", True)
                          and self.cache.codec in (None, "fp8"))
        self.eos = eos_token_id
        self.reqs: Dict[int, Request] = {}
        self._next_id = 1
        self._static: Dict[tuple, _StaticStep] = {}
        self._attn_scratch: Optional[A.PagedAttnScratch] = None
        self.draft = model.draft_view(draft_layers) if draft_layers > 0 else None
        self.draft_cache: Optional[PagedKvCache] = None
        if draft_model is not None:
            if draft_model.cfg.vocab_size != model.cfg.vocab_size:
                raise ValueError("the draft model must share the target's vocabulary")
            self.draft = draft_model
            self.draft_cache = PagedKvCache(draft_model.n_layers, draft_num_blocks or num_blocks, draft_model.Hkv,
                                            draft_model.D, page, kv_dtype, self.device)
        # Prompts that begin with already-prefilled tokens reuse those KV blocks (not with a sliding window, whose
        # trimming releases the very blocks a later prompt would share).
        self.prefix: Optional[PrefixCache] = None
        if prefix_cache and not getattr(model.cfg, "sliding_window", 0):
            self.prefix = PrefixCache(self.cache.alloc, page, prefix_cache_entries)
        self.spec_k = spec_k
        self.spec = SpecStats()
        self.counts: Optional[torch.Tensor] = None  # [max_batch, V] int16 penalty table, allocated lazily
        self._rows_free = list(range(max_batch))
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.steps = 0
        self._gen = torch.Generator(device=self.device)
        self.timing = {"prefill_s": 0.0, "decode_s": 0.0}

    # ------------------------------------------------------------------------------------------------
    def add_request(self, prompt: Sequence[int], params: SamplingParams, soft: Optional[dict] = None) -> int:
        """``soft`` describes a multimodal prompt: ``rows`` (prompt positions of the placeholder tokens), ``vals``
        (their embeddings, [len(rows), hidden]), ``pos3`` (rotary streams [3, len(prompt)]) and ``delta``.  Such
        prompts neither use nor feed the prefix cache (equal token ids do not mean equal images)."""
        rid = self._next_id
        self._next_id += 1
        shared = 0
        if soft is not None:
            if self.draft is not None:
                raise ValueError("speculative decoding is not available for prompts with images")
            if len(soft["rows"]) != soft["vals"].shape[0] or (
                    soft.get("pos3") is not None and soft["pos3"].shape != (3, len(prompt))):
                raise ValueError("soft-token description does not match the prompt")
        if self.prefix is not None and soft is None:
            eid, n = self.prefix.lookup(prompt)
            if eid is not None:
                try:
                    self.cache.alloc.attach_shared(rid, eid, n)
                    shared = n
                except (KvOutOfBlocks, KeyError):
                    shared = 0
        if not shared:
            self.cache.alloc.attach(rid)
        try:
            self.sched.admit(rid, len(prompt), params.max_tokens, prompt_done=shared)
        except Exception:
            self.cache.alloc.detach(rid)
            raise
        r = Request(rid, list(prompt), params, t_admit=time.perf_counter())
        if soft is not None:
            r.soft_rows, r.soft_vals = [int(i) for i in soft["rows"]], soft["vals"].to(self.device)
            if soft.get("pos3") is not None:
                r.pos3, r.rope_delta = soft["pos3"].to(torch.int64).cpu(), int(soft.get("delta", 0))
            if soft.get("bidir"):
                r.bidir_spans = [(int(a), int(b)) for a, b in soft["bidir"]]
                self.sched.set_atomic_prefill(rid)       # a run must see its later tokens: no chunking
        if params.needs_penalties:
            r.row = self._rows_free.pop()
            if self.counts is None:
                self.counts = torch.zeros((self.max_batch, self.model.cfg.vocab_size), dtype=torch.int16,
                                          device=self.device)
            self.counts[r.row].zero_()
            toks = torch.tensor(r.prompt, dtype=torch.int32, device=self.device)
            S.count_tokens(self.counts, toks, torch.full_like(toks, r.row))
        self.reqs[rid] = r
        return rid

    def _retire(self, r: Request, reason: str) -> None:
        r.finished, r.finish_reason = True, reason
        self.cache.alloc.detach(r.rid)
        if self.draft_cache is not None and r.draft_attached:
            self.draft_cache.alloc.detach(r.rid)
            r.draft_attached = False
        if r.row >= 0:
            self._rows_free.append(r.row)
            r.row = -1

    def has_work(self) -> bool:
        return any(not r.finished for r in self.reqs.values())

    # ------------------------------------------------------------------------------------------------
    def _after_capture(self) -> None:
        """Tensor-parallel ranks meet on the host after capturing a graph: capture allocates and takes tens of
        milliseconds, and a rank that is already replaying would otherwise sit in its kernels' cross-GPU waits for
        as long as the slowest rank still captures."""
        if self.model.tp_size > 1 and getattr(self.model, "comm", None) is not None:
            torch.cuda.synchronize()
            self.model.comm.barrier()

    def _attn_splits(self, B: int, max_kv: int) -> int:
        ctas = B * self.model.Hkv
        if max_kv < 1024:
            return 1
        if ctas >= 256:
            # Enough CTAs already; a 2-way split evens out the last wave (3 CTAs fit per SM).
            return 2 if ctas < 1500 else 1
        return int(min(8, max(1, 444 // max(ctas, 1)), max(1, max_kv // 512)))

    def _scratch_for(self, T: int, splits: int) -> Optional[A.PagedAttnScratch]:
        if splits <= 1:
            return None
        s = self._attn_scratch
        if s is None or s.max_tokens < T or s.max_splits < splits:
            s = A.PagedAttnScratch(max(T, self.max_batch * (self.spec_k + 1)), self.model.Hq, self.model.D,
                                   max(splits, 8), self.device)
            self._attn_scratch = s
        return s

    def _build_batch(self, items: List[StepItem], seq_tokens: List[List[int]]) -> StepBatch:
        """General path: arbitrary mix of prefill chunks and decode tokens.  One pinned staging buffer, one copy."""
        B = len(items)
        alloc = self.cache.alloc
        ids, pos, slots, qs, ql, kvl, rows = [], [], [], [], [], [], []
        tables = np.zeros((B, self.max_blocks), dtype=np.int32)
        t0 = 0
        for i, (it, toks) in enumerate(zip(items, seq_tokens)):
            n = len(toks)
            sl = alloc.append(it.request_id, n)
            ids.extend(toks)
            pos.extend(range(it.kv_before, it.kv_before + n))
            slots.extend(sl.tolist())
            qs.append(t0); ql.append(n); kvl.append(it.kv_before + n - self.reqs[it.request_id].kv_removed)
            bt = alloc.block_table(it.request_id)
            tables[i, : len(bt)] = bt
            rows.append(t0 + n - 1)
            t0 += n
        T = t0
        flat = np.concatenate([np.asarray(ids, np.int32), np.asarray(pos, np.int32), np.asarray(slots, np.int32),
                               np.asarray(qs, np.int32), np.asarray(ql, np.int32), np.asarray(kvl, np.int32),
                               np.asarray(rows, np.int32), tables.reshape(-1)])
        host = torch.from_numpy(flat)
        if self.device.type == "cuda":
            host = host.pin_memory()
        dev = host.to(self.device, non_blocking=True)
        self.h2d_bytes += flat.nbytes
        o = 0
        def take(k):
            nonlocal o
            v = dev[o:o + k]
            o += k
            return v
        d_ids, d_pos, d_slots = take(T), take(T), take(T)
        d_qs, d_ql, d_kvl, d_rows = take(B), take(B), take(B), take(B)
        d_tab = take(B * self.max_blocks).view(B, self.max_blocks)
        max_q = max(ql)
        splits = self._attn_splits(B, max(kvl)) if max_q * (self.model.Hq // self.model.Hkv) <= 16 else 1
        return StepBatch(d_ids, d_pos, d_slots, d_qs, d_ql, d_kvl, d_tab, d_rows, max_q, splits, max_kv=max(kvl))

    def _add_multimodal(self, batch: StepBatch, items: List[StepItem], reqs: List[Request]) -> None:
        """Rotary streams for every token of the step, and the soft-token rows that fall inside its prefill chunks."""
        pos, rows, vals = [], [], []
        runs = []                                   # (first row in the step, length, keys up to the run's end, item)
        t0 = 0
        for i, (it, r) in enumerate(zip(items, reqs)):
            n = 1 if it.mode == "decode" else it.q_len
            a = it.kv_before
            if r.soft_rows is not None and it.mode != "decode":
                for j, p in enumerate(r.soft_rows):
                    if a <= p < a + n:
                        rows.append(t0 + p - a)
                        vals.append(r.soft_vals[j])
                for s0, s1 in r.bidir_spans or []:
                    if a <= s0 and s1 <= a + n:
                        runs.append((t0 + s0 - a, s1 - s0, s1 - r.kv_removed, i))
            if r.pos3 is not None and it.mode != "decode":
                pos.append(r.pos3[:, a:a + n])
            else:
                pos.append((torch.arange(a, a + n) + r.rope_delta)[None].expand(3, n))
            t0 += n
        if any(r.pos3 is not None for r in reqs):
            batch.pos3 = torch.cat(pos, 1).to(self.device)
        if rows:
            batch.embed_rows = torch.tensor(rows, dtype=torch.int64, device=self.device)
            batch.embed_vals = torch.stack(vals)
        if runs:
            i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=self.device)
            which = torch.tensor([u[3] for u in runs], dtype=torch.int64, device=self.device)
            row_idx = torch.cat([torch.arange(u[0], u[0] + u[1]) for u in runs]).to(self.device)
            batch.bidir = (i32([u[0] for u in runs]), i32([u[1] for u in runs]), i32([u[2] for u in runs]),
                           batch.block_tables.index_select(0, which).contiguous(), max(u[1] for u in runs), row_idx)

    def _pick_tokens(self, logits: torch.Tensor, reqs: List[Request]) -> torch.Tensor:
        if any(r.params.grammar is not None for r in reqs):
            # Grammar-constrained rows: every token the grammar cannot continue with goes to -inf.  The masks are
            # computed on the host (C++ recogniser stepped over the vocabulary) and applied on the device.
            V = logits.shape[-1]
            m = np.ones((len(reqs), V), dtype=np.uint8)
            for i, r in enumerate(reqs):
                if r.params.grammar is not None:
                    gm = r.params.grammar.mask()
                    m[i, : min(V, gm.shape[0])] = gm[:V]
                    m[i, gm.shape[0]:] = 0
            md = torch.from_numpy(m).to(logits.device, non_blocking=True).bool()
            self.h2d_bytes += m.nbytes
            logits = logits.float().masked_fill(~md, float("-inf"))
        if all(r.params.greedy and not r.params.needs_penalties for r in reqs):
            return self.model.greedy_tokens(logits)
        lg = logits
        dev = logits.device
        if any(r.params.needs_penalties for r in reqs):
            rows = torch.tensor([max(r.row, 0) for r in reqs], device=dev)
            cnt = self.counts.index_select(0, rows) if self.counts is not None else None
            f = lambda key: torch.tensor([getattr(r.params, key) for r in reqs], dtype=torch.float32, device=dev)
            lg = S.penalties(logits, cnt, f("repetition_penalty"), f("frequency_penalty"), f("presence_penalty"))
        else:
            lg = logits.float()
        f = lambda key, dt: torch.tensor([getattr(r.params, key) for r in reqs], dtype=dt, device=dev)
        seeds = [r.params.seed for r in reqs]
        if any(s is not None for s in seeds):
            self._gen.manual_seed(int(sum((s or 0) * (i + 1) for i, s in enumerate(seeds)) + self.steps))
        u = torch.rand(len(reqs), device=dev, generator=self._gen)
        return S.sample(lg.contiguous(), f("temperature", torch.float32), f("top_k", torch.int32),
                        f("top_p", torch.float32), f("min_p", torch.float32), u)

    def _accept(self, r: Request, tok: int, now: float) -> bool:
        """Append one sampled token; returns True when the request is finished."""
        r.out.append(tok)
        if r.params.grammar is not None:
            r.params.grammar.accept(tok)
        if r.t_first is None:
            r.t_first = now
        if r.row >= 0:
            S.count_tokens(self.counts, torch.tensor([tok], dtype=torch.int32, device=self.device),
                           torch.tensor([r.row], dtype=torch.int32, device=self.device))
        if not r.params.ignore_eos and (tok == self.eos or tok in r.params.stop_token_ids):
            self._retire(r, "stop")
            return True
        if len(r.out) >= r.params.max_tokens:
            self._retire(r, "length")
            return True
        return False

    # ------------------------------------------------------------------------------------------------
    def _decode_static(self, items: List[StepItem]) -> Optional[torch.Tensor]:
        """Steady-state decode through static buffers and a captured graph.  Returns sampled tokens (device)."""
        B = len(items)
        reqs = [self.reqs[it.request_id] for it in items]
        max_kv = max(it.kv_before for it in items) + 1
        splits = self._attn_splits(B, max_kv)
        # The split count is baked into the graph; bucket it by the context length so a graph is reused.
        key = (B, splits)
        st = self._static.get(key)
        if st is None:
            st = _StaticStep(B, self.max_blocks, self.device)
            self._static[key] = st
        seqs = np.array([it.request_id for it in items], dtype=np.int64)
        ones = np.ones(B, dtype=np.int32)
        tab_np = st.h_tab.numpy()
        slots, lens = self.cache.alloc.append_batch(seqs, ones, self.max_blocks, tab_np)
        st.h_slots.numpy()[:] = slots
        st.h_kvl.numpy()[:] = lens
        st.h_pos.numpy()[:] = lens - 1 + np.array([r.kv_removed for r in reqs], dtype=np.int32)
        st.h_ids.numpy()[:] = [r.out[-1] if r.out else r.prompt[-1] for r in reqs]
        st.dev.copy_(st.host, non_blocking=True)
        self.h2d_bytes += st.h2d_bytes()
        scratch = self._scratch_for(B, splits)
        batch = StepBatch(st.ids, st.pos, st.slots, st.qs, st.ql, st.kvl, st.tab, st.qs, 1, splits)

        def run():
            logits = self.model.forward(batch, self.cache.k, self.cache.v, scratch)
            st.logits = logits
            st.out_tokens = self.model.greedy_tokens(logits)

        greedy = all(r.params.greedy and not r.params.needs_penalties and r.params.grammar is None for r in reqs)
        if self.use_graph and greedy:
            if st.graph is None:
                from .. import _native as N

                run()  # warm-up: configures kernel attributes outside the capture
                torch.cuda.synchronize()
                n0 = N.launches()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    run()
                st.launches = N.launches() - n0
                st.graph = g
                self._after_capture()
                # The warm-up and capture passes rewrote the same KV slots with the same values; replay for real.
            st.graph.replay()
            from .. import _native as N

            N.count_launch(st.launches)
            return st.out_tokens
        logits = self.model.forward(batch, self.cache.k, self.cache.v, scratch)
        return self._pick_tokens(logits, reqs)

    def step(self) -> int:
        """Run one scheduler step.  Returns the number of tokens produced."""
        if self.draft is not None and not any(r.params.grammar is not None and not r.finished
                                              for r in self.reqs.values()):
            snap = self.sched.snapshot()
            if snap["decode"] > 0 and snap["waiting"] + snap["prefill"] == 0 and not any(
                    r.soft_rows is not None for r in self.reqs.values()):
                return self._spec_round()
        items = self.sched.claim_step()
        if not items:
            return 0
        t_start = time.perf_counter()
        reqs = [self.reqs[it.request_id] for it in items]
        try:
            multimodal = any(r.soft_rows is not None for r in reqs)
            if all(it.mode == "decode" and it.q_len == 1 for it in items) and self.device.type == "cuda" \
                    and not multimodal:
                toks_dev = self._decode_static(items)
                producing = list(range(len(items)))
            else:
                seq_tokens = []
                for it, r in zip(items, reqs):
                    if it.mode == "decode":
                        seq_tokens.append([r.out[-1]])
                    else:
                        seq_tokens.append(r.prompt[it.kv_before: it.kv_before + it.q_len])
                batch = self._build_batch(items, seq_tokens)
                if multimodal:
                    self._add_multimodal(batch, items, reqs)
                scratch = self._scratch_for(batch.ids.numel(), batch.attn_splits)
                producing = [i for i, (it, r) in enumerate(zip(items, reqs))
                             if it.mode == "decode" or it.kv_before + it.q_len >= len(r.prompt)]
                if producing:
                    batch.logit_rows = batch.logit_rows[torch.tensor(producing, device=self.device)] \
                        if len(producing) != len(items) else batch.logit_rows
                    logits = self.model.forward(batch, self.cache.k, self.cache.v, scratch)
                    toks_dev = self._pick_tokens(logits, [reqs[i] for i in producing])
                else:
                    batch.logit_rows = batch.logit_rows[:1]
                    self.model.forward(batch, self.cache.k, self.cache.v, scratch)
                    toks_dev = None
        except KvOutOfBlocks:
            self.sched.fail_step()
            # Slots reserved for the items packed before the one that failed go back to the pool.
            for it in items:
                if self.cache.alloc.length(it.request_id) > it.kv_before:
                    self.cache.alloc.truncate(it.request_id, it.kv_before)
            # Cached prefixes are the first thing to give up under memory pressure: drop one and retry the step.
            if self.prefix is not None and self.prefix.evict_one():
                return 0
            raise
        for it, r in zip(items, reqs):
            if it.mode != "decode" and it.kv_before + it.q_len >= len(r.prompt):
                ratio = r.params.cache_compaction_ratio
                if ratio is not None and 0.0 < ratio < 1.0:
                    self.compact_request(it.request_id, ratio)
                elif self.prefix is not None and r.soft_rows is None:
                    self.prefix.insert(it.request_id, r.prompt)
        toks = toks_dev.cpu().tolist() if toks_dev is not None else []
        self.d2h_bytes += 4 * len(toks)
        now = time.perf_counter()
        tokens_out = [0] * len(items)
        finished = [False] * len(items)
        for j, i in enumerate(producing):
            tokens_out[i] = 1
            finished[i] = self._accept(reqs[i], int(toks[j]), now)
        self.sched.complete_step(items, tokens_out, finished)
        self.steps += 1
        dt = time.perf_counter() - t_start
        self.timing["decode_s" if all(it.mode == "decode" for it in items) else "prefill_s"] += dt
        return len(producing)

    # ------------------------------------------------------------------------------------------------
    def compact_request(self, rid: int, ratio: float, n_ref: int = 64, keep_recent: int = 16) -> int:
        """Attention-matching compaction of one sequence's KV cache (all layers, every KV head) to about ``ratio``
        of its tokens (plain bf16 / f32 caches only); the sequence moves to fresh blocks (its old ones may be
        shared with cached prefixes) and the freed blocks return to the pool.  Returns the number of tokens removed.  Not combined with
        speculative decoding."""
        from .kv_compaction import compact_layer

        if self.draft is not None:
            raise ValueError("KV compaction cannot be combined with speculative decoding")
        if self.cache.codec is not None:
            raise ValueError(f"KV compaction needs a plain cache; this engine keeps its cache as {self.cache.codec}")
        r = self.reqs[rid]
        alloc, page = self.cache.alloc, self.page
        N = alloc.length(rid)
        if N < 4 * page:
            return 0
        table = torch.from_numpy(alloc.block_table(rid).astype(np.int64)).to(self.device)
        slots = (table[:, None] * page + torch.arange(page, device=self.device)[None]).reshape(-1)[:N]
        L = self.cache.k.shape[0]
        Hkv, D = self.cache.k.shape[3], self.cache.k.shape[4]
        new_k, new_v = [], []
        for l in range(L):
            K = self.cache.k[l].view(-1, Hkv, D).index_select(0, slots)
            V = self.cache.v[l].view(-1, Hkv, D).index_select(0, slots)
            kh, vh = compact_layer(K, V, ratio, n_ref, keep_recent)
            new_k.append(kh)
            new_v.append(vh)
        M = new_k[0].shape[0]
        alloc.detach(rid)
        alloc.attach(rid)
        dst = torch.from_numpy(alloc.append(rid, M).astype(np.int64)).to(self.device)
        for l in range(L):
            self.cache.k[l].view(-1, Hkv, D)[dst] = new_k[l].to(self.cache.k.dtype)
            self.cache.v[l].view(-1, Hkv, D)[dst] = new_v[l].to(self.cache.v.dtype)
        r.kv_removed += N - M
        return N - M

    # ------------------------------------------------------------------------------------------------
    def _spec_round(self) -> int:
        """One speculative round for every decoding sequence: K greedy draft steps on the shallow model (which
        shares the target's first layers and their KV cache), one target pass over K+1 positions, verify/accept,
        KV rollback of the rejected tail."""
        items = self.sched.claim_step()
        if not items:
            return 0
        reqs = [self.reqs[it.request_id] for it in items]
        # Draft length of the round: the smallest of what the requests ask for (default: the engine's), 1..16.
        K = max(1, min(16, min((r.params.speculative_k or self.spec_k) for r in reqs)))
        B = len(items)
        alloc = self.cache.alloc
        separate = self.draft_cache is not None
        if separate:
            self._draft_catch_up(items, reqs)
        # Reserve K+1 slots per sequence up front; the draft fills the first K progressively.
        base_len = [it.kv_before for it in items]
        all_slots, tables = [], np.zeros((B, self.max_blocks), dtype=np.int32)
        for i, it in enumerate(items):
            all_slots.append(alloc.append(it.request_id, K + 1))
            bt = alloc.block_table(it.request_id)
            tables[i, : len(bt)] = bt
        d_tab = torch.from_numpy(tables).to(self.device)
        self.h2d_bytes += tables.nbytes
        last = torch.tensor([r.out[-1] for r in reqs], dtype=torch.int32, device=self.device)
        ar = torch.arange(B, dtype=torch.int32, device=self.device)
        ones = torch.ones(B, dtype=torch.int32, device=self.device)
        base = torch.tensor(base_len, dtype=torch.int32, device=self.device)
        slots_t = torch.from_numpy(np.stack(all_slots)).to(self.device)  # [B, K+1]
        drafts = []
        cur = last
        splits = self._attn_splits(B, max(base_len) + K + 1)
        scratch = self._scratch_for(B * (K + 1), splits)
        if separate:
            # The draft model writes K entries (last, d0 .. d_{K-2}) into ITS cache through ITS block tables.
            dalloc = self.draft_cache.alloc
            dtab_np = np.zeros((B, self.max_blocks), dtype=np.int32)
            dslots = []
            for i, it in enumerate(items):
                dslots.append(dalloc.append(it.request_id, K))
                bt = dalloc.block_table(it.request_id)
                dtab_np[i, : len(bt)] = bt
            dk, dv = self.draft_cache.k, self.draft_cache.v
            draft_tab = torch.from_numpy(dtab_np).to(self.device)
            draft_slots = torch.from_numpy(np.stack(dslots)).to(self.device)  # [B, K]
            self.h2d_bytes += dtab_np.nbytes
        else:
            dk, dv, draft_tab, draft_slots = self.cache.k, self.cache.v, d_tab, slots_t
        for j in range(K):
            b = StepBatch(cur, base + j, draft_slots[:, j].contiguous(), ar, ones, base + j + 1, draft_tab, ar, 1,
                          splits)
            lg = self.draft.forward(b, dk, dv, scratch)
            cur = self.draft.greedy_tokens(lg)
            drafts.append(cur)
        draft = torch.stack(drafts, 1).contiguous()  # [B, K]
        # Target verifies [last, d0..d_{K-1}] in one pass.
        ver_ids = torch.cat([last[:, None], draft], 1).reshape(-1).contiguous()
        pos = (base[:, None] + torch.arange(K + 1, dtype=torch.int32, device=self.device)[None]).reshape(-1)
        G = self.model.Hq // self.model.Hkv
        vb = StepBatch(ver_ids, pos.contiguous(), slots_t.reshape(-1).contiguous(), ar * (K + 1),
                       ones * (K + 1), base + K + 1, d_tab,
                       torch.arange(B * (K + 1), dtype=torch.int32, device=self.device), K + 1,
                       splits if (K + 1) * G <= 16 else 1, max_kv=max(base_len) + K + 1)
        logits = self.model.forward(vb, self.cache.k, self.cache.v, scratch)
        if all(r.params.greedy and not r.params.needs_penalties for r in reqs):
            target = self.model.greedy_tokens(logits)
        else:
            rep = [r for r in reqs for _ in range(K + 1)]
            target = self._pick_tokens(logits, rep)
        n_m, nxt = S.spec_verify(draft, target.view(B, K + 1).contiguous())
        res = torch.stack([n_m, nxt], 1).cpu().tolist()
        dr = draft.cpu().tolist()
        self.d2h_bytes += 8 * B + 4 * B * K
        now = time.perf_counter()
        produced = 0
        tokens_out, finished = [0] * B, [False] * B
        self.spec.rounds += 1
        for i, (it, r) in enumerate(zip(items, reqs)):
            m, nx = res[i]
            self.spec.drafted += K
            self.spec.matched += m
            self.spec.rejected += K - m
            if m == K:
                self.spec.bonus += 1
            else:
                self.spec.corrections += 1
            new = dr[i][:m] + [nx]
            done = False
            n_added = 0
            for t in new:
                n_added += 1
                if self._accept(r, int(t), now):
                    done = True
                    break
            self.spec.accepted += n_added
            produced += n_added
            tokens_out[i], finished[i] = n_added, done
            if not done:
                # KV holds last + the m matched drafts; the correction/bonus token enters the cache next round.
                alloc.truncate(it.request_id, base_len[i] + n_added)
                if separate:
                    # The draft wrote last, d0 .. d_{K-2}: keep last + the matched drafts it has seen.  When all K
                    # matched it is one entry short (d_{K-1}); the next round's catch-up feeds it.
                    self.draft_cache.alloc.truncate(it.request_id, base_len[i] + min(n_added, K))
        self.sched.complete_step(items, tokens_out, finished)
        self.steps += 1
        return produced

    def _draft_catch_up(self, items: List[StepItem], reqs: List[Request]) -> None:
        """Brings the separate draft model's KV cache up to the target's: every token of a sequence except the one
        about to be fed (prompt on the first round, tokens produced by non-speculative steps, the last matched
        draft after a fully accepted round) runs through the draft model as a prefill chunk."""
        dalloc = self.draft_cache.alloc
        chunk = 2048
        while True:
            rows, seqs = [], []
            budget = chunk
            for it, r in zip(items, reqs):
                if not r.draft_attached:
                    dalloc.attach(r.rid)
                    r.draft_attached = True
                have, want = dalloc.length(r.rid), it.kv_before
                if have > want:            # the target rolled back further than the draft (never with equal K)
                    dalloc.truncate(r.rid, want)
                    have = want
                if have < want and budget > 0:
                    n = min(want - have, budget)
                    budget -= n
                    rows.append((r.rid, have, n))
                    seqs.append(r.tokens[have: have + n])
            if not rows:
                return
            B = len(rows)
            ids, pos, slots, qs, ql, kvl, last_rows = [], [], [], [], [], [], []
            tables = np.zeros((B, self.max_blocks), dtype=np.int32)
            t0 = 0
            for i, ((rid, have, n), toks) in enumerate(zip(rows, seqs)):
                sl = dalloc.append(rid, n)
                ids.extend(toks); pos.extend(range(have, have + n)); slots.extend(sl.tolist())
                qs.append(t0); ql.append(n); kvl.append(have + n); last_rows.append(t0 + n - 1)
                bt = dalloc.block_table(rid)
                tables[i, : len(bt)] = bt
                t0 += n
            dev = self.device
            ti = lambda a: torch.tensor(a, dtype=torch.int32, device=dev)
            self.h2d_bytes += 4 * (3 * t0 + 4 * B) + tables.nbytes
            b = StepBatch(ti(ids), ti(pos), ti(slots), ti(qs), ti(ql), ti(kvl), torch.from_numpy(tables).to(dev),
                          ti(last_rows[:1]), max(ql), 1)
            self.draft.forward(b, self.draft_cache.k, self.draft_cache.v, None)

    # ------------------------------------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], params, on_token: Optional[Callable] = None,
                 soft: Optional[Sequence[Optional[dict]]] = None) -> List[GenerationResult]:
        """Run prompts to completion.  ``params`` is one SamplingParams or one per prompt; ``soft`` holds, per
        prompt, the multimodal description :meth:`add_request` takes (or None)."""
        plist = params if isinstance(params, (list, tuple)) else [params] * len(prompts)
        slist = list(soft) if soft is not None else [None] * len(prompts)
        rids = [self.add_request(p, sp, sf) for p, sp, sf in zip(prompts, plist, slist)]
        emitted = {rid: 0 for rid in rids}
        while any(not self.reqs[rid].finished for rid in rids):
            n = self.step()
            if on_token is not None:
                for rid in rids:
                    r = self.reqs[rid]
                    while emitted[rid] < len(r.out):
                        on_token(rid, r.out[emitted[rid]])
                        emitted[rid] += 1
            if n == 0 and not self.has_work():
                break
        out = []
        for rid in rids:
            r = self.reqs.pop(rid)
            out.append(GenerationResult(r.out, r.finish_reason or "length", len(r.prompt),
                                        (r.t_first - r.t_admit) if r.t_first else 0.0))
        return out


def decode_burst(engine: "LLMEngine", n_steps: int):
    """Run ``n_steps`` greedy decode steps for every sequence that is currently decoding without a host round
    trip per step: KV slots for all steps are reserved up front, the per-step integer inputs are staged on the
    device once, each step is a device-to-device refresh of the static buffers plus one graph replay, and the
    sampled tokens of all steps come back in a single read at the end.  Stop conditions are applied afterwards
    (tokens past a stop are dropped and their KV released).  Returns (tokens [n_steps, B] on the host, device
    milliseconds measured with CUDA events, kernel launches)."""
    from .. import _native as N

    items = engine.sched.claim_step()
    assert items and all(it.mode == "decode" and it.q_len == 1 for it in items), "burst needs a pure decode batch"
    reqs = [engine.reqs[it.request_id] for it in items]
    B = len(items)
    alloc = engine.cache.alloc
    base = np.array([it.kv_before for it in items], dtype=np.int32)
    max_kv = int(base.max()) + n_steps
    splits = engine._attn_splits(B, max_kv)
    key = (B, splits)
    st = engine._static.get(key)
    if st is None:
        st = _StaticStep(B, engine.max_blocks, engine.device)
        engine._static[key] = st
    slots = np.stack([alloc.append(it.request_id, n_steps) for it in items], 1)  # [n_steps, B]
    for i, it in enumerate(items):
        bt = alloc.block_table(it.request_id)
        st.h_tab.numpy()[i, : len(bt)] = bt
    st.h_ids.numpy()[:] = [r.out[-1] if r.out else r.prompt[-1] for r in reqs]
    st.h_slots.numpy()[:] = slots[0]
    st.h_pos.numpy()[:] = base
    removed = np.array([r.kv_removed for r in reqs], dtype=np.int32)
    st.h_kvl.numpy()[:] = base + 1 - removed
    st.dev.copy_(st.host, non_blocking=True)
    steps = np.arange(n_steps, dtype=np.int32)[:, None]
    per_step = np.stack([base[None] + steps, slots, ], 1)  # [n_steps, 2, B]: positions, slots
    per_step_dev = torch.from_numpy(per_step.astype(np.int32)).pin_memory().to(engine.device, non_blocking=True)
    kvl_dev = torch.from_numpy((base[None] + steps + 1 - removed[None]).astype(np.int32)).pin_memory().to(engine.device,
                                                                                         non_blocking=True)
    engine.h2d_bytes += st.h2d_bytes() + per_step.nbytes + kvl_dev.numel() * 4
    scratch = engine._scratch_for(B, splits)
    batch = StepBatch(st.ids, st.pos, st.slots, st.qs, st.ql, st.kvl, st.tab, st.qs, 1, splits)

    def run():
        logits = engine.model.forward(batch, engine.cache.k, engine.cache.v, scratch)
        st.out_tokens = engine.model.greedy_tokens(logits)

    if st.graph is None:
        run()
        torch.cuda.synchronize()
        n0 = N.launches()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            run()
        st.launches = N.launches() - n0
        st.graph = g
        engine._after_capture()
    out = torch.empty((n_steps, B), dtype=torch.int32, device=engine.device)
    assert st.pos.data_ptr() + 4 * B == st.slots.data_ptr()
    ps_view = st.dev[B:3 * B]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    n0 = N.launches()
    e0.record()
    for i in range(n_steps):
        if i > 0:
            st.ids.copy_(st.out_tokens)
            ps_view.copy_(per_step_dev[i].reshape(-1))
            st.kvl.copy_(kvl_dev[i])
        st.graph.replay()
        N.count_launch(st.launches)
        out[i].copy_(st.out_tokens)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    launches = N.launches() - n0
    host = out.cpu()
    engine.d2h_bytes += host.numel() * 4
    now = time.perf_counter()
    tokens_out, finished = [0] * B, [False] * B
    toks = host.tolist()
    for i, (it, r) in enumerate(zip(items, reqs)):
        n_added, done = 0, False
        for s in range(n_steps):
            n_added += 1
            if engine._accept(r, int(toks[s][i]), now):
                done = True
                break
        tokens_out[i], finished[i] = n_added, done
        if not done and n_added < n_steps:
            alloc.truncate(it.request_id, int(base[i]) + n_added)
    engine.sched.complete_step(items, tokens_out, finished)
    engine.steps += n_steps
    return host, ms, launches
