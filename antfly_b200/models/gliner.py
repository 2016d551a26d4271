"""GLiNER: zero-shot span extraction.  A DeBERTa encoder reads ``( [P] entities ( [E] label ... ) ) [SEP_TEXT] words``
and a small head scores every (word span, label) pair.

Head (weight names as in the checkpoints, zig/pkg/inference/src/architectures/gliner_head.zig:165-1178):

* word vectors: the hidden state of each word's first sub-token;
* span vectors: ``out_project(relu([project_start(w[start]) ; project_end(w[end])]))`` where the three projections
  are two-layer ReLU MLPs (``span_rep.span_rep_layer.*``), for every start word and every width up to ``max_width``;
* label vectors: the hidden state at each label marker ``h`` goes through one GRU step whose input is a learned
  position vector and whose state is ``h`` (``count_embed.gru``), a residual, a 128-wide two-layer post-norm
  transformer over the labels (``count_embed.transformer``), and a three-layer MLP on ``[transformer ; residual]``;
* logits: ``span_vectors @ label_vectors.T``.

The encoder layers and every MLP run on the bf16 GEMM with bias / ReLU epilogues; gathers, the GRU gate arithmetic
and the four-head attention over a handful of labels are tensor arithmetic.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Sequence, Tuple

import torch

from ..ops import dense as Dn
from .bert import pack_sequences
from .deberta import DebertaConfig, DebertaModel

HEAD_PREFIXES = ("span_rep.", "count_embed.")


@dataclass
class GlinerInput:
    ids: List[int]            # schema tokens, then the words' sub-tokens
    words_mask: List[int]     # 0 for schema tokens, 1-based word number for text tokens
    num_words: int


class GlinerModel:
    def __init__(self, encoder: DebertaModel, weights: Dict[str, torch.Tensor], label_heads: int = 4):
        self.encoder, self.w, self.label_heads = encoder, weights, label_heads
        self.device = weights["span_rep.span_rep_layer.out_project.0.weight"].device
        self.hidden = weights["span_rep.span_rep_layer.out_project.3.weight"].shape[0]
        self.label_layers = 1 + max(int(k.split(".")[4]) for k in weights
                                    if k.startswith("count_embed.transformer.transformer.layers."))

    @classmethod
    def from_state_dict(cls, cfg: DebertaConfig, sd: Dict[str, torch.Tensor], device="cuda",
                        dtype=torch.bfloat16) -> "GlinerModel":
        """Encoder tensors are stored under ``encoder.embeddings.*`` / ``encoder.encoder.*``; head tensors keep
        their names."""
        enc_sd = {k[len("encoder."):]: v for k, v in sd.items()
                  if k.startswith("encoder.embeddings.") or k.startswith("encoder.encoder.")}
        if not enc_sd:
            raise KeyError("no encoder.* tensors in the checkpoint")
        encoder = DebertaModel.from_state_dict(cfg, enc_sd, device=device, dtype=dtype)
        w = {k: v.to(dtype).to(device).contiguous() for k, v in sd.items() if k.startswith(HEAD_PREFIXES)}
        return cls(encoder, w)

    # -- head pieces ---------------------------------------------------------------------------------------
    def _mlp2(self, x: torch.Tensor, prefix: str) -> torch.Tensor:
        w = self.w
        h = Dn.gemm_bf16(x, w[prefix + ".0.weight"], bias=w[prefix + ".0.bias"], act="relu")
        return Dn.gemm_bf16(h, w[prefix + ".3.weight"], bias=w[prefix + ".3.bias"])

    def span_vectors(self, words: torch.Tensor, starts: torch.Tensor, ends: torch.Tensor) -> torch.Tensor:
        """Word vectors [W, H] and span endpoints (word indices, [S]) -> span vectors [S, H]."""
        p = "span_rep.span_rep_layer."
        a = self._mlp2(words, p + "project_start").index_select(0, starts)
        b = self._mlp2(words, p + "project_end").index_select(0, ends)
        cat = torch.relu(torch.cat([a, b], -1)).contiguous()
        return self._mlp2(cat, p + "out_project")

    def label_vectors(self, h: torch.Tensor) -> torch.Tensor:
        """Label marker states [N, H] -> label vectors [N, H]."""
        w = self.w
        N, H = h.shape
        dt = h.dtype
        x = w["count_embed.pos_embedding.weight"][:1].expand(N, H).contiguous()
        gi = Dn.gemm_bf16(x, w["count_embed.gru.weight_ih_l0"], bias=w["count_embed.gru.bias_ih_l0"],
                          out_dtype=torch.float32).float()
        gh = Dn.gemm_bf16(h, w["count_embed.gru.weight_hh_l0"], bias=w["count_embed.gru.bias_hh_l0"],
                          out_dtype=torch.float32).float()
        r = torch.sigmoid(gi[:, :H] + gh[:, :H])
        z = torch.sigmoid(gi[:, H:2 * H] + gh[:, H:2 * H])
        n = torch.tanh(gi[:, 2 * H:] + r * gh[:, 2 * H:])
        hf = h.float()
        combined = ((1 - z) * n + z * hf + hf).to(dt).contiguous()          # GRU state plus the residual
        t = "count_embed.transformer."
        y = Dn.gemm_bf16(combined, w[t + "in_projector.weight"], bias=w[t + "in_projector.bias"])
        D = y.shape[1]
        nh = self.label_heads
        for l in range(self.label_layers):
            p = t + f"transformer.layers.{l}."
            qkv = Dn.gemm_bf16(y, w[p + "self_attn.in_proj_weight"], bias=w[p + "self_attn.in_proj_bias"],
                               out_dtype=torch.float32).float().view(N, 3, nh, D // nh)
            q, k, v = qkv[:, 0].transpose(0, 1), qkv[:, 1].transpose(0, 1), qkv[:, 2].transpose(0, 1)
            att = torch.softmax(q @ k.transpose(-1, -2) * (D // nh) ** -0.5, -1) @ v        # [nh, N, D / nh]
            ctx = att.transpose(0, 1).reshape(N, D).to(dt).contiguous()
            y = Dn.gemm_bf16(ctx, w[p + "self_attn.out_proj.weight"], bias=w[p + "self_attn.out_proj.bias"], residual=y)
            y = Dn.norm(y, w[p + "norm1.weight"], w[p + "norm1.bias"], eps=1e-5)
            f = Dn.gemm_bf16(y, w[p + "linear1.weight"], bias=w[p + "linear1.bias"], act="relu")
            y = Dn.gemm_bf16(f, w[p + "linear2.weight"], bias=w[p + "linear2.bias"], residual=y)
            y = Dn.norm(y, w[p + "norm2.weight"], w[p + "norm2.bias"], eps=1e-5)
        cat = torch.cat([y, combined], -1).contiguous()
        o = t + "out_projector."
        a = Dn.gemm_bf16(cat, w[o + "0.weight"], bias=w[o + "0.bias"], act="relu")
        a = Dn.gemm_bf16(a, w[o + "2.weight"], bias=w[o + "2.bias"], act="relu")
        return Dn.gemm_bf16(a, w[o + "4.weight"], bias=w[o + "4.bias"])

    # -- full forward --------------------------------------------------------------------------------------
    def span_logits(self, inputs: Sequence[GlinerInput], marker_ids: Sequence[int],
                    max_width: int) -> List[torch.Tensor]:
        """One fp32 tensor [num_words, max_width, num_labels] per input; spans that run past the last word hold
        the score of the (0, 0) span and are ignored by decoders."""
        if not inputs:
            return []
        dev = self.device
        b = pack_sequences([x.ids for x in inputs]).to(dev)
        hidden = self.encoder.encode(b)                                     # [T, H] packed
        markers = set(int(m) for m in marker_ids if m)
        out: List[torch.Tensor] = []
        word_rows: List[int] = []
        span_s: List[int] = []
        span_e: List[int] = []
        label_rows: List[int] = []
        shapes: List[Tuple[int, int, int, int]] = []                        # (words, labels, span offset, label offset)
        for x, st in zip(inputs, b.starts.tolist()):
            first = {}
            for t, wid in enumerate(x.words_mask):
                if wid > 0 and wid not in first:
                    first[wid] = st + t
            base = len(word_rows)
            nw = x.num_words
            word_rows += [first.get(i + 1, st) for i in range(nw)]
            lab = [st + t for t, tok in enumerate(x.ids) if tok in markers]
            shapes.append((nw, len(lab), len(span_s), len(label_rows)))
            label_rows += lab
            for wd in range(nw):
                for k in range(max_width):
                    ok = wd + k < nw
                    span_s.append(base + (wd if ok else 0))
                    span_e.append(base + (wd + k if ok else 0))
        if not span_s or not label_rows:
            return [torch.zeros((s[0], max_width, s[1])) for s in shapes]
        idx = lambda v: torch.tensor(v, dtype=torch.long, device=dev)
        words = hidden.index_select(0, idx(word_rows)).contiguous()
        spans = self.span_vectors(words, idx(span_s), idx(span_e))
        labels = self.label_vectors_grouped(hidden.index_select(0, idx(label_rows)).contiguous(),
                                            [s[1] for s in shapes])
        for nw, nl, so, lo in shapes:
            if nw == 0 or nl == 0:
                out.append(torch.zeros((nw, max_width, nl)))
                continue
            sv = spans[so:so + nw * max_width].contiguous()
            lg = Dn.gemm_bf16(sv, labels[lo:lo + nl].contiguous(), out_dtype=torch.float32).float()
            out.append(lg.view(nw, max_width, nl))
        return out

    def label_vectors_grouped(self, h: torch.Tensor, counts: Sequence[int]) -> torch.Tensor:
        """Label vectors for several inputs at once: the label transformer attends within one input's labels."""
        parts, o = [], 0
        for n in counts:
            if n:
                parts.append(self.label_vectors(h[o:o + n].contiguous()))
            o += n
        return torch.cat(parts, 0)
