"""Training objectives: chunked next-token cross-entropy, sequence log-probabilities, DPO, GRPO, InfoNCE, reranker
losses.

The reference's set (zig/pkg/inference/docs/finetuning/FINETUNING.md "Loss Functions", "Unified Recipes": SFT with
chunked cross-entropy so that the [tokens, vocabulary] logits never exist at once, preference (DPO with ``beta``),
GRPO with group-normalised advantages, a clipped ratio and a KL term, contrastive InfoNCE with in-batch negatives,
pointwise / pairwise reranker losses).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint


def chunked_token_logps(net, hidden: torch.Tensor, targets: torch.Tensor, chunk: int = 1024) -> torch.Tensor:
    """log p(targets[t] | ...) for every position, computing the vocabulary projection ``chunk`` positions at a time
    (each chunk's logits are recomputed in the backward pass instead of being kept).  hidden [N, H], targets [N]
    (entries < 0 are ignored and come back as 0)."""
    out = []
    safe = targets.clamp_min(0)

    def piece(h, t):
        return torch.log_softmax(net.logits(h), -1).gather(-1, t[:, None])[:, 0]

    for i in range(0, hidden.shape[0], chunk):
        h, t = hidden[i:i + chunk], safe[i:i + chunk]
        if torch.is_grad_enabled() and hidden.requires_grad:
            out.append(checkpoint(piece, h, t, use_reentrant=False))
        else:
            out.append(piece(h, t))
    lp = torch.cat(out) if out else hidden.new_zeros(0)
    return lp * (targets >= 0)


def causal_lm_loss(net, hidden: torch.Tensor, ids: torch.Tensor, loss_mask: torch.Tensor,
                   doc_ids: Optional[torch.Tensor] = None, chunk: int = 1024) -> Tuple[torch.Tensor, int]:
    """Mean next-token cross-entropy over positions whose *target* token has ``loss_mask`` set.  hidden [B, S, H],
    ids / loss_mask [B, S].  With packing, the last token of a document does not predict the next document's first."""
    tgt = ids[:, 1:].clone()
    keep = loss_mask[:, 1:].bool()
    if doc_ids is not None:
        keep = keep & (doc_ids[:, 1:] == doc_ids[:, :-1])
    tgt[~keep] = -1
    lp = chunked_token_logps(net, hidden[:, :-1].reshape(-1, hidden.shape[-1]), tgt.reshape(-1), chunk)
    n = int(keep.sum())
    return -lp.sum() / max(n, 1), n


def sequence_logps(net, hidden, ids, loss_mask, chunk: int = 1024) -> torch.Tensor:
    """Sum of target log-probabilities per row -> [B]."""
    tgt = ids[:, 1:].clone()
    tgt[~loss_mask[:, 1:].bool()] = -1
    lp = chunked_token_logps(net, hidden[:, :-1].reshape(-1, hidden.shape[-1]), tgt.reshape(-1), chunk)
    return lp.view(ids.shape[0], -1).sum(1)


def dpo_loss(policy_chosen, policy_rejected, ref_chosen, ref_rejected, beta: float = 0.1):
    """-log sigmoid(beta * ((pi_c - pi_r) - (ref_c - ref_r))); also returns the mean reward margin and accuracy."""
    margin = (policy_chosen - policy_rejected) - (ref_chosen - ref_rejected)
    loss = -F.logsigmoid(beta * margin).mean()
    m = margin.detach()
    return loss, {"reward_margin": float((beta * m).mean()), "accuracy": float((m > 0).float().mean())}


def grpo_advantages(rewards: torch.Tensor, group_size: int, normalize: bool = True) -> torch.Tensor:
    """rewards [P * G] (G completions per prompt, grouped) -> reward minus its group's mean, divided by the group's
    standard deviation when ``normalize``."""
    r = rewards.view(-1, group_size)
    adv = r - r.mean(1, keepdim=True)
    if normalize:
        adv = adv / (r.std(1, keepdim=True, unbiased=False) + 1e-6)
    return adv.reshape(-1)


def grpo_loss(new_logps, old_logps, ref_logps, advantages, token_mask, clip_epsilon: float = 0.2,
              kl_coef: float = 0.04):
    """Token-level clipped surrogate with a KL penalty towards the reference policy.  new / old / ref log-probs and
    token_mask are [N, T]; advantages [N] (one per completion)."""
    m = token_mask.float()
    ratio = torch.exp(new_logps - old_logps)
    adv = advantages[:, None]
    surrogate = torch.minimum(ratio * adv, ratio.clamp(1 - clip_epsilon, 1 + clip_epsilon) * adv)
    d = ref_logps - new_logps
    kl = torch.exp(d) - d - 1.0                                          # non-negative estimator of KL(new || ref)
    per_tok = -(surrogate - kl_coef * kl) * m
    per_seq = per_tok.sum(1) / m.sum(1).clamp_min(1.0)
    return per_seq.mean(), {"kl": float((kl * m).sum() / m.sum().clamp_min(1.0)),
                            "clip_fraction": float((((ratio - 1).abs() > clip_epsilon).float() * m).sum()
                                                   / m.sum().clamp_min(1.0))}


def info_nce(query: torch.Tensor, positive: torch.Tensor, negatives: Optional[torch.Tensor] = None,
             temperature: float = 0.05, bank: Optional[torch.Tensor] = None,
             bank_exclude: Optional[torch.Tensor] = None):
    """Contrastive loss with in-batch negatives: row i's positive is positive[i]; every other positive, the optional
    hard negatives [B, N, D] and a bank of earlier embeddings [M, D] (a cross-batch memory) are negatives, except
    the bank entries marked in ``bank_exclude`` [B, M] (an earlier embedding of the row's own positive must not
    count against it).  Inputs are L2-normalised vectors."""
    cands = positive
    n_bank = 0
    if bank is not None and bank.numel():
        cands = torch.cat([cands, bank.to(cands.dtype)], 0)
        n_bank = bank.shape[0]
    logits = query @ cands.t() / temperature
    if n_bank and bank_exclude is not None:
        pad = torch.zeros(query.shape[0], positive.shape[0], dtype=torch.bool, device=query.device)
        logits = logits.masked_fill(torch.cat([pad, bank_exclude], 1), float("-inf"))
    if negatives is not None:
        hard = torch.einsum("bd,bnd->bn", query, negatives) / temperature
        logits = torch.cat([logits, hard], 1)
    target = torch.arange(query.shape[0], device=query.device)
    return F.cross_entropy(logits, target), {"accuracy": float((logits.argmax(1) == target).float().mean())}


def reranker_loss(scores: torch.Tensor, labels: torch.Tensor, groups: Optional[torch.Tensor] = None, mode: str = "bce"):
    """scores [N] (one logit per query-document pair), labels [N] in [0, 1].  ``bce``: pointwise.  ``pairwise``:
    within each group (same query), -log sigmoid(s_pos - s_neg) over every (positive, negative) pair."""
    if mode == "bce":
        return F.binary_cross_entropy_with_logits(scores, labels.float())
    if mode != "pairwise":
        raise ValueError(f"unknown reranker loss {mode!r}")
    if groups is None:
        groups = torch.zeros_like(labels, dtype=torch.long)
    same = groups[:, None] == groups[None, :]
    pairs = same & (labels[:, None] > 0.5) & (labels[None, :] <= 0.5)
    if not bool(pairs.any()):
        return scores.sum() * 0.0
    diff = scores[:, None] - scores[None, :]
    return -(F.logsigmoid(diff) * pairs).sum() / pairs.sum()
