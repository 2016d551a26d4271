"""Gated delta-rule linear attention (the recurrent layers of Qwen3.5 / Qwen3-Next decoders).

One layer keeps, per sequence, a short convolution tail and a matrix state ``S`` [value heads, key dim, value dim]
instead of a key / value cache.  For each token: Q, K, V come from one projection followed by a causal depth-wise
convolution (kernel 4) and SiLU; Q and K are L2-normalised per head; the state decays by ``exp(g)`` with
``g = -exp(A_log) * softplus(a + dt_bias)``, is corrected towards the new value by the delta rule
``S += k (x) ((v - S^T k) * beta)`` with ``beta = sigmoid(b)``, and is read with ``o = S^T q / sqrt(d_k)``; the
output is RMS-normalised per head, gated by ``SiLU(z)`` and projected back.  The reference carries the same op on
its CPU and Metal paths (zig/pkg/inference/src/architectures/gpt.zig:4462-4775).

The projections run on the bf16 GEMM.  Decode runs the recurrence one step per token over all heads at once
(state in fp32); prefill uses the chunked form (:func:`gated_delta_rule_chunked`): per 64-token chunk one
triangular solve and a handful of batched matrix products, so a prompt costs T / 64 sequential steps instead of T.
``forward`` takes and returns the state, so prefill and single-token decode share it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from ..ops import dense as Dn


@dataclass
class DeltaNetConfig:
    hidden_size: int
    linear_num_key_heads: int
    linear_num_value_heads: int
    linear_key_head_dim: int
    linear_value_head_dim: int
    linear_conv_kernel_dim: int = 4
    rms_norm_eps: float = 1e-6

    @classmethod
    def from_hf(cls, d: dict) -> "DeltaNetConfig":
        return cls(**{k: d[k] for k in cls.__dataclass_fields__ if k in d and d[k] is not None})


def gated_delta_rule(q, k, v, g, beta, state: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """q, k [T, H, Dk], v [T, H, Dv], g, beta [T, H]; state [H, Dk, Dv] or None -> (outputs [T, H, Dv] fp32, state).
    Q and K are L2-normalised here."""
    T, H, Dk = k.shape
    nrm = lambda x: x.float() * torch.rsqrt(x.float().pow(2).sum(-1, keepdim=True) + 1e-6)
    qf, kf, vf = nrm(q) * Dk ** -0.5, nrm(k), v.float()
    S = torch.zeros((H, Dk, v.shape[-1]), dtype=torch.float32, device=q.device) if state is None else state.float().clone()
    out = torch.empty((T, H, v.shape[-1]), dtype=torch.float32, device=q.device)
    decay, bt = g.float().exp(), beta.float()
    for t in range(T):
        S = S * decay[t][:, None, None]
        mem = (S * kf[t][:, :, None]).sum(1)                         # what the state already returns for this key
        S = S + kf[t][:, :, None] * ((vf[t] - mem) * bt[t][:, None])[:, None, :]
        out[t] = (S * qf[t][:, :, None]).sum(1)
    return out, S


def gated_delta_rule_chunked(q, k, v, g, beta, state: Optional[torch.Tensor] = None,
                             chunk: int = 64) -> Tuple[torch.Tensor, torch.Tensor]:
    """Same function as :func:`gated_delta_rule`, computed chunk by chunk with matrix products (prefill).

    Inside a chunk with entry state S0, write G_t for the running sum of the log decays and u_t for the vector the
    rule adds at step t (S_t = e^{G_t} S0 + sum_{i<=t} e^{G_t - G_i} k_i u_i^T).  The u_t obey a unit lower-triangular
    system (I + A) U = beta * (V - e^{G} * (K S0)) with A_ij = beta_i e^{G_i - G_j} (k_i . k_j) for j < i, so with
    T = (I + A)^-1 (one triangular solve per chunk and head, independent of S0):
        U = T (beta V) - T (beta e^{G} K) S0
        O = e^{G} (Q S0) + tril(e^{G_t - G_i} (q_t . k_i)) U
        S_end = e^{G_C} S0 + (e^{G_C - G} K)^T U
    Everything except the S0 terms is computed for all chunks at once; the loop over chunks carries only S0.
    All exponents are differences G_t - G_i with i <= t, i.e. <= 0."""
    T, H, Dk = k.shape
    Dv = v.shape[-1]
    dev = q.device
    nrm = lambda x: x.float() * torch.rsqrt(x.float().pow(2).sum(-1, keepdim=True) + 1e-6)
    qf, kf, vf = nrm(q) * Dk ** -0.5, nrm(k), v.float()
    S = torch.zeros((H, Dk, Dv), dtype=torch.float32, device=dev) if state is None else state.float().clone()
    C = chunk
    N = (T + C - 1) // C
    pad = N * C - T
    if pad:                                    # padded steps: no decay (g = 0), nothing written (k = 0, beta = 0)
        z = lambda x: torch.nn.functional.pad(x, (0, 0) * (x.dim() - 1) + (0, pad))
        qf, kf, vf = z(qf), z(kf), z(vf)
        g, beta = z(g.float()), z(beta.float())
    hc = lambda x: x.reshape(N, C, H, -1).permute(2, 0, 1, 3)                 # [H, N, C, D]
    Q, K, V = hc(qf), hc(kf), hc(vf)
    G = g.float().reshape(N, C, H).permute(2, 0, 1).cumsum(-1)                # [H, N, C] running log decay
    B = beta.float().reshape(N, C, H).permute(2, 0, 1)
    diff = (G[..., :, None] - G[..., None, :])                                # G_t - G_i
    lower = torch.ones((C, C), dtype=torch.bool, device=dev).tril()
    D = torch.where(lower, diff, torch.full_like(diff, float("-inf"))).exp()  # e^{G_t - G_i} for i <= t, else 0
    KK = K @ K.transpose(-1, -2)
    A = (B[..., :, None] * D * KK).tril(-1)
    eye = torch.eye(C, dtype=torch.float32, device=dev).expand(H, N, C, C)
    Tm = torch.linalg.solve_triangular(eye + A, eye, upper=False, unitriangular=True)
    eG = G.exp()
    W1 = Tm @ (B[..., None] * V)                                              # [H, N, C, Dv]
    W2 = Tm @ ((B * eG)[..., None] * K)                                       # [H, N, C, Dk]
    QK = (Q @ K.transpose(-1, -2)) * D                                        # already lower-triangular through D
    Kend = K * (G[..., -1:, None] - G[..., None]).exp()                       # e^{G_C - G_i} k_i
    out = torch.empty((H, N, C, Dv), dtype=torch.float32, device=dev)
    for n in range(N):
        U = W1[:, n] - W2[:, n] @ S                                           # [H, C, Dv]
        out[:, n] = eG[:, n, :, None] * (Q[:, n] @ S) + QK[:, n] @ U
        S = eG[:, n, -1, None, None] * S + Kend[:, n].transpose(-1, -2) @ U
    o = out.permute(1, 2, 0, 3).reshape(N * C, H, Dv)[:T]
    return o.contiguous(), S


CHUNKED_FROM = 32          # tokens per call from which the chunked form is used (single-token decode stays recurrent)


class GatedDeltaNetLayer:
    def __init__(self, cfg: DeltaNetConfig, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, weights

    @classmethod
    def from_state_dict(cls, cfg: DeltaNetConfig, sd: Dict[str, torch.Tensor], prefix: str = "", device="cuda",
                        dtype=torch.bfloat16) -> "GatedDeltaNetLayer":
        t = lambda x: x.to(dtype).to(device).contiguous()
        f = lambda x: x.float().to(device).contiguous()
        # one GEMM for all four input projections: [q | k | v | z | b | a] rows
        w = {"in.w": t(torch.cat([sd[prefix + f"in_proj_{n}.weight"] for n in ("qkv", "z", "b", "a")], 0)),
             "conv.w": f(sd[prefix + "conv1d.weight"].squeeze(1)),                # [channels, kernel]
             "A_log": f(sd[prefix + "A_log"]), "dt_bias": f(sd[prefix + "dt_bias"]),
             "norm.w": f(sd[prefix + "norm.weight"]), "out.w": t(sd[prefix + "out_proj.weight"])}
        return cls(cfg, w)

    def init_state(self, device) -> Tuple[torch.Tensor, torch.Tensor]:
        c = self.cfg
        conv_dim = 2 * c.linear_num_key_heads * c.linear_key_head_dim + c.linear_num_value_heads * c.linear_value_head_dim
        return (torch.zeros((c.linear_conv_kernel_dim - 1, conv_dim), dtype=torch.float32, device=device),
                torch.zeros((c.linear_num_value_heads, c.linear_key_head_dim, c.linear_value_head_dim),
                            dtype=torch.float32, device=device))

    def forward(self, x: torch.Tensor, state: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
        """x [T, hidden] (one sequence, in order) -> (y [T, hidden], new state)."""
        c, w = self.cfg, self.w
        Hk, Hv, Dk, Dv, K = (c.linear_num_key_heads, c.linear_num_value_heads, c.linear_key_head_dim,
                             c.linear_value_head_dim, c.linear_conv_kernel_dim)
        T = x.shape[0]
        conv_tail, S = state if state is not None else self.init_state(x.device)
        proj = Dn.gemm_bf16(x.to(w["in.w"].dtype).contiguous(), w["in.w"], out_dtype=torch.float32).float()
        kd, vd = Hk * Dk, Hv * Dv
        mixed, z, b, a = proj[:, : 2 * kd + vd], proj[:, 2 * kd + vd: 2 * kd + 2 * vd], \
            proj[:, 2 * kd + 2 * vd: 2 * kd + 2 * vd + Hv], proj[:, 2 * kd + 2 * vd + Hv:]
        # causal depth-wise convolution over [tail ; new tokens]
        seq = torch.cat([conv_tail, mixed], 0)                                        # [K - 1 + T, channels]
        win = seq.unfold(0, K, 1)                                                     # [T, channels, K]
        mixed = torch.nn.functional.silu((win * w["conv.w"][None]).sum(-1))
        q = mixed[:, :kd].view(T, Hk, Dk)
        k = mixed[:, kd:2 * kd].view(T, Hk, Dk)
        v = mixed[:, 2 * kd:].view(T, Hv, Dv)
        if Hv != Hk:
            q, k = q.repeat_interleave(Hv // Hk, 1), k.repeat_interleave(Hv // Hk, 1)
        g = -w["A_log"].exp() * torch.nn.functional.softplus(a + w["dt_bias"])
        rule = gated_delta_rule_chunked if T >= CHUNKED_FROM else gated_delta_rule
        o, S = rule(q, k, v, g, torch.sigmoid(b), S)
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + c.rms_norm_eps) * w["norm.w"]
        o = o * torch.nn.functional.silu(z.view(T, Hv, Dv))
        y = Dn.gemm_bf16(o.reshape(T, vd).to(w["out.w"].dtype).contiguous(), w["out.w"])
        return y, (seq[-(K - 1):].contiguous(), S)
