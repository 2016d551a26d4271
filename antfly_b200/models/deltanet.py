"""Gated delta-rule linear attention (the recurrent layers of Qwen3.5 / Qwen3-Next decoders).

One layer keeps, per sequence, a short convolution tail and a matrix state ``S`` [value heads, key dim, value dim]
instead of a key / value cache.  For each token: Q, K, V come from one projection followed by a causal depth-wise
convolution (kernel 4) and SiLU; Q and K are L2-normalised per head; the state decays by ``exp(g)`` with
``g = -exp(A_log) * softplus(a + dt_bias)``, is corrected towards the new value by the delta rule
``S += k (x) ((v - S^T k) * beta)`` with ``beta = sigmoid(b)``, and is read with ``o = S^T q / sqrt(d_k)``; the
output is RMS-normalised per head, gated by ``SiLU(z)`` and projected back.  The reference carries the same op on
its CPU and Metal paths (zig/pkg/inference/src/architectures/gpt.zig:4462-4775).

The projections run on the bf16 GEMM; the recurrence is tensor arithmetic over all heads at once, one step per
token (state in fp32).  ``forward`` takes and returns the state, so prefill and single-token decode are the same
code.
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
        o, S = gated_delta_rule(q, k, v, g, torch.sigmoid(b), S)
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + c.rms_norm_eps) * w["norm.w"]
        o = o * torch.nn.functional.silu(z.view(T, Hv, Dv))
        y = Dn.gemm_bf16(o.reshape(T, vd).to(w["out.w"].dtype).contiguous(), w["out.w"])
        return y, (seq[-(K - 1):].contiguous(), S)
