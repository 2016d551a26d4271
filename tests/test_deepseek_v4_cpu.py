"""DeepSeek-V4 decoder: the building blocks against the reference's own worked examples
(zig/pkg/inference/src/architectures/deepseek_v4_host.zig tests), and the whole model against a row-by-row
restatement of the reference's loops (architectures/gpt.zig deepSeekV4* functions)."""
import math

import pytest
import torch

from antfly_b200.models import deepseek_v4 as V4


def _sig(x):
    return 1.0 / (1.0 + math.exp(-x))


def _silu(x):
    return x * _sig(x)


# -- worked examples from the reference's tests ------------------------------------------------------------------
def test_route_selection_bias_steers_choice_weights_stay_unbiased():
    pick, w = V4.select_routes(torch.tensor([[-2.0, 1.0, 4.0, 0.5]]), torch.tensor([0.0, 10.0, 0.0, 0.0]), 2,
                               "sqrtsoftplus", True, 1.5)
    assert pick.tolist() == [[1, 2]]
    assert abs(float(w.sum()) - 1.5) < 1e-5
    sp = lambda x: math.sqrt(math.log1p(math.exp(x)))
    assert abs(float(w[0, 0]) - 1.5 * sp(1.0) / (sp(1.0) + sp(4.0))) < 1e-5


def test_hyper_head_weights_and_collapse():
    streams = torch.tensor([[[3.0, 4.0], [0.0, 0.0]], [[6.0, 8.0], [0.0, 0.0]]])
    fn = torch.tensor([[1.0, 0, 0, 0], [0, 0, 1.0, 0]])
    w = V4.hyper_head_weights(streams, fn, torch.zeros(2), torch.tensor([1.0]), 1e-6, 0.0)
    assert abs(float(w[0, 0]) - (_sig(1.2) + 1e-6)) < 1e-6 and abs(float(w[0, 1]) - (0.5 + 1e-6)) < 1e-6
    torch.testing.assert_close(w[0], w[1])
    streams = torch.tensor([[[1.0, 2.0, 3.0], [10.0, 20.0, 30.0]]])
    w = V4.hyper_head_weights(streams, torch.zeros(2, 6), torch.tensor([0.0, math.log(3.0)]), torch.tensor([1.0]),
                              0.0, 1e-6)
    out = torch.einsum("ts,tsh->th", w, streams)
    torch.testing.assert_close(out, torch.tensor([[8.0, 16.0, 24.0]]), atol=1e-5, rtol=0)


def test_hyper_connection_update_with_zero_projections():
    cfg = V4.DeepseekV4Config(hc_mult=2, hc_sinkhorn_iters=1, hc_eps=0.0, rms_norm_eps=1e-6, hidden_size=2)
    m = V4.DeepseekV4Model.__new__(V4.DeepseekV4Model)
    m.cfg, m.w = cfg, {"k.fn": torch.zeros(8, 4), "k.base": torch.zeros(8), "k.scale": torch.ones(3)}
    streams = torch.tensor([[[1.0, 2.0], [9.0, 18.0]]])
    out = m._hc_post(streams, torch.tensor([[3.0, 4.0]]), "k")
    torch.testing.assert_close(out, torch.tensor([[[3.25, 6.0], [3.25, 6.0]]]))
    # the head form broadcasts a weighted update into every stream
    m.w = {"k.fn": torch.zeros(2, 4), "k.base": torch.tensor([0.0, math.log(3.0)]), "k.scale": torch.ones(1)}
    out = m._hc_post(torch.tensor([[[1.0, 2.0], [10.0, 20.0]]]), torch.tensor([[4.0, 8.0]]), "k")
    torch.testing.assert_close(out, torch.tensor([[[3.0, 6.0], [13.0, 26.0]]]))


def test_trailing_rope_and_its_inverse():
    x = torch.tensor([[[11.0, 12.0, 1.0, 0.0], [21.0, 22.0, 0.0, 1.0]]])
    y = V4.trailing_rope(x, torch.tensor([1]), 2, 10000.0)
    want = torch.tensor([[[11.0, 12.0, math.cos(1), math.sin(1)], [21.0, 22.0, -math.sin(1), math.cos(1)]]])
    torch.testing.assert_close(y, want)
    x = torch.arange(1.0, 9.0).view(1, 2, 4)
    back = V4.trailing_rope(V4.trailing_rope(x, torch.tensor([3]), 2, 10000.0), torch.tensor([3]), 2, 10000.0, True)
    torch.testing.assert_close(back, x, atol=1e-5, rtol=0)
    # second pair turns slower: angle = pos / theta^(2/4)
    y = V4.trailing_rope(torch.tensor([[[1.0, 0.0, 1.0, 0.0]]]), torch.tensor([5]), 4, 100.0)
    torch.testing.assert_close(y, torch.tensor([[[math.cos(5), math.sin(5), math.cos(0.5), math.sin(0.5)]]]))


def test_sinkhorn_clamped_swiglu_grouped_projection():
    m = V4.sinkhorn(torch.tensor([[0.2, 0.8], [0.4, 0.6]]), 20, 1e-6)
    assert torch.allclose(m.sum(0), torch.ones(2), atol=1e-4) and torch.allclose(m.sum(1), torch.ones(2), atol=1e-4)
    y = V4.clamped_swiglu(torch.tensor([20.0, -1.0]), torch.tensor([3.0, -20.0]), 10.0)
    torch.testing.assert_close(y, torch.tensor([_silu(10.0) * 3.0, _silu(-1.0) * -10.0]))
    w = torch.zeros(2, 2, 2)                                    # (group, out, in)
    w[0, 0, 0] = w[0, 1, 1] = 1.0
    w[1, 0, 0] = w[1, 1, 1] = 10.0
    out = V4.grouped_output_projection(torch.tensor([[1.0, 2.0, 3.0, 4.0]]), w.view(4, 2), 2)
    # per group [1, 2] and [30, 40]; the reference's helper sums the groups (31, 42), the model concatenates them
    # and lets o_b mix: summing is o_b = [I I]
    torch.testing.assert_close(out, torch.tensor([[1.0, 2.0, 30.0, 40.0]]))
    torch.testing.assert_close(out.view(2, 2).sum(0), torch.tensor([31.0, 42.0]))


# -- the whole model against per-row loops ------------------------------------------------------------------------
def _tiny(hc_mult=2, hash_layers=1, topk=2, full_hc=True, seed=0):
    g = torch.Generator().manual_seed(seed)
    H, heads, D, rope, qr, orank, groups, E, I, V = 16, 4, 8, 4, 12, 6, 2, 4, 10, 50
    idx_h, idx_d = 2, 6
    cfg = V4.DeepseekV4Config(
        vocab_size=V, hidden_size=H, num_hidden_layers=3, num_attention_heads=heads, head_dim=D, q_lora_rank=qr,
        qk_rope_head_dim=rope, o_groups=groups, o_lora_rank=orank, sliding_window=5, rope_theta=10000.0,
        compress_rope_theta=4000.0, compress_rate_csa=2, compress_rate_hca=3, index_n_heads=idx_h,
        index_head_dim=idx_d, index_topk=topk, hc_mult=hc_mult, hc_sinkhorn_iters=3, hc_eps=1e-4, swiglu_limit=1.5,
        num_local_experts=E, num_experts_per_tok=2, moe_intermediate_size=I, scoring_func="sqrtsoftplus",
        norm_topk_prob=True, routed_scaling_factor=1.3, num_hash_layers=hash_layers,
        layer_types=[V4.SLIDING, V4.SPARSE, V4.HEAVY], rms_norm_eps=1e-6)
    r = lambda *s, k=0.4: torch.randn(*s, generator=g) * k
    sd = {"model.embed_tokens.weight": r(V, H, k=1.0), "model.norm.weight": 1 + r(H, k=0.1), "lm_head.weight": r(V, H)}
    if hc_mult:
        sd.update({"model.hc_head.hc_fn": r(hc_mult, hc_mult * H), "model.hc_head.hc_base": r(hc_mult),
                   "model.hc_head.hc_scale": torch.tensor([0.7])})
    for l in range(3):
        s = f"model.layers.{l}."
        sd[s + "input_layernorm.weight"], sd[s + "post_attention_layernorm.weight"] = 1 + r(H, k=0.1), 1 + r(H, k=0.1)
        a = s + "self_attn."
        sd.update({a + "q_a_proj.weight": r(qr, H), a + "q_a_norm.weight": 1 + r(qr, k=0.1),
                   a + "q_b_proj.weight": r(heads * D, qr), a + "kv_proj.weight": r(D, H),
                   a + "kv_norm.weight": 1 + r(D, k=0.1), a + "o_a_proj.weight": r(groups * orank, heads * D // groups),
                   a + "o_b_proj.weight": r(H, groups * orank), a + "sinks": r(heads, k=1.0)})
        if hc_mult:
            rows = (2 + hc_mult) * hc_mult if full_hc else hc_mult
            for hc in ("attn_hc", "ffn_hc"):
                sd.update({s + hc + ".fn": r(rows, hc_mult * H), s + hc + ".base": r(rows),
                           s + hc + ".scale": torch.tensor([0.9, 1.1, 0.8])})
        kind = cfg.layer_types[l]
        if kind != V4.SLIDING:
            rate = cfg.rate(l)
            pools = [("compressor", D)] + ([("compressor.indexer", idx_d)] if kind == V4.SPARSE else [])
            for pool, dim in pools:
                gw = rate if pool == "compressor" else 1
                sd.update({a + pool + ".kv_proj.weight": r(dim, H), a + pool + ".gate_proj.weight": r(gw, H),
                           a + pool + ".kv_norm.weight": 1 + r(dim, k=0.1),
                           a + pool + ".position_bias": r(rate, dim) if pool == "compressor" else r(dim)})
            if kind == V4.SPARSE:
                sd[a + "compressor.indexer.q_b_proj.weight"] = r(idx_h * idx_d, qr)
                sd[a + "compressor.indexer.weights_proj.weight"] = r(idx_h, H)
        m = s + "mlp."
        sd[m + "gate.weight"] = r(E, H, k=1.0)
        if l < hash_layers:
            sd[m + "gate.tid2eid"] = torch.randint(0, E, (V, 2), generator=g).float().flatten()
        else:
            sd[m + "gate.e_score_correction_bias"] = r(E, k=1.0)
        sd[m + "experts.gate_up_proj"] = r(E, 2, I, H)
        sd[m + "experts.down_proj"] = r(E, H, I)
        sd.update({m + "shared_experts.gate_proj.weight": r(I, H), m + "shared_experts.up_proj.weight": r(I, H),
                   m + "shared_experts.down_proj.weight": r(H, I)})
    return cfg, sd


def _rms(v, w, eps):
    y = v / math.sqrt(sum(float(x) ** 2 for x in v) / len(v) + eps)
    return y * w if w is not None else y


def _rope_row(v, pos, rope, theta, sign=1.0):
    v = v.clone()
    D = v.numel()
    for pair in range(rope // 2):
        ang = sign * pos / theta ** (pair * 2 / rope)
        i = D - rope + 2 * pair
        x0, x1 = float(v[i]), float(v[i + 1])
        v[i], v[i + 1] = x0 * math.cos(ang) - x1 * math.sin(ang), x0 * math.sin(ang) + x1 * math.cos(ang)
    return v


class LoopOracle:
    """The reference's algorithm with its loops: every call recomputes from the whole token history, the way its
    cached path would after the same sequence of calls (``calls`` = lengths of the successive forward calls)."""

    def __init__(self, cfg, sd):
        self.c, self.sd = cfg, {k: v.float() for k, v in sd.items()}

    def pool(self, hs, l, pool, rate, dim, theta, total):
        c, sd = self.c, self.sd
        a = f"model.layers.{l}.self_attn.{pool}."
        rows, positions = [], []
        for b in range((total + rate - 1) // rate):
            start, end = b * rate, min(total, b * rate + rate)
            acc, den = torch.zeros(dim), 0.0
            for p in range(start, end):
                gl = sd[a + "gate_proj.weight"] @ hs[p]
                g = _sig(float(gl[p - start] if gl.numel() == rate else gl[0]))
                bias = sd[a + "position_bias"]
                bias = bias.view(rate, dim)[p - start] if bias.numel() == rate * dim else bias
                acc += g * (sd[a + "kv_proj.weight"] @ hs[p] + bias)
                den += g
            if den > 0:
                acc = acc / den
            pos = min(total - 1, end - 1)
            rows.append(_rope_row(_rms(acc, sd[a + "kv_norm.weight"], c.rms_norm_eps), pos, min(c.qk_rope_head_dim, dim),
                                  theta))
            positions.append(pos)
        return rows, positions

    def attention(self, l, hs_all, q_rows, total_after_call):
        """hs_all: normed inputs of all tokens up to the end of the current call; q_rows: positions of this call."""
        c, sd = self.c, self.sd
        a = f"model.layers.{l}.self_attn."
        H, D, rope, theta = c.num_attention_heads, c.head_dim, c.qk_rope_head_dim, c.theta(l)
        kind = c.layer_types[l]
        kv = [_rope_row(_rms(sd[a + "kv_proj.weight"] @ h, sd[a + "kv_norm.weight"], c.rms_norm_eps), p, rope, theta)
              for p, h in enumerate(hs_all)]
        comp = idx = None
        if kind != V4.SLIDING:
            comp = self.pool(hs_all, l, "compressor", c.rate(l), D, theta, total_after_call)
            if kind == V4.SPARSE:
                idx = self.pool(hs_all, l, "compressor.indexer", c.rate(l), c.index_head_dim, theta, total_after_call)
        outs = []
        for qp in q_rows:
            h = hs_all[qp]
            ql = _rms(sd[a + "q_a_proj.weight"] @ h, sd[a + "q_a_norm.weight"], c.rms_norm_eps)
            q = (sd[a + "q_b_proj.weight"] @ ql).view(H, D)
            q = torch.stack([_rope_row(_rms(q[i], None, c.rms_norm_eps), qp, rope, theta) for i in range(H)])
            keys = [kv[k] for k in range(max(0, qp + 1 - c.sliding_window), qp + 1)]
            if comp is not None:
                rows, positions = comp
                cand = [i for i, p in enumerate(positions) if p <= qp]
                if kind == V4.SPARSE and c.index_topk > 0:
                    iq = (sd[a + "compressor.indexer.q_b_proj.weight"] @ ql).view(c.index_n_heads, c.index_head_dim)
                    hw = sd[a + "compressor.indexer.weights_proj.weight"] @ h
                    sc = {i: sum(_sig(float(hw[j])) * float(iq[j] @ idx[0][i]) for j in range(c.index_n_heads)) /
                          math.sqrt(c.index_head_dim) for i in cand}
                    cand = sorted(cand, key=lambda i: -sc[i])[: c.index_topk]
                keys += [rows[i] for i in cand]
            K = torch.stack(keys)
            ctx = torch.zeros(H, D)
            for i in range(H):
                lg = (K @ q[i]) / math.sqrt(D)
                sink = float(sd[a + "sinks"][i])
                mx = max(sink, float(lg.max()))
                e = torch.exp(lg - mx)
                ctx[i] = (e[:, None] * K).sum(0) / (math.exp(sink - mx) + float(e.sum()))
                ctx[i] = _rope_row(ctx[i], qp, rope, theta, -1.0)
            G = max(1, c.o_groups)
            gw = H * D // G
            oa = sd[a + "o_a_proj.weight"].view(G, -1, gw)
            mid = torch.cat([oa[g] @ ctx.flatten()[g * gw:(g + 1) * gw] for g in range(G)])
            outs.append(sd[a + "o_b_proj.weight"] @ mid)
        return outs

    def ffn(self, l, x, tok):
        c, sd = self.c, self.sd
        m = f"model.layers.{l}.mlp."
        lg = sd[m + "gate.weight"] @ x
        score = lambda v: math.sqrt(max(math.log1p(math.exp(float(v))), 0.0))
        E, k = c.num_local_experts, c.num_experts_per_tok
        if m + "gate.tid2eid" in sd and l < c.num_hash_layers:
            ids = [int(sd[m + "gate.tid2eid"][tok * k + i]) for i in range(k)]
        else:
            b = sd[m + "gate.e_score_correction_bias"]
            ids = sorted(range(E), key=lambda e: -(score(lg[e]) + float(b[e])))[:k]
        wts = [score(lg[e]) for e in ids]
        tot = sum(wts)
        wts = [w / tot * c.routed_scaling_factor for w in wts]
        out = torch.zeros_like(x)
        gu_all, down = sd[m + "experts.gate_up_proj"], sd[m + "experts.down_proj"]
        for e, wt in zip(ids, wts):
            gate = (gu_all[e, 0] @ x).clamp(max=c.swiglu_limit)
            up = (gu_all[e, 1] @ x).clamp(-c.swiglu_limit, c.swiglu_limit)
            out += wt * (down[e] @ (torch.nn.functional.silu(gate) * up))
        sh = torch.nn.functional.silu(sd[m + "shared_experts.gate_proj.weight"] @ x) * \
            (sd[m + "shared_experts.up_proj.weight"] @ x)
        return out + sd[m + "shared_experts.down_proj.weight"] @ sh

    def hc(self, stream, key):
        """-> (pre [hc], post [hc] | None, comb [hc, hc] | None) for one token's streams [hc, H]."""
        c, sd = self.c, self.sd
        hc = c.hc_mult
        flat = stream.flatten()
        r = 1.0 / math.sqrt(float(flat.pow(2).mean()) + c.rms_norm_eps)
        fn, base, scale = sd[key + ".fn"], sd[key + ".base"], sd[key + ".scale"]
        if fn.shape[0] == hc:
            return [_sig(float(fn[s] @ flat) * r * float(scale[0]) + float(base[s])) + c.hc_eps for s in range(hc)], None, None
        pre = [_sig(float(fn[d] @ flat) * r * float(scale[0]) + float(base[d])) + c.hc_eps for d in range(hc)]
        post = [_sig(float(fn[hc + d] @ flat) * r * float(scale[1]) + float(base[hc + d])) + c.hc_eps for d in range(hc)]
        comb = torch.tensor([[_sig(float(fn[2 * hc + d * hc + s] @ flat) * r * float(scale[2]) +
                                   float(base[2 * hc + d * hc + s])) + c.hc_eps for s in range(hc)] for d in range(hc)])
        for _ in range(c.hc_sinkhorn_iters):
            comb = comb / (comb.sum(1, keepdim=True) + c.hc_eps)
            comb = comb / (comb.sum(0, keepdim=True) + c.hc_eps)
        return pre, post, comb

    def run(self, ids, calls):
        c, sd = self.c, self.sd
        hc, L = c.hc_mult, c.num_hidden_layers
        normed = [[] for _ in range(L)]                      # per layer: attention-normed inputs of all tokens so far
        logits = []
        done = 0
        for n in calls:
            rows = list(range(done, done + n))
            xs = [sd["model.embed_tokens.weight"][ids[p]] for p in rows]
            streams = [x[None].repeat(hc, 1) for x in xs] if hc else None
            for l in range(L):
                s = f"model.layers.{l}."
                ins = []
                for i in range(n):
                    if hc:
                        pre, post, comb = self.hc(streams[i], s + "attn_hc")
                        a_in = sum(pre[d] * streams[i][d] for d in range(hc)) if comb is None else \
                            sum(pre[d] * comb[d, k] * streams[i][k] for d in range(hc) for k in range(hc))
                    else:
                        a_in = xs[i]
                    ins.append(_rms(a_in, sd[s + "input_layernorm.weight"], c.rms_norm_eps))
                normed[l] += ins
                upd = self.attention(l, normed[l], rows, done + n)
                for i in range(n):
                    if hc:
                        streams[i] = self.post(streams[i], upd[i], s + "attn_hc")
                        pre, post, comb = self.hc(streams[i], s + "ffn_hc")
                        f_in = sum(pre[d] * streams[i][d] for d in range(hc)) if comb is None else \
                            sum(pre[d] * comb[d, k] * streams[i][k] for d in range(hc) for k in range(hc))
                    else:
                        xs[i] = xs[i] + upd[i]
                        f_in = xs[i]
                    u = self.ffn(l, _rms(f_in, sd[s + "post_attention_layernorm.weight"], c.rms_norm_eps), ids[rows[i]])
                    if hc:
                        streams[i] = self.post(streams[i], u, s + "ffn_hc")
                    else:
                        xs[i] = xs[i] + u
            for i in range(n):
                if hc:
                    flat = streams[i].flatten()
                    r = 1.0 / math.sqrt(float(flat.pow(2).mean()) + c.rms_norm_eps)
                    fn, base, sc = sd["model.hc_head.hc_fn"], sd["model.hc_head.hc_base"], sd["model.hc_head.hc_scale"]
                    x = sum((_sig(float(fn[d] @ flat) * r * float(sc[0]) + float(base[d])) + c.hc_eps) * streams[i][d]
                            for d in range(hc))
                else:
                    x = xs[i]
                logits.append(sd["lm_head.weight"] @ _rms(x, sd["model.norm.weight"], c.rms_norm_eps))
            done += n
        return torch.stack(logits)

    def post(self, stream, update, key):
        pre, post, comb = self.hc(stream, key)
        hc = self.c.hc_mult
        if comb is None:
            return torch.stack([stream[d] + pre[d] * update for d in range(hc)])
        return torch.stack([pre[d] * (sum(comb[d, k] * stream[k] for k in range(hc)) + post[d] * update)
                            for d in range(hc)])


@pytest.mark.parametrize("variant", ["full_hc", "head_hc", "no_hc", "topk_all"])
@pytest.mark.parametrize("calls", [[9], [1] * 9, [4, 1, 3, 1]])
def test_model_matches_the_row_by_row_algorithm(variant, calls):
    kw = {"full_hc": {}, "head_hc": dict(full_hc=False), "no_hc": dict(hc_mult=0, hash_layers=0),
          "topk_all": dict(topk=0)}[variant]
    cfg, sd = _tiny(**kw)
    ids = torch.randint(0, cfg.vocab_size, (9,), generator=torch.Generator().manual_seed(5)).tolist()
    want = LoopOracle(cfg, sd).run(ids, calls)
    model = V4.DeepseekV4Model.from_state_dict(cfg, sd, device="cpu", dtype=torch.float32)
    st, got, at = None, [], 0
    for n in calls:
        lg, st = model.forward(torch.tensor(ids[at:at + n]), st)
        got.append(lg)
        at += n
    torch.testing.assert_close(torch.cat(got), want, atol=2e-4, rtol=2e-3)
    assert st.length == 9 and st.local[0].shape[0] == cfg.sliding_window
    assert st.comp[1].rows.shape[0] == 5 and st.comp[2].rows.shape[0] == 3 and 0 not in st.comp


def test_prefill_in_one_call_differs_from_token_steps_only_through_open_blocks():
    """A block's compressed row sits at the newest token of the block, so during a long prefill the tokens inside
    an unfinished block do not see it; sliding layers are unaffected.  The reference behaves the same."""
    cfg, sd = _tiny()
    cfg.layer_types = [V4.SLIDING] * 3
    sd2 = {k: v for k, v in sd.items() if ".compressor." not in k}
    model = V4.DeepseekV4Model.from_state_dict(cfg, sd2, device="cpu", dtype=torch.float32)
    ids = torch.arange(3, 12)
    whole, _ = model.forward(ids)
    st, rows = None, []
    for t in ids:
        lg, st = model.forward(t.view(1), st)
        rows.append(lg[0])
    torch.testing.assert_close(torch.stack(rows), whole, atol=1e-5, rtol=1e-4)


def test_config_aliases_and_schedules():
    c = V4.DeepseekV4Config.from_hf({"model_type": "deepseek_v4", "num_hidden_layers": 4, "rope_head_dim": 32,
                                     "score_func": "sigmoid", "route_scale": 2.5, "n_routed_experts": 16,
                                     "compress_rates": {"csa": 4, "hca": 64}, "compress_ratios": [0, 4, 64, 4],
                                     "num_hash_layers": 1, "eos_token_id": [7, 8]})
    assert (c.qk_rope_head_dim, c.scoring_func, c.routed_scaling_factor, c.num_local_experts) == (32, "sigmoid", 2.5, 16)
    assert c.layer_types == [V4.SLIDING, V4.SPARSE, V4.HEAVY, V4.SPARSE]
    assert [c.rate(i) for i in range(4)] == [0, 4, 64, 4] and c.hash_routed(0) and not c.hash_routed(1)
    assert c.eos_token_id == 7
    c = V4.DeepseekV4Config.from_hf({"num_hidden_layers": 2, "compress_rope_theta": 5e4, "rope_theta": 1e4,
                                     "layer_types": [V4.SLIDING, V4.HEAVY], "mlp_layer_types": ["moe", "hash_moe"]})
    assert c.theta(0) == 1e4 and c.theta(1) == 5e4 and not c.hash_routed(0) and c.hash_routed(1)


def test_loads_through_the_model_manager_and_generates(tmp_path):
    import json

    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.formats import safetensors_io as st
    from antfly_b200.runtime.sampling_params import SamplingParams

    cfg, sd = _tiny()
    cfg.vocab_size = 600
    g = torch.Generator().manual_seed(9)
    sd["model.embed_tokens.weight"] = torch.randn(600, 16, generator=g)
    sd["lm_head.weight"] = torch.randn(600, 16, generator=g) * 0.4
    sd["model.layers.0.mlp.gate.tid2eid"] = torch.randint(0, 4, (600, 2), generator=g).float().flatten()
    d = tmp_path / "generators" / "tiny-v4"
    d.mkdir(parents=True)
    st.save_file({k: v.contiguous() for k, v in sd.items()}, str(d / "model.safetensors"))
    conf = {k: getattr(cfg, k) for k in cfg.__dataclass_fields__}
    conf["model_type"] = "deepseek_v4_flash"
    (d / "config.json").write_text(json.dumps(conf))
    pipe = ModelManager(models_dir=str(tmp_path), device="cpu").get("tiny-v4", "generator").pipeline
    out = pipe.generate("hello there", SamplingParams(max_tokens=6, ignore_eos=True), raw_prompt=True)
    model = V4.DeepseekV4Model.from_state_dict(cfg, sd, device="cpu", dtype=torch.float32)
    ids = pipe.tokenizer.encode_prompt("hello there", add_bos=True)
    logits, state = model.forward(torch.tensor(ids))
    want = []
    for _ in range(6):
        want.append(int(logits[-1].argmax()))
        logits, state = model.forward(torch.tensor([want[-1]]), state)
    assert out.token_ids == want and out.completion_tokens == 6
