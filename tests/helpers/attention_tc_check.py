"""Child process of tests/test_zy_attention_tc_gpu.py: runs the tcgen05 attention kernel on one case and compares
it with the fp32 reference op.  Prints one JSON line.  Runs in a process of its own so that the kernel's first
runs on a device cannot take the test session's CUDA context with them."""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from antfly_b200 import _native as N  # noqa: E402
from antfly_b200.ops import attention as A  # noqa: E402
from antfly_b200.ops import reference as R  # noqa: E402


def varlen_case(D, Hq, Hkv, lens, causal, window, seed):
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    H = Hq * D
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, generator=g).to(torch.bfloat16)
    q = qkv[:, :H].view(T, Hq, D)
    k = qkv[:, H:H + Hkv * D].view(T, Hkv, D)
    v = qkv[:, H + Hkv * D:].view(T, Hkv, D)
    L = torch.tensor(lens, dtype=torch.int32)
    starts = (torch.cumsum(L, 0) - L).int()
    cu = torch.cat([starts.long(), torch.tensor([T])])
    want = R.varlen_attention(q, k, v, cu, D ** -0.5, causal, window)
    dq = qkv.cuda()
    got = A.attention_tc(dq[:, :H].view(T, Hq, D), dq[:, H:H + Hkv * D].view(T, Hkv, D),
                         dq[:, H + Hkv * D:].view(T, Hkv, D), starts.cuda(), L.cuda(), L.cuda(), max(lens), causal,
                         window)
    torch.cuda.synchronize()
    return got.float().cpu(), want.float()


def paged_case(D, Hq, Hkv, q_lens, ctx_lens, window, page, seed):
    g = torch.Generator().manual_seed(seed)
    B = len(q_lens)
    kv = [a + b for a, b in zip(q_lens, ctx_lens)]
    nblk = sum((n + page - 1) // page for n in kv) + 3
    kc = torch.randn(nblk, page, Hkv, D, generator=g).to(torch.bfloat16)
    vc = torch.randn(nblk, page, Hkv, D, generator=g).to(torch.bfloat16)
    perm = torch.randperm(nblk, generator=g)
    tables = torch.zeros((B, max((n + page - 1) // page for n in kv) + 1), dtype=torch.int32)
    off = 0
    for b, n in enumerate(kv):
        nb = (n + page - 1) // page
        tables[b, :nb] = perm[off:off + nb].int()
        off += nb
    T = sum(q_lens)
    q = torch.randn(T, Hq, D, generator=g).to(torch.bfloat16)
    ql = torch.tensor(q_lens, dtype=torch.int32)
    qs = (torch.cumsum(ql, 0) - ql).int()
    kl = torch.tensor(kv, dtype=torch.int32)
    want = R.paged_attention(q, kc, vc, tables, qs, ql, kl, D ** -0.5, window)
    got = A.attention_tc(q.cuda(), None, None, qs.cuda(), ql.cuda(), kl.cuda(), max(q_lens), True, window,
                         k_cache=kc.cuda(), v_cache=vc.cuda(), block_tables=tables.cuda())
    torch.cuda.synchronize()
    return got.float().cpu(), want.float()


def main():
    spec = json.loads(sys.argv[1])
    if spec["kind"] == "varlen":
        got, want = varlen_case(spec["D"], spec["Hq"], spec["Hkv"], spec["lens"], spec["causal"], spec["window"], spec["seed"])
    else:
        got, want = paged_case(spec["D"], spec["Hq"], spec["Hkv"], spec["q_lens"], spec["ctx_lens"], spec["window"],
                               spec["page"], spec["seed"])
    err = (got - want).abs()
    tol = 2e-2 + 2e-2 * want.abs()
    print(json.dumps({"max_err": float(err.max()), "bad": int((err > tol).sum()), "n": int(err.numel()),
                      "finite": bool(torch.isfinite(got).all()), "status": int(N.status())}))


if __name__ == "__main__":
    main()
