"""GPU numerics: the IVF list-scan kernel and the device-side probe (no host synchronisation)."""
import pytest
import torch

from antfly_b200.ops import reference as R

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("metric", ["cosine", "l2_squared", "inner_product"])
@pytest.mark.parametrize("dim", [64, 200, 768])
def test_ivf_list_scan_kernel_matches_reference(metric, dim):
    """afb_ivf_scan against a plain fp32 evaluation of the same grouped scoring: every (list, query) pair's members
    below the query's threshold are appended (order free), nothing else."""
    from antfly_b200 import _native as N
    from antfly_b200.index.distance import score_form
    from antfly_b200.ops import index_ops as IX

    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(dim)
    n_lists, nq = 37, 21
    sizes = torch.randint(0, 150, (n_lists,), generator=g, device=dev)
    sizes[5] = 0
    sizes[9] = 700
    off = torch.zeros(n_lists + 1, dtype=torch.int64, device=dev)
    off[1:] = torch.cumsum(sizes, 0)
    n = int(off[-1])
    x = torch.randn(n, dim, generator=g, device=dev).bfloat16()
    q = torch.randn(nq, dim, generator=g, device=dev).bfloat16()
    form = score_form(metric)
    row = IX.row_sqnorm(q) if form.use_row_norm else None
    col = IX.row_sqnorm(x) if form.use_col_norm else None
    probes = torch.stack([torch.randperm(n_lists, generator=g, device=dev)[:6] for _ in range(nq)]).int()
    probes[3, 4:] = -1
    pl = torch.where(probes.reshape(-1) >= 0, probes.reshape(-1).long(), torch.full((nq * 6,), n_lists, device=dev))
    pq = torch.arange(nq, device=dev, dtype=torch.int32)[:, None].expand(nq, 6).reshape(-1)
    pls, order = torch.sort(pl, stable=True)
    pair_q = pq[order].contiguous()
    pair_off = torch.searchsorted(pls, torch.arange(n_lists + 1, device=dev)).int()
    d_all = form.scale * (q.float() @ x.float().t())
    if row is not None:
        d_all = d_all + row[:, None]
    if col is not None:
        d_all = d_all + col[None, :]
    if form.clamp_zero:
        d_all = d_all.clamp_min(0)
    for thr_q in (None, 0.35):
        thr = None
        if thr_q is not None:
            thr = torch.quantile(d_all, thr_q, dim=1).contiguous()
        cap = 2048
        cv = torch.full((nq, cap), float("nan"), device=dev)
        ci = torch.full((nq, cap), -7, dtype=torch.int32, device=dev)
        cc = torch.zeros(nq, dtype=torch.int32, device=dev)
        IX.ivf_scan(x, col, q, row, thr, off, pair_off, pair_q, cv, ci, cc, form.scale, form.clamp_zero)
        torch.cuda.synchronize()
        assert N.status() == 0
        for qi in range(nq):
            want = {}
            for l in probes[qi].tolist():
                if l < 0:
                    continue
                for r in range(int(off[l]), int(off[l + 1])):
                    dv = float(d_all[qi, r])
                    if thr is None or dv < float(thr[qi]) - 1e-3:
                        want[r] = dv
            cnt = int(cc[qi])
            got = {int(i): float(v) for i, v in zip(ci[qi, :cnt].tolist(), cv[qi, :cnt].tolist())}
            assert len(got) == cnt                       # no row appended twice
            missing = [r for r in want if r not in got]
            assert not missing, (qi, missing[:5])
            for r, v in got.items():
                assert abs(v - float(d_all[qi, r])) < 2e-2 + 2e-2 * abs(v)
                if thr is not None:
                    assert v < float(thr[qi])


def test_ivf_search_on_gpu_equals_host_walk_and_never_synchronises():
    from antfly_b200 import _native as N
    from antfly_b200.index.ivf import IVFIndex

    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(2)
    centers = torch.randn(64, 96, generator=g, device=dev)
    x = centers[torch.randint(0, 64, (20000,), generator=g, device=dev)] + 0.3 * torch.randn(20000, 96, generator=g, device=dev)
    q = centers[torch.randint(0, 64, (50,), generator=g, device=dev)] + 0.3 * torch.randn(50, 96, generator=g, device=dev)
    idx = IVFIndex(x, 128, metric="cosine")
    a = idx.search(q, 10, nprobe=16)
    b = idx._search_host(q, 10, nprobe=16)
    assert N.status() == 0
    same = (a.ids == b.ids).float().mean()
    assert float(same) > 0.999          # equal up to ties between equal bf16 scores
    torch.testing.assert_close(a.distances, b.distances, atol=2e-3, rtol=2e-3)
    idx.search(q, 10, nprobe=16, check=False)                 # warm: allocator, module loads
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        r = idx.search(q, 10, nprobe=16, check=False)         # any host synchronisation would raise here
    finally:
        torch.cuda.set_sync_debug_mode("default")
    assert int(r.overflow) == 0
