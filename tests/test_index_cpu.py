"""Index logic on the CPU: fusion / pruner, search-effort mapping, wire codecs, RaBitQ, HBC tree and artifacts."""
import math
import zlib

import pytest
import torch

from antfly_b200.index import artifact, codec, fusion
from antfly_b200.index.distance import resolve_search_effort
from antfly_b200.index.flat import FlatIndex, exact_search_fp32, recall_at_k
from antfly_b200.index.hbc import HBCConfig, HBCIndex
from antfly_b200.index.rabitq import RaBitQuantizer, bit_product


def test_rrf_rsf_failover_and_pruner():
    res = {"dense": [("a", 0.9), ("b", 0.8), ("c", 0.1)], "text": [("b", 12.0), ("d", 3.0)]}
    rrf = fusion.fuse(res, fusion.MergeConfig("rrf"))
    assert [h.doc_id for h in rrf] == ["b", "a", "d", "c"]
    assert rrf[0].score == pytest.approx(1 / 62 + 1 / 61) and rrf[0].index_count == 2
    w = fusion.fuse(res, fusion.MergeConfig("rrf", weights={"text": 0.0}))
    assert [h.doc_id for h in w][:3] == ["a", "b", "c"]
    rsf = fusion.fuse(res, fusion.MergeConfig("rsf"))
    assert rsf[0].doc_id == "b" and rsf[0].score == pytest.approx((0.8 - 0.1) / 0.8 + 1.0)
    assert fusion.fuse({"x": [], "y": [("q", 1.0)]}, fusion.MergeConfig("failover"))[0].doc_id == "q"
    pr = fusion.prune(rrf, fusion.Pruner(require_multi_index=True))
    assert [h.doc_id for h in pr] == ["b"]
    pr = fusion.prune(rrf, fusion.Pruner(min_score_ratio=0.6))
    assert [h.doc_id for h in pr] == ["b"]
    hits = [fusion.FusedHit(i, s) for i, s in enumerate([1.0, 0.95, 0.9, 0.3, 0.25])]
    assert len(fusion.prune(hits, fusion.Pruner(max_score_gap_percent=50.0))) == 3
    assert len(fusion.prune(hits, fusion.Pruner(min_absolute_score=0.28))) == 4
    assert len(fusion.prune(hits, fusion.Pruner(std_dev_threshold=0.5))) == 3


def test_search_effort_mapping():
    w0, e0 = resolve_search_effort(10, 0.0)
    wh, eh = resolve_search_effort(10, 0.5)
    w1, e1 = resolve_search_effort(10, 1.0)
    assert w0 == 64 and e0 == 1.0
    assert wh == round(64 + 0.5 * (4096 - 64)) and eh == 7.0
    assert w1 == 4096 and e1 == 100.0
    assert resolve_search_effort(500, 0.0)[0] == 500


def test_vector_wire_codecs():
    v = torch.randn(3, 8)
    assert torch.equal(codec.decode_packed(codec.encode_packed(v), 8), v)
    assert codec.decode_vectors([1.0, 2.0]).shape == (1, 2) and codec.decode_vectors([[1, 2], [3, 4]]).shape == (2, 2)
    sp = codec.encode_sparse_packed([7, 2], [0.5, 1.5])
    assert codec.decode_sparse(sp) == {"indices": [2, 7], "values": [1.5, 0.5]}
    with pytest.raises(ValueError):
        codec.decode_packed("AAAA", 3)


@pytest.mark.parametrize("metric", ["l2_squared", "inner_product", "cosine"])
def test_rabitq_estimates_track_exact_distances(metric):
    from antfly_b200.ops import reference as R

    g = torch.Generator().manual_seed(0)
    D, n = 256, 400
    c = torch.randn(D, generator=g) * 0.1
    x = c + torch.randn(n, D, generator=g)
    q = c + torch.randn(D, generator=g)
    rq = RaBitQuantizer(D, metric)
    qs = rq.quantize(c, x)
    assert qs.codes.shape == (n, 4) and int(qs.code_counts[0]) == int((x[0] - c >= 0).sum())
    d, e = rq.estimate(qs, q)
    exact = R.distances(q[None], x, metric)[0]
    # within a few error bounds for almost every vector, and the ranking is strongly correlated
    within = ((d - exact).abs() <= 4 * e + 1e-3).float().mean()
    assert float(within) > 0.9
    rk = torch.corrcoef(torch.stack([d, exact]))[0, 1]
    assert float(rk) > 0.7
    # the weighted popcount agrees with a per-bit restatement
    planes = rq._query_planes(qs, q)[0]
    bp = bit_product(qs.codes[:5], planes)
    for i in range(5):
        bits = lambda w: [(int(w[j]) >> (63 - b)) & 1 for j in range(4) for b in range(64)]
        cb = bits(qs.codes[i])
        ref = sum((1 << p) * sum(a & b for a, b in zip(cb, bits(planes[p]))) for p in range(4))
        assert int(bp[i]) == ref


def test_hbc_build_search_recall_and_artifact_roundtrip(tmp_path):
    g = torch.Generator().manual_seed(1)
    centers = torch.randn(20, 32, generator=g)
    x = centers[torch.randint(0, 20, (3000,), generator=g)] + 0.3 * torch.randn(3000, 32, generator=g)
    q = centers[torch.randint(0, 20, (40,), generator=g)] + 0.3 * torch.randn(40, 32, generator=g)
    cfg = HBCConfig(32, "l2_squared", branching_factor=8, leaf_size=60, search_width=16)
    idx = HBCIndex.bulk_build(x, cfg)
    st = idx.stats()
    assert st["vectors"] == 3000 and st["leaves"] >= 3000 // 60 * 0.5 and st["levels"] >= 2
    truth = exact_search_fp32(q, x, 10, "l2_squared")
    found = torch.tensor([idx.search(q[i], 10)[0] + [-1] * 10 for i in range(40)])[:, :10]
    r = recall_at_k(found, truth.ids, 10)
    assert r > 0.8, r
    wide = torch.tensor([idx.search(q[i], 10, search_width=64)[0] for i in range(40)])
    assert recall_at_k(wide, truth.ids, 10) >= r
    artifact.save_hbc(idx, str(tmp_path / "hbc"))
    md = artifact.unpack_metadata(artifact.pack_metadata(cfg, idx.root, 3000, len(idx.nodes)))
    assert md["dims"] == 32 and md["leaf_size"] == 60 and md["metric"] == "l2_squared" and md["root_node"] == idx.root
    back = artifact.load_hbc(str(tmp_path / "hbc"))
    assert back.stats() == st
    assert back.search(q[0], 10)[0] == idx.search(q[0], 10)[0]
    nd = idx.nodes[idx.root]
    rt = artifact.unpack_node(nd.id, artifact.pack_node(nd))
    assert rt.children == nd.children and rt.level == nd.level and torch.equal(rt.centroid, nd.centroid.cpu())
    # quantised payloads are stored as protobuf messages and come back bit for bit
    for a, b in ((idx.nodes[i].quant, back.nodes[i].quant) for i in idx.nodes):
        assert torch.equal(a.codes, b.codes) and torch.equal(a.code_counts, b.code_counts)
        assert torch.equal(a.centroid_distances, b.centroid_distances) and torch.equal(a.inv_dot, b.inv_dot)
        assert torch.equal(a.centroid, b.centroid) and a.metric == b.metric


@pytest.mark.parametrize("metric", ["l2_squared", "inner_product", "cosine"])
def test_rabitq_payload_protobuf_wire_format(metric):
    """The payload is a protobuf message: checked field by field against a hand-assembled encoding, including
    code words with the top bit set (10-byte varints) and packed repeated scalars."""
    import struct

    from antfly_b200.index.rabitq import RaBitQuantizer

    g = torch.Generator().manual_seed(4)
    x = torch.randn(7, 130, generator=g)                       # 130 dims -> 3 code words per vector
    qz = RaBitQuantizer(130, metric)
    qs = qz.quantize(x.mean(0), x)
    blob = artifact.encode_rabitq_set(qs)
    back = artifact.decode_rabitq_set(blob)
    assert back.metric == metric and torch.equal(back.codes, qs.codes) and back.codes.shape == (7, 3)
    assert bool((qs.codes < 0).any())                          # top bit set somewhere: exercised the u64 path
    assert torch.equal(back.code_counts, qs.code_counts) and torch.equal(back.inv_dot, qs.inv_dot)
    if metric == "l2_squared":
        assert back.centroid_dot is None and back.centroid_norm == 0.0 and blob[0] == 0x12   # field 1 omitted (0)
    else:
        assert torch.equal(back.centroid_dot, qs.centroid_dot)
        assert abs(back.centroid_norm - qs.centroid_norm) < 1e-6 and blob[:2] == bytes([0x08, {"inner_product": 1,
                                                                                                "cosine": 2}[metric]])
    # field 2 (centroid) is a length-delimited run of little-endian floats right after the metric
    off = 0 if metric == "l2_squared" else 2
    assert blob[off] == 0x12
    n, p = artifact._read_varint(blob, off + 1)
    assert n == 130 * 4 and struct.unpack("<f", blob[p:p + 4])[0] == float(qs.centroid[0])
    # estimates from the decoded payload equal the originals
    q = torch.randn(130, generator=g)
    back.data_norms = qs.data_norms
    d0, e0 = qz.estimate(qs, q)
    d1, e1 = qz.estimate(back, q)
    assert torch.equal(d0, d1) and torch.equal(e0, e1)
    vs = artifact.decode_vector_set(artifact.encode_vector_set(x))
    assert torch.equal(vs, x)


def test_flat_index_cpu_path_is_exact():
    g = torch.Generator().manual_seed(2)
    x = torch.randn(5000, 32, generator=g)
    q = torch.randn(16, 32, generator=g)
    idx = FlatIndex(x.to(torch.bfloat16).float(), metric="l2_squared")
    idx.seed_cols, idx.cand_cap = 256, 512
    res = idx.search(q.to(torch.bfloat16).float(), 10)
    truth = exact_search_fp32(q.to(torch.bfloat16).float(), x.to(torch.bfloat16).float(), 10, "l2_squared")
    assert recall_at_k(res.ids, truth.ids, 10) == 1.0


def test_hilbert_keys_match_an_independent_restatement_and_order_is_local():
    import numpy as np

    from antfly_b200.index.hilbert import hilbert_keys, hilbert_order, random_orthogonal

    def py_key(vec):
        # Skilling's transform written independently (lists of Python ints), then MSB-first bit interleave
        x = [int(np.float32(v).view(np.uint32)) for v in vec]
        n, m = len(x), 1 << 31
        q = m
        while q > 1:
            p = q - 1
            for i in range(n):
                if x[i] & q:
                    x[0] ^= p
                else:
                    t = (x[0] ^ x[i]) & p
                    x[0] ^= t
                    x[i] ^= t
            q >>= 1
        for i in range(1, n):
            x[i] ^= x[i - 1]
        t, q = 0, m
        while q > 1:
            if x[n - 1] & q:
                t ^= q - 1
            q >>= 1
        x = [v ^ t for v in x]
        bits = [(x[i] >> b) & 1 for b in range(31, -1, -1) for i in range(n)]
        return bytes(int("".join(map(str, bits[k:k + 8])), 2) for k in range(0, len(bits), 8))

    g = torch.Generator().manual_seed(0)
    v = torch.rand(40, 3, generator=g)
    keys = hilbert_keys(v)
    assert keys.shape == (40, 12)
    for r in range(40):
        assert bytes(keys[r]) == py_key(v[r].tolist())
    # locality: neighbours along the curve are much closer than neighbours in random order (positive coordinates,
    # where float bit patterns are monotonic in value)
    pts = torch.rand(4000, 2, generator=g) + 1.0
    order = hilbert_order(pts)
    assert sorted(order.tolist()) == list(range(4000))
    along = (pts[order][1:] - pts[order][:-1]).norm(dim=-1).mean()
    rand = (pts[1:] - pts[:-1]).norm(dim=-1).mean()
    assert float(along) < 0.1 * float(rand)
    q = random_orthogonal(48, seed=7)
    torch.testing.assert_close(q @ q.T, torch.eye(48), atol=1e-5, rtol=1e-5)
    assert torch.equal(q, random_orthogonal(48, seed=7)) and not torch.equal(q, random_orthogonal(48, seed=8))


def test_hbc_hilbert_bulk_builds():
    g = torch.Generator().manual_seed(2)
    centers = torch.rand(20, 16, generator=g) * 4 + 1.0
    x = centers[torch.randint(0, 20, (3000,), generator=g)] + 0.1 * torch.randn(3000, 16, generator=g)
    q = centers[torch.randint(0, 20, (40,), generator=g)] + 0.1 * torch.randn(40, 16, generator=g)
    truth = exact_search_fp32(q, x, 10, "l2_squared")

    def recall(mode, width):
        idx = HBCIndex.bulk_build(x, HBCConfig(16, "l2_squared", branching_factor=8, leaf_size=60, search_width=width,
                                               bulk_build=mode))
        assert idx.stats()["vectors"] == 3000 and idx.stats()["levels"] >= 2
        found = torch.tensor([idx.search(q[i], 10)[0] + [-1] * 10 for i in range(40)])[:, :10]
        return recall_at_k(found, truth.ids, 10), idx

    r_seeded, idx = recall("hilbert_seeded", 16)
    assert r_seeded > 0.8, r_seeded                       # clustered leaves: as good as the k-means build
    r_pure, idx_pure = recall("hilbert", 16)
    assert idx_pure.stats()["leaves"] == 50 and r_pure > 0.3   # loose leaves: usable, clearly worse
    assert r_seeded > r_pure


def test_hbc_online_insert_split_and_delete():
    g = torch.Generator().manual_seed(3)
    centers = torch.randn(12, 24, generator=g)
    def draw(n):
        return centers[torch.randint(0, 12, (n,), generator=g)] + 0.25 * torch.randn(n, 24, generator=g)
    x0, x1 = draw(600), draw(2400)
    cfg = HBCConfig(24, "l2_squared", branching_factor=6, leaf_size=40, search_width=24)
    idx = HBCIndex.bulk_build(x0, cfg)
    before = idx.stats()
    for lo in range(0, 2400, 800):                      # three online batches
        idx.insert(x1[lo:lo + 800])
    st = idx.stats()
    assert st["vectors"] == 3000 and st["leaves"] > before["leaves"] and st["levels"] >= before["levels"]
    assert max(len(n.children) for n in idx.nodes.values() if n.is_leaf) <= 2 * cfg.leaf_size
    assert max(len(n.children) for n in idx.nodes.values() if not n.is_leaf) <= 2 * cfg.branching_factor
    # every vector sits in exactly one leaf and parents / children agree
    seen = sorted(v for n in idx.nodes.values() if n.is_leaf for v in n.children)
    assert seen == list(range(3000))
    for n in idx.nodes.values():
        if not n.is_leaf:
            assert all(idx.nodes[c].parent == n.id for c in n.children)
    allx = torch.cat([x0, x1])
    q = draw(40)
    truth = exact_search_fp32(q, allx, 10, "l2_squared")
    found = torch.tensor([idx.search(q[i], 10)[0] + [-1] * 10 for i in range(40)])[:, :10]
    assert recall_at_k(found, truth.ids, 10) > 0.8
    # per-query profile: wider search scores more leaves and re-ranks more vectors
    pa, pb = {}, {}
    idx.search(q[0], 10, search_width=4, epsilon=3.0, profile=pa)
    idx.search(q[0], 10, search_width=32, epsilon=3.0, profile=pb)
    assert 1 <= pa["leaves"] <= 4 < pb["leaves"] <= 32 and pb["reranked"] >= pa["reranked"] >= 10
    assert pa["internal_nodes"] >= 1 and pa["total_ns"] >= pa["leaf_ns"] + pa["internal_ns"] + pa["rerank_ns"] > 0
    # deletion: the deleted ids never come back
    gone = truth.ids[0, :5].tolist()
    assert idx.delete(gone) == 5 and idx.delete(gone) == 0
    assert not set(idx.search(q[0], 10)[0]) & set(gone)


def test_hbc_flat_directory_mode_recursive_build_and_leaf_merge():
    g = torch.Generator().manual_seed(5)
    centers = torch.randn(16, 24, generator=g)
    x = centers[torch.randint(0, 16, (2500,), generator=g)] + 0.25 * torch.randn(2500, 24, generator=g)
    q = centers[torch.randint(0, 16, (30,), generator=g)] + 0.25 * torch.randn(30, 24, generator=g)
    truth = exact_search_fp32(q, x, 10, "l2_squared")

    def recall(idx, **kw):
        found = torch.tensor([(idx.search(q[i], 10, **kw)[0] + [-1] * 10)[:10] for i in range(30)])
        return recall_at_k(found, truth.ids, 10)

    # top-down recursive build: every leaf fits, recall is in the same range as the bottom-up build
    rec = HBCIndex.bulk_build(x, HBCConfig(24, "l2_squared", branching_factor=8, leaf_size=50, search_width=16,
                                           bulk_build="recursive", epsilon=1.0))
    assert max(len(n.children) for n in rec.nodes.values() if n.is_leaf) <= 50 and recall(rec) > 0.8
    # flat directory: all leaf centroids are scored in blocks, the best `probe` leaves are opened
    cfg = HBCConfig(24, "l2_squared", branching_factor=8, leaf_size=50, search_width=16,
                    centroid_directory_mode="flat_rabitq", flat_centroid_block_size=16, epsilon=0.5)
    flat = HBCIndex.bulk_build(x, cfg)
    prof = {}
    flat.search(q[0], 10, profile=prof)
    n_leaves = sum(1 for n in flat.nodes.values() if n.is_leaf)
    assert prof["internal_nodes"] == -(-n_leaves // 16) and 1 <= prof["leaves"] <= 16
    r_flat = recall(flat)
    assert r_flat > 0.7                   # 1-bit codes of 24-d centroids in 16-centroid blocks: a coarse directory
    few = HBCIndex.bulk_build(x, HBCConfig(24, "l2_squared", branching_factor=8, leaf_size=50, search_width=16,
                                           centroid_directory_mode="flat_rabitq", flat_centroid_probe_count=2))
    p2 = {}
    few.search(q[0], 10, profile=p2)
    assert p2["leaves"] <= 2 and recall(few) <= r_flat + 1e-9
    # the directory follows inserts and deletes
    extra = centers[3] + 0.05 * torch.randn(40, 24, generator=g)
    flat.insert(extra, torch.arange(10000, 10040))
    ids, _ = flat.search(centers[3], 10)
    assert len(set(ids) & set(range(10000, 10040))) >= 8
    # deleting most of a leaf merges the rest into a sibling; nothing is lost, nothing deleted comes back
    leaf = next(n for n in flat.nodes.values() if n.is_leaf and len(n.children) >= 20)
    victims = [int(flat.ids[v]) for v in leaf.children[:-3]]
    survivors = [int(flat.ids[v]) for v in leaf.children[-3:]]
    before = sum(1 for n in flat.nodes.values() if n.is_leaf)
    assert flat.delete(victims) == len(victims)
    assert leaf.id not in flat.nodes and sum(1 for n in flat.nodes.values() if n.is_leaf) == before - 1
    seen = [int(flat.ids[v]) for n in flat.nodes.values() if n.is_leaf for v in n.children]
    assert set(survivors) <= set(seen) and not set(victims) & set(seen) and len(seen) == len(set(seen))
    for s_id in survivors:
        vec = flat.vectors[(flat.ids == s_id).nonzero()[0, 0]]
        assert flat.search(vec, 1, search_width=64)[0] == [s_id]
    for n in flat.nodes.values():
        if not n.is_leaf:
            assert all(c in flat.nodes and flat.nodes[c].parent == n.id for c in n.children)


def _dataset(kind: str, n: int, d: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    if kind == "clustered":
        c = torch.randn(24, d, generator=g)
        x = c[torch.randint(0, 24, (n,), generator=g)] + 0.3 * torch.randn(n, d, generator=g)
        q = c[torch.randint(0, 24, (32,), generator=g)] + 0.3 * torch.randn(32, d, generator=g)
    elif kind == "uniform":
        x, q = torch.rand(n, d, generator=g) - 0.5, torch.rand(32, d, generator=g) - 0.5
    else:                                  # heavy-tailed norms: what inner-product search has to cope with
        x = torch.randn(n, d, generator=g) * torch.rand(n, 1, generator=g).pow(3) * 3
        q = torch.randn(32, d, generator=g)
    return x, q


# expected recall@10 per (dataset, metric, index) with the tolerance the reference's recall tables use (a floor)
RECALL_CASES = [
    ("clustered", "l2_squared", "hbc", 0.85), ("clustered", "cosine", "hbc", 0.85),
    ("clustered", "inner_product", "hbc", 0.75), ("uniform", "l2_squared", "hbc", 0.7),
    ("uniform", "cosine", "hbc", 0.45), ("skewed", "inner_product", "hbc", 0.6),
    ("clustered", "l2_squared", "hbc_hilbert_seeded", 0.85), ("clustered", "cosine", "hbc_flat", 0.7),
    ("clustered", "l2_squared", "ivf", 0.9), ("clustered", "cosine", "ivf", 0.9),
    ("uniform", "inner_product", "ivf", 0.7), ("clustered", "l2_squared", "flat", 1.0),
    ("skewed", "inner_product", "flat", 1.0), ("uniform", "cosine", "flat", 0.99),
]


@pytest.mark.parametrize("dataset,metric,kind,floor", RECALL_CASES)
def test_recall_table(dataset, metric, kind, floor):
    from antfly_b200.index.ivf import IVFIndex

    x, q = _dataset(dataset, 3000, 32, seed=zlib.crc32(f"{dataset}-{metric}".encode()) % 997)
    xb, qb = x.to(torch.bfloat16).float(), q.to(torch.bfloat16).float()
    truth = exact_search_fp32(qb, xb, 10, metric)
    if kind == "flat":
        idx = FlatIndex(xb, metric=metric)
        idx.seed_cols, idx.cand_cap = 256, 512
        found = idx.search(qb, 10).ids
    elif kind == "ivf":
        found = IVFIndex(xb, 40, metric=metric).search(qb, 10, nprobe=12).ids
    else:
        extra = {"hbc": {}, "hbc_hilbert_seeded": {"bulk_build": "hilbert_seeded"},
                 "hbc_flat": {"centroid_directory_mode": "flat_rabitq"}}[kind]
        # epsilon widens the centroid-distance pruning band; data without cluster structure needs a wide one
        eps = 3.0 if dataset == "uniform" else 1.0
        idx = HBCIndex.bulk_build(xb, HBCConfig(32, metric, branching_factor=8, leaf_size=60, search_width=24,
                                                epsilon=eps, **extra))
        found = torch.tensor([(idx.search(qb[i], 10)[0] + [-1] * 10)[:10] for i in range(32)])
    r = recall_at_k(found, truth.ids, 10)
    assert r >= floor, (dataset, metric, kind, r)


@pytest.mark.parametrize("metric", ["l2_squared", "cosine", "inner_product"])
@pytest.mark.parametrize("nprobe", [1, 5, 12])
def test_ivf_fixed_launch_sequence_equals_the_host_driven_walk(metric, nprobe):
    """The one-sequence search (pair sort, seed list-scan, thresholded list-scan, select) returns exactly what the
    host-driven walk over the probed lists returns."""
    from antfly_b200.index.ivf import IVFIndex

    x, q = _dataset("clustered", 3000, 32, seed=11)
    xb, qb = x.to(torch.bfloat16).float(), q.to(torch.bfloat16).float()
    idx = IVFIndex(xb, 40, metric=metric)
    a = idx.search(qb, 10, nprobe=nprobe)
    b = idx._search_host(qb, 10, nprobe=nprobe)
    assert torch.equal(a.ids, b.ids)
    torch.testing.assert_close(a.distances, b.distances, atol=1e-5, rtol=1e-5)


def test_ivf_search_makes_no_host_round_trip_between_its_launches():
    """Inside ``search(check=False)`` nothing reads a device value on the host: the kernel wrappers (whose CPU
    fallbacks are exempt here) are the only places where data is touched."""
    from antfly_b200.index import ivf as IVF
    from antfly_b200.ops import index_ops as IX

    x, q = _dataset("clustered", 2000, 32, seed=5)
    idx = IVF.IVFIndex(x.to(torch.bfloat16).float(), 32, metric="cosine")
    counts = {"n": 0, "exempt": 0}

    def counting(name):
        orig = getattr(torch.Tensor, name)

        def f(self, *a, **k):
            if not counts["exempt"]:
                counts["n"] += 1
            return orig(self, *a, **k)
        return name, orig, f

    def exempt(fn):
        def g(*a, **k):
            counts["exempt"] += 1
            try:
                return fn(*a, **k)
            finally:
                counts["exempt"] -= 1
        return g

    patched = [counting(n) for n in ("item", "tolist", "cpu", "numpy", "__int__", "__bool__", "__float__", "__index__")]
    wrapped = {n: getattr(IX, n) for n in ("ivf_scan", "topk_select", "score_filter", "row_sqnorm")}
    try:
        for n, fn in wrapped.items():
            setattr(IX, n, exempt(fn))
        for n, _, f in patched:
            setattr(torch.Tensor, n, f)
        res = idx.search(q.to(torch.bfloat16).float(), 10, nprobe=8, check=False)
    finally:
        for n, orig, _ in patched:
            setattr(torch.Tensor, n, orig)
        for n, fn in wrapped.items():
            setattr(IX, n, fn)
    assert counts["n"] == 0
    assert res.overflow is not None and int(res.overflow) == 0


def test_ivf_overflow_is_reported_and_repaired():
    """A candidate buffer that is too small for the thresholded pass: ``check=False`` reports it, ``check=True``
    repeats on the safe path and returns the exact probed-list result."""
    from antfly_b200.index.ivf import IVFIndex

    x, q = _dataset("uniform", 3000, 32, seed=9)
    xb, qb = x.to(torch.bfloat16).float(), q.to(torch.bfloat16).float()
    idx = IVFIndex(xb, 8, metric="l2_squared")
    want = idx._search_host(qb, 10, nprobe=8)
    idx.cand_cap = 16
    flagged = idx.search(qb, 10, nprobe=8, check=False)
    assert int(flagged.overflow) == 1
    got = idx.search(qb, 10, nprobe=8)
    assert torch.equal(got.ids, want.ids)
