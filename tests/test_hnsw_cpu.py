"""Graph index: recall against exact search for the three metrics, filtered search (graph walk and direct scan),
deletion with repair, upsert, persistence, structural self-check, and its use as a table's dense index."""
import numpy as np
import pytest
import torch

from antfly_b200.index.flat import recall_at_k
from antfly_b200.index.hnsw import HNSWIndex


def _exact(x, q, metric, k):
    x, q = x.double(), q.double()
    if metric == "l2_squared":
        d = (q[:, None] - x[None]).pow(2).sum(-1)
    elif metric == "inner_product":
        d = -(q @ x.T)
    else:
        d = 1 - torch.nn.functional.normalize(q, dim=-1) @ torch.nn.functional.normalize(x, dim=-1).T
    v, i = torch.topk(d, k, dim=-1, largest=False)
    return v.float(), i


def _data(n=3000, d=24, nq=40, seed=0):
    g = torch.Generator().manual_seed(seed)
    centers = torch.randn(30, d, generator=g) * 3
    x = centers[torch.randint(0, 30, (n,), generator=g)] + torch.randn(n, d, generator=g)
    q = centers[torch.randint(0, 30, (nq,), generator=g)] + torch.randn(nq, d, generator=g)
    return x, q


@pytest.mark.parametrize("metric", ["l2_squared", "inner_product", "cosine"])
def test_recall_and_distances_against_exact_search(metric):
    x, q = _data()
    idx = HNSWIndex(x.shape[1], metric, neighbors=16, ef_construction=120, ef_search=80, seed=1)
    idx.batch_insert(range(1000, 1000 + len(x)), x)
    assert len(idx) == len(x) and idx.check() == 0
    st = idx.stats()
    assert st["max_layer"] >= 1 and 0 < st["upper_layer_nodes"] < len(x) // 4 and st["edges"] <= len(x) * 32 + st["upper_layer_nodes"] * 16 * 8
    res = idx.search(q, 10)
    dv, di = _exact(x, q, metric, 10)
    rec = recall_at_k(res.ids - 1000, di, 10)
    assert rec >= (0.9 if metric == "inner_product" else 0.97), rec
    # the distance reported for a hit is the metric's own value for that vector
    got = res.distances[0, 0].item()
    j = int(res.ids[0, 0]) - 1000
    want = _exact(x[j:j + 1], q[:1], metric, 1)[0].item()
    assert abs(got - want) < 1e-3 * max(1.0, abs(want))
    assert bool((res.distances[:, 1:] >= res.distances[:, :-1]).all())
    # more effort does not lose recall; a single query vector is accepted as well
    wide = idx.search(q, 10, effort=1.0)
    assert recall_at_k(wide.ids - 1000, di, 10) >= rec
    assert idx.search(q[0], 3).ids.shape == (1, 3)
    with pytest.raises(ValueError):
        idx.search(torch.zeros(1, 5), 3)


def test_parallel_search_equals_serial_search():
    x, q = _data(n=1500, nq=33, seed=3)
    a = HNSWIndex(x.shape[1], "l2_squared", seed=5, threads=1)
    a.batch_insert(range(len(x)), x)
    one = a.search(q, 7)
    a.threads = 8
    many = a.search(q, 7)
    assert torch.equal(one.ids, many.ids) and torch.equal(one.distances, many.distances)


def test_filtered_search_walks_the_graph_or_scans_directly():
    x, q = _data(n=2400, nq=20, seed=7)
    meta = [(b"tenant-a/" if i % 3 == 0 else b"tenant-b/" if i % 3 == 1 else b"rare/") + str(i).encode()
            for i in range(len(x))]
    for i in range(len(x)):
        if meta[i].startswith(b"rare/") and i % 60 != 2:
            meta[i] = b"tenant-b/" + str(i).encode()
    idx = HNSWIndex(x.shape[1], "l2_squared", ef_search=96, seed=2)
    idx.batch_insert(range(len(x)), x, metadata=meta)
    assert idx.metadata(3) == meta[3] and idx.metadata(10 ** 9) is None
    torch.testing.assert_close(idx.get_vector(3), x[3])
    assert idx.get_vector(10 ** 9) is None
    # a broad filter: graph walk, every hit carries the prefix, recall against the exact filtered answer
    keep = torch.tensor([m.startswith(b"tenant-a/") for m in meta])
    res = idx.search(q, 10, filter_prefix=b"tenant-a/")
    assert all(meta[i].startswith(b"tenant-a/") for i in res.ids.flatten().tolist())
    sub = keep.nonzero().flatten()
    _, di = _exact(x[sub], q, "l2_squared", 10)
    assert recall_at_k(res.ids, sub[di], 10) >= 0.95
    # a selective filter (40 matches): the direct scan is exact
    rare = torch.tensor([m.startswith(b"rare/") for m in meta]).nonzero().flatten()
    assert len(rare) == 40
    res = idx.search(q, 10, filter_prefix=b"rare/")
    _, di = _exact(x[rare], q, "l2_squared", 10)
    assert torch.equal(res.ids, rare[di])
    # fewer matches than k: the rest is padding; no match at all: all padding
    res = idx.search(q[:2], 50, filter_prefix=b"rare/")
    assert bool((res.ids[:, :40] >= 0).all()) and bool((res.ids[:, 40:] == -1).all())
    assert bool(torch.isinf(res.distances[:, 40:]).all())
    assert bool((idx.search(q[:2], 5, filter_prefix=b"nobody/").ids == -1).all())


def test_delete_repairs_the_graph_and_upsert_replaces():
    x, q = _data(n=2000, nq=30, seed=11)
    meta = [b"doc-%d" % (i // 4) for i in range(len(x))]               # four chunks per document
    idx = HNSWIndex(x.shape[1], "cosine", neighbors=12, ef_search=80, seed=4)
    idx.batch_insert(range(len(x)), x, metadata=meta)
    entry = idx.stats()["entry_point"]
    gone = set(range(0, len(x), 2)) | {entry}                          # half of the index, the entry point included
    assert idx.delete(sorted(gone) + [10 ** 9]) == len(gone)
    assert len(idx) == len(x) - len(gone) and idx.check() == 0
    assert idx.stats()["entry_point"] not in gone
    live = torch.tensor(sorted(set(range(len(x))) - gone))
    res = idx.search(q, 10)
    assert not (set(res.ids.flatten().tolist()) & gone)
    _, di = _exact(x[live], q, "cosine", 10)
    assert recall_at_k(res.ids, live[di], 10) >= 0.93
    # a document's chunks go together
    assert idx.delete_by_metadata(b"doc-7") == sum(1 for i in range(28, 32) if i not in gone)
    assert idx.check() == 0
    # freed slots are reused; re-inserting an id moves it
    before = idx.stats()["slots"]
    idx.batch_insert([1, 3, 3], torch.stack([x[5], x[6], q[0]]))       # an id repeated in a batch: the last one stays
    assert idx.stats()["slots"] == before and idx.check() == 0
    hit = idx.search(q[:1], 1)
    assert hit.ids[0, 0].item() == 3 and hit.distances[0, 0].item() < 1e-5
    # everything can go, and the index starts over
    left = len(idx)
    assert idx.delete(range(len(x))) == left
    assert len(idx) == 0 and idx.check() == 0 and bool((idx.search(q[:1], 3).ids == -1).all())
    idx.batch_insert([42], x[:1])
    assert idx.search(x[:1], 1).ids.item() == 42


def test_save_and_load_round_trip(tmp_path):
    x, q = _data(n=800, nq=10, seed=13)
    idx = HNSWIndex(x.shape[1], "inner_product", neighbors=8, neighbors_layer0=20, ef_search=50, seed=9)
    idx.batch_insert(range(len(x)), x, metadata=[b"m%d" % i for i in range(len(x))])
    idx.delete(range(0, 100))
    path = str(tmp_path / "graph.hnsw")
    idx.save(path)
    back = HNSWIndex.load(path)
    assert (back.dim, back.metric, back.ef_search) == (idx.dim, idx.metric, idx.ef_search)
    assert back.stats() == idx.stats() and back.check() == 0 and back.metadata(500) == b"m500"
    a, b = idx.search(q, 5), back.search(q, 5)
    assert torch.equal(a.ids, b.ids) and torch.equal(a.distances, b.distances)
    back.batch_insert([5], x[5:6])                                      # a loaded index keeps accepting writes
    assert back.check() == 0 and len(back) == len(idx) + 1
    raw = bytearray(open(path, "rb").read())
    raw[0] ^= 0xFF
    bad = str(tmp_path / "bad.hnsw")
    open(bad, "wb").write(bytes(raw))
    with pytest.raises(ValueError):
        HNSWIndex.load(bad)
    open(bad, "wb").write(bytes(raw[:200]))
    with pytest.raises(ValueError):
        HNSWIndex.load(bad)


def test_forced_levels_give_a_reproducible_shape():
    x = torch.eye(6)
    idx = HNSWIndex(6, "l2_squared", neighbors=2, seed=0)
    idx.batch_insert(range(6), x, levels=[0, 2, 0, 1, 0, 0])
    st = idx.stats()
    assert st["max_layer"] == 2 and st["entry_point"] == 1 and st["upper_layer_nodes"] == 2 and idx.check() == 0
    with pytest.raises(ValueError):
        HNSWIndex(0)
    with pytest.raises(ValueError):
        HNSWIndex(4, "manhattan")


def test_graph_index_as_a_tables_dense_index():
    from antfly_b200.index.table import Table, TableQuery

    g = torch.Generator().manual_seed(0)
    emb = torch.randn(50, 16, generator=g)
    t = Table("docs", dense_index=HNSWIndex(16, "cosine", seed=0))
    t.upsert({f"k{i}": {"text": f"document number {i}"} for i in range(50)}, embeddings=emb)
    hits = t.query(TableQuery(embedding=emb[17], limit=3))
    assert hits[0].id == "k17"
    t.delete("k17")
    assert all(h.id != "k17" for h in t.query(TableQuery(embedding=emb[17], limit=3)))
