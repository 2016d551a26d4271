"""Sparse inverted index, BM25 full-text index and the hybrid table query (dense + sparse + full text, fusion,
pruning, rerank)."""
import math

import torch

from antfly_b200.index.flat import GrowableFlatIndex
from antfly_b200.index.fusion import MergeConfig, Pruner
from antfly_b200.index.sparse import FullTextIndex, SparseIndex, analyze
from antfly_b200.index.table import Table, TableQuery


def test_sparse_index_scores_are_dot_products_with_updates_and_deletes():
    g = torch.Generator().manual_seed(0)
    V, N = 50, 40
    dense = torch.rand(N, V, generator=g) * (torch.rand(N, V, generator=g) < 0.15)
    idx = SparseIndex(V, merge_threshold=64)                 # small threshold: exercises buffer merges
    idx.add_dense_rows([f"d{i}" for i in range(N)], dense)
    q = {3: 0.5, 7: 1.0, 11: 0.25, 49: 2.0}
    qv = torch.zeros(V)
    for t, w in q.items():
        qv[t] = w
    want = dense @ qv
    got = idx.search(q, 5)
    top = torch.topk(want, 5)
    assert [d for d, _ in got] == [f"d{i}" for i in top.indices.tolist() if want[i] > 0][: len(got)]
    for (d, s) in got:
        assert abs(s - float(want[int(d[1:])])) < 1e-5
    best = got[0][0]
    assert idx.delete(best) and not idx.delete(best) and len(idx) == N - 1
    assert best not in [d for d, _ in idx.search(q, 5)]
    idx.add(best, {49: 100.0})                                # re-add with a new vector
    assert idx.search(q, 1)[0] == (best, 200.0) and idx.doc_freq(49) == int((dense[:, 49] > 0).sum()) + (
        0 if dense[int(best[1:]), 49] > 0 else 1)


def test_bm25_ranking_and_formula():
    docs = {"a": "the quick brown fox jumps over the lazy dog", "b": "a fast brown fox", "c": "lazy dogs sleep all day",
            "d": "quantum computing with superconducting qubits", "e": "fox fox fox hunting foxes"}
    ft = FullTextIndex()
    for k, t in docs.items():
        ft.add(k, t)
    assert analyze("The Foxes are JUMPING") == ["fox", "jump"] or analyze("The Foxes are JUMPING") == ["foxe", "jump"]
    hits = ft.search("brown fox", 10)
    ids = [d for d, _ in hits]
    assert set(ids) == {"a", "b", "e"} and ids[0] == "b"      # both terms in the shortest document
    assert ft.search("qubits", 3)[0][0] == "d" and ft.search("nonexistent", 3) == []
    # one-term score against the formula
    toks = {k: analyze(t) for k, t in docs.items()}
    term = analyze("sleep")[0]
    df = sum(term in v for v in toks.values())
    avg = sum(len(v) for v in toks.values()) / len(toks)
    tf, dl = toks["c"].count(term), len(toks["c"])
    want = math.log(1 + (5 - df + 0.5) / (df + 0.5)) * tf * 2.2 / (tf + 1.2 * (1 - 0.75 + 0.75 * dl / avg))
    assert abs(ft.search("sleep", 1)[0][1] - want) < 1e-5
    ft.delete("b")
    assert [d for d, _ in ft.search("brown fox", 10)][0] in ("a", "e") and "b" not in dict(ft.search("brown fox", 10))


def _toy_embed(texts):
    # bag of hashed words -> 32-d vectors: texts sharing words are close
    out = torch.zeros(len(texts), 32)
    for i, t in enumerate(texts):
        for w in analyze(t, stopwords=False):
            out[i, sum(map(ord, w)) % 32] += 1.0
    return out


def test_table_hybrid_query_fuses_prunes_and_reranks():
    docs = {f"doc{i}": {"text": t, "n": i} for i, t in enumerate([
        "red apples and green apples", "how to bake an apple pie", "the history of the roman empire",
        "roman roads and aqueducts", "apple releases a new phone", "empire state building height",
        "green tea health benefits", "pie charts in spreadsheets"])}
    tbl = Table("t", dense_index=GrowableFlatIndex(32, "cosine"), embed=_toy_embed, sparse_terms=64,
                sparse_encode=lambda ts: torch.nn.functional.pad(_toy_embed(ts), (0, 32)),
                rerank=lambda q, ds: [float(len(set(analyze(q)) & set(analyze(d)))) for d in ds])
    tbl.upsert(docs)
    assert len(tbl) == 8
    # dense only
    hits = tbl.query(TableQuery(semantic_search="apple pie", limit=3))
    assert hits[0].id == "doc1" and set(hits[0].index_scores) == {"dense", "sparse"} and hits[0].document["n"] == 1
    # full text only, with documents attached
    hits = tbl.query(TableQuery(full_text_search="roman empire", limit=5))
    assert hits[0].id == "doc2" and {h.id for h in hits} == {"doc2", "doc3", "doc5"}
    assert all(set(h.index_scores) == {"full_text"} for h in hits)
    # hybrid RRF: documents found by several indexes rise; require_multi_index drops single-index hits
    q = TableQuery(semantic_search="green apples", full_text_search="green apples", limit=8,
                   pruner=Pruner(require_multi_index=True))
    hits = tbl.query(q)
    assert hits[0].id == "doc0" and all(len(h.index_scores) > 1 for h in hits)
    rrf = tbl.query(TableQuery(semantic_search="green apples", full_text_search="green apples", limit=1))[0]
    assert abs(rrf.score - 3 / 61.0) < 1e-9                  # rank 0 in all three indexes
    # RSF with weights, failover
    hits = tbl.query(TableQuery(semantic_search="apple", full_text_search="phone", limit=3,
                                merge=MergeConfig("rsf", weights={"full_text": 5.0})))
    assert hits[0].id == "doc4"
    hits = tbl.query(TableQuery(full_text_search="zzz", semantic_search="pie charts", limit=2,
                                merge=MergeConfig("failover")))
    assert hits and set(hits[0].index_scores) == {"dense"}
    # rerank stage re-scores the fused candidates
    hits = tbl.query(TableQuery(semantic_search="apple", full_text_search="apple", limit=3,
                                rerank_query="bake pie"))
    assert hits[0].id == "doc1" and hits[0].index_scores["reranker"] == 2.0
    # distance bound, delete, upsert replaces
    bounded = tbl.query(TableQuery(semantic_search="apple pie", limit=3, distance_under=-1.0))
    assert all("dense" not in h.index_scores for h in bounded)      # the bound filters the dense ranking only
    assert tbl.delete("doc1") and not tbl.delete("doc1")
    assert "doc1" not in [h.id for h in tbl.query(TableQuery(semantic_search="apple pie",
                                                              full_text_search="apple pie", limit=8))]
    tbl.upsert({"doc0": {"text": "volcanoes of iceland", "n": 0}})
    assert tbl.query(TableQuery(full_text_search="iceland volcanoes", semantic_search="iceland volcanoes",
                                limit=1))[0].id == "doc0"
