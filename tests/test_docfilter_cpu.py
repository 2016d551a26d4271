"""Document filters of table queries (query strings and query objects), and the query fields built on them: key
prefix, filter / exclusion before scoring, ordering with a cursor, counting, profiling."""
import pytest
import torch

from antfly_b200.index.docfilter import compile_filter
from antfly_b200.index.flat import GrowableFlatIndex
from antfly_b200.index.table import Table, TableQuery

DOCS = {
    "article:1": {"text": "red apples and green apples", "status": "published", "year": 2021, "tags": ["fruit", "food"],
                  "created_at": "2023-05-01", "meta": {"lang": "en"}, "deprecated": False},
    "article:2": {"text": "how to bake an apple pie", "status": "draft", "year": 2019, "tags": ["food"],
                  "created_at": "2022-11-20", "meta": {"lang": "en"}, "deprecated": False},
    "article:3": {"text": "roman roads and aqueducts", "status": "published", "year": 2024, "tags": ["history"],
                  "created_at": "2024-02-02", "meta": {"lang": "de"}, "deprecated": True},
    "note:1": {"text": "apple harvest notes", "status": "archived", "year": 2020, "tags": [],
               "created_at": "2020-01-01", "meta": {"lang": "en"}, "deprecated": False},
}


def keys(q):
    f = compile_filter(q)
    return sorted(k for k, d in DOCS.items() if f(d))


def test_query_strings():
    assert keys("status:published") == ["article:1", "article:3"]
    assert keys("year:>2020") == ["article:1", "article:3"] and keys("year:<=2020") == ["article:2", "note:1"]
    assert keys("created_at:>2023-01-01") == ["article:1", "article:3"]          # ISO dates order as strings
    assert keys("+status:published +meta.lang:en") == ["article:1"]
    assert keys("status:published AND year:>2022") == ["article:3"]
    assert keys("status:draft OR status:archived") == ["article:2", "note:1"]
    assert keys("-status:draft") == ["article:1", "article:3", "note:1"]
    assert keys("+tags:food -status:draft") == ["article:1"]
    assert keys("tags:history") == ["article:3"] and keys("deprecated:true") == ["article:3"]
    assert keys('text:"apple pie"') == ["article:2"] and keys("text:apple") == ["article:2", "note:1"]
    assert keys("text:app*") == ["note:1"] and keys("aqueducts") == ["article:3"]
    assert keys("status:published NOT deprecated:true") == ["article:1"]
    assert keys("") == sorted(DOCS) and keys(None) == sorted(DOCS)
    assert keys("missing:1") == []


def test_query_objects():
    assert keys({"query": "+status:published +year:>2022"}) == ["article:3"]
    assert keys({"term": "draft", "field": "status"}) == ["article:2"]
    assert keys({"match": "apple pie", "field": "text"}) == ["article:2", "note:1"]
    assert keys({"match_phrase": "green apples", "field": "text"}) == ["article:1"]
    assert keys({"prefix": "roman", "field": "text"}) == ["article:3"]
    assert keys({"field": "year", "min": 2020, "max": 2024}) == ["article:1", "note:1"]
    assert keys({"field": "year", "min": 2020, "max": 2024, "inclusive_max": True}) == ["article:1", "article:3", "note:1"]
    assert keys({"conjuncts": [{"term": "published", "field": "status"}, {"field": "year", "min": 2022}]}) == ["article:3"]
    assert keys({"disjuncts": [{"term": "draft", "field": "status"}, {"bool": True, "field": "deprecated"}]}) == [
        "article:2", "article:3"]
    assert keys({"must": {"term": "published", "field": "status"}, "must_not": {"bool": True, "field": "deprecated"}}) == [
        "article:1"]
    assert keys({"match_all": {}}) == sorted(DOCS) and keys({"match_none": {}}) == []
    with pytest.raises(ValueError):
        compile_filter({"fuzzy": "x"})


def _table():
    g = torch.Generator().manual_seed(0)
    emb = torch.nn.functional.normalize(torch.randn(len(DOCS), 16, generator=g), dim=-1)
    t = Table("t", dense_index=GrowableFlatIndex(16, "cosine", device="cpu"))
    t.upsert(DOCS, embeddings=emb)
    return t, dict(zip(DOCS, emb))


def test_filters_apply_before_scoring_in_every_index():
    t, emb = _table()
    # the nearest vector is filtered out: the hit list still fills from what is allowed
    hits = t.query(TableQuery(embedding=emb["article:2"], limit=2, filter_query="status:published"))
    assert [h.id for h in hits] and all(DOCS[h.id]["status"] == "published" for h in hits) and len(hits) == 2
    hits = t.query(TableQuery(full_text_search="apple apples", limit=5, exclusion_query="status:draft OR status:archived"))
    assert [h.id for h in hits] == ["article:1"]
    hits = t.query(TableQuery(full_text_search="apple apples", limit=5, filter_prefix="note:"))
    assert [h.id for h in hits] == ["note:1"]
    # no scoring query at all: everything that passes the filter
    prof = {}
    hits = t.query(TableQuery(filter_query={"field": "year", "min": 2020}, limit=10, profile=prof))
    assert sorted(h.id for h in hits) == ["article:1", "article:3", "note:1"]
    assert prof["filter_matches"] == 3 and prof["total_ms"] >= prof["filter_ms"] >= 0
    assert t.query(TableQuery(full_text_search="apple", filter_query="status:nothing")) == []


def test_order_by_cursor_and_the_endpoint_fields():
    from fastapi.testclient import TestClient

    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.api.server import create_app

    t, emb = _table()
    page = t.query(TableQuery(full_text_search="apple apples roman", limit=2, order_by=[{"field": "year", "desc": True}]))
    assert [h.id for h in page] == ["article:3", "article:1"] and page[1].sort == ["2021", "article:1"]
    nxt = t.query(TableQuery(full_text_search="apple apples roman", limit=2, order_by=[{"field": "year", "desc": True}],
                             search_after=page[-1].sort))
    assert [h.id for h in nxt] == ["note:1", "article:2"]
    asc = t.query(TableQuery(full_text_search="apple apples roman", limit=4, order_by=[{"field": "created_at"}]))
    assert [h.id for h in asc] == ["note:1", "article:2", "article:1", "article:3"]
    app = create_app(ModelManager(models_dir="/nonexistent", device="cpu"))
    app.state.tables["t"] = t
    c = TestClient(app)
    r = c.post("/db/v1/tables/t/query", json={"full_text_search": "apple apples roman", "limit": 2, "profile": True,
                                              "order_by": [{"field": "year", "desc": True}], "filter_prefix": "article:"})
    body = r.json()["responses"][0]
    assert r.status_code == 200 and [h["_id"] for h in body["hits"]["hits"]] == ["article:3", "article:1"]
    assert body["hits"]["hits"][0]["_sort"] == ["2024", "article:3"] and "full_text_ms" in body["profile"]
    r = c.post("/db/v1/tables/t/query", json={"full_text_search": "apple apples roman", "limit": 2,
                                              "order_by": [{"field": "year", "desc": True}], "filter_prefix": "article:",
                                              "search_after": body["hits"]["hits"][-1]["_sort"]})
    assert [h["_id"] for h in r.json()["responses"][0]["hits"]["hits"]] == ["article:2"]
    r = c.post("/db/v1/tables/t/query", json={"filter_query": "status:published", "count": True})
    assert r.json()["responses"][0]["hits"] == {"total": 2, "hits": [], "max_score": 0.0}
    for bad in ({"full_text_search": "x", "search_after": ["1"]},
                {"full_text_search": "x", "order_by": [{"field": "year"}], "search_after": ["1"], "offset": 1},
                {"embeddings": emb["note:1"].tolist(), "order_by": [{"field": "year"}]},
                {"full_text_search": "x", "filter_query": {"fuzzy": 1}}):
        assert c.post("/db/v1/tables/t/query", json=bad).status_code == 400, bad


def test_aggregations_over_the_matched_documents():
    from fastapi.testclient import TestClient

    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.api.server import create_app
    from antfly_b200.index.aggregations import aggregate

    docs = list(DOCS.values())
    out = aggregate(docs, {"y": {"type": "stats", "field": "year"}, "n": {"type": "count"},
                           "langs": {"type": "cardinality", "field": "meta.lang"},
                           "total": {"type": "sum", "field": "year"}, "top": {"type": "max", "field": "year"}})
    assert out["y"]["count"] == 4 and out["y"]["min"] == 2019 and out["y"]["max"] == 2024 and out["y"]["avg"] == 2021.0
    assert abs(out["y"]["std_deviation"] - (sum((v - 2021) ** 2 for v in (2021, 2019, 2024, 2020)) / 4) ** 0.5) < 1e-9
    assert out["n"]["value"] == 4 and out["langs"]["value"] == 2 and out["total"]["value"] == 8084 and out["top"]["value"] == 2024
    out = aggregate(docs, {"by_status": {"type": "terms", "field": "status", "size": 2,
                                         "sub_aggregations": {"avg_year": {"type": "avg", "field": "year"}}},
                           "by_tag": {"type": "terms", "field": "tags"}})
    assert out["by_status"]["buckets"][0] == {"key": "published", "doc_count": 2,
                                              "sub_aggregations": {"avg_year": {"value": 2022.5}}}
    assert len(out["by_status"]["buckets"]) == 2
    assert out["by_tag"]["buckets"][0] == {"key": "food", "doc_count": 2}
    out = aggregate(docs, {"eras": {"type": "range", "field": "year", "ranges": [
        {"name": "old", "to": 2021}, {"name": "new", "from": 2021}]},
        "per_2y": {"type": "histogram", "field": "year", "interval": 2, "min_doc_count": 1},
        "by_year": {"type": "date_histogram", "field": "created_at", "calendar_interval": "year"},
        "recent": {"type": "date_range", "field": "created_at", "date_ranges": [{"name": "since-2023", "from": "2023-01-01"}]}})
    assert [(b["key"], b["doc_count"]) for b in out["eras"]["buckets"]] == [("old", 2), ("new", 2)]
    assert [(b["key"], b["doc_count"]) for b in out["per_2y"]["buckets"]] == [(2018.0, 1), (2020.0, 2), (2024.0, 1)]
    assert [(b["key"], b["doc_count"]) for b in out["by_year"]["buckets"]] == [("2020", 1), ("2022", 1), ("2023", 1), ("2024", 1)]
    assert out["recent"]["buckets"][0]["doc_count"] == 2
    for bad in ({"g": {"type": "geohash_grid", "field": "loc"}}, {"s": {"type": "sum"}},
                {"h": {"type": "histogram", "field": "year"}}):
        with pytest.raises(ValueError):
            aggregate(docs, bad)
    t, _ = _table()
    app = create_app(ModelManager(models_dir="/nonexistent", device="cpu"))
    app.state.tables["t"] = t
    r = TestClient(app).post("/db/v1/tables/t/query", json={
        "full_text_search": "apple apples", "limit": 1, "filter_prefix": "article:",
        "aggregations": {"by_status": {"type": "terms", "field": "status"}}})
    body = r.json()["responses"][0]
    assert r.status_code == 200 and len(body["hits"]["hits"]) == 1 and body["hits"]["total"] == 2
    assert sorted((b["key"], b["doc_count"]) for b in body["aggregations"]["by_status"]["buckets"]) == [
        ("draft", 1), ("published", 1)]
