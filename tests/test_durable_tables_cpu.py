"""Tables kept in a data directory: documents, embeddings and definitions come back after the server restarts."""
import os

import pytest
import torch
from fastapi.testclient import TestClient

from antfly_b200.api.model_manager import ModelManager
from antfly_b200.api.server import create_app
from antfly_b200.index.flat import GrowableFlatIndex
from antfly_b200.index.lsm_store import LsmStore
from antfly_b200.index.table import Table, TableQuery


def _docs(n, dim=8, seed=0):
    g = torch.Generator().manual_seed(seed)
    emb = torch.nn.functional.normalize(torch.randn(n, dim, generator=g), dim=-1)
    docs = {f"doc{i}": {"text": f"document number {i} about {'cats' if i % 2 else 'dogs'}", "n": i} for i in range(n)}
    return docs, emb


def test_a_table_over_a_store_recovers_documents_embeddings_and_deletes(tmp_path):
    docs, emb = _docs(40)
    calls = []

    def embed(texts):
        calls.append(len(texts))
        return torch.stack([emb[int(t.split()[2])] for t in texts])

    d = str(tmp_path / "store")
    with LsmStore(d, background=False) as store:
        t = Table("t", dense_index=GrowableFlatIndex(8, "cosine", device="cpu"), embed=embed, store=store)
        t.upsert(docs)
        assert t.delete("doc3") and t.delete("doc4") and not t.delete("nope")
        t.upsert({"doc5": {"text": "document number 5 about birds", "n": 500}})
        before = [(h.id, round(h.score, 5)) for h in t.query(TableQuery(embedding=emb[7], limit=5))]
        assert before[0][0] == "doc7" and calls == [40, 1]
    with LsmStore(d, background=False) as store:
        t2 = Table("t", dense_index=GrowableFlatIndex(8, "cosine", device="cpu"), embed=embed, store=store)
        assert t2.recover() == 38 and len(t2) == 38
        assert calls == [40, 1]                                  # nothing was embedded again
        assert t2.docs["doc5"] == {"text": "document number 5 about birds", "n": 500} and "doc3" not in t2.docs
        assert [(h.id, round(h.score, 5)) for h in t2.query(TableQuery(embedding=emb[7], limit=5))] == before
        assert [h.id for h in t2.query(TableQuery(full_text_search="birds", limit=3))] == ["doc5"]
        wal = store.stats()["wal_records"]
        t2.recover()
        assert store.stats()["wal_records"] == wal               # a replay writes nothing back
    with pytest.raises(TypeError):
        Table._store_key(3.5)
    assert Table._from_store_key(Table._store_key(12345)) == 12345 and Table._from_store_key(Table._store_key("é")) == "é"


def test_tables_of_a_server_with_a_data_directory_survive_a_restart(tmp_path):
    data = str(tmp_path / "data")
    docs, emb = _docs(30)
    mgr = lambda: ModelManager(models_dir="/nonexistent", device="cpu")
    with TestClient(create_app(mgr(), data_dir=data)) as c:
        r = c.post("/db/v1/tables/articles", json={"dimension": 8, "metric": "cosine", "index_type": "hnsw",
                                                  "neighbors": 8})
        assert r.status_code == 200 and r.json()["durable"] is True and r.json()["restored"] == 0
        assert c.post("/db/v1/tables/bad name!", json={"dimension": 8}).status_code >= 400
        r = c.post("/db/v1/tables/articles/batch",
                   json={"inserts": docs, "embeddings": {k: emb[i].tolist() for i, k in enumerate(docs)}})
        assert r.status_code == 200 and r.json()["count"] == 30
        assert c.post("/db/v1/tables/articles/batch", json={"deletes": ["doc0", "doc1"]}).json()["deleted"] == 2
        c.post("/db/v1/tables/scratch", json={"dimension": 8})
        assert c.delete("/db/v1/tables/scratch").json() == {"table": "scratch", "dropped": True}
        assert c.delete("/db/v1/tables/scratch").status_code == 404
        q = {"embeddings": {"v": emb[9].tolist()}, "limit": 4}
        before = c.post("/db/v1/tables/articles/query", json=q).json()["responses"][0]["hits"]["hits"]
        assert before[0]["_id"] == "doc9"
        for t in c.app.state.tables.values():                    # what a shutdown does
            t.store.close()
    assert sorted(os.listdir(os.path.join(data, "tables"))) == ["articles"]
    with TestClient(create_app(mgr(), data_dir=data)) as c:
        assert c.get("/db/v1/tables").json()["tables"] == [{"name": "articles", "count": 28}]
        after = c.post("/db/v1/tables/articles/query", json=q).json()["responses"][0]["hits"]["hits"]
        assert [(h["_id"], round(h["_score"], 5)) for h in after] == [(h["_id"], round(h["_score"], 5)) for h in before]
        r = c.post("/db/v1/tables/articles/query", json={"full_text_search": "cats", "filter_query": "n:>20", "limit": 50})
        ids = sorted(h["_id"] for h in r.json()["responses"][0]["hits"]["hits"])
        assert ids == sorted(f"doc{i}" for i in range(21, 30, 2))
        assert c.post("/db/v1/tables/articles", json={"dimension": 8}).status_code == 409
        for t in c.app.state.tables.values():
            t.store.close()
