"""Entity resolution into a knowledge graph and mention cleanup."""
from types import SimpleNamespace as NS

import pytest
import torch

from antfly_b200.pipelines import resolver as R


def test_string_similarity():
    assert R.jaro_winkler("hello", "hello") == 1.0 and R.jaro_winkler("", "hello") == 0.0
    assert R.jaro_winkler("martha", "marhta") == pytest.approx(0.9611, abs=1e-4)      # the textbook pair
    assert R.jaro_winkler("dixon", "dicksonx") == pytest.approx(0.8133, abs=1e-4)
    assert R.jaro("abc", "xyz") == 0.0
    # every word of the shorter name occurs in the longer one: lifted above plain Jaro-Winkler
    s = R.entity_similarity("marie curie", "marie sklodowska curie")
    assert s >= 0.7 + 0.3 * len("marie curie") / len("marie sklodowska curie") - 1e-12
    assert R.entity_similarity("a", "") == 0.0 and R.normalize_name("  Ada LOVELACE\n") == "ada lovelace"


def test_knowledge_graph_merges_mentions_and_relations():
    E = lambda t, l, s: NS(text=t, label=l, score=s, start=0, end=len(t))
    texts = [[E("Marie Curie", "person", 0.9), E("Paris", "place", 0.8), E("Curie", "device", 0.4)],
             [E("marie curie", "person", 0.95), E("Marie Sklodowska Curie", "person", 0.7), E("Paris", "place", 0.6),
              E("noise", "person", 0.05)]]
    rel = lambda h, t, l, s: NS(head=h, tail=t, label=l, score=s)
    rels = [[rel(texts[0][0], texts[0][1], "lives in", 0.6)],
            [rel(texts[1][1], texts[1][2], "lives in", 0.8), rel(E("Nobody", "person", 1.0), texts[1][2], "lives in", 0.9)]]
    kg = R.build_knowledge_graph(texts, rels, R.ResolverConfig(similarity_threshold=0.8, min_entity_confidence=0.1))
    by = {e.canonical_name: e for e in kg.entities}
    assert set(by) == {"Marie Sklodowska Curie", "Paris", "Curie"}                   # labels must match to merge
    p = by["Marie Sklodowska Curie"]
    assert p.score == pytest.approx(0.95) and p.text_indices == [0, 1]
    assert p.mentions == ["Marie Curie", "Marie Sklodowska Curie"]                     # normalised duplicates once
    assert len(kg.relations) == 1                                                      # unknown head dropped, rest merged
    r = kg.relations[0]
    assert (r.head_id, r.tail_id, r.label) == (p.id, by["Paris"].id, "lives in") and r.score == pytest.approx(0.8)
    assert r.text_indices == [0, 1]
    loose = R.build_knowledge_graph(texts, None, R.ResolverConfig(similarity_threshold=0.8, type_must_match=False,
                                                                  track_provenance=False))
    assert len(loose.entities) < len(kg.entities) + 1 and loose.entities[0].mentions is None
    assert R.build_knowledge_graph([], None).entities == []


def test_cleanup_drops_invalid_mentions_and_clusters_by_embedding():
    E = lambda t, l, s: NS(text=t, label=l, score=s, start=1, end=1 + len(t))
    v = lambda *x: torch.tensor(x, dtype=torch.float32)
    ms = [R.CleanupMention(E("IBM", "org", 0.9), 0.9, 0.5, v(1, 0, 0)),
          R.CleanupMention(E("I.B.M.", "org", 0.8), 0.8, 0.7, v(0.99, 0.1, 0)),
          R.CleanupMention(E("Big Blue", "org", 0.7), 0.7, 0.6, v(0.95, 0.32, 0)),    # close to the second only
          R.CleanupMention(E("IBM", "product", 0.9), 0.9, 0.9, v(1, 0, 0)),           # other type
          R.CleanupMention(E("junk", "org", 0.9), 0.2, 0.9, v(1, 0, 0)),              # invalid
          R.CleanupMention(E("zero", "org", 0.9), 0.9, 0.9, v(0, 0, 0))]              # no direction: alone
    res = R.cleanup_mentions(ms, R.CleanupConfig(dedup_similarity_threshold=0.95))
    assert [d["text"] for d in res.dropped_mentions] == ["junk"]
    got = {e.text: e for e in res.resolved_entities}
    assert set(got) == {"I.B.M.", "IBM", "zero"}                                       # chain 1-2-3 is one cluster
    assert got["I.B.M."].mentions == ["IBM", "I.B.M.", "Big Blue"] and got["I.B.M."].label == "org"
    assert got["IBM"].label == "product" and got["I.B.M."].id == "cleanup-entity-0"
    assert R.cleanup_mentions([], None).resolved_entities == []
