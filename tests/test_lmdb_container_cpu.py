"""The LMDB container of vector indexes: an environment written by the stock LMDB library is read entry for entry,
environments written here come back the same, and an HBC index survives the trip through one."""
import gzip
import os
import struct

import pytest
import torch

from antfly_b200.formats.lmdb_io import F_BIGDATA, LmdbError, LmdbReader, write_lmdb

FIXTURE = os.path.join(os.path.dirname(__file__), "data", "lmdb_stock_env.mdb.gz")


def _stock_contents():
    """What the fixture's generator stored with the stock library: three named databases filled in one transaction
    (keys ``k:%08d`` of (7919 i) mod 100003; values of 40, 1500 or 10000 bytes whose byte j is i + 31 j), then a
    second transaction deleting every third key of ``hbc_nodes``."""
    dbs = {}
    for name, n in (("hbc_nodes", 150), ("hbc_meta", 1), ("hbc_quant", 150)):
        kv = {}
        for i in range(n):
            size = 10000 if i % 97 == 0 else 1500 if i % 5 == 0 else 40
            kv[b"k:%08d" % ((i * 7919) % 100003)] = bytes((i + 31 * j) & 0xFF for j in range(size))
        dbs[name] = kv
    for i in range(0, 150, 3):
        del dbs["hbc_nodes"][b"k:%08d" % ((i * 7919) % 100003)]
    return dbs


def test_environment_written_by_the_stock_library_is_read_entry_for_entry(tmp_path):
    path = tmp_path / "data.mdb"
    path.write_bytes(gzip.decompress(open(FIXTURE, "rb").read()))
    want = _stock_contents()
    with LmdbReader(str(tmp_path)) as r:
        assert r.page_size == 4096 and r.txnid == 2                     # the second commit's meta page is current
        assert sorted(r.databases()) == sorted(want)
        for name, kv in want.items():
            got = list(r.items(name))
            assert [k for k, _ in got] == sorted(kv) and r.entries(name) == len(kv)
            assert all(kv[k] == v for k, v in got)
            for k in list(kv)[::7]:
                assert r.get(name, k) == kv[k]
            assert r.get(name, b"k:99999999") is None and r.get(name, b"a") is None
        with pytest.raises(KeyError):
            list(r.items("hbc_vecs"))
        assert list(r.items(None)) == []                                 # the main database only holds the names


def test_written_environments_round_trip_with_overflow_values_and_deep_trees(tmp_path):
    g = torch.Generator().manual_seed(0)
    rnd = lambda n: bytes(torch.randint(0, 256, (n,), generator=g, dtype=torch.uint8).tolist())
    big = {struct.pack(">Q", i): rnd([24, 700, 2029, 2030, 2031, 5000][i % 6]) for i in range(400)}
    many = {rnd(12): rnd(8) for _ in range(30000)}                       # three levels at 4096-byte pages
    dbs = {"hbc_nodes": big, "hbc_quant": many, "hbc_meta": {b"hbc:meta": b"m" * 50}, "hbc_vecs": {}}
    write_lmdb(str(tmp_path / "env"), dbs)
    with LmdbReader(str(tmp_path / "env")) as r:
        assert r.databases() == sorted(dbs)
        for name, kv in dbs.items():
            got = list(r.items(name))
            assert [k for k, _ in got] == sorted(kv) and all(kv[k] == v for k, v in got)
        for k in list(many)[:200]:
            assert r.get("hbc_quant", k) == many[k]
        assert r.get("hbc_nodes", struct.pack(">Q", 3)) == big[struct.pack(">Q", 3)]
    # small pages force more levels and exercise the same code with other limits
    write_lmdb(str(tmp_path / "env512"), {"d": big}, page_size=512)
    with LmdbReader(str(tmp_path / "env512")) as r:
        assert r.page_size == 512 and dict(r.items("d")) == big
    with pytest.raises(LmdbError):
        write_lmdb(str(tmp_path / "bad"), {"d": {b"": b"x"}})
    with pytest.raises(LmdbError):
        write_lmdb(str(tmp_path / "bad"), {"d": {b"k" * 512: b"x"}})


def test_reader_rejects_files_that_are_not_lmdb(tmp_path):
    (tmp_path / "data.mdb").write_bytes(b"\0" * 8192)
    with pytest.raises(LmdbError):
        LmdbReader(str(tmp_path))
    # a cycle between pages is reported, not followed forever
    write_lmdb(str(tmp_path / "env"), {"d": {struct.pack(">I", i): b"v" * 100 for i in range(500)}})
    raw = bytearray((tmp_path / "env" / "data.mdb").read_bytes())
    with LmdbReader(str(tmp_path / "env")) as r:
        root = r._db_root("d")
    first_ptr = struct.unpack_from("<H", raw, root * 4096 + 16)[0]
    struct.pack_into("<HHH", raw, root * 4096 + first_ptr, root & 0xFFFF, root >> 16, 0)   # child 0 := the root itself
    (tmp_path / "env" / "data.mdb").write_bytes(bytes(raw))
    with LmdbReader(str(tmp_path / "env")) as r, pytest.raises(LmdbError):
        list(r.items("d"))


def test_hbc_index_through_the_lmdb_container(tmp_path):
    from antfly_b200.index import artifact
    from antfly_b200.index.hbc import HBCConfig, HBCIndex

    g = torch.Generator().manual_seed(2)
    x = torch.randn(1200, 24, generator=g)
    idx = HBCIndex.bulk_build(x, HBCConfig(24, "cosine", branching_factor=6, leaf_size=40, search_width=12,
                                           use_quantization=True))
    artifact.save_hbc(idx, str(tmp_path / "a"), container="lmdb")
    artifact.save_hbc(idx, str(tmp_path / "b"), container="files")
    assert sorted(os.listdir(tmp_path / "a")) == ["data.mdb", "lock.mdb"]
    with LmdbReader(str(tmp_path / "a")) as r:
        assert sorted(r.databases()) == ["hbc_meta", "hbc_nodes", "hbc_quant", "hbc_vecs"]
        assert artifact.unpack_metadata(r.get("hbc_meta", artifact.META_KEY))["dims"] == 24
        assert r.entries("hbc_nodes") == len(idx.nodes) and r.entries("hbc_vecs") == 2 * 1200
    a, b = artifact.load_hbc(str(tmp_path / "a")), artifact.load_hbc(str(tmp_path / "b"))
    assert a.stats() == b.stats() == idx.stats()
    for q in x[:5]:
        assert a.search(q, 8)[0] == b.search(q, 8)[0] == idx.search(q, 8)[0]
    with pytest.raises(FileNotFoundError):
        artifact.load_hbc(str(tmp_path))
