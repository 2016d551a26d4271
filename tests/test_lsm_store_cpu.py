"""The log-structured merge store: model-based checks against a dictionary, cursor moves, snapshot isolation,
recovery from the write-ahead log (whole and torn), damaged files, read-only opens, bulk loading, concurrent use."""
import bisect
import os
import random
import threading

import pytest

from antfly_b200.index.lsm_store import LsmError, LsmStore

SMALL = dict(memtable_bytes=8 << 10, block_bytes=512, target_file_bytes=16 << 10, level1_bytes=48 << 10,
             level0_compact_files=3, sync=False)


def _key(i: int) -> bytes:
    return b"k%06d" % i


def _check_against(store: LsmStore, model: dict, ns="vecs"):
    with store.begin_read() as r:
        keys = sorted(model)
        assert [k for k, _ in r.items(ns)] == keys
        for k in keys[:: max(1, len(keys) // 50)]:
            assert r.get(ns, k) == model[k]
        c = r.open_cursor(ns)
        back = []
        e = c.last()
        while e is not None:
            back.append(e[0])
            e = c.prev()
        assert back == keys[::-1]


@pytest.mark.parametrize("background", [False, True])
def test_random_operations_match_a_dictionary_through_flushes_merges_and_reopens(tmp_path, background):
    rng = random.Random(7)
    d = str(tmp_path / "db")
    model = {}
    store = LsmStore(d, background=background, **SMALL)
    for round_ in range(12):
        for _ in range(40):
            with store.begin_write() as w:
                for _ in range(rng.randrange(1, 12)):
                    k = _key(rng.randrange(600))
                    if rng.random() < 0.25:
                        w.delete("vecs", k)
                        model.pop(k, None)
                    else:
                        v = bytes(rng.randrange(256) for _ in range(rng.randrange(0, 120)))
                        w.put("vecs", k, v)
                        model[k] = v
        if round_ % 4 == 1:
            store.flush()
        if round_ % 4 == 2:
            store.compact(full=round_ == 10)
        if round_ % 3 == 0:
            store.close()
            store = LsmStore(d, background=background, **SMALL)
        _check_against(store, model)
    st = store.stats()
    assert st["flushes"] + st["recovered_records"] > 0 and st["last_sequence"] > 0
    store.compact(full=True)
    st = store.stats()
    assert sum(st[f"level{i}_files"] for i in range(6)) >= 1 and st["level0_files"] == 0
    _check_against(store, model)
    store.close()


def test_cursor_moves_agree_with_bisect_over_the_sorted_keys(tmp_path):
    rng = random.Random(3)
    with LsmStore(str(tmp_path / "db"), background=False, **SMALL) as store:
        model = {}
        for chunk in range(6):                                   # rows spread over memory, level 0 and deeper levels
            with store.begin_write() as w:
                for _ in range(150):
                    k = _key(rng.randrange(0, 4000, 3))
                    w.put("nodes", k, k[::-1])
                    model[k] = k[::-1]
                for k in rng.sample(sorted(model), 20):
                    w.delete("nodes", k)
                    del model[k]
            if chunk in (1, 3):
                store.flush()
            if chunk == 2:
                store.compact()
        with store.begin_write() as w:                           # neighbours in other namespaces must stay invisible
            w.put("meta", b"zzzz", b"1")
            w.put("quant", b"", b"empty key")
            w.put("vecs", b"a", b"2")
        keys = sorted(model)
        with store.begin_read() as r:
            c = r.open_cursor("nodes")
            assert c.first() == (keys[0], model[keys[0]]) and c.last() == (keys[-1], model[keys[-1]])
            assert c.next() is None and c.seek_at_or_before(b"a") is None and c.seek_at_or_after(b"z") is None
            for _ in range(300):
                probe = _key(rng.randrange(-5, 4010))
                i = bisect.bisect_left(keys, probe)
                e = c.seek_at_or_after(probe)
                assert (e[0] if e else None) == (keys[i] if i < len(keys) else None)
                if e is not None and rng.random() < 0.5:         # change of direction right after a seek
                    p = c.prev()
                    assert (p[0] if p else None) == (keys[i - 1] if i > 0 else None)
                    if p is not None:
                        assert c.next()[0] == keys[i]
                j = bisect.bisect_right(keys, probe) - 1
                e = c.seek_at_or_before(probe)
                assert (e[0] if e else None) == (keys[j] if j >= 0 else None)
                if e is not None and rng.random() < 0.5:
                    n = c.next()
                    assert (n[0] if n else None) == (keys[j + 1] if j + 1 < len(keys) else None)
            assert r.get("quant", b"") == b"empty key" and list(r.items("quant")) == [(b"", b"empty key")]
            assert r.get_many_sorted("nodes", [keys[0], b"nope", keys[-1]]) == [model[keys[0]], None, model[keys[-1]]]
            assert [k for k, _ in r.items("nodes", prefix=b"k0001")] == [k for k in keys if k.startswith(b"k0001")]


def test_a_read_transaction_keeps_its_view_while_writes_flushes_and_merges_go_on(tmp_path):
    with LsmStore(str(tmp_path / "db"), background=False, **SMALL) as store:
        with store.begin_write() as w:
            for i in range(200):
                w.put("vecs", _key(i), b"old%d" % i)
        r = store.begin_read()
        before = dict(r.items("vecs"))
        for rep in range(3):
            with store.begin_write() as w:
                for i in range(0, 200, 2):
                    w.put("vecs", _key(i), b"new%d-%d" % (rep, i) + b"x" * 100)
                for i in range(1, 200, 10):
                    w.delete("vecs", _key(i))
                w.put("vecs", _key(1000 + rep), b"added")
            if rep == 1:
                store.flush()
        store.compact(full=True)
        assert dict(r.items("vecs")) == before and r.get("vecs", _key(0)) == b"old0" and r.get("vecs", _key(1001)) is None
        assert store.stats()["live_snapshots"] == 1
        r.abort()
        with store.begin_read() as r2:
            assert r2.get("vecs", _key(0)).startswith(b"new2-0") and r2.get("vecs", _key(1)) is None
            assert r2.get("vecs", _key(1001)) == b"added"
        assert store.stats()["live_snapshots"] == 0


def test_a_write_transaction_reads_its_own_writes_and_an_abort_leaves_nothing(tmp_path):
    with LsmStore(str(tmp_path / "db"), background=False, **SMALL) as store:
        with store.begin_write() as w:
            for i in range(0, 20, 2):
                w.put("meta", _key(i), b"base")
        w = store.begin_write()
        w.put("meta", _key(3), b"mine")
        w.put("meta", _key(4), b"changed")
        w.delete("meta", _key(6))
        w.put("meta", _key(99), b"tail")
        assert w.get("meta", _key(3)) == b"mine" and w.get("meta", _key(6)) is None and w.get("meta", _key(8)) == b"base"
        want = [_key(0), _key(2), _key(3), _key(4), _key(8), _key(10), _key(12), _key(14), _key(16), _key(18), _key(99)]
        c = w.open_cursor("meta")
        assert [k for k, _ in c] == want
        assert c.seek_at_or_after(_key(5)) == (_key(8), b"base") and c.prev() == (_key(4), b"changed")
        assert c.seek_at_or_before(_key(7)) == (_key(4), b"changed") and c.next() == (_key(8), b"base")
        assert c.last() == (_key(99), b"tail") and c.next() is None
        back, e = [], c.last()
        while e is not None:
            back.append(e[0])
            e = c.prev()
        assert back == want[::-1]
        with store.begin_read() as r:                            # nothing is visible outside before the commit
            assert r.get("meta", _key(3)) is None and r.get("meta", _key(6)) == b"base"
        w.abort()
        with store.begin_read() as r:
            assert r.get("meta", _key(3)) is None and len(list(r.items("meta"))) == 10
        with pytest.raises(ZeroDivisionError):
            with store.begin_write() as w2:
                w2.put("meta", b"never", b"1")
                1 / 0
        with store.begin_read() as r:
            assert r.get("meta", b"never") is None


def _wal_files(d):
    return sorted(f for f in os.listdir(d) if f.startswith("wal-"))


def test_commits_survive_a_reopen_from_the_log_and_a_torn_tail_loses_only_the_last_commit(tmp_path):
    d = str(tmp_path / "db")
    store = LsmStore(d, background=False, memtable_bytes=1 << 20, sync=True)
    for i in range(30):
        with store.begin_write() as w:
            w.put("vecs", _key(i), b"v%d" % i * 20)
            w.put("meta", b"count", b"%d" % (i + 1))
    assert store.stats()["level0_files"] == 0                    # everything is still only in the log and memory
    store.close()
    (wal,) = _wal_files(d)
    size = os.path.getsize(os.path.join(d, wal))
    with open(os.path.join(d, wal), "r+b") as f:                 # a crash in the middle of the last record
        f.truncate(size - 7)
    store = LsmStore(d, background=False, memtable_bytes=1 << 20, sync=True)
    st = store.stats()
    assert st["recovered_records"] == 29 and st["level0_files"] == 1
    with store.begin_read() as r:
        assert r.get("meta", b"count") == b"29" and r.get("vecs", _key(28)) is not None and r.get("vecs", _key(29)) is None
    assert _wal_files(d) != [wal]                                 # the replayed log is gone, a fresh one is open
    with store.begin_write() as w:
        w.put("vecs", _key(29), b"again")
    store.close()
    with LsmStore(d, read_only=True) as ro:
        with ro.begin_read() as r:
            assert r.get("vecs", _key(29)) == b"again" and r.get("meta", b"count") == b"29"


def test_a_flipped_byte_in_a_log_record_ends_the_replay_there(tmp_path):
    d = str(tmp_path / "db")
    with LsmStore(d, background=False, memtable_bytes=1 << 20) as store:
        for i in range(10):
            with store.begin_write() as w:
                w.put("vecs", _key(i), b"payload-%d" % i)
    (wal,) = _wal_files(d)
    raw = bytearray(open(os.path.join(d, wal), "rb").read())
    raw[len(raw) // 2] ^= 0x40
    open(os.path.join(d, wal), "wb").write(bytes(raw))
    with LsmStore(d, background=False) as store:
        n = store.stats()["recovered_records"]
        assert 0 < n < 10
        with store.begin_read() as r:
            assert [k for k, _ in r.items("vecs")] == [_key(i) for i in range(n)]


def test_damaged_table_files_and_manifests_are_refused_with_an_error(tmp_path):
    d = str(tmp_path / "db")
    with LsmStore(d, background=False, **SMALL) as store:
        with store.begin_write() as w:
            for i in range(500):
                w.put("vecs", _key(i), b"x" * 50)
        store.compact(full=True)
    tables = [f for f in os.listdir(d) if f.endswith(".tbl")]
    assert tables
    path = os.path.join(d, tables[0])
    good = open(path, "rb").read()
    # footer magic, index block, filter: refused at open
    for off in (len(good) - 3, len(good) - 64 - 20):
        bad = bytearray(good)
        bad[off] ^= 0xFF
        open(path, "wb").write(bytes(bad))
        with pytest.raises(LsmError):
            LsmStore(d, background=False)
    open(path, "wb").write(good[: len(good) // 2])
    with pytest.raises(LsmError):
        LsmStore(d, read_only=True)
    # a data block: the file opens, the read that touches the block fails
    bad = bytearray(good)
    bad[len(good) // 3] ^= 0x01
    open(path, "wb").write(bytes(bad))
    with LsmStore(d, read_only=True) as store:
        with store.begin_read() as r:
            with pytest.raises(LsmError, match="checksum"):
                list(r.items("vecs"))
    open(path, "wb").write(good)
    manifest = os.path.join(d, "MANIFEST")
    text = open(manifest).read()
    open(manifest, "w").write(text.replace("seq ", "seq 1", 1))
    with pytest.raises(LsmError, match="MANIFEST"):
        LsmStore(d, background=False)
    open(manifest, "w").write(text)
    with LsmStore(d, background=False) as store:
        with store.begin_read() as r:
            assert len(list(r.items("vecs"))) == 500


def test_one_writer_many_read_only_opens(tmp_path):
    d = str(tmp_path / "db")
    with pytest.raises(LsmError, match="MANIFEST"):
        LsmStore(str(tmp_path / "nothing"), read_only=True)
    with LsmStore(d, background=False, **SMALL) as store:
        with store.begin_write() as w:
            w.put("meta", b"a", b"1")
        with pytest.raises(LsmError, match="another process"):
            LsmStore(d, background=False)
        before = sorted(os.listdir(d))
        with LsmStore(d, read_only=True) as ro:                  # sees the log's content, writes nothing
            with ro.begin_read() as r:
                assert r.get("meta", b"a") == b"1"
            with pytest.raises(LsmError, match="read-only"):
                ro.begin_write()
            with pytest.raises(LsmError, match="read-only"):
                ro.begin_batch()
        assert sorted(os.listdir(d)) == before


def test_bulk_ingest_writes_one_table_file_and_no_log_record(tmp_path):
    d = str(tmp_path / "db")
    with LsmStore(d, background=False, **SMALL) as store:
        with store.begin_write() as w:
            w.put("vecs", _key(5), b"older")
            w.put("vecs", _key(7), b"to be deleted")
        wal_before = store.stats()["wal_records"]
        b = store.begin_batch("bulk_ingest")
        rng = random.Random(1)
        order = list(range(3000))
        rng.shuffle(order)                                       # any order; the engine sorts
        for i in order:
            b.append_put("vecs", _key(i), b"bulk%d" % i)
        b.put("vecs", _key(5), b"bulk wins twice")              # the last write of a key wins
        b.delete("vecs", _key(7))
        assert b.get("vecs", _key(5)) == b"older"                # a batch reads the committed state
        b.commit()
        st = store.stats()
        assert st["ingests"] == 1 and st["wal_records"] == wal_before
        with store.begin_read() as r:
            assert r.get("vecs", _key(5)) == b"bulk wins twice" and r.get("vecs", _key(7)) is None
            assert len(list(r.items("vecs"))) == 2999
    with LsmStore(d, read_only=True) as ro, ro.begin_read() as r:
        assert r.get("vecs", _key(2999)) == b"bulk2999" and r.get("vecs", _key(7)) is None


def test_a_full_merge_drops_deleted_rows_and_filters_skip_files(tmp_path):
    with LsmStore(str(tmp_path / "db"), background=False, **SMALL) as store:
        for lo in (0, 1000, 2000):
            with store.begin_write() as w:
                for i in range(lo, lo + 300):
                    w.put("vecs", _key(i), b"y" * 40)
            store.flush()
        with store.begin_write() as w:
            for i in range(0, 300):
                w.delete("vecs", _key(i))
        store.flush()
        size_before = sum(store.stats()[f"level{i}_bytes"] for i in range(6))
        with store.begin_read() as r:
            for i in range(5000, 5200):                          # absent keys inside no file's range cost nothing;
                assert r.get("vecs", _key(i)) is None
            for i in range(1000, 2300, 7):                       # absent keys inside a range are turned away by filters
                r.get("vecs", _key(i) + b"?")
        assert store.stats()["bloom_skips"] >= 80             # about 86 of the probes fall inside a file
        store.compact(full=True)
        st = store.stats()
        assert st["dropped_tombstones"] == 300 and sum(st[f"level{i}_bytes"] for i in range(6)) < size_before
        with store.begin_read() as r:
            assert len(list(r.items("vecs"))) == 600


def test_writers_and_readers_on_threads_with_background_flushes_and_merges(tmp_path):
    d = str(tmp_path / "db")
    store = LsmStore(d, background=True, **SMALL)
    errors, done = [], threading.Event()

    def writer(t):
        try:
            for i in range(150):
                with store.begin_write() as w:
                    # both rows of a commit carry the same stamp: a reader must never see them differ
                    w.put("vecs", b"pair-a-%d" % t, b"%d" % i)
                    w.put("vecs", b"pair-b-%d" % t, b"%d" % i)
                    w.put("nodes", b"t%d-%05d" % (t, i), b"z" * 200)
        except Exception as e:                                   # pragma: no cover
            errors.append(e)

    def reader():
        try:
            while not done.is_set():
                with store.begin_read() as r:
                    for t in range(3):
                        assert r.get("vecs", b"pair-a-%d" % t) == r.get("vecs", b"pair-b-%d" % t)
                    keys = [k for k, _ in r.items("nodes")]
                    assert keys == sorted(keys)
        except Exception as e:                                   # pragma: no cover
            errors.append(e)

    ws = [threading.Thread(target=writer, args=(t,)) for t in range(3)]
    rs = [threading.Thread(target=reader) for _ in range(2)]
    for t in ws + rs:
        t.start()
    for t in ws:
        t.join()
    done.set()
    for t in rs:
        t.join()
    assert not errors, errors
    st = store.stats()
    assert st["flushes"] > 0 and st["compactions"] > 0
    with store.begin_read() as r:
        assert len(list(r.items("nodes"))) == 450
    store.close()
    with LsmStore(d, read_only=True) as ro, ro.begin_read() as r:
        assert len(list(r.items("nodes"))) == 450 and r.get("vecs", b"pair-a-2") == b"149"


def test_hbc_index_through_the_lsm_container_and_a_rebuild_in_the_same_directory(tmp_path):
    import torch

    from antfly_b200.index import artifact
    from antfly_b200.index.hbc import HBCConfig, HBCIndex

    g = torch.Generator().manual_seed(2)
    x = torch.randn(1200, 24, generator=g)
    cfg = HBCConfig(24, "cosine", branching_factor=6, leaf_size=40, search_width=12, use_quantization=True)
    idx = HBCIndex.bulk_build(x, cfg)
    d = str(tmp_path / "a")
    artifact.save_hbc(idx, d, container="lsm")
    names = os.listdir(d)
    assert "MANIFEST" in names and sum(n.endswith(".tbl") for n in names) == 1
    with LsmStore(d, read_only=True) as store, store.begin_read() as r:
        assert artifact.unpack_metadata(r.get("meta", artifact.META_KEY))["dims"] == 24
        assert len(list(r.items("nodes"))) == len(idx.nodes) and len(list(r.items("vecs"))) == 2 * 1200
        assert len(list(r.items("vecs", prefix=b"v:"))) == 1200
    a = artifact.load_hbc(d)
    assert a.stats() == idx.stats()
    for q in x[:5]:
        assert a.search(q, 8)[0] == idx.search(q, 8)[0]
    small = HBCIndex.bulk_build(x[:300], cfg)                    # a smaller index over the old one: no stale rows
    artifact.save_hbc(small, d, container="lsm")
    b = artifact.load_hbc(d)
    assert b.stats() == small.stats() and b.search(x[0], 5)[0] == small.search(x[0], 5)[0]


def test_an_hbc_index_kept_in_the_store_commits_each_batch_and_reopens_to_the_same_tree(tmp_path):
    import torch

    from antfly_b200.index.hbc import HBCConfig, HBCIndex
    from antfly_b200.index.hbc_store import PersistentHBC

    g = torch.Generator().manual_seed(5)
    x = torch.randn(1500, 16, generator=g)
    cfg = HBCConfig(16, "l2_squared", branching_factor=6, leaf_size=24, search_width=16, use_quantization=True)
    d = str(tmp_path / "idx")
    twin = HBCIndex.bulk_build(x[:800], cfg)                     # the same operations on a plain in-memory index
    p = PersistentHBC.create(d, x[:800], cfg, background=False, sync=False)
    total_rows = sum(len(list(r)) for r in [p._sig]) + len(p._vectors)
    commits = p.store.stats()["wal_records"]
    new_ids = torch.arange(5000, 5300).flip(0)                   # ids in descending order, far from the positions
    twin.insert(x[800:1100], new_ids)
    wrote = p.insert(x[800:1100], new_ids)
    assert p.store.stats()["wal_records"] == commits + 1         # one commit for the whole batch
    small = p.insert(x[1100:1103], torch.tensor([9001, 9002, 9003]))
    twin.insert(x[1100:1103], torch.tensor([9001, 9002, 9003]))
    assert 3 <= small < total_rows // 4 and small < wrote        # a small batch rewrites a small part of the rows
    gone = list(range(0, 400, 3)) + [5000, 5299, 9002]
    assert p.delete(gone) == twin.delete(gone) == len(gone)
    for q in x[1200:1210]:
        assert p.search(q, 10)[0] == twin.search(q, 10)[0]
    want = [twin.search(q, 10) for q in x[1200:1230]]
    stats = twin.stats()
    p.close()
    with PersistentHBC(d, background=False, sync=False) as again:
        assert again.index.stats() == stats
        for q, (ids, dist) in zip(x[1200:1230], want):
            got = again.search(q, 10)
            assert got[0] == ids and got[1] == pytest.approx(dist, rel=1e-5, abs=1e-5)
        assert not set(gone) & set(again.index.ids.tolist())    # deleted vectors left the store too
        with again.store.begin_read() as r:
            assert r.get("vecs", b"v:" + (5000).to_bytes(8, "big")) is None
            assert r.get("vecs", b"v:" + (5001).to_bytes(8, "big")) is not None
        again.insert(x[1300:1310], torch.arange(20000, 20010))
        after = [again.search(q, 5)[0] for q in x[1300:1310]]
        twin.insert(x[1300:1310], torch.arange(20000, 20010))
        assert after == [twin.search(q, 5)[0] for q in x[1300:1310]]     # the reloaded tree behaves as the original
    with PersistentHBC(d, background=False, sync=False) as third:
        assert 20005 in third.index.ids.tolist() and [third.search(q, 5)[0] for q in x[1300:1310]] == after
    with pytest.raises(FileNotFoundError):
        PersistentHBC(str(tmp_path / "nothing"))


def test_random_damage_to_any_file_of_a_store_gives_an_error_or_a_working_store(tmp_path):
    import shutil

    good = str(tmp_path / "good")
    opts = dict(SMALL, background=False)
    with LsmStore(good, **opts) as s:
        for rep in range(5):
            with s.begin_write() as w:
                for i in range(300):
                    w.put("vecs", b"k%05d" % ((i * 7 + rep * 13) % 1500), bytes([rep]) * 40)
                for i in range(0, 300, 9):
                    w.delete("vecs", b"k%05d" % i)
            if rep in (1, 3):
                s.flush()
        s.compact()
        with s.begin_write() as w:
            w.put("meta", b"tail", b"in the log only")
    files = [f for f in sorted(os.listdir(good)) if f != "LOCK"]
    assert any(f.endswith(".tbl") for f in files) and any(f.startswith("wal-") for f in files)
    rng = random.Random(11)
    outcomes = set()
    for case in range(45):
        d = str(tmp_path / "bad")
        shutil.rmtree(d, ignore_errors=True)
        shutil.copytree(good, d)
        name = files[case % len(files)]
        raw = bytearray(open(os.path.join(d, name), "rb").read())
        if not raw:
            continue
        mode = case // len(files) % 3
        if mode == 0:
            raw = raw[: rng.randrange(0, len(raw))]
        elif mode == 1:
            for _ in range(rng.randrange(1, 6)):
                raw[rng.randrange(len(raw))] ^= 1 + rng.randrange(255)
        else:
            o = rng.randrange(len(raw))
            raw[o:o + 32] = bytes(rng.randrange(256) for _ in range(min(32, len(raw) - o)))
        open(os.path.join(d, name), "wb").write(bytes(raw))
        try:
            with LsmStore(d, read_only=case % 2 == 0, **opts) as s:
                with s.begin_read() as r:
                    keys = [k for k, _ in r.items("vecs")]
                    assert keys == sorted(keys)
                    c = r.open_cursor("vecs")
                    e = c.last()
                    while e is not None:
                        e = c.prev()
                if case % 2:
                    with s.begin_write() as w:
                        w.put("vecs", b"new", b"1")
                    s.compact(full=True)
            outcomes.add(("ok", name.split(".")[-1]))
        except LsmError:
            outcomes.add(("refused", name.split(".")[-1]))
    assert ("refused", "tbl") in outcomes and ("refused", "MANIFEST") in outcomes and ("ok", "log") in outcomes
