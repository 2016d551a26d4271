"""Property tests (hypothesis): parsers and packers hold their invariants on arbitrary inputs and fail only in the
ways they document -- the counterpart of the reference's codec-corpus / fuzz tier."""
import os
import struct

import numpy as np
import pytest
import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from antfly_b200.finetune.data import TokenExample, pack_examples
from antfly_b200.formats import gguf as GG
from antfly_b200.formats import safetensors_io as ST
from antfly_b200.index.docfilter import compile_filter
from antfly_b200.pipelines.chunking import chunk_text, merge_vad_frames

FAST = settings(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.too_slow])


@FAST
@given(st.text(alphabet=st.characters(blacklist_categories=("Cs",)), max_size=600), st.integers(4, 60), st.integers(0, 3))
def test_chunks_are_spans_of_the_source_in_order(text, target, overlap):
    chunks = chunk_text(text, target_tokens=target, overlap_tokens=overlap)
    last_start = -1
    for i, c in enumerate(chunks):
        assert c["id"] == i and text[c["start_char"]:c["end_char"]] == c["text"] and c["text"]
        assert c["start_char"] >= last_start
        last_start = c["start_char"]
    if text.strip():
        assert chunks and chunks[0]["start_char"] <= len(text) - len(text.lstrip()) + 1
    assert len(chunks) <= 50


@FAST
@given(st.text(max_size=80))
def test_filter_strings_always_compile_and_evaluate(q):
    f = compile_filter(q)
    assert f({"a": 1, "text": "some words", "tags": ["x"], "n": None}) in (True, False)


@FAST
@given(st.lists(st.integers(1, 40), min_size=1, max_size=30), st.integers(40, 64))
def test_packing_places_every_example_once_within_the_row_length(lengths, row):
    ex = [TokenExample(list(range(n)), [1] * n) for n in lengths]
    rows = pack_examples(ex, row, pad_id=0)
    seen = sorted(i for r in rows for i in r["examples"])
    assert seen == list(range(len(ex)))
    for r in rows:
        assert len(r["ids"]) == len(r["loss_mask"]) == len(r["doc_ids"]) == row
        used = sum(lengths[i] for i in r["examples"])
        assert used <= row and sum(r["loss_mask"]) == used
        assert r["doc_ids"][:used] == [d for d, i in enumerate(r["examples"]) for _ in range(lengths[i])]
    assert sum(lengths) <= len(rows) * row and (len(rows) - 1) * row < 2 * sum(lengths) + row   # not wasteful


@FAST
@given(st.lists(st.floats(0, 1), max_size=200), st.integers(0, 500), st.integers(0, 500), st.integers(0, 100),
       st.integers(0, 2000))
def test_vad_segments_are_ordered_disjoint_and_inside_the_recording(probs, sil, speech, pad, cap):
    segs = merge_vad_frames(probs, 512, 16000, 0.5, sil, speech, pad, cap)
    total = len(probs) * 512
    prev = 0
    for a, b in segs:
        assert 0 <= a < b <= total
        assert a >= prev - 2 * (pad * 16) - 1          # padding may make neighbours touch or overlap by the pads
        prev = b
        if cap > 0:
            assert b - a <= cap * 16


@FAST
@given(st.sampled_from(sorted(GG.QUANT_NAMES)), st.integers(0, 2 ** 31 - 1), st.floats(1e-3, 1e3))
def test_quantisers_stay_finite_and_within_the_block_range(name, seed, scale):
    ty = GG.QUANT_NAMES[name]
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal(512) * scale).astype(np.float32)
    x[rng.integers(0, 512, 5)] = 0.0
    raw = GG.quantize(x, ty)
    import ctypes

    from antfly_b200 import _native as N

    back = np.empty_like(x)
    assert N.host().afb_gguf_dequantize(ctypes.c_int(ty), raw.ctypes.data_as(ctypes.c_void_p),
                                        back.ctypes.data_as(ctypes.c_void_p), ctypes.c_long(x.size)) == 0
    assert np.isfinite(back).all()
    for b in range(0, 512, 256):
        amax = np.abs(x[b:b + 256]).max()
        assert np.abs(back[b:b + 256]).max() <= amax * 1.3 + 1e-6
        assert np.abs(back[b:b + 256] - x[b:b + 256]).max() <= amax * (0.75 if name in ("q2_k", "q3_k") else 0.2) + 1e-6


@FAST
@given(st.binary(max_size=200))
def test_broken_safetensors_files_are_refused_not_crashed_on(tmp_path_factory, blob):
    p = str(tmp_path_factory.mktemp("st") / "x.safetensors")
    good = str(tmp_path_factory.mktemp("st") / "good.safetensors")
    ST.save_file({"a": torch.arange(6, dtype=torch.float32).view(2, 3)}, good)
    raw = open(good, "rb").read()
    for data in (blob, raw[: len(raw) // 2], struct.pack("<Q", 10 ** 12) + blob, raw[:8] + blob + raw[8:]):
        with open(p, "wb") as f:
            f.write(data)
        try:
            out = ST.load_file(p)
        except (ValueError, KeyError, OSError, UnicodeDecodeError, struct.error, TypeError, RuntimeError):
            continue
        for t in out.values():
            assert isinstance(t, torch.Tensor)


@settings(max_examples=15, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(st.integers(0, 2 ** 31 - 1))
def test_graph_index_survives_random_inserts_and_deletes(seed):
    from antfly_b200.index.hnsw import HNSWIndex

    rng = np.random.default_rng(seed)
    idx = HNSWIndex(8, "l2_squared", neighbors=4, ef_construction=20, ef_search=20, seed=seed % 1000)
    live = {}
    for _ in range(6):
        ids = rng.integers(0, 60, rng.integers(1, 25)).tolist()
        vecs = rng.standard_normal((len(ids), 8)).astype(np.float32)
        idx.batch_insert(ids, torch.from_numpy(vecs))
        for i, v in zip(ids, vecs):
            live[i] = v
        gone = [i for i in list(live) if rng.random() < 0.3]
        assert idx.delete(gone) == len(gone)
        for i in gone:
            del live[i]
        assert idx.check() == 0 and len(idx) == len(live)
        if live:
            q = torch.from_numpy(rng.standard_normal((3, 8)).astype(np.float32))
            res = idx.search(q, 5, ef=64)
            got = set(res.ids.flatten().tolist()) - {-1}
            assert got <= set(live)
            # an exact hit on a stored vector is found
            k = next(iter(live))
            assert idx.search(torch.from_numpy(live[k])[None], 1, ef=64).ids.item() == k


@settings(max_examples=120, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(st.integers(0, 2), st.integers(0, 2 ** 31 - 1))
def test_corrupt_gguf_files_are_refused_with_value_errors(tmp_path_factory, kind, seed):
    """Truncations, flipped header bytes and overwritten counts: the reader raises ValueError or reads a file whose
    tensors all lie inside it; nothing else escapes."""
    d = tmp_path_factory.mktemp("gguf")
    good = str(d / "good.gguf")
    GG.write_gguf(good, {"general.architecture": "llama", "llama.block_count": 1, "tokenizer.ggml.tokens": ["a", "b"]},
                  {"token_embd.weight": (8, torch.ones(4, 32)), "n.weight": (0, torch.ones(4))})
    raw = bytearray(open(good, "rb").read())
    rng = np.random.default_rng(seed)
    if kind == 0:
        raw = raw[: int(rng.integers(0, len(raw)))]
    elif kind == 1:
        for _ in range(3):
            raw[int(rng.integers(0, min(len(raw), 220)))] = int(rng.integers(0, 256))
    else:
        raw[int(rng.integers(4, 40))] = int(rng.integers(0, 256))
    bad = str(d / "bad.gguf")
    with open(bad, "wb") as f:
        f.write(bytes(raw))
    try:
        f = GG.GGUFFile(bad)
    except ValueError:
        return
    for name, info in f.tensors.items():
        try:
            t = f.tensor(name)
        except (ValueError, NotImplementedError):
            continue
        assert t.numel() == int(np.prod(info.shape)) if info.shape else True


@settings(max_examples=120, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(st.integers(0, 2), st.integers(0, 2 ** 31 - 1))
def test_damaged_lmdb_files_are_refused_with_lmdb_errors(tmp_path_factory, kind, seed):
    """A stock LMDB data file cut short or with bytes overwritten: every read either works or raises LmdbError (a
    database name that no longer decodes may also be reported missing)."""
    import gzip
    import os

    from antfly_b200.formats.lmdb_io import LmdbError, LmdbReader

    raw = bytearray(gzip.open(os.path.join(os.path.dirname(__file__), "data", "lmdb_stock_env.mdb.gz")).read())
    rng = np.random.default_rng(seed)
    if kind == 0:
        raw = raw[: int(rng.integers(1, len(raw)))]
    elif kind == 1:
        for _ in range(int(rng.integers(1, 20))):
            raw[int(rng.integers(0, len(raw)))] = int(rng.integers(0, 256))
    else:
        o = int(rng.integers(0, len(raw) - 64))
        raw[o:o + 64] = bytes(rng.integers(0, 256, 64, dtype=np.uint8))
    bad = str(tmp_path_factory.mktemp("lmdb") / "data.mdb")
    with open(bad, "wb") as f:
        f.write(bytes(raw))
    try:
        with LmdbReader(bad) as r:
            for name in [None] + r.databases():
                for _ in r.items(name):
                    pass
                r.entries(name)
    except (LmdbError, KeyError):
        pass
