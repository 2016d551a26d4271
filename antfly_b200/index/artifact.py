"""Index artifacts on disk.

(1) HBC records in the reference's key/value layout (zig/lib/vectorindex/src/hbc.zig:20-198,
store.zig:23-28): four ordered namespaces ``nodes, meta, quant, vecs``; metadata key ``hbc:meta`` holding a 50-byte
little-endian record {version u32 = 1, dims u32, branching_factor u32, leaf_size u32, root_node u64,
active_count u64, node_count u64, use_quantization u8, quantizer_seed u64, metric u8}; node keys
``n:<u64 BE id>:<suffix>`` with the packed node value ``HBN1`` + header {is_leaf u8, level u16, parent u64} +
centroid_len u32 + ids_len u32 + centroid f32s + ids u64s; ``v:<id>`` raw f32 vector; ``l:<id>`` vector -> leaf.
The namespaces are persisted either as one sorted key/value file each, or as the named databases ``hbc_nodes``,
``hbc_meta``, ``hbc_quant``, ``hbc_vecs`` of an LMDB environment, the container the reference's default storage
backend uses (zig/pkg/antfly/src/storage/hbc_adapter.zig:1435-1438; formats/lmdb_io.py reads and writes the file
format), so an index directory written by either side opens on the other.
(2) GPU index shards (flat / IVF) as safetensors bundles: centroids, posting offsets, sorted vectors, ids.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, Tuple

import torch

from ..formats import safetensors_io as ST
from .hbc import HBCConfig, HBCIndex, Node

META_KEY = b"hbc:meta"
_METRICS = {"l2_squared": 0, "inner_product": 1, "cosine": 2}
_METRIC_NAMES = {v: k for k, v in _METRICS.items()}
_META = struct.Struct("<IIIIQQQBQB")
assert _META.size == 50


def pack_metadata(cfg: HBCConfig, root: int, active: int, nodes: int) -> bytes:
    return _META.pack(1, cfg.dims, cfg.branching_factor, cfg.leaf_size, root, active, nodes,
                      1 if cfg.use_quantization else 0, cfg.quantizer_seed, _METRICS[cfg.metric])


def unpack_metadata(b: bytes) -> dict:
    v, dims, bf, ls, root, active, nodes, uq, seed, metric = _META.unpack(b)
    if v != 1:
        raise ValueError(f"unsupported HBC metadata version {v}")
    return {"dims": dims, "branching_factor": bf, "leaf_size": ls, "root_node": root, "active_count": active,
            "node_count": nodes, "use_quantization": bool(uq), "quantizer_seed": seed, "metric": _METRIC_NAMES[metric]}


def node_key(node_id: int, suffix: str) -> bytes:
    return b"n:" + struct.pack(">Q", node_id) + b":" + suffix.encode()


def pack_node(nd: Node) -> bytes:
    c = nd.centroid.detach().float().cpu()
    ids = [int(i) for i in nd.children]
    return (b"HBN1" + struct.pack("<BHQ", 1 if nd.is_leaf else 0, nd.level, nd.parent) +
            struct.pack("<II", c.numel(), len(ids)) + c.numpy().astype("<f4").tobytes() +
            struct.pack(f"<{len(ids)}Q", *ids))


def unpack_node(node_id: int, b: bytes) -> Node:
    if b[:4] != b"HBN1":
        raise ValueError("bad packed node magic")
    is_leaf, level, parent = struct.unpack_from("<BHQ", b, 4)
    cl, il = struct.unpack_from("<II", b, 15)
    off = 23
    cent = torch.frombuffer(bytearray(b[off:off + 4 * cl]), dtype=torch.float32).clone()
    off += 4 * cl
    ids = list(struct.unpack_from(f"<{il}Q", b, off))
    return Node(node_id, bool(is_leaf), level, parent, cent, ids)


# ----------------------------------------------------------------------------------------------------------
# Quantised payloads: protobuf wire format of RaBitQuantizedVectorSet / NonQuantizedVectorSet
# (go/pkg/antfly/lib/vector/quantize/quantize.proto, zig/lib/vector/src/proto.zig:38-200).  Scalars repeat packed
# (edition 2023 default): floats as fixed32, uint64 code words and uint32 counts as varints.
# ----------------------------------------------------------------------------------------------------------
def _varint(v: int) -> bytes:
    v &= (1 << 64) - 1
    out = bytearray()
    while True:
        b7 = v & 0x7F
        v >>= 7
        out.append(b7 | (0x80 if v else 0))
        if not v:
            return bytes(out)


def _read_varint(b: bytes, pos: int) -> Tuple[int, int]:
    v, shift = 0, 0
    while True:
        c = b[pos]
        pos += 1
        v |= (c & 0x7F) << shift
        if not c & 0x80:
            return v, pos
        shift += 7
        if shift > 63:
            raise ValueError("varint too long")


def _field(num: int, wire: int, payload: bytes) -> bytes:
    head = _varint(num << 3 | wire)
    return head + (_varint(len(payload)) if wire == 2 else b"") + payload


def _floats(t: torch.Tensor) -> bytes:
    return t.detach().float().cpu().contiguous().numpy().astype("<f4").tobytes()


def encode_rabitq_set(qs) -> bytes:
    """RaBitQSet -> RaBitQuantizedVectorSet bytes."""
    n, width = qs.codes.shape
    words = qs.codes.detach().cpu().reshape(-1).tolist()
    codes = _field(1, 0, _varint(n)) + _field(2, 0, _varint(width)) + _field(3, 2, b"".join(_varint(w) for w in words))
    out = b""
    m = _METRICS[qs.metric]
    if m:
        out += _field(1, 0, _varint(m))
    out += _field(2, 2, _floats(qs.centroid)) + _field(3, 2, codes)
    out += _field(4, 2, b"".join(_varint(int(c)) for c in qs.code_counts.tolist()))
    out += _field(5, 2, _floats(qs.centroid_distances)) + _field(6, 2, _floats(qs.inv_dot))
    if qs.centroid_dot is not None:
        out += _field(7, 2, _floats(qs.centroid_dot))
    if qs.centroid_norm:
        out += _field(8, 5, struct.pack("<f", float(qs.centroid_norm)))
    return out


def _parse(b: bytes):
    pos = 0
    while pos < len(b):
        key, pos = _read_varint(b, pos)
        num, wire = key >> 3, key & 7
        if wire == 0:
            v, pos = _read_varint(b, pos)
        elif wire == 2:
            n, pos = _read_varint(b, pos)
            v, pos = b[pos:pos + n], pos + n
        elif wire == 5:
            v, pos = b[pos:pos + 4], pos + 4
        elif wire == 1:
            v, pos = b[pos:pos + 8], pos + 8
        else:
            raise ValueError(f"unsupported wire type {wire}")
        yield num, wire, v


def _unpack_floats(b: bytes) -> torch.Tensor:
    return torch.frombuffer(bytearray(b), dtype=torch.float32).clone() if b else torch.zeros(0)


def _unpack_varints(b: bytes) -> list:
    out, pos = [], 0
    while pos < len(b):
        v, pos = _read_varint(b, pos)
        out.append(v)
    return out


def decode_rabitq_set(b: bytes):
    from .rabitq import RaBitQSet

    f: Dict[int, object] = {}
    for num, _wire, v in _parse(b):
        f[num] = v
    count = width = 0
    words: list = []
    for num, _wire, v in _parse(f.get(3, b"")):
        if num == 1:
            count = v
        elif num == 2:
            width = v
        elif num == 3:
            words = _unpack_varints(v)
    if len(words) != count * width:
        raise ValueError("code set size does not match count * width")
    signed = [w - (1 << 64) if w >= 1 << 63 else w for w in words]       # int64 tensor holding the u64 bit pattern
    codes = torch.tensor(signed, dtype=torch.int64).view(count, width) if count else torch.zeros((0, width),
                                                                                                   dtype=torch.int64)
    return RaBitQSet(_METRIC_NAMES[f.get(1, 0)], _unpack_floats(f.get(2, b"")), codes,
                     torch.tensor(_unpack_varints(f.get(4, b"")), dtype=torch.int32), _unpack_floats(f.get(5, b"")),
                     _unpack_floats(f.get(6, b"")), _unpack_floats(f[7]) if 7 in f else None,
                     struct.unpack("<f", f[8])[0] if 8 in f else 0.0)


def encode_vector_set(x: torch.Tensor) -> bytes:
    """NonQuantizedVectorSet{vectors: Set{dims, count, data}} (the root's payload when it is kept exact)."""
    n, d = x.shape
    inner = _field(1, 0, _varint(d)) + _field(2, 0, _varint(n)) + _field(3, 2, _floats(x))
    return _field(1, 2, inner)


def decode_vector_set(b: bytes) -> torch.Tensor:
    """NonQuantizedVectorSet (field 1 wraps the Set) or a bare Set{dims, count, data}, the form of the reference's
    checked-in ``.pbvec`` recall fixtures (zig/lib/vector/src/proto.zig, zig/bench/vectors/recall_common.zig:56)."""
    fields = list(_parse(b))
    if fields and fields[0][0] == 1 and fields[0][1] == 2:
        fields = list(_parse(fields[0][2]))
    f = {num: v for num, _w, v in fields}
    x = _unpack_floats(f.get(3, b""))
    dims, count = int(f.get(1, 0)), int(f.get(2, 0))
    if x.numel() != dims * count:
        raise ValueError("vector set size does not match dims * count")
    return x.view(count, dims)


def _write_ns(path: str, kv: Dict[bytes, bytes]) -> None:
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(kv)))
        for k in sorted(kv):
            f.write(struct.pack("<II", len(k), len(kv[k])) + k + kv[k])


def _read_ns(path: str) -> Dict[bytes, bytes]:
    out = {}
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        for _ in range(n):
            kl, vl = struct.unpack("<II", f.read(8))
            k = f.read(kl)
            out[k] = f.read(vl)
    return out


LMDB_NAMES = {"nodes": "hbc_nodes", "meta": "hbc_meta", "quant": "hbc_quant", "vecs": "hbc_vecs"}


def _namespaces(directory: str) -> Dict[str, Dict[bytes, bytes]]:
    """The four namespaces of an index directory, from whichever container it holds."""
    if os.path.exists(os.path.join(directory, "data.mdb")):
        from ..formats.lmdb_io import LmdbReader

        with LmdbReader(directory) as r:
            have = set(r.databases())
            return {ns: dict(r.items(name)) if name in have else {} for ns, name in LMDB_NAMES.items()}
    if os.path.exists(os.path.join(directory, "MANIFEST")):
        from .lsm_store import LsmStore

        with LsmStore(directory, read_only=True) as store, store.begin_read() as r:
            return {ns: dict(r.items(ns)) for ns in LMDB_NAMES}
    out = {}
    for ns in LMDB_NAMES:
        path = os.path.join(directory, ns + ".kv")
        out[ns] = _read_ns(path) if os.path.exists(path) else {}
    return out


def hbc_rows(index: HBCIndex, known_vectors=()) -> Dict[str, Dict[bytes, bytes]]:
    """Every row of an index, by namespace.  Leaves list their members by vector id (stable under deletes and any
    id order); vectors no leaf holds any more are left out.  ``known_vectors``: ids whose ``v:`` row the caller
    already has (their bytes are not produced again)."""
    import copy

    ids = index.ids.tolist()
    nodes: Dict[bytes, bytes] = {}
    for nd in index.nodes.values():
        if nd.is_leaf:
            nd = copy.copy(nd)
            nd.children = [ids[m] for m in nd.children]
        nodes[node_key(nd.id, "p")] = pack_node(nd)
    live = sorted(index.leaf_of)
    meta = {META_KEY: pack_metadata(index.cfg, index.root, len(live), len(index.nodes))}
    vecs: Dict[bytes, bytes] = {}
    x = index.vectors.detach().float().cpu()
    known = set(known_vectors)
    for i in live:
        vid = int(ids[i])
        if vid not in known:
            vecs[b"v:" + struct.pack(">Q", vid)] = x[i].numpy().astype("<f4").tobytes()
        vecs[b"l:" + struct.pack(">Q", vid)] = struct.pack("<Q", index.leaf_of[i])
    quant = {b"q:" + struct.pack(">Q", nd.id): encode_rabitq_set(nd.quant) for nd in index.nodes.values()
             if getattr(nd, "quant", None) is not None}
    return {"nodes": nodes, "meta": meta, "vecs": vecs, "quant": quant}


def save_hbc(index: HBCIndex, directory: str, container: str = "files") -> None:
    """``container``: "files" (one sorted file per namespace), "lmdb" (one LMDB environment) or "lsm" (a
    log-structured merge store directory, loaded as one sorted table file)."""
    if container not in ("files", "lmdb", "lsm"):
        raise ValueError(f"unknown index container {container!r}")
    os.makedirs(directory, exist_ok=True)
    spaces = hbc_rows(index)
    if container == "lmdb":
        from ..formats.lmdb_io import write_lmdb

        write_lmdb(directory, {LMDB_NAMES[ns]: kv for ns, kv in spaces.items()})
        return
    if container == "lsm":
        from .lsm_store import LsmStore

        with LsmStore(directory, background=False) as store:
            with store.begin_write() as w:                       # rows of an earlier index in this directory go
                for ns in spaces:
                    for k, _ in list(w.open_cursor(ns)):
                        if k not in spaces[ns]:
                            w.delete(ns, k)
            with store.begin_batch("bulk_ingest") as b:
                for ns, kv in spaces.items():
                    for k, v in kv.items():
                        b.put(ns, k, v)
            store.compact(full=True)
        return
    for ns, kv in spaces.items():
        _write_ns(os.path.join(directory, ns + ".kv"), kv)


def load_hbc(directory: str) -> HBCIndex:
    spaces = _namespaces(directory)
    if META_KEY not in spaces["meta"]:
        raise FileNotFoundError(f"{directory}: no HBC index metadata (no *.kv files, LMDB environment or merge store)")
    return load_hbc_from(spaces)


def load_hbc_from(spaces: Dict[str, Dict[bytes, bytes]]) -> HBCIndex:
    """The index from its rows ({namespace: {key: value}})."""
    if META_KEY not in spaces["meta"]:
        raise FileNotFoundError("no HBC index metadata among the rows")
    md = unpack_metadata(spaces["meta"][META_KEY])
    cfg = HBCConfig(md["dims"], md["metric"], md["branching_factor"], md["leaf_size"],
                    use_quantization=md["use_quantization"], quantizer_seed=md["quantizer_seed"])
    idx = HBCIndex(cfg)
    for k, v in spaces["nodes"].items():
        if not k.startswith(b"n:") or not k.endswith(b":p"):
            continue
        nid = struct.unpack(">Q", k[2:10])[0]
        idx.nodes[nid] = unpack_node(nid, v)
    idx.root = md["root_node"]
    vecs = spaces["vecs"]
    vids = sorted(struct.unpack(">Q", k[2:])[0] for k in vecs if k.startswith(b"v:"))
    rows = [torch.frombuffer(bytearray(vecs[b"v:" + struct.pack(">Q", v)]), dtype=torch.float32) for v in vids]
    idx.vectors = torch.stack(rows) if rows else torch.zeros(0, cfg.dims)
    idx.ids = torch.tensor(vids)
    pos = {v: i for i, v in enumerate(vids)}
    leaves = [nd for nd in idx.nodes.values() if nd.is_leaf]
    # leaves list vector ids; files written before that listed row positions (the same thing whenever the ids
    # were 0..n-1), which shows as a member that is no stored id
    by_id = all(m in pos for nd in leaves for m in nd.children)
    for nd in leaves:
        if by_id:
            nd.children = [pos[m] for m in nd.children]
        for m in nd.children:
            idx.leaf_of[m] = nd.id
    if cfg.use_quantization:
        stored = spaces["quant"]
        for nd in idx.nodes.values():
            blob = stored.get(b"q:" + struct.pack(">Q", nd.id))
            pts = None
            if blob is not None:
                nd.quant = decode_rabitq_set(blob)
                if nd.quant.codes.shape[0] != len(nd.children):
                    blob = None                      # stale payload: fall back to re-quantising
                elif cfg.metric == "cosine":
                    pts = idx.vectors[torch.tensor(nd.children)] if nd.is_leaf else torch.stack(
                        [idx.nodes[c].centroid for c in nd.children])
                    nd.quant.data_norms = pts.norm(dim=-1)
            if blob is None:
                pts = idx.vectors[torch.tensor(nd.children)] if nd.is_leaf else torch.stack(
                    [idx.nodes[c].centroid for c in nd.children])
                nd.quant = idx.quantizer.quantize(nd.centroid, pts)
    return idx


def save_ivf(index, path: str) -> None:
    ST.save_file({"centroids": index.centroids, "offsets": index.offsets, "order": index.order, "vectors": index.x},
                 path, {"metric": index.metric, "n_lists": index.n_lists, "kind": "ivf", "id_offset": index.id_offset})


def load_ivf(path: str, device="cuda"):
    from .distance import score_form
    from .flat import FlatIndex
    from .ivf import IVFIndex
    from ..ops import index_ops as IX

    f = ST.SafetensorsFile(path)
    md = f.metadata
    idx = IVFIndex.__new__(IVFIndex)
    idx.metric, idx.form = md["metric"], score_form(md["metric"])
    idx.id_offset = int(md.get("id_offset", 0))
    idx.centroids = f.tensor("centroids").to(device)
    idx.offsets = f.tensor("offsets").to(device)
    idx.order = f.tensor("order").to(device)
    idx.x = f.tensor("vectors").to(device)
    idx.n_lists, idx.n, idx.dim = int(md["n_lists"]), idx.x.shape[0], idx.x.shape[1]
    idx.col_norm = IX.row_sqnorm(idx.x) if idx.form.use_col_norm else None
    idx.centroid_index = FlatIndex(idx.centroids, metric=idx.metric)
    idx.list_sizes = idx.offsets[1:] - idx.offsets[:-1]
    idx.kmeans_iterations = 0
    return idx
