"""Bindings of the C++ CPU reference path (``csrc/host/oracle.cpp``): BERT-style encoder forward with pooling and
exact top-k search, in fp32, multithreaded, with no PyTorch in the compute path."""
from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np
import torch

from .. import _native as N


def bert_embed(model, ids: torch.Tensor, type_ids: Optional[torch.Tensor], mask: Optional[torch.Tensor],
               threads: int = 0) -> torch.Tensor:
    """model: antfly_b200.models.bert.BertModel (weights converted to fp32 here); ids/type_ids/mask: [B, S] int."""
    lib = N.host()
    cfg, w = model.cfg, model.w
    f = lambda t: np.ascontiguousarray(t.detach().float().cpu().numpy())
    arrs = [f(w["emb.word"]), f(w["emb.pos"]), f(w["emb.type"]), f(w["emb.ln.g"]), f(w["emb.ln.b"])]
    for l in range(cfg.num_hidden_layers):
        p = f"l{l}."
        for k in ("qkv.w", "qkv.b", "o.w", "o.b", "ln1.g", "ln1.b", "ff1.w", "ff1.b", "ff2.w", "ff2.b", "ln2.g",
                  "ln2.b"):
            arrs.append(f(w[p + k]))
    ptrs = (ctypes.c_void_p * len(arrs))(*[a.ctypes.data for a in arrs])
    B, S = ids.shape
    ii = np.ascontiguousarray(ids.cpu().numpy().astype(np.int32))
    tt = np.ascontiguousarray(type_ids.cpu().numpy().astype(np.int32)) if type_ids is not None else None
    mm = np.ascontiguousarray(mask.cpu().numpy().astype(np.int32)) if mask is not None else None
    out = np.empty((B, cfg.hidden_size), dtype=np.float32)
    if threads:
        lib.afb_cpu_set_threads(ctypes.c_int(threads))
    vp = lambda a: a.ctypes.data_as(ctypes.c_void_p) if a is not None else None
    rc = lib.afb_cpu_bert_embed(ptrs, ctypes.c_int(cfg.num_hidden_layers), ctypes.c_int(cfg.hidden_size),
                                ctypes.c_int(cfg.num_attention_heads), ctypes.c_int(cfg.intermediate_size),
                                ctypes.c_float(cfg.layer_norm_eps), vp(ii), vp(tt), vp(mm), ctypes.c_int(B),
                                ctypes.c_int(S), vp(out))
    assert rc == 0
    return torch.from_numpy(out)


def topk(q: torch.Tensor, x: torch.Tensor, k: int, metric: str = "cosine"):
    lib = N.host()
    qa = np.ascontiguousarray(q.detach().float().cpu().numpy())
    xa = np.ascontiguousarray(x.detach().float().cpu().numpy())
    Qn, D = qa.shape
    idx = np.empty((Qn, k), dtype=np.int32)
    dist = np.empty((Qn, k), dtype=np.float32)
    m = {"l2_squared": 0, "inner_product": 1, "cosine": 2}[metric]
    lib.afb_cpu_topk(qa.ctypes.data_as(ctypes.c_void_p), xa.ctypes.data_as(ctypes.c_void_p), ctypes.c_int(Qn),
                     ctypes.c_long(xa.shape[0]), ctypes.c_int(D), ctypes.c_int(k), ctypes.c_int(m),
                     idx.ctypes.data_as(ctypes.c_void_p), dist.ctypes.data_as(ctypes.c_void_p))
    return torch.from_numpy(idx), torch.from_numpy(dist)
