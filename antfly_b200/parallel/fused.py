"""Fused compute + collective path for tensor-parallel decode (peer memory over NVLink / NVSwitch).

One symmetric workspace per rank (``torch.distributed._symmetric_memory``; every rank maps every other rank's copy)
holds (a) the partial-sum slices pushed by the row-parallel GEMMs' epilogues, (b) the MX-fp8 activation rows pushed
by the norm kernels, (c) arrival counters.  The collectives disappear into the kernels around them:

  GEMM -> reduce-scatter   o_proj / down epilogues store each fp32 partial tile into the buffer of the rank that
                           owns the token (mode 3 of ``afb_gemm_mxfp8_tp``) and bump a counter there; the residual +
                           RMSNorm kernel of the owner waits for the counters and sums the slices it already has
                           to read.
  all-gather -> GEMM       that same norm kernel quantises its rows and stores them into every rank's activation
                           buffers; the next column-parallel GEMM (QKV, gate/up, LM head) streams its weight tiles
                           immediately and only waits for the row counter before its first activation load.

For the skinniest batches a one-shot variant halves the number of NVLink hops per collective:

  GEMM -> all-reduce       o_proj / down reduce their split-K slices inside a thread-block cluster (distributed
                           shared memory), round to bf16 and store the tile into slot `rank` of EVERY rank's buffer
                           (``afb_gemm_mxfp8_bcast``);
                           each rank's residual + RMSNorm kernel polls the slots themselves (they hold a sentinel
                           until data lands -- no flags, no fences), sums them in rank order, so the replicated
                           residual stream stays bit-identical on all ranks, and puts the sentinel back; the next
                           column-parallel GEMM reads local activations with no second hop.  Two buffers alternate
                           between the two collectives of a layer.

Counters are re-armed by the last CTA of the consuming kernel, so a CUDA graph of the step replays without host
involvement.  All waits are bounded; an expired wait sets the kernel status word (``_native.status()``).
Transfers are plain peer loads / stores -- no TMA multicast, no multimem.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _native as N
from ..ops import quant as Q
from ..ops.dense import ACT

_c_int = ctypes.c_int
_c_long = ctypes.c_long
_c_float = ctypes.c_float


def _ptr_array(ptrs: List[int]):
    return (ctypes.c_void_p * 8)(*(list(ptrs) + [0] * (8 - len(ptrs))))


class SymmetricWorkspace:
    """Peer-mapped scratch of a tensor-parallel group, carved into named regions with identical offsets on all
    ranks."""

    def __init__(self, rank: int, world: int, device, hidden: int, max_tokens: int = 128, max_slices: int = 8,
                 group=None):
        import torch.distributed._symmetric_memory as symm

        assert max_tokens % world == 0
        self.rank, self.world, self.device = rank, world, device
        self.hidden, self.max_tokens, self.max_slices = hidden, max_tokens, max_slices
        self.tl_max = max_tokens // world
        off = 0

        def region(nbytes):
            nonlocal off
            o = off
            off = (off + nbytes + 1023) // 1024 * 1024
            return o

        self.off_flags = region(4096)
        self.off_parts = region(world * max_slices * self.tl_max * hidden * 4)
        self.off_q0 = region(max_tokens * hidden)
        self.off_q1 = region(max_tokens * hidden)
        tiles = (max_tokens + 127) // 128
        self.sf_bytes = tiles * (hidden // 128) * 512
        self.off_sf0 = region(self.sf_bytes)
        self.off_sf1 = region(self.sf_bytes)
        # one-shot all-reduce: two alternating [world][max_tokens][hidden] bf16 slot buffers
        self.off_bcast = [region(world * max_tokens * hidden * 2) for _ in range(2)]
        # in-kernel arg-max merge: [world][ARGMAX_ROWS] 64-bit keys, zero = empty
        self.off_argmax = region(world * self.ARGMAX_ROWS * 8)
        self.nbytes = off
        group = group or dist.group.WORLD
        self.buf = symm.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.hdl = symm.rendezvous(self.buf, group)
        self.buf.zero_()
        # scale bytes of rows that are never written must still be a valid exponent
        self.local(self.off_sf0, self.sf_bytes).fill_(127)
        self.local(self.off_sf1, self.sf_bytes).fill_(127)
        self.clear_one_shot_slots()
        torch.cuda.synchronize(device)
        dist.barrier(group)
        self.base_ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        # 0 when the buffer is not bound to an NVLink multicast object (what this package asks for)
        self.multicast_ptr = int(getattr(self.hdl, "multicast_ptr", 0) or 0)
        assert self.base_ptrs[rank] == self.buf.data_ptr()

    def clear_one_shot_slots(self) -> None:
        """Puts the 'nothing here yet' sentinel (bf16 -0.0) into every one-shot slot.  Done at construction; the
        consumer kernels restore it after every read, so this is only needed again after a failed step."""
        for off in self.off_bcast:
            self.local(off, self.world * self.max_tokens * self.hidden * 2).view(torch.int16).fill_(-32768)

    def local(self, off: int, nbytes: int) -> torch.Tensor:
        return self.buf[off:off + nbytes]

    def peers(self, off: int):
        return _ptr_array([b + off for b in self.base_ptrs])

    # flag slots (int32 indices inside the flag region)
    PART_FLAGS, PART_ARRIVED, X_READY, X_CONSUMED = 0, 8, 9, 10
    ARGMAX_ROWS = 1024

    def flag_ptr(self, slot: int) -> ctypes.c_void_p:
        return ctypes.c_void_p(self.buf.data_ptr() + self.off_flags + 4 * slot)

    def peer_flag_ptrs(self, slot: int):
        return _ptr_array([b + self.off_flags + 4 * slot for b in self.base_ptrs])


class FusedTp:
    """The three fused operations of a tensor-parallel decode step."""

    def __init__(self, ws: SymmetricWorkspace, terms: int = 2, one_shot: bool = True):
        self.ws, self.terms, self.one_shot = ws, terms, one_shot
        self.rank, self.world = ws.rank, ws.world

    def tokens_per_rank(self, T: int) -> int:
        assert T % self.world == 0 and T <= self.ws.max_tokens
        return T // self.world

    # -- GEMM -> reduce-scatter -----------------------------------------------------------------------------
    def gemm_push(self, x: Q.MxAct, w: Q.Fp8Weight, T: int, split_k: int) -> int:
        """Row-parallel GEMM whose epilogue pushes the partial tiles to the owners.  Returns the slice count."""
        ws = self.ws
        M, K = x.q0.shape
        Nn = w.out_features
        assert Nn == ws.hidden, "row-parallel outputs are hidden-sized"
        lib = N.cuda()
        S = int(lib.afb_mx_effective_splits(_c_int(K), _c_int(max(split_k, 1))))
        assert S <= ws.max_slices
        rc = lib.afb_gemm_mxfp8_tp(
            N.ptr(x.q0), N.ptr(x.q1), N.ptr(x.sf0), N.ptr(x.sf1), N.ptr(w.q), N.ptr(Q.weight_sf_atoms(w)), None, None,
            None, _c_int(M), _c_int(Nn), _c_int(K), _c_int(Nn), _c_int(0), _c_int(0), _c_int(3), _c_int(S),
            _c_int(x.terms), ws.peers(ws.off_parts), ws.peer_flag_ptrs(ws.PART_FLAGS), _c_int(self.world),
            _c_int(self.rank), _c_int(self.tokens_per_rank(T)), _c_int(S), None, _c_int(0), None, N.stream_ptr())
        N.check(rc, "afb_gemm_mxfp8_tp(push)")
        N.count_launch()
        return S

    # -- reduce (own rows) + residual + RMSNorm + all-gather push ---------------------------------------------
    def norm_reduce_gather(self, gamma: torch.Tensor, residual: torch.Tensor, T: int, slices: int, n_out: int,
                           eps: float, gather: bool = True):
        """Waits for every rank's partial slices of this rank's rows, returns the new residual rows [T/world, H]
        and (when ``gather``) leaves the normalised MX rows of all ranks in the gathered activation buffers."""
        ws = self.ws
        tl = self.tokens_per_rank(T)
        H = ws.hidden
        parts = ws.local(ws.off_parts, self.world * slices * tl * H * 4).view(torch.float32)
        sum_out = torch.empty((tl, H), dtype=torch.bfloat16, device=ws.device)
        expected = ((n_out + 127) // 128) * slices
        two = self.terms == 2
        rc = N.cuda().afb_norm_tp(
            None, N.ptr(parts), _c_int(self.world * slices), _c_long(tl * H), _c_int(0), N.ptr(residual), None,
            N.ptr(gamma), None,
            N.ptr(sum_out), None, None, _c_int(tl), _c_int(H), _c_float(eps), _c_int(1), _c_int(0), None, None, None,
            None, ws.flag_ptr(ws.PART_FLAGS), _c_int(self.world), _c_int(expected), ws.flag_ptr(ws.PART_ARRIVED),
            ws.peers(ws.off_q0), ws.peers(ws.off_q1) if two else None, ws.peers(ws.off_sf0),
            ws.peers(ws.off_sf1) if two else None, ws.peer_flag_ptrs(ws.X_READY), _c_int(self.world if gather else 0),
            _c_int(self.rank * tl), N.stream_ptr())
        N.check(rc, "afb_norm_tp")
        N.count_launch()
        return sum_out

    def gathered(self, T: int) -> Q.MxAct:
        ws = self.ws
        H = ws.hidden
        q0 = ws.local(ws.off_q0, T * H).view(T, H)
        sf0 = ws.local(ws.off_sf0, ws.sf_bytes).view(-1, H // 128, 512)
        if self.terms == 2:
            return Q.MxAct(q0, sf0, ws.local(ws.off_q1, T * H).view(T, H), ws.local(ws.off_sf1, ws.sf_bytes).view(
                -1, H // 128, 512))
        return Q.MxAct(q0, sf0)

    # -- all-gather -> GEMM ---------------------------------------------------------------------------------
    def gemm_gathered(self, w: Q.Fp8Weight, T: int, split_k: int = 1, swiglu: bool = False, partials: bool = False,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Column-parallel GEMM on the gathered activations; waits for all T rows to arrive."""
        ws = self.ws
        x = self.gathered(T)
        K, Nn = ws.hidden, w.out_features
        lib = N.cuda()
        dev = ws.device
        if split_k > 1 or partials:
            S = int(lib.afb_mx_effective_splits(_c_int(K), _c_int(max(split_k, 1))))
            mode, ldc = 1, Nn
            out = torch.empty((S, T, Nn), dtype=torch.float32, device=dev) if out is None else out
        elif swiglu:
            S, mode = 1, 2
            out = torch.empty((T, Nn // 2), dtype=torch.bfloat16, device=dev) if out is None else out
            ldc = out.stride(0)
        else:
            S, mode = 1, 0
            out = torch.empty((T, Nn), dtype=torch.bfloat16, device=dev) if out is None else out
            ldc = out.stride(0)
        rc = lib.afb_gemm_mxfp8_tp(
            N.ptr(x.q0), N.ptr(x.q1), N.ptr(x.sf0), N.ptr(x.sf1), N.ptr(w.q), N.ptr(Q.weight_sf_atoms(w)), N.ptr(out),
            None, None, _c_int(T), _c_int(Nn), _c_int(K), _c_int(ldc), _c_int(0), _c_int(0), _c_int(mode), _c_int(S),
            _c_int(x.terms), None, None, _c_int(0), _c_int(0), _c_int(0), _c_int(0), ws.flag_ptr(ws.X_READY), _c_int(T),
            ws.flag_ptr(ws.X_CONSUMED), N.stream_ptr())
        N.check(rc, "afb_gemm_mxfp8_tp(gathered)")
        N.count_launch()
        return out

    # -- one-shot: GEMM -> all-reduce (broadcast of the reduced bf16 tile) ------------------------------------
    def gemm_bcast(self, x: Q.MxAct, w: Q.Fp8Weight, T: int, split_k: int, buf: int) -> None:
        """Row-parallel GEMM whose reduced bf16 tiles land in slot ``rank`` of every rank's buffer ``buf``.
        No flag accompanies the data: the consumer polls the slots themselves."""
        ws = self.ws
        M, K = x.q0.shape
        Nn = w.out_features
        assert Nn == ws.hidden and M == T and T <= ws.max_tokens
        lib = N.cuda()
        S = int(lib.afb_mx_effective_splits(_c_int(K), _c_int(max(split_k, 1))))
        assert S <= 8
        rc = lib.afb_gemm_mxfp8_bcast(
            N.ptr(x.q0), N.ptr(x.q1), N.ptr(x.sf0), N.ptr(x.sf1), N.ptr(w.q), N.ptr(Q.weight_sf_atoms(w)),
            _c_int(M), _c_int(Nn), _c_int(K), _c_int(Nn), _c_int(S), _c_int(x.terms), ws.peers(ws.off_bcast[buf]),
            _c_int(self.world), _c_int(self.rank), N.stream_ptr())
        N.check(rc, "afb_gemm_mxfp8_bcast")
        N.count_launch()

    def norm_bcast(self, gamma: torch.Tensor, residual: torch.Tensor, T: int, eps: float, buf: int,
                   want_norm: bool = True):
        """Polls the world's slots of buffer ``buf`` until every element has landed, sums them in rank order with
        the (replicated) residual, restores the slots' sentinel, and returns (new residual [T, H] bf16, normalised rows as MX activations or None)."""
        ws = self.ws
        H = ws.hidden
        parts = ws.local(ws.off_bcast[buf], self.world * T * H * 2).view(torch.bfloat16)
        sum_out = torch.empty((T, H), dtype=torch.bfloat16, device=ws.device)
        mx = Q.new_mx(T, H, self.terms, ws.device) if want_norm else None
        rc = N.cuda().afb_norm_tp(
            None, N.ptr(parts), _c_int(self.world), _c_long(T * H), _c_int(2), N.ptr(residual), None, N.ptr(gamma),
            None, N.ptr(sum_out), None, None, _c_int(T), _c_int(H), _c_float(eps), _c_int(1), _c_int(0),
            N.ptr(mx.q0 if mx else None), N.ptr(mx.q1 if mx else None), N.ptr(mx.sf0 if mx else None),
            N.ptr(mx.sf1 if mx else None), None, _c_int(0), _c_int(0), None, None, None, None, None, None, _c_int(0),
            _c_int(0), N.stream_ptr())
        N.check(rc, "afb_norm_tp(bcast)")
        N.count_launch()
        return sum_out, mx

    # -- vocabulary-sharded arg-max merged across ranks inside the kernel ---------------------------------------
    def argmax(self, logits: torch.Tensor, vocab_offset: int) -> torch.Tensor:
        from ..ops import sampling as S

        ws = self.ws
        assert logits.shape[0] <= ws.ARGMAX_ROWS
        return S.argmax_tp(logits, vocab_offset, ws.peers(ws.off_argmax), self.world, self.rank, ws.ARGMAX_ROWS)

    # -- pre-flight -------------------------------------------------------------------------------------------------
    def self_check(self, group=None) -> bool:
        """Runs each fused hand-off once on small random data with a host synchronise in between and compares it
        with the same arithmetic done through NCCL: row-parallel GEMM -> all-reduce -> residual + RMSNorm, and the
        sharded arg-max merge.  Returns True only if every rank saw matching results and no wait expired.  Meant
        to be called once before a serving loop or a benchmark commits to the fused path; a missing or misbehaving
        rank costs one wait limit here instead of wedging a queue of graphs."""
        ws = self.ws
        dev, H = ws.device, ws.hidden
        T, K = 16, 256
        ok = True
        try:
            g = torch.Generator(device=dev).manual_seed(1000 + self.rank)
            x = (torch.randn(T, K, generator=g, device=dev) * 0.5).to(torch.bfloat16)
            w = Q.random_fp8(H, K, dev, seed=77 + self.rank)
            gamma = torch.ones(H, dtype=torch.bfloat16, device=dev)
            residual = torch.zeros((T, H), dtype=torch.bfloat16, device=dev)
            xq = Q.quantize_mx(x, terms=self.terms)
            local = Q.gemm_mxfp8(xq, w).float()                       # this rank's partial product, bf16-rounded
            want = local.clone()
            dist.all_reduce(want, group=group)
            for buf in (0, 1):
                self.gemm_bcast(xq, w, T, 1, buf)
                got, _ = self.norm_bcast(gamma, residual, T, 1e-5, buf)
                torch.cuda.synchronize(dev)
                err = float((got.float() - want).abs().max())
                ok = ok and err <= 0.05 * max(1.0, float(want.abs().max()))
            V = 4096
            logits = torch.randn(T, V, generator=g, device=dev)  # fp32: ties between ranks are negligible
            tok = self.argmax(logits, self.rank * V)
            vals = logits.float().max(-1)
            all_v = [torch.empty_like(vals.values) for _ in range(self.world)]
            all_i = [torch.empty_like(vals.indices) for _ in range(self.world)]
            dist.all_gather(all_v, vals.values.contiguous(), group=group)
            dist.all_gather(all_i, (vals.indices + self.rank * V).contiguous(), group=group)
            av, ai = torch.stack(all_v), torch.stack(all_i)
            best = av.max(0).values
            want_tok = torch.where(av == best[None], ai, torch.full_like(ai, 2 ** 40)).min(0).values
            torch.cuda.synchronize(dev)
            ok = ok and bool(torch.equal(tok.long(), want_tok.long()))
            ok = ok and N.status() == 0
        except Exception:
            ok = False
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if int(flag.item()) == 0:
            N.status()  # clear whatever the failed attempt recorded
            ws.clear_one_shot_slots()
            ws.local(ws.off_argmax, self.world * ws.ARGMAX_ROWS * 8).zero_()
            torch.cuda.synchronize(dev)
            dist.barrier(group=group)
            return False
        return True
