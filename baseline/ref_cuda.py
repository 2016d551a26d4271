"""Reference arm: a BERT-base forward through the REFERENCE's own CUDA kernels, launched the reference's way.

Nothing from this repository's package is imported here.  The kernels are the unmodified
``inference_cuda_kernels.cu`` of the reference (built by ``baseline/build_ref.py``), loaded as a module through the
CUDA driver API and launched with the grid / block shapes of the reference's launcher
(``zig/pkg/inference/src/ops/cuda/kernels.zig``):

  launch1d     grid ceil(n / 256), block 256                          kernels.zig:1913
  launchBlocks grid = blocks, block = threads                         kernels.zig:1919
  launch2d     grid (gx, gy), block = threads                         kernels.zig:1925
  tiled linear grid (ceil(out / 4), ceil(rows / 2)), block 256        kernels.zig:402-470, chosen when
               rows >= 2, in >= 256, out >= 4                         cuda_compute.zig:573
  attention    block kernel, grid = batch * seq * heads, block 128,
               when seq <= 512 and head_dim <= 128                    kernels.zig:1068-1131

The op sequence is the reference's encoder (``architectures/bert.zig:131-300``): three embedding lookups + two adds
+ LayerNorm; per layer linear q / k / v, scaled-dot-product attention with the int64 key mask (uploaded per call,
``cuda_compute.zig:1050-1084``, head-major flag set as that function sets it), linear, add, LayerNorm, linear,
GELU (element-wise op 3), linear, add, LayerNorm; every op writes a fresh fp32 buffer.  Inputs are padded to
``max_length`` = 512 as the reference's pipelines do by default (``pipelines/embedding.zig:47-51,197-208``) and a
batch is fed in requests of 32 sequences, the pipelines' ``batch_size``: one 256 x 512 call would need a grid of
65,536 in y for the tiled linear, beyond what ``launch2d`` can launch.  The hidden states are downloaded and pooled
on the host (``pipelines/embedding.zig:282-322``; ``bert.zig:125``).

torch is used for device / pinned allocations, events and the host-side pooling only.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Dict, List, Tuple

HERE = os.path.dirname(os.path.abspath(__file__))
CUBIN = os.path.join(HERE, "_ref", "inference_cuda_kernels.sm_100a.cubin")

F32_COL_TILE, F32_ROW_TILE, TILED_THREADS = 4, 2, 256     # kernels.zig f32_col_tile / f32_row_tile / f32_tiled_threads
MAX_LENGTH, PIPELINE_BATCH = 512, 32                       # pipelines/embedding.zig:50-51
OP_ADD, OP_GELU = 0, 3                                     # kernels.zig:1864-1872


# ---- launch geometry (pure arithmetic; unit-tested on CPU against the formulas above) -------------------------
def grid_1d(count: int) -> Tuple[Tuple[int, int, int], int]:
    return ((count + 255) // 256, 1, 1), 256


def grid_blocks(blocks: int, threads: int) -> Tuple[Tuple[int, int, int], int]:
    return (blocks, 1, 1), threads


def grid_tiled_linear(rows: int, out_dim: int) -> Tuple[Tuple[int, int, int], int]:
    return ((out_dim + F32_COL_TILE - 1) // F32_COL_TILE, (rows + F32_ROW_TILE - 1) // F32_ROW_TILE, 1), TILED_THREADS


def linear_uses_tiles(rows: int, in_dim: int, out_dim: int) -> bool:
    return rows >= 2 and in_dim >= 256 and out_dim >= 4


def attention_uses_block_kernel(seq_len: int, head_dim: int) -> bool:
    return seq_len <= 512 and head_dim <= 128


def grid_fits(grid: Tuple[int, int, int]) -> bool:
    """The limits cuLaunchKernel enforces: 2^31 - 1 in x, 65,535 in y and z."""
    return 0 < grid[0] <= 2 ** 31 - 1 and 0 < grid[1] <= 65535 and 0 < grid[2] <= 65535


def request_chunks(n_docs: int, batch: int = PIPELINE_BATCH) -> List[Tuple[int, int]]:
    return [(lo, min(n_docs, lo + batch)) for lo in range(0, n_docs, batch)]


@dataclass
class RefBertConfig:
    vocab_size: int = 30522
    hidden: int = 768
    layers: int = 12
    heads: int = 12
    intermediate: int = 3072
    max_pos: int = 512
    type_vocab: int = 2
    num_labels: int = 0


class RefModule:
    """The reference's kernel module, loaded the way ``KernelModule.load`` does: driver API, one module, functions by
    name."""

    NAMES = ["termite_linear_bias_f32", "termite_linear_bias_f32_tile4_r2", "termite_layer_norm_f32",
             "termite_elementwise_f32", "termite_embedding_lookup_f32", "termite_attention_f32_block",
             "termite_attention_f32"]

    def __init__(self):
        import torch
        from cuda.bindings import driver as cu

        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device")
        if not os.path.exists(CUBIN):
            raise RuntimeError(f"{CUBIN} missing: run python baseline/build_ref.py")
        torch.cuda.init()
        torch.zeros(1, device="cuda")  # primary context current in this thread
        self.cu = cu
        with open(CUBIN, "rb") as f:
            image = f.read()
        err, self.module = cu.cuModuleLoadData(image)
        self._check(err, "cuModuleLoadData")
        self.fn: Dict[str, object] = {}
        for n in self.NAMES:
            err, f_ = cu.cuModuleGetFunction(self.module, n.encode())
            self._check(err, f"cuModuleGetFunction({n})")
            self.fn[n] = f_
        self.launches = 0

    def _check(self, err, what):
        if int(err) != 0:
            raise RuntimeError(f"{what} failed with CUDA driver error {int(err)}")

    def launch(self, name: str, grid, block: int, args, types) -> None:
        import torch

        if not grid_fits(grid):
            raise RuntimeError(f"{name}: grid {grid} exceeds what cuLaunchKernel accepts")
        err, = self.cu.cuLaunchKernel(self.fn[name], grid[0], grid[1], grid[2], block, 1, 1, 0,
                                      torch.cuda.current_stream().cuda_stream, (tuple(args), tuple(types)), 0)
        self._check(err, f"cuLaunchKernel({name})")
        self.launches += 1


P, U32, F32 = ctypes.c_void_p, ctypes.c_uint, ctypes.c_float


class RefBert:
    """Random-init BERT-base weights in the reference's layout (fp32, [out, in] row-major) and the forward above."""

    def __init__(self, cfg: RefBertConfig, seed: int = 0):
        import torch

        self.cfg, self.mod = cfg, RefModule()
        g = torch.Generator(device="cuda").manual_seed(seed)
        dev = "cuda"

        def w(*shape, std=0.02):
            return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * std).contiguous()

        H, I = cfg.hidden, cfg.intermediate
        self.word, self.pos, self.typ = w(cfg.vocab_size, H), w(cfg.max_pos, H), w(cfg.type_vocab, H)
        self.emb_g, self.emb_b = torch.ones(H, device=dev), torch.zeros(H, device=dev)
        self.layers = []
        for _ in range(cfg.layers):
            self.layers.append({
                "q": (w(H, H), w(H)), "k": (w(H, H), w(H)), "v": (w(H, H), w(H)), "o": (w(H, H), w(H)),
                "ln1": (torch.ones(H, device=dev), torch.zeros(H, device=dev)),
                "i": (w(I, H), w(I)), "d": (w(H, I), w(H)),
                "ln2": (torch.ones(H, device=dev), torch.zeros(H, device=dev))})
        self.cls = (w(max(cfg.num_labels, 1), H), w(max(cfg.num_labels, 1))) if cfg.num_labels else None

    # ---- the reference's ops -------------------------------------------------------------------------------------
    def linear(self, x, wb, rows, in_dim, out_dim):
        import torch

        wt, b = wb
        y = torch.empty((rows, out_dim), dtype=torch.float32, device="cuda")
        if linear_uses_tiles(rows, in_dim, out_dim):
            grid, block = grid_tiled_linear(rows, out_dim)
            name = "termite_linear_bias_f32_tile4_r2"
        else:
            grid, block = grid_1d(rows * out_dim)
            name = "termite_linear_bias_f32"
        self.mod.launch(name, grid, block, (y.data_ptr(), x.data_ptr(), wt.data_ptr(), b.data_ptr(), rows, in_dim, out_dim),
                        (P, P, P, P, U32, U32, U32))
        return y

    def elementwise(self, a, b, op):
        import torch

        y = torch.empty_like(a)
        n = a.numel()
        grid, block = grid_1d(n)
        self.mod.launch("termite_elementwise_f32", grid, block,
                        (y.data_ptr(), a.data_ptr(), b.data_ptr() if b is not None else 0, n, op), (P, P, P, U32, U32))
        return y

    def layer_norm(self, x, gb, dim, eps=1e-12):
        import torch

        y = torch.empty_like(x)
        rows = x.numel() // dim
        grid, block = grid_blocks(rows, TILED_THREADS)
        self.mod.launch("termite_layer_norm_f32", grid, block,
                        (y.data_ptr(), x.data_ptr(), gb[0].data_ptr(), gb[1].data_ptr(), rows, dim, eps),
                        (P, P, P, P, U32, U32, F32))
        return y

    def embedding_lookup(self, table, ids_host_i64, total, dim):
        import torch

        ids = ids_host_i64.to("cuda", non_blocking=False)          # uploadTempI64
        y = torch.empty((total, dim), dtype=torch.float32, device="cuda")
        grid, block = grid_1d(total * dim)
        self.mod.launch("termite_embedding_lookup_f32", grid, block, (y.data_ptr(), table.data_ptr(), ids.data_ptr(), total, dim),
                        (P, P, P, U32, U32))
        return y

    def sdpa(self, q, k, v, mask_host_i64, batch, seq, heads, head_dim):
        import torch

        mask = mask_host_i64.to("cuda", non_blocking=False)        # uploaded per call, as sdpaLaunch does
        y = torch.empty_like(q)
        args = (y.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), mask.data_ptr(), 0, batch, seq, heads, head_dim,
                0, 1, 0, 1)
        types = (P, P, P, P, P, P, U32, U32, U32, U32, U32, U32, U32, U32)
        if attention_uses_block_kernel(seq, head_dim):
            grid, block = grid_blocks(batch * seq * heads, 128)
            self.mod.launch("termite_attention_f32_block", grid, block, args, types)
        else:
            grid, block = grid_1d(batch * seq * heads * head_dim)
            self.mod.launch("termite_attention_f32", grid, block, args, types)
        return y

    # ---- forward ---------------------------------------------------------------------------------------------------
    def forward(self, ids_host, mask_host, type_host=None):
        """ids / mask: pinned host int64 [B, S].  Returns the device fp32 hidden states [B * S, H]."""
        import torch

        c = self.cfg
        B, S = ids_host.shape
        total, H = B * S, c.hidden
        x = self.embedding_lookup(self.word, ids_host.reshape(-1), total, H)
        pos_ids = (torch.arange(total, dtype=torch.int64) % S)
        x = self.elementwise(x, self.embedding_lookup(self.pos, pos_ids, total, H), OP_ADD)
        tt = type_host.reshape(-1) if type_host is not None else torch.zeros(total, dtype=torch.int64)
        x = self.elementwise(x, self.embedding_lookup(self.typ, tt, total, H), OP_ADD)
        x = self.layer_norm(x, (self.emb_g, self.emb_b), H)
        hd = H // c.heads
        mask_flat = mask_host.reshape(-1)
        for L in self.layers:
            q = self.linear(x, L["q"], total, H, H)
            k = self.linear(x, L["k"], total, H, H)
            v = self.linear(x, L["v"], total, H, H)
            a = self.sdpa(q, k, v, mask_flat, B, S, c.heads, hd)
            o = self.linear(a, L["o"], total, H, H)
            x1 = self.layer_norm(self.elementwise(o, x, OP_ADD), L["ln1"], H)
            f = self.elementwise(self.linear(x1, L["i"], total, H, c.intermediate), None, OP_GELU)
            d = self.linear(f, L["d"], total, c.intermediate, H)
            x = self.layer_norm(self.elementwise(d, x1, OP_ADD), L["ln2"], H)
        return x

    def embed_request(self, ids_host, mask_host):
        """One pipeline request: forward, download of the hidden states, masked mean pool + L2 normalise on the host
        (the reference's stock path does both on the CPU)."""
        import torch

        B, S = ids_host.shape
        h = self.forward(ids_host, mask_host).view(B, S, self.cfg.hidden)
        host = h.cpu()
        m = mask_host.to(torch.float32)[:, :, None]
        e = (host * m).sum(1) / m.sum(1).clamp_min(1.0)
        return torch.nn.functional.normalize(e, dim=-1)

    def rerank_request(self, ids_host, mask_host, type_host):
        """Cross-encoder request: forward, then the 1-logit head on the [CLS] rows and a sigmoid (host)."""
        import torch

        B, S = ids_host.shape
        h = self.forward(ids_host, mask_host, type_host).view(B, S, self.cfg.hidden)
        cls = h[:, 0, :].contiguous()
        logit = self.linear(cls, self.cls, B, self.cfg.hidden, 1)
        return torch.sigmoid(logit.cpu())


def synthetic_docs(n_docs: int, lo: int, hi: int, vocab=(1000, 30000), seed: int = 0):
    """Token ids uniform in vocab, lengths uniform in [lo, hi], padded to MAX_LENGTH as the reference does; pinned."""
    import torch

    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(lo, hi + 1, (n_docs,), generator=g)
    ids = torch.zeros((n_docs, MAX_LENGTH), dtype=torch.int64)
    mask = torch.zeros((n_docs, MAX_LENGTH), dtype=torch.int64)
    for i, n in enumerate(lens.tolist()):
        ids[i, :n] = torch.randint(vocab[0], vocab[1], (n,), generator=g)
        ids[i, 0], ids[i, n - 1] = 101, 102
        mask[i, :n] = 1
    return ids.pin_memory(), mask.pin_memory(), lens
