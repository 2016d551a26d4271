"""GGUF v3 reader: magic ``GGUF``, typed metadata key/values (13 value types), tensor directory, 32-byte aligned
data section (zig/pkg/inference/src/gguf/format.zig:18-60).  Tensor payloads are dequantised by the C++ codecs
(``csrc/host/codecs.cpp``) for F32 / F16 / BF16 / Q8_0 / Q4_0 / Q4_K / MXFP4; other encodings are listed in the
directory and reported as unsupported when asked for.  A small writer exists for tests and for exporting."""
from __future__ import annotations

import ctypes
import mmap
import struct
from dataclasses import dataclass
from typing import Optional, Any, Dict, List, Tuple

import numpy as np
import torch

from .. import _native as N

GGUF_MAGIC = b"GGUF"
TYPE_NAMES = {0: "F32", 1: "F16", 2: "Q4_0", 3: "Q4_1", 6: "Q5_0", 7: "Q5_1", 8: "Q8_0", 9: "Q8_1", 10: "Q2_K",
              11: "Q3_K", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K", 15: "Q8_K", 16: "IQ2_XXS", 17: "IQ2_XS", 18: "IQ3_XXS",
              19: "IQ1_S", 20: "IQ4_NL", 21: "IQ3_S", 22: "IQ2_S", 23: "IQ4_XS", 24: "I8", 25: "I16", 26: "I32",
              27: "I64", 28: "F64", 29: "IQ1_M", 30: "BF16", 34: "TQ1_0", 35: "TQ2_0", 36: "I2_S", 37: "I8_S", 38: "TL1", 39: "MXFP4",
              40: "NVFP4", 41: "Q1_0"}
SUPPORTED = {0, 1, 2, 3, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16, 17, 18, 19, 20, 21, 22, 23, 24, 25, 26, 27, 28, 29, 30,
             34, 35, 36, 37, 39, 40, 41}
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}


@dataclass
class GGUFTensorInfo:
    name: str
    shape: Tuple[int, ...]  # row-major (outermost first)
    type: int
    offset: int

    @property
    def type_name(self) -> str:
        return TYPE_NAMES.get(self.type, f"type{self.type}")


class GGUFFile:
    def __init__(self, path: str):
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        mm = self._mm
        if mm[:4] != GGUF_MAGIC:
            raise ValueError(f"{path}: not a GGUF file")
        try:
            self._parse(mm)
        except (struct.error, OverflowError, IndexError, MemoryError, RecursionError) as e:
            raise ValueError(f"{path}: truncated or corrupt GGUF header ({type(e).__name__}: {e})") from e
        # every tensor must lie inside the file: a directory that points past the end is refused here, not when a
        # kernel reads the bytes
        lib = N.host()
        lib.afb_gguf_block_bytes.restype = ctypes.c_long
        lib.afb_gguf_block_values.restype = ctypes.c_long
        for info in self.tensors.values():
            n = 1
            for d in info.shape:
                n *= int(d)
            bv, bb = int(lib.afb_gguf_block_values(info.type)), int(lib.afb_gguf_block_bytes(info.type))
            if bv > 0 and bb > 0 and (n < 0 or self.data_start + info.offset + (n // bv) * bb > len(mm)):
                raise ValueError(f"{path}: tensor {info.name!r} extends past the end of the file")

    def _parse(self, mm) -> None:
        self.version, n_tensors, n_kv = struct.unpack_from("<IQQ", mm, 4)
        if n_tensors > len(mm) or n_kv > len(mm):             # each entry takes at least a few bytes
            raise ValueError("GGUF header counts exceed the file size")
        self._pos = 24
        self.metadata: Dict[str, Any] = {}
        for _ in range(n_kv):
            key = self._string()
            (vt,) = struct.unpack_from("<I", mm, self._pos)
            self._pos += 4
            self.metadata[key] = self._value(vt)
        self.tensors: Dict[str, GGUFTensorInfo] = {}
        for _ in range(n_tensors):
            name = self._string()
            (nd,) = struct.unpack_from("<I", mm, self._pos)
            self._pos += 4
            if nd > 8:
                raise ValueError(f"tensor {name!r} declares {nd} dimensions")
            dims = struct.unpack_from(f"<{nd}Q", mm, self._pos)
            self._pos += 8 * nd
            ty, off = struct.unpack_from("<IQ", mm, self._pos)
            self._pos += 12
            self.tensors[name] = GGUFTensorInfo(name, tuple(reversed(dims)), ty, off)
        align = self.metadata.get("general.alignment", 32)
        if not isinstance(align, int) or align <= 0 or align > (1 << 20):
            raise ValueError(f"bad general.alignment {align!r}")
        self.data_start = (self._pos + align - 1) // align * align

    def _string(self) -> str:
        (n,) = struct.unpack_from("<Q", self._mm, self._pos)
        if self._pos + 8 + n > len(self._mm):
            raise ValueError("string runs past the end of the file")
        s = self._mm[self._pos + 8:self._pos + 8 + n].decode("utf-8", errors="replace")
        self._pos += 8 + n
        return s

    def _value(self, vt: int):
        if vt in _SCALARS:
            fmt = _SCALARS[vt]
            (v,) = struct.unpack_from(fmt, self._mm, self._pos)
            self._pos += struct.calcsize(fmt)
            return v
        if vt == 8:
            return self._string()
        if vt == 9:
            et, n = struct.unpack_from("<IQ", self._mm, self._pos)
            self._pos += 12
            if n > len(self._mm) - self._pos:                  # every element takes at least one byte
                raise ValueError("array runs past the end of the file")
            return [self._value(et) for _ in range(n)]
        raise ValueError(f"unknown GGUF metadata value type {vt}")

    def tensor(self, name: str) -> torch.Tensor:
        """Dequantised fp32 tensor."""
        info = self.tensors[name]
        bitnet = str(self.metadata.get("general.architecture", "")) in ("bitnet", "bitnet-b1.58")
        if info.type == 38 or (info.type == 39 and bitnet):
            # BitNet lookup-table layouts: whole-tensor tilings, not block formats (formats/bitnet_tl.py)
            from . import bitnet_tl as TL

            if len(info.shape) != 2:
                raise NotImplementedError("TL1 / TL2 tensors are matrices")
            rows, cols = info.shape
            nbytes = TL.tl1_nbytes(rows, cols) if info.type == 38 else TL.tl2_nbytes(rows, cols)
            src = np.frombuffer(self._mm, dtype=np.uint8, count=nbytes, offset=self.data_start + info.offset)
            fn = TL.dequantize_tl1 if info.type == 38 else TL.dequantize_tl2
            return torch.from_numpy(fn(src, rows, cols))
        if info.type not in SUPPORTED:
            raise NotImplementedError(f"GGUF tensor type {info.type_name} is not supported")
        lib = N.host()
        lib.afb_gguf_block_bytes.restype = ctypes.c_long
        lib.afb_gguf_block_values.restype = ctypes.c_long
        n = int(np.prod(info.shape)) if info.shape else 1
        bv, bb = lib.afb_gguf_block_values(info.type), lib.afb_gguf_block_bytes(info.type)
        start = self.data_start + info.offset
        if info.type == 36:
            # BitNet I2_S: whole 128-value blocks (the last one padded), then the tensor's fp32 scale at byte n / 4
            # of a 32-byte tail (zig/pkg/inference/src/gguf/tensor_types.zig:248 byteLen)
            padded = -(-n // bv) * bv
            src = np.frombuffer(self._mm, dtype=np.uint8, count=padded // bv * bb, offset=start)
            full = np.empty(padded, dtype=np.float32)
            rc = lib.afb_gguf_dequantize(ctypes.c_int(36), src.ctypes.data_as(ctypes.c_void_p),
                                         full.ctypes.data_as(ctypes.c_void_p), ctypes.c_long(padded))
            if rc != 0:
                raise NotImplementedError("GGUF tensor type I2_S is not supported")
            out = full[:n].copy()
            tail = start + -(-n // 4)
            if tail + 4 <= len(self._mm):
                scale = float(np.frombuffer(self._mm, dtype="<f4", count=1, offset=tail)[0])
                if np.isfinite(scale) and scale != 0.0:
                    out *= scale
            return torch.from_numpy(out).view(info.shape)
        nbytes = n // bv * bb
        src = np.frombuffer(self._mm, dtype=np.uint8, count=nbytes, offset=start)
        out = np.empty(n, dtype=np.float32)
        rc = lib.afb_gguf_dequantize(ctypes.c_int(info.type), src.ctypes.data_as(ctypes.c_void_p),
                                     out.ctypes.data_as(ctypes.c_void_p), ctypes.c_long(n))
        if rc != 0:
            raise NotImplementedError(f"GGUF tensor type {info.type_name} is not supported")
        return torch.from_numpy(out).view(info.shape)

    def raw(self, name: str) -> np.ndarray:
        info = self.tensors[name]
        lib = N.host()
        lib.afb_gguf_block_bytes.restype = ctypes.c_long
        lib.afb_gguf_block_values.restype = ctypes.c_long
        n = int(np.prod(info.shape))
        nbytes = n // lib.afb_gguf_block_values(info.type) * lib.afb_gguf_block_bytes(info.type)
        return np.frombuffer(self._mm, dtype=np.uint8, count=nbytes, offset=self.data_start + info.offset)


# HF <- GGUF tensor names for llama-family checkpoints (the loader-side normalisation the reference performs).
_GGUF_TO_HF = {
    "token_embd.weight": "model.embed_tokens.weight", "output_norm.weight": "model.norm.weight",
    "output.weight": "lm_head.weight",
}
_LAYER = {"attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj",
          "attn_output": "self_attn.o_proj", "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj",
          "ffn_down": "mlp.down_proj", "attn_norm": "input_layernorm", "ffn_norm": "post_attention_layernorm",
          "attn_sub_norm": "self_attn.attn_sub_norm", "ffn_sub_norm": "mlp.ffn_sub_norm",   # BitNet
          "attn_q_norm": "self_attn.q_norm", "attn_k_norm": "self_attn.k_norm",              # Qwen3, Gemma-3
          "attn_qkv": "self_attn.qkv_proj"}                                                   # Phi-3 (fused)
# per architecture: names that mean something else there
_GEMMA_POST = {"ffn_norm": "pre_feedforward_layernorm", "post_attention_norm": "post_attention_layernorm",
               "post_ffw_norm": "post_feedforward_layernorm"}                                 # norms on both sides
_LAYER_ARCH = {"phi3": {"ffn_up": "mlp.gate_up_proj"},                                        # gate and up stacked
               "gemma2": _GEMMA_POST, "gemma3": _GEMMA_POST, "gemma3_text": _GEMMA_POST}
GEMMA_ARCHS = ("gemma", "gemma2", "gemma3")


def hf_name(gguf_name: str, arch: Optional[str] = None) -> str:
    if gguf_name in _GGUF_TO_HF:
        return _GGUF_TO_HF[gguf_name]
    parts = gguf_name.split(".")
    if parts[0] == "blk" and len(parts) >= 4:
        mid = _LAYER_ARCH.get(arch or "", {}).get(parts[2]) or _LAYER.get(parts[2])
        if mid:
            return f"model.layers.{parts[1]}.{mid}.{parts[3]}"
    return gguf_name


def gguf_name(hf: str, arch: Optional[str] = None) -> str:
    """Inverse of :func:`hf_name` for the Llama-family tensor names."""
    for g, h in _GGUF_TO_HF.items():
        if h == hf:
            return g
    parts = hf.split(".")
    if len(parts) >= 5 and parts[0] == "model" and parts[1] == "layers":
        mid = ".".join(parts[3:-1])
        for g, h in list(_LAYER_ARCH.get(arch or "", {}).items()) + list(_LAYER.items()):
            if h == mid:
                return f"blk.{parts[2]}.{g}.{parts[-1]}"
    return hf


# Architectures whose converted files store the Q / K projection rows re-ordered so that the rotary pairs of a head
# are adjacent (row 2j and 2j + 1 of a head are rows j and j + D/2 of the Hugging Face layout): llama.cpp's converter
# does this for its "llama" architecture (Llama and Mistral checkpoints) and rotates consecutive pairs at run time; the
# reference follows the same convention (zig/pkg/inference/src/models/gpt.zig:1277-1281).  The attention scores are
# the same either way -- a permutation applied to both q and k -- so such files are served as they are, with the
# consecutive-pair rotation, and only a comparison against a Hugging Face model needs the rows put back.
PAIRED_ROPE_ARCHS = ("llama", "mistral")


def pair_rope_rows(w: torch.Tensor, n_head: int) -> torch.Tensor:
    """Hugging Face row order of a Q / K projection -> rotary pairs adjacent (the stored order of those files)."""
    rows = w.shape[0]
    return w.reshape(n_head, 2, rows // n_head // 2, *w.shape[1:]).transpose(1, 2).reshape(w.shape)


def unpair_rope_rows(w: torch.Tensor, n_head: int) -> torch.Tensor:
    """Inverse of :func:`pair_rope_rows`."""
    rows = w.shape[0]
    return w.reshape(n_head, rows // n_head // 2, 2, *w.shape[1:]).transpose(1, 2).reshape(w.shape)


def to_hf_row_order(sd: Dict[str, torch.Tensor], config: dict) -> Dict[str, torch.Tensor]:
    """A state dict read from a file of one of :data:`PAIRED_ROPE_ARCHS` (Hugging Face tensor names) with the Q / K
    rows back in the Hugging Face order, for loading into a transformers model."""
    if config.get("model_type") not in PAIRED_ROPE_ARCHS:
        return dict(sd)
    nh, nkv = int(config["num_attention_heads"]), int(config.get("num_key_value_heads") or config["num_attention_heads"])
    out = {}
    for k, v in sd.items():
        if k.endswith(("self_attn.q_proj.weight", "self_attn.q_proj.bias")):
            v = unpair_rope_rows(v, nh)
        elif k.endswith(("self_attn.k_proj.weight", "self_attn.k_proj.bias")):
            v = unpair_rope_rows(v, nkv)
        out[k] = v
    return out


_EXPERT_STACKS = {"ffn_gate_exps": "gate", "ffn_up_exps": "up", "ffn_down_exps": "down"}
_SHARED_EXPERT = {"ffn_gate_shexp": "mlp.shared_expert.gate_proj", "ffn_up_shexp": "mlp.shared_expert.up_proj",
                  "ffn_down_shexp": "mlp.shared_expert.down_proj", "ffn_gate_inp_shexp": "mlp.shared_expert_gate",
                  "ffn_gate_inp": "mlp.gate"}


def fuse_expert_tensors(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """The expert tensors of a mixture-of-experts file under the names the decoder loader reads:
    ``blk.N.ffn_gate_exps`` [E, F, H] and ``ffn_up_exps`` become ``mlp.experts.gate_up_proj`` [E, 2F, H] (gate rows,
    then up rows), ``ffn_down_exps`` [E, H, F] becomes ``mlp.experts.down_proj``, the router ``ffn_gate_inp`` becomes
    ``mlp.gate``, a shared expert keeps its three projections and its gate."""
    out, stacks = {}, {}
    for name, t in sd.items():
        parts = name.split(".")
        if parts[0] == "blk" and len(parts) == 4 and parts[2] in _EXPERT_STACKS:
            stacks.setdefault(parts[1], {})[_EXPERT_STACKS[parts[2]]] = t
        elif parts[0] == "blk" and len(parts) == 4 and parts[2] in _SHARED_EXPERT:
            out[f"model.layers.{parts[1]}.{_SHARED_EXPERT[parts[2]]}.{parts[3]}"] = t
        else:
            out[name] = t
    for layer, st in stacks.items():
        out[f"model.layers.{layer}.mlp.experts.gate_up_proj"] = torch.cat([st["gate"], st["up"]], 1)
        out[f"model.layers.{layer}.mlp.experts.down_proj"] = st["down"]
    return out


def split_expert_tensors(sd: Dict[str, torch.Tensor], n_experts: int) -> Dict[str, torch.Tensor]:
    """Inverse of :func:`fuse_expert_tensors` for export: fused or per-expert Hugging Face names -> the stacked
    per-projection tensors (under their file names) plus everything else unchanged."""
    out = {}
    per = {}
    for name, t in sd.items():
        parts = name.split(".")
        if len(parts) >= 5 and parts[0] == "model" and parts[1] == "layers":
            layer, rest = parts[2], ".".join(parts[3:])
            moe = rest.split(".", 1)[1] if rest.startswith(("mlp.", "block_sparse_moe.")) else None
            if moe == "experts.gate_up_proj":
                F = t.shape[1] // 2
                out[f"blk.{layer}.ffn_gate_exps.weight"], out[f"blk.{layer}.ffn_up_exps.weight"] = t[:, :F], t[:, F:]
                continue
            if moe == "experts.down_proj":
                out[f"blk.{layer}.ffn_down_exps.weight"] = t
                continue
            if moe and moe.startswith("experts.") and moe.count(".") == 3:            # experts.<e>.<proj>.weight
                _, e, proj, _w = moe.split(".")
                kind = {"w1": "gate", "gate_proj": "gate", "w3": "up", "up_proj": "up", "w2": "down",
                        "down_proj": "down"}[proj]
                per.setdefault((layer, kind), {})[int(e)] = t
                continue
            if moe == "gate.weight":
                out[f"blk.{layer}.ffn_gate_inp.weight"] = t
                continue
            inv = {v: k for k, v in _SHARED_EXPERT.items()}
            if rest.rsplit(".", 1)[0] in inv:
                out[f"blk.{layer}.{inv[rest.rsplit('.', 1)[0]]}.{parts[-1]}"] = t
                continue
        out[name] = t
    for (layer, kind), ts in per.items():
        out[f"blk.{layer}.ffn_{kind}_exps.weight"] = torch.stack([ts[e] for e in range(n_experts)])
    return out


def export_llama_gguf(path: str, sd: Dict[str, torch.Tensor], config: dict, quant: str = "q8_0",
                      tokens: Optional[List[str]] = None, extra_metadata: Optional[Dict[str, Any]] = None,
                      include: Optional[List[str]] = None, exclude: Optional[List[str]] = None,
                      dry_run: bool = False) -> Dict[str, int]:
    """Write a Llama-family Hugging Face state dict as a GGUF v3 file: 2-D projection weights in ``quant`` (f32,
    f16, q8_0, q4_0), norms and embeddings in f32 / f16; metadata keys are the ones :func:`llama_config_from_gguf`
    reads back; Q / K rows of the :data:`PAIRED_ROPE_ARCHS` in the stored order of those files.  ``include`` /
    ``exclude`` are prefixes of (Hugging Face) tensor names that restrict which eligible tensors are quantised (the
    others stay f16); ``dry_run`` plans without writing (the reference's --quantize-include / --quantize-exclude /
    --dry-run, zig/pkg/inference/src/native_export_gguf.zig:4814).  Returns {tensor type id: count}."""
    ty = {"f32": 0, "f16": 1, "i2_s": 36, **QUANT_NAMES}[quant.lower()]           # i2_s: BitNet ternary projections
    block = 256 if ty in (10, 11, 12, 13, 14, 15) else 32
    arch = {"mixtral": "llama", "qwen2_moe": "qwen2moe", "qwen3_moe": "qwen3moe", "gemma3_text": "gemma3"}.get(
        config.get("model_type", "llama"), config.get("model_type", "llama"))
    n_exp = int(config.get("num_local_experts") or config.get("num_experts") or 0)
    if n_exp:
        sd = split_expert_tensors(sd, n_exp)
    md = {"general.architecture": arch, "general.name": str(config.get("_name_or_path", "model")),
          f"{arch}.block_count": int(config["num_hidden_layers"]),
          f"{arch}.embedding_length": int(config["hidden_size"]),
          f"{arch}.feed_forward_length": int(config["intermediate_size"]),
          f"{arch}.attention.head_count": int(config["num_attention_heads"]),
          f"{arch}.attention.head_count_kv": int(config.get("num_key_value_heads", config["num_attention_heads"])),
          f"{arch}.rope.freq_base": float(config.get("rope_theta", 10000.0)),
          f"{arch}.attention.layer_norm_rms_epsilon": float(config.get("rms_norm_eps", 1e-5)),
          f"{arch}.vocab_size": int(config["vocab_size"])}
    if tokens:
        md["tokenizer.ggml.tokens"] = list(tokens)
    if arch in ("gemma2", "gemma3"):
        if config.get("sliding_window"):
            md[f"{arch}.attention.sliding_window"] = int(config["sliding_window"])
        for key in ("attn_logit_softcapping", "final_logit_softcapping"):
            if config.get(key):
                md[f"{arch}.{key}"] = float(config[key])
        if config.get("query_pre_attn_scalar"):
            md[f"{arch}.attention.query_pre_attn_scalar"] = float(config["query_pre_attn_scalar"])
        if arch == "gemma3":
            rp = config.get("rope_parameters") or {}
            full, local = rp.get("full_attention", rp), rp.get("sliding_attention", {})
            md[f"{arch}.rope.freq_base"] = float(full.get("rope_theta") or config.get("rope_theta") or 1000000.0)
            md[f"{arch}.rope.local_freq_base"] = float(local.get("rope_theta") or config.get("rope_local_base_freq")
                                                       or 10000.0)
            if full.get("rope_type") == "linear" and full.get("factor"):
                md[f"{arch}.rope.scaling.type"], md[f"{arch}.rope.scaling.factor"] = "linear", float(full["factor"])
            kinds = config.get("layer_types")
            if kinds:
                md[f"{arch}.attention.layer_types"] = [1 if k == "sliding_attention" else 0 for k in kinds]
    if n_exp:
        md[f"{arch}.expert_count"] = n_exp
        md[f"{arch}.expert_used_count"] = int(config.get("num_experts_per_tok", 2))
        md[f"{arch}.expert_feed_forward_length"] = int(config.get("moe_intermediate_size") or config["intermediate_size"])
        if config.get("shared_expert_intermediate_size"):
            md[f"{arch}.expert_shared_feed_forward_length"] = int(config["shared_expert_intermediate_size"])
    md.update(extra_metadata or {})              # tokenizer tables, chat template, ...
    if config.get("max_position_embeddings"):
        md[f"{arch}.context_length"] = int(config["max_position_embeddings"])
    if config.get("head_dim"):
        md[f"{arch}.attention.key_length"] = int(config["head_dim"])
    tensors, counts = {}, {}
    # frequency-dependent rotary scaling travels the way converted Llama-3.1 files carry it: one divisor per rotary
    # pair in rope_freqs.weight (plus the attention factor, when there is one)
    rope = config.get("rope_parameters") or config.get("rope_scaling") or {}
    kind = rope.get("rope_type", rope.get("type"))
    if kind == "linear" and rope.get("factor"):
        md[f"{arch}.rope.scaling.type"], md[f"{arch}.rope.scaling.factor"] = "linear", float(rope["factor"])
    elif kind in ("llama3", "yarn", "longrope", "su", "factors"):
        from ..models.rope_scaling import rope_frequencies

        hd = int(config.get("head_dim") or config["hidden_size"] // config["num_attention_heads"])
        theta = float(config.get("rope_theta") or rope.get("rope_theta") or 10000.0)
        full = dict(rope)
        if "original_max_position_embeddings" not in full and config.get("original_max_position_embeddings"):
            full["original_max_position_embeddings"] = config["original_max_position_embeddings"]
        inv, att = rope_frequencies(full, theta, hd, int(config.get("max_position_embeddings") or 0))
        base = [theta ** (-2.0 * j / hd) for j in range(hd // 2)]
        tensors["rope_freqs.weight"] = (0, torch.tensor([b / f for b, f in zip(base, inv)], dtype=torch.float32))
        if att != 1.0:
            md[f"{arch}.rope.scaling.attn_factor"] = float(att)
    nh = int(config["num_attention_heads"])
    nkv = int(config.get("num_key_value_heads", nh))
    for name, t in sd.items():
        if not isinstance(t, torch.Tensor) or not t.is_floating_point():
            continue
        if arch in PAIRED_ROPE_ARCHS:
            if name.endswith(("self_attn.q_proj.weight", "self_attn.q_proj.bias")):
                t = pair_rope_rows(t, nh)
            elif name.endswith(("self_attn.k_proj.weight", "self_attn.k_proj.bias")):
                t = pair_rope_rows(t, nkv)
        if arch in GEMMA_ARCHS and name.endswith("norm.weight"):
            t = t.float() + 1.0      # converted Gemma files hold 1 + gamma (the loader takes the 1 off again)
        quantisable = t.dim() in (2, 3) and t.shape[-1] % block == 0 and "embed_tokens" not in name and \
            "norm" not in name and "ffn_gate_inp" not in name
        if ty == 36:      # ternary only where the model is ternary (the projections), whole 128-value blocks
            quantisable = quantisable and name.endswith("_proj.weight") and t.numel() % 128 == 0
        if include and not any(name.startswith(pre) for pre in include):
            quantisable = False
        if exclude and any(name.startswith(pre) for pre in exclude):
            quantisable = False
        tt = ty if quantisable else (1 if t.dim() == 2 and ty != 0 and "ffn_gate_inp" not in name else 0)
        tensors[gguf_name(name, arch)] = (tt, t.float())
        counts[tt] = counts.get(tt, 0) + 1
    if not dry_run:
        write_gguf(path, md, tensors)
    return counts


def llama_config_from_gguf(md: Dict[str, Any]) -> dict:
    arch = md.get("general.architecture", "llama")
    g = lambda k, d=None: md.get(f"{arch}.{k}", d)
    if arch.startswith("bitnet"):          # "bitnet" / "bitnet-b1.58": keys carry the file's own spelling
        return {**llama_config_from_gguf({**md, "general.architecture": "llama",
                                          **{"llama." + k[len(arch) + 1:]: v for k, v in md.items()
                                             if k.startswith(arch + ".")}}),
                "model_type": "bitnet", "tie_word_embeddings": True, "rope_half_split": True}
    out = {"model_type": arch, "hidden_size": g("embedding_length"), "num_hidden_layers": g("block_count"),
           "num_attention_heads": g("attention.head_count"),
           "num_key_value_heads": g("attention.head_count_kv", g("attention.head_count")),
           "intermediate_size": g("feed_forward_length"), "rope_theta": g("rope.freq_base", 10000.0),
           "rms_norm_eps": g("attention.layer_norm_rms_epsilon", 1e-5),
           "vocab_size": g("vocab_size", len(md.get("tokenizer.ggml.tokens", [])) or None),
           "head_dim": g("attention.key_length"), "max_position_embeddings": g("context_length")}
    if arch in PAIRED_ROPE_ARCHS:
        out["rope_half_split"] = False          # Q / K rows are stored with their rotary pairs adjacent
    n_exp = int(g("expert_count") or 0)
    if n_exp > 0:
        # mixture-of-experts files: Mixtral is written under the "llama" architecture, the Qwen families under
        # their own; expert weights come as one stacked tensor per projection (see fuse_expert_tensors)
        out["model_type"] = {"llama": "mixtral", "qwen2moe": "qwen2_moe", "qwen3moe": "qwen3_moe"}.get(arch, arch)
        out["num_local_experts"] = out["num_experts"] = n_exp
        out["num_experts_per_tok"] = int(g("expert_used_count") or 2)
        out["moe_intermediate_size"] = int(g("expert_feed_forward_length") or g("feed_forward_length") or 0) or None
        out["shared_expert_intermediate_size"] = int(g("expert_shared_feed_forward_length") or 0) or None
        out["norm_topk_prob"] = arch != "qwen2moe"
        out["decoder_sparse_step"], out["mlp_only_layers"] = 1, []
    # context extension declared in the metadata: linear position scaling or yarn (a per-pair divisor tensor,
    # rope_freqs.weight, is attached by the loader that has the tensors at hand: see rope_factors_config)
    if g("rope.scaling.attn_factor") and not g("rope.scaling.type"):
        out["rope_attention_factor"] = float(g("rope.scaling.attn_factor"))     # goes with a rope_freqs.weight tensor
    kind = g("rope.scaling.type")
    if kind in ("linear", "yarn") and g("rope.scaling.factor"):
        rope = {"rope_type": kind, "factor": float(g("rope.scaling.factor"))}
        if g("rope.scaling.original_context_length"):
            rope["original_max_position_embeddings"] = int(g("rope.scaling.original_context_length"))
        if g("rope.scaling.attn_factor"):
            rope["attention_factor"] = float(g("rope.scaling.attn_factor"))
        out["rope_scaling"] = rope
    if arch in ("gemma2", "gemma3"):
        # Converted files carry the window and the soft caps; the layer pattern, the local rotary base and the
        # query scale are fixed per family there, so the defaults of the configuration reader apply when the
        # optional keys this module's own exporter adds (layer_types, local_freq_base, query_pre_attn_scalar) are absent.
        out["sliding_window"] = g("attention.sliding_window")
        out["attn_logit_softcapping"], out["final_logit_softcapping"] = g("attn_logit_softcapping"), g("final_logit_softcapping")
        out["query_pre_attn_scalar"] = g("attention.query_pre_attn_scalar") or g("attention.key_length")
        if arch == "gemma3":
            glob = {"rope_type": "default", "rope_theta": float(g("rope.freq_base", 1000000.0))}
            if out.get("rope_scaling", {}).get("rope_type") == "linear":
                glob = dict(out.pop("rope_scaling"), rope_theta=glob["rope_theta"])
            out["rope_parameters"] = {"full_attention": glob, "sliding_attention": {
                "rope_type": "default", "rope_theta": float(g("rope.local_freq_base", 10000.0))}}
            out.pop("rope_theta", None)
            kinds = g("attention.layer_types")
            if kinds:
                out["layer_types"] = ["sliding_attention" if k else "full_attention" for k in kinds]
    return out


def rope_factors_config(factors, attention_factor: float = 1.0) -> dict:
    """The ``rope_freqs.weight`` tensor of a GGUF file (one divisor per rotary pair; how converted Llama-3.1 files carry
    their frequency scaling) as a ``rope_scaling`` entry."""
    return {"rope_type": "factors", "factors": [float(v) for v in factors], "attention_factor": float(attention_factor)}


def pack_i2s(values: np.ndarray) -> bytes:
    """fp32 values -> BitNet I2_S bytes: the tensor is ternarised against its mean magnitude (``round(v / mean|v|)``
    clipped to [-1, 1]), 128 values go into 32 bytes (byte ``g`` holds values ``g``, ``g + 32``, ``g + 64``,
    ``g + 96`` in bits 7-6, 5-4, 3-2, 1-0 as value + 1), and a 32-byte tail starts with the fp32 scale."""
    a = np.asarray(values, dtype=np.float32).reshape(-1)
    if a.size % 128:
        raise ValueError("I2_S tensors hold a multiple of 128 values")
    scale = max(float(np.abs(a).mean()), 1e-5) if a.size else 1.0
    codes = (np.clip(np.rint(a / scale), -1, 1) + 1).astype(np.uint8).reshape(-1, 4, 32)
    packed = (codes[:, 0] << 6) | (codes[:, 1] << 4) | (codes[:, 2] << 2) | codes[:, 3]
    return packed.astype(np.uint8).tobytes() + struct.pack("<f", scale) + b"\0" * 28


# tensor types the export tool can write besides F32 / F16 (ggml numbering): Q4_0 Q4_1 Q5_0 Q5_1 Q8_0 Q8_1 and the
# K-quants Q2_K .. Q6_K, Q8_K
QUANTIZABLE = (2, 3, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15)
QUANT_NAMES = {"q4_0": 2, "q4_1": 3, "q5_0": 6, "q5_1": 7, "q8_0": 8, "q8_1": 9, "q2_k": 10, "q3_k": 11, "q4_k": 12,
               "q5_k": 13, "q6_k": 14, "q8_k": 15}


def quantize(values: np.ndarray, type_id: int) -> np.ndarray:
    """fp32 values (a whole number of blocks of the type) -> the type's block bytes (csrc/host/gguf_quantize.cpp)."""
    lib = N.host()
    lib.afb_gguf_block_bytes.restype = ctypes.c_long
    lib.afb_gguf_block_values.restype = ctypes.c_long
    a = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
    bv, bb = int(lib.afb_gguf_block_values(type_id)), int(lib.afb_gguf_block_bytes(type_id))
    if type_id not in QUANTIZABLE or bv <= 0:
        raise NotImplementedError(f"no quantiser for GGUF tensor type {type_id}")
    if a.size % bv:
        raise ValueError(f"{a.size} values are not a whole number of {bv}-value blocks")
    out = np.empty(a.size // bv * bb, dtype=np.uint8)
    rc = lib.afb_gguf_quantize(ctypes.c_int(type_id), a.ctypes.data_as(ctypes.c_void_p),
                               out.ctypes.data_as(ctypes.c_void_p), ctypes.c_long(a.size))
    if rc != 0:
        raise RuntimeError(f"GGUF quantiser failed for type {type_id} (code {rc})")
    return out


def write_gguf(path: str, metadata: Dict[str, Any], tensors: Dict[str, Tuple[int, torch.Tensor]]) -> None:
    """tensors: name -> (type id, fp32 tensor); quantises with the C++ codecs (F32, F16, Q8_0, Q4_0)."""
    lib = N.host()

    def s(x: str) -> bytes:
        b = x.encode("utf-8")
        return struct.pack("<Q", len(b)) + b

    def val(v) -> bytes:
        if isinstance(v, bool):
            return struct.pack("<I?", 7, v)
        if isinstance(v, int):
            return struct.pack("<Iq", 11, v) if v < 0 else struct.pack("<II", 4, v) if v < 2 ** 32 else struct.pack("<IQ", 10, v)
        if isinstance(v, float):
            return struct.pack("<If", 6, v)
        if isinstance(v, str):
            return struct.pack("<I", 8) + s(v)
        if isinstance(v, (list, tuple)):
            if all(isinstance(e, str) for e in v):
                return struct.pack("<IIQ", 9, 8, len(v)) + b"".join(s(e) for e in v)
            return struct.pack("<IIQ", 9, 6, len(v)) + b"".join(struct.pack("<f", float(e)) for e in v)
        raise TypeError(type(v))

    blobs, infos, off = [], [], 0
    for name, (ty, t) in tensors.items():
        a = t.detach().float().cpu().contiguous().numpy().reshape(-1)
        if ty == 0:
            raw = a.tobytes()
        elif ty == 1:
            raw = a.astype(np.float16).tobytes()
        elif ty in QUANTIZABLE:
            raw = quantize(a, ty).tobytes()
        elif ty == 36:
            raw = pack_i2s(a)
        else:
            raise NotImplementedError(ty)
        pad = (32 - len(raw) % 32) % 32
        infos.append((name, tuple(t.shape), ty, off))
        blobs.append(raw + b"\0" * pad)
        off += len(raw) + pad
    head = GGUF_MAGIC + struct.pack("<IQQ", 3, len(infos), len(metadata))
    for k, v in metadata.items():
        head += s(k) + val(v)
    for name, shape, ty, o in infos:
        dims = tuple(reversed(shape))
        head += s(name) + struct.pack("<I", len(dims)) + struct.pack(f"<{len(dims)}Q", *dims) + struct.pack("<IQ", ty, o)
    head += b"\0" * ((32 - len(head) % 32) % 32)
    with open(path, "wb") as f:
        f.write(head)
        for b in blobs:
            f.write(b)
