"""Model manager: resolves model names to directories, loads and caches models with their tokenizer and
pipelines (the reference's ModelManager.loadFromDir / LoadedModel, zig/pkg/inference/src/server/
model_manager.zig:641-1100), bounded by ``max_loaded_models`` with least-recently-used eviction.  Models can also be
registered in memory (random-init models for tests and benchmarks)."""
from __future__ import annotations

import json
import os
import threading
import time
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, Optional

import torch

from ..formats import manifest as MF
from ..formats import safetensors_io as ST
from ..models.bert import BertConfig, BertModel
from ..models.llama import LlamaConfig, LlamaModel
from ..pipelines.embedding import Embedder
from ..pipelines.generation import Generator
from ..pipelines.reranking import CrossEncoderReranker
from ..runtime.engine import LLMEngine
from ..tokenizer import ByteTokenizer, load_tokenizer


COMPILED_ARTIFACT = "compiled.antfly_b200.safetensors"


class ModelNotFound(KeyError):
    pass


@dataclass
class LoadedModel:
    name: str
    task: str  # embedder | reranker | generator
    pipeline: object
    tokenizer: object
    path: Optional[str] = None
    loaded_at: float = field(default_factory=time.time)
    info: Dict = field(default_factory=dict)
    last_used: float = field(default_factory=time.time)
    pinned: bool = False      # eager strategy / registered in memory: never unloaded for idleness or room
    bytes: int = 0            # parameter bytes (advisory memory accounting)


def _param_bytes(pipeline) -> int:
    model = getattr(pipeline, "model", None) or getattr(getattr(pipeline, "engine", None), "model", None)
    total = 0
    for v in getattr(model, "w", {}).values():
        if isinstance(v, torch.Tensor):
            total += v.numel() * v.element_size()
        else:  # block-fp8 weight: codes + scales
            total += sum(t.numel() * t.element_size() for t in (getattr(v, "q", None), getattr(v, "scales", None))
                         if isinstance(t, torch.Tensor))
    return total


class ModelManager:
    def __init__(self, models_dir: Optional[str] = None, device: Optional[str] = None, max_loaded_models: int = 8,
                 kv_blocks: int = 4096, max_batch: int = 64, prefix_cache: bool = True, keep_alive_s: float = 0.0,
                 max_memory_mb: int = 0, strategies: Optional[Dict[str, str]] = None, clock=time.time,
                 tensor_parallel: Optional[tuple] = None, gguf_native: Optional[bool] = None,
                 adapters: Optional[Dict[str, str]] = None):
        """``max_loaded_models`` 0 = unlimited; ``keep_alive_s`` > 0 unloads directory-backed models idle for that
        long (checked on every access and by :meth:`evict_idle`); ``max_memory_mb`` > 0 is an advisory budget on
        parameter bytes, enforced by unloading least-recently-used models; ``strategies`` maps model names to
        eager (never unloaded) / lazy / bounded."""
        self.models_dir = models_dir or MF.default_models_dir()
        self.device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
        self.max_loaded = max_loaded_models
        self.keep_alive_s, self.max_memory_mb = keep_alive_s, max_memory_mb
        self.strategies, self._clock = dict(strategies or {}), clock
        self.evictions = 0
        self.kv_blocks, self.max_batch, self.prefix_cache = kv_blocks, max_batch, prefix_cache
        self._models: "OrderedDict[str, LoadedModel]" = OrderedDict()
        self._lock = threading.Lock()
        # (rank, world, comm): BERT-family encoders and cross-encoders are sharded over the ranks of a
        # tensor-parallel job (every rank serves the same requests in lockstep), the reference's
        # TERMITE_MLX_DISTRIBUTED_MODE=tensor_parallel deployment (zig/pkg/inference/docs/RERANKING.md:32-43)
        self.tensor_parallel = tensor_parallel
        # model name -> adapter name under <model>/adapters/ (default: the adapter in the model directory itself,
        # else adapters/retrieval; the ANTFLY_B200_ADAPTER environment variable names one for every model)
        self.adapters = dict(adapters or {})
        self._tls = threading.local()          # per-thread note of the adapter merged by the load in progress
        # GGUF generators: keep the projections in their block formats and expand them inside the kernels instead
        # of re-packing to block fp8 at load time (default: the ANTFLY_B200_GGUF_NATIVE environment switch)
        self.gguf_native = os.environ.get("ANTFLY_B200_GGUF_NATIVE", "0") == "1" if gguf_native is None else gguf_native

    def _tp(self, model):
        if self.tensor_parallel is not None and isinstance(model, BertModel):
            rank, world, comm = self.tensor_parallel
            return model.tensor_parallel(rank, world, comm)
        return model

    # -- registration of in-memory models ------------------------------------------------------------------
    def register(self, name: str, task: str, pipeline, tokenizer, info: Optional[dict] = None) -> LoadedModel:
        lm = LoadedModel(name, task, pipeline, tokenizer, info=info or {}, pinned=True)
        with self._lock:
            self._models[f"{task}:{name}"] = lm
        return lm

    def register_random(self, name: str, task: str, size: str = "tiny", seed: int = 0) -> LoadedModel:
        """Random-init model of a named size, with the byte tokenizer (no artifacts needed)."""
        dev = self.device
        if task in ("embedder", "reranker"):
            cfgs = {"tiny": BertConfig(hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                                       intermediate_size=256, vocab_size=512),
                    "base": BertConfig.base()}
            cfg = cfgs[size]
            if task == "reranker":
                cfg.num_labels = 1
            model = self._tp(BertModel.random_init(cfg, device=dev, seed=seed))
            tok = ByteTokenizer(cfg.vocab_size)
            pipe = Embedder(model, tok) if task == "embedder" else CrossEncoderReranker(model, tok)
            return self.register(name, task, pipe, tok, {"hidden_size": cfg.hidden_size, "random_init": True})
        cfgs = {"tiny": LlamaConfig.tiny(), "8b": LlamaConfig.llama3_8b(), "70b": LlamaConfig.llama3_70b()}
        cfg = cfgs[size]
        model = LlamaModel.random_init(cfg, device=dev, seed=seed, fast_init=(size != "tiny"))
        tok = ByteTokenizer(cfg.vocab_size)
        eng = LLMEngine(model, num_blocks=self.kv_blocks, max_batch=self.max_batch,
                        use_cuda_graph=dev.type == "cuda", eos_token_id=tok.special.eos_id,
                        prefix_cache=self.prefix_cache)
        return self.register(name, "generator", Generator(eng, tok), tok, {"random_init": True})

    # -- directory-backed models ---------------------------------------------------------------------------
    def _load_dir(self, name: str, task: str, path: str) -> LoadedModel:
        mf = MF.read_manifest(path)
        tok = load_tokenizer(path, mf.config.get("vocab_size", 0))
        if mf.chat_template is None:                 # a GGUF-only directory: the template travels in the file's metadata
            mf.chat_template = getattr(tok, "chat_template", None)
        packed = os.path.join(path, COMPILED_ARTIFACT)
        if task == "generator" and os.path.exists(packed):
            # a compiled artifact holds the weights in the kernels' own layout: read and upload, nothing to pack
            model = LlamaModel.from_artifact(packed, device=self.device)
            eng = LLMEngine(model, num_blocks=self.kv_blocks, max_batch=self.max_batch,
                            use_cuda_graph=self.device.type == "cuda", eos_token_id=tok.special.eos_id,
                            prefix_cache=self.prefix_cache)
            return LoadedModel(name, task, Generator(eng, tok, mf.chat_template), tok, path,
                               info={"weights": "compiled", "capabilities": mf.capabilities})
        if mf.weights == "gguf":
            from ..formats import gguf as GG

            f = GG.GGUFFile(os.path.join(path, mf.weight_files[0]))
            cfg_d = {k: v for k, v in GG.llama_config_from_gguf(f.metadata).items() if v is not None}
            cfg_d.setdefault("tie_word_embeddings", "output.weight" not in f.tensors)   # no output matrix: tied
            if "rope_freqs.weight" in f.tensors and "rope_scaling" not in cfg_d:
                cfg_d["rope_scaling"] = GG.rope_factors_config(f.tensor("rope_freqs.weight").float().flatten().tolist(),
                                                               cfg_d.pop("rope_attention_factor", 1.0))
            if task == "generator" and self.gguf_native and cfg_d.get("model_type") in (
                    "llama", "mistral", "qwen2", "qwen3"):
                model = LlamaModel.from_gguf_native(LlamaConfig.from_hf(cfg_d), f, device=self.device)
                eng = LLMEngine(model, num_blocks=self.kv_blocks, max_batch=self.max_batch,
                                use_cuda_graph=self.device.type == "cuda", eos_token_id=tok.special.eos_id,
                                prefix_cache=self.prefix_cache)
                return LoadedModel(name, task, Generator(eng, tok, mf.chat_template), tok, path,
                                   info={"weights": "gguf-native", "capabilities": mf.capabilities})
            arch = cfg_d.get("model_type")
            sd = {GG.hf_name(n, arch): f.tensor(n) for n in f.tensors if f.tensors[n].type in GG.SUPPORTED}
            if cfg_d.get("num_experts"):
                sd = GG.fuse_expert_tensors(sd)
            if arch in GG.GEMMA_ARCHS:
                # converted Gemma files store 1 + gamma in their norm tensors; the model adds the 1 itself
                sd = {k: (v - 1.0 if k.endswith("norm.weight") else v) for k, v in sd.items()}
        elif mf.weights == "safetensors":
            sd, cfg_d = ST.load_model_dir(path), mf.config
        else:
            raise ModelNotFound(f"{name}: no loadable weights (found {mf.weights})")
        # a low-rank adapter in the model directory (or the one named for this model) is folded into the weights
        # before they are packed, so the adapted model runs at the base model's cost
        from ..formats import lora as LORA

        self._tls.adapter = LORA.apply_adapter(sd, path, self.adapters.get(name) or os.environ.get("ANTFLY_B200_ADAPTER"))
        if task == "embedder" and cfg_d.get("model_type") == "clip":
            from ..models.clip import ClipConfig, ClipModel
            from ..pipelines.multimodal import ClipEmbedder

            model = ClipModel.from_state_dict(ClipConfig.from_hf(cfg_d), sd, device=self.device)
            pipe = ClipEmbedder(model, tok)
        elif task == "embedder" and cfg_d.get("model_type") == "clap":
            from ..models.clap import ClapConfig, ClapModel
            from ..pipelines.multimodal import ClapEmbedder

            model = ClapModel.from_state_dict(ClapConfig.from_hf(cfg_d), sd, device=self.device)
            pipe = ClapEmbedder(model, tok)
        elif task == "embedder" and cfg_d.get("model_type") in ("qwen2", "qwen3", "llama", "mistral", "gemma", "phi3"):
            # decoder-based embedding models (Qwen3-Embedding, E5-Mistral, ...): last-token pooling
            from ..pipelines.embedding import DecoderEmbedder

            model = LlamaModel.from_state_dict(LlamaConfig.from_hf(cfg_d), sd, device=self.device)
            pipe = DecoderEmbedder(model, tok)
        elif task == "generator" and cfg_d.get("model_type") in ("qwen3_5", "qwen3_5_text", "qwen3_next"):
            # hybrid decoder (delta-rule + gated attention layers): per-sequence state kept by the model
            from ..models.qwen35 import Qwen35Config, Qwen35Model
            from ..pipelines.generation import StatefulGenerator

            dt = torch.bfloat16 if self.device.type == "cuda" else torch.float32
            model = Qwen35Model.from_state_dict(Qwen35Config.from_hf(cfg_d), sd, device=self.device, dtype=dt)
            pipe = StatefulGenerator(model, tok, mf.chat_template)
        elif task == "generator" and str(cfg_d.get("model_type", "")).replace("-", "_").startswith("deepseek_v4"):
            # single-latent attention with compressed long-range rows: the cache is the model's own state
            from ..models.deepseek_v4 import DeepseekV4Config, DeepseekV4Model
            from ..pipelines.generation import StatefulGenerator

            dt = torch.bfloat16 if self.device.type == "cuda" else torch.float32
            model = DeepseekV4Model.from_state_dict(DeepseekV4Config.from_hf(cfg_d), sd, device=self.device, dtype=dt)
            pipe = StatefulGenerator(model, tok, mf.chat_template)
        elif task == "generator" and cfg_d.get("model_type") in ("gemma4", "gemma4_text"):
            # Gemma-4: per-layer cache geometries and KV-shared layers, so it carries its own per-sequence state.
            from ..models.gemma4 import Gemma4Config, Gemma4TextModel
            from ..models.gemma4v import Gemma4Multimodal
            from ..pipelines.generation import StatefulGenerator

            dt = torch.bfloat16 if self.device.type == "cuda" else torch.float32
            if cfg_d.get("model_type") == "gemma4" and cfg_d.get("vision_config") and \
                    any(k.startswith("model.vision_tower.") for k in sd):
                model = Gemma4Multimodal.from_state_dict(cfg_d, sd, device=self.device, dtype=dt)
                pre = {}
                pp = os.path.join(path, "preprocessor_config.json") if os.path.isdir(path) else None
                if pp and os.path.exists(pp):
                    import json as _json
                    with open(pp, encoding="utf-8") as f:
                        pre = _json.load(f)
                model.max_soft_tokens = int(pre.get("max_soft_tokens", 280))
            else:
                text_d = cfg_d.get("text_config") or cfg_d
                model = Gemma4TextModel.from_state_dict(Gemma4Config.from_hf(text_d), sd, device=self.device, dtype=dt)
            pipe = StatefulGenerator(model, tok, mf.chat_template)
        elif task == "rewriter" or (task == "generator" and cfg_d.get("model_type") in ("t5", "mt5", "bart",
                                                                                         "mbart")):
            from ..models.t5 import T5Config, T5Model
            from ..pipelines.seq2seq import Seq2SeqGenerator

            if cfg_d.get("model_type") in ("bart", "mbart"):
                from ..models.bart import BartConfig, BartModel

                model = BartModel.from_state_dict(BartConfig.from_hf(cfg_d), sd, device=self.device)
            elif cfg_d.get("model_type") in ("t5", "mt5"):
                model = T5Model.from_state_dict(T5Config.from_hf(cfg_d), sd, device=self.device)
            else:
                raise ModelNotFound(f"{name}: rewriters are T5- or BART-family encoder-decoder models "
                                    f"(found {cfg_d.get('model_type')!r})")
            pipe = Seq2SeqGenerator(model, tok)
        elif task == "reader" and cfg_d.get("model_type") == "florence2":
            from ..models.florence2 import Florence2Model
            from ..pipelines.reading import FlorenceReader

            pp = {}
            ppath = os.path.join(path, "preprocessor_config.json")
            if os.path.exists(ppath):
                with open(ppath, encoding="utf-8") as f:
                    pp = json.load(f)
            dt = torch.bfloat16 if self.device.type == "cuda" else torch.float32
            model = Florence2Model.from_state_dict(cfg_d, sd, device=self.device, dtype=dt)
            size = pp.get("size") or {}
            pipe = FlorenceReader(model, tok, pp.get("image_mean", (0.485, 0.456, 0.406)),
                                  pp.get("image_std", (0.229, 0.224, 0.225)),
                                  "bilinear" if pp.get("resample") == 2 else "bicubic",
                                  int(size.get("height", model.vcfg.image_size)))
        elif task == "reader":
            from ..models.trocr import TrOCRConfig, TrOCRModel
            from ..pipelines.reading import Reader

            if cfg_d.get("model_type") != "vision-encoder-decoder" or \
                    (cfg_d.get("decoder") or {}).get("model_type") != "trocr":
                raise ModelNotFound(f"{name}: readers are ViT + TrOCR vision encoder-decoder models")
            pp = {}
            ppath = os.path.join(path, "preprocessor_config.json")
            if os.path.exists(ppath):
                with open(ppath, encoding="utf-8") as f:
                    pp = json.load(f)
            model = TrOCRModel.from_state_dict(TrOCRConfig.from_hf(cfg_d), sd, device=self.device)
            pipe = Reader(model, tok, pp.get("image_mean", (0.5, 0.5, 0.5)), pp.get("image_std", (0.5, 0.5, 0.5)),
                          "bicubic" if pp.get("resample") == 3 else "bilinear")
        elif task == "transcriber":
            import json as _json

            from ..models.whisper import WhisperConfig, WhisperModel
            from ..pipelines.transcription import Transcriber

            if cfg_d.get("model_type") != "whisper":
                raise ModelNotFound(f"{name}: transcribers are Whisper models (found {cfg_d.get('model_type')!r})")
            gen = {}
            gp = os.path.join(path, "generation_config.json")
            if os.path.exists(gp):
                with open(gp, encoding="utf-8") as f:
                    gen = _json.load(f)
            model = WhisperModel.from_state_dict(WhisperConfig.from_hf(cfg_d), sd, device=self.device)
            pipe = Transcriber(model, tok, gen)
        elif task in ("recognizer", "classifier") and any(k.startswith("count_embed.") for k in sd):
            # GLiNER: labels are given per request, one model serves recognition, label scoring and relations
            import json as _json

            from ..models.deberta import DebertaConfig
            from ..models.gliner import GlinerModel
            from ..pipelines.gliner import GlinerConfig, GlinerPipeline

            enc_cfg = cfg_d.get("encoder_config") or cfg_d
            model = GlinerModel.from_state_dict(DebertaConfig.from_hf(enc_cfg), sd, device=self.device)
            added: dict = {}
            ap = os.path.join(path, "added_tokens.json")
            if os.path.exists(ap):
                with open(ap, encoding="utf-8") as f:
                    added = _json.load(f)
            gcfg = dict(cfg_d)
            if "max_len" in gcfg and "max_length" not in gcfg:
                gcfg["max_length"] = gcfg["max_len"]
            pipe = GlinerPipeline(model, tok, GlinerConfig.from_files(gcfg, added))
        elif task == "classifier" and cfg_d.get("model_type") == "layoutlmv3":
            from ..models.layoutlmv3 import LayoutLMv3Config, LayoutLMv3Model
            from ..pipelines.layout import DocumentClassifier

            model = LayoutLMv3Model.from_state_dict(LayoutLMv3Config.from_hf(cfg_d), sd, device=self.device)
            id2label = {int(k): v for k, v in (cfg_d.get("id2label") or {}).items()} or \
                {i: f"LABEL_{i}" for i in range(model.cfg.num_labels)}
            pipe = DocumentClassifier(model, tok, id2label, int(cfg_d.get("bos_token_id", 0) or 0),
                                      int(cfg_d.get("eos_token_id", 2) or 2))
        elif task == "recognizer" and cfg_d.get("model_type") == "layoutlmv3":
            from ..models.layoutlmv3 import LayoutLMv3Config, LayoutLMv3Model
            from ..pipelines.layout import LayoutTokenClassifier

            model = LayoutLMv3Model.from_state_dict(LayoutLMv3Config.from_hf(cfg_d), sd, device=self.device)
            id2label = {int(k): v for k, v in (cfg_d.get("id2label") or {}).items()} or \
                {i: f"LABEL_{i}" for i in range(model.cfg.num_labels)}
            pipe = LayoutTokenClassifier(model, tok, id2label, int(cfg_d.get("bos_token_id", 0) or 0),
                                         int(cfg_d.get("eos_token_id", 2) or 2))
        elif task in ("recognizer", "classifier", "chunker"):
            from ..pipelines.classification import TextClassifier, TokenClassifier

            model = self._encoder(cfg_d, sd)
            id2label = {int(k): v for k, v in (cfg_d.get("id2label") or {}).items()} or \
                {i: f"LABEL_{i}" for i in range(model.cfg.num_labels)}
            if task in ("recognizer", "chunker"):
                pipe = TokenClassifier(model, id2label, tok)
            else:
                pipe = TextClassifier(model, tok, id2label,
                                      multi_label=cfg_d.get("problem_type") == "multi_label_classification")
        elif task in ("embedder", "reranker") and cfg_d.get("model_type") == "colqwen2":
            # page-image retrieval by late interaction over a Qwen2-VL backbone
            from ..models import qwen2vl as QV
            from ..pipelines.vlm import ColQwenEmbedder, Qwen2VLAdapter, VlmTokens

            vd = cfg_d.get("vlm_config") or {}
            text_d = dict(vd.get("text_config") or {k: v for k, v in vd.items() if k != "vision_config"})
            text_d.setdefault("model_type", "qwen2_vl_text")
            core = {k[len("vlm."):] if k.startswith("vlm.") else k: v for k, v in sd.items()}
            model = LlamaModel.from_state_dict(
                LlamaConfig.from_hf(text_d),
                QV.text_state_dict({k: v for k, v in core.items() if not k.startswith("embedding_proj_layer")}),
                device=self.device)
            vision = QV.Qwen2VLVisionModel.from_state_dict(QV.Qwen2VLVisionConfig.from_hf(vd.get("vision_config") or {}),
                                                           core, device=self.device)
            adapter = Qwen2VLAdapter(vision, VlmTokens(int(vd.get("image_token_id", 151655))))
            dt = torch.bfloat16 if self.device.type == "cuda" else torch.float32
            pw = core["embedding_proj_layer.weight"].to(dt).to(self.device)
            pb = core["embedding_proj_layer.bias"].to(dt).to(self.device) if "embedding_proj_layer.bias" in core else None
            pipe = ColQwenEmbedder(model, adapter, pw, pb, tok)
        elif task in ("embedder", "reranker") and cfg_d.get("model_type") == "modernbert":
            from ..models.modernbert import ModernBertConfig, ModernBertModel

            model = ModernBertModel.from_state_dict(ModernBertConfig.from_hf(cfg_d), sd, device=self.device)
            pipe = Embedder(model, tok) if task == "embedder" else CrossEncoderReranker(model, tok)
        elif task in ("embedder", "reranker") and cfg_d.get("model_type") == "deberta-v2":
            from ..models.deberta import DebertaConfig, DebertaModel

            model = DebertaModel.from_state_dict(DebertaConfig.from_hf(cfg_d), sd, device=self.device)
            pipe = Embedder(model, tok) if task == "embedder" else CrossEncoderReranker(model, tok)
        elif task in ("embedder", "reranker"):
            cfg = BertConfig.from_hf(cfg_d)
            model = self._tp(BertModel.from_state_dict(cfg, sd, device=self.device))
            pipe = Embedder(model, tok) if task == "embedder" else CrossEncoderReranker(model, tok)
        else:
            vlm = None
            if cfg_d.get("model_type") in ("gpt2", "gpt_neo", "gpt_neox", "opt", "gptj", "phi", "falcon", "bloom"):
                from ..models.gpt import GptConfig, GptModel

                model = GptModel.from_state_dict(GptConfig.from_hf(cfg_d), sd, device=self.device)
            elif cfg_d.get("model_type") == "qwen2_vl":
                # decoder + vision tower in one checkpoint; images reach the decoder as soft tokens
                import json as _json

                from ..models import qwen2vl as QV
                from ..pipelines.vlm import Qwen2VLAdapter, VlmTokens

                text_d = dict(cfg_d.get("text_config") or {k: v for k, v in cfg_d.items() if k != "vision_config"})
                text_d.setdefault("model_type", "qwen2_vl_text")
                if "rope_scaling" not in text_d and cfg_d.get("rope_scaling"):
                    text_d["rope_scaling"] = cfg_d["rope_scaling"]
                model = LlamaModel.from_state_dict(LlamaConfig.from_hf(text_d), QV.text_state_dict(sd),
                                                   device=self.device)
                vision = QV.Qwen2VLVisionModel.from_state_dict(
                    QV.Qwen2VLVisionConfig.from_hf(cfg_d.get("vision_config") or {}), sd, device=self.device)
                pre = {}
                pp = os.path.join(path, "preprocessor_config.json")
                if os.path.exists(pp):
                    with open(pp, encoding="utf-8") as f:
                        pre = _json.load(f)
                vlm = Qwen2VLAdapter(
                    vision, VlmTokens(int(cfg_d.get("image_token_id", 151655)), cfg_d.get("vision_start_token_id"),
                                      cfg_d.get("vision_end_token_id")),
                    int(pre.get("min_pixels", 56 * 56)), int(pre.get("max_pixels", 14 * 14 * 4 * 1280)))
            elif cfg_d.get("model_type") == "gemma3" and cfg_d.get("vision_config"):
                from ..models.gemma3v import Gemma3VisionModel, SiglipVisionConfig
                from ..models.qwen2vl import text_state_dict
                from ..pipelines.vlm import Gemma3Adapter

                text_d = dict(cfg_d.get("text_config") or {})
                text_d.setdefault("model_type", "gemma3_text")
                model = LlamaModel.from_state_dict(LlamaConfig.from_hf(text_d), text_state_dict(sd), device=self.device)
                vision = Gemma3VisionModel.from_state_dict(
                    SiglipVisionConfig.from_hf(cfg_d["vision_config"]), sd, device=self.device,
                    tokens_per_image=int(cfg_d.get("mm_tokens_per_image", 256)),
                    norm_eps=float(text_d.get("rms_norm_eps", 1e-6)))
                vlm = Gemma3Adapter(vision, int(cfg_d.get("image_token_index", 262144)),
                                    int(cfg_d.get("boi_token_index", 255999)), int(cfg_d.get("eoi_token_index", 256000)),
                                    tok.encode("\n\n"))
            else:
                cfg = LlamaConfig.from_hf(cfg_d)
                model = LlamaModel.from_state_dict(cfg, sd, device=self.device)
            eng = LLMEngine(model, num_blocks=self.kv_blocks, max_batch=self.max_batch,
                            use_cuda_graph=self.device.type == "cuda", eos_token_id=tok.special.eos_id,
                            prefix_cache=self.prefix_cache)
            pipe = Generator(eng, tok, mf.chat_template, vlm=vlm)
        return LoadedModel(name, task, pipe, tok, path, info={"weights": mf.weights, "capabilities": mf.capabilities})

    def _encoder(self, cfg_d: dict, sd):
        """BERT-family / ModernBERT / DeBERTa encoder with its classification head, picked by model_type."""
        mt = cfg_d.get("model_type")
        if "num_labels" not in cfg_d and cfg_d.get("id2label"):
            cfg_d = dict(cfg_d, num_labels=len(cfg_d["id2label"]))
        if mt == "modernbert":
            from ..models.modernbert import ModernBertConfig, ModernBertModel

            return ModernBertModel.from_state_dict(ModernBertConfig.from_hf(cfg_d), sd, device=self.device)
        if mt == "deberta-v2":
            from ..models.deberta import DebertaConfig, DebertaModel

            return DebertaModel.from_state_dict(DebertaConfig.from_hf(cfg_d), sd, device=self.device)
        return self._tp(BertModel.from_state_dict(BertConfig.from_hf(cfg_d), sd, device=self.device))

    def get(self, name: str, task: str) -> LoadedModel:
        key = f"{task}:{name}"
        now = self._clock()
        with self._lock:
            self._evict_idle_locked(now, keep=key)
            if key in self._models:
                self._models.move_to_end(key)
                self._models[key].last_used = now
                return self._models[key]
        path = MF.resolve_model_path(name, self.models_dir, task + "s")
        if path is None:
            raise ModelNotFound(f"model {name!r} not found under {self.models_dir} ({task}s/)")
        self._tls.adapter = None
        lm = self._load_dir(name, task, path)
        ad = self._tls.adapter
        if ad:
            lm.info["adapter"] = {k: v for k, v in ad.items() if k != "path"}
            lm.info["adapter"]["name"] = os.path.basename(ad["path"]) \
                if os.path.basename(os.path.dirname(ad["path"])) == "adapters" else "default"
        lm.last_used = now
        lm.pinned = self.strategies.get(name) == "eager"
        lm.bytes = _param_bytes(lm.pipeline)
        with self._lock:
            self._models[key] = lm
            self._make_room_locked(keep=key)
        return lm

    def get_generator(self, name: str, draft_model: Optional[str] = None,
                      cache_dtype: Optional[str] = None) -> LoadedModel:
        """The generator ``name`` as the request wants it served: with a separate draft model for speculative
        decoding (``draft_model``, loaded like any generator) and / or a KV cache of another dtype
        (``cache_dtype``: f16 / bf16 plain, fp8 / int8 / int4 / polar4 / turbo3 quantised, f32 on the CPU path).
        A variant shares the base model's weights and gets an engine -- KV pool, scheduler, graphs -- of its own;
        variants are cached and evicted like models.  Reference: per-request ``draft_model`` / ``cache_dtype``
        (specs/openapi/inference/api.yaml:2299-2443; zig/pkg/inference/src/runtime/kv/pool.zig:26-35)."""
        from ..runtime.kv_cache import KV_CODECS, KV_DTYPES

        base = self.get(name, "generator")
        kv = None if cache_dtype in (None, "", "bf16", "bfloat16", "f16") else cache_dtype
        if kv is not None and kv not in KV_CODECS and kv not in KV_DTYPES:
            raise ValueError(f"unknown cache_dtype {cache_dtype!r}")
        if kv == "f32" and self.device.type == "cuda":
            raise ValueError("cache_dtype 'f32' is not available on the GPU (the kernels read bf16 or quantised caches)")
        if not draft_model and kv is None:
            return base
        key = f"generator:{name}|draft={draft_model or ''}|kv={kv or ''}"
        now = self._clock()
        with self._lock:
            if key in self._models:
                self._models.move_to_end(key)
                self._models[key].last_used = now
                return self._models[key]
        if not hasattr(base.pipeline, "engine"):
            lm = self._stateful_variant(base, name, draft_model, kv, now)
            with self._lock:
                self._models[key] = lm
                self._make_room_locked(keep=key)
            return lm
        eng0 = base.pipeline.engine
        draft = None
        if draft_model:
            if draft_model == name:
                raise ValueError("draft_model must differ from the model it drafts for")
            draft = self.get(draft_model, "generator").pipeline.engine.model
            if draft.cfg.vocab_size != eng0.model.cfg.vocab_size:
                raise ValueError(f"draft model {draft_model!r} has a different vocabulary than {name!r}")
        eng = LLMEngine(eng0.model, num_blocks=self.kv_blocks, page=eng0.page, max_batch=self.max_batch,
                        use_cuda_graph=self.device.type == "cuda", eos_token_id=eng0.eos,
                        prefix_cache=self.prefix_cache, kv_dtype=kv or "bf16", draft_model=draft)
        pipe = Generator(eng, base.tokenizer, base.pipeline.template.source, add_bos=base.pipeline.add_bos,
                         vlm=base.pipeline.vlm)
        lm = LoadedModel(name, "generator", pipe, base.tokenizer, base.path,
                         info=dict(base.info, draft_model=draft_model, cache_dtype=kv or "bf16"), last_used=now)
        with self._lock:
            self._models[key] = lm
            self._make_room_locked(keep=key)
        return lm

    def _stateful_variant(self, base: LoadedModel, name: str, draft_model: Optional[str], kv: Optional[str],
                          now: float) -> LoadedModel:
        """Variants of a generator that keeps its own per-sequence cache (no paged engine): the only one is Gemma-4
        with its multi-token-prediction assistant as ``draft_model``
        (zig/pkg/inference/src/pipelines/generation.zig:1566, 3028-3110)."""
        from ..models.gemma4 import Gemma4Assistant, Gemma4TextModel
        from ..pipelines.generation import StatefulGenerator

        if kv is not None:
            raise ValueError(f"{name!r} keeps a cache layout of its own; cache_dtype is not available for it")
        target = getattr(base.pipeline.model, "text", base.pipeline.model)
        if not isinstance(target, Gemma4TextModel):
            raise ValueError(f"speculative decoding with a draft model is not available for {name!r}")
        path = MF.resolve_model_path(draft_model, self.models_dir, "generators")
        if path is None:
            raise ModelNotFound(f"model {draft_model!r} not found under {self.models_dir} (generators/)")
        mf = MF.read_manifest(path)
        if mf.config.get("model_type") != "gemma4_assistant":
            raise ValueError(f"{name!r} drafts with a Gemma-4 assistant checkpoint; {draft_model!r} is "
                             f"{mf.config.get('model_type')!r}")
        dt = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        asst = Gemma4Assistant.from_state_dict(mf.config, ST.load_model_dir(path), target, device=self.device, dtype=dt)
        if asst.body.cfg.vocab_size != target.cfg.vocab_size:
            raise ValueError(f"draft model {draft_model!r} has a different vocabulary than {name!r}")
        pipe = StatefulGenerator(base.pipeline.model, base.tokenizer, base.pipeline.template.source,
                                 add_bos=base.pipeline.add_bos, assistant=asst)
        return LoadedModel(name, "generator", pipe, base.tokenizer, base.path,
                           info=dict(base.info, draft_model=draft_model), last_used=now)

    # -- eviction ------------------------------------------------------------------------------------------
    def _drop_locked(self, key: str) -> None:
        self._models.pop(key, None)
        self.evictions += 1

    def _evict_idle_locked(self, now: float, keep: Optional[str] = None) -> int:
        if self.keep_alive_s <= 0:
            return 0
        idle = [k for k, m in self._models.items()
                if k != keep and not m.pinned and now - m.last_used > self.keep_alive_s]
        for k in idle:
            self._drop_locked(k)
        return len(idle)

    def _make_room_locked(self, keep: str) -> None:
        def over() -> bool:
            if self.max_loaded and len(self._models) > self.max_loaded:
                return True
            return bool(self.max_memory_mb) and sum(m.bytes for m in self._models.values()) > self.max_memory_mb << 20

        while over():
            victim = next((k for k, m in self._models.items() if k != keep and not m.pinned), None)
            if victim is None:
                break                      # only pinned models and the new one are left: the limits are advisory
            self._drop_locked(victim)

    def evict_idle(self) -> int:
        """Unload models idle for longer than keep_alive; returns how many were unloaded."""
        with self._lock:
            return self._evict_idle_locked(self._clock())

    def unload(self, name: str, task: str) -> bool:
        with self._lock:
            found = f"{task}:{name}" in self._models
            if found:
                self._drop_locked(f"{task}:{name}")
            return found

    def list_models(self) -> Dict[str, Dict[str, dict]]:
        out: Dict[str, Dict[str, dict]] = {t: {} for t in MF.TASK_DIRS}
        out["extractors"] = {}
        with self._lock:
            for lm in self._models.values():
                out[lm.task + "s"][lm.name] = {"name": lm.name, "loaded": True, **lm.info}
        if os.path.isdir(self.models_dir):
            for t in MF.TASK_DIRS:
                root = os.path.join(self.models_dir, t)
                if not os.path.isdir(root):
                    continue
                for dirpath, dirs, files in os.walk(root):
                    if "config.json" in files or any(f.endswith((".safetensors", ".gguf")) for f in files):
                        nm = os.path.relpath(dirpath, root)
                        out[t].setdefault(nm, {"name": nm, "loaded": False})
                        dirs[:] = []
            # pulled models live under <owner>/<name>; their manifest says what they are
            from .. import registry

            for e in registry.discover(self.models_dir):
                group = e.kind + "s"
                if group in out and not any(e.name in names for names in out.values()):
                    out[group].setdefault(e.name, {"name": e.name, "loaded": False, "variant": e.variant})
        out["chunkers"].setdefault("fixed", {"name": "fixed", "loaded": True})
        return out

    def loaded_count(self) -> int:
        with self._lock:
            return len(self._models)
