"""Command line: ``python -m antfly_b200 <command>`` (the reference's ``antfly inference {run, embed, generate,
...}``, zig/pkg/inference/src/main.zig:92-157; generate / embed flags follow native_generate.zig / native_embed.zig).

  export    safetensors checkpoint -> GGUF    --in DIR --out FILE --quant f32|f16|q8_0|q4_0
  classify / recognize / rewrite            --model NAME --text ...
  compare   embedder parity across devices    --model NAME --text ... --device-a cpu --device-b cuda
  run       start the HTTP server            --host --port --models-dir --preload task:name[:size]
  embed     embed texts                      --model --text ... [--dimensions N] [--print-timing]
  rerank    score documents against a query  --model --query Q --doc ... 
  generate  generate text                    --model --prompt P [--max-tokens --temperature --top-k --top-p --min-p
                                             --repetition-penalty --speculative-k --draft-layers --draft-model --cache-dtype
                                             --prefill-chunk-size --kv-budget-mb --host-budget-mb --backend-budget-mb
                                             --scratch-budget-mb --combined-budget-mb --image --no-bos --no-chat-template
                                             --print-timing --print-token-ids --print-finish-reason]
  search    query a saved index              --index PATH --vector "0.1,0.2,..." | --packed B64 [--k --nprobe]
  quantize  pack a safetensors checkpoint to block-scaled fp8   --in DIR --out FILE
  list      list models                      --models-dir
  smoke     tiny end-to-end run on the GPU
  bench     forwards to bench.py workloads   --workload decode|embed|knn ...

Model names resolve like the server's; ``random:<size>`` builds a random-init model (tiny | base | 8b | 70b).
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List, Optional


def _manager(args):
    from .api.model_manager import ModelManager

    return ModelManager(models_dir=getattr(args, "models_dir", None), device=getattr(args, "device", None),
                        kv_blocks=getattr(args, "kv_blocks", 4096),
                        prefix_cache=not getattr(args, "no_prefix_cache", False))


def _get(mgr, name: str, task: str):
    if name.startswith("random:"):
        size = name.split(":", 1)[1] or "tiny"
        return mgr.register_random(name, task, size)
    return mgr.get(name, task)


def cmd_run(args) -> int:
    from .api.server import serve

    from .api.model_manager import ModelManager
    from .config import load_config

    # file < environment < flags that were given on the command line
    over = {k: v for k, v in (("models_dir", args.models_dir), ("preload", args.preload),
                              ("max_concurrent_requests", args.max_concurrent_requests),
                              ("max_queue_size", args.max_queue_size)) if v is not None}
    if args.host is not None or args.port is not None:
        over["api_url"] = f"http://{args.host or '127.0.0.1'}:{args.port or 11433}"
    elif not args.config:
        over["api_url"] = "http://127.0.0.1:11433"
    cfg = load_config(args.config, **over)
    host, port = cfg.host_port
    from .utils import logs

    logs.event(logs.setup(cfg.log.level, cfg.log.style), 20, "starting", host=host, port=port,
               models_dir=cfg.models_dir, keep_alive=cfg.keep_alive, max_loaded_models=cfg.max_loaded_models)
    mgr = ModelManager(models_dir=cfg.models_dir, device=args.device or cfg.device(), kv_blocks=args.kv_blocks,
                       prefix_cache=not args.no_prefix_cache, max_loaded_models=cfg.max_loaded_models,
                       keep_alive_s=cfg.keep_alive_s, max_memory_mb=cfg.max_memory_mb,
                       strategies=cfg.model_strategies)
    eager = [f"{t}:{n}" for n, s in cfg.model_strategies.items() if s == "eager"
             for t in ("embedder", "reranker", "generator") if _resolvable(mgr, n, t)]
    for spec in list(cfg.preload) + eager:
        task, _, name = spec.partition(":")
        if not name:                       # a bare model name: look it up under every task directory
            name, tasks = task, [t for t in ("embedder", "reranker", "generator") if _resolvable(mgr, task, t)]
        else:
            tasks = [task]
        for t in tasks:
            _get(mgr, name, t)
    serve(host, port, manager=mgr, max_concurrent_requests=cfg.max_concurrent_requests or 64,
          max_queue_size=cfg.max_queue_size or 256, request_timeout_s=cfg.request_timeout_s,
          api_key=cfg.api_key, content_security=dict(cfg.content_security, allow_downloads=cfg.allow_downloads),
          data_dir=cfg.data_dir)
    return 0


def _resolvable(mgr, name: str, task: str) -> bool:
    from .formats import manifest as MF

    return name.startswith("random:") or MF.resolve_model_path(name, mgr.models_dir, task + "s") is not None


def cmd_embed(args) -> int:
    mgr = _manager(args)
    lm = _get(mgr, args.model, "embedder")
    t0 = time.perf_counter()
    rows, ntok = [], 0
    if args.text:
        emb, ntok = lm.pipeline.embed(args.text, dimensions=args.dimensions)
        rows += [("text", r) for r in emb]
    # --image / --audio: files embedded by a dual-tower model into the same space as the texts
    for kind, paths, fn in (("image", args.image, "embed_images"), ("audio", args.audio, "embed_audio")):
        if not paths:
            continue
        if not hasattr(lm.pipeline, fn):
            print(f"model {args.model!r} does not embed {kind} inputs", file=sys.stderr)
            return 2
        e = getattr(lm.pipeline, fn)(paths).cpu()
        if args.dimensions:
            import torch

            e = torch.nn.functional.normalize(e[:, : args.dimensions], dim=-1)
        rows += [(kind, r) for r in e]
    if not rows:
        print("nothing to embed: give --text, --image or --audio", file=sys.stderr)
        return 2
    dt = time.perf_counter() - t0
    for i, (kind, row) in enumerate(rows):
        print(json.dumps({"index": i, "input": kind, "embedding": [round(x, 6) for x in row.tolist()]}))
    if args.print_timing:
        print(f"embed_timing_ms: total={dt * 1e3:.1f} inputs={len(rows)} tokens={ntok}", file=sys.stderr)
    return 0


def cmd_rerank(args) -> int:
    mgr = _manager(args)
    lm = _get(mgr, args.model, "reranker")
    scores, _ = lm.pipeline.rerank(args.query, args.doc)
    for i in sorted(range(len(scores)), key=lambda j: -scores[j]):
        print(json.dumps({"index": i, "score": scores[i], "text": args.doc[i]}))
    return 0


def cmd_generate(args) -> int:
    from .runtime.sampling_params import SamplingParams

    mgr = _manager(args)
    lm = _get(mgr, args.model, "generator")
    if args.draft_model or args.cache_dtype not in (None, "bf16", "f16"):
        # --draft-model: a second generator drafts for speculative decoding; --cache-dtype: KV cache codec
        try:
            lm = mgr.get_generator(args.model, args.draft_model, args.cache_dtype)
        except ValueError as e:
            print(str(e), file=sys.stderr)
            return 2
    gen = lm.pipeline
    eng = getattr(gen, "engine", None)           # None: a model that keeps its own sequence state (no paged engine)
    if eng is None and (args.draft_layers or any((args.kv_budget_mb, args.host_budget_mb, args.backend_budget_mb,
                                                  args.scratch_budget_mb, args.combined_budget_mb))):
        print("--draft-layers and the memory budgets apply to models served by the paged engine", file=sys.stderr)
        return 2
    if args.draft_model and eng is not None:
        eng.spec_k = args.speculative_k
    if args.draft_layers:
        if args.draft_model:
            print("--draft-layers and --draft-model are alternatives", file=sys.stderr)
            return 2
        eng.draft = eng.model.draft_view(args.draft_layers)
        eng.spec_k = args.speculative_k
    if args.no_bos:
        gen.add_bos = False
    if any((args.kv_budget_mb, args.host_budget_mb, args.backend_budget_mb, args.scratch_budget_mb,
            args.combined_budget_mb)):
        from .runtime.tiering import Limits, MemoryBudgetExceeded, budget_for_engine

        try:
            budget_for_engine(eng, Limits.from_mb(args.host_budget_mb, args.backend_budget_mb, args.combined_budget_mb,
                                                  args.kv_budget_mb, args.scratch_budget_mb))
        except MemoryBudgetExceeded as e:
            print(str(e), file=sys.stderr)
            return 3
    sp = SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                        min_p=args.min_p, repetition_penalty=args.repetition_penalty, seed=args.seed,
                        cache_compaction_ratio=args.cache_compaction_ratio)
    if eng is None and args.draft_model:
        sp.speculative_k = args.speculative_k
    out = gen.generate(args.prompt, sp, raw_prompt=args.no_chat_template or args.raw_prompt,
                       on_delta=(lambda d: (sys.stdout.write(d), sys.stdout.flush())) if args.stream else None,
                       images=args.image or None)
    if not args.stream:
        print(out.text)
    else:
        print()
    if args.print_token_ids:
        print("token_ids:", out.token_ids, file=sys.stderr)
    if args.print_finish_reason:
        print("finish_reason:", out.finish_reason, file=sys.stderr)
    if args.print_timing:
        print(out.timing_line(), file=sys.stderr)
        if eng is not None and eng.draft is not None:
            print(eng.spec.line(), file=sys.stderr)
    return 0


def cmd_run_artifact(args) -> int:
    """Generate straight from a compiled artifact file (weights already in the kernels' layout): the reference's
    ``run-artifact`` (zig/pkg/inference/src/native_run_artifact.zig)."""
    import os

    from .models.llama import LlamaModel
    from .pipelines.generation import Generator
    from .runtime.engine import LLMEngine
    from .runtime.sampling_params import SamplingParams
    from .tokenizer import load_tokenizer

    import torch

    device = args.device or ("cuda" if torch.cuda.is_available() else "cpu")
    model = LlamaModel.from_artifact(args.artifact, device=device)
    tok = load_tokenizer(args.tokenizer_dir or os.path.dirname(os.path.abspath(args.artifact)), model.cfg.vocab_size)
    eng = LLMEngine(model, num_blocks=args.kv_blocks, use_cuda_graph=device == "cuda", eos_token_id=tok.special.eos_id)
    out = Generator(eng, tok).generate(args.prompt, SamplingParams(max_tokens=args.max_tokens,
                                                                    temperature=args.temperature, seed=args.seed),
                                       raw_prompt=args.raw_prompt)
    print(out.text)
    if args.print_timing:
        print(out.timing_line(), file=sys.stderr)
    return 0


def cmd_extract(args) -> int:
    """Schema-driven extraction (entities, relations, classifications) over texts: the request the ``/ai/v1/extract``
    endpoint takes, answered in-process (zig/pkg/inference/src/main.zig ``extract``)."""
    from fastapi.testclient import TestClient

    from .api.server import create_app

    schema = {}
    if args.entities:
        schema["entities"] = args.entities
    if args.relations:
        schema["relations"] = [{"type": r} for r in args.relations]
    if args.classify:
        schema["classifications"] = [{"name": "label", "labels": args.classify}]
    if args.schema:
        with open(args.schema, encoding="utf-8") as f:
            schema = json.load(f)
    body = {"model": args.model, "inputs": [{"id": str(i), "content": t} for i, t in enumerate(args.text)],
            "schema": schema, "options": {"threshold": args.threshold, "resolve": args.resolve}}
    r = TestClient(create_app(_manager(args))).post("/ai/v1/extract", json=body)
    print(json.dumps(r.json(), indent=None if args.compact else 2))
    return 0 if r.status_code == 200 else 2


def cmd_cuda_info(args) -> int:
    """Device report in the reference's ``cuda-info`` key: value form (zig/pkg/inference/src/cuda_info.zig), plus
    what this build adds (SM count, memory, library paths); ``--smoke`` runs the tiny end-to-end check."""
    import torch

    if not torch.cuda.is_available():
        print("cuda: unavailable\nreason: no CUDA device visible to this process")
        return 1
    from . import _native as N

    dev = torch.cuda.current_device()
    prop = torch.cuda.get_device_properties(dev)
    print("cuda: available")
    print(f"driver_version: {torch.version.cuda}")
    print(f"device_count: {torch.cuda.device_count()}")
    print(f"selected_device: {dev}")
    print(f"device_name: {prop.name}")
    print(f"compute_capability: sm_{prop.major}{prop.minor}")
    print(f"multiprocessors: {prop.multi_processor_count}")
    print(f"memory_bytes: {prop.total_memory}")
    print(f"artifacts: {N._LIB_DIR}")
    if prop.major != 10:
        print("note: the kernels are built for sm_100a only")
    if args.smoke:
        rc = cmd_smoke(args)
        print("smoke: ok" if rc == 0 else "smoke: failed")
        return rc
    return 0


def cmd_dequant(args) -> int:
    """Raw blocks of one GGUF tensor type on stdin -> fp32 values on stdout (the reference's ``dequant_cli``,
    zig/pkg/inference/src/dequant_cli.zig)."""
    import numpy as np
    import torch

    from .formats import gguf as GG
    from .ops import gguf_ops as G

    names = {v.lower(): k for k, v in GG.TYPE_NAMES.items()}
    key = args.format.lower()
    if key not in names and not key.isdigit():
        print(f"unknown format: {args.format}", file=sys.stderr)
        return 2
    type_id = int(key) if key.isdigit() else names[key]
    try:
        bv, bb = G.block_geometry(type_id)
    except NotImplementedError:
        print(f"no block size for {args.format}", file=sys.stderr)
        return 2
    raw = (open(args.input, "rb") if args.input else sys.stdin.buffer).read()
    if len(raw) % bb:
        print(f"input size {len(raw)} not a multiple of block size {bb}", file=sys.stderr)
        return 2
    n = len(raw) // bb * bv
    out = G.dequantize(torch.from_numpy(np.frombuffer(raw, dtype=np.uint8).copy()), type_id, (n,), torch.float32)
    data = out.numpy().astype("<f4").tobytes()
    if args.output:
        with open(args.output, "wb") as f:
            f.write(data)
    else:
        sys.stdout.buffer.write(data)
        sys.stdout.buffer.flush()
    return 0


def cmd_bench(args) -> int:
    """Forwards to ``bench.py`` at the repository root (one process; multi-GPU runs go through torchrun)."""
    import os
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    return subprocess.call([sys.executable, os.path.join(root, "bench.py")] + list(args.rest))


def cmd_search(args) -> int:
    import torch

    from .index import artifact, codec

    idx = artifact.load_ivf(args.index, device="cuda" if torch.cuda.is_available() else "cpu")
    q = codec.decode_packed(args.packed, idx.dim) if args.packed else codec.decode_vectors(
        [float(x) for x in args.vector.split(",")])
    res = idx.search(q.to(idx.x.device), args.k, nprobe=args.nprobe)
    for d, i in zip(res.distances[0].tolist(), res.ids[0].tolist()):
        print(json.dumps({"id": i, "distance": d}))
    return 0


def cmd_quantize(args) -> int:
    """Pack every 2-D weight of a safetensors checkpoint to block-scaled fp8 (e4m3 + e8m0 per 32 along K)."""
    from .formats import safetensors_io as ST
    from .ops import quant as Q

    sd = ST.load_model_dir(args.inp)
    out = {}
    for name, t in sd.items():
        if t.dim() == 2 and t.shape[1] % 32 == 0 and not name.endswith("embed_tokens.weight"):
            p = Q.pack_fp8(t.float())
            out[name + ".q"], out[name + ".scales"] = p.q.view(t.shape).view(dtype=p.q.dtype), p.scales
        else:
            out[name] = t
    ST.save_file(out, args.out, {"format": "antfly_b200.block_fp8", "block": "32", "scale": "e8m0"})
    print(f"wrote {args.out}: {len(out)} tensors")
    return 0


def cmd_export(args) -> int:
    """Export a Llama-family safetensors checkpoint directory as one GGUF file (f32 / f16, the 32-value block types
    q4_0 .. q8_1 and the K-quants q2_k .. q6_k, q8_k; rows that are not a whole number of blocks stay f16)."""
    import os

    from .formats import gguf as GG
    from .formats import manifest as MF
    from .formats import safetensors_io as ST

    mf = MF.read_manifest(args.inp)
    split = lambda v: [p.strip() for p in (v or "").split(",") if p.strip()] or None
    counts = GG.export_llama_gguf(args.out, ST.load_model_dir(args.inp), mf.config, args.quant,
                                  include=split(args.quantize_include), exclude=split(args.quantize_exclude),
                                  dry_run=args.dry_run)
    print(json.dumps({"out": args.out, "bytes": None if args.dry_run else os.path.getsize(args.out),
                      "tensor_types": counts, "dry_run": args.dry_run}))
    return 0


def cmd_compile_artifact(args) -> int:
    """Pack a Llama-family checkpoint directory into the kernels' own layout (fused, block-fp8) next to the original
    weights; the server then loads that file instead of re-packing at every start."""
    import os

    from .api.model_manager import COMPILED_ARTIFACT
    from .formats import manifest as MF
    from .formats import safetensors_io as ST
    from .models.llama import LlamaConfig, LlamaModel

    t0 = time.perf_counter()
    mf = MF.read_manifest(args.inp)
    model = LlamaModel.from_state_dict(LlamaConfig.from_hf(mf.config), ST.load_model_dir(args.inp),
                                       device=args.device or "cpu")
    out = args.out or os.path.join(args.inp, COMPILED_ARTIFACT)
    model.save_artifact(out)
    print(json.dumps({"out": out, "bytes": os.path.getsize(out), "seconds": round(time.perf_counter() - t0, 2)}))
    return 0


def cmd_classify(args) -> int:
    lm = _manager(args).get(args.model, "classifier")
    for text, ranked in zip(args.text, lm.pipeline.classify(args.text, top_k=args.top_k)):
        print(json.dumps({"text": text, "labels": ranked}))
    return 0


def cmd_recognize(args) -> int:
    lm = _manager(args).get(args.model, "recognizer")
    if hasattr(lm.pipeline, "recognize"):                 # zero-shot span model: the labels come from --labels
        for text, ents in zip(args.text, lm.pipeline.recognize(args.text, args.labels or None,
                                                               threshold=args.threshold)):
            print(json.dumps({"text": text, "entities": [
                {"label": e.label, "text": e.text, "score": round(e.score, 4), "start": e.start, "end": e.end}
                for e in ents]}))
        return 0
    for text, ents in zip(args.text, lm.pipeline.entities(args.text)):
        print(json.dumps({"text": text, "entities": [
            {"label": e.label, "text": e.text, "score": round(e.score, 4), "start_token": e.start_token,
             "end_token": e.end_token} for e in ents]}))
    return 0


def cmd_rewrite(args) -> int:
    from .runtime.sampling_params import SamplingParams

    lm = _manager(args).get(args.model, "rewriter")
    for text in args.text:
        out = lm.pipeline.generate(text, SamplingParams(max_tokens=args.max_tokens), raw_prompt=True)
        print(json.dumps({"input": text, "text": out.text, "tokens": out.completion_tokens}))
        if args.print_timing:
            print(out.timing_line(), file=sys.stderr)
    return 0


def cmd_transcribe(args) -> int:
    lm = _manager(args).get(args.model, "transcriber")
    for path in args.audio:
        out = lm.pipeline.transcribe(path, language=args.language, max_new_tokens=args.max_tokens)
        print(json.dumps({"audio": path, "text": out.text, "segments": [
            {k: v for k, v in s.items() if k != "tokens"} for s in out.segments]}))
        if args.print_timing:
            t = out.timing_ms
            print("transcribe_timing_ms: decode_audio=%.1f transcribe=%.1f total=%.1f" %
                  (t["decode_audio"], t["transcribe"], t["total"]), file=sys.stderr)
    return 0


def cmd_read(args) -> int:
    import numpy as np
    import torch
    from PIL import Image

    lm = _manager(args).get(args.model, "reader")
    imgs = [torch.from_numpy(np.asarray(Image.open(p).convert("RGB")).copy()) for p in args.image]
    for path, r in zip(args.image, lm.pipeline.read(imgs, args.max_tokens, prompt=args.prompt)):
        print(json.dumps({"image": path, "text": r.text}))
    return 0


def cmd_compare(args) -> int:
    """Run the same embedder on two devices (by default the CPU oracle path and the GPU kernels) and report how far
    the embeddings are apart: the parity check a deployment runs after changing hardware or build."""
    import torch

    from .api.model_manager import ModelManager

    devs = [args.device_a, args.device_b or ("cuda" if torch.cuda.is_available() else "cpu")]
    embs = []
    for d in devs:
        mgr = ModelManager(models_dir=args.models_dir, device=d)
        lm = _get(mgr, args.model, "embedder")
        embs.append(lm.pipeline.embed(args.text)[0].float().cpu())
    cos = torch.nn.functional.cosine_similarity(embs[0], embs[1], dim=-1)
    rep = {"model": args.model, "devices": devs, "texts": len(args.text), "min_cosine": float(cos.min()),
           "max_abs_diff": float((embs[0] - embs[1]).abs().max())}
    print(json.dumps(rep))
    return 0 if rep["min_cosine"] >= args.min_cosine else 1


def cmd_list(args) -> int:
    print(json.dumps(_manager(args).list_models(), indent=2))
    return 0


def cmd_finetune(args) -> int:
    """``finetune run recipe.json [--dry-run] [--resume-from DIR]``: the recipe runner (the reference's
    ``finetune run``, zig/pkg/inference/docs/finetuning/FINETUNING.md "Unified Recipes").  Under ``torchrun`` (RANK /
    WORLD_SIZE set) the ranks train data-parallel: gloo on CPU, NCCL on GPUs."""
    import os

    from .finetune import recipes as R

    if args.action == "smoke-fast":
        import tempfile

        root = args.recipe or os.path.join(tempfile.gettempdir(), "antfly-b200-finetune-smoke-fast")
        summary = R.smoke_fast(root)
        print(json.dumps(summary))
        return 0 if summary["ok"] else 1
    if not args.recipe:
        print("finetune run / plan need a recipe file", file=sys.stderr)
        return 2
    with open(args.recipe, encoding="utf-8") as f:
        recipe = json.load(f)
    try:
        if args.dry_run or args.action == "plan":
            print(json.dumps({"recipe": R.normalize(recipe)["recipe"], "steps": R.plan(recipe)}, indent=1))
            return 0
        dist, device = None, args.device or "cpu"
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world > 1:
            import torch
            import torch.distributed as D

            if device.startswith("cuda"):
                device = f"cuda:{os.environ.get('LOCAL_RANK', '0')}"
                torch.cuda.set_device(device)
            D.init_process_group("nccl" if device.startswith("cuda") else "gloo")
            dist = (D.get_rank(), world)
        lead = dist is None or dist[0] == 0

        def log(rec):
            if lead:
                print("step {step} loss {loss:.4f} lr {lr:.2e} grad_norm {grad_norm:.3f}".format(**rec), file=sys.stderr)

        rep = R.run_recipe(recipe, dist, device, args.resume_from, log)
        if lead:
            print(json.dumps({k: rep.get(k) for k in ("status", "train", "eval", "packing") if k in rep}))
        if dist is not None:
            import torch.distributed as D

            D.barrier()
            D.destroy_process_group()
    except R.RecipeError as e:
        print(f"recipe error: {e}", file=sys.stderr)
        return 2
    return 0


def cmd_pull(args) -> int:
    """Fetch a model (``[hf:]owner/name[:variant]``) into the models directory from a hub or a mirror directory
    (the reference's ``pull``, zig/pkg/inference/src/registry/registry.zig:225-251)."""
    from . import registry as R

    last = {"name": None}

    def progress(name, done, total):
        if last["name"] != name:
            last["name"] = name
            print(f"  {name}" + (f" ({total} bytes)" if total else ""), file=sys.stderr)

    try:
        for ref in args.refs:
            dest = R.pull(ref, args.models_dir, R.Hub(args.hub, args.token), args.tasks, args.capabilities, progress)
            print(dest)
    except R.RegistryError as e:
        print(f"pull failed: {e}", file=sys.stderr)
        return 1
    return 0


def cmd_smoke(args) -> int:
    import importlib.util
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("graft_entry", os.path.join(root, "__graft_entry__.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()
    mod.smoke()
    return 0


def cmd_store_bench(args) -> int:
    import tempfile

    from .index.lsm_store import bench

    with tempfile.TemporaryDirectory(dir=args.dir) as d:
        print(json.dumps(bench(d, args.rows, args.value_bytes, args.batch, args.sync)))
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="antfly_b200", description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)

    def common(p):
        p.add_argument("--models-dir")
        p.add_argument("--device")
        p.add_argument("--kv-blocks", type=int, default=4096)
        p.add_argument("--no-prefix-cache", action="store_true",
                       help="do not reuse the KV blocks of prompt prefixes that were prefilled before")

    p = sub.add_parser("run"); common(p)
    p.add_argument("--config", help="YAML / JSON configuration file (api_url, models_dir, keep_alive, "
                                    "max_loaded_models, max_memory_mb, preload, model_strategies, ...)")
    p.add_argument("--host"); p.add_argument("--port", type=int)
    p.add_argument("--preload", nargs="*"); p.add_argument("--max-concurrent-requests", type=int)
    p.add_argument("--max-queue-size", type=int); p.set_defaults(fn=cmd_run)
    p = sub.add_parser("export", help="safetensors checkpoint directory -> GGUF")
    p.add_argument("--in", dest="inp", required=True); p.add_argument("--out", required=True)
    p.add_argument("--quant", default="q8_0", choices=["f32", "f16", "i2_s", "q4_0", "q4_1", "q5_0", "q5_1", "q8_0",
                                                        "q8_1", "q2_k", "q3_k", "q4_k", "q5_k", "q6_k", "q8_k"])
    p.add_argument("--quantize-include", help="comma-separated tensor-name prefixes: quantise only these")
    p.add_argument("--quantize-exclude", help="comma-separated tensor-name prefixes: leave these in f16")
    p.add_argument("--dry-run", action="store_true", help="report the tensor types without writing the file")
    p.set_defaults(fn=cmd_export)
    p = sub.add_parser("compile-artifact", help="pack a checkpoint into the kernels' layout for fast loading")
    p.add_argument("--in", dest="inp", required=True); p.add_argument("--out"); p.add_argument("--device")
    p.set_defaults(fn=cmd_compile_artifact)
    p = sub.add_parser("classify"); common(p)
    p.add_argument("--model", required=True); p.add_argument("--text", nargs="+", required=True)
    p.add_argument("--top-k", type=int, default=1); p.set_defaults(fn=cmd_classify)
    p = sub.add_parser("recognize"); common(p)
    p.add_argument("--model", required=True); p.add_argument("--text", nargs="+", required=True)
    p.add_argument("--labels", nargs="+", default=[]); p.add_argument("--threshold", type=float)
    p.set_defaults(fn=cmd_recognize)
    p = sub.add_parser("rewrite"); common(p)
    p.add_argument("--model", required=True); p.add_argument("--text", nargs="+", required=True)
    p.add_argument("--max-tokens", type=int, default=128); p.add_argument("--print-timing", action="store_true")
    p.set_defaults(fn=cmd_rewrite)
    p = sub.add_parser("transcribe"); common(p)
    p.add_argument("--model", required=True); p.add_argument("--audio", nargs="+", required=True, help="WAV files")
    p.add_argument("--language"); p.add_argument("--max-tokens", type=int, default=224)
    p.add_argument("--print-timing", action="store_true"); p.set_defaults(fn=cmd_transcribe)
    p = sub.add_parser("read", help="OCR: text of each image"); common(p)
    p.add_argument("--model", required=True); p.add_argument("--image", nargs="+", required=True)
    p.add_argument("--prompt", help="task prompt of models that take one (Florence-2: <OCR>, <CAPTION>, ...)")
    p.add_argument("--max-tokens", type=int, default=256); p.set_defaults(fn=cmd_read)
    p = sub.add_parser("compare", help="same embedder on two devices: embedding parity report")
    p.add_argument("--models-dir"); p.add_argument("--model", required=True)
    p.add_argument("--text", nargs="+", required=True); p.add_argument("--device-a", default="cpu")
    p.add_argument("--device-b"); p.add_argument("--min-cosine", type=float, default=0.99)
    p.set_defaults(fn=cmd_compare)
    p = sub.add_parser("embed"); common(p)
    p.add_argument("--model", required=True); p.add_argument("--text", nargs="+", default=[])
    p.add_argument("--image", nargs="+", default=[]); p.add_argument("--audio", nargs="+", default=[])
    p.add_argument("--dimensions", type=int); p.add_argument("--print-timing", action="store_true")
    p.set_defaults(fn=cmd_embed)
    p = sub.add_parser("rerank"); common(p)
    p.add_argument("--model", required=True); p.add_argument("--query", required=True)
    p.add_argument("--doc", nargs="+", required=True); p.set_defaults(fn=cmd_rerank)
    p = sub.add_parser("generate"); common(p)
    p.add_argument("--model", required=True); p.add_argument("--prompt", required=True)
    p.add_argument("--max-tokens", type=int, default=256); p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--top-k", type=int, default=0); p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--min-p", type=float, default=0.0); p.add_argument("--repetition-penalty", type=float, default=1.0)
    p.add_argument("--seed", type=int); p.add_argument("--speculative-k", type=int, default=4)
    p.add_argument("--draft-layers", type=int, default=0)
    p.add_argument("--draft-model", help="a second generator that drafts tokens for speculative decoding")
    p.add_argument("--cache-dtype", default="bf16",
                   choices=["bf16", "f16", "f32", "fp8", "int8", "int4", "polar4", "turbo3"])
    p.add_argument("--prefill-chunk-size", type=int, default=2048); p.add_argument("--kv-budget-mb", type=int, default=0)
    p.add_argument("--cache-compaction-ratio", type=float,
                   help="after prefill keep this fraction of the KV cache (attention-matching compaction)")
    p.add_argument("--no-bos", action="store_true"); p.add_argument("--no-chat-template", action="store_true")
    p.add_argument("--raw-prompt", action="store_true"); p.add_argument("--stream", action="store_true")
    p.add_argument("--image", nargs="+", default=[])
    for flag in ("--host-budget-mb", "--backend-budget-mb", "--scratch-budget-mb", "--combined-budget-mb"):
        p.add_argument(flag, type=int, default=0)
    p.add_argument("--print-timing", action="store_true"); p.add_argument("--print-token-ids", action="store_true")
    p.add_argument("--print-finish-reason", action="store_true"); p.set_defaults(fn=cmd_generate)
    p = sub.add_parser("run-artifact", help="generate from a compiled artifact file")
    p.add_argument("--artifact", required=True); p.add_argument("--prompt", required=True)
    p.add_argument("--tokenizer-dir"); p.add_argument("--device"); p.add_argument("--kv-blocks", type=int, default=1024)
    p.add_argument("--max-tokens", type=int, default=128); p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--seed", type=int); p.add_argument("--raw-prompt", action="store_true")
    p.add_argument("--print-timing", action="store_true"); p.set_defaults(fn=cmd_run_artifact)
    p = sub.add_parser("extract", help="entities / relations / classifications by schema"); common(p)
    p.add_argument("--model", required=True); p.add_argument("--text", nargs="+", required=True)
    p.add_argument("--entities", nargs="*", default=[]); p.add_argument("--relations", nargs="*", default=[])
    p.add_argument("--classify", nargs="*", default=[], help="labels of one classification task")
    p.add_argument("--schema", help="JSON file with the full schema"); p.add_argument("--threshold", type=float, default=0.0)
    p.add_argument("--resolve", action="store_true"); p.add_argument("--compact", action="store_true")
    p.set_defaults(fn=cmd_extract)
    p = sub.add_parser("cuda-info", help="device report"); p.add_argument("--smoke", action="store_true")
    p.set_defaults(fn=cmd_cuda_info)
    p = sub.add_parser("dequant", help="GGUF blocks on stdin -> fp32 on stdout")
    p.add_argument("format", help="tensor type name (q4_k, iq2_xs, ...) or id"); p.add_argument("--input")
    p.add_argument("--output"); p.set_defaults(fn=cmd_dequant)
    sub.add_parser("kv-distortion", help="score error of the quantised KV-cache key codecs")
    p = sub.add_parser("bench", help="forwards its arguments to bench.py")
    p.add_argument("rest", nargs=argparse.REMAINDER); p.set_defaults(fn=cmd_bench)
    p = sub.add_parser("search")
    p.add_argument("--index", required=True); p.add_argument("--vector"); p.add_argument("--packed")
    p.add_argument("--k", type=int, default=10); p.add_argument("--nprobe", type=int, default=64)
    p.set_defaults(fn=cmd_search)
    p = sub.add_parser("quantize")
    p.add_argument("--in", dest="inp", required=True); p.add_argument("--out", required=True)
    p.set_defaults(fn=cmd_quantize)
    p = sub.add_parser("list"); common(p); p.set_defaults(fn=cmd_list)
    p = sub.add_parser("finetune", help="run a fine-tuning recipe (LoRA / QLoRA SFT, DPO, GRPO, reranker, embedder)")
    p.add_argument("action", choices=["run", "plan", "smoke-fast"])
    p.add_argument("recipe", nargs="?", help="recipe JSON file (smoke-fast: output directory, optional)")
    p.add_argument("--dry-run", action="store_true", help="print the plan and stop")
    p.add_argument("--resume-from", help="checkpoint directory of an earlier run of the same recipe")
    p.add_argument("--device"); p.set_defaults(fn=cmd_finetune)
    p = sub.add_parser("pull", help="fetch models into the models directory")
    p.add_argument("refs", nargs="+", help="[hf:]owner/name[:variant] (auto, gguf, gguf:Q4_K_M, safetensors, mmproj)")
    p.add_argument("--models-dir"); p.add_argument("--token")
    p.add_argument("--hub", help="hub URL, or a mirror directory laid out owner/name ($HF_ENDPOINT by default)")
    p.add_argument("--tasks", help="comma-separated tasks for the manifest (embed, rerank, generate, ...)")
    p.add_argument("--capabilities", help="comma-separated capabilities for the manifest")
    p.set_defaults(fn=cmd_pull)
    p = sub.add_parser("store-bench", help="write / read throughput of the log-structured merge store")
    p.add_argument("--dir", default=None); p.add_argument("--rows", type=int, default=200_000)
    p.add_argument("--value-bytes", type=int, default=256); p.add_argument("--batch", type=int, default=500)
    p.add_argument("--sync", action="store_true"); p.set_defaults(fn=cmd_store_bench)
    p = sub.add_parser("smoke"); p.set_defaults(fn=cmd_smoke)
    raw = list(sys.argv[1:] if argv is None else argv)
    if raw and raw[0] == "bench":              # everything after the command belongs to bench.py, options included
        return cmd_bench(argparse.Namespace(rest=raw[1:]))
    if raw and raw[0] == "kv-distortion":      # score error of the KV-cache key codecs (utils/kv_distortion.py)
        from .utils import kv_distortion
        kv_distortion.main(raw[1:])
        return 0
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
