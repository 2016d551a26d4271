"""Model references, discovery of the models directory and ``pull`` from a model hub.

What the reference does (zig/pkg/inference/src/registry/registry.zig:53-84 references, :100-223 discovery, :225-251
pull, :725-816 the manifest written after a pull; registry/download.zig:44-187 file lists and quant preference,
:800-905 which files a variant needs):

* a reference is ``[hf:]owner/name[:variant]``; the variant is ``auto``, ``gguf``, ``gguf:<QUANT>``, ``mmproj``,
  ``safetensors``, or one of the ONNX names;
* the hub lists a repository's files (``/api/models/<owner>/<name>``, with size and LFS sha256) and serves them under
  ``/<owner>/<name>/resolve/main/<file>``;
* configuration and tokenizer files are always taken; of the weights, one GGUF file (the requested quantisation, else
  the first of a preference list that favours small deployable files), and / or the safetensors payload (an index
  with all of its shards, else the single file);
* the model lands in ``models_dir/<owner>/<name>``; when it has no ``model_manifest.json`` (or tasks / capabilities
  were given) one is written with the type derived from the tasks.

This build has no ONNX lane, so ONNX payloads are never selected: ``auto`` means GGUF and / or safetensors, and an
explicit ONNX variant falls back to safetensors as the reference's legacy rule does.  Besides ``http(s)://`` the hub
can be a directory (or ``file://`` URL) laid out ``<root>/<owner>/<name>/...``: a mirror on local or shared storage,
which is what an air-gapped deployment pulls from.
"""
from __future__ import annotations

import hashlib
import json
import os
import urllib.error
import urllib.parse
import urllib.request
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Sequence

from .formats import manifest as MF

ALWAYS_FILES = (
    "config.json", "clip_config.json", "generation_config.json", "processor_config.json",
    "preprocessor_config.json", "tokenizer.json", "tokenizer_config.json", "special_tokens_map.json",
    "tokenizer.model", "vocab.txt", "vocab.json", "merges.txt", "modules.json",
    "config_sentence_transformers.json", "1_SpladePooling/config.json", "1_Pooling/config.json",
    "chat_template.jinja", "added_tokens.json", "model_manifest.json", "antfly_metadata.json",
    "antfly_inference_variants.json",
)
SAFETENSORS_INDEXES = ("model.safetensors.index.json", "pytorch_model.safetensors.index.json")
SAFETENSORS_FILES = ("model.safetensors", "pytorch_model.safetensors")
GGUF_QUANT_PREFERENCE = ("Q4_K_S", "UD-Q4_K_S", "Q4_K", "Q4_K_M", "UD-Q4_K_M", "UD-Q4_K_XL", "Q5_K_S", "Q5_K_M",
                         "Q6_K", "Q8_0", "Q3_K_M", "Q2_K")
PROJECTOR_PREFERENCE = ("f16", "bf16", "q8_0", "q6_k", "q5_k_m", "q4_k_m")
ONNX_VARIANTS = ("onnx", "f32", "i8")
KINDS = ("embedder", "chunker", "reranker", "generator", "recognizer", "classifier", "rewriter", "reader",
         "transcriber", "extractor")
# first match wins, in this order
_TASK_TYPES = (("recognize", "recognizer"), ("extract", "recognizer"), ("classify", "classifier"),
               ("rerank", "reranker"), ("read", "reader"), ("transcribe", "transcriber"), ("rewrite", "rewriter"),
               ("chunk", "chunker"), ("generate", "generator"), ("embed", "embedder"))
_TYPE_TASK = {"embedder": "embed", "reranker": "rerank", "generator": "generate", "chunker": "chunk",
              "recognizer": "recognize", "classifier": "classify", "rewriter": "rewrite", "reader": "read",
              "transcriber": "transcribe", "extractor": "extract"}


class RegistryError(RuntimeError):
    pass


@dataclass(frozen=True)
class ModelRef:
    owner: str
    name: str
    variant: str = "auto"

    @staticmethod
    def parse(ref: str) -> "ModelRef":
        text = ref[3:] if ref.startswith("hf:") else ref
        variant = "auto"
        if ":" in text:
            text, variant = text.split(":", 1)
        if "/" not in text:
            raise RegistryError(f"invalid model reference {ref!r}: expected owner/name[:variant]")
        owner, name = text.split("/", 1)
        if not owner or not name or not variant:
            raise RegistryError(f"invalid model reference {ref!r}: expected owner/name[:variant]")
        return ModelRef(owner, name, variant)


@dataclass
class HubFile:
    name: str
    size: Optional[int] = None
    sha256: Optional[str] = None


# ----------------------------------------------------------------------------------------------------------
# which files a variant needs
# ----------------------------------------------------------------------------------------------------------
def _is_gguf(name: str) -> bool:
    return name.lower().endswith(".gguf")


def _is_projector(name: str) -> bool:
    base = os.path.basename(name).lower()
    return _is_gguf(name) and ("mmproj" in base or "projector" in base)


def _quant_matches(name: str, quant: str) -> bool:
    """``quant`` as a whole tag of the file name: delimited by ``-``, ``.`` or ``_`` on the left and ``.`` / ``-`` on
    the right, so Q4_K does not claim a Q4_K_M file."""
    base = os.path.basename(name)
    stem = base[:-5] if _is_gguf(base) else base
    up, q = stem.upper(), quant.upper()
    i = up.find(q)
    while i >= 0:
        left_ok = i == 0 or up[i - 1] in "-._"
        j = i + len(q)
        right_ok = j == len(up) or up[j] in ".-"
        if left_ok and right_ok:
            return True
        i = up.find(q, i + 1)
    return False


def _gguf_group(files: Sequence[HubFile], first: HubFile) -> List[HubFile]:
    """A split GGUF (``-00001-of-00003``) travels whole."""
    base = first.name
    marker = base.lower().rfind("-of-")
    if marker < 0:
        return [first]
    prefix = base[: base.lower().rfind("-", 0, marker)]
    return sorted((f for f in files if _is_gguf(f.name) and f.name.startswith(prefix + "-")), key=lambda f: f.name)


def select_gguf(files: Sequence[HubFile], quant: Optional[str]) -> List[HubFile]:
    cands = sorted((f for f in files if _is_gguf(f.name) and not _is_projector(f.name)), key=lambda f: f.name)
    if not cands:
        return []
    if quant:
        for f in cands:
            if _quant_matches(f.name, quant):
                return _gguf_group(files, f)
        return []
    for q in GGUF_QUANT_PREFERENCE:
        for f in cands:
            if _quant_matches(f.name, q):
                return _gguf_group(files, f)
    return _gguf_group(files, cands[0])


def select_projector(files: Sequence[HubFile]) -> List[HubFile]:
    cands = [f for f in files if _is_projector(f.name)]
    for tag in PROJECTOR_PREFERENCE:
        for f in cands:
            if _quant_matches(f.name, tag):
                return [f]
    return cands[:1]


def select_safetensors(files: Sequence[HubFile], shards_of: Callable[[str], Iterable[str]]) -> List[HubFile]:
    """The index with every shard it names (``shards_of`` reads the index's weight map), else the single file."""
    by_name = {f.name: f for f in files}
    for idx in SAFETENSORS_INDEXES:
        if idx in by_name:
            out = [by_name[idx]]
            for shard in sorted(set(shards_of(idx))):
                if shard not in by_name:
                    raise RegistryError(f"{idx} names {shard}, which the repository does not list")
                out.append(by_name[shard])
            return out
    for name in SAFETENSORS_FILES:
        if name in by_name:
            return [by_name[name]]
    return []


def select_files(files: Sequence[HubFile], variant: str,
                 shards_of: Callable[[str], Iterable[str]] = lambda idx: ()) -> List[HubFile]:
    variant = variant or "auto"
    want_mmproj = variant in ("mmproj", "projector")
    want_gguf = variant == "gguf" or variant.startswith("gguf:")
    want_onnx = variant in ONNX_VARIANTS
    want_st = variant == "safetensors" or variant in ("hybrid", "onnx+native", "native+onnx") or want_onnx
    auto = not (want_mmproj or want_gguf or want_st)
    if auto and variant != "auto":
        raise RegistryError(f"unknown variant {variant!r}")
    by_name = {f.name: f for f in files}
    out: List[HubFile] = []
    if not want_mmproj:
        out += [by_name[n] for n in ALWAYS_FILES if n in by_name]
        out += [f for f in files if os.path.basename(f.name) in ("adapter_config.json", "adapter_model.safetensors")]
    payload: List[HubFile] = []
    if want_gguf or auto:
        payload += select_gguf(files, variant[5:] if variant.startswith("gguf:") else None)
    if want_mmproj:
        payload += select_projector(files)
    if want_st or auto:
        payload += select_safetensors(files, shards_of)
    if not payload:
        raise RegistryError(f"no model files for variant {variant!r} in the repository"
                            + (" (ONNX payloads are not served by this build)" if want_onnx else ""))
    seen, uniq = set(), []
    for f in out + payload:
        if f.name not in seen:
            seen.add(f.name)
            uniq.append(f)
    return uniq


# ----------------------------------------------------------------------------------------------------------
# the hub: HTTP (the public API layout) or a mirror directory
# ----------------------------------------------------------------------------------------------------------
class Hub:
    """``base_url``: ``https://...`` / ``http://...`` (listing under ``/api/models``, files under ``/resolve/main``)
    or a directory / ``file://`` URL holding ``<owner>/<name>/`` trees."""

    def __init__(self, base_url: Optional[str] = None, token: Optional[str] = None, timeout: float = 30.0):
        base_url = base_url or os.environ.get("HF_ENDPOINT") or "https://huggingface.co"
        self.token, self.timeout = token or os.environ.get("HF_TOKEN"), timeout
        if base_url.startswith("file://"):
            base_url = urllib.parse.unquote(urllib.parse.urlparse(base_url).path)
        self.local = not base_url.startswith(("http://", "https://"))
        self.base = base_url.rstrip("/")

    def _open(self, url: str, headers: Optional[Dict[str, str]] = None):
        req = urllib.request.Request(url, headers=dict(headers or {}))
        if self.token:
            req.add_header("Authorization", f"Bearer {self.token}")
        try:
            return urllib.request.urlopen(req, timeout=self.timeout)
        except urllib.error.HTTPError as e:
            if e.code in (401, 403):
                raise RegistryError(f"{url}: access denied (HTTP {e.code}); a token is needed") from e
            if e.code == 404:
                raise RegistryError(f"{url}: not found") from e
            raise RegistryError(f"{url}: HTTP {e.code}") from e
        except (urllib.error.URLError, OSError) as e:
            raise RegistryError(f"{url}: {getattr(e, 'reason', e)}") from e

    def list_files(self, ref: ModelRef) -> List[HubFile]:
        if self.local:
            root = os.path.join(self.base, ref.owner, ref.name)
            if not os.path.isdir(root):
                raise RegistryError(f"{root}: not found")
            out = []
            for d, _, names in os.walk(root):
                for n in names:
                    p = os.path.join(d, n)
                    out.append(HubFile(os.path.relpath(p, root).replace(os.sep, "/"), os.path.getsize(p)))
            return sorted(out, key=lambda f: f.name)
        with self._open(f"{self.base}/api/models/{ref.owner}/{ref.name}?blobs=true") as r:
            info = json.load(r)
        out = []
        for s in info.get("siblings") or []:
            lfs = s.get("lfs") or {}
            out.append(HubFile(s["rfilename"], lfs.get("size", s.get("size")), lfs.get("sha256") or lfs.get("oid")))
        return out

    def read_small(self, ref: ModelRef, name: str) -> bytes:
        if self.local:
            with open(os.path.join(self.base, ref.owner, ref.name, name), "rb") as f:
                return f.read()
        with self._open(f"{self.base}/{ref.owner}/{ref.name}/resolve/main/{urllib.parse.quote(name)}") as r:
            return r.read()

    def fetch(self, ref: ModelRef, f: HubFile, dest: str, progress: Optional[Callable[[str, int, Optional[int]], None]]
              = None) -> None:
        """Into ``dest`` through ``dest + '.part'``; an interrupted transfer resumes from the bytes already there (a
        Range request), and a listed sha256 is checked before the rename."""
        os.makedirs(os.path.dirname(dest) or ".", exist_ok=True)
        if os.path.exists(dest) and (f.size is None or os.path.getsize(dest) == f.size) and \
                (f.sha256 is None or _sha256(dest) == f.sha256):
            if progress:
                progress(f.name, f.size or os.path.getsize(dest), f.size)
            return
        part = dest + ".part"
        have = os.path.getsize(part) if os.path.exists(part) else 0
        if f.size is not None and have > f.size:
            have = 0
        if self.local:
            src = os.path.join(self.base, ref.owner, ref.name, f.name)
            with open(src, "rb") as r, open(part, "ab" if have else "wb") as w:
                r.seek(have)
                done = have
                while True:
                    buf = r.read(8 << 20)
                    if not buf:
                        break
                    w.write(buf)
                    done += len(buf)
                    if progress:
                        progress(f.name, done, f.size)
        else:
            url = f"{self.base}/{ref.owner}/{ref.name}/resolve/main/{urllib.parse.quote(f.name)}"
            with self._open(url, {"Range": f"bytes={have}-"} if have else None) as r:
                resumed = have and r.status == 206
                with open(part, "ab" if resumed else "wb") as w:
                    done = have if resumed else 0
                    while True:
                        buf = r.read(1 << 20)
                        if not buf:
                            break
                        w.write(buf)
                        done += len(buf)
                        if progress:
                            progress(f.name, done, f.size)
        got = os.path.getsize(part)
        if f.size is not None and got != f.size:
            raise RegistryError(f"{f.name}: {got} bytes received, {f.size} expected (run the pull again to resume)")
        if f.sha256 is not None and _sha256(part) != f.sha256:
            os.remove(part)
            raise RegistryError(f"{f.name}: sha256 mismatch")
        os.replace(part, dest)


def _sha256(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for buf in iter(lambda: f.read(8 << 20), b""):
            h.update(buf)
    return h.hexdigest()


# ----------------------------------------------------------------------------------------------------------
# manifest of a pulled model
# ----------------------------------------------------------------------------------------------------------
def manifest_type(tasks: Sequence[str], fallback: str) -> str:
    for task, kind in _TASK_TYPES:
        if task in tasks:
            return kind
    return fallback


def _csv(text: Optional[str]) -> List[str]:
    out: List[str] = []
    for t in (text or "").split(","):
        t = t.strip()
        if t and t not in out:
            out.append(t)
    return out


def synthesize_manifest(model_dir: str, tasks: Optional[str] = None, capabilities: Optional[str] = None) -> dict:
    m = MF.read_manifest(model_dir)
    kind = m.model_type
    task_list = _csv(tasks) or [_TYPE_TASK.get(t, t) for t in m.tasks] or [_TYPE_TASK.get(kind, "embed")]
    caps = list(m.capabilities)
    cfg = m.config
    inputs = ["text"]
    if "vision_config" in cfg or os.path.exists(os.path.join(model_dir, "preprocessor_config.json")):
        inputs.append("image")
    if "audio_config" in cfg or cfg.get("model_type") in ("whisper", "clap", "wav2vec2"):
        inputs.append("audio")
    if "generate" in task_list and m.chat_template and "chat" not in caps:
        caps.append("chat")
    if "image" in inputs and "generate" in task_list and "vision" not in caps:
        caps.append("vision")
    for c in _csv(capabilities):
        if c not in caps:
            caps.append(c)
    out = {"type": manifest_type(task_list, kind), "tasks": task_list}
    if caps:
        out["capabilities"] = caps
    if inputs != ["text"]:
        out["inputs"] = inputs
    return out


def pull(ref_text: str, models_dir: Optional[str] = None, hub: Optional[Hub] = None, tasks: Optional[str] = None,
         capabilities: Optional[str] = None, progress: Optional[Callable[[str, int, Optional[int]], None]] = None
         ) -> str:
    """Fetch what ``ref_text`` names into ``models_dir/<owner>/<name>``; returns that directory."""
    ref = ModelRef.parse(ref_text)
    hub = hub or Hub()
    root = os.path.realpath(models_dir or MF.default_models_dir())
    dest = os.path.join(root, ref.owner, ref.name)
    files = hub.list_files(ref)

    def shards_of(index_name: str):
        return json.loads(hub.read_small(ref, index_name)).get("weight_map", {}).values()

    chosen = select_files(files, ref.variant, shards_of)
    os.makedirs(dest, exist_ok=True)
    for f in chosen:
        target = os.path.normpath(os.path.join(dest, f.name))
        if not target.startswith(dest + os.sep):
            raise RegistryError(f"{f.name}: path leaves the model directory")
        hub.fetch(ref, f, target, progress)
    has_manifest = os.path.exists(os.path.join(dest, "model_manifest.json"))
    if not has_manifest or tasks or capabilities:
        body = synthesize_manifest(dest, tasks, capabilities)
        with open(os.path.join(dest, "model_manifest.json"), "w", encoding="utf-8") as w:
            json.dump(body, w)
    return dest


# ----------------------------------------------------------------------------------------------------------
# discovery
# ----------------------------------------------------------------------------------------------------------
@dataclass
class ModelEntry:
    name: str
    kind: str
    path: str
    variant: str


def _is_model_dir(path: str) -> bool:
    try:
        names = os.listdir(path)
    except OSError:
        return False
    return "config.json" in names or "model_manifest.json" in names or any(
        n.endswith((".gguf", ".safetensors")) for n in names)


def _entry(path: str, name: str, hint: Optional[str]) -> ModelEntry:
    try:
        m = MF.read_manifest(path)
        kind = manifest_type([_TYPE_TASK.get(t, t) for t in m.tasks], hint or m.model_type) if m.tasks else \
            (hint or m.model_type)
        variant = m.weights or "none"
    except (OSError, ValueError):
        kind, variant = hint or "embedder", "none"
    return ModelEntry(name, kind, path, variant)


def discover(models_dir: Optional[str] = None) -> List[ModelEntry]:
    """Models under ``models_dir``: ``<owner>/<name>`` and bare ``<name>`` directories, then the per-task layout
    ``<task>s/<name>`` and ``<task>s/<owner>/<name>`` (whose directory gives the kind)."""
    root = models_dir or MF.default_models_dir()
    out: List[ModelEntry] = []
    seen = set()

    def add(path, name, hint=None):
        real = os.path.realpath(path)
        if real not in seen and _is_model_dir(path):
            seen.add(real)
            out.append(_entry(path, name, hint))
            return True
        return False

    def walk(base, prefix, hint):
        if not os.path.isdir(base):
            return
        for a in sorted(os.listdir(base)):
            pa = os.path.join(base, a)
            if not os.path.isdir(pa) or (hint is None and a in MF.TASK_DIRS):
                continue
            if add(pa, prefix + a, hint):
                continue
            for b in sorted(os.listdir(pa)):
                pb = os.path.join(pa, b)
                if os.path.isdir(pb):
                    add(pb, f"{prefix}{a}/{b}", hint)

    walk(root, "", None)
    for t in MF.TASK_DIRS:
        walk(os.path.join(root, t), "", t[:-1])
    return out


def resolve_variant(models_dir: str, requested: str) -> Optional[str]:
    """``owner/name[:variant]`` or a bare name -> the directory that holds it, if it is there."""
    name = requested[3:] if requested.startswith("hf:") else requested
    name = name.split(":", 1)[0]
    return MF.resolve_model_path(name, models_dir)
