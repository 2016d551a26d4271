"""Request / response models of the inference API (specs/openapi/inference/api.yaml: EmbedRequest :740,
EmbedResponse :800, RerankRequest :999, RerankResponse :1054, GenerateRequest :2299, GenerateResponse :2472,
GenerateChunk, ModelsResponse :2099, Error :722) and the vector-search subset of the DB QueryRequest
(specs/openapi/antfly/metadata.yaml:4077-4420)."""
from __future__ import annotations

from typing import Any, Dict, List, Literal, Optional, Union

from pydantic import BaseModel, ConfigDict, Field


class ContentPart(BaseModel):
    model_config = ConfigDict(extra="allow")
    type: str
    text: Optional[str] = None


class EmbedRequest(BaseModel):
    model: str
    input: Union[str, List[str], List[ContentPart]]
    encoding_format: Literal["float"] = "float"
    dimensions: Optional[int] = Field(default=None, gt=0)
    task_type: Optional[str] = None
    input_type: Optional[str] = None


class SparseVector(BaseModel):
    indices: List[int]
    values: List[float]


class EmbeddingObject(BaseModel):
    object: Literal["embedding"] = "embedding"
    embedding: Union[List[float], SparseVector]
    index: int


class EmbeddingUsage(BaseModel):
    prompt_tokens: int
    total_tokens: int


class EmbedResponse(BaseModel):
    object: Literal["list"] = "list"
    data: List[EmbeddingObject]
    model: str
    usage: EmbeddingUsage


class RerankRequest(BaseModel):
    model: str
    query: str
    prompts: List[str]


class RerankObject(BaseModel):
    object: Literal["rerank.score"] = "rerank.score"
    index: int
    score: float


class GenerateUsage(BaseModel):
    prompt_tokens: int
    completion_tokens: int
    total_tokens: int


class RerankResponse(BaseModel):
    object: Literal["list"] = "list"
    data: List[RerankObject]
    model: str
    usage: GenerateUsage


class ChatMessage(BaseModel):
    model_config = ConfigDict(extra="allow")
    role: str
    content: Union[str, List[ContentPart], None] = None


class GenerateRequest(BaseModel):
    model_config = ConfigDict(extra="allow")
    model: str
    messages: List[ChatMessage]
    max_tokens: int = 256
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    stop: Union[str, List[str], None] = None
    seed: Optional[int] = None
    stream: bool = False
    draft_model: Optional[str] = None
    speculative_k: Optional[int] = Field(default=None, ge=1, le=16)
    cache_dtype: Optional[Literal["f16", "f32", "int8", "fp8", "int4", "bf16"]] = None
    cache_compaction_ratio: Optional[float] = None
    backend: Optional[str] = None
    mode: Optional[str] = None
    grammar: Optional[str] = None
    response_format: Optional[Dict[str, Any]] = None
    compiled_target: Optional[str] = None       # the reference's compiled-graph hint (partitioned | whole-model); no effect here
    tools: Optional[List[Dict[str, Any]]] = None
    tool_choice: Optional[Union[str, Dict[str, Any]]] = None


class GenerateMessage(BaseModel):
    role: str = "assistant"
    content: Optional[str] = None
    tool_calls: Optional[List[Dict[str, Any]]] = None


class GenerateChoice(BaseModel):
    index: int = 0
    message: GenerateMessage
    finish_reason: str


class GenerateResponse(BaseModel):
    id: str
    object: Literal["chat.completion"] = "chat.completion"
    created: int
    model: str
    choices: List[GenerateChoice]
    usage: GenerateUsage


class ChunkRequest(BaseModel):
    """``input`` (a string, or a content part: ``{"type": "text", "text": ...}`` /
    ``{"type": "media", "mime_type": "audio/wav", "data": <base64>}``) with ``config`` {model, max_chunks, threshold,
    text: {target_tokens, overlap_tokens, separator}, audio: {window_duration_ms, overlap_duration_ms}}; ``text``
    and the flat option fields are the older spelling and still accepted."""
    input: Union[str, Dict[str, Any], None] = None
    text: Optional[str] = None
    config: Dict[str, Any] = Field(default_factory=dict)
    model: Optional[str] = None
    target_tokens: Optional[int] = None
    overlap_tokens: Optional[int] = None
    max_chunks: Optional[int] = None


class ErrorBody(BaseModel):
    error: str
    message: str


class SearchRequest(BaseModel):
    """Vector-search subset of QueryRequest: one dense query per index name, or packed base64 little-endian f32."""
    model_config = ConfigDict(extra="allow")
    index: str
    embeddings: Union[List[List[float]], List[float], str, None] = None
    semantic_search: Optional[str] = None
    embedder: Optional[str] = None
    limit: int = Field(default=10, gt=0)
    search_effort: float = 0.5
    distance_under: Optional[float] = None
    distance_over: Optional[float] = None


class SearchHit(BaseModel):
    id: int
    distance: float


class SearchResponse(BaseModel):
    hits: List[List[SearchHit]]
    took_ms: float
    index: str


class TableCreateRequest(BaseModel):
    """Subset of the table-creation body: one dense embedding index (dimension, metric, embedder model, exact or
    HBC) and an optional sparse index."""
    model_config = ConfigDict(extra="allow")
    dimension: Optional[int] = None
    metric: str = "cosine"
    embedder: Optional[str] = None
    index_type: str = "flat"            # flat | hbc | hnsw (neighbors, ef_construction, ef_search as extra fields)
    reranker: Optional[str] = None
    text_field: str = "text"


class BatchRequest(BaseModel):
    model_config = ConfigDict(extra="allow")
    inserts: Dict[str, Dict[str, Any]] = Field(default_factory=dict)
    deletes: List[str] = Field(default_factory=list)
    embeddings: Optional[Dict[str, List[float]]] = None     # precomputed dense vectors per inserted key


class TableQueryRequest(BaseModel):
    """Hybrid-search subset of QueryRequest (metadata.yaml:4077-4400)."""
    model_config = ConfigDict(extra="allow")
    semantic_search: Optional[str] = None
    full_text_search: Union[str, Dict[str, Any], None] = None
    embeddings: Union[Dict[str, Any], List[float], str, None] = None
    limit: int = Field(default=10, gt=0)
    offset: int = Field(default=0, ge=0)
    search_effort: float = 0.5
    distance_under: Optional[float] = None
    distance_over: Optional[float] = None
    merge_config: Optional[Dict[str, Any]] = None
    pruner: Optional[Dict[str, Any]] = None
    reranker: Optional[Dict[str, Any]] = None
    fields: Optional[List[str]] = None
    filter_prefix: Optional[str] = None
    filter_query: Union[str, Dict[str, Any], None] = None
    exclusion_query: Union[str, Dict[str, Any], None] = None
    order_by: Optional[List[Dict[str, Any]]] = None
    search_after: Optional[List[str]] = None
    count: bool = False
    profile: bool = False
    aggregations: Optional[Dict[str, Dict[str, Any]]] = None


class ClassifyRequest(BaseModel):
    model_config = ConfigDict(extra="allow")
    model: str
    texts: List[str]
    labels: List[str] = Field(default_factory=list)
    hypothesis_template: Optional[str] = None
    multi_label: bool = False


class RecognizeRequest(BaseModel):
    model_config = ConfigDict(extra="allow")
    model: str
    texts: List[str]
    labels: List[str] = Field(default_factory=list)
    relation_labels: List[str] = Field(default_factory=list)
    threshold: Optional[float] = None
    resolver: Optional[Dict[str, Any]] = None


class RewriteRequest(BaseModel):
    model_config = ConfigDict(extra="allow")
    model: str
    inputs: List[str]
    max_tokens: int = Field(default=128, gt=0)


class ExtractionInput(BaseModel):
    model_config = ConfigDict(extra="allow")
    id: Optional[str] = None
    content: Union[str, List[Dict[str, Any]]]


class ExtractionRequest(BaseModel):
    """Schema-driven extraction (specs/openapi/ai/extraction.yaml): entity labels for a token-classification
    model, classification tasks for a sequence-classification model."""
    model_config = ConfigDict(extra="allow", protected_namespaces=())
    model: str
    inputs: List[ExtractionInput]
    schema_: Dict[str, Any] = Field(alias="schema")
    options: Dict[str, Any] = Field(default_factory=dict)


class TranscribeRequest(BaseModel):
    model_config = ConfigDict(extra="allow")
    model: str
    audio: str                          # base64-encoded WAV
    language: Optional[str] = None
    task: str = "transcribe"
    max_tokens: int = Field(default=224, gt=0)


class RerankMultimodalDocument(BaseModel):
    model_config = ConfigDict(extra="allow")
    id: Optional[str] = None
    content: Union[str, List[Dict[str, Any]]]


class RerankMultimodalRequest(BaseModel):
    model_config = ConfigDict(extra="allow")
    model: str
    query: str
    documents: List[RerankMultimodalDocument]


class LayoutPage(BaseModel):
    model_config = ConfigDict(extra="allow")
    words: List[str]
    boxes: List[List[float]]                       # one [x0, y0, x1, y1] per word
    width: Optional[float] = None                  # page size the boxes are measured in; without it boxes are 0..1000
    height: Optional[float] = None
    image: Optional[Union[str, Dict[str, Any]]] = None   # data URL of the page, optional


class LayoutRequest(BaseModel):
    model_config = ConfigDict(extra="allow")
    model: str
    pages: List[LayoutPage]
    group: bool = True                             # join B- / I- tagged words into fields


class ReadRequest(BaseModel):
    model_config = ConfigDict(extra="allow")
    model: str
    images: List[Union[str, Dict[str, Any]]]      # {"url": "data:image/png;base64,..."} or the data URL itself
    prompt: Optional[str] = None
    max_tokens: int = Field(default=256, gt=0)
