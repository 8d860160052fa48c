"""FastAPI application: ``POST /v1/chat/completions``, ``POST /v1/messages``, ``GET /health``, ``GET /stats``, ``GET /v1/models``, ``POST /v1/completions``.

Request schemas and defaults follow ``astrai/inference/network/app.py:33-206`` (OpenAI: temperature 1.0, top_p 1.0,
top_k 50, max_tokens 2048; Anthropic: max_tokens 1024; 503 ``{"detail": "Engine not initialized"}`` before the engine
exists).  The engine is created with the paged KV cache and radix prefix index on; page size, cache size and the prefill
token budget are server options.
"""

from __future__ import annotations

import logging
from contextlib import asynccontextmanager
from pathlib import Path
from typing import Any, Dict, List, Optional, Union

import torch
from fastapi import APIRouter, FastAPI, HTTPException
from pydantic import BaseModel, Field, model_validator

from astrai_b200.inference.engine import InferenceEngine
from astrai_b200.inference.network.anthropic import AnthropicResponseBuilder
from astrai_b200.inference.network.openai import OpenAIResponseBuilder
from astrai_b200.inference.network.protocol import ProtocolHandler

logger = logging.getLogger(__name__)
_app: Optional[FastAPI] = None


class ChatMessage(BaseModel):
    role: str
    content: Optional[str] = None
    tool_calls: Optional[List[Dict[str, Any]]] = None
    tool_call_id: Optional[str] = None


class FunctionDef(BaseModel):
    name: str
    description: Optional[str] = None
    parameters: Optional[Dict[str, Any]] = None


class ToolDef(BaseModel):
    type: str = "function"
    function: FunctionDef


class ChatCompletionRequest(BaseModel):
    model: str = "astrai"
    messages: List[ChatMessage]
    temperature: Optional[float] = Field(default=1.0, ge=0.0, le=2.0)
    top_p: Optional[float] = Field(default=1.0, ge=0.0, le=1.0)
    top_k: Optional[int] = Field(default=50, ge=1)
    stream: Optional[bool] = False
    stop: Optional[Union[str, List[str]]] = None
    max_tokens: Optional[int] = Field(default=2048, ge=1)
    max_completion_tokens: Optional[int] = Field(default=None, ge=1)  # the newer OpenAI name; wins over max_tokens when given
    n: Optional[int] = Field(default=1, ge=1)
    presence_penalty: Optional[float] = Field(default=0.0, ge=-2.0, le=2.0)
    frequency_penalty: Optional[float] = Field(default=0.0, ge=-2.0, le=2.0)
    logit_bias: Optional[Dict[int, float]] = None
    user: Optional[str] = None
    tools: Optional[List[ToolDef]] = None
    tool_choice: Optional[Union[str, Dict[str, Any]]] = "auto"

    @model_validator(mode="after")
    def _one_token_budget(self):
        if self.max_completion_tokens is not None:
            self.max_tokens = self.max_completion_tokens
        return self


class CompletionRequest(BaseModel):
    model: str = "astrai"
    prompt: Union[str, List[str]]
    max_tokens: Optional[int] = Field(default=16, ge=1)
    temperature: Optional[float] = Field(default=1.0, ge=0.0, le=2.0)
    top_p: Optional[float] = Field(default=1.0, ge=0.0, le=1.0)
    top_k: Optional[int] = Field(default=50, ge=1)
    frequency_penalty: Optional[float] = Field(default=0.0, ge=-2.0, le=2.0)
    stream: Optional[bool] = False
    stop: Optional[Union[str, List[str]]] = None
    echo: Optional[bool] = False


class AnthropicMessage(BaseModel):
    role: str
    content: Union[str, List[Dict[str, Any]]]


class MessagesRequest(BaseModel):
    model: str = "astrai"
    max_tokens: int = Field(default=1024, ge=1)
    messages: List[AnthropicMessage]
    system: Optional[str] = None
    temperature: Optional[float] = Field(default=1.0, ge=0.0, le=2.0)
    top_p: Optional[float] = Field(default=1.0, ge=0.0, le=1.0)
    top_k: Optional[int] = Field(default=50, ge=1)
    stream: Optional[bool] = False
    stop_sequences: Optional[List[str]] = None


def create_engine(param_path: Path, device: str = "cuda", dtype: torch.dtype = torch.bfloat16, max_batch_size: int = 16,
                  max_seq_len: Optional[int] = None, page_size: int = 16, kv_cache_tokens: Optional[int] = None,
                  paged: bool = True, max_prefill_tokens: int = 8192, enable_cuda_graph: bool = True,
                  **scheduler_kwargs) -> InferenceEngine:
    """Model + tokenizer from ``param_path`` behind an engine.  ``scheduler_kwargs`` go to the scheduler unchanged
    (``chunked_prefill``, ``prefill_defer_steps`` ...)."""
    from astrai_b200.models import AutoModel
    from astrai_b200.tokenize import AutoTokenizer

    param_path = Path(param_path)
    if not param_path.exists():
        raise FileNotFoundError(f"Parameter directory not found: {param_path}")
    tokenizer = AutoTokenizer.from_pretrained(param_path)
    model = AutoModel.from_pretrained(param_path).to(device=device, dtype=dtype).eval()
    return InferenceEngine(model=model, tokenizer=tokenizer, max_batch_size=max_batch_size, max_seq_len=max_seq_len,
                           enable_cuda_graph=enable_cuda_graph, page_size=page_size, kv_cache_tokens=kv_cache_tokens,
                           paged=paged, max_prefill_tokens=max_prefill_tokens, **scheduler_kwargs)


@asynccontextmanager
async def lifespan(app: FastAPI):
    cfg = dict(app.state.server_config)
    if not cfg.pop("_test", False):
        app.state.engine = create_engine(**cfg)
    yield
    if app.state.engine:
        app.state.engine.shutdown()


router = APIRouter()


def get_app() -> FastAPI:
    """The process-wide app, built on first use (importing this module creates nothing)."""
    global _app
    if _app is None:
        _app = FastAPI(title="astrai_b200 inference server", version="0.1.0", lifespan=lifespan)
        _app.include_router(router)
        _app.state.server_config = {}
        _app.state.engine = None
    return _app


def _engine() -> InferenceEngine:
    engine = get_app().state.engine
    if engine is None:
        raise HTTPException(status_code=503, detail="Engine not initialized")
    return engine


@router.get("/health")
async def health():
    return {"status": "ok", "model_loaded": get_app().state.engine is not None}


@router.get("/stats")
async def stats():
    return _engine().get_stats()


@router.get("/v1/models")
async def models():
    """The one model this server holds, in the shape OpenAI clients list models in (not a route of the reference; clients
    such as SDKs and UIs call it before their first request)."""
    _engine()
    name = Path(str(get_app().state.server_config.get("param_path") or "astrai")).name or "astrai"
    return {"object": "list", "data": [{"id": name, "object": "model", "created": 0, "owned_by": "astrai_b200"}]}


@router.post("/v1/chat/completions")
async def chat_completion(request: ChatCompletionRequest):
    return await ProtocolHandler(request, _engine(), OpenAIResponseBuilder()).handle()


@router.post("/v1/completions")
async def completion(request: CompletionRequest):
    from astrai_b200.inference.network.completions import CompletionResponseBuilder

    return await ProtocolHandler(request, _engine(), CompletionResponseBuilder()).handle()


@router.post("/v1/messages")
async def create_message(request: MessagesRequest):
    return await ProtocolHandler(request, _engine(), AnthropicResponseBuilder()).handle()


def run_tensor_parallel_server(param_path: Path, tp_size: int, host: str = "0.0.0.0", port: int = 8000, device: str = "cuda",
                               dtype: torch.dtype = torch.bfloat16, max_batch_size: int = 16, max_seq_len: Optional[int] = None,
                               **engine_kwargs):
    """One serving replica over ``tp_size`` processes (launch with ``python -m torch.distributed.run --nproc-per-node
    tp_size -m astrai_b200.cli.serve --tp_size tp_size ...``): every rank loads the checkpoint and keeps its share of every
    layer; the first rank runs the HTTP front end, the others follow its scheduling loop until it shuts down."""
    import os

    import uvicorn

    from astrai_b200.parallel.setup import setup_parallel

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world != tp_size:
        raise RuntimeError(f"--tp_size {tp_size} needs exactly that many processes (torchrun --nproc-per-node {tp_size}); found {world}")
    cuda = str(device).startswith("cuda")
    with setup_parallel(rank, world, local, "nccl" if cuda else "gloo", os.environ.get("MASTER_ADDR", "127.0.0.1"),
                        os.environ.get("MASTER_PORT", "29500"), "cuda" if cuda else "cpu"):
        engine = create_engine(param_path, device=f"cuda:{local}" if cuda else "cpu", dtype=dtype, max_batch_size=max_batch_size,
                               max_seq_len=max_seq_len, tp_size=tp_size, **engine_kwargs)
        if rank != 0:
            engine.follow()
            return
        app = get_app()
        app.state.server_config = {"_test": True}  # the engine exists already: the lifespan hook must not build another
        app.state.engine = engine
        try:
            uvicorn.run(app, host=host, port=port)
        finally:
            app.state.engine = None
            engine.shutdown()


def run_server(param_path: Path, host: str = "0.0.0.0", port: int = 8000, reload: bool = False, device: str = "cuda",
               dtype: torch.dtype = torch.bfloat16, max_batch_size: int = 16, max_seq_len: Optional[int] = None, **engine_kwargs):
    import uvicorn

    tp_size = int(engine_kwargs.pop("tp_size", 1) or 1)
    if tp_size > 1:
        return run_tensor_parallel_server(param_path, tp_size, host=host, port=port, device=device, dtype=dtype,
                                          max_batch_size=max_batch_size, max_seq_len=max_seq_len, **engine_kwargs)
    app = get_app()
    app.state.server_config = {"device": device, "dtype": dtype, "param_path": param_path, "max_batch_size": max_batch_size,
                               "max_seq_len": max_seq_len, **engine_kwargs}
    uvicorn.run(app, host=host, port=port, reload=reload)
