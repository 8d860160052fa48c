"""Protocol-independent request handling: run the generation, watch for stop sequences, hand text to a builder.

Loop and event order follow ``astrai/inference/network/protocol.py:18-197``: stop sequences are matched as substrings of
the accumulated text and the matching piece is not emitted; a stream always ends with ``data: [DONE]``.
"""

from __future__ import annotations

import json
from contextlib import aclosing
from dataclasses import dataclass, field
from typing import Any, AsyncGenerator, Dict, List, Optional, Tuple, Union

from fastapi.responses import StreamingResponse
from pydantic import BaseModel


def sse_event(data: Dict[str, Any], event: Optional[str] = None) -> str:
    head = f"event: {event}\n" if event else ""
    return f"{head}data: {json.dumps(data, ensure_ascii=False)}\n"


def sse_done() -> str:
    return "data: [DONE]\n\n"


@dataclass
class GenContext:
    resp_id: str
    created: int
    model: str
    prompt_tokens: int = 0
    completion_tokens: int = 0
    finish_reason: Optional[str] = None  # "stop" / "length" once the engine ran the request to its end; None if cut short
    engine_usage: Dict[str, Any] = field(default_factory=dict)

    def settle(self, matched: Optional[str]):
        """After the last piece: take the engine's token count (the handler counted pieces of text, and a token that gives
        no text of its own was not among them) unless a stop sequence ended the answer before the engine did."""
        if matched is None and self.engine_usage:
            self.completion_tokens = max(self.completion_tokens, int(self.engine_usage.get("completion_tokens", 0)))
            self.finish_reason = self.engine_usage.get("finish_reason")


@dataclass
class StopInfo:
    matched: Optional[str] = None
    body: str = ""
    yielded: str = ""


class StopChecker:
    def __init__(self, sequences: List[str]):
        self._sequences = [s for s in sequences if s]

    def check(self, text: str) -> Optional[str]:
        return next((s for s in self._sequences if s in text), None)


class ResponseBuilder:
    """A wire protocol = five formatting methods."""

    def prepare(self, request: BaseModel, engine) -> Tuple[str, GenContext, List[str]]:
        raise NotImplementedError

    def format_stream_start(self, ctx: GenContext) -> List[str]:
        raise NotImplementedError

    def format_chunk(self, token: str, **kwargs) -> List[str]:
        raise NotImplementedError

    def format_stream_end(self, ctx: GenContext, stop: StopInfo) -> List[str]:
        raise NotImplementedError

    def format_response(self, ctx: GenContext, content: str, stop: StopInfo) -> Dict[str, Any]:
        raise NotImplementedError


class ProtocolHandler:
    def __init__(self, request: BaseModel, engine, builder: ResponseBuilder):
        self.request, self.engine, self.builder = request, engine, builder

    async def handle(self) -> Union[StreamingResponse, Dict[str, Any]]:
        prompt, ctx, stops = self.builder.prepare(self.request, self.engine)
        ctx.prompt_tokens = len(self.engine.tokenizer.encode(prompt))
        r = self.request
        agen = self.engine.generate_async(prompt=prompt, max_tokens=r.max_tokens, temperature=r.temperature, top_p=r.top_p,
                                          top_k=r.top_k, frequency_penalty=getattr(r, "frequency_penalty", 0.0) or 0.0,
                                          usage=ctx.engine_usage)
        if r.stream:
            return StreamingResponse(self._events(agen, ctx, stops), media_type="text/event-stream",
                                     headers={"Cache-Control": "no-cache", "Connection": "keep-alive"})
        return await self._collect(agen, ctx, stops)

    async def _events(self, agen: AsyncGenerator, ctx: GenContext, stops: List[str]):
        checker = StopChecker(stops)
        for ev in self.builder.format_stream_start(ctx):
            yield ev
        body = sent = ""
        matched = None
        ids: List[int] = []
        # closing the generator (a stop sequence matched, or the client went away and this coroutine was cancelled) takes
        # the request out of the scheduler
        async with aclosing(agen) as pieces:
            async for piece in pieces:
                body += piece
                new_ids = self.engine.tokenizer.encode(piece)
                ids.extend(new_ids)
                matched = checker.check(body)
                if matched:
                    break
                ctx.completion_tokens += 1
                for ev in self.builder.format_chunk(piece, body=body, current_token_ids=ids, delta_token_ids=new_ids):
                    yield ev
                sent += piece
        ctx.settle(matched)
        for ev in self.builder.format_stream_end(ctx, StopInfo(matched, body, sent)):
            yield ev
        yield sse_done()

    async def _collect(self, agen: AsyncGenerator, ctx: GenContext, stops: List[str]) -> Dict[str, Any]:
        checker = StopChecker(stops)
        body, matched = "", None
        async with aclosing(agen) as pieces:
            async for piece in pieces:
                body += piece
                matched = checker.check(body)
                if matched:
                    break
                ctx.completion_tokens += 1
        ctx.settle(matched)
        return self.builder.format_response(ctx, body, StopInfo(matched, body))
