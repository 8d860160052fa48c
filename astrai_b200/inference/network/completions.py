"""OpenAI ``/v1/completions`` wire format: plain text in, plain text out (no chat template).

Not a route of the reference (its server speaks the two chat protocols only); evaluation harnesses and older clients
use it.  It is the same :class:`~astrai_b200.inference.network.protocol.ProtocolHandler` loop with a third builder: the
prompt is the request's text as it stands, a stop sequence ends the text before its first character,
``finish_reason`` is ``length`` when the token budget ran out and ``stop`` otherwise.
"""

from __future__ import annotations

import time
import uuid
from typing import Any, Dict, List, Optional

from astrai_b200.inference.network.protocol import GenContext, ResponseBuilder, StopInfo, sse_event


class CompletionResponseBuilder(ResponseBuilder):
    def prepare(self, request, engine):
        prompt = request.prompt if isinstance(request.prompt, str) else "".join(request.prompt)
        self._id, self._model = f"cmpl-{uuid.uuid4().hex[:12]}", request.model
        self._echo = prompt if getattr(request, "echo", False) else ""
        stop = request.stop
        stops = [] if stop is None else ([stop] if isinstance(stop, str) else list(stop))
        return prompt, GenContext(self._id, int(time.time()), self._model), stops

    def _object(self, text: str, created: int, finish: Optional[str]) -> Dict[str, Any]:
        return {"id": self._id, "object": "text_completion", "created": created, "model": self._model,
                "choices": [{"index": 0, "text": text, "logprobs": None, "finish_reason": finish}]}

    @staticmethod
    def _reason(ctx: GenContext, stop: StopInfo) -> str:
        """``length`` when the engine ended the answer for want of room (token budget or context), ``stop`` otherwise."""
        return "length" if stop.matched is None and ctx.finish_reason == "length" else "stop"

    @staticmethod
    def _usage(ctx: GenContext) -> Dict[str, int]:
        return {"prompt_tokens": ctx.prompt_tokens, "completion_tokens": ctx.completion_tokens,
                "total_tokens": ctx.prompt_tokens + ctx.completion_tokens}

    @staticmethod
    def _before_stop(stop: StopInfo) -> str:
        return stop.body if stop.matched is None else stop.body[: stop.body.index(stop.matched)]

    def format_stream_start(self, ctx):
        return [sse_event(self._object(self._echo, ctx.created, None))] if self._echo else []

    def format_chunk(self, token, **kw):
        return [sse_event(self._object(token, 0, None))]

    def format_stream_end(self, ctx, stop):
        events: List[str] = []
        rest = self._before_stop(stop)[len(stop.yielded):]  # text of the piece that completed a stop sequence, up to the sequence
        if rest:
            events.append(sse_event(self._object(rest, 0, None)))
        last = self._object("", ctx.created, self._reason(ctx, stop))
        last["usage"] = self._usage(ctx)
        return events + [sse_event(last)]

    def format_response(self, ctx, content, stop):
        out = self._object(self._echo + self._before_stop(stop), ctx.created, self._reason(ctx, stop))
        out["usage"] = self._usage(ctx)
        return out
