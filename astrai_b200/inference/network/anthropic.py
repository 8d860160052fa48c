"""Anthropic ``/v1/messages`` wire format (reference ``astrai/inference/network/anthropic.py:28-142``).

Stream: ``message_start``, ``content_block_start``, ``content_block_delta``*, (text still unsent before a matched stop
sequence), ``content_block_stop``, ``message_delta`` (``end_turn`` | ``stop_sequence``), ``message_stop``.
"""

from __future__ import annotations

import time
import uuid
from typing import Any, Dict, List, Union

from astrai_b200.inference.network.protocol import GenContext, ResponseBuilder, StopInfo, sse_event


def first_text(content: Union[str, List[Dict[str, Any]]]) -> str:
    if isinstance(content, str):
        return content
    for block in content if isinstance(content, list) else ():
        if isinstance(block, dict) and block.get("type") == "text":
            return block.get("text", "")
    return ""


def _delta(text: str) -> str:
    return sse_event({"type": "content_block_delta", "index": 0, "delta": {"type": "text_delta", "text": text}},
                     event="content_block_delta")


class AnthropicResponseBuilder(ResponseBuilder):
    def prepare(self, request, engine):
        messages = []
        if getattr(request, "system", None):
            messages.append({"role": "system", "content": request.system})
        for m in request.messages:
            text = first_text(m.content)
            if text:
                messages.append({"role": m.role, "content": text})
        prompt = engine.tokenizer.apply_chat_template(messages, tokenize=False)
        ctx = GenContext(f"msg_{uuid.uuid4().hex[:24]}", int(time.time()), request.model)
        return prompt, ctx, list(getattr(request, "stop_sequences", None) or [])

    def format_stream_start(self, ctx):
        start = {"type": "message_start", "message": {"id": ctx.resp_id, "type": "message", "role": "assistant",
                                                       "model": ctx.model, "content": [],
                                                       "usage": {"input_tokens": ctx.prompt_tokens}}}
        block = {"type": "content_block_start", "index": 0, "content_block": {"type": "text", "text": ""}}
        return [sse_event(start, event="message_start"), sse_event(block, event="content_block_start")]

    def format_chunk(self, token, **kw):
        return [_delta(token)]

    @staticmethod
    def _stop_reason(ctx, stop) -> str:
        """``stop_sequence``, ``max_tokens`` (the engine ran out of token budget or context; the reference says
        ``end_turn`` there too) or ``end_turn``."""
        if stop.matched:
            return "stop_sequence"
        return "max_tokens" if ctx.finish_reason == "length" else "end_turn"

    def format_stream_end(self, ctx, stop):
        events = []
        if stop.matched:
            pending = stop.body[: stop.body.rfind(stop.matched)][len(stop.yielded):]
            if pending:
                events.append(_delta(pending))
        events.append(sse_event({"type": "content_block_stop", "index": 0}, event="content_block_stop"))
        events.append(sse_event({"type": "message_delta",
                                 "delta": {"stop_reason": self._stop_reason(ctx, stop),
                                           "stop_sequence": stop.matched},
                                 "usage": {"output_tokens": ctx.completion_tokens}}, event="message_delta"))
        events.append(sse_event({"type": "message_stop"}, event="message_stop"))
        return events

    def format_response(self, ctx, content, stop):
        if stop.matched:
            content = content[: content.rfind(stop.matched)]
        return {"id": ctx.resp_id, "type": "message", "role": "assistant", "model": ctx.model,
                "content": [{"type": "text", "text": content}],
                "stop_reason": self._stop_reason(ctx, stop), "stop_sequence": stop.matched,
                "usage": {"input_tokens": ctx.prompt_tokens, "output_tokens": ctx.completion_tokens}}
