"""OpenAI ``/v1/chat/completions`` wire format (reference ``astrai/inference/network/openai.py:51-277``).

Stream: role chunk -> content / tool-call chunks (``created: 0`` on middle chunks) -> finish chunk
(``finish_reason`` ``stop``, ``tool_calls``, or ``length`` when the engine ran out of token budget or context: the
reference says ``stop`` there too) -> a bare usage object.  ``n``, ``presence_penalty``, ``logit_bias`` and
``user`` are accepted and ignored with a warning.
"""

from __future__ import annotations

import logging
import time
import uuid
from typing import Any, Dict, List, Optional

from astrai_b200.inference.network.protocol import GenContext, ResponseBuilder, StopInfo, sse_event
from astrai_b200.inference.network.tool_parser import BaseToolParser, ToolParserFactory

logger = logging.getLogger(__name__)
IGNORED_PARAMS = ("n", "presence_penalty", "logit_bias", "user")


class OpenAIResponseBuilder(ResponseBuilder):
    def prepare(self, request, engine):
        messages = [{"role": m.role, "content": m.content} for m in request.messages]
        raw_tools = getattr(request, "tools", None) or []
        tools = [t.model_dump() if hasattr(t, "model_dump") else t for t in raw_tools] or None
        prompt = engine.tokenizer.apply_chat_template(messages, tokenize=False, tools=tools or [])
        self._id, self._model = f"chatcmpl-{uuid.uuid4().hex[:12]}", request.model
        fields = getattr(type(request), "model_fields", {})
        for name in IGNORED_PARAMS:
            value = getattr(request, name, None)
            default = fields[name].default if name in fields else None
            if value is not None and value != default:
                logger.warning("ChatCompletionRequest param '%s'=%r is not supported and will be ignored", name, value)
        self._parser: Optional[BaseToolParser] = None
        if tools:
            choice = getattr(request, "tool_choice", None)
            choice = choice if isinstance(choice, (str, dict)) else "auto"
            self._parser = ToolParserFactory.create("simple_json", tools=tools, tool_choice=choice)
        self._role_sent = False
        stop = request.stop
        stops = [] if stop is None else ([stop] if isinstance(stop, str) else list(stop))
        return prompt, GenContext(self._id, int(time.time()), self._model), stops

    def _chunk(self, delta: Dict[str, Any], created: int = 0, finish: Optional[str] = None) -> str:
        return sse_event({"id": self._id, "object": "chat.completion.chunk", "created": created, "model": self._model,
                          "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]})

    def format_stream_start(self, ctx):
        return [self._chunk({"role": "assistant"}, ctx.created)]

    def format_chunk(self, token, **kw):
        if self._parser is None:
            return [self._chunk({"content": token})]
        events: List[str] = []
        for delta in self._parser.feed(kw.get("body", ""), current_token_ids=kw.get("current_token_ids"),
                                       delta_token_ids=kw.get("delta_token_ids")):
            key = "content" if "content" in delta else ("tool_calls" if "tool_calls" in delta else None)
            if key is None:
                continue
            if not self._role_sent:
                self._role_sent = True
                events.append(self._chunk({"role": "assistant"}))
            events.append(self._chunk({key: delta[key]}))
        return events

    @staticmethod
    def _usage(ctx: GenContext) -> Dict[str, int]:
        return {"prompt_tokens": ctx.prompt_tokens, "completion_tokens": ctx.completion_tokens,
                "total_tokens": ctx.prompt_tokens + ctx.completion_tokens}

    @staticmethod
    def _plain_reason(ctx: GenContext, stop) -> str:
        return "length" if stop.matched is None and ctx.finish_reason == "length" else "stop"

    def format_stream_end(self, ctx, stop):
        reason = "tool_calls" if (self._parser is not None and self._parser.has_tool_calls) else self._plain_reason(ctx, stop)
        return [self._chunk({}, ctx.created, reason), sse_event(self._usage(ctx))]

    def format_response(self, ctx, content, stop):
        message: Dict[str, Any] = {"role": "assistant", "content": content}
        reason = self._plain_reason(ctx, stop)
        parsed = self._parser.parse_complete(content) if self._parser is not None else None
        if parsed and parsed.get("tool_calls"):
            message = {"role": "assistant", "content": parsed.get("content"), "tool_calls": parsed["tool_calls"]}
            reason = "tool_calls"
        return {"id": self._id, "object": "chat.completion", "created": ctx.created, "model": self._model,
                "choices": [{"index": 0, "message": message, "finish_reason": reason}], "usage": self._usage(ctx)}
