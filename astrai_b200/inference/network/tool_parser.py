"""Incremental extraction of tool calls from generated text.

The built-in parser recognises ``{"name": "<function>", "arguments": {...}}`` objects anywhere in the output and
streams them as OpenAI-style deltas: text before the first call as ``content``, then for each call one delta carrying
its id + name and further deltas carrying the growth of its argument string.  Observable behaviour (including the
argument string being the INNER text of the arguments object) follows ``astrai/inference/network/tool_parser.py:19-339``.
"""

from __future__ import annotations

import json
import re
import uuid
from typing import Dict, List, Optional, Tuple

from astrai_b200.factory import BaseFactory


class BaseToolParser:
    """One instance per request; ``feed`` receives the full text generated so far on every call."""

    def __init__(self, tools: Optional[List[Dict]] = None, tool_choice="auto"):
        self.tools = tools or []
        self.tool_choice = tool_choice

    def feed(self, body: str, current_token_ids: Optional[List[int]] = None,
             delta_token_ids: Optional[List[int]] = None) -> List[Dict]:
        raise NotImplementedError

    def parse_complete(self, body: str) -> Optional[Dict]:
        raise NotImplementedError

    @property
    def has_tool_calls(self) -> bool:
        raise NotImplementedError


class ToolParserFactory(BaseFactory["BaseToolParser"]):
    pass


def _object_end(text: str, start: int) -> Tuple[int, bool]:
    """Index one past the brace closing the object that opens at ``start`` (string- and escape-aware)."""
    depth, in_str, esc = 0, False, False
    for i in range(start, len(text)):
        ch = text[i]
        if esc:
            esc = False
        elif ch == "\\":
            esc = True
        elif ch == '"':
            in_str = not in_str
        elif not in_str:
            if ch == "{":
                depth += 1
            elif ch == "}":
                depth -= 1
                if depth == 0:
                    return i + 1, True
    return len(text), False


def _argument_text(args) -> str:
    if isinstance(args, dict):
        return json.dumps(args, ensure_ascii=False)[1:-1].rstrip() if args else ""
    if isinstance(args, list):
        return json.dumps(args, ensure_ascii=False) if args else ""
    if isinstance(args, str):
        return args
    return "" if args is None else str(args)


def _complete_call(blob: str) -> Optional[Tuple[str, str]]:
    try:
        obj = json.loads(blob)
    except json.JSONDecodeError:
        return None
    name = obj.get("name") if isinstance(obj, dict) else None
    if not isinstance(name, str) or not name:
        return None
    return name, _argument_text(obj.get("arguments"))


def _partial_call(blob: str) -> Optional[Tuple[str, str]]:
    m = re.search(r'"name"\s*:\s*"([^"]*)"', blob)
    if not m:
        return None
    a = re.search(r'"arguments"\s*:\s*(.*)', blob, re.DOTALL)
    if not a:
        return m.group(1), ""
    raw = a.group(1).rstrip()
    if raw.startswith("{"):
        raw = raw[1:].rstrip()
        if raw.endswith("}"):
            raw = raw[:-1].rstrip()
    return m.group(1), raw


def find_tool_calls(text: str, start: int = 0) -> List[Dict]:
    """Every complete tool-call object from ``start`` on; scanning stops at the first unclosed object."""
    found, pos = [], start
    while True:
        brace = text.find("{", pos)
        if brace < 0:
            return found
        end, closed = _object_end(text, brace)
        if not closed:
            return found
        call = _complete_call(text[brace:end])
        if call is not None:
            found.append({"start": brace, "end": end, "name": call[0], "args": call[1], "complete": True})
        pos = end


def find_partial_tool_call(text: str, start: int = 0) -> Optional[Dict]:
    brace = text.find("{", start)
    if brace < 0 or '"name"' not in text[brace:]:
        return None
    call = _partial_call(text[brace:])
    if call is None or call[0] is None:
        return None
    return {"start": brace, "name": call[0], "args": call[1], "complete": False}


_CALL_HEAD = re.compile(r'^\{\s*(?:"(?:n(?:a(?:m(?:e(?:"(?:\s*(?::(?:\s*(?:"[^"]*)?)?)?)?)?)?)?)?)?)?$')


@ToolParserFactory.register("simple_json")
class SimpleJsonToolParser(BaseToolParser):
    def __init__(self, tools=None, tool_choice="auto"):
        super().__init__(tools, tool_choice)
        self._content_sent = 0
        self._calls: List[Dict] = []
        self._seen = False

    def feed(self, body, current_token_ids=None, delta_token_ids=None):
        done = find_tool_calls(body)
        tail = find_partial_tool_call(body, done[-1]["end"] if done else 0)
        calls = done + ([tail] if tail else [])
        out: List[Dict] = []
        if not calls:
            # Hold back an unclosed "{" that may still turn into a tool call (it reads like the head of
            # {"name": "...), so that half a call is never streamed as plain content.
            limit = len(body)
            brace = body.rfind("{", self._content_sent)
            if brace >= 0 and not _object_end(body, brace)[1] and _CALL_HEAD.match(body[brace:]):
                limit = brace
            fresh = body[self._content_sent:limit]
            body = body[:limit]
            if fresh:
                self._content_sent = len(body)
                out.append({"content": fresh})
            return out
        first = calls[0]["start"]
        if first > self._content_sent:
            text = body[self._content_sent:first]
            self._content_sent = first
            if text:
                out.append({"content": text})
        for i, call in enumerate(calls):
            if i >= len(self._calls):
                self._calls.append({"id": f"call_{uuid.uuid4().hex[:12]}", "named": False, "sent": 0})
                self._seen = True
            st = self._calls[i]
            if not st["named"]:
                st["named"] = True
                out.append({"tool_calls": [{"index": i, "id": st["id"], "type": "function",
                                            "function": {"name": call["name"], "arguments": ""}}]})
            if len(call["args"]) > st["sent"]:
                piece = call["args"][st["sent"]:]
                st["sent"] = len(call["args"])
                out.append({"tool_calls": [{"index": i, "function": {"arguments": piece}}]})
        return out

    def parse_complete(self, body):
        done = find_tool_calls(body)
        if not done:
            return None
        calls = [{"id": f"call_{uuid.uuid4().hex[:12]}", "type": "function",
                  "function": {"name": c["name"], "arguments": c["args"]}} for c in done]
        return {"content": body[: done[0]["start"]].strip() or None, "tool_calls": calls}

    @property
    def has_tool_calls(self) -> bool:
        return self._seen
