"""Incremental tool-call extraction (``SimpleJsonToolParser``): what is streamed, when, and in which pieces."""

import json

import pytest

from astrai_b200.inference.network.tool_parser import (
    BaseToolParser, SimpleJsonToolParser, ToolParserFactory, find_partial_tool_call, find_tool_calls,
)

CALL = '{"name": "get_weather", "arguments": {"city": "Paris", "unit": "C"}}'


def _stream(text, step=1):
    """Feed ``text`` in chunks of ``step`` characters; returns the list of all deltas."""
    p = SimpleJsonToolParser()
    out = []
    for end in range(step, len(text) + step, step):
        out += p.feed(text[:min(end, len(text))])
    return p, out


def _content(deltas):
    return "".join(d["content"] for d in deltas if "content" in d)


def _calls(deltas):
    calls = {}
    for d in deltas:
        for tc in d.get("tool_calls", []):
            st = calls.setdefault(tc["index"], {"name": None, "id": None, "args": ""})
            fn = tc.get("function", {})
            if fn.get("name"):
                st["name"], st["id"] = fn["name"], tc.get("id")
            st["args"] += fn.get("arguments", "")
    return calls


def test_factory_registration_and_base_contract():
    assert "simple_json" in ToolParserFactory.list_registered()
    p = ToolParserFactory.create("simple_json", tools=[{"type": "function"}], tool_choice="auto")
    assert isinstance(p, BaseToolParser) and p.tools and not p.has_tool_calls
    with pytest.raises(NotImplementedError):
        BaseToolParser().feed("x")


def test_plain_text_is_streamed_as_content_only():
    p, deltas = _stream("The weather is nice today.")
    assert _content(deltas) == "The weather is nice today." and not p.has_tool_calls
    assert all("tool_calls" not in d for d in deltas)


@pytest.mark.parametrize("step", [1, 2, 3, 7, 1000])
def test_call_is_reassembled_for_any_chunking(step):
    p, deltas = _stream(CALL, step)
    calls = _calls(deltas)
    assert p.has_tool_calls and list(calls) == [0]
    assert calls[0]["name"] == "get_weather" and calls[0]["id"].startswith("call_")
    assert json.loads("{" + calls[0]["args"] + "}") == {"city": "Paris", "unit": "C"}
    assert _content(deltas) == ""  # no half call leaks into the content


@pytest.mark.parametrize("step", [1, 5])
def test_text_before_a_call_is_content_and_the_call_is_not(step):
    p, deltas = _stream("Let me check. " + CALL, step)
    assert _content(deltas) == "Let me check. "
    assert _calls(deltas)[0]["name"] == "get_weather"


def test_name_delta_comes_once_and_before_argument_deltas():
    _, deltas = _stream(CALL)
    named = [i for i, d in enumerate(deltas) if any(tc.get("function", {}).get("name") for tc in d.get("tool_calls", []))]
    args = [i for i, d in enumerate(deltas) if any(tc.get("function", {}).get("arguments") for tc in d.get("tool_calls", []))]
    assert len(named) == 1 and args and named[0] < args[0]
    first = deltas[named[0]]["tool_calls"][0]
    assert first["type"] == "function" and first["function"]["arguments"] == ""


def test_two_calls_get_two_indices_and_distinct_ids():
    second = '{"name": "get_time", "arguments": {"tz": "UTC"}}'
    p, deltas = _stream(CALL + " " + second, 4)
    calls = _calls(deltas)
    assert sorted(calls) == [0, 1] and calls[1]["name"] == "get_time" and calls[0]["id"] != calls[1]["id"]
    assert json.loads("{" + calls[1]["args"] + "}") == {"tz": "UTC"}


def test_json_that_is_not_a_call_stays_content():
    text = 'Here is data: {"value": 3, "items": [1, 2]} done'
    p, deltas = _stream(text, 3)
    assert _content(deltas) == text and not p.has_tool_calls


def test_braces_inside_strings_do_not_close_the_object():
    text = '{"name": "echo", "arguments": {"text": "a } b { c \\" d"}}'
    calls = find_tool_calls(text)
    assert len(calls) == 1 and calls[0]["end"] == len(text)
    assert json.loads("{" + calls[0]["args"] + "}") == {"text": 'a } b { c " d'}


def test_empty_and_missing_arguments():
    assert find_tool_calls('{"name": "ping", "arguments": {}}')[0]["args"] == ""
    assert find_tool_calls('{"name": "ping"}')[0]["args"] == ""
    assert find_tool_calls('{"name": "", "arguments": {}}') == []
    assert find_tool_calls('{"name": 5}') == []


def test_string_and_list_arguments_pass_through():
    assert find_tool_calls('{"name": "f", "arguments": "raw text"}')[0]["args"] == "raw text"
    assert find_tool_calls('{"name": "f", "arguments": [1, 2]}')[0]["args"] == "[1, 2]"


def test_nested_arguments_keep_their_inner_text():
    text = '{"name": "plan", "arguments": {"steps": [{"a": 1}, {"b": {"c": 2}}], "ok": true}}'
    got = find_tool_calls(text)[0]["args"]
    assert json.loads("{" + got + "}") == {"steps": [{"a": 1}, {"b": {"c": 2}}], "ok": True}


def test_partial_call_detection():
    assert find_partial_tool_call("no braces here") is None
    assert find_partial_tool_call('{"value": 1') is None
    part = find_partial_tool_call('{"name": "get_weather", "arguments": {"city": "Par')
    assert part["name"] == "get_weather" and part["args"] == '"city": "Par' and part["complete"] is False
    assert find_partial_tool_call('{"name": "get_weather"')["args"] == ""


def test_scan_stops_at_the_first_unclosed_object():
    text = CALL + ' {"name": "second", "arguments": {"x": '
    assert [c["name"] for c in find_tool_calls(text)] == ["get_weather"]


def test_unicode_arguments_are_not_escaped():
    text = '{"name": "say", "arguments": {"text": "héllo ☃"}}'
    assert "héllo ☃" in find_tool_calls(text)[0]["args"]


def test_argument_deltas_only_ever_append():
    p = SimpleJsonToolParser()
    sent = ""
    for end in range(1, len(CALL) + 1):
        for d in p.feed(CALL[:end]):
            for tc in d.get("tool_calls", []):
                sent += tc.get("function", {}).get("arguments", "")
    assert json.loads("{" + sent + "}") == {"city": "Paris", "unit": "C"}


def test_feeding_the_same_text_twice_emits_nothing_new():
    p = SimpleJsonToolParser()
    p.feed("hello " + CALL)
    assert p.feed("hello " + CALL) == []


def test_held_back_brace_is_released_when_it_turns_out_to_be_text():
    p = SimpleJsonToolParser()
    first = p.feed('result: {"na')          # could still become {"name": ...: held back
    assert _content(first) == "result: "
    rest = p.feed('result: {"nation": "FR"} end')
    assert _content(first + rest) == 'result: {"nation": "FR"} end'


def test_parse_complete_for_non_streaming_responses():
    p = SimpleJsonToolParser()
    assert p.parse_complete("just text") is None
    res = p.parse_complete("I will call it. " + CALL)
    assert res["content"] == "I will call it." and len(res["tool_calls"]) == 1
    fn = res["tool_calls"][0]["function"]
    assert fn["name"] == "get_weather" and json.loads("{" + fn["arguments"] + "}")["city"] == "Paris"
    assert p.parse_complete(CALL)["content"] is None


def test_whitespace_and_key_order_variants():
    text = '{ "arguments" : {"a":1} , "name" : "f" }'
    calls = find_tool_calls(text)
    assert calls[0]["name"] == "f" and calls[0]["args"] == '"a": 1'


def test_call_followed_by_text_keeps_the_call_complete():
    p, deltas = _stream(CALL + "\nDone.", 6)
    assert json.loads("{" + _calls(deltas)[0]["args"] + "}") == {"city": "Paris", "unit": "C"}
