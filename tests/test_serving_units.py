"""Serving building blocks in isolation: the producer / consumer hand-over of ``generate``, tasks and their queues, the
protocol builders' wire formats, and the synchronous ``run_batch`` path (behaviours the reference checks in
``tests/inference/test_engine.py``, ``test_task.py``, ``test_protocol.py`` and ``test_scheduler.py``)."""

import json
import threading
import time
from types import SimpleNamespace

import pytest
import torch

from helpers import build_tokenizer_dir, tiny_config


# ------------------------------------------------------------------------------------------------- GenerateResult
def test_result_collects_pieces_per_prompt_and_in_arrival_order():
    from astrai_b200.inference.engine import GenerateResult
    from astrai_b200.inference.task import STOP

    r = GenerateResult(count=2)
    r.append("a", 0)
    r.append("x", 1)
    r.append("b", 0)
    assert r.pop_all() == [(0, "a"), (1, "x"), (0, "b")] and r.pop_all() == []
    r.append(STOP, 1)
    r.append("c", 0)
    assert r.get_results() == ["abc", "x"]
    assert [i for i, t in r.pop_all() if t is STOP] == [1]


def test_result_completion_counts_each_prompt_once():
    from astrai_b200.inference.engine import GenerateResult
    from astrai_b200.inference.task import STOP

    r = GenerateResult(count=2)
    r.append(STOP, 0)
    r.append(STOP, 0)  # a second end marker for the same prompt must not release the waiter
    with pytest.raises(TimeoutError, match="1 of 2"):
        r.wait_completion(timeout=0.05)
    r.append(STOP, 1)
    r.wait_completion(timeout=0.05)
    GenerateResult(count=0).wait_completion(timeout=0.01)  # nothing to wait for


def test_result_wait_blocks_until_a_producer_delivers():
    from astrai_b200.inference.engine import GenerateResult

    r = GenerateResult()
    assert r.wait(timeout=0.02) is False
    t0 = time.time()
    threading.Timer(0.05, lambda: r.append("late")).start()
    assert r.wait(timeout=2.0) is True and time.time() - t0 < 1.5
    assert r.wait(timeout=0.0) is True  # what wait() took out of the inbox is still there for pop_all()
    assert r.pop_all() == [(0, "late")]


def test_result_is_safe_under_concurrent_producers():
    from astrai_b200.inference.engine import GenerateResult
    from astrai_b200.inference.task import STOP

    n, per = 8, 200
    r = GenerateResult(count=n)

    def produce(i):
        for k in range(per):
            r.append(f"{k},", i)
        r.append(STOP, i)

    threads = [threading.Thread(target=produce, args=(i,)) for i in range(n)]
    for t in threads:
        t.start()
    r.wait_completion(timeout=10)
    for t in threads:
        t.join()
    assert r.get_results() == ["".join(f"{k}," for k in range(per))] * n
    assert len(r.pop_all()) == n * (per + 1)


# ---------------------------------------------------------------------------------------------------------- tasks
class _Tok:
    stop_ids = [2]

    def encode(self, text):
        return [ord(c) % 50 + 3 for c in text]

    def decode(self, ids):
        return "".join(chr(97 + i % 26) for i in ids)


def test_task_lifecycle_fields():
    from astrai_b200.inference.task import Task, TaskStatus

    t = Task("t", [5, 6, 7], max_tokens=2)
    assert t.status is TaskStatus.PENDING and t.next_pos == 0 and not t.prefill_done
    t.input_tokens = 3
    t.mark_prefill_done()
    assert t.prefill_done and t.next_pos == 3
    t.advance_kv()
    assert t.next_pos == 4
    assert not t.is_finished({2})
    t.output_ids.append(9)
    t.output_tokens = 1
    assert not t.is_finished({2})
    t.output_ids.append(2)
    assert t.is_finished({2})  # stop id
    u = Task("u", [1], max_tokens=1)
    u.output_ids.append(8)
    u.output_tokens = 1
    assert u.is_finished(set())  # budget reached
    assert not Task("v", [1], max_tokens=None).is_finished({2})


def test_manager_truncates_long_prompts_from_the_left_and_caps_max_tokens():
    from astrai_b200.inference.task import TaskManager

    m = TaskManager(_Tok(), max_batch_size=2, max_seq_len=8)
    long = m.make_task(list(range(20)), max_tokens=5)
    assert long.prompt_ids == list(range(12, 20)) and long.max_tokens == 0  # the last 8 tokens, no room to generate
    short = m.make_task([1, 2, 3], max_tokens=100)
    assert short.max_tokens == 5
    assert m.make_task([1, 2, 3], max_tokens=None).max_tokens == 5
    assert m.make_task([1, 2, 3], max_tokens=2).max_tokens == 2


def test_manager_queues_are_fifo_and_rejections_go_back_to_the_front():
    from astrai_b200.inference.task import TaskManager, TaskStatus

    m = TaskManager(_Tok(), max_batch_size=4, max_seq_len=32)
    ids = [m.add_task([i + 3]) for i in range(5)]
    assert m.get_stats()["waiting_queue"] == 5 and m.has_work()
    got = m.pull_candidates(3)
    assert [t.task_id for t in got] == ids[:3]
    m.activate(got[0])
    assert got[0].status is TaskStatus.RUNNING and m.get_stats()["active_tasks"] == 1
    m.return_to_waiting(got[1:])
    assert [t.task_id for t in m.get_waiting_tasks()] == ids[1:]  # original order restored
    assert m.pull_candidates(10)[0].task_id == ids[1]


def test_manager_accepts_text_or_ids_and_registers_callbacks():
    from astrai_b200.inference.task import TaskManager

    m = TaskManager(_Tok(), max_seq_len=64)
    seen = []
    a = m.add_task("hey", stream_callback=seen.append)
    b = m.add_task([7, 8, 9])
    tasks = {t.task_id: t for t in m.get_waiting_tasks()}
    assert tasks[a].prompt_ids == _Tok().encode("hey") and tasks[b].prompt_ids == [7, 8, 9]
    m.invoke_callback(a, "x")
    m.invoke_callback(b, "ignored")  # no callback registered: a no-op
    assert seen == ["x"]


def test_manager_remove_task_from_either_queue():
    from astrai_b200.inference.task import TaskManager

    m = TaskManager(_Tok(), max_seq_len=64)
    a, b = m.add_task([3]), m.add_task([4])
    first = m.pull_candidates(1)[0]
    m.activate(first)
    assert [t.task_id for t in m.remove_task(a)] == [a]  # active tasks are handed back so their cache can be freed
    assert m.remove_task(b) == [] and not m.has_work()
    assert m.remove_task("unknown") == []


def test_manager_retires_finished_and_aborted_tasks_and_counts_tokens():
    from astrai_b200.inference.task import TaskManager, TaskStatus

    m = TaskManager(_Tok(), max_seq_len=64)
    for i in range(3):
        m.add_task([i + 3], max_tokens=4)
    a, b, c = m.pull_candidates(3)
    for t in (a, b, c):
        m.activate(t)
    a.output_ids, a.output_tokens = [9, 2], 2          # stop id
    b.status = TaskStatus.ABORTED                      # ran out of cache
    c.output_ids, c.output_tokens = [9], 1             # still running
    done = m.remove_finished_tasks({2})
    assert {t.task_id for t in done} == {a.task_id, b.task_id} and a.status is TaskStatus.FINISHED
    assert [t.task_id for t in m.get_active_tasks()] == [c.task_id]
    assert m.get_stats()["total_tokens"] == 2  # aborted tasks do not count


def test_manager_wait_returns_on_wake_and_on_new_work():
    from astrai_b200.inference.task import TaskManager

    m = TaskManager(_Tok(), max_seq_len=64)
    t0 = time.time()
    threading.Timer(0.05, m.wake).start()
    m.wait_for_tasks(timeout=5.0)
    assert time.time() - t0 < 2.0
    m.add_task([3])
    t0 = time.time()
    m.wait_for_tasks(timeout=5.0)  # work is queued: returns at once
    assert time.time() - t0 < 0.5
    m.clear_queues()
    assert not m.has_work()


# ------------------------------------------------------------------------------------------------------- protocol
def test_stop_checker_matches_substrings_and_ignores_empty_sequences():
    from astrai_b200.inference.network.protocol import StopChecker

    c = StopChecker(["END", "", "\n\n"])
    assert c.check("the END is near") == "END" and c.check("a\n\nb") == "\n\n" and c.check("nothing") is None
    assert StopChecker([]).check("anything") is None and StopChecker([""]).check("") is None


def test_sse_helpers():
    from astrai_b200.inference.network.protocol import GenContext, StopInfo, sse_done, sse_event

    assert sse_done() == "data: [DONE]\n\n"
    ev = sse_event({"a": "é"}, event="message_start")
    assert ev.startswith("event: message_start\ndata: ") and json.loads(ev.split("data: ", 1)[1]) == {"a": "é"} and "é" in ev
    assert sse_event({"a": 1}).startswith("data: ")
    ctx = GenContext("id", 1, "m")
    assert (ctx.prompt_tokens, ctx.completion_tokens) == (0, 0)
    assert StopInfo().matched is None and StopInfo("x", "ax", "a").yielded == "a"


class _ChatTok:
    def apply_chat_template(self, messages, tokenize=False, tools=None):
        return "|".join(f"{m['role']}:{m['content']}" for m in messages) + (f"|tools={len(tools)}" if tools else "")

    def encode(self, text):
        return list(text.encode())


def _data(event: str):
    return json.loads(event.split("data: ", 1)[1])


def test_openai_builder_formats():
    from astrai_b200.inference.network.app import ChatCompletionRequest, ChatMessage
    from astrai_b200.inference.network.openai import OpenAIResponseBuilder
    from astrai_b200.inference.network.protocol import StopInfo

    b = OpenAIResponseBuilder()
    req = ChatCompletionRequest(model="m1", messages=[ChatMessage(role="system", content="be brief"), ChatMessage(role="user", content="hi")],
                                stop="END")
    prompt, ctx, stops = b.prepare(req, SimpleNamespace(tokenizer=_ChatTok()))
    assert prompt == "system:be brief|user:hi" and stops == ["END"] and ctx.model == "m1" and ctx.resp_id.startswith("chatcmpl-")
    assert b.prepare(ChatCompletionRequest(messages=[ChatMessage(role="user", content="x")], stop=["a", "b"]),
                     SimpleNamespace(tokenizer=_ChatTok()))[2] == ["a", "b"]
    assert b.prepare(ChatCompletionRequest(messages=[ChatMessage(role="user", content="x")]),
                     SimpleNamespace(tokenizer=_ChatTok()))[2] == []
    prompt, ctx, _ = b.prepare(req, SimpleNamespace(tokenizer=_ChatTok()))
    start = _data(b.format_stream_start(ctx)[0])
    assert start["object"] == "chat.completion.chunk" and start["choices"][0]["delta"] == {"role": "assistant"}
    assert start["created"] == ctx.created and start["id"] == ctx.resp_id
    chunk = _data(b.format_chunk("tok")[0])
    assert chunk["choices"][0]["delta"] == {"content": "tok"} and chunk["choices"][0]["finish_reason"] is None and chunk["created"] == 0
    ctx.prompt_tokens, ctx.completion_tokens = 7, 3
    end = b.format_stream_end(ctx, StopInfo())
    assert _data(end[0])["choices"][0]["finish_reason"] == "stop" and _data(end[0])["choices"][0]["delta"] == {}
    assert _data(end[1]) == {"prompt_tokens": 7, "completion_tokens": 3, "total_tokens": 10}
    full = b.format_response(ctx, "answer", StopInfo())
    assert full["object"] == "chat.completion" and full["choices"][0]["message"] == {"role": "assistant", "content": "answer"}
    assert full["choices"][0]["finish_reason"] == "stop" and full["usage"]["total_tokens"] == 10


def test_openai_builder_warns_about_ignored_parameters(caplog):
    from astrai_b200.inference.network.app import ChatCompletionRequest, ChatMessage
    from astrai_b200.inference.network.openai import OpenAIResponseBuilder

    eng = SimpleNamespace(tokenizer=_ChatTok())
    with caplog.at_level("WARNING"):
        OpenAIResponseBuilder().prepare(ChatCompletionRequest(messages=[ChatMessage(role="user", content="x")]), eng)
    assert "not supported" not in caplog.text  # defaults are silent
    with caplog.at_level("WARNING"):
        OpenAIResponseBuilder().prepare(ChatCompletionRequest(messages=[ChatMessage(role="user", content="x")], n=2, user="u",
                                                              presence_penalty=0.5), eng)
    for name in ("'n'", "'user'", "'presence_penalty'"):
        assert name in caplog.text


def test_anthropic_builder_prepare_and_stream_events():
    from astrai_b200.inference.network.anthropic import AnthropicResponseBuilder, first_text
    from astrai_b200.inference.network.app import AnthropicMessage, MessagesRequest
    from astrai_b200.inference.network.protocol import StopInfo

    assert first_text("plain") == "plain"
    assert first_text([{"type": "image", "source": {}}, {"type": "text", "text": "second"}]) == "second"
    assert first_text([]) == "" and first_text([{"type": "image"}]) == ""
    b = AnthropicResponseBuilder()
    req = MessagesRequest(model="claude-ish", system="sys", stop_sequences=["STOP"],
                          messages=[AnthropicMessage(role="user", content=[{"type": "text", "text": "hello"}]),
                                    AnthropicMessage(role="assistant", content=[{"type": "image"}])])
    prompt, ctx, stops = b.prepare(req, SimpleNamespace(tokenizer=_ChatTok()))
    assert prompt == "system:sys|user:hello" and stops == ["STOP"] and ctx.resp_id.startswith("msg_")  # the empty turn is dropped
    ctx.prompt_tokens = 4
    start = b.format_stream_start(ctx)
    assert [e.split("\n")[0] for e in start] == ["event: message_start", "event: content_block_start"]
    assert _data(start[0])["message"]["usage"] == {"input_tokens": 4} and _data(start[0])["message"]["content"] == []
    assert _data(b.format_chunk("hi")[0])["delta"] == {"type": "text_delta", "text": "hi"}
    ctx.completion_tokens = 2
    end = b.format_stream_end(ctx, StopInfo())
    assert [e.split("\n")[0] for e in end] == ["event: content_block_stop", "event: message_delta", "event: message_stop"]
    assert _data(end[1])["delta"] == {"stop_reason": "end_turn", "stop_sequence": None} and _data(end[1])["usage"] == {"output_tokens": 2}


def test_anthropic_stop_sequence_trims_and_flushes_unsent_text():
    from astrai_b200.inference.network.anthropic import AnthropicResponseBuilder
    from astrai_b200.inference.network.protocol import GenContext, StopInfo

    b, ctx = AnthropicResponseBuilder(), GenContext("msg_1", 0, "m", 3, 5)
    # "Hello wor" was streamed, the piece "ld STOP tail" completed the stop sequence: "ld " must still reach the client
    end = b.format_stream_end(ctx, StopInfo(matched="STOP", body="Hello world STOP tail", yielded="Hello wor"))
    assert _data(end[0])["delta"]["text"] == "ld " and end[1].startswith("event: content_block_stop")
    assert _data(end[2])["delta"] == {"stop_reason": "stop_sequence", "stop_sequence": "STOP"}
    # everything before the stop sequence was already sent: no extra delta
    end = b.format_stream_end(ctx, StopInfo(matched="STOP", body="abcSTOP", yielded="abc"))
    assert end[0].startswith("event: content_block_stop")
    full = b.format_response(ctx, "Hello world STOP tail", StopInfo(matched="STOP", body="Hello world STOP tail"))
    assert full["content"] == [{"type": "text", "text": "Hello world "}] and full["stop_reason"] == "stop_sequence"
    assert full["usage"] == {"input_tokens": 3, "output_tokens": 5}
    plain = b.format_response(ctx, "all of it", StopInfo())
    assert plain["content"][0]["text"] == "all of it" and plain["stop_reason"] == "end_turn" and plain["stop_sequence"] is None


# ------------------------------------------------------------------------------------------------------ run_batch
@pytest.fixture(scope="module")
def served(tmp_path_factory):
    from astrai_b200.models import AutoRegressiveLM
    from astrai_b200.tokenize import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(build_tokenizer_dir(str(tmp_path_factory.mktemp("tok"))))
    torch.manual_seed(0)
    model = AutoRegressiveLM(tiny_config(vocab_size=512, hidden_size=32, intermediate_size=64, max_position_embeddings=128)).eval()
    return model, tok


def _sched(served, **kw):
    from astrai_b200.inference import InferenceScheduler

    model, tok = served
    return InferenceScheduler(model, tok, enable_cuda_graph=False, **{"max_batch_size": 4, "max_seq_len": 64, **kw})


def test_run_batch_edge_cases(served):
    s = _sched(served)
    assert s.run_batch([], max_tokens=4) == []
    assert s.run_batch([[5, 6, 7]], max_tokens=0) == [[]]
    out = s.run_batch([[5, 6, 7], [], [9] * 100], max_tokens=3, temperature=0.0)
    assert len(out[0]) == 3 and out[1] == []  # an empty prompt yields nothing
    assert len(out[2]) <= 3  # the over-long prompt keeps its tail and whatever room is left
    assert s.get_stats()["active_tasks"] == 0 and s.get_stats()["waiting_queue"] == 0


def test_run_batch_logprobs_are_aligned_with_tokens(served):
    model, _ = served
    s = _sched(served)
    prompt = [11, 12, 13, 14]
    toks, lps = s.run_batch([prompt], max_tokens=5, temperature=0.0, return_logprobs=True)[0]
    assert len(toks) == len(lps) == 5 and all(lp <= 0 for lp in lps)
    with torch.no_grad():
        logits = model(torch.tensor([prompt + toks[:-1]]))["logits"][0, len(prompt) - 1:].float()
    ref = torch.log_softmax(logits, -1).gather(1, torch.tensor(toks)[:, None])[:, 0]
    assert torch.allclose(torch.tensor(lps), ref, atol=1e-4)


def test_run_batch_more_prompts_than_batch_slots(served):
    """The synchronous path takes what fits at once (one cache row per prompt) and answers the rest with empty lists, as
    the reference's ``run_batch`` does; the prompts it takes decode exactly as they do alone."""
    s = _sched(served, max_batch_size=2)
    prompts = [[20 + i, 21 + i, 22 + i] for i in range(5)]
    together = s.run_batch(prompts, max_tokens=4, temperature=0.0)
    alone = [_sched(served, max_batch_size=1).run_batch([p], max_tokens=4, temperature=0.0)[0] for p in prompts]
    assert together[:2] == alone[:2] and together[2:] == [[], [], []]
    assert s.run_batch(prompts[2:4], max_tokens=4, temperature=0.0) == alone[2:4]  # the rows were given back


def test_decode_steps_do_not_leak_state_between_batches(served):
    s = _sched(served)
    a = s.run_batch([[30, 31, 32], [40, 41]], max_tokens=6, temperature=0.0)
    b = s.run_batch([[40, 41]], max_tokens=6, temperature=0.0)  # same request alone, after the first batch is gone
    assert b[0] == a[1]
    c = s.run_batch([[50], [30, 31, 32]], max_tokens=6, temperature=0.0)
    assert c[1] == a[0]


def test_streaming_callbacks_deliver_text_then_stop(served):
    from astrai_b200.inference.task import STOP

    s = _sched(served)
    s.start()
    try:
        got, done = [], threading.Event()

        def cb(piece):
            got.append(piece)
            if piece is STOP:
                done.set()

        s.add_task([60, 61, 62], max_tokens=5, temperature=0.0, stream_callback=cb)
        assert done.wait(timeout=30)
        assert got[-1] is STOP and got.count(STOP) == 1 and all(isinstance(p, str) for p in got[:-1])
        stats = s.get_stats()
        assert stats["total_tasks"] == 1 and stats["active_tasks"] == 0
    finally:
        s.stop()


# ------------------------------------------------------------------------------------- admission policy under load
def test_prefill_is_deferred_only_under_load(served):
    from astrai_b200.inference.task import Task

    s = _sched(served, max_batch_size=64, prefill_defer_steps=4, prefill_defer_min_batch=8, prefill_defer_tokens=100)
    fresh = [Task("f", list(range(3, 23)))]
    assert not s._defer_prefill([], 50)                      # nothing waiting
    assert not s._defer_prefill(fresh, 7)                    # small decode batch: prefill at once
    assert s._defer_prefill(fresh, 8)                        # under load: wait for company
    assert not s._defer_prefill([Task("g", list(range(3, 200)))], 8)  # enough prompt tokens pending for a forward of their own
    s._steps_since_prefill = 4
    assert not s._defer_prefill(fresh, 8)                    # waited long enough
    off = _sched(served, prefill_defer_steps=0)
    assert not off._defer_prefill(fresh, 1000)


def test_deferred_admission_does_not_change_greedy_outputs(served):
    """Prompts that arrive while others decode are held back for a few steps under the deferral policy; every request
    still gets exactly the tokens it gets alone."""
    from astrai_b200.inference.task import STOP

    prompts = [[30 + i, 31 + i, 32 + i, 33 + i] for i in range(6)]
    alone = [_sched(served, max_batch_size=1).run_batch([p], max_tokens=12, temperature=0.0)[0] for p in prompts]
    model, tok = served
    s = _sched(served, max_batch_size=8, prefill_defer_steps=3, prefill_defer_min_batch=2, prefill_defer_tokens=1000)
    got = {i: [] for i in range(len(prompts))}
    done = {i: threading.Event() for i in range(len(prompts))}
    tasks = {}

    def make_cb(i):
        def cb(piece):
            if piece is STOP:
                done[i].set()
        return cb

    s.start()
    try:
        for i, p in enumerate(prompts):
            tasks[i] = s.add_task(p, max_tokens=12, temperature=0.0, stream_callback=make_cb(i))
            time.sleep(0.01)  # staggered arrivals: later prompts meet a running decode batch
        for ev in done.values():
            assert ev.wait(timeout=60)
    finally:
        s.stop()
    # token ids are not streamed (text is); compare through the scheduler's own bookkeeping of finished tasks
    finished = {t["task_id"]: t for t in s.get_stats().get("recent_tasks", [])}
    assert len(finished) == len(prompts) and all(t["output_tokens"] == 12 for t in finished.values())
    again = _sched(served, max_batch_size=8, prefill_defer_steps=3, prefill_defer_min_batch=2, prefill_defer_tokens=1000)
    assert again.run_batch(prompts, max_tokens=12, temperature=0.0) == alone


def test_create_engine_takes_the_serve_cli_options(tmp_path, served):
    """The options the serve command forwards reach the scheduler, and the engine built from a model directory answers
    over HTTP."""
    from fastapi.testclient import TestClient

    from astrai_b200.inference.network import get_app
    from astrai_b200.inference.network.app import create_engine
    from astrai_b200.serialization import Checkpoint

    model, _ = served
    d = tmp_path / "params"
    build_tokenizer_dir(str(d))
    Checkpoint(state_dict=model.state_dict(), config=model.config.to_dict()).save(str(d))
    with pytest.raises(FileNotFoundError):
        create_engine(tmp_path / "nowhere", device="cpu")
    eng = create_engine(d, device="cpu", dtype=torch.float32, max_batch_size=2, max_seq_len=64, page_size=4, paged=True,
                        enable_cuda_graph=False, chunked_prefill=True, max_prefill_tokens=16, prefill_defer_steps=0)
    try:
        assert eng.scheduler.chunked_prefill and eng.scheduler.max_prefill_tokens == 16 and eng.scheduler.prefill_defer_steps == 0
        app = get_app()
        app.state.server_config = {"_test": True}
        with TestClient(app) as c:
            app.state.engine = eng
            assert c.get("/health").json() == {"status": "ok", "model_loaded": True}
            r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hello"}], "max_tokens": 4})
            assert r.status_code == 200 and r.json()["choices"][0]["message"]["role"] == "assistant"
            assert r.json()["usage"]["completion_tokens"] <= 4
            r = c.post("/v1/messages", json={"messages": [{"role": "user", "content": "hello"}], "max_tokens": 4, "stream": True})
            assert r.status_code == 200 and "event: message_stop" in r.text and r.text.rstrip().endswith("data: [DONE]")
            app.state.engine = None
    finally:
        eng.shutdown()


# ------------------------------------------------------------------------------------- abandoned answers are cancelled
def _wait_until(cond, timeout=20.0):
    end = time.time() + timeout
    while time.time() < end:
        if cond():
            return True
        time.sleep(0.01)
    return False


def _slow_down(scheduler, seconds=0.01):
    """Make every scheduling step take a while, so that a test can act while an answer is still being generated."""
    step = scheduler._step

    def slow(*args, **kwargs):
        time.sleep(seconds)
        return step(*args, **kwargs)

    scheduler._step = slow


def test_remove_task_during_generation_goes_through_the_loop_and_frees_the_slot(served):
    s = _sched(served, max_batch_size=2)
    _slow_down(s)
    s.start()
    try:
        heard = []
        tid = s.add_task([60, 61, 62], max_tokens=50, temperature=0.0, stream_callback=heard.append)
        assert _wait_until(lambda: len(heard) >= 2)
        s.remove_task(tid)
        count = len(heard)
        assert _wait_until(lambda: s.get_stats()["active_tasks"] == 0)
        time.sleep(0.1)
        assert len(heard) == count  # silenced at once: nothing after the call returned, not even the end marker
        assert s._cancelled == []
        s.remove_task(tid)  # unknown by now: nothing is staged
        s.remove_task("never-existed")
        assert s._cancelled == []
        # the freed slot and pages serve the next requests
        done = threading.Event()
        s.add_task([60, 61, 62], max_tokens=3, temperature=0.0, stream_callback=lambda p: done.set() if not isinstance(p, str) else None)
        assert done.wait(timeout=30)
    finally:
        s.stop()


def test_waiting_request_can_be_cancelled_before_it_runs(served):
    s = _sched(served, max_batch_size=1)
    _slow_down(s)
    s.start()
    try:
        first, second = [], []
        a = s.add_task([60, 61, 62], max_tokens=40, temperature=0.0, stream_callback=first.append)
        b = s.add_task([70, 71], max_tokens=40, temperature=0.0, stream_callback=second.append)
        assert _wait_until(lambda: len(first) >= 2)
        s.remove_task(b)
        assert _wait_until(lambda: s.get_stats()["waiting_queue"] == 0)
        s.remove_task(a)
        assert _wait_until(lambda: s.get_stats()["active_tasks"] == 0)
        assert second == []
    finally:
        s.stop()


def test_abandoned_stream_gives_its_batch_slot_back(served):
    from astrai_b200.inference import InferenceEngine

    model, tok = served
    engine = InferenceEngine(model, tok, max_batch_size=2, max_seq_len=96, enable_cuda_graph=False)
    _slow_down(engine.scheduler)
    try:
        stream = engine.generate("hello", stream=True, max_tokens=80, temperature=0.0)
        assert isinstance(next(stream), str)
        assert engine.get_stats()["active_tasks"] == 1
        stream.close()  # the consumer walks away
        assert _wait_until(lambda: engine.get_stats()["active_tasks"] == 0)
        # a stream that is read to its end removes nothing twice and leaves nothing behind
        assert "".join(engine.generate("hello", stream=True, max_tokens=4, temperature=0.0)) == engine.generate("hello", max_tokens=4, temperature=0.0)
        assert engine.get_stats()["active_tasks"] == 0 and engine.scheduler._cancelled == []
    finally:
        engine.shutdown()


def test_closing_the_async_generator_cancels_the_request(served):
    import asyncio

    from astrai_b200.inference import InferenceEngine

    model, tok = served
    engine = InferenceEngine(model, tok, max_batch_size=2, max_seq_len=96, enable_cuda_graph=False)
    _slow_down(engine.scheduler)

    async def read_two_then_leave():
        agen = engine.generate_async("hello", max_tokens=80, temperature=0.0)
        got = []
        async for piece in agen:
            got.append(piece)
            if len(got) == 2:
                break
        await agen.aclose()
        return got

    async def cancelled_in_mid_read():
        agen = engine.generate_async("hello there", max_tokens=80, temperature=0.0)

        async def reader():
            async for _ in agen:
                pass

        task = asyncio.ensure_future(reader())
        await asyncio.sleep(0.2)
        task.cancel()
        with pytest.raises(asyncio.CancelledError):
            await task

    try:
        assert len(asyncio.run(read_two_then_leave())) == 2
        assert _wait_until(lambda: engine.get_stats()["active_tasks"] == 0)
        asyncio.run(cancelled_in_mid_read())
        assert _wait_until(lambda: engine.get_stats()["active_tasks"] == 0)
        assert engine.generate("hello", max_tokens=3, temperature=0.0) is not None  # the engine still serves
    finally:
        engine.shutdown()


def test_http_stop_sequence_ends_the_generation_not_only_the_answer(served):
    """A matched stop sequence answers the client at once; the request must not keep decoding up to max_tokens."""
    from fastapi.testclient import TestClient

    from astrai_b200.inference import InferenceEngine
    from astrai_b200.inference.network import app as app_mod

    model, tok = served
    engine = InferenceEngine(model, tok, max_batch_size=2, max_seq_len=120, enable_cuda_graph=False)
    _slow_down(engine.scheduler, 0.005)
    app = app_mod.get_app()
    old = app.state.engine, app.state.server_config
    app.state.engine, app.state.server_config = engine, {"_test": True}
    try:
        client = TestClient(app)
        full = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 12, "temperature": 0.0}).json()
        text = full["choices"][0]["message"]["content"]
        assert len(text) >= 4
        stop = text[2:4]
        before = engine.get_stats()["total_tokens"]
        cut = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 100, "temperature": 0.0,
                                                        "stop": [stop]}).json()
        # this wire format keeps the piece that completed the stop sequence in the answer (as the reference does)
        assert cut["choices"][0]["finish_reason"] == "stop" and cut["choices"][0]["message"]["content"] == text[:4]
        assert cut["usage"]["completion_tokens"] < 12
        assert _wait_until(lambda: engine.get_stats()["active_tasks"] == 0, timeout=0.3)  # 100 more steps would take half a second
        assert engine.get_stats()["total_tokens"] - before < 100
    finally:
        app.state.engine, app.state.server_config = old
        engine.shutdown()


def test_finished_requests_are_counted_even_when_the_caller_removes_them_at_once(served):
    """``generate`` removes its requests as soon as the last piece arrived, which is before the loop has retired them:
    the removal must not swallow the token count or the prefix index entry of a request that finished."""
    from astrai_b200.inference import InferenceEngine

    model, tok = served
    engine = InferenceEngine(model, tok, max_batch_size=2, max_seq_len=96, enable_cuda_graph=False)
    try:
        for n in range(1, 6):
            engine.generate("count me", max_tokens=4, temperature=0.0)
            assert _wait_until(lambda: engine.get_stats()["active_tasks"] == 0)
            stats = engine.get_stats()
            assert stats["total_tasks"] == n and 0 < stats["total_tokens"] <= 4 * n
            assert stats["total_tokens"] >= n
    finally:
        engine.shutdown()


# ------------------------------------------------------------------------------ attention back end per scheduler / request
def test_scheduler_backend_is_active_on_the_loop_thread_and_named(served, monkeypatch):
    from astrai_b200.ops import backend as ab

    monkeypatch.delenv("ASTR_BACKEND", raising=False)
    monkeypatch.delenv("ASTRAI_B200_ATTN", raising=False)
    s = _sched(served, backend="torch_native")
    assert s.backend_name == "torch_native" and ab.get_backend("cuda", use_default=False) is None  # nothing leaks to this thread
    seen = []
    step = s._step
    s._step = lambda *a, **k: (seen.append(ab.get_backend("cuda", use_default=False)), step(*a, **k))[1]
    done = threading.Event()
    s.start()
    try:
        s.add_task([60, 61], max_tokens=2, temperature=0.0, stream_callback=lambda p: done.set() if not isinstance(p, str) else None)
        assert done.wait(timeout=30)
    finally:
        s.stop()
    assert seen and set(seen) == {ab.ATTN_BACKEND.TORCH_NATIVE}
    assert _sched(served).backend_name == "torch_native"  # a CPU model: the only back end there is
    with pytest.raises(ValueError):
        _sched(served, backend="metal")


def test_requests_are_stepped_in_groups_of_their_own_backend(served, monkeypatch):
    """A request carries the back end its submitter had selected; a step runs one forward group per back end, each under
    that selection, and the tokens are what they are without any selection (on the CPU every back end is the same math)."""
    from astrai_b200.inference.task import Task
    from astrai_b200.ops import backend as ab

    monkeypatch.delenv("ASTR_BACKEND", raising=False)
    monkeypatch.delenv("ASTRAI_B200_ATTN", raising=False)
    plain = _sched(served).run_batch([[30, 31, 32], [40, 41], [50, 51, 52, 53]], max_tokens=5, temperature=0.0)

    s = _sched(served)
    calls = []
    decode, prefill = s._executor.execute_decode, s._executor.execute_prefill
    s._executor.execute_decode = lambda tasks, **k: (calls.append(("decode", ab.get_backend("cuda", use_default=False), len(tasks))), decode(tasks, **k))[1]
    s._executor.execute_prefill = lambda tasks, **k: (calls.append(("prefill", ab.get_backend("cuda", use_default=False), len(tasks))), prefill(tasks, **k))[1]
    tasks = [Task("a", [30, 31, 32], 5, 0.0, backend=ab.ATTN_BACKEND.TORCH_NATIVE), Task("b", [40, 41], 5, 0.0),
             Task("c", [50, 51, 52, 53], 5, 0.0, backend=ab.ATTN_BACKEND.TORCH_NATIVE)]
    for t in tasks:
        assert s._task_cache.task_alloc(t.task_id, t.prompt_ids)
    for _ in range(5):
        stepped, aborted = s._step(tasks)
        assert len(stepped) == 3 and not aborted
    assert [t.output_ids for t in tasks] == plain
    assert {c for c in calls if c[0] == "prefill"} == {("prefill", ab.ATTN_BACKEND.TORCH_NATIVE, 2), ("prefill", None, 1)}
    assert [c for c in calls if c[0] == "decode"].count(("decode", ab.ATTN_BACKEND.TORCH_NATIVE, 2)) == 4
    assert [c for c in calls if c[0] == "decode"].count(("decode", None, 1)) == 4
    assert ab.get_backend("cuda", use_default=False) is None


def test_generate_hands_the_callers_backend_to_the_request(served, monkeypatch):
    from astrai_b200.inference import InferenceEngine
    from astrai_b200.ops import backend as ab

    monkeypatch.delenv("ASTR_BACKEND", raising=False)
    monkeypatch.delenv("ASTRAI_B200_ATTN", raising=False)
    model, tok = served
    engine = InferenceEngine(model, tok, max_batch_size=2, max_seq_len=96, enable_cuda_graph=False)
    seen = []
    add = engine.scheduler.add_task
    engine.scheduler.add_task = lambda *a, **k: (seen.append(k.get("backend")), add(*a, **k))[1]
    try:
        first = engine.generate("hello", max_tokens=3, temperature=0.0)
        with ab.attn_backend("torch_native"):
            second = engine.generate("hello", max_tokens=3, temperature=0.0)
            streamed = "".join(engine.generate("hello", stream=True, max_tokens=3, temperature=0.0))
        assert seen == [None, ab.ATTN_BACKEND.TORCH_NATIVE, ab.ATTN_BACKEND.TORCH_NATIVE] and first == second == streamed
    finally:
        engine.shutdown()


def test_http_rejects_malformed_requests_before_they_reach_the_engine(served):
    from fastapi.testclient import TestClient

    from astrai_b200.inference import InferenceEngine
    from astrai_b200.inference.network import app as app_mod

    model, tok = served
    engine = InferenceEngine(model, tok, max_batch_size=2, max_seq_len=96, enable_cuda_graph=False)
    app = app_mod.get_app()
    old = app.state.engine, app.state.server_config
    app.state.engine, app.state.server_config = engine, {"_test": True}
    try:
        client = TestClient(app)
        before = engine.get_stats()["total_tasks"]
        ok = {"messages": [{"role": "user", "content": "hi"}]}
        for bad in ({}, {"messages": "hi"}, {**ok, "max_tokens": 0}, {**ok, "temperature": 2.5}, {**ok, "top_p": 1.5}, {**ok, "top_k": 0},
                    {**ok, "frequency_penalty": 3.0}, {"messages": [{"content": "no role"}]}):
            assert client.post("/v1/chat/completions", json=bad).status_code == 422, bad
        for bad in ({}, {"messages": [{"role": "user"}]}, {"messages": [{"role": "user", "content": "x"}], "max_tokens": 0},
                    {"messages": [{"role": "user", "content": "x"}], "stop_sequences": "END"}):
            assert client.post("/v1/messages", json=bad).status_code == 422, bad
        assert client.post("/v1/chat/completions", content=b"{not json", headers={"content-type": "application/json"}).status_code == 422
        assert engine.get_stats()["total_tasks"] == before
        assert client.get("/nowhere").status_code == 404 and client.get("/v1/chat/completions").status_code == 405
        listed = client.get("/v1/models").json()
        assert listed["object"] == "list" and [m["object"] for m in listed["data"]] == ["model"] and listed["data"][0]["id"]
        # an empty conversation is a valid request: the model answers the bare generation prompt
        r = client.post("/v1/chat/completions", json={"messages": [], "max_tokens": 2, "temperature": 0.0})
        assert r.status_code == 200 and r.json()["usage"]["completion_tokens"] <= 2
        stats = client.get("/stats").json()
        assert {"total_tasks", "total_tokens", "active_tasks", "waiting_queue"} <= set(stats) and stats["total_tasks"] == before + 1
    finally:
        app.state.engine, app.state.server_config = old
        engine.shutdown()


def test_submit_stream_and_cancel_from_many_threads_leaks_nothing(served):
    """Callers on eight threads submit, read a little, walk away, finish, or cancel by id, all at once; afterwards every
    page and every request row is back, nothing is queued, and the engine still answers."""
    import random

    from astrai_b200.inference import InferenceEngine

    model, tok = served
    engine = InferenceEngine(model, tok, max_batch_size=4, max_seq_len=64, enable_cuda_graph=False, kv_cache_tokens=4 * 64, page_size=16)
    pool = engine.scheduler._cache
    pages_at_rest = pool.allocator.available()
    errors, finished = [], []

    def caller(seed):
        rng = random.Random(seed)
        try:
            for i in range(6):
                prompt = "hello " * rng.randint(1, 4) + str(seed)
                kind = rng.choice(["full", "abandon", "cancel_id", "stream_full"])
                if kind == "full":
                    finished.append(engine.generate(prompt, max_tokens=rng.randint(1, 6), temperature=0.0))
                elif kind == "stream_full":
                    finished.append("".join(engine.generate(prompt, stream=True, max_tokens=rng.randint(1, 6), temperature=0.0)))
                elif kind == "abandon":
                    stream = engine.generate(prompt, stream=True, max_tokens=30, temperature=0.0)
                    for n, _ in enumerate(stream):
                        if n >= rng.randint(0, 2):
                            break
                    stream.close()
                else:
                    tid = engine.scheduler.add_task(prompt, max_tokens=30, temperature=0.0, stream_callback=lambda piece: None)
                    time.sleep(rng.random() * 0.02)
                    engine.scheduler.remove_task(tid)
        except Exception as exc:  # noqa: BLE001 - reported below
            errors.append(repr(exc))

    try:
        threads = [threading.Thread(target=caller, args=(s,)) for s in range(8)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=120)
        assert not any(t.is_alive() for t in threads) and errors == []
        assert _wait_until(lambda: engine.get_stats()["active_tasks"] == 0 and engine.get_stats()["waiting_queue"] == 0, timeout=30)
        assert _wait_until(lambda: pool.allocator.available() == pages_at_rest, timeout=10)  # retained prefix pages count as available
        assert engine.scheduler._cancelled == [] and all(isinstance(x, str) for x in finished)
        assert engine.generate("still here", max_tokens=2, temperature=0.0) is not None
        # every request row is free again: a full batch can be admitted
        assert len(engine.generate(["a", "b", "c", "d"], max_tokens=1, temperature=0.0)) == 4
    finally:
        engine.shutdown()


def test_text_completions_route(served):
    """Plain text in and out: no chat template around the prompt, the text ends before a stop sequence, the finish reason
    tells a spent budget from an end, streams carry the same text in pieces."""
    from fastapi.testclient import TestClient

    from astrai_b200.inference import InferenceEngine
    from astrai_b200.inference.network import app as app_mod

    PROMPT = "the quick brown fox"
    model, tok = served
    engine = InferenceEngine(model, tok, max_batch_size=2, max_seq_len=96, enable_cuda_graph=False)
    app = app_mod.get_app()
    old = app.state.engine, app.state.server_config
    app.state.engine, app.state.server_config = engine, {"_test": True}
    try:
        client = TestClient(app)
        r = client.post("/v1/completions", json={"prompt": PROMPT, "max_tokens": 8, "temperature": 0.0}).json()
        text = r["choices"][0]["text"]
        assert r["object"] == "text_completion" and r["id"].startswith("cmpl-")
        ids = engine.scheduler.run_batch([tok.encode(PROMPT)], max_tokens=8, temperature=0.0)[0]
        spent = len(ids) == 8 and ids[-1] not in tok.stop_ids
        # tokens, not pieces of text (this random model emits tokens that decode to nothing on their own)
        assert r["usage"] == {"prompt_tokens": len(tok.encode(PROMPT)), "completion_tokens": len(ids),
                              "total_tokens": len(tok.encode(PROMPT)) + len(ids)}
        assert r["choices"][0]["finish_reason"] == ("length" if spent else "stop")
        assert text == engine.generate(PROMPT, max_tokens=8, temperature=0.0)  # the bare prompt, not a chat turn
        echoed = client.post("/v1/completions", json={"prompt": [PROMPT[:4], PROMPT[4:]], "max_tokens": 8, "temperature": 0.0, "echo": True}).json()
        assert echoed["choices"][0]["text"] == PROMPT + text
        assert len(text) >= 4  # this prompt's greedy continuation has text to cut
        stop = text[2:4]
        cut = client.post("/v1/completions", json={"prompt": PROMPT, "max_tokens": 50, "temperature": 0.0, "stop": stop}).json()
        assert cut["choices"][0]["text"] == text[:text.index(stop)] and cut["choices"][0]["finish_reason"] == "stop"
        with client.stream("POST", "/v1/completions", json={"prompt": PROMPT, "max_tokens": 50, "temperature": 0.0, "stop": [stop],
                                                            "stream": True}) as resp:
            events = [line[6:] for line in resp.iter_lines() if line.startswith("data: ")]
        assert events[-1] == "[DONE]"
        chunks = [json.loads(e) for e in events[:-1]]
        assert "".join(c["choices"][0]["text"] for c in chunks) == text[:text.index(stop)]
        assert chunks[-1]["choices"][0]["finish_reason"] == "stop" and chunks[-1]["usage"]["completion_tokens"] >= 1
        assert all(c["choices"][0]["finish_reason"] is None for c in chunks[:-1])
        assert client.post("/v1/completions", json={"max_tokens": 3}).status_code == 422
        # the chat protocols name a spent budget too
        chat = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": PROMPT}], "max_tokens": 5, "temperature": 0.0}).json()
        msg = client.post("/v1/messages", json={"messages": [{"role": "user", "content": PROMPT}], "max_tokens": 5, "temperature": 0.0}).json()
        assert chat["usage"]["completion_tokens"] == msg["usage"]["output_tokens"] <= 5
        newer = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": PROMPT}], "max_tokens": 40,
                                                          "max_completion_tokens": 5, "temperature": 0.0}).json()
        assert newer["usage"] == chat["usage"] and newer["choices"][0]["message"] == chat["choices"][0]["message"]
        if chat["usage"]["completion_tokens"] == 5:
            assert chat["choices"][0]["finish_reason"] == "length" and msg["stop_reason"] == "max_tokens"
        else:  # ended by an end-of-sequence token
            assert chat["choices"][0]["finish_reason"] == "stop" and msg["stop_reason"] == "end_turn"
    finally:
        app.state.engine, app.state.server_config = old
        engine.shutdown()


def test_finish_callback_reports_tokens_and_reason(served):
    """The scheduler tells a finished request's ``finish_callback`` the number of generated tokens and whether an
    end-of-sequence token or the budget ended it, before the stream's STOP; a cancelled request hears nothing."""
    from astrai_b200.inference.task import STOP

    model, tok = served
    s = _sched(served)
    s.start()
    try:
        log, done = [], threading.Event()

        def heard(x):
            log.append(x)
            if x is STOP:
                done.set()

        s.add_task(prompt="the quick brown fox", max_tokens=5, temperature=0.0, stream_callback=heard, finish_callback=heard)
        assert done.wait(30)
        info = log[-2]
        assert log[-1] is STOP and isinstance(info, dict) and set(info) == {"completion_tokens", "finish_reason"}
        assert 1 <= info["completion_tokens"] <= 5
        assert info["finish_reason"] == ("length" if info["completion_tokens"] == 5 else "stop")
        assert sum(isinstance(x, dict) for x in log) == 1
        mgr = s._task_mgr
        deadline = time.time() + 10
        while (mgr._callbacks or mgr._finish_callbacks) and time.time() < deadline:
            time.sleep(0.01)  # the loop forgets both callbacks when it retires the request
        assert not mgr._callbacks and not mgr._finish_callbacks

        quiet = []
        _slow_down(s)
        tid = s.add_task(prompt="the quick brown fox", max_tokens=40, temperature=0.0, stream_callback=lambda x: None, finish_callback=quiet.append)
        time.sleep(0.05)
        s.remove_task(tid)
        deadline = time.time() + 10
        while s.get_stats()["active_tasks"] and time.time() < deadline:
            time.sleep(0.01)
        assert quiet == [] and not mgr._finish_callbacks
    finally:
        s.stop()
