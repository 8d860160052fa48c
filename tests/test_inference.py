"""Cache allocator / radix index, sampling, scheduler equivalence, engine, HTTP protocol formats."""

import asyncio
import json
import threading

import pytest
import torch

from helpers import build_tokenizer_dir, tiny_config


@pytest.fixture(scope="module")
def tok(tmp_path_factory):
    from astrai_b200.tokenize import AutoTokenizer

    return AutoTokenizer.from_pretrained(build_tokenizer_dir(str(tmp_path_factory.mktemp("tok"))))


@pytest.fixture(scope="module")
def model():
    from astrai_b200.models import AutoRegressiveLM

    torch.manual_seed(0)
    return AutoRegressiveLM(tiny_config()).eval()


def test_allocator_refcount_and_lru():
    from astrai_b200.inference.cache import Allocator

    a = Allocator(3)
    evicted = []
    a.on_evict = evicted.append
    p0, p1, p2 = a.alloc(), a.alloc(), a.alloc()
    assert {p0, p1, p2} == {0, 1, 2} and a.alloc() == -1
    a.inc_ref(p0)
    a.free(p0)
    assert a.ref_count(p0) == 1 and a.alloc() == -1
    a.free(p0, keep_cached=True)
    a.free(p1, keep_cached=True)
    assert a.alloc() == p0 and evicted == [p0]  # least recently released cached page goes first
    a.inc_ref(p1)  # a cache hit takes the page out of the LRU
    assert a.alloc() == -1
    a.free(p2)
    assert a.alloc() == p2


def test_radix_cache_prefix_semantics():
    from astrai_b200.inference.cache import RadixCache

    r = RadixCache(page_size=2)
    ids = [1, 2, 3, 4, 5]
    r.record(10, ids, 0)
    r.record(11, ids, 1)
    r.record(99, ids, 2)  # the third page is not full: ignored
    assert r.lookup(ids) == [10, 11] and r.lookup([1, 2, 9, 9]) == [10] and r.lookup([7, 7]) == []
    r.record(12, [1, 2, 8, 8], 1)  # a branch under the shared first page
    assert r.lookup([1, 2, 8, 8, 0]) == [10, 12]
    r.evict(10)
    assert r.lookup(ids) == [] and not r.has_page(10) and r.has_page(11)


@pytest.mark.parametrize("page_size", [1, 2, 16])
def test_paged_alloc_extend_free_roundtrip(page_size):
    from astrai_b200.inference.cache import PagePool, TaskCacheManager
    from astrai_b200.inference.workspace import InferenceWorkspace

    pool = PagePool(2, 1, 8, max_batch_size=2, max_seq_len=40, device="cpu", dtype=torch.float32, page_size=page_size, n_tokens=64)
    mgr = TaskCacheManager(pool)
    ws = InferenceWorkspace(2, 40, 2, 8, "cpu", torch.float32, n_kv_heads=1, max_prefill_tokens=80)
    prompt = list(range(100, 119))
    assert mgr.task_alloc("a", prompt) and mgr.task_alloc("b", prompt[:5])
    assert not mgr.task_alloc("c", [1])  # no request row left
    kv = mgr.bind(["a", "b"], ws, start_pos=0)
    assert kv.out_cache_loc.numel() == 24 and kv.q_lens == [19, 5] and kv.qo_indptr.tolist() == [0, 19, 24]
    assert len(set(kv.out_cache_loc.tolist())) == 24  # distinct slots
    st = mgr.state("a")
    row = pool.req_pool.host[st.req_idx]
    for pos in (0, 7, 18):
        assert row[pos].item() == st.pages[pos // page_size] * page_size + pos % page_size
    assert mgr.task_extend("a", 19) and mgr.task_extend("b", 5)
    kv = mgr.bind(["a", "b"], ws)
    assert kv.seq_lens.tolist() == [20, 6] and not mgr.bind_was_steady
    assert mgr.task_extend("a", 20) and mgr.task_extend("b", 6)
    kv = mgr.bind(["a", "b"], ws)
    assert mgr.bind_was_steady and kv.seq_lens.tolist() == [21, 7]
    assert not mgr.task_extend("a", 40)  # beyond max_seq_len
    free_before = pool.allocator.available()
    mgr.task_free("a")
    mgr.task_free("b")
    assert pool.allocator.available() > free_before and mgr.task_alloc("c", [1])


def test_sampling_rules():
    from astrai_b200.inference.runtime.sample import SamplingPipeline, TemperatureStrategy, TopKStrategy, TopPStrategy, sample

    logits = torch.tensor([[1.0, 3.0, 2.0, 0.0], [0.5, 0.1, 0.2, 4.0]])
    assert sample(logits.clone(), temperature=0.0).tolist() == [1, 3]
    assert sample(logits.clone(), temperature=torch.zeros(2), top_k=1).tolist() == [1, 3]
    k = TopKStrategy(torch.tensor([2, 0])).apply(logits.clone())
    assert torch.isinf(k[0, [0, 3]]).all() and torch.isfinite(k[1]).all()
    k1 = TopKStrategy(1).apply(logits.clone())
    assert torch.isfinite(k1).sum(dim=-1).tolist() == [1, 1]
    probs = torch.tensor([[0.5, 0.3, 0.15, 0.05]]).log()
    p = TopPStrategy(0.7).apply(probs.clone())
    assert torch.isfinite(p[0]).tolist() == [True, True, False, False]  # the token that crosses 0.7 stays
    assert torch.isfinite(TopPStrategy(1.0).apply(probs.clone())).all()
    t = TemperatureStrategy(torch.tensor([0.0, 2.0])).apply(logits.clone())
    assert torch.isfinite(t).all() and torch.allclose(t[1], logits[1] / 2)
    hist = torch.tensor([[1, 1, 2], [3, 0, 0]])
    mask = torch.tensor([[True, True, True], [True, False, False]])
    torch.manual_seed(0)
    toks, lp = sample(logits.clone(), temperature=1.0, top_k=0, frequency_penalty=torch.tensor([100.0, 100.0]),
                      input_ids=hist, input_mask=mask, return_logprobs=True)
    assert toks[0].item() not in (1, 2) and toks[1].item() != 3 and (lp <= 0).all()
    torch.manual_seed(0)
    draws = torch.stack([sample(logits.clone(), temperature=1.0, top_k=2) for _ in range(200)])
    assert set(draws[:, 0].tolist()) <= {1, 2} and set(draws[:, 1].tolist()) <= {0, 3}
    pipe = SamplingPipeline([TemperatureStrategy(0.0)])
    tk, lps = pipe.sample(logits.clone(), return_logprobs=True)
    assert torch.allclose(lps, torch.log_softmax(logits, -1).gather(-1, tk[:, None])[:, 0])


@pytest.mark.parametrize("paged,page_size", [(True, 4), (True, 16), (False, 1)])
def test_run_batch_matches_full_forward(model, tok, paged, page_size):
    from astrai_b200.inference import InferenceScheduler

    s = InferenceScheduler(model, tok, max_batch_size=4, max_seq_len=64, enable_cuda_graph=False, page_size=page_size, paged=paged)
    prompts = [[5, 6, 7, 8, 9, 10, 11, 12, 13], [20, 21, 22], [5, 6, 7, 8, 9, 10, 11, 12, 30, 31]]
    outs, lps = zip(*s.run_batch(prompts, max_tokens=5, temperature=0.0, return_logprobs=True))
    for p, o, lp in zip(prompts, outs, lps):
        seq = list(p)
        for step in range(len(o)):
            with torch.no_grad():
                logits = model(torch.tensor([seq]))["logits"][0, -1]
            assert logits.argmax().item() == o[step]
            assert lp[step] == pytest.approx(torch.log_softmax(logits, -1)[o[step]].item(), abs=1e-4)
            seq.append(o[step])
    assert s.run_batch(prompts, max_tokens=5, temperature=0.0) == list(outs)  # second pass reuses cached prefix pages
    if paged and page_size == 4:
        assert s.cache.prefix.lookup(prompts[0]) != []
    assert s.run_batch([[1] * 64, [1, 2]], max_tokens=3, temperature=0.0)[0] == []  # prompt fills the context: skipped


@pytest.mark.parametrize("budget", [3, 7, 64])
def test_chunked_prefill_gives_the_same_tokens(model, tok, budget):
    """Prompts cut into chunks of at most `budget` tokens per step (decodes of the others running in between) produce
    exactly what whole-prompt prefill produces."""
    from astrai_b200.inference import InferenceScheduler

    prompts = [list(range(5, 30)), [20, 21, 22], list(range(5, 17)) + [40, 41], [7]]
    plain = InferenceScheduler(model, tok, max_batch_size=4, max_seq_len=64, enable_cuda_graph=False, page_size=4, paged=True)
    want = plain.run_batch(prompts, max_tokens=6, temperature=0.0, return_logprobs=True)
    chunked = InferenceScheduler(model, tok, max_batch_size=4, max_seq_len=64, enable_cuda_graph=False, page_size=4, paged=True,
                                 max_prefill_tokens=budget, chunked_prefill=True)
    got = chunked.run_batch(prompts, max_tokens=6, temperature=0.0, return_logprobs=True)
    for (o, lp), (o2, lp2) in zip(want, got):
        assert o == o2
        assert lp2 == pytest.approx(lp, abs=1e-4)
    assert chunked.run_batch(prompts, max_tokens=6, temperature=0.0) == [o for o, _ in want]  # prefix pages reused


def test_stop_ids_and_max_tokens(model, tok):
    from astrai_b200.inference import InferenceScheduler

    s = InferenceScheduler(model, tok, max_batch_size=2, max_seq_len=32, enable_cuda_graph=False)
    out = s.run_batch([[5, 6, 7]], max_tokens=4, temperature=0.0)[0]
    assert len(out) == 4
    first = out[0]

    class StopTok:
        stop_ids = [first]

        def __getattr__(self, name):
            return getattr(tok, name)

    s2 = InferenceScheduler(model, StopTok(), max_batch_size=2, max_seq_len=32, enable_cuda_graph=False)
    assert s2.run_batch([[5, 6, 7]], max_tokens=4, temperature=0.0)[0] == [first]


def test_engine_generate_stream_batch_and_stats(model, tok):
    from astrai_b200.inference import InferenceEngine

    with InferenceEngine(model, tok, max_batch_size=4, max_seq_len=64, enable_cuda_graph=False) as eng:
        text = eng.generate("hello world", max_tokens=5, temperature=0.0)
        assert isinstance(text, str)
        pieces = list(eng.generate("hello world", stream=True, max_tokens=5, temperature=0.0))
        assert "".join(pieces) == text
        both = eng.generate(["hello", "the quick brown fox"], max_tokens=4, temperature=0.0)
        assert isinstance(both, list) and len(both) == 2
        assert eng.generate("x", max_tokens=0) == "" and list(eng.generate("x", stream=True, max_tokens=0)) == []

        async def drain():
            return [p async for p in eng.generate_async("hello world", max_tokens=5, temperature=0.0)]

        assert "".join(asyncio.run(drain())) == text
        stats = eng.get_stats()
        assert stats["total_tasks"] >= 5 and "avg_ttft_ms" in stats and stats["active_tasks"] == 0


def test_scheduler_thread_safety_under_concurrent_submitters(model, tok):
    from astrai_b200.inference import InferenceEngine

    results, errors = {}, []
    with InferenceEngine(model, tok, max_batch_size=3, max_seq_len=48, enable_cuda_graph=False) as eng:
        def worker(i):
            try:
                results[i] = eng.generate(f"hello {i}", max_tokens=3 + i % 3, temperature=0.0)
            except Exception as exc:  # noqa: BLE001
                errors.append(exc)

        threads = [threading.Thread(target=worker, args=(i,)) for i in range(10)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=120)
    assert not errors and len(results) == 10


def test_scheduler_crash_releases_waiters(model, tok):
    from astrai_b200.inference import InferenceEngine

    eng = InferenceEngine(model, tok, max_batch_size=2, max_seq_len=32, enable_cuda_graph=False)
    eng.scheduler._executor.execute_prefill = lambda *a, **k: (_ for _ in ()).throw(RuntimeError("injected executor failure"))
    assert eng.generate("hello", max_tokens=3) == ""  # STOP delivered, caller not left hanging
    eng.shutdown()


class _FakeEngine:
    def __init__(self, tokenizer, pieces):
        self.tokenizer, self.pieces, self.calls = tokenizer, pieces, []

    def generate_async(self, prompt, **kw):
        self.calls.append((prompt, kw))
        pieces = self.pieces

        async def agen():
            for p in pieces:
                yield p

        return agen()

    def get_stats(self):
        return {"total_tasks": 1}

    def shutdown(self):
        pass


@pytest.fixture
def client(tok):
    from fastapi.testclient import TestClient

    from astrai_b200.inference.network import get_app

    app = get_app()
    app.state.server_config = {"_test": True}
    app.state.engine = None
    with TestClient(app) as c:
        yield c, app
    app.state.engine = None


def _sse_payloads(text):
    return [line[6:] for line in text.splitlines() if line.startswith("data: ")]


def test_http_health_and_503(client):
    c, app = client
    assert c.get("/health").json() == {"status": "ok", "model_loaded": False}
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}]})
    assert r.status_code == 503 and r.json() == {"detail": "Engine not initialized"}
    assert c.post("/v1/chat/completions", json={"messages": "oops"}).status_code == 422


def test_http_openai_formats(client, tok):
    c, app = client
    app.state.engine = _FakeEngine(tok, ["Hel", "lo", " END", " tail"])
    body = {"messages": [{"role": "user", "content": "hi"}], "stop": ["END"], "max_tokens": 7, "temperature": 0.5}
    r = c.post("/v1/chat/completions", json=body).json()
    assert r["object"] == "chat.completion" and r["choices"][0]["message"] == {"role": "assistant", "content": "Hello END"}
    assert r["choices"][0]["finish_reason"] == "stop" and r["usage"]["completion_tokens"] == 2
    prompt, kw = app.state.engine.calls[0]
    assert "<|im_start|>user" in prompt and kw["max_tokens"] == 7 and kw["top_k"] == 50 and kw["temperature"] == 0.5
    s = c.post("/v1/chat/completions", json={**body, "stream": True})
    assert s.headers["content-type"].startswith("text/event-stream")
    data = _sse_payloads(s.text)
    assert data[-1] == "[DONE]"
    chunks = [json.loads(d) for d in data[:-1]]
    assert chunks[0]["choices"][0]["delta"] == {"role": "assistant"}
    assert [ch["choices"][0]["delta"].get("content") for ch in chunks[1:3]] == ["Hel", "lo"] and chunks[1]["created"] == 0
    assert chunks[3]["choices"][0]["finish_reason"] == "stop" and chunks[3]["choices"][0]["delta"] == {}
    assert "choices" not in chunks[4] and chunks[4]["total_tokens"] == chunks[4]["prompt_tokens"] + 2
    assert c.get("/stats").json() == {"total_tasks": 1}


def test_http_openai_tool_calls(client, tok):
    c, app = client
    pieces = ["I will ", '{"name": "lookup", ', '"arguments": {"q": "x"}}']
    app.state.engine = _FakeEngine(tok, pieces)
    tools = [{"type": "function", "function": {"name": "lookup", "parameters": {}}}]
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "tools": tools}).json()
    assert r["choices"][0]["finish_reason"] == "tool_calls"
    call = r["choices"][0]["message"]["tool_calls"][0]
    assert call["function"] == {"name": "lookup", "arguments": '"q": "x"'} and r["choices"][0]["message"]["content"] == "I will"
    s = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "tools": tools, "stream": True})
    chunks = [json.loads(d) for d in _sse_payloads(s.text)[:-1]]
    finish = [ch for ch in chunks if ch.get("choices") and ch["choices"][0]["finish_reason"]]
    assert finish[0]["choices"][0]["finish_reason"] == "tool_calls"
    names = [ch["choices"][0]["delta"]["tool_calls"][0]["function"].get("name") for ch in chunks
             if ch.get("choices") and "tool_calls" in ch["choices"][0]["delta"]]
    assert "lookup" in names


def test_http_anthropic_formats(client, tok):
    c, app = client
    app.state.engine = _FakeEngine(tok, ["Hi", " there", " STOP now"])
    body = {"messages": [{"role": "user", "content": [{"type": "text", "text": "hey"}]}], "system": "be brief", "stop_sequences": ["STOP"]}
    r = c.post("/v1/messages", json=body).json()
    assert r["type"] == "message" and r["content"] == [{"type": "text", "text": "Hi there "}]
    assert r["stop_reason"] == "stop_sequence" and r["stop_sequence"] == "STOP" and r["usage"]["output_tokens"] == 2
    prompt, kw = app.state.engine.calls[0]
    assert "be brief" in prompt and kw["max_tokens"] == 1024
    s = c.post("/v1/messages", json={**body, "stream": True})
    events = [l[7:] for l in s.text.splitlines() if l.startswith("event: ")]
    assert events == ["message_start", "content_block_start", "content_block_delta", "content_block_delta",
                      "content_block_delta", "content_block_stop", "message_delta", "message_stop"]
    data = _sse_payloads(s.text)
    assert data[-1] == "[DONE]" and json.loads(data[4])["delta"]["text"] == " "  # unsent text before the stop sequence
    assert json.loads(data[6])["delta"]["stop_reason"] == "stop_sequence"
    app.state.engine = _FakeEngine(tok, ["plain"])
    assert c.post("/v1/messages", json={"messages": [{"role": "user", "content": "x"}]}).json()["stop_reason"] == "end_turn"


def test_fused_projection_weights_keep_names_values_and_outputs(model):
    from astrai_b200.inference.runtime.executor import fuse_projection_weights
    import copy

    m = copy.deepcopy(model).eval()
    before = {k: v.clone() for k, v in m.state_dict().items()}
    ids = torch.tensor([[5, 6, 7, 8, 9]])
    with torch.no_grad():
        want = m(ids)["logits"]
    n = fuse_projection_weights(m)
    assert n == 2 * len(m.layers)
    attn = m.layers[0].attention
    assert attn.fused_qkv.shape[0] == attn.q_proj.weight.shape[0] + 2 * attn.k_proj.weight.shape[0]
    assert attn.q_proj.weight.data_ptr() == attn.fused_qkv.data_ptr()  # the parameters are views of the fused matrix
    after = m.state_dict()
    assert set(after) == set(before) and all(torch.equal(after[k], before[k]) for k in before)
    with torch.no_grad():
        assert torch.equal(m(ids)["logits"], want)
    assert fuse_projection_weights(m) == 0  # idempotent


def test_fused_projection_weights_stack_moe_experts():
    import copy
    import sys

    sys.path.insert(0, str(__import__("pathlib").Path(__file__).parent))
    from helpers import tiny_config

    from astrai_b200.inference.runtime.executor import fuse_projection_weights
    from astrai_b200.models import AutoRegressiveLM

    torch.manual_seed(0)
    m = AutoRegressiveLM(tiny_config(ffn_type="moe", n_routed_experts=4, n_activated_experts=2, moe_intermediate_size=16,
                                     n_shared_experts=1)).eval()
    before = {k: v.clone() for k, v in m.state_dict().items()}
    ids = torch.tensor([[5, 6, 7, 8, 9, 10]])
    with torch.no_grad():
        want = m(ids)["logits"]
    assert fuse_projection_weights(m) > 0
    moe_layer = m.layers[0].mlp
    w_gu, w_dn = moe_layer.stacked_experts
    assert w_gu.shape[0] == 4 and moe_layer.routed_experts[2].down.weight.data_ptr() == w_dn[2].data_ptr()
    assert moe_layer.routed_experts[1].gate.weight.data_ptr() == w_gu[1].data_ptr()  # still a view after the MLP pass
    after = m.state_dict()
    assert all(torch.equal(after[k], before[k]) for k in before)
    with torch.no_grad():
        assert torch.equal(m(ids)["logits"], want)
