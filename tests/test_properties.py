"""Property-based checks (hypothesis, fixed seed): invariants that must hold for any input, not only the hand-picked ones."""

import json
import random

import pytest
import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

PROFILE = settings(max_examples=60, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.too_slow])


# ------------------------------------------------------------------------------------------------ paged pool + prefix index
class _PoolModel:
    """What the pool promises, stated naively: which token sequence every page of every live request holds."""

    def __init__(self):
        self.content = {}  # physical page -> tuple of the tokens whose K / V it holds (full pages only)


@PROFILE
@given(st.lists(st.tuples(st.sampled_from(["alloc", "extend", "finish", "drop"]), st.integers(0, 5), st.integers(1, 40)), min_size=1, max_size=60),
       st.integers(0, 3))
def test_paged_pool_never_hands_a_page_to_two_requests_and_prefix_hits_hold_the_right_tokens(ops, seed):
    from astrai_b200.inference.cache import PagePool, TaskCacheManager

    page = 4
    pool = PagePool(n_layers=1, n_kv_heads=1, head_dim=2, max_batch_size=4, max_seq_len=48, device="cpu", dtype=torch.float32,
                    page_size=page, n_tokens=page * 20)
    mgr = TaskCacheManager(pool)
    rng = random.Random(seed)
    live = {}          # task id -> list of token ids whose K / V are in the cache
    holds = {}         # physical page -> tokens it was last filled with (as the index may remember them)
    serial = 0
    for kind, which, n in ops:
        if kind == "alloc":
            serial += 1
            # prompts share prefixes: they are cut from three fixed streams
            stream = [(which * 7 + i * (which + 1)) % 11 for i in range(64)]
            prompt = stream[: max(1, min(n, 40))]
            tid = f"t{serial}"
            if mgr.task_alloc(tid, prompt):
                state = mgr.state(tid)
                # the cached prefix is whole pages, strictly shorter than the prompt, and holds exactly these tokens
                assert state.cached % page == 0 and state.cached < len(prompt) + page
                for i in range(state.cached // page):
                    assert holds.get(state.pages[i]) == tuple(prompt[i * page:(i + 1) * page])
                mgr.task_record_hashes(tid, prompt, state.cached // page)
                for i in range(len(prompt) // page):
                    holds[state.pages[i]] = tuple(prompt[i * page:(i + 1) * page])
                live[tid] = list(prompt)
        elif live:
            tid = sorted(live)[which % len(live)]
            if kind == "extend":
                for _ in range(min(n, 6)):
                    pos = len(live[tid])
                    if not mgr.task_extend(tid, pos):
                        break
                    live[tid].append(rng.randrange(11))
            else:
                if kind == "finish":  # a finished request leaves its full pages in the index
                    state = mgr.state(tid)
                    mgr.task_record_hashes(tid, live[tid])
                    for i in range(len(live[tid]) // page):
                        holds[state.pages[i]] = tuple(live[tid][i * page:(i + 1) * page])
                mgr.task_free(tid)
                del live[tid]
        # invariants after every operation
        owners = {}
        for tid, tokens in live.items():
            state = mgr.state(tid)
            assert state.length == len(tokens) and len(state.pages) * page >= len(tokens)
            for i, p in enumerate(state.pages):
                owners.setdefault(p, []).append((tid, i))
        for p, users in owners.items():
            assert pool.allocator.ref_count(p) == len(users)
            if len(users) > 1:  # a shared page is a shared prefix page: the same position, the same tokens, full
                assert len({i for _, i in users}) == 1
                i = users[0][1]
                spans = {tuple(live[t][i * page:(i + 1) * page]) for t, _ in users}
                assert len(spans) == 1 and len(next(iter(spans))) == page
        in_use = len(owners)
        assert pool.allocator.available() == 20 - in_use
    for tid in list(live):
        mgr.task_free(tid)
    assert pool.allocator.available() == 20


# ----------------------------------------------------------------------------------------------------------- packing
@PROFILE
@given(st.lists(st.integers(1, 30), min_size=1, max_size=40), st.integers(4, 24), st.sampled_from(["keep_start", "keep_end"]))
def test_bfd_bins_hold_every_document_once_and_never_overflow(lengths, limit, mode):
    from astrai_b200.preprocessing.packing import plan_bfd

    docs = [[i] * n for i, n in enumerate(lengths)]
    bins = plan_bfd(docs, limit, mode)
    seen = sorted(i for b in bins for i in b)
    assert seen == list(range(len(docs)))
    for b in bins:
        assert sum(min(lengths[i], limit) for i in b) <= limit
    # no two bins could have been merged at the time the later one was opened: every bin after the first is more than
    # the room left in some earlier one only if ... (best fit): at least, no bin is empty
    assert all(b for b in bins)


@PROFILE
@given(st.lists(st.lists(st.integers(1, 99), min_size=1, max_size=25), min_size=1, max_size=12), st.integers(4, 16),
       st.sampled_from(["simple", "bfd", "bfd_split"]))
def test_packers_keep_columns_aligned_and_lose_tokens_only_by_truncation(docs, limit, name):
    from astrai_b200.preprocessing.packing import PackingStrategyFactory

    keys = {"sequence": [list(d) for d in docs], "loss_mask": [[t % 2 for t in d] for d in docs]}
    out = PackingStrategyFactory.create(name).apply(keys, limit, "keep_start")
    assert len(out["sequence"]) == len(out["loss_mask"])
    for seq, mask in zip(out["sequence"], out["loss_mask"]):
        assert len(seq) == len(mask) and [t % 2 for t in seq] == mask  # the mask travelled with its tokens
        assert len(seq) <= limit
    kept = sorted(t for seq in out["sequence"] for t in seq)
    if name == "bfd_split":  # long documents are cut into pieces, nothing is lost
        assert kept == sorted(t for d in docs for t in d)
    else:  # "simple" does not pack at all, "bfd" packs whole documents: both cut a long document to the limit
        assert kept == sorted(t for d in docs for t in d[:limit])
    if name == "simple":
        assert out["sequence"] == [d[:limit] for d in docs]


# ------------------------------------------------------------------------------------------------- tool-call parser
@PROFILE
@given(st.lists(st.integers(1, 9), min_size=1, max_size=40), st.booleans(), st.integers(0, 2))
def test_tool_parser_gives_the_same_calls_for_any_chunking(cuts, with_text, n_calls):
    from astrai_b200.inference.network import ToolParserFactory

    calls = [{"name": f"fn_{i}", "arguments": {"x": i, "s": 'a "quoted" } brace', "nested": {"k": [1, 2, {"z": "}"}]}}} for i in range(n_calls)]
    text = ("Let me look that up. " if with_text else "") + " ".join(json.dumps(c, ensure_ascii=False) for c in calls)
    whole = ToolParserFactory.create("simple_json").parse_complete(text) or {}
    parser = ToolParserFactory.create("simple_json")
    names, args, content, pos, i = {}, {}, "", 0, 0
    while pos < len(text):
        pos = min(pos + cuts[i % len(cuts)], len(text))
        i += 1
        for delta in parser.feed(text[:pos]):  # the parser is handed everything generated so far
            content += delta.get("content", "")
            for tc in delta.get("tool_calls", []):
                fn = tc.get("function", {})
                if fn.get("name"):
                    assert tc["index"] not in names  # the name comes once, before any argument text
                    names[tc["index"]] = fn["name"]
                args[tc["index"]] = args.get(tc["index"], "") + fn.get("arguments", "")
    got = [{"name": names[k], "arguments": json.loads("{" + args[k] + "}")} for k in sorted(names)]  # deltas carry the inner text
    assert got == calls
    # as in the reference, "arguments" is the text between the outer braces of the arguments object
    whole_calls = [{"name": c["function"]["name"], "arguments": json.loads("{" + c["function"]["arguments"] + "}")}
                   for c in whole.get("tool_calls", [])]
    assert whole_calls == calls
    if with_text:
        assert content.strip() == "Let me look that up."
    elif calls:
        assert content.strip() == ""
    assert parser.has_tool_calls == bool(calls)


# --------------------------------------------------------------------------------------------------------- sampler
@PROFILE
@given(st.integers(1, 97), st.integers(1, 6), st.integers(0, 5), st.integers(0, 3), st.booleans())
def test_sampler_ranks_cover_the_data_and_a_resumed_rank_continues_where_it_stopped(n, world, seed, epoch, shuffle):
    from astrai_b200.data import RDSampler

    data = list(range(n))
    per_rank = []
    for rank in range(world):
        s = RDSampler(data, partition=(rank, world), seed=seed, shuffle=shuffle, start_epoch=epoch)
        assert len(s) == -(-n // world)
        idx = list(s)
        assert len(idx) == -(-n // world)
        per_rank.append(idx)
        cut = len(idx) // 2
        resumed = RDSampler(data, partition=(rank, world), seed=seed, shuffle=shuffle, start_epoch=epoch, start_iter=cut)
        assert list(resumed) == idx[cut:]
    flat = [i for idx in per_rank for i in idx]
    assert set(flat) == set(data)                       # everything is drawn
    assert len(flat) - n < world                        # padding by wrapping: fewer than one extra sample per rank
    if n % world == 0:                                  # no padding: the ranks' shares are disjoint
        assert len(set(flat)) == len(flat)


# ------------------------------------------------------------------------------------------------ streaming detokeniser
@pytest.fixture(scope="module")
def tokenizer(tmp_path_factory):
    from astrai_b200.tokenize import AutoTokenizer
    from helpers import build_tokenizer_dir

    return AutoTokenizer.from_pretrained(build_tokenizer_dir(str(tmp_path_factory.mktemp("tok"))))


@PROFILE
@given(st.lists(st.sampled_from(list("abc xyz,.!?\n") + ["é", "ß", "漢", "字", "🙂", "the ", "quick ", "hello world"]), max_size=30))
def test_streamed_pieces_add_up_to_the_decoded_text(tokenizer, parts):
    text = "".join(parts)
    from astrai_b200.inference.task import StreamDecoder

    ids = tokenizer.encode(text)
    decoder = StreamDecoder(tokenizer)
    pieces = [decoder.push(i) for i in ids]
    assert all(isinstance(p, str) for p in pieces)
    joined = "".join(pieces)
    whole = tokenizer.decode(ids)
    assert whole.startswith(joined)  # nothing wrong is ever emitted; an unfinished multi-byte character may be held back
    assert "�" not in joined
    if ids and whole and not whole.endswith("�"):
        assert joined == whole


# ------------------------------------------------------------------------------------------------------ stop sequences
@PROFILE
@given(st.lists(st.text(alphabet="ab|", min_size=0, max_size=3), max_size=4), st.text(alphabet="ab|", max_size=12))
def test_stop_checker_finds_a_sequence_exactly_when_one_occurs(stops, text):
    from astrai_b200.inference.network import StopChecker

    found = StopChecker(stops).check(text)
    real = [s for s in stops if s]
    if found is None:
        assert not any(s in text for s in real)
    else:
        assert found in real and found in text


# ------------------------------------------------------------------------------ continuous batching does not change answers
@pytest.fixture(scope="module")
def tiny_lm():
    from astrai_b200.models import AutoRegressiveLM
    from helpers import tiny_config

    torch.manual_seed(0)
    return AutoRegressiveLM(tiny_config(vocab_size=256, hidden_size=32, intermediate_size=64, max_position_embeddings=128)).eval()


class _Ids:
    stop_ids = [1]

    def encode(self, text):
        return [int(t) for t in str(text).split()]

    def decode(self, ids, skip_special_tokens=True):
        return " ".join(map(str, ids))


_ALONE = {}


def _alone(model, prompt, budget):
    """Greedy answer of one prompt on its own, contiguous cache, whole-prompt prefill: the statement to agree with."""
    from astrai_b200.inference import InferenceScheduler

    key = (tuple(prompt), budget)
    if key not in _ALONE:
        s = InferenceScheduler(model, _Ids(), max_batch_size=1, max_seq_len=96, enable_cuda_graph=False, paged=False, page_size=1)
        _ALONE[key] = s.run_batch([list(prompt)], max_tokens=budget, temperature=0.0)[0]
    return _ALONE[key]


@settings(max_examples=25, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.too_slow, HealthCheck.function_scoped_fixture])
@given(st.lists(st.tuples(st.integers(0, 2), st.integers(1, 30), st.integers(1, 8)), min_size=1, max_size=6),
       st.sampled_from([4, 8, 16]), st.booleans(), st.sampled_from([8, 24, 4096]), st.integers(1, 6))
def test_answers_do_not_depend_on_batch_mates_page_size_or_prefill_chunking(tiny_lm, requests, page, chunked, prefill_budget, slots):
    from astrai_b200.inference import InferenceScheduler

    # prompts are cut from three streams, so that several share page-aligned prefixes and hit the prefix index
    prompts = [[(stream * 37 + i * (stream + 3)) % 250 + 2 for i in range(n)] for stream, n, _ in requests]
    budgets = [b for _, _, b in requests]
    sched = InferenceScheduler(tiny_lm, _Ids(), max_batch_size=slots, max_seq_len=96, enable_cuda_graph=False, paged=True, page_size=page,
                               kv_cache_tokens=96 * 8, chunked_prefill=chunked, max_prefill_tokens=prefill_budget)
    want = [_alone(tiny_lm, p, b) for p, b in zip(prompts, budgets)]
    # the synchronous path takes one budget for the batch: group the requests by budget, twice over to reuse cached prefixes
    for _ in range(2):
        for budget in sorted(set(budgets)):
            group = [i for i, b in enumerate(budgets) if b == budget]
            for start in range(0, len(group), slots):
                part = group[start:start + slots]
                got = sched.run_batch([prompts[i] for i in part], max_tokens=budget, temperature=0.0)
                assert got == [want[i] for i in part]
    assert sched._cache.allocator.available() == 96 * 8 // page  # every page came back


@settings(max_examples=8, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.too_slow, HealthCheck.function_scoped_fixture])
@given(st.lists(st.tuples(st.integers(0, 2), st.integers(1, 30), st.integers(1, 8), st.integers(0, 3)), min_size=1, max_size=10),
       st.sampled_from([4, 16]), st.booleans(), st.integers(1, 4), st.sampled_from([0, 2]))
def test_the_serving_loop_gives_every_request_its_own_answer_whenever_it_arrives(tiny_lm, requests, page, chunked, slots, defer):
    import threading
    import time

    from astrai_b200.inference import InferenceScheduler
    from astrai_b200.inference.task import STOP

    prompts = [[(stream * 37 + i * (stream + 3)) % 250 + 2 for i in range(n)] for stream, n, _, _ in requests]
    want = [_alone(tiny_lm, p, b) for p, (_, _, b, _) in zip(prompts, requests)]
    sched = InferenceScheduler(tiny_lm, _Ids(), max_batch_size=slots, max_seq_len=96, enable_cuda_graph=False, paged=True, page_size=page,
                               kv_cache_tokens=96 * 6, chunked_prefill=chunked, max_prefill_tokens=16, prefill_defer_steps=defer,
                               prefill_defer_min_batch=1, prefill_defer_tokens=64)
    got = [[] for _ in prompts]
    done = [threading.Event() for _ in prompts]

    def collector(i):
        def on_piece(piece):
            if piece is STOP:
                done[i].set()
            else:
                got[i].extend(int(t) for t in piece.split())
        return on_piece

    sched.start()
    try:
        for i, (prompt, (_, _, budget, pause)) in enumerate(zip(prompts, requests)):
            sched.add_task(prompt, max_tokens=budget, temperature=0.0, stream_callback=collector(i))
            time.sleep(pause * 0.003)  # some arrive together, some while others decode
        assert all(e.wait(timeout=60) for e in done)
    finally:
        sched.stop()
    assert got == want
    assert sched._cache.allocator.available() == 96 * 6 // page


# ------------------------------------------------------------------------------------------- learning-rate schedules
@PROFILE
@given(st.sampled_from(["cosine", "sgdr", "wsd"]), st.integers(0, 20), st.integers(1, 60), st.floats(0.0, 0.5), st.integers(0, 90))
def test_schedules_stay_in_bounds_warm_up_monotonically_and_resume_exactly(kind, warmup, span, floor, resume_at):
    from astrai_b200.trainer import SchedulerFactory

    def make():
        opt = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=2.0)
        extra = {"cosine": {"lr_decay_steps": span}, "sgdr": {"cycle_length": span, "t_mult": 2},
                 "wsd": {"stable_steps": span // 2, "decay_steps": max(span - span // 2, 1)}}[kind]
        return opt, SchedulerFactory.create(kind, opt, warmup_steps=warmup, min_rate=floor, **extra)

    opt, sched = make()
    lrs = []
    for _ in range(100):
        lrs.append(opt.param_groups[0]["lr"])
        opt.step()
        sched.step()
    assert all(2.0 * floor - 1e-9 <= lr <= 2.0 + 1e-9 for lr in lrs)
    assert all(b >= a - 1e-12 for a, b in zip(lrs[:warmup], lrs[1:warmup + 1]))  # never falls while warming up
    if warmup < 100:
        assert lrs[warmup] == pytest.approx(2.0)  # the peak is reached right after the warm-up
    # a scheduler rebuilt from the state saved after `resume_at` steps continues the same curve
    opt2, sched2 = make()
    for _ in range(resume_at):
        opt2.step()
        sched2.step()
    state = sched2.state_dict()
    opt3, sched3 = make()
    sched3.load_state_dict(state)
    for g, lr in zip(opt3.param_groups, sched3.get_last_lr()):
        g["lr"] = lr
    tail = []
    for _ in range(100 - resume_at):
        tail.append(opt3.param_groups[0]["lr"])
        opt3.step()
        sched3.step()
    assert tail == pytest.approx(lrs[resume_at:], abs=1e-12)


# ------------------------------------------------------------------------------------------------- sampling filters
@PROFILE
@given(st.integers(1, 4), st.integers(2, 40), st.integers(0, 45), st.floats(0.05, 1.0), st.floats(0.1, 3.0), st.integers(0, 10))
def test_filters_keep_the_most_likely_tokens_and_enough_probability_mass(rows, vocab, k, p, temperature, seed):
    from astrai_b200.inference.runtime.sample import SamplingPipeline, TemperatureStrategy, TopKStrategy, TopPStrategy

    logits = torch.randn(rows, vocab, generator=torch.Generator().manual_seed(seed)) * 3
    scaled = logits / temperature
    after_k = TopKStrategy(k).apply(TemperatureStrategy(temperature).apply(logits))
    kept_k = torch.isfinite(after_k)
    for r in range(rows):
        n = int(kept_k[r].sum())
        assert n >= 1 and (k <= 0 or k >= vocab or n >= min(k, vocab))       # ties may keep more than k, never fewer
        if 0 < k < vocab:
            assert scaled[r][kept_k[r]].min() >= scaled[r][~kept_k[r]].max() if (~kept_k[r]).any() else True
    out = SamplingPipeline([TemperatureStrategy(temperature), TopKStrategy(k), TopPStrategy(p)]).apply(logits)
    kept = torch.isfinite(out)
    probs_after_k = torch.softmax(after_k, -1)
    for r in range(rows):
        assert kept[r].any() and (kept[r] <= kept_k[r]).all()                  # top-p only removes
        assert kept[r][out[r].argmax()] and out[r].argmax() == logits[r].argmax()  # the most likely token always survives
        mass = float(probs_after_k[r][kept[r]].sum())
        assert mass >= min(p, 1.0) - 1e-5                                      # the kept set carries at least p of the mass
        if (~kept[r] & kept_k[r]).any():                                       # whatever was removed is no likelier than what stayed
            assert probs_after_k[r][kept[r]].min() >= probs_after_k[r][~kept[r] & kept_k[r]].max() - 1e-7


# --------------------------------------------------------------------------------- packed-document attention relations
@PROFILE
@given(st.lists(st.lists(st.integers(1, 6), min_size=1, max_size=5), min_size=1, max_size=4))
def test_run_boundaries_describe_the_same_relation_as_the_dense_document_mask(doc_lengths):
    from astrai_b200.ops.segments import from_position_ids
    from astrai_b200.trainer.strategy import make_doc_boundary_mask

    width = max(sum(row) for row in doc_lengths)
    rows = []
    for row in doc_lengths:
        pos = [i for n in row for i in range(n)]
        pos += list(range(width - len(pos)))  # the tail is one more document (possibly empty)
        rows.append(pos)
    position_ids = torch.tensor(rows)
    seg = from_position_ids(position_ids)
    assert torch.equal(seg.to_dense(), make_doc_boundary_mask(position_ids))
    assert seg.bounds[0] == 0 and seg.bounds[-1] == len(rows) * width and seg.bounds == sorted(set(seg.bounds))
    assert seg.max_len == max(b - a for a, b in zip(seg.bounds[:-1], seg.bounds[1:]))
    if width > 1:  # the inputs of a next-token objective lose their last column; so do the runs
        assert torch.equal(seg.drop_last().to_dense(), make_doc_boundary_mask(position_ids)[:, :, :-1, :-1])


# ------------------------------------------------------------------------------------------------ zig-zag sequence sharding
@PROFILE
@given(st.integers(1, 4), st.integers(1, 5), st.integers(1, 3))
def test_zigzag_split_and_merge_are_inverse_and_balance_causal_work(world, chunk, batch):
    from astrai_b200.parallel.context_parallel import zigzag_merge, zigzag_positions, zigzag_split

    seq = 2 * world * chunk
    x = torch.arange(batch * seq * 3).view(batch, seq, 3)
    parts = [zigzag_split(x, world, r) for r in range(world)]
    assert all(p.shape == (batch, 2 * chunk, 3) for p in parts)
    assert torch.equal(zigzag_merge(parts), x)
    for r in range(world):
        pos = zigzag_positions(seq, world, r)
        assert torch.equal(parts[r][0, :, 0] // 3, pos)  # a rank's rows sit at exactly these positions
    work = [int(zigzag_positions(seq, world, r).add(1).sum()) for r in range(world)]
    assert len(set(work)) == 1  # keys visible to a rank's queries under causal attention: the same for every rank


# -------------------------------------------------------------------------------------------- expert capacity limit
@PROFILE
@given(st.integers(1, 24), st.integers(1, 3), st.sampled_from([(4, 2), (8, 4), (6, 3), (4, 4)]), st.floats(1.0, 3.0), st.integers(0, 20))
def test_capacity_limit_never_overfills_a_destination_and_only_drops_what_does_not_fit(tokens, k, shape, factor, seed):
    from astrai_b200.parallel.expert_parallel import limit_rows_per_rank

    experts, world = shape
    g = torch.Generator().manual_seed(seed)
    idx = torch.randint(0, experts, (tokens, k), generator=g)
    if seed % 3 == 0:
        idx[: tokens // 2 + 1] = 0  # a hot expert
    w = torch.rand(tokens, k, generator=g) + 0.1
    new_idx, new_w, counts, dropped = limit_rows_per_rank(idx, w, experts, world, factor)
    cap = int(factor * tokens * k) // world
    local = experts // world
    per_rank = counts.view(world, local).sum(1)
    assert int(counts.sum()) == tokens * k and (per_rank <= max(cap, 0)).all() or cap * world < tokens * k
    kept = new_w > 0
    assert torch.equal(new_idx[kept], idx[kept]) and torch.equal(new_w[kept], w[kept])  # kept pairs are untouched
    assert int((~kept).sum()) == int(dropped)
    sent = torch.bincount((idx // local).flatten(), minlength=world)
    assert int(dropped) == int((sent - cap).clamp(min=0).sum())  # exactly the overflow is dropped, nothing more
    assert torch.equal(counts, torch.bincount(new_idx.flatten(), minlength=experts).int())


# -------------------------------------------------------------------------------------------------- training windows
@PROFILE
@given(st.lists(st.integers(1, 40), min_size=1, max_size=5), st.integers(1, 24), st.integers(1, 30))
def test_windows_tile_the_token_stream_across_shards_and_shift_targets_by_one(tmp_path_factory, shard_sizes, window, stride):
    from astrai_b200.data import DatasetFactory
    from astrai_b200.serialization import save_bin

    root = tmp_path_factory.mktemp("windows")
    total, start = sum(shard_sizes), 0
    for i, n in enumerate(shard_sizes):  # the stream 0, 1, 2, ... cut into shards of uneven size
        save_bin(str(root / f"shard_{i:04d}"), {"sequence": [torch.arange(start, start + n, dtype=torch.int32)]})
        start += n
    ds = DatasetFactory.load("seq", str(root), window_size=window, stride=stride)
    want = 0 if total <= window else (total - 1 - window) // stride + 1
    assert len(ds) == want
    covered = set()
    for i in range(len(ds)):
        item = ds[i]
        x, y = item["input_ids"].tolist(), item["target_ids"].tolist()
        assert len(x) == len(y) == window and y == [t + 1 for t in x]        # next-token targets
        assert x == list(range(x[0], x[0] + window)) and x[-1] <= total - 2   # contiguous, across shard boundaries, inside the data
        assert x[0] == min(i * stride, total - 1 - window)
        covered.update(x)
    if want and stride <= window:
        assert covered == set(range(0, max(covered) + 1)) and max(covered) >= total - 1 - stride  # no holes; the tail is short of a stride


# ------------------------------------------------------------------------------------------------------ chat masking
@settings(max_examples=40, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.too_slow, HealthCheck.function_scoped_fixture])
@given(st.lists(st.tuples(st.sampled_from(["system", "user", "assistant", "tool"]), st.sampled_from(["hello world", "the quick brown fox", "a", "é ß", "x " * 9])),
                min_size=1, max_size=7),
       st.sampled_from(["mask", "train"]), st.integers(4, 80))
def test_chat_records_train_exactly_the_roles_the_config_names(tokenizer, turns, default, limit):
    from astrai_b200.config import PipelineConfig
    from astrai_b200.preprocessing import MaskBuilderFactory

    cfg = PipelineConfig.from_dict({"input": {"sections": [{"field": "messages", "action": "$role", "template": True}]},
                                    "mask": {"user": "mask", "assistant": "train"}, "mask_default": default,
                                    "preprocessing": {"max_seq_len": limit}})
    messages = [{"role": r, "content": c} for r, c in turns]
    builder = MaskBuilderFactory.create("single")
    rec = builder.build({"messages": messages}, cfg, tokenizer)
    pieces = [tokenizer.encode(tokenizer.apply_chat_template([m], tokenize=False, add_generation_prompt=False), add_special_tokens=False)
              for m in messages]
    ids = [tokenizer.bos_token_id] + [t for p in pieces for t in p]
    trains = {"user": 0, "assistant": 1}
    mask = [0] + [trains.get(m["role"], int(default == "train")) for m, p in zip(messages, pieces) for _ in p]
    assert rec is not None and rec["sequence"] == ids[:limit]
    if "loss_mask" in rec:
        assert rec["loss_mask"] == mask[:limit]
    else:  # every token trains: the mask is left out
        assert all(mask[:limit])
    assert builder.build_batch([{"messages": messages}, {"messages": messages[:1]}], cfg, tokenizer)[0] == rec


# --------------------------------------------------------------------------------------- padding never changes a loss
def _frozen_copy(model):
    import copy

    return copy.deepcopy(model).requires_grad_(False).eval()


@settings(max_examples=15, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.too_slow, HealthCheck.function_scoped_fixture])
@given(st.integers(1, 3), st.integers(5, 12), st.integers(0, 5), st.integers(0, 4), st.integers(0, 30))
def test_preference_loss_does_not_depend_on_the_amount_of_padding(tiny_lm, pairs, length, extra_right, shorter, seed):
    from astrai_b200.data import dpo_collate_fn
    from astrai_b200.trainer import StrategyFactory

    g = torch.Generator().manual_seed(seed)
    items = []
    for i in range(pairs):
        n_c, n_r = length - (i * shorter) % 4, length - ((i + 1) * shorter) % 3
        chosen, rejected = torch.randint(2, 250, (n_c,), generator=g), torch.randint(2, 250, (n_r,), generator=g)
        rejected[:3] = chosen[:3]
        cm, rm = torch.ones(n_c, dtype=torch.bool), torch.ones(n_r, dtype=torch.bool)
        cm[:3], rm[:3] = False, False
        items.append({"chosen": chosen, "rejected": rejected, "chosen_mask": cm, "rejected_mask": rm})
    batch = dpo_collate_fn(items)
    wide = {k: torch.nn.functional.pad(v, (0, extra_right)) for k, v in batch.items()}
    policy = _frozen_copy(tiny_lm).train()
    with torch.no_grad():  # move the policy away from the reference so that the margin is not identically zero
        for p in policy.parameters():
            p.add_(0.05 * torch.randn(p.shape, generator=g))
    s = StrategyFactory.create("dpo", model=policy, device="cpu", ref_model=_frozen_copy(tiny_lm), beta=0.3)
    a, b = float(s(batch)["loss"]), float(s(wide)["loss"])
    assert a == pytest.approx(b, abs=2e-5) and abs(a - 0.6931) > 1e-6
    # one pair at a time: the batch loss is the mean of the pairs' losses
    singles = [float(s(dpo_collate_fn([it]))["loss"]) for it in items]
    assert a == pytest.approx(sum(singles) / len(singles), abs=2e-5)


@settings(max_examples=12, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.too_slow, HealthCheck.function_scoped_fixture])
@given(st.integers(1, 2), st.integers(2, 3), st.integers(3, 7), st.integers(3, 7), st.integers(0, 4), st.integers(0, 3), st.integers(0, 30))
def test_group_loss_does_not_depend_on_the_amount_of_padding(tiny_lm, prompts, group, plen, rlen, extra_left, extra_right, seed):
    from astrai_b200.data import grpo_collate_fn
    from astrai_b200.trainer import StrategyFactory

    g = torch.Generator().manual_seed(seed)
    items = []
    for i in range(prompts):
        p = torch.randint(2, 250, (plen - i % 2,), generator=g)
        resp = [torch.randint(2, 250, (rlen - (i + j) % 3,), generator=g) for j in range(group)]
        items.append({"prompts": p, "responses": resp, "masks": [torch.ones_like(r, dtype=torch.bool) for r in resp],
                      "rewards": torch.rand(group, generator=g)})
    batch = grpo_collate_fn(items)
    wide = dict(batch)
    wide["prompts"] = torch.nn.functional.pad(batch["prompts"], (extra_left, 0))
    wide["prompt_mask"] = torch.nn.functional.pad(batch["prompt_mask"], (extra_left, 0))
    wide["responses"] = torch.nn.functional.pad(batch["responses"], (0, extra_right))
    wide["masks"] = torch.nn.functional.pad(batch["masks"], (0, extra_right))
    policy = _frozen_copy(tiny_lm).train()
    with torch.no_grad():
        for p in policy.parameters():
            p.add_(0.05 * torch.randn(p.shape, generator=g))

    class Exec:
        use_distributed = False

        def unwrap_model(self, m):
            return m.state_dict()

    s = StrategyFactory.create("grpo", model=policy, device="cpu", old_model=_frozen_copy(tiny_lm), ref_model=_frozen_copy(tiny_lm),
                               group_size=group, clip_eps=0.2, kl_coef=0.05, executor=Exec())
    a, b = s(batch), s(wide)
    assert float(a["loss"]) == pytest.approx(float(b["loss"]), abs=2e-5)
    assert float(a["metrics"]["kl_loss"]) == pytest.approx(float(b["metrics"]["kl_loss"]), abs=2e-5) and float(a["metrics"]["kl_loss"]) > 0


# ------------------------------------------------------------------------------------ packing never leaks across documents
@settings(max_examples=15, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.too_slow, HealthCheck.function_scoped_fixture])
@given(st.lists(st.lists(st.integers(2, 9), min_size=1, max_size=4), min_size=1, max_size=3), st.integers(0, 30))
def test_packed_supervised_loss_is_the_token_weighted_mean_of_the_documents_alone(tiny_lm, rows, seed):
    """Rows of packed documents (positions restart, attention stays inside a document): the batch loss must be what the
    documents give one by one - the sum of their trained tokens' losses over the number of trained tokens."""
    from astrai_b200.trainer import StrategyFactory

    g = torch.Generator().manual_seed(seed)
    width = max(sum(r) for r in rows)
    model = _frozen_copy(tiny_lm)
    strategy = StrategyFactory.create("sft", model=model, device="cpu")
    ids = torch.zeros(len(rows), width + 1, dtype=torch.long)
    pos = torch.zeros(len(rows), width, dtype=torch.long)
    keep = torch.zeros(len(rows), width, dtype=torch.bool)
    total, count = 0.0, 0
    for r, lens in enumerate(rows):
        lens = list(lens) + ([width - sum(lens)] if sum(lens) < width else [])  # the rest of the row is one more document
        start = 0
        for n in lens:
            doc = torch.randint(2, 250, (n + 1,), generator=g)
            trained = torch.rand(n, generator=g) < 0.6
            ids[r, start:start + n + 1] = doc  # the next document overwrites the last token: it is only ever a target
            pos[r, start:start + n] = torch.arange(n)
            keep[r, start:start + n] = trained
            start += n
        # the documents alone, with the tokens as they ended up in the row
        start = 0
        for n in lens:
            x, y = ids[r, start:start + n][None], ids[r, start + 1:start + n + 1][None]
            k = keep[r, start:start + n][None]
            if k.any():
                logits = model(x)["logits"].float()
                rows_loss = torch.nn.functional.cross_entropy(logits[0], y[0], reduction="none")
                total += float((rows_loss * k[0]).sum())
                count += int(k.sum())
            start += n
    if count == 0:
        return
    batch = {"input_ids": ids[:, :-1], "target_ids": ids[:, 1:], "position_ids": pos, "loss_mask": keep}
    with torch.no_grad():
        loss = float(strategy(batch)["loss"])
    assert loss == pytest.approx(total / count, abs=3e-5)
