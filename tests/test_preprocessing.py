"""Mask builders, packing, position ids and the preprocessing pipeline in depth (behaviours the reference checks in
``tests/data/test_preprocess_builder.py`` and ``tests/data/test_preprocess_pipeline.py``, restated for this package)."""

import json

import pytest
import torch

from helpers import build_tokenizer_dir


@pytest.fixture(scope="module")
def tok_dir(tmp_path_factory):
    return build_tokenizer_dir(str(tmp_path_factory.mktemp("tok")))


@pytest.fixture(scope="module")
def tok(tok_dir):
    from astrai_b200.tokenize import AutoTokenizer

    return AutoTokenizer.from_pretrained(tok_dir)


def _cfg(**d):
    from astrai_b200.config import PipelineConfig

    return PipelineConfig.from_dict(d)


CHAT = {"input": {"sections": [{"field": "messages", "action": "$role", "template": True}]},
        "mask": {"system": "mask", "user": "mask", "assistant": "train"}}
CONV = [{"role": "system", "content": "be kind"}, {"role": "user", "content": "hello there"},
        {"role": "assistant", "content": "general greeting"}, {"role": "user", "content": "again"},
        {"role": "assistant", "content": "once more"}]


# ------------------------------------------------------------------------------------------------------------ chat
def test_chat_trains_exactly_the_assistant_turns(tok):
    from astrai_b200.preprocessing import MaskBuilderFactory

    rec = MaskBuilderFactory.create("single").build({"messages": CONV}, _cfg(**CHAT), tok)
    ids, mask = rec["sequence"], rec["loss_mask"]
    assert ids[0] == tok.bos_token_id and mask[0] == 0 and len(ids) == len(mask)
    pieces = [tok.encode(tok.apply_chat_template([m], tokenize=False, add_generation_prompt=False), add_special_tokens=False) for m in CONV]
    assert ids[1:] == [t for p in pieces for t in p]  # message by message through the chat template, nothing in between
    expect = [0] + [int(m["role"] == "assistant") for m, p in zip(CONV, pieces) for _ in p]
    assert mask == expect


def test_chat_uniform_masks_and_default_role_action(tok):
    from astrai_b200.preprocessing import MaskBuilderFactory

    b = MaskBuilderFactory.create("single")
    everything = b.build({"messages": CONV}, _cfg(**{**CHAT, "mask": {"system": "train", "user": "train", "assistant": "train"}}), tok)
    assert everything["loss_mask"][0] == 0 and all(everything["loss_mask"][1:])  # the BOS token never trains
    nothing = b.build({"messages": CONV}, _cfg(**{**CHAT, "mask": {}}), tok)  # unknown roles take mask_default = "mask"
    assert not any(nothing["loss_mask"])
    flipped = b.build({"messages": CONV}, _cfg(**{**CHAT, "mask": {}, "mask_default": "train"}), tok)
    assert all(flipped["loss_mask"][1:])


def test_chat_empty_missing_and_truncated(tok):
    from astrai_b200.preprocessing import MaskBuilderFactory

    b = MaskBuilderFactory.create("single")
    cfg = _cfg(**CHAT)
    assert b.build({"messages": []}, cfg, tok) is None and b.build({}, cfg, tok) is None and b.build({"messages": "text"}, cfg, tok) is None
    short = _cfg(**{**CHAT, "preprocessing": {"max_seq_len": 10}})
    rec = b.build({"messages": CONV}, short, tok)
    full = b.build({"messages": CONV}, cfg, tok)
    assert len(rec["sequence"]) == 10 == len(rec["loss_mask"]) and rec["sequence"] == full["sequence"][:10]


def test_batch_equals_one_by_one(tok):
    from astrai_b200.preprocessing import MaskBuilderFactory

    b = MaskBuilderFactory.create("sectioned")
    cfg = _cfg(**CHAT)
    items = [{"messages": CONV[:3]}, {"messages": []}, {"messages": CONV}, {"messages": CONV[1:2]}]
    assert b.build_batch(items, cfg, tok) == [b.build(it, cfg, tok) for it in items]


def test_domain_comes_from_the_configured_key(tok):
    from astrai_b200.preprocessing import MaskBuilderFactory

    b = MaskBuilderFactory.create("single")
    cfg = _cfg(**{**CHAT, "output": {"domain_key": "source"}})
    assert b.build({"messages": CONV, "source": "wiki"}, cfg, tok)["domain"] == "wiki"
    assert b.build({"messages": CONV}, cfg, tok)["domain"] == "__default__"
    assert b.build({"messages": CONV, "source": 7}, cfg, tok)["domain"] == "__default__"  # only strings name a domain
    assert b.build({"messages": CONV, "source": "wiki"}, _cfg(**CHAT), tok)["domain"] == "__default__"


# ----------------------------------------------------------------------------------------------------- instruction
INSTR = {"input": {"sections": [{"field": "instruction", "action": "mask"}, {"field": "output", "action": "train"}]},
         "preprocessing": {"min_chars": 0}}


def test_instruction_masks_the_prompt_and_trains_the_answer(tok):
    from astrai_b200.preprocessing import MaskBuilderFactory

    rec = MaskBuilderFactory.create("single").build({"instruction": "add 2 and 2", "output": "four"}, _cfg(**INSTR), tok)
    n_prompt = len(tok.encode("add 2 and 2", add_special_tokens=True))
    n_out = len(tok.encode("four", add_special_tokens=False))
    assert rec["loss_mask"] == [0] * n_prompt + [1] * n_out
    both = {"input": {"sections": [{"field": "instruction", "action": "train"}, {"field": "output", "action": "train"}]},
            "preprocessing": {"min_chars": 0}}
    rec = MaskBuilderFactory.create("single").build({"instruction": "add 2 and 2", "output": "four"}, _cfg(**both), tok)
    assert "loss_mask" not in rec and len(rec["sequence"]) == n_prompt + n_out  # every token trains: no mask column


def test_instruction_skips_blank_fields(tok):
    from astrai_b200.preprocessing import MaskBuilderFactory

    b = MaskBuilderFactory.create("single")
    only_out = b.build({"instruction": "   ", "output": "four"}, _cfg(**INSTR), tok)
    assert only_out["sequence"] == tok.encode("four", add_special_tokens=True)  # first rendered section carries the specials
    assert b.build({"instruction": "", "output": ""}, _cfg(**INSTR), tok) is None


# ------------------------------------------------------------------------------------------------------------ text
def test_text_filters_by_character_count_and_truncates(tok):
    from astrai_b200.preprocessing import MaskBuilderFactory

    b = MaskBuilderFactory.create("single")
    cfg = _cfg(input={"sections": [{"field": "text", "action": "train"}]}, preprocessing={"min_chars": 10, "max_chars": 40, "max_seq_len": 6})
    assert b.build({"text": "too short"}, cfg, tok) is None
    assert b.build({"text": "x" * 41}, cfg, tok) is None
    assert b.build({"text": ""}, cfg, tok) is None and b.build({}, cfg, tok) is None
    rec = b.build({"text": "just long enough to pass"}, cfg, tok)
    assert rec["sequence"] == tok.encode("just long enough to pass")[:6] and "loss_mask" not in rec
    # the character filters are for plain-text corpora only: a masked section is never filtered by length
    masked = _cfg(input={"sections": [{"field": "text", "action": "mask"}, {"field": "more", "action": "train"}]}, preprocessing={"min_chars": 10})
    assert b.build({"text": "tiny", "more": "x"}, masked, tok) is not None


def test_filter_by_length_helper():
    from astrai_b200.preprocessing.pipeline import filter_by_length

    assert filter_by_length("a" * 50) and not filter_by_length("a" * 49)
    assert filter_by_length("abc", min_len=1, max_len=3) and not filter_by_length("abcd", min_len=1, max_len=3)


# ------------------------------------------------------------------------------------------------------- dpo / grpo
DPO = {"input": {"sources": {
    "chosen": {"sections": [{"field": "messages", "action": "mask", "template": True}, {"field": "chosen", "action": "train"}]},
    "rejected": {"sections": [{"field": "messages", "action": "mask", "template": True}, {"field": "rejected", "action": "train"}]}}},
    "preprocessing": {"min_chars": 0}}


def test_dpo_pairs_share_a_masked_prompt(tok):
    from astrai_b200.preprocessing import MaskBuilderFactory

    b = MaskBuilderFactory.create("multi")
    rec = b.build({"messages": CONV[:2], "chosen": "a fine answer", "rejected": "no"}, _cfg(**DPO), tok)
    n_prompt = rec["chosen_mask"].index(1)
    assert n_prompt == rec["rejected_mask"].index(1) and rec["chosen"][:n_prompt] == rec["rejected"][:n_prompt]
    assert rec["chosen"][0] == tok.bos_token_id
    assert all(rec["chosen_mask"][n_prompt:]) and all(rec["rejected_mask"][n_prompt:])
    assert rec["chosen"][n_prompt:] == tok.encode("a fine answer", add_special_tokens=False)


@pytest.mark.parametrize("missing", ["chosen", "rejected"])
def test_dpo_incomplete_records_are_dropped(tok, missing):
    from astrai_b200.preprocessing import MaskBuilderFactory

    item = {"chosen": "yes", "rejected": "no"}
    item.pop(missing)
    plain = {"input": {"sources": {"chosen": {"sections": [{"field": "chosen", "action": "train"}]},
                                   "rejected": {"sections": [{"field": "rejected", "action": "train"}]}}},
             "preprocessing": {"min_chars": 0}}
    assert MaskBuilderFactory.create("multi").build(item, _cfg(**plain), tok) is None


GRPO = {"input": {"sources": {
    "prompts": {"sections": [{"field": "prompt", "action": "mask"}]},
    "responses": {"sections": [{"field": "responses", "action": "train"}], "list_field": True, "mask_key": "masks"},
    "rewards": {"sections": [{"field": "rewards", "action": "value"}]}}},
    "preprocessing": {"min_chars": 0}}


def test_grpo_keeps_one_list_per_response(tok):
    from astrai_b200.preprocessing import MaskBuilderFactory

    b = MaskBuilderFactory.create("sectioned")
    item = {"prompt": "solve", "responses": ["first try", "second", "the third attempt"], "rewards": [0.1, 1, -2]}
    rec = b.build(item, _cfg(**GRPO), tok)
    assert [tok.decode(r) for r in rec["responses"]] == item["responses"]  # boundaries and order preserved, no specials
    assert [len(m) for m in rec["masks"]] == [len(r) for r in rec["responses"]] and all(all(m) for m in rec["masks"])
    assert rec["rewards"] == [0.1, 1.0, -2.0] and not any(rec.get("prompts_mask", [0]))
    single = b.build({"prompt": "p", "responses": ["only"], "rewards": 0.5}, _cfg(**GRPO), tok)
    assert single["rewards"] == [0.5] and len(single["responses"]) == 1
    assert b.build({"prompt": "p", "responses": "not a list", "rewards": [1]}, _cfg(**GRPO), tok) is None
    assert b.build({"prompt": "p", "responses": ["x"]}, _cfg(**GRPO), tok) is None  # rewards missing
    items = [item, {"prompt": "q", "responses": ["z"], "rewards": [3]}]
    assert b.build_batch(items, _cfg(**GRPO), tok) == [b.build(it, _cfg(**GRPO), tok) for it in items]


def test_builders_refuse_the_other_kind_of_config(tok):
    from astrai_b200.preprocessing import MaskBuilderFactory

    assert MaskBuilderFactory.create("single").build({"prompt": "p"}, _cfg(**GRPO), tok) is None
    assert MaskBuilderFactory.create("multi").build({"messages": CONV}, _cfg(**CHAT), tok) is None
    for name in ("single", "multi", "sectioned"):
        assert MaskBuilderFactory.create(name) is not None
    with pytest.raises((KeyError, ValueError)):
        MaskBuilderFactory.create("nope")


# ---------------------------------------------------------------------------------------------------------- packing
def test_bfd_never_overfills_and_keeps_every_document():
    from astrai_b200.preprocessing import plan_bfd

    g = torch.Generator().manual_seed(0)
    seqs = [[i] * int(n) for i, n in enumerate(torch.randint(1, 40, (200,), generator=g))]
    bins = plan_bfd(seqs, 64)
    assert sorted(i for b in bins for i in b) == list(range(200))
    fill = [sum(len(seqs[i]) for i in b) for b in bins]
    assert max(fill) <= 64
    assert len(bins) <= -(-sum(len(s) for s in seqs) // 64) * 1.2  # close to the lower bound on the number of bins


def test_bfd_truncates_oversized_documents_by_mode():
    from astrai_b200.preprocessing import PackingStrategyFactory

    cols = {"sequence": [list(range(10))], "loss_mask": [[1] * 10]}
    start = PackingStrategyFactory.create("bfd").apply(cols, 4, "keep_start")
    end = PackingStrategyFactory.create("bfd").apply(cols, 4, "keep_end")
    assert start["sequence"] == [[0, 1, 2, 3]] and end["sequence"] == [[6, 7, 8, 9]]


def test_bfd_split_keeps_all_tokens_in_aligned_chunks():
    from astrai_b200.preprocessing import PackingStrategyFactory

    seqs = [list(range(100, 123)), [1, 2, 3], list(range(200, 216)), [9]]
    cols = {"sequence": seqs, "position_ids": [list(range(len(s))) for s in seqs]}
    out = PackingStrategyFactory.create("bfd_split").apply(cols, 8, "keep_start")
    flat = [t for s in out["sequence"] for t in s]
    assert sorted(flat) == sorted(t for s in seqs for t in s)  # a long document is cut into pieces, never truncated
    assert all(len(s) <= 8 for s in out["sequence"])
    assert [len(s) for s in out["sequence"]] == [len(s) for s in out["position_ids"]]
    plain = PackingStrategyFactory.create("bfd").apply(cols, 8, "keep_start")
    assert sum(len(s) for s in plain["sequence"]) < len(flat)  # plain BFD drops what does not fit
    short = {"sequence": [[1, 2], [3]]}
    assert sorted(map(tuple, PackingStrategyFactory.create("bfd_split").apply(short, 8, "keep_start")["sequence"])) in ([(1, 2, 3)], [(3, 1, 2)], [(1, 2), (3,)])


def test_position_id_strategies():
    from astrai_b200.preprocessing.position_id import PositionIdStrategyFactory

    docs = [[5, 5, 5], [6], [7, 7]]
    assert PositionIdStrategyFactory.create("doc_reset").generate(docs) == [0, 1, 2, 0, 0, 1]
    assert PositionIdStrategyFactory.create("continuous").generate(docs) == [0, 1, 2, 3, 4, 5]
    assert PositionIdStrategyFactory.create("none").generate(docs) == []


# --------------------------------------------------------------------------------------------------------- pipeline
def _jsonl(path, records):
    with open(path, "w") as fh:
        for r in records:
            fh.write(json.dumps(r) + "\n")


def test_text_pipeline_counts_filters_and_max_items(tok_dir, tmp_path):
    from astrai_b200.data import DatasetFactory
    from astrai_b200.preprocessing import Pipeline

    recs = [{"text": f"document number {i} " * 4} for i in range(30)] + [{"text": "tiny"}] * 5
    _jsonl(tmp_path / "in.jsonl", recs)
    cfg = _cfg(input={"sections": [{"field": "text", "action": "train"}]}, preprocessing={"min_chars": 20, "batch_size": 8},
               output={"position_ids_mode": "none"})
    assert Pipeline(cfg, [str(tmp_path / "in.jsonl")], str(tmp_path / "all"), tok_dir).run() == 30
    shard = tmp_path / "all" / "__default__" / "shard_0000"
    assert (shard / "sequence.bin").exists() and not (shard / "loss_mask.bin").exists() and not (shard / "position_ids.bin").exists()
    ds = DatasetFactory.load("seq", str(tmp_path / "all"), window_size=16)
    assert len(ds) > 0 and ds[0]["input_ids"].dtype == torch.long
    capped = _cfg(input={"sections": [{"field": "text", "action": "train"}]}, preprocessing={"min_chars": 20, "max_items": 7, "batch_size": 4})
    assert Pipeline(capped, [str(tmp_path / "in.jsonl")], str(tmp_path / "cap"), tok_dir).run() == 7


def test_pipeline_shards_by_domain_and_token_budget(tok_dir, tmp_path):
    from astrai_b200.preprocessing import Pipeline

    recs = [{"text": "alpha beta gamma delta " * 3, "src": "a" if i % 3 else "b"} for i in range(24)]
    _jsonl(tmp_path / "in.jsonl", recs)
    cfg = _cfg(input={"sections": [{"field": "text", "action": "train"}]}, preprocessing={"min_chars": 0, "batch_size": 5},
               output={"domain_key": "src", "max_tokens_per_shard": 150})
    assert Pipeline(cfg, [str(tmp_path / "in.jsonl")], str(tmp_path / "out"), tok_dir).run() == 24
    a = sorted(p.name for p in (tmp_path / "out" / "a").iterdir())
    b = sorted(p.name for p in (tmp_path / "out" / "b").iterdir())
    assert a[0] == "shard_0000" and len(a) > 1 and b[0] == "shard_0000"  # several shards once the token budget is reached
    meta = json.load(open(tmp_path / "out" / "a" / "shard_0000" / "meta.json"))
    assert meta["sequence"]["dtype"] == "int32"


def test_pipeline_dtype_override(tok_dir, tmp_path):
    from astrai_b200.preprocessing import Pipeline

    _jsonl(tmp_path / "in.jsonl", [{"messages": CONV}] * 6)
    cfg = _cfg(**{**CHAT, "output": {"dtype": {"sequence": "int64", "loss_mask": "uint8"}}})
    Pipeline(cfg, [str(tmp_path / "in.jsonl")], str(tmp_path / "out"), tok_dir).run()
    meta = json.load(open(tmp_path / "out" / "__default__" / "shard_0000" / "meta.json"))
    assert meta["sequence"]["dtype"] == "int64" and meta["loss_mask"]["dtype"] == "uint8" and meta["position_ids"]["dtype"] == "int32"


def test_dpo_pipeline_writes_record_offsets(tok_dir, tmp_path):
    from astrai_b200.data import DatasetFactory
    from astrai_b200.preprocessing import Pipeline

    recs = [{"messages": CONV[:2], "chosen": "good " * (i + 1), "rejected": "bad"} for i in range(9)]
    _jsonl(tmp_path / "in.jsonl", recs)
    Pipeline(_cfg(**{**DPO, "output": {"position_ids_mode": "none"}}), [str(tmp_path / "in.jsonl")], str(tmp_path / "out"), tok_dir).run()
    ds = DatasetFactory.load("dpo", str(tmp_path / "out"))
    assert len(ds) == 9
    lens = [ds[i]["chosen"].numel() for i in range(9)]
    assert lens == sorted(lens) and lens[0] < lens[-1]  # records come back one by one, in input order
    assert ds[3]["chosen_mask"].dtype == torch.bool and ds[3]["chosen_mask"].numel() == ds[3]["chosen"].numel()


def test_grpo_pipeline_roundtrip_through_jsonl_storage(tok_dir, tmp_path):
    from astrai_b200.data import DatasetFactory, grpo_collate_fn
    from astrai_b200.preprocessing import Pipeline

    recs = [{"prompt": f"task {i}", "responses": ["a" * (i + 1), "bb", "ccc"], "rewards": [1.0, 0.0, 0.5]} for i in range(5)]
    _jsonl(tmp_path / "in.jsonl", recs)
    cfg = _cfg(**{**GRPO, "output": {"storage_format": "jsonl", "position_ids_mode": "none"}})
    assert Pipeline(cfg, [str(tmp_path / "in.jsonl")], str(tmp_path / "out"), tok_dir).run() == 5
    ds = DatasetFactory.load("grpo", str(tmp_path / "out"))
    assert len(ds) == 5
    item = ds[2]
    assert len(item["responses"]) == 3 and item["rewards"].tolist() == [1.0, 0.0, 0.5] and item["prompts"].dtype == torch.long
    batch = grpo_collate_fn([ds[0], ds[4]])
    assert batch["responses"].shape[:2] == (2, 3) and batch["rewards"].shape == (2, 3)


def test_pipeline_survives_malformed_records(tok_dir, tmp_path):
    from astrai_b200.preprocessing import Pipeline

    with open(tmp_path / "in.jsonl", "w") as fh:
        fh.write(json.dumps({"messages": CONV}) + "\n")
        fh.write("{broken json\n")
        fh.write(json.dumps({"messages": "not a list"}) + "\n")
        fh.write(json.dumps({"unrelated": 1}) + "\n")
        fh.write(json.dumps({"messages": CONV[:3]}) + "\n")
    assert Pipeline(_cfg(**CHAT), [str(tmp_path / "in.jsonl")], str(tmp_path / "out"), tok_dir).run() == 2
