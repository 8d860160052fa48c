"""Stores, datasets, collate functions, tokenizer, preprocessing pipeline."""

import json
import os

import pytest
import torch

from helpers import build_tokenizer_dir


@pytest.fixture(scope="module")
def tok_dir(tmp_path_factory):
    return build_tokenizer_dir(str(tmp_path_factory.mktemp("tok")))


def test_bin_roundtrip_and_stream_windows(tmp_path):
    from astrai_b200.data import DatasetFactory, MmapStore
    from astrai_b200.serialization import load_bin, save_bin

    a, b = torch.arange(0, 50, dtype=torch.int32), torch.arange(50, 103, dtype=torch.int32)
    save_bin(str(tmp_path / "d" / "shard_0000"), {"sequence": [a]})
    save_bin(str(tmp_path / "d" / "shard_0001"), {"sequence": [b]})
    assert torch.equal(load_bin(str(tmp_path / "d" / "shard_0000"))["sequence"][0], a)
    store = MmapStore(window_size=16, stride=16)
    store.load(str(tmp_path))
    total, w = 103, 16
    assert store.token_count == total and len(store) == (total - 1 - w) // 16 + 1
    ds = DatasetFactory.load("seq", str(tmp_path), window_size=16)
    s = ds[3]
    assert torch.equal(s["input_ids"], torch.arange(48, 64)) and torch.equal(s["target_ids"], torch.arange(49, 65))
    last = ds[len(ds) - 1]
    assert last["target_ids"][-1].item() <= 102
    with pytest.raises(IndexError):
        store.sample_window(len(store))
    short = MmapStore(window_size=200)
    short.load(str(tmp_path))
    assert len(short) == 0


def test_record_offsets_and_dpo_dataset(tmp_path):
    from astrai_b200.data import DatasetFactory, dpo_collate_fn
    from astrai_b200.serialization import save_bin

    chosen = [torch.tensor([1, 2, 3]), torch.tensor([4, 5])]
    rejected = [torch.tensor([1, 9]), torch.tensor([4, 8, 7, 6])]
    cm = [torch.tensor([0, 1, 1]), torch.tensor([0, 1])]
    rm = [torch.tensor([0, 1]), torch.tensor([0, 1, 1, 1])]
    save_bin(str(tmp_path / "s"), {"chosen": chosen, "rejected": rejected, "chosen_mask": cm, "rejected_mask": rm},
             record_keys=["chosen", "rejected", "chosen_mask", "rejected_mask"])
    ds = DatasetFactory.load("dpo", str(tmp_path))
    assert len(ds) == 2 and torch.equal(ds[1]["rejected"], torch.tensor([4, 8, 7, 6]))
    batch = dpo_collate_fn([ds[0], ds[1]])
    assert batch["chosen"].shape == (2, 4) and batch["chosen"][1].tolist() == [4, 5, 0, 0]
    assert batch["rejected_mask"][1].tolist() == [False, True, True, True]


def test_grpo_collate_left_pads_prompts():
    from astrai_b200.data import grpo_collate_fn

    rec = lambda p, rs: {"prompts": torch.tensor(p), "responses": [torch.tensor(r) for r in rs],  # noqa: E731
                         "masks": [torch.ones(len(r), dtype=torch.bool) for r in rs], "rewards": torch.tensor([1.0, 0.0])}
    out = grpo_collate_fn([rec([5, 6, 7], [[1], [2, 3]]), rec([8], [[4, 4, 4], [9]])])
    assert out["prompts"].tolist() == [[5, 6, 7], [0, 0, 8]]
    assert out["prompt_mask"].tolist() == [[True, True, True], [False, False, True]]
    assert out["responses"].shape == (2, 2, 3) and out["masks"][0, 0].tolist() == [True, False, False]


def test_tokenizer_special_tokens_and_chat_template(tok_dir, tmp_path):
    from astrai_b200.tokenize import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(tok_dir)
    assert tok.bos_token == "<|bos|>" and isinstance(tok.bos_token_id, int) and tok.missing_token_id is None
    assert set(tok.stop_ids) == {tok.bos_token_id, tok.eos_token_id, tok.pad_token_id, tok.im_start_id}
    ids = tok.encode("hello world")
    assert tok.decode(ids) == "hello world"
    assert tok.encode(["hello", "world"]) == [tok.encode("hello"), tok.encode("world")]
    text = tok.apply_chat_template([{"role": "user", "content": "hi"}], tokenize=False)
    assert text.endswith("<|im_start|>assistant\n") and "<|im_start|>user\nhi<|im_end|>" in text
    batch = tok.apply_chat_template([[{"role": "user", "content": "a"}], [{"role": "user", "content": "b"}]], tokenize=True)
    assert len(batch) == 2 and all(isinstance(x, list) for x in batch)
    tok.save_pretrained(tmp_path / "copy")
    again = AutoTokenizer.from_pretrained(tmp_path / "copy")
    assert again.encode("hello world") == ids and again.eos_token == tok.eos_token
    import pickle

    assert pickle.loads(pickle.dumps(tok)).encode("hello") == tok.encode("hello")
    with pytest.raises(FileNotFoundError):
        AutoTokenizer.from_pretrained(tmp_path / "nowhere")


def test_plan_bfd_and_packers():
    from astrai_b200.preprocessing import PackingStrategyFactory, plan_bfd

    seqs = [[1] * 5, [2] * 3, [3] * 4, [4] * 2, [5] * 9]
    bins = plan_bfd(seqs, 8)
    assert sorted(i for b in bins for i in b) == [0, 1, 2, 3, 4]
    assert all(sum(min(len(seqs[i]), 8) for i in b) <= 8 for b in bins)
    cols = {"sequence": seqs, "loss_mask": [[0] * len(s) for s in seqs]}
    simple = PackingStrategyFactory.create("simple").apply(cols, 8, "keep_end")
    assert simple["sequence"][4] == [5] * 8
    packed = PackingStrategyFactory.create("bfd").apply(cols, 8, "keep_start")
    assert all(len(s) <= 8 for s in packed["sequence"]) and [len(x) for x in packed["sequence"]] == [len(x) for x in packed["loss_mask"]]
    split = PackingStrategyFactory.create("bfd_split").apply(cols, 8, "keep_start")
    assert sum(len(s) for s in split["sequence"]) == sum(len(s) for s in seqs)  # nothing dropped


def test_mask_builder_single_and_multi(tok_dir):
    from astrai_b200.config import PipelineConfig
    from astrai_b200.preprocessing import SectionedMaskBuilder
    from astrai_b200.tokenize import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(tok_dir)
    cfg = PipelineConfig.from_dict({
        "input": {"sections": [{"field": "messages", "action": "$role", "template": True}]},
        "mask": {"user": "mask", "assistant": "train"}, "output": {"domain_key": "src"},
    })
    item = {"messages": [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"}], "src": "chat"}
    b = SectionedMaskBuilder()
    one = b.build(item, cfg, tok)
    assert one["domain"] == "chat" and one["sequence"][0] == tok.bos_token_id and one["loss_mask"][0] == 0
    assert 0 < sum(one["loss_mask"]) < len(one["loss_mask"])
    assert b.build_batch([item, {"messages": []}], cfg, tok) == [one, None]
    text_cfg = PipelineConfig.from_dict({"input": {"sections": [{"field": "text", "action": "train"}]}, "preprocessing": {"min_chars": 5}})
    assert b.build({"text": "abc"}, text_cfg, tok) is None
    full = b.build({"text": "hello world"}, text_cfg, tok)
    assert "loss_mask" not in full and full["sequence"] == tok.encode("hello world")
    dpo_cfg = PipelineConfig.from_dict({"input": {"sources": {
        "chosen": {"sections": [{"field": "prompt", "action": "mask"}, {"field": "chosen", "action": "train"}]},
        "rejected": {"sections": [{"field": "prompt", "action": "mask"}, {"field": "rejected", "action": "train"}]},
    }}, "preprocessing": {"min_chars": 0}})
    rec = b.build({"prompt": "q: ", "chosen": "good", "rejected": "bad"}, dpo_cfg, tok)
    assert {"chosen", "rejected", "chosen_mask", "rejected_mask"} <= set(rec)
    assert b.build({"chosen": "x"}, dpo_cfg, tok) is None  # nothing to build "rejected" from
    grpo_cfg = PipelineConfig.from_dict({"input": {"sources": {
        "prompts": {"sections": [{"field": "prompt", "action": "mask"}]},
        "responses": {"sections": [{"field": "responses", "action": "train"}], "list_field": True, "mask_key": "masks"},
        "rewards": {"sections": [{"field": "rewards", "action": "value"}]},
    }}, "preprocessing": {"min_chars": 0}})
    g = b.build({"prompt": "p", "responses": ["aa", "bbb"], "rewards": [1, 0.5]}, grpo_cfg, tok)
    assert len(g["responses"]) == 2 and g["rewards"] == [1.0, 0.5] and len(g["masks"]) == 2


def test_pipeline_writes_loadable_shards(tok_dir, tmp_path):
    from astrai_b200.config import PipelineConfig
    from astrai_b200.data import DatasetFactory
    from astrai_b200.preprocessing import Pipeline

    src = tmp_path / "in.jsonl"
    with open(src, "w") as fh:
        for i in range(40):
            fh.write(json.dumps({"messages": [{"role": "user", "content": f"question {i}"}, {"role": "assistant", "content": "answer " * (i % 5 + 1)}]}) + "\n")
    cfg = PipelineConfig.from_dict({
        "input": {"sections": [{"field": "messages", "action": "$role", "template": True}]},
        "mask": {"user": "mask", "assistant": "train"},
        "preprocessing": {"packing_strategy": "bfd", "max_packed_len": 64, "batch_size": 7},
        "output": {"position_ids_mode": "doc_reset"},
    })
    n = Pipeline(cfg, [str(src)], str(tmp_path / "out"), tok_dir).run()
    assert n == 40
    shard = tmp_path / "out" / "__default__" / "shard_0000"
    assert (shard / "sequence.bin").exists() and (shard / "loss_mask.bin").exists() and (shard / "position_ids.bin").exists()
    ds = DatasetFactory.load("sft", str(tmp_path / "out"), window_size=32)
    s = ds[0]
    assert s["input_ids"].shape == (32,) and s["loss_mask"].dtype == torch.bool and s["position_ids"][0].item() == 0


def test_jsonl_store_eager_and_lazy(tok_dir, tmp_path):
    from astrai_b200.data import DatasetFactory

    d = tmp_path / "chat"
    d.mkdir()
    with open(d / "a.jsonl", "w") as fh:
        for i in range(6):
            fh.write(json.dumps({"messages": [{"role": "user", "content": "hello there " * 3}, {"role": "assistant", "content": "general " * 4}]}) + "\n")
        fh.write("not json\n")
    ds = DatasetFactory.load("sft", str(d), window_size=16, tokenizer_path=tok_dir)
    assert len(ds) > 0 and ds[0]["input_ids"].shape == (16,)
    p = tmp_path / "pref"
    p.mkdir()
    with open(p / "p.jsonl", "w") as fh:
        fh.write(json.dumps({"prompt": "what?", "chosen": "this", "rejected": "that one"}) + "\n")
    dpo = DatasetFactory.load("dpo", str(p), tokenizer_path=tok_dir)
    rec = dpo[0]
    assert rec["chosen_mask"].sum() > 0 and rec["chosen_mask"][0].item() is False
