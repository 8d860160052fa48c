"""Stores, datasets and the resumable sampler in depth: window arithmetic, segment chaining, record access, error paths,
format detection, lazy / eager JSONL, collate functions (behaviours the reference checks in ``tests/data/test_dataset.py``
and ``tests/data/test_sampler.py``, restated for this package's API)."""

import json

import pytest
import torch

from helpers import build_tokenizer_dir


@pytest.fixture(scope="module")
def tok_dir(tmp_path_factory):
    return build_tokenizer_dir(str(tmp_path_factory.mktemp("tok")))


def _bin(tmp_path, name, **keys):
    from astrai_b200.serialization import save_bin

    save_bin(str(tmp_path / name), {k: v for k, v in keys.items()})
    return str(tmp_path)


# ------------------------------------------------------------------------------------------------------- windows
@pytest.mark.parametrize("total,window,stride", [(100, 16, 16), (100, 16, 4), (65, 64, 64), (1000, 128, 96), (33, 32, 7)])
def test_window_count_and_last_window_stays_inside(tmp_path, total, window, stride):
    from astrai_b200.data import MmapStore

    _bin(tmp_path, "s", sequence=[torch.arange(total, dtype=torch.int32)])
    store = MmapStore(window_size=window, stride=stride)
    store.load(str(tmp_path))
    n = len(store)
    assert n == (total - 1 - window) // stride + 1
    seen_last = 0
    for i in range(n):
        b, e = store.sample_window(i)
        assert e - b == window and e <= total - 1  # one token is always left for the shifted targets
        seen_last = max(seen_last, e)
    assert seen_last >= total - 1 - stride  # the tail is not dropped by more than a stride


def test_stride_defaults_to_the_window(tmp_path):
    from astrai_b200.data import MmapStore

    _bin(tmp_path, "s", sequence=[torch.arange(200, dtype=torch.int32)])
    a, b = MmapStore(window_size=32), MmapStore(window_size=32, stride=32)
    a.load(str(tmp_path))
    b.load(str(tmp_path))
    assert a.stride == 32 and len(a) == len(b)


def test_overlapping_windows_with_a_custom_stride(tmp_path):
    from astrai_b200.data import DatasetFactory

    _bin(tmp_path, "s", sequence=[torch.arange(100, dtype=torch.int32)])
    ds = DatasetFactory.load("seq", str(tmp_path), window_size=16, stride=4)
    assert ds[1]["input_ids"][0].item() == 4 and ds[2]["input_ids"][0].item() == 8
    assert torch.equal(ds[1]["target_ids"], ds[1]["input_ids"] + 1)


def test_data_shorter_than_the_window_gives_an_empty_dataset(tmp_path):
    from astrai_b200.data import DatasetFactory

    _bin(tmp_path, "s", sequence=[torch.arange(10, dtype=torch.int32)])
    ds = DatasetFactory.load("seq", str(tmp_path), window_size=32)
    assert len(ds) == 0 and ds.token_count == 10
    with pytest.raises(IndexError):
        ds.store.sample_window(0)


def test_windows_cross_shard_boundaries(tmp_path):
    from astrai_b200.data import MmapStore

    for i, (lo, hi) in enumerate([(0, 10), (10, 11), (11, 40), (40, 64)]):
        _bin(tmp_path, f"shard_{i:04d}", sequence=[torch.arange(lo, hi, dtype=torch.int32)])
    store = MmapStore(window_size=8, stride=8)
    store.load(str(tmp_path))
    assert store.token_count == 64
    for b, e in [(0, 8), (5, 13), (9, 12), (8, 41), (39, 64), (63, 64)]:
        assert store.fetch(b, e, "sequence").tolist() == list(range(b, e))


def test_multi_key_fetch_returns_aligned_slices(tmp_path):
    from astrai_b200.data import MmapStore

    seq = torch.arange(50, dtype=torch.int32)
    _bin(tmp_path, "s", sequence=[seq], loss_mask=[(seq % 2).to(torch.uint8)], position_ids=[seq % 7])
    store = MmapStore(window_size=8)
    store.load(str(tmp_path))
    got = store.fetch(10, 18, ["sequence", "loss_mask"])
    assert set(got) == {"sequence", "loss_mask"}
    assert got["loss_mask"].tolist() == [int(x) % 2 for x in got["sequence"].tolist()]
    assert set(store[0]) == {"sequence", "loss_mask", "position_ids"}
    assert store[-1]["sequence"].shape == (8,)


def test_token_count_is_the_shortest_key(tmp_path):
    from astrai_b200.data import MmapStore

    _bin(tmp_path, "s", sequence=[torch.arange(50, dtype=torch.int32)], loss_mask=[torch.ones(40, dtype=torch.uint8)])
    store = MmapStore(window_size=8)
    store.load(str(tmp_path))
    assert store.token_count == 40


# ----------------------------------------------------------------------------------------------------- error paths
def test_unloaded_store_is_empty_and_refuses_access():
    from astrai_b200.data import MmapStore

    store = MmapStore(window_size=8)
    assert len(store) == 0 and store.keys == []
    with pytest.raises(RuntimeError, match="not loaded"):
        store.fetch(0, 4, "sequence")
    with pytest.raises(IndexError):
        store.sample_window(0)
    with pytest.raises(RuntimeError, match="window_size"):
        MmapStore().sample_window(0)


def test_fetch_bounds_are_checked(tmp_path):
    from astrai_b200.data import MmapStore

    _bin(tmp_path, "s", sequence=[torch.arange(20, dtype=torch.int32)])
    store = MmapStore(window_size=4)
    store.load(str(tmp_path))
    assert store.fetch(3, 3, "sequence").numel() == 0
    for b, e in [(-1, 4), (0, 21), (20, 20), (25, 30)]:
        with pytest.raises(ValueError, match="out of bounds"):
            store.fetch(b, e, "sequence")
    with pytest.raises(IndexError):
        store[len(store)]
    with pytest.raises(ValueError, match="Record index"):
        store.fetch_record(0, "sequence")  # no offsets were written: no record mode


def test_format_detection(tmp_path):
    from astrai_b200.data.storage import detect_format

    with pytest.raises(FileNotFoundError):
        detect_format(str(tmp_path / "missing"))
    (tmp_path / "notes.txt").write_text("x")
    with pytest.raises(ValueError, match="Unsupported"):
        detect_format(str(tmp_path / "notes.txt"))
    with pytest.raises(FileNotFoundError):
        detect_format(str(tmp_path))  # a directory without data files
    one = tmp_path / "a.jsonl"
    one.write_text("{}\n")
    assert detect_format(str(one)) == "jsonl" and detect_format(str(tmp_path)) == "jsonl"
    _bin(tmp_path / "bins", "deep/shard_0000", sequence=[torch.arange(4, dtype=torch.int32)])
    assert detect_format(str(tmp_path / "bins")) == "bin"  # found below nested directories
    assert detect_format(str(tmp_path)) == "bin"  # shards win over loose jsonl files


def test_unknown_store_or_dataset_type():
    from astrai_b200.data import DatasetFactory, StoreFactory

    with pytest.raises((KeyError, ValueError)):
        StoreFactory.create("parquet")
    with pytest.raises((KeyError, ValueError)):
        DatasetFactory.load("seq", None)
    with pytest.raises(FileNotFoundError):
        StoreFactory.create("bin").load("/nonexistent/place")


def test_dataset_reports_missing_keys(tmp_path):
    from astrai_b200.data import DatasetFactory

    _bin(tmp_path, "s", sequence=[torch.arange(64, dtype=torch.int32)])
    with pytest.raises(KeyError, match="loss_mask"):
        DatasetFactory.load("sft", str(tmp_path), window_size=8)
    with pytest.raises(KeyError, match="chosen"):
        DatasetFactory.load("dpo", str(tmp_path))


def test_nested_keys_are_refused_by_the_bin_writer(tmp_path):
    from astrai_b200.serialization import save_bin

    with pytest.raises(ValueError, match="JSONL"):
        save_bin(str(tmp_path / "s"), {"responses": [[torch.tensor([1, 2])], [torch.tensor([3])]]})


# ------------------------------------------------------------------------------------------------------ record mode
def test_record_offsets_slice_single_records_back_out(tmp_path):
    from astrai_b200.data import MmapStore
    from astrai_b200.serialization import load_bin_offsets, save_bin

    recs = [torch.arange(n, dtype=torch.int32) + 100 * i for i, n in enumerate([3, 1, 7, 2])]
    save_bin(str(tmp_path / "s"), {"chosen": recs}, record_keys=["chosen"])
    assert load_bin_offsets(str(tmp_path / "s"))["chosen"] == [0, 3, 4, 11, 13]
    store = MmapStore()
    store.load(str(tmp_path))
    assert store.num_records == 4 and len(store) == 4
    for i, r in enumerate(recs):
        assert torch.equal(store.fetch_record(i, "chosen"), r)
    with pytest.raises(ValueError):
        store.fetch_record(4, "chosen")


def test_records_are_numbered_across_shards(tmp_path):
    from astrai_b200.data import MmapStore
    from astrai_b200.serialization import save_bin

    save_bin(str(tmp_path / "shard_0"), {"chosen": [torch.tensor([1, 2]), torch.tensor([3])]}, record_keys=["chosen"])
    save_bin(str(tmp_path / "shard_1"), {"chosen": [torch.tensor([4, 5, 6]), torch.tensor([7]), torch.tensor([8, 9])]}, record_keys=["chosen"])
    store = MmapStore()
    store.load(str(tmp_path))
    assert store.num_records == 5
    assert [store.fetch_record(i, "chosen").tolist() for i in range(5)] == [[1, 2], [3], [4, 5, 6], [7], [8, 9]]


def test_shards_without_offsets_disable_record_mode_with_a_warning(tmp_path, caplog):
    from astrai_b200.data import MmapStore
    from astrai_b200.serialization import save_bin

    save_bin(str(tmp_path / "shard_0"), {"chosen": [torch.tensor([1, 2]), torch.tensor([3])]}, record_keys=["chosen"])
    save_bin(str(tmp_path / "shard_1"), {"chosen": [torch.tensor([4, 5, 6])]})  # an old shard: no offsets
    store = MmapStore()
    with caplog.at_level("WARNING"):
        store.load(str(tmp_path))
    assert store.num_records == 0 and "record mode disabled" in caplog.text


def test_bin_dtypes_survive_the_roundtrip(tmp_path):
    from astrai_b200.serialization import load_bin, save_bin

    data = {"a": [torch.arange(5, dtype=torch.int32)], "b": [torch.tensor([1, 0, 1], dtype=torch.uint8)],
            "c": [torch.tensor([0.5, -1.25], dtype=torch.float32)], "d": [torch.arange(3, dtype=torch.int64)]}
    save_bin(str(tmp_path / "s"), data)
    back = load_bin(str(tmp_path / "s"))
    for k, v in data.items():
        assert back[k][0].dtype == v[0].dtype and torch.equal(back[k][0], v[0])
    meta = json.load(open(tmp_path / "s" / "meta.json"))
    assert meta["a"]["shape"] == [5] and meta["c"]["dtype"] == "float32"


# ------------------------------------------------------------------------------------------------------------ jsonl
def _write_jsonl(path, records, junk=False):
    with open(path, "w") as fh:
        for r in records:
            fh.write(json.dumps(r) + "\n")
        if junk:
            fh.write("{not json\n\n")


def test_jsonl_source_skips_bad_lines_and_reads_directories(tmp_path):
    from astrai_b200.data.storage import JsonlSource

    _write_jsonl(tmp_path / "b.jsonl", [{"i": 2}], junk=True)
    _write_jsonl(tmp_path / "a.jsonl", [{"i": 0}, {"i": 1}])
    assert [r["i"] for r in JsonlSource(str(tmp_path)).load()] == [0, 1, 2]  # files in name order
    assert [r["i"] for r in JsonlSource(str(tmp_path / "b.jsonl")).load()] == [2]


def test_jsonl_eager_needs_a_transform_and_lazy_refuses_streams(tmp_path, tok_dir):
    from astrai_b200.data import DatasetFactory, JsonlStore

    _write_jsonl(tmp_path / "p.jsonl", [{"prompt": "a?", "chosen": "yes", "rejected": "no no"}] * 3)
    with pytest.raises(ValueError, match="transform"):
        JsonlStore().load(str(tmp_path))
    with pytest.raises(FileNotFoundError, match="dataset_config"):
        DatasetFactory.load("sft", str(tmp_path), window_size=8)
    ds = DatasetFactory.load("dpo", str(tmp_path), tokenizer_path=tok_dir)
    assert len(ds) == 3 and set(ds.keys) >= {"chosen", "rejected", "chosen_mask", "rejected_mask"}
    with pytest.raises(RuntimeError, match="lazy"):
        ds.store.fetch(0, 1, "chosen")
    with pytest.raises(ValueError):
        ds.store.fetch_record(3, "chosen")


def test_dpo_tokenize_masks_the_shared_prompt(tok_dir):
    from astrai_b200.data.dataset import dpo_tokenize
    from astrai_b200.tokenize import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(tok_dir)
    rec = dpo_tokenize({"prompt": "why is the sky blue?", "chosen": "scattering", "rejected": "paint"}, tok)
    n_prompt = rec["chosen_mask"].index(1) if isinstance(rec["chosen_mask"], list) else int((rec["chosen_mask"] == 0).sum())
    assert n_prompt > 0
    assert list(rec["chosen"][:n_prompt]) == list(rec["rejected"][:n_prompt])  # same prompt tokens in both sequences
    assert dpo_tokenize({"prompt": "x"}, tok) is None and dpo_tokenize({"chosen": "a", "rejected": "b"}, tok) is None
    short = dpo_tokenize({"prompt": "p " * 50, "chosen": "c " * 50, "rejected": "r " * 50}, tok, max_len=24)
    assert len(short["chosen"]) <= 24 and len(short["rejected"]) <= 24


def test_sft_jsonl_uses_the_builtin_messages_config_unless_a_config_file_exists(tmp_path, tok_dir):
    from astrai_b200.data import DatasetFactory

    d = tmp_path / "chat"
    d.mkdir()
    msgs = [{"role": "user", "content": "hello there"}, {"role": "assistant", "content": "general greeting, hello"}]
    _write_jsonl(d / "a.jsonl", [{"messages": msgs}] * 8)
    ds = DatasetFactory.load("sft", str(d), window_size=8, tokenizer_path=tok_dir)
    assert len(ds) > 0
    s = ds[0]
    assert s["loss_mask"].dtype == torch.bool and s["position_ids"].dtype == torch.long
    total_trained = sum(int(ds[i]["loss_mask"].sum()) for i in range(len(ds)))
    assert 0 < total_trained < len(ds) * 8  # assistant tokens only


# ----------------------------------------------------------------------------------------------------------- collate
def test_dpo_collate_pads_right_with_zero_masks():
    from astrai_b200.data import dpo_collate_fn

    batch = dpo_collate_fn([
        {"chosen": torch.tensor([5, 6, 7]), "rejected": torch.tensor([5, 9]), "chosen_mask": torch.tensor([False, True, True]),
         "rejected_mask": torch.tensor([False, True])},
        {"chosen": torch.tensor([1]), "rejected": torch.tensor([1, 2, 3, 4]), "chosen_mask": torch.tensor([True]),
         "rejected_mask": torch.tensor([False, True, True, True])}])
    assert batch["chosen"].shape == batch["rejected"].shape == batch["chosen_mask"].shape == (2, 4)
    assert batch["chosen"][0].tolist() == [5, 6, 7, 0] and batch["chosen_mask"][1].tolist() == [True, False, False, False]
    assert batch["chosen_mask"].dtype == torch.bool


def test_grpo_collate_shapes_for_ragged_groups():
    from astrai_b200.data import grpo_collate_fn

    item = lambda p, rs: {"prompts": torch.arange(1, p + 1), "responses": [torch.arange(1, n + 1) for n in rs],  # noqa: E731
                          "masks": [torch.ones(n, dtype=torch.bool) for n in rs], "rewards": torch.arange(len(rs)).float()}
    batch = grpo_collate_fn([item(3, [2, 5]), item(6, [4, 1])])
    assert batch["prompts"].shape == (2, 6) and batch["responses"].shape == (2, 2, 5) and batch["rewards"].shape == (2, 2)
    assert batch["prompts"][0].tolist() == [0, 0, 0, 1, 2, 3] and batch["prompt_mask"][0].tolist() == [False] * 3 + [True] * 3
    assert batch["masks"][0, 0].tolist() == [True, True, False, False, False]
    assert batch["masks"][1, 1].tolist() == [True, False, False, False, False]


def test_synthetic_dataset_is_deterministic_per_index():
    from astrai_b200.data.dataset import SyntheticTokenDataset

    a, b = SyntheticTokenDataset(10, 32, 500, seed=3), SyntheticTokenDataset(10, 32, 500, seed=3)
    assert len(a) == 10 and torch.equal(a[4]["input_ids"], b[4]["input_ids"])
    assert torch.equal(a[4]["input_ids"][1:], a[4]["target_ids"][:-1])
    assert not torch.equal(a[4]["input_ids"], a[5]["input_ids"])
    assert not torch.equal(a[4]["input_ids"], SyntheticTokenDataset(10, 32, 500, seed=4)[4]["input_ids"])
    assert int(a[0]["input_ids"].max()) < 500


# ----------------------------------------------------------------------------------------------------------- sampler
def test_sampler_is_a_permutation_and_repeats_for_the_same_seed():
    from astrai_b200.data import RDSampler

    data = list(range(37))
    a, b = list(RDSampler(data, seed=5)), list(RDSampler(data, seed=5))
    assert a == b and sorted(a) == data
    assert list(RDSampler(data, seed=6)) != a
    assert list(RDSampler(data, seed=5, shuffle=False)) == data


def test_sampler_reshuffles_every_epoch_and_resumes_mid_epoch():
    from astrai_b200.data import RDSampler

    data = list(range(50))
    s = RDSampler(data, seed=1)
    first, second = list(s), list(s)
    assert sorted(first) == sorted(second) == data and first != second  # a new order per epoch
    fresh = RDSampler(data, seed=1, start_epoch=1)
    assert list(fresh) == second  # an epoch's order depends on (seed, epoch) only
    resumed = RDSampler(data, seed=1, start_epoch=0, start_iter=20)
    assert list(resumed) == first[20:]
    assert list(resumed) == second  # after the partial epoch the next one is whole again


def test_sampler_partitions_are_disjoint_and_cover_the_data():
    from astrai_b200.data import RDSampler

    data = list(range(41))
    parts = [list(RDSampler(data, seed=9, partition=(i, 4))) for i in range(4)]
    sizes = {len(p) for p in parts}
    assert len(sizes) == 1  # every data-parallel position steps the same number of times
    flat = [x for p in parts for x in p]
    assert len(set(flat)) >= len(data) - 3 and set(flat) <= set(data)
    dropped = [list(RDSampler(data, seed=9, partition=(i, 4), drop_last=True)) for i in range(4)]
    assert sum(len(p) for p in dropped) == 40 and len({x for p in dropped for x in p}) == 40
    assert len(RDSampler(data, seed=9, partition=(0, 4), drop_last=True)) == 10


def test_stores_satisfy_the_stream_and_record_protocols(tmp_path):
    from astrai_b200.data import MmapStore, Recordable, Streamable

    store = MmapStore()
    assert isinstance(store, Streamable) and isinstance(store, Recordable)
    assert not isinstance(object(), Streamable) and not isinstance([], Recordable)
