"""Configuration objects: defaults, validation messages, dictionary and file round trips (model, training, pipeline)."""

import json

import pytest

from astrai_b200.config import AutoRegressiveLMConfig, ConfigFactory, EncoderConfig, PipelineConfig, TrainConfig
from astrai_b200.config.preprocess_config import InputConfig, OutputConfig, ProcessingConfig


def test_pipeline_defaults():
    c = PipelineConfig()
    assert c.version == 1 and c.mask == {} and c.mask_default == "mask" and c.input.sections is None and c.input.sources is None
    assert (c.preprocessing.max_seq_len, c.preprocessing.min_chars, c.preprocessing.max_chars) == (2048, 50, 2_000_000)
    assert (c.preprocessing.batch_size, c.preprocessing.packing_strategy, c.preprocessing.max_packed_len) == (256, "simple", 8192)
    assert (c.output.storage_format, c.output.position_ids_mode, c.output.max_tokens_per_shard) == ("bin", "doc_reset", 100_000_000)


def test_pipeline_from_dict_builds_the_nested_sections_and_keeps_unset_defaults():
    c = PipelineConfig.from_dict({"version": 1, "input": {"sections": [{"field": "messages", "action": "$role", "template": True}]},
                                  "mask": {"system": "mask", "assistant": "train"}, "preprocessing": {"max_seq_len": 1024},
                                  "output": {"storage_format": "jsonl"}})
    assert isinstance(c.input, InputConfig) and isinstance(c.preprocessing, ProcessingConfig) and isinstance(c.output, OutputConfig)
    assert c.input.sections == [{"field": "messages", "action": "$role", "template": True}]
    assert c.preprocessing.max_seq_len == 1024 and c.preprocessing.batch_size == 256 and c.output.storage_format == "jsonl"


@pytest.mark.parametrize("sources", [False, True])
def test_pipeline_round_trips_through_dict_and_file(tmp_path, sources):
    if sources:
        raw = {"input": {"sources": {"chosen": {"sections": [{"field": "chosen", "action": "train"}]},
                                     "rejected": {"sections": [{"field": "rejected", "action": "train"}]}}}}
    else:
        raw = {"input": {"sections": [{"field": "prompt", "action": "mask"}, {"field": "response", "action": "train"}]},
               "mask": {"prompt": "mask", "response": "train"}, "output": {"dtype": {"sequence": "int64"}, "domain_key": "source"}}
    c = PipelineConfig.from_dict(raw)
    again = PipelineConfig.from_dict(c.to_dict())
    assert again == c
    path = tmp_path / "pipeline.json"
    c.to_file(path)
    loaded = PipelineConfig.from_file(path)
    assert loaded == c and (loaded.input.sources is not None) == sources and (loaded.input.sections is None) == sources
    assert json.loads(path.read_text())["preprocessing"]["packing_strategy"] == "simple"  # a plain, readable JSON file


@pytest.mark.parametrize("section,key,value,message", [
    ("preprocessing", "packing_strategy", "tetris", "packing_strategy"), ("preprocessing", "truncation_mode", "middle", "truncation_mode"),
    ("preprocessing", "max_seq_len", 0, "positive"), ("preprocessing", "batch_size", -1, "positive"), ("preprocessing", "min_chars", -1, "non-negative"),
    ("output", "storage_format", "parquet", "storage_format"), ("output", "position_ids_mode", "random", "position_ids_mode")])
def test_pipeline_rejects_bad_values_by_name(section, key, value, message):
    with pytest.raises(ValueError, match=message):
        PipelineConfig.from_dict({section: {key: value}})


def test_model_config_file_round_trip_and_factory(tmp_path):
    c = AutoRegressiveLMConfig(vocab_size=100, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                               intermediate_size=64, max_position_embeddings=128, ffn_type="moe", n_routed_experts=4, n_activated_experts=2)
    path = tmp_path / "config.json"
    c.to_file(path)
    loaded = ConfigFactory.load(path)
    assert isinstance(loaded, AutoRegressiveLMConfig) and loaded.to_dict() == c.to_dict()
    raw = json.loads(path.read_text())
    assert raw["model_type"] is None and raw["n_routed_experts"] == 4  # an unnamed type reads back as the decoder LM
    assert isinstance(ConfigFactory.load(raw), AutoRegressiveLMConfig)  # a dictionary works like the file
    enc = EncoderConfig(model_type="embedding", vocab_size=50, hidden_size=16, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=2, intermediate_size=32,
                        max_position_embeddings=32)
    enc.to_file(tmp_path / "enc.json")
    assert isinstance(ConfigFactory.load(tmp_path / "enc.json"), EncoderConfig)


def test_model_config_ignores_unknown_keys_of_foreign_files(tmp_path):
    path = tmp_path / "config.json"
    path.write_text(json.dumps({"model_type": "autoregressive_lm", "vocab_size": 10, "hidden_size": 8, "num_hidden_layers": 1,
                                "num_attention_heads": 2, "num_key_value_heads": 1, "intermediate_size": 16, "max_position_embeddings": 16,
                                "architectures": ["Whatever"], "torch_dtype": "bfloat16", "transformers_version": "9.9"}))
    c = ConfigFactory.load(path)
    assert c.vocab_size == 10 and not hasattr(c, "architectures")


def _train(**over):
    base = dict(model_fn=lambda: None, strategy="seq", dataset=[1], optimizer_fn=lambda m: None)
    base.update(over)
    return TrainConfig(**base)


def test_train_config_defaults_match_the_reference():
    c = _train()
    assert (c.n_epoch, c.batch_per_device, c.grad_accum_steps, c.max_grad_norm) == (1, 4, 1, 1.0)
    assert (c.ckpt_dir, c.ckpt_interval, c.random_seed) == ("./checkpoint", 5000, 3407)
    assert (c.nprocs, c.backend, c.parallel_mode, c.start_method, c.device_type) == (1, "nccl", "none", "spawn", "cuda")
    assert c.metrics == ["loss", "lr", "grad_norm"] and c.val_split is None and c.moe_aux_loss_coef == 0.01


@pytest.mark.parametrize("field,value", [("strategy", "ppo"), ("parallel_mode", "zero3"), ("backend", "mpi"), ("start_method", "thread"),
                                         ("compile_mode", "fastest"), ("val_split", 1.5), ("val_split", 0.0), ("moe_aux_loss_coef", -0.1)])
def test_train_config_rejects_bad_values(field, value):
    with pytest.raises(ValueError):
        _train(**{field: value})


def test_train_config_to_dict_holds_only_what_json_can_hold():
    c = _train(dataset=object(), optimizer_name="fused_adamw", optimizer_hyperparameters={"lr": 1e-3}, executor_kwargs={"comm": "nccl"})
    d = c.to_dict()
    json.dumps(d)  # no callables, no datasets
    assert d["strategy"] == "seq" and d["optimizer_name"] == "fused_adamw" and d["optimizer_hyperparameters"] == {"lr": 1e-3}
    assert "model_fn" not in d and "dataset" not in d and "optimizer_fn" not in d
