"""The user guides stay true: every command-line option is documented, and the configuration examples load."""

import json
import os
import re

import click
import pytest
from click.testing import CliRunner

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DOCS = os.path.join(ROOT, "docs")


def _read(*parts):
    with open(os.path.join(DOCS, *parts), encoding="utf-8") as fh:
        return fh.read()


def _blocks(text, lang):
    return re.findall(r"```" + lang + r"\n(.*?)```", text, flags=re.S)


def _commands():
    from astrai_b200.cli.generate import generate_command
    from astrai_b200.cli.preprocess import preprocess_command
    from astrai_b200.cli.serve import serve_command
    from astrai_b200.cli.train import train_command

    return {"train": train_command, "serve": serve_command, "generate": generate_command, "preprocess": preprocess_command}


@pytest.mark.parametrize("name", ["train", "serve", "generate", "preprocess"])
def test_every_option_is_in_the_options_reference_with_its_default(name):
    text = _read("guides", "params.md")
    section = text.split(f"## `python -m astrai_b200.cli.{name}")[1].split("\n## ")[0]
    for p in _commands()[name].params:
        if isinstance(p, click.Argument):
            continue
        row = next((line for line in section.splitlines() if line.startswith("| ") and f"`{p.opts[-1]}`" in line.split("|")[1]), None)
        assert row is not None, f"--{p.name} is missing from docs/guides/params.md"
        if p.default not in (None, (), False, True) and not isinstance(p.default, (tuple, list)):
            assert f"`{p.default}`" in row, (p.name, row)
        assert row.split("|")[4].strip(), f"--{p.name} has no description"


def test_every_option_has_help_text():
    for name, cmd in _commands().items():
        for p in cmd.params:
            if isinstance(p, click.Option) and p.name not in ("config",):
                assert p.help or name != "train", f"{name} --{p.name}"


def test_pipeline_examples_are_valid_configurations():
    from astrai_b200.config import PipelineConfig

    blocks = [b for b in _blocks(_read("guides", "preprocessing.md"), "json") if '"input"' in b]
    assert len(blocks) >= 5
    for block in blocks:
        cfg = PipelineConfig.from_dict(json.loads(block))
        assert (cfg.input.sections is None) != (cfg.input.sources is None)


def test_training_yaml_example_is_accepted_by_the_command(tmp_path):
    from astrai_b200.cli.train import train_command

    blocks = [b for b in _blocks(_read("guides", "training.md"), "yaml") if "train_type" in b]
    assert blocks
    cfg = tmp_path / "train.yaml"
    cfg.write_text(blocks[0])
    res = CliRunner().invoke(train_command, ["-c", str(cfg), "--dry-run"])
    assert res.exit_code == 0, res.output
    plan = json.loads(res.output)
    assert plan["train_type"] == "sft" and plan["optimizer"] == "fused_adamw" and plan["nprocs"] == 8 and plan["max_lr"] == 2e-4


def test_serving_yaml_example_is_accepted_by_the_command(tmp_path, monkeypatch):
    from astrai_b200.cli.serve import serve_command

    blocks = [b for b in _blocks(_read("guides", "inference.md"), "yaml") if "server:" in b]
    assert blocks
    cfg = tmp_path / "serve.yaml"
    cfg.write_text(blocks[0])
    seen = {}
    monkeypatch.setattr("astrai_b200.inference.run_server", lambda **kw: seen.update(kw))
    res = CliRunner().invoke(serve_command, ["-c", str(cfg)])
    assert res.exit_code == 0, res.output
    assert seen["max_batch_size"] == 128 and seen["chunked_prefill"] is True and seen["page_size"] == 16 and seen["port"] == 8000


def test_model_config_example_builds_a_model_config():
    from astrai_b200.config import AutoRegressiveLMConfig

    block = next(b for b in _blocks(_read("get-started.md"), "json") if "hidden_size" in b)
    cfg = AutoRegressiveLMConfig(**json.loads(block))
    assert cfg.hidden_size // cfg.num_attention_heads == 128


def test_modules_and_files_named_in_the_guides_exist():
    import importlib

    text = "\n".join(_read(*p) for p in (("get-started.md",), ("guides", "training.md"), ("guides", "inference.md"), ("guides", "evaluation.md"),
                                           ("guides", "distributed.md"), ("guides", "preprocessing.md")))
    for module in sorted(set(re.findall(r"python -m (astrai_b200[\w.]*)", text))):
        assert importlib.util.find_spec(module) is not None, module
    for path in sorted(set(re.findall(r"\b(deploy/[\w.\-]+)", text))):
        assert os.path.exists(os.path.join(ROOT, path)), path
    for link in re.findall(r"\]\(((?:guides|developer)/[\w\-]+\.md)\)", _read("get-started.md")):
        assert os.path.exists(os.path.join(DOCS, link)), link


def test_options_page_is_what_the_generator_writes():
    from astrai_b200.cli.options_doc import render

    assert _read("guides", "params.md") == render(), "run: python -m astrai_b200.cli.options_doc > docs/guides/params.md"


def test_runtime_section_examples_produce_exports(tmp_path):
    import yaml

    from astrai_b200.cli import runtime

    blocks = [b for b in _blocks(_read("developer", "docker.md"), "yaml") if b.lstrip().startswith("runtime:")]
    assert len(blocks) == 2
    flat = runtime.exports("train", yaml.safe_load(blocks[0]), tmp_path)
    assert "export ASTRAI_GPUS=0,1,2,3" in flat and "export ASTRAI_AUTO_RESUME=1" in flat and "export ASTRAI_MAX_HOURS=47.5" in flat
    nested_cfg = yaml.safe_load(blocks[1])
    nested = runtime.exports("train", nested_cfg, tmp_path)
    assert "export ASTRAI_NPROCS=4" in nested and "export ASTRAI_CONTAINER=pretrain-1b" in nested
    assert any(line.startswith("export ASTRAI_DATA_DIR=" + str(tmp_path)) for line in nested)  # resolved against the config's directory
    assert runtime.environment_of(nested_cfg) == {"NCCL_DEBUG": "WARN"}
