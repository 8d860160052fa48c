"""``python -m astrai_b200.cli.options_doc > docs/guides/params.md``: the option reference, written from the commands.

One table per command (option, values, default, description) taken from the click definitions, so the page cannot drift
from ``--help``; ``tests/test_docs.py`` compares the committed page with this module's output.
"""

from __future__ import annotations

import sys

import click

def fmt_default(p):
    d = p.default
    if p.is_flag and p.secondary_opts:
        return f"`{'on' if d else 'off'}`"
    if p.is_flag:
        return "`off`" if not d else "`on`"
    if d is None or d == ():
        return "—"
    if isinstance(d, (tuple, list)):
        return "`" + " ".join(map(str, d)) + "`"
    return f"`{d}`"

def fmt_type(p):
    t = p.type
    if isinstance(t, click.Choice):
        return " \\| ".join(f"`{c}`" for c in t.choices)
    if p.is_flag:
        return "flag" + (f" (`--no-{p.name}` turns it off)" if p.secondary_opts else "")
    return {"INT": "int", "FLOAT": "float", "STRING": "text", "BOOL": "bool"}.get(t.name.upper(), t.name)

def table(cmd, notes):
    rows = ["| option | values | default | |", "|---|---|---|---|"]
    for p in cmd.params:
        if isinstance(p, click.Argument):
            continue
        name = " / ".join(f"`{o}`" for o in p.opts if not o.startswith("--no-"))
        if getattr(p, "multiple", False):
            name += " (repeatable)"
        help_ = (p.help or notes.get(p.name, "")).replace("|", "\\|")
        rows.append(f"| {name} | {fmt_type(p)} | {fmt_default(p)} | {help_} |")
    return "\n".join(rows)

NOTES = {"host": "Address to bind.", "port": "Port to bind.", "param_path": "Model directory.", "device": "cuda or cpu.",
         "dtype": "Weights and activations.", "max_batch_size": "Requests decoded together.",
         "max_seq_len": "Prompt + answer tokens per request (default: the model's max_position_embeddings).",
         "cuda_graph": "Replay decode steps from CUDA graphs captured at start-up.",
         "max_prefill_tokens": "Prompt tokens processed per step (per forward without --chunked_prefill).",
         "reload": "uvicorn auto-reload (development).", "config": "YAML file; explicit options win.",
         "input_json_file": "JSON Lines: one object per line with the question.", "output_json_file": "Where the answers go (JSON Lines).",
         "question_key": "Field holding the question.", "response_key": "Field to put the answer in.",
         "temperature": "Sampling temperature (0 = greedy).", "top_k": "Keep the k most likely tokens.", "top_p": "Keep the smallest set of tokens with this probability mass.",
         "batch_size": "Questions per batch.", "num_samples": "Answers per question.", "max_tokens": "Longest answer (default: the room left in --max_seq_len).",
         "frequency_penalty": "Penalty per earlier occurrence of a token in the last --rep_window tokens.", "rep_window": "Window of the frequency penalty.",
         "output_dir": "Where the shards go.", "tokenizer_path": "Directory with tokenizer.json and tokenizer_config.json."}

def render() -> str:
    from astrai_b200.cli.generate import generate_command
    from astrai_b200.cli.preprocess import preprocess_command
    from astrai_b200.cli.serve import serve_command
    from astrai_b200.cli.train import train_command

    return f"""# Command-line options

Generated from the commands themselves; `python -m astrai_b200.cli.<command> --help` prints the same.
Every option can also be given in the YAML file passed with `-c` (the name without the dashes; see the guides for the
file layouts); an option given on the command line wins over the file, the file wins over the default.

## `python -m astrai_b200.cli.train`

{table(train_command, NOTES)}

## `python -m astrai_b200.cli.serve`

{table(serve_command, NOTES)}

## `python -m astrai_b200.cli.generate`

{table(generate_command, NOTES)}

## `python -m astrai_b200.cli.preprocess INPUT_FILES...`

{table(preprocess_command, NOTES)}

## Environment variables

| variable | effect |
|---|---|
| `ASTR_LOG_LEVEL` | level of the package logger (`DEBUG`, `INFO`, `WARNING` …) |
| `ASTR_BACKEND` (or `ASTRAI_B200_ATTN`) | attention back end: `tcgen05` (default on CUDA: the hand-written kernels; `cuda` and `flash` are accepted as aliases) or `torch_native` / `sdpa` (PyTorch's scaled-dot-product attention, the comparison arm). In Python: `with astrai_b200.ops.attn_backend("torch_native"):` |
| `ASTRAI_B200_SDPA` | order of PyTorch attention back ends tried by the `sdpa` path, e.g. `cudnn,flash,efficient,math` |
| `ASTRAI_B200_FSDP_COMM` | default of `bench.py --comm` (`p2p`, `nvls`, `nccl`) |
| `ASTRAI_B200_TRACE` | `1`: named NVTX ranges per layer, step phase and collective (see `astrai_b200.utils.trace`, which can also export a Chrome trace with device times) |
| `ASTRAI_B200_NO_BUILD` | `1`: never compile the extension on import; fail if `_C.so` is missing |
| `ASTRAI_B200_BUILD_EXT` | `pip install`: `0` skips the extension build, `1` makes a failed build an error |
"""


def main() -> int:
    sys.stdout.write(render())
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
