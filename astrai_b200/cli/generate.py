"""``python -m astrai_b200.cli.generate``: batch generation from a JSONL file of questions.

Counterpart of ``scripts/tools/generate.py:117-159`` of the reference: each input line holds ``{question_key: text}``;
each output line repeats the input with ``response_key`` added (a list when ``--num_samples`` > 1).
"""

from __future__ import annotations

import json

import click


def _chunks(items, n):
    for i in range(0, len(items), n):
        yield items[i:i + n]


@click.command(context_settings={"show_default": True})
@click.option("--param_path", type=str, required=True)
@click.option("--input_json_file", type=click.Path(exists=True, dir_okay=False), required=True)
@click.option("--output_json_file", type=click.Path(dir_okay=False), required=True)
@click.option("--question_key", type=str, default="question")
@click.option("--response_key", type=str, default="response")
@click.option("--temperature", type=float, default=0.8)
@click.option("--top_k", type=int, default=50)
@click.option("--top_p", type=float, default=0.95)
@click.option("--batch_size", type=int, default=1)
@click.option("--num_samples", type=int, default=1)
@click.option("--max_seq_len", type=int, default=2048)
@click.option("--max_tokens", type=int, default=None)
@click.option("--frequency_penalty", type=float, default=0.0)
@click.option("--rep_window", type=int, default=64)
@click.option("--device", type=str, default="cuda")
def generate_command(param_path, input_json_file, output_json_file, question_key, response_key, temperature, top_k, top_p,
                     batch_size, num_samples, max_seq_len, max_tokens, frequency_penalty, rep_window, device):
    """Answer every question of a JSONL file with the model in PARAM_PATH."""
    import torch

    from astrai_b200.inference import InferenceEngine
    from astrai_b200.models import AutoModel
    from astrai_b200.tokenize import AutoTokenizer

    with open(input_json_file) as fh:
        records = [json.loads(line) for line in fh if line.strip()]
    tokenizer = AutoTokenizer.from_pretrained(param_path)
    model = AutoModel.from_pretrained(param_path).to(device=device, dtype=torch.bfloat16 if device != "cpu" else torch.float32).eval()
    engine = InferenceEngine(model, tokenizer, max_batch_size=max(batch_size * num_samples, 1), max_seq_len=max_seq_len)
    try:
        with open(output_json_file, "w") as out:
            for batch in _chunks(records, batch_size):
                prompts = [tokenizer.apply_chat_template([{"role": "user", "content": str(r[question_key])}], tokenize=False,
                                                         add_generation_prompt=True) for r in batch for _ in range(num_samples)]
                answers = engine.generate(prompts, max_tokens=max_tokens, temperature=temperature, top_k=top_k, top_p=top_p,
                                          frequency_penalty=frequency_penalty, rep_window=rep_window)
                for i, rec in enumerate(batch):
                    mine = answers[i * num_samples:(i + 1) * num_samples]
                    out.write(json.dumps({**rec, response_key: mine[0] if num_samples == 1 else mine}, ensure_ascii=False) + "\n")
    finally:
        engine.shutdown()


if __name__ == "__main__":
    generate_command()
