"""``python -m astrai_b200.cli.preprocess``: tokenise / mask / pack JSON(L) files into training shards.

Counterpart of ``scripts/tools/preprocess.py:9-50`` of the reference.
"""

from __future__ import annotations

import click


@click.command(context_settings={"show_default": True})
@click.argument("input_files", nargs=-1, required=True, type=click.Path(exists=True, dir_okay=False))
@click.option("--output_dir", "-o", type=click.Path(file_okay=False), required=True)
@click.option("--config", "-c", type=click.Path(exists=True, dir_okay=False), required=True, help="Pipeline config (JSON).")
@click.option("--tokenizer_path", type=str, default="params")
@click.option("--batch_size", type=click.IntRange(min=1), default=None, help="Records per tokenisation batch (overrides the config).")
def preprocess_command(input_files, output_dir, config, tokenizer_path, batch_size):
    """Run the preprocessing pipeline over INPUT_FILES and write ``<output_dir>/<domain>/shard_NNNN/``."""
    from astrai_b200.config import PipelineConfig
    from astrai_b200.preprocessing import Pipeline

    cfg = PipelineConfig.from_file(config)
    if batch_size is not None:
        cfg.preprocessing.batch_size = batch_size
    click.echo(f"Preprocessing {len(input_files)} file(s) -> {output_dir}")
    kept = Pipeline(cfg, list(input_files), output_dir, tokenizer_path).run()
    click.echo(f"Done: {kept} record(s) kept.")


if __name__ == "__main__":
    preprocess_command()
