"""``python -m astrai_b200.cli.serve``: start the OpenAI / Anthropic compatible HTTP server.

Options of the reference's ``scripts/tools/server.py:90-193`` plus the cache controls its CLI does not expose
(``astrai/inference/scheduler.py:56-67`` always builds a contiguous pool): ``--page_size`` (default 16: paged KV
cache with the radix prefix cache; 1 selects the contiguous cache) and ``--kv_cache_tokens``.
"""

from __future__ import annotations

from pathlib import Path
from typing import Optional

import click

from astrai_b200.cli.common import flatten_sections, load_yaml, merge_config, torch_dtype


@click.command(context_settings={"show_default": True})
@click.option("--config", "-c", type=click.Path(exists=True, dir_okay=False), default=None)
@click.option("--host", type=str, default="0.0.0.0")
@click.option("--port", type=int, default=8000)
@click.option("--param_path", type=click.Path(), default="params")
@click.option("--device", type=str, default="cuda")
@click.option("--dtype", type=click.Choice(["bfloat16", "float16", "float32"]), default="bfloat16")
@click.option("--max_batch_size", type=int, default=16)
@click.option("--max_seq_len", type=int, default=None)
@click.option("--page_size", type=int, default=16, help="Tokens per KV page (1 = contiguous cache).")
@click.option("--kv_cache_tokens", type=int, default=None, help="Size of the paged KV pool in tokens.")
@click.option("--cuda_graph/--no-cuda_graph", default=True)
@click.option("--chunked_prefill/--no-chunked_prefill", default=False,
              help="Spread long prompts over several steps (at most --max_prefill_tokens prompt tokens per step).")
@click.option("--max_prefill_tokens", type=int, default=8192)
@click.option("--prefill_defer_steps", type=int, default=8,
              help="Under load (32 or more requests decoding) new prompts wait up to this many decode steps so that "
                   "several are prefilled in one forward; 0 prefills every prompt at once.")
@click.option("--tp_size", type=int, default=1,
              help="Tensor-parallel serving: one replica over this many GPUs; start the command under "
                   "`python -m torch.distributed.run --nproc-per-node TP_SIZE -m astrai_b200.cli.serve ...`.")
@click.option("--reload", is_flag=True, default=False)
@click.pass_context
def serve_command(ctx: click.Context, config: Optional[str], **opts):
    """Serve a model directory over HTTP (POST /v1/chat/completions, POST /v1/messages, GET /health, GET /stats)."""
    o = merge_config(ctx, opts, flatten_sections(load_yaml(config), ("server",)))
    from astrai_b200.inference import run_server

    engine_kwargs = {"enable_cuda_graph": o["cuda_graph"], "paged": o["page_size"] > 1, "page_size": o["page_size"],
                     "kv_cache_tokens": o["kv_cache_tokens"], "chunked_prefill": o["chunked_prefill"],
                     "max_prefill_tokens": o["max_prefill_tokens"], "prefill_defer_steps": o["prefill_defer_steps"], "tp_size": o["tp_size"]}
    run_server(param_path=Path(o["param_path"]), host=o["host"], port=o["port"], reload=o["reload"], device=o["device"],
               dtype=torch_dtype(o["dtype"]), max_batch_size=o["max_batch_size"], max_seq_len=o["max_seq_len"], **engine_kwargs)


if __name__ == "__main__":
    serve_command()
