"""``python -m astrai_b200.cli.benchmark``: inference benchmarks on a random-init model.

* ``prefill`` / ``decode``: the measurements of the reference's ``scripts/tools/benchmark.py:169-286`` (prefill
  tokens/s of one packed forward; decode tokens/s through the real scheduler, sampler and CUDA graphs).
* ``serve``: a continuous-batching load test - Poisson arrivals, log-normal prompt lengths, shared prefixes, uniform
  output lengths - reporting output tokens/s, p50 / p99 time to first token and p50 time per output token.  Requests
  are injected straight into the scheduler (token ids, no HTTP) from a timer thread; every timestamp is taken on the
  host when a token is handed to the request's callback.

Presets: ``1b`` = 24 layers, d 2048, 16 query / 4 KV heads, head_dim 128, FFN 5632, vocab 32000 (the training
benchmark's model); ``ref1b`` = the preset of the reference's benchmark (d 1536, 24 layers, 24q / 4kv, FFN 6912,
vocab 100000).
"""

from __future__ import annotations

import json
import os
import math
import random
import threading
import time
from typing import Dict, List, Optional

import click

PRESETS = {
    "1b": dict(vocab_size=32000, hidden_size=2048, num_hidden_layers=24, intermediate_size=5632, num_attention_heads=16,
               num_key_value_heads=4, max_position_embeddings=8192),
    "ref1b": dict(vocab_size=100000, hidden_size=1536, num_hidden_layers=24, intermediate_size=6912, num_attention_heads=24,
                  num_key_value_heads=4, max_position_embeddings=32768),
    "tiny": dict(vocab_size=4096, hidden_size=256, num_hidden_layers=2, intermediate_size=688, num_attention_heads=4,
                 num_key_value_heads=2, max_position_embeddings=4096),
}


class _IdTokenizer:
    """Stands in for a tokenizer when requests are token ids: no stop ids, decode renders ids."""

    stop_ids: List[int] = []

    def encode(self, text):
        return [int(t) for t in str(text).split()]

    def decode(self, ids, skip_special_tokens=True):
        return " ".join(str(i) for i in ids)


def build_model(preset: str, device: str, dtype):
    import torch

    from astrai_b200.config import AutoRegressiveLMConfig
    from astrai_b200.models import AutoRegressiveLM

    cfg = AutoRegressiveLMConfig(rms_norm_eps=1e-6, tie_word_embeddings=True, rope_theta=10000.0, **PRESETS[preset])
    torch.manual_seed(0)
    return AutoRegressiveLM(cfg).to(device=device, dtype=dtype).eval()


def _pct(values: List[float], q: float) -> Optional[float]:
    if not values:
        return None
    s = sorted(values)
    return s[min(len(s) - 1, max(0, math.ceil(q * len(s)) - 1))]


def make_requests(n: int, rate: float, vocab: int, seed: int, prompt_mean: float = 512.0, sigma: float = 0.6,
                  prompt_range=(16, 4096), shared_fraction: float = 0.5, n_prefixes: int = 8, prefix_len: int = 1024,
                  out_range=(64, 512)) -> List[Dict]:
    """The synthetic request stream: arrival time, prompt ids, output budget."""
    rng = random.Random(seed)
    mu = math.log(prompt_mean) - sigma * sigma / 2  # log-normal with the requested mean
    prefixes = [[rng.randrange(2, vocab) for _ in range(prefix_len)] for _ in range(n_prefixes)]
    t, reqs = 0.0, []
    for _ in range(n):
        t += rng.expovariate(rate)
        plen = int(min(max(rng.lognormvariate(mu, sigma), prompt_range[0]), prompt_range[1]))
        if rng.random() < shared_fraction:
            head = prefixes[rng.randrange(n_prefixes)]
            ids = (head + [rng.randrange(2, vocab) for _ in range(max(plen - prefix_len, 16))])
        else:
            ids = [rng.randrange(2, vocab) for _ in range(plen)]
        reqs.append({"arrival": t, "ids": ids, "max_tokens": rng.randint(*out_range)})
    return reqs


def run_serve(scheduler, requests: List[Dict], temperature: float, top_p: float, top_k: int, time_scale: float = 1.0,
              stop=None, as_text: bool = False) -> Dict:
    """Replay ``requests`` against a started scheduler; returns the aggregate metrics.  ``stop`` is the scheduler's
    end-of-stream sentinel (default: this package's); ``as_text`` submits prompts as space-separated id strings for a
    scheduler whose ``add_task`` tokenises text."""
    if stop is None:
        from astrai_b200.inference import STOP as stop
    STOP = stop

    lock = threading.Lock()
    records = [{"arrival": None, "first": None, "last": None, "tokens": 0} for _ in requests]
    done = threading.Event()
    remaining = [len(requests)]

    def callback_for(i):
        def cb(token):
            now = time.perf_counter()
            rec = records[i]
            if token is STOP:
                with lock:
                    remaining[0] -= 1
                    if remaining[0] == 0:
                        done.set()
                return
            if rec["first"] is None:
                rec["first"] = now
            rec["last"] = now
            rec["tokens"] += 1
        return cb

    t0 = time.perf_counter()

    def feeder():
        for i, req in enumerate(requests):
            delay = t0 + req["arrival"] * time_scale - time.perf_counter()
            if delay > 0:
                time.sleep(delay)
            records[i]["arrival"] = time.perf_counter()
            prompt = " ".join(map(str, req["ids"])) if as_text else req["ids"]
            scheduler.add_task(prompt, max_tokens=req["max_tokens"], temperature=temperature, top_p=top_p, top_k=top_k,
                               stream_callback=callback_for(i))

    th = threading.Thread(target=feeder, daemon=True)
    th.start()
    th.join()
    done.wait(timeout=3600)
    wall = time.perf_counter() - t0
    ttft = [(r["first"] - r["arrival"]) * 1e3 for r in records if r["first"] is not None]
    tpot = [(r["last"] - r["first"]) * 1e3 / (r["tokens"] - 1) for r in records if r["tokens"] > 1]
    out_tokens = sum(r["tokens"] for r in records)
    return {"requests": len(requests), "completed": sum(1 for r in records if r["tokens"] > 0), "wall_s": wall,
            "output_tokens": out_tokens, "output_tok_per_s": out_tokens / wall if wall > 0 else None,
            "ttft_ms_p50": _pct(ttft, 0.5), "ttft_ms_p99": _pct(ttft, 0.99), "tpot_ms_p50": _pct(tpot, 0.5),
            "prompt_tokens": sum(len(r["ids"]) for r in requests)}


def _id_tokenizer_dir(vocab: int) -> str:
    """A tokenizer.json whose tokens are the decimal strings "0" .. str(vocab-1) with matching ids (whitespace split), so
    that a scheduler which tokenises text sees exactly the requested ids and can stream any sampled id back."""
    import tempfile

    from tokenizers import Tokenizer, decoders, models, pre_tokenizers

    tk = Tokenizer(models.WordLevel({str(i): i for i in range(vocab)}, unk_token="0"))
    tk.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tk.decoder = decoders.Fuse()
    path = tempfile.mkdtemp(prefix="id_tokenizer_")
    tk.save(os.path.join(path, "tokenizer.json"))
    with open(os.path.join(path, "tokenizer_config.json"), "w") as fh:
        json.dump({}, fh)
    return path


def _serve_reference(preset, device, n_requests, rate, max_batch_size, max_seq_len, kv_cache_tokens, temperature, top_p, top_k,
                     seed, time_scale, backend) -> Dict:
    """The same load test against the reference's own scheduler, model and paged cache (its public API, stock code path)."""
    import torch
    from astrai.config import AutoRegressiveLMConfig  # the reference package
    from astrai.inference import STOP, InferenceScheduler
    from astrai.inference.cache.pool import PagePool
    from astrai.model import AutoRegressiveLM
    from astrai.tokenize import AutoTokenizer

    cfg = AutoRegressiveLMConfig(rms_norm_eps=1e-6, tie_word_embeddings=True, rope_theta=10000.0, **PRESETS[preset])
    torch.manual_seed(0)
    model = AutoRegressiveLM(cfg).to(device=device, dtype=torch.bfloat16).eval()
    tok = AutoTokenizer.from_pretrained(_id_tokenizer_dir(cfg.vocab_size))
    pool = PagePool(cfg.num_hidden_layers, cfg.num_key_value_heads, cfg.hidden_size // cfg.num_attention_heads, max_batch_size,
                    max_seq_len, torch.device(device), torch.bfloat16, page_size=16,
                    n_tokens=kv_cache_tokens or max_batch_size * 4608)
    sched = InferenceScheduler(model, tok, max_batch_size=max_batch_size, max_seq_len=max_seq_len, cache=pool, backend=backend)
    reqs = make_requests(n_requests, rate, cfg.vocab_size, seed)
    sched.start()
    try:
        res = run_serve(sched, reqs, temperature, top_p, top_k, time_scale, stop=STOP, as_text=True)
    finally:
        sched.stop()
    res.update({"benchmark": "serve", "impl": "reference", "backend": backend, "preset": preset, "rate": rate,
                "max_batch_size": max_batch_size, "page_size": 16,
                "sampling": {"temperature": temperature, "top_p": top_p, "top_k": top_k, "seed": seed}})
    return res


@click.group()
def benchmark():
    """Inference benchmarks on random-init weights."""


def _model_options(fn):
    """Options shared by ``prefill`` and ``decode``: which model, in which precision, over which cache, on which back end
    (the reference's ``--ckpt / --config / --dtype / --cache / --backend / --compare``, ``scripts/tools/benchmark.py:409-455``)."""
    for opt in reversed([
        click.option("--preset", type=click.Choice(sorted(PRESETS)), default="1b", help="Architecture when neither --ckpt nor --config is given."),
        click.option("--ckpt", type=click.Path(exists=True, file_okay=False), default=None, help="Model directory to load instead of random weights."),
        click.option("--config", "config_path", type=click.Path(exists=True, dir_okay=False), default=None,
                     help="Model config JSON: random weights of that architecture."),
        click.option("--device", default="cuda"),
        click.option("--dtype", type=click.Choice(["bfloat16", "float16", "float32"]), default=None, help="Default: bfloat16 on CUDA, float32 on the CPU."),
        click.option("--cache", type=click.Choice(["paged", "contiguous"]), default="paged", help="KV cache layout."),
        click.option("--backend", type=str, default=None, help="Attention back end (tcgen05, torch_native, or a registered name); default: the process default."),
        click.option("--compare", is_flag=True, default=False, help="Run under tcgen05 and torch_native and print both with their ratio."),
    ]):
        fn = opt(fn)
    return fn


def _load_model(preset, ckpt, config_path, device, dtype):
    import torch

    from astrai_b200.cli.common import torch_dtype

    dt = torch_dtype(dtype) if dtype else (torch.bfloat16 if device != "cpu" else torch.float32)
    if ckpt:
        from astrai_b200.models import AutoModel

        return AutoModel.from_pretrained(ckpt).to(device=device, dtype=dt).eval(), os.path.basename(os.path.normpath(ckpt))
    if config_path:
        from astrai_b200.config import AutoRegressiveLMConfig
        from astrai_b200.models import AutoRegressiveLM

        torch.manual_seed(0)
        return AutoRegressiveLM(AutoRegressiveLMConfig.from_file(config_path)).to(device=device, dtype=dt).eval(), os.path.basename(config_path)
    return build_model(preset, device, dt), preset


def _arms(backend, compare):
    return ["tcgen05", "torch_native"] if compare else [backend]


def _report(rows, key):
    for row in rows:
        click.echo(json.dumps(row))
    if len(rows) == 2:
        click.echo(json.dumps({"compare": key, rows[0]["backend"] + "_over_" + rows[1]["backend"]: rows[0][key] / max(rows[1][key], 1e-12)}))


def _scheduler(model, batch_size, max_seq_len, cache, backend, **kw):
    from astrai_b200.inference import InferenceScheduler

    return InferenceScheduler(model, _IdTokenizer(), max_batch_size=batch_size, max_seq_len=max_seq_len, paged=cache == "paged",
                              page_size=16 if cache == "paged" else 1, backend=backend, **kw)


def _sync(device):
    import torch

    if device != "cpu":
        torch.cuda.synchronize()


@benchmark.command()
@_model_options
@click.option("--batch_size", type=int, default=8)
@click.option("--prompt_len", type=int, default=1024)
@click.option("--trials", type=int, default=5)
def prefill(preset, ckpt, config_path, device, dtype, cache, backend, compare, batch_size, prompt_len, trials):
    """Tokens/s of packed prefill forwards through the scheduler's executor."""
    import torch

    from astrai_b200.ops import backend as attn_backends

    model, name = _load_model(preset, ckpt, config_path, device, dtype)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(2, model.config.vocab_size, (prompt_len,), generator=g).tolist() for _ in range(batch_size)]
    rows = []
    for arm in _arms(backend, compare):
        sched = _scheduler(model, batch_size, prompt_len + 8, cache, arm)
        times = []
        with sched._backend_context():
            for i in range(trials + 3):
                _sync(device)
                t0 = time.perf_counter()
                sched.run_batch(prompts, max_tokens=1, temperature=0.0)
                _sync(device)
                if i >= 3:
                    times.append(time.perf_counter() - t0)
        best = min(times)
        rows.append({"benchmark": "prefill", "model": name, "backend": sched.backend_name, "cache": cache, "batch": batch_size,
                     "prompt_len": prompt_len, "tok_per_s": batch_size * prompt_len / best, "ms": best * 1e3})
        del sched
    _report(rows, "tok_per_s")


@benchmark.command()
@_model_options
@click.option("--batch_size", type=int, default=16)
@click.option("--prompt_len", type=int, default=128)
@click.option("--gen_len", type=int, default=256)
@click.option("--cuda_graph/--no-cuda_graph", default=True)
def decode(preset, ckpt, config_path, device, dtype, cache, backend, compare, batch_size, prompt_len, gen_len, cuda_graph):
    """Decode tokens/s through scheduler + sampler (+ CUDA graphs)."""
    import torch

    model, name = _load_model(preset, ckpt, config_path, device, dtype)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(2, model.config.vocab_size, (prompt_len,), generator=g).tolist() for _ in range(batch_size)]
    rows = []
    for arm in _arms(backend, compare):
        sched = _scheduler(model, batch_size, prompt_len + gen_len + 8, cache, arm, enable_cuda_graph=cuda_graph)
        with sched._backend_context():
            sched.run_batch(prompts, max_tokens=8, temperature=0.0)  # warm-up
            _sync(device)
            t0 = time.perf_counter()
            out = sched.run_batch(prompts, max_tokens=gen_len, temperature=0.0)
            _sync(device)
            dt = time.perf_counter() - t0
        n = sum(len(o[0]) if isinstance(o, tuple) else len(o) for o in out)
        rows.append({"benchmark": "decode", "model": name, "backend": sched.backend_name, "cache": cache, "cuda_graph": sched.cuda_graph_enabled,
                     "batch": batch_size, "gen_len": gen_len, "tok_per_s": n / dt, "ms_per_step": dt * 1e3 / max(gen_len, 1)})
        del sched
    _report(rows, "tok_per_s")


@benchmark.command()
@click.option("--preset", type=click.Choice(sorted(PRESETS)), default="1b")
@click.option("--device", default="cuda")
@click.option("--requests", "n_requests", type=int, default=2048)
@click.option("--rate", type=float, default=32.0, help="Poisson arrival rate (requests / s).")
@click.option("--max_batch_size", type=int, default=64)
@click.option("--max_seq_len", type=int, default=8192)
@click.option("--kv_cache_tokens", type=int, default=None)
@click.option("--temperature", type=float, default=0.8)
@click.option("--top_p", type=float, default=0.95)
@click.option("--top_k", type=int, default=50)
@click.option("--seed", type=int, default=0)
@click.option("--time_scale", type=float, default=1.0, help="Stretch (>1) or compress (<1) the arrival times.")
@click.option("--chunked_prefill/--no-chunked_prefill", default=False)
@click.option("--max_prefill_tokens", type=int, default=8192)
@click.option("--impl", type=click.Choice(["ours", "reference"]), default="ours",
              help="'reference' drives the unmodified reference package (importable as `astrai`, e.g. PYTHONPATH=baseline/_ref) "
                   "with the same request stream.")
@click.option("--ref_backend", type=str, default="flash", help="Attention backend of the reference arm.")
def serve(preset, device, n_requests, rate, max_batch_size, max_seq_len, kv_cache_tokens, temperature, top_p, top_k, seed,
          time_scale, chunked_prefill, max_prefill_tokens, impl, ref_backend):
    """Continuous-batching load test with a paged KV cache (16-token pages) and the radix prefix cache."""
    import torch

    if impl == "reference":
        click.echo(json.dumps(_serve_reference(preset, device, n_requests, rate, max_batch_size, max_seq_len, kv_cache_tokens,
                                               temperature, top_p, top_k, seed, time_scale, ref_backend)))
        return
    from astrai_b200.inference import InferenceScheduler

    model = build_model(preset, device, torch.bfloat16 if device != "cpu" else torch.float32)
    sched = InferenceScheduler(model, _IdTokenizer(), max_batch_size=max_batch_size, max_seq_len=max_seq_len, page_size=16,
                               kv_cache_tokens=kv_cache_tokens or max_batch_size * 4608, paged=True,
                               chunked_prefill=chunked_prefill, max_prefill_tokens=max_prefill_tokens)
    reqs = make_requests(n_requests, rate, model.config.vocab_size, seed)
    sched.run_batch([reqs[0]["ids"][:64]], max_tokens=4, temperature=0.0)  # warm-up
    sched.start()
    try:
        res = run_serve(sched, reqs, temperature, top_p, top_k, time_scale)
    finally:
        sched.stop()
    res.update({"benchmark": "serve", "preset": preset, "rate": rate, "max_batch_size": max_batch_size, "page_size": 16,
                "chunked_prefill": chunked_prefill, "max_prefill_tokens": max_prefill_tokens,
                "sampling": {"temperature": temperature, "top_p": top_p, "top_k": top_k, "seed": seed}})
    click.echo(json.dumps(res))


if __name__ == "__main__":
    benchmark()
