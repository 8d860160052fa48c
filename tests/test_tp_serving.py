"""Tensor-parallel serving on gloo ranks: the replica cut over two ranks answers exactly as one process does."""

import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(tmp_path, port, *extra):
    out = str(tmp_path / "res.json")
    from helpers import launch_ranks

    code, log = launch_ranks(2, os.path.join(ROOT, "tests", "workers", "tp_serve.py"), ["--out", out, *extra], port, cwd=ROOT)
    assert code == 0, log
    return json.load(open(out))


@pytest.mark.parametrize("moe", [False, True])
def test_two_rank_replica_generates_what_one_process_generates(tmp_path, moe):
    res = _run(tmp_path, 29770 + int(moe), *(["--moe"] if moe else []))
    assert res["finished"] and res["got"] == res["want"]          # greedy streams, token for token
    assert res["local_heads"] == 2 and res["pool_heads"] == 1     # 4 query / 2 key-value heads cut in two
    assert res["sampled_pieces"] == 6 and res["active"] == 0 and res["n_ids"] == 5


def test_inference_sharding_keeps_the_math_and_refuses_what_it_cannot_cut():
    """Cut a model for two ranks inside one process (no process group: the sum is done by hand) and compare the summed
    partial outputs of one block with the whole block."""
    from helpers import tiny_config

    from astrai_b200.models import AutoRegressiveLM
    from astrai_b200.parallel import tp_inference as tpi

    torch.manual_seed(0)
    cfg = tiny_config(num_attention_heads=4, num_key_value_heads=2, hidden_size=16, intermediate_size=32)
    whole = AutoRegressiveLM(cfg).eval()
    x = torch.randn(1, 5, 16)
    rot = whole.rotary_embedding(x, None)
    ref_attn = whole.layers[0].attention(x, rot, None, None, True, None)
    ref_ffn = whole.layers[0].mlp(x)["hidden_states"]
    parts_attn, parts_ffn = [], []
    for rank in range(2):
        part = AutoRegressiveLM(cfg).eval()
        part.load_state_dict(whole.state_dict())
        tpi._shard_attention(part.layers[0].attention, 2, rank)
        tpi._shard_mlp(part.layers[0].mlp, 2, rank)
        parts_attn.append(part.layers[0].attention(x, rot, None, None, True, None))
        parts_ffn.append(part.layers[0].mlp(x)["hidden_states"])
        assert part.layers[0].attention.q_proj.weight.shape == (8, 16) and part.layers[0].mlp.down.weight.shape == (16, 16)
    assert torch.allclose(sum(parts_attn), ref_attn, atol=1e-5) and torch.allclose(sum(parts_ffn), ref_ffn, atol=1e-5)
    with pytest.raises(ValueError, match="do not divide"):
        tpi._shard_attention(AutoRegressiveLM(cfg).layers[0].attention, 4, 0)  # two key-value heads over four ranks
    local = tpi.LocalHeads(cfg, 2)
    assert (local.num_attention_heads, local.num_key_value_heads, local.hidden_size // local.num_attention_heads) == (2, 1, 4)
    assert local.num_hidden_layers == cfg.num_hidden_layers


def test_serve_command_with_two_tensor_parallel_processes_answers_over_http(tmp_path):
    """``torchrun --nproc-per-node 2 -m astrai_b200.cli.serve --tp_size 2`` on the CPU: the first rank answers HTTP requests,
    the second follows; the answer equals the single-process engine's."""
    import signal
    import time
    import urllib.request

    from helpers import build_tokenizer_dir, tiny_config

    from astrai_b200.inference import InferenceEngine
    from astrai_b200.models import AutoRegressiveLM
    from astrai_b200.serialization import Checkpoint
    from astrai_b200.tokenize import AutoTokenizer

    params = tmp_path / "params"
    build_tokenizer_dir(str(params))
    torch.manual_seed(0)
    model = AutoRegressiveLM(tiny_config(vocab_size=512, hidden_size=32, intermediate_size=64, num_attention_heads=4,
                                         num_key_value_heads=2, max_position_embeddings=128)).eval()
    Checkpoint(state_dict=model.state_dict(), config=model.config.to_dict()).save(str(params))
    tok = AutoTokenizer.from_pretrained(params)
    messages = [{"role": "user", "content": "hello"}]
    with InferenceEngine(model, tok, max_batch_size=2, max_seq_len=96, enable_cuda_graph=False) as eng:
        want = eng.generate(tok.apply_chat_template(messages, tokenize=False), max_tokens=6, temperature=0.0)
        want_ids = eng.scheduler.run_batch([tok.encode(tok.apply_chat_template(messages, tokenize=False))], max_tokens=6, temperature=0.0)[0]
    port = 18473
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29779", "-m", "astrai_b200.cli.serve", "--tp_size", "2", "--device", "cpu", "--dtype", "float32",
           "--param_path", str(params), "--host", "127.0.0.1", "--port", str(port), "--max_batch_size", "2", "--max_seq_len", "96",
           "--no-cuda_graph"]
    proc = subprocess.Popen(cmd, env=dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1"), cwd=ROOT,
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, start_new_session=True)
    try:
        deadline = time.time() + 120
        while True:
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=2) as r:
                    if json.load(r).get("model_loaded"):
                        break
            except OSError:
                pass
            assert proc.poll() is None, proc.stdout.read()[-3000:]
            assert time.time() < deadline, "the server did not come up"
            time.sleep(0.5)
        body = json.dumps({"messages": messages, "max_tokens": 6, "temperature": 0.0}).encode()
        req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/chat/completions", data=body, headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=60) as r:
            answer = json.load(r)
        assert answer["choices"][0]["message"]["content"] == want
        # the finish report reaches the first rank's handler through the staged (every-rank) request path too
        assert answer["usage"]["completion_tokens"] == len(want_ids)
        assert answer["choices"][0]["finish_reason"] == ("stop" if want_ids[-1] in tok.stop_ids else "length")
    finally:
        os.killpg(proc.pid, signal.SIGTERM)  # the exact process group started above
        try:
            proc.wait(timeout=30)
        except subprocess.TimeoutExpired:
            os.killpg(proc.pid, signal.SIGKILL)
            proc.wait(timeout=10)
