"""Shared fixtures: tiny model config, a character-level BPE tokenizer built in-test, random token data."""

import json
import os

import torch

TINY = dict(vocab_size=1000, hidden_size=8, num_hidden_layers=2, rms_norm_eps=1e-5, intermediate_size=16,
            tie_word_embeddings=False, max_position_embeddings=64, rope_theta=10000.0, num_attention_heads=2,
            num_key_value_heads=1)

CHAT_TEMPLATE = ("{% for m in messages %}<|im_start|>{{ m['role'] }}\n{{ m['content'] }}<|im_end|>\n{% endfor %}"
                 "{% if add_generation_prompt %}<|im_start|>assistant\n{% endif %}")
SPECIAL = {"bos_token": "<|bos|>", "eos_token": "<|im_end|>", "pad_token": "<|pad|>", "im_start": "<|im_start|>"}


def tiny_config(**over):
    from astrai_b200.config import AutoRegressiveLMConfig

    return AutoRegressiveLMConfig(**{**TINY, **over})


def build_tokenizer_dir(path: str) -> str:
    """Train a small BPE tokenizer over single characters and write tokenizer.json + tokenizer_config.json."""
    from tokenizers import Tokenizer, models, pre_tokenizers, trainers, decoders

    tk = Tokenizer(models.BPE(unk_token="<|unk|>"))
    tk.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tk.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=400, special_tokens=["<|unk|>"] + list(SPECIAL.values()),
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    corpus = [chr(c) for c in range(32, 127)] + ["hello world", "the quick brown fox", "user assistant system"]
    tk.train_from_iterator(corpus, trainer)
    os.makedirs(path, exist_ok=True)
    tk.save(os.path.join(path, "tokenizer.json"))
    with open(os.path.join(path, "tokenizer_config.json"), "w") as fh:
        json.dump({"special_tokens": SPECIAL, "chat_template": CHAT_TEMPLATE}, fh)
    return path


class RandomTokens(torch.utils.data.Dataset):
    def __init__(self, n=32, seq=16, vocab=1000, seed=0, fail_after=None):
        g = torch.Generator().manual_seed(seed)
        self.data = torch.randint(1, vocab, (n, seq + 1), generator=g)
        self.fail_after = fail_after
        self.served = 0

    def __len__(self):
        return self.data.shape[0]

    def __getitem__(self, i):
        self.served += 1
        if self.fail_after is not None and self.served > self.fail_after:
            raise RuntimeError("injected data failure")
        row = self.data[i]
        return {"input_ids": row[:-1], "target_ids": row[1:]}


def launch_ranks(nproc: int, script: str, args, port: int, timeout: float = 600.0, env=None, cwd=None):
    """Run ``script`` as ``nproc`` rank processes on this machine (RANK / WORLD_SIZE / LOCAL_RANK / MASTER_* in their
    environment, as an external launcher sets them) and wait for all of them.  Returns ``(returncode, output)``: the first
    non-zero exit code (0 if none) and every rank's output.  Starting the ranks directly instead of through
    ``torch.distributed.run`` saves that launcher's own start-up in every test; the tests that are about the launcher use it."""
    import socket
    import subprocess
    import sys
    import time

    # the asked-for port if it can be had; otherwise (a run a moment ago still holds it) one the system picks
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as probe:
        try:
            probe.bind(("127.0.0.1", int(port)))
        except OSError:
            probe.bind(("127.0.0.1", 0))
            port = probe.getsockname()[1]
    base = dict(os.environ if env is None else env, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(nproc),
                LOCAL_WORLD_SIZE=str(nproc))
    base.setdefault("OMP_NUM_THREADS", "1")
    procs = []
    for rank in range(nproc):
        rank_env = dict(base, RANK=str(rank), LOCAL_RANK=str(rank))
        procs.append(subprocess.Popen([sys.executable, script, *map(str, args)], env=rank_env, cwd=cwd, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    deadline = time.time() + timeout
    code, outputs = 0, []
    for rank, p in enumerate(procs):
        try:
            out, _ = p.communicate(timeout=max(deadline - time.time(), 1.0))
        except subprocess.TimeoutExpired:
            for q in procs:  # the exact processes started above
                if q.poll() is None:
                    q.kill()
            out, _ = p.communicate()
            out = (out or "") + f"\n[rank {rank}: killed after {timeout:.0f} s]"
            code = code or -9
        outputs.append(f"--- rank {rank} (exit {p.returncode}) ---\n{(out or '')[-3000:]}")
        if p.returncode and not code:
            code = p.returncode
    return code, "\n".join(outputs)
