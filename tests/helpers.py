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
