from __future__ import annotations

import argparse

import torch


def engine_from_args(description: str, extra=None):
    ap = argparse.ArgumentParser(description=description)
    ap.add_argument("--param_path", default="params")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--max_seq_len", type=int, default=2048)
    ap.add_argument("--max_batch_size", type=int, default=8)
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--top_p", type=float, default=0.95)
    ap.add_argument("--top_k", type=int, default=50)
    ap.add_argument("--max_tokens", type=int, default=256)
    if extra:
        extra(ap)
    args = ap.parse_args()
    from astrai_b200.inference import InferenceEngine
    from astrai_b200.models import AutoModel
    from astrai_b200.tokenize import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(args.param_path)
    dtype = torch.bfloat16 if args.device.startswith("cuda") else torch.float32
    model = AutoModel.from_pretrained(args.param_path).to(device=args.device, dtype=dtype).eval()
    return InferenceEngine(model, tok, max_batch_size=args.max_batch_size, max_seq_len=args.max_seq_len), tok, args


def chat_prompt(tok, messages):
    return tok.apply_chat_template(messages, tokenize=False, add_generation_prompt=True)


def sampling(args):
    return dict(max_tokens=args.max_tokens, temperature=args.temperature, top_p=args.top_p, top_k=args.top_k)
