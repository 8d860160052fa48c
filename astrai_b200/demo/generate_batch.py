"""Several prompts through the continuous-batching scheduler at once."""
from astrai_b200.demo._common import chat_prompt, engine_from_args, sampling

PROMPTS = ["What is the capital of France?", "Write a haiku about autumn.", "Explain what a GPU is in one sentence.",
           "Give me three names for a cat."]


def main():
    engine, tok, args = engine_from_args(__doc__)
    try:
        outs = engine.generate([chat_prompt(tok, [{"role": "user", "content": p}]) for p in PROMPTS], **sampling(args))
        for p, o in zip(PROMPTS, outs):
            print(f"> {p}\n{o}\n")
    finally:
        engine.shutdown()


if __name__ == "__main__":
    main()
