"""One prompt, one completion."""
from astrai_b200.demo._common import chat_prompt, engine_from_args, sampling


def main():
    engine, tok, args = engine_from_args(__doc__, lambda ap: ap.add_argument("--prompt", default="Tell me a short story."))
    try:
        print(engine.generate(chat_prompt(tok, [{"role": "user", "content": args.prompt}]), **sampling(args)))
    finally:
        engine.shutdown()


if __name__ == "__main__":
    main()
