"""Interactive chat with token streaming (empty line or Ctrl-D to quit)."""
from astrai_b200.demo._common import chat_prompt, engine_from_args, sampling


def main():
    engine, tok, args = engine_from_args(__doc__)
    history = []
    try:
        while True:
            try:
                text = input("you> ").strip()
            except EOFError:
                break
            if not text:
                break
            history.append({"role": "user", "content": text})
            print("bot> ", end="", flush=True)
            reply = ""
            for piece in engine.generate(chat_prompt(tok, history), stream=True, **sampling(args)):
                reply += piece
                print(piece, end="", flush=True)
            print()
            history.append({"role": "assistant", "content": reply})
    finally:
        engine.shutdown()


if __name__ == "__main__":
    main()
