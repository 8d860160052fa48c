"""Fetch a released checkpoint from the Hugging Face hub into ``--out`` (needs network access and ``huggingface_hub``).

The reference's demo downloads ``ViperEkura/AstrAI-V1-instruct`` (``scripts/demo/download.py``); the directory layout it
produces (``config.json``, ``model.safetensors``, ``tokenizer.json``, ``tokenizer_config.json``) loads here unchanged."""
import argparse


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--repo_id", default="ViperEkura/AstrAI-V1-instruct")
    ap.add_argument("--out", default="params")
    args = ap.parse_args()
    try:
        from huggingface_hub import snapshot_download
    except ImportError as exc:  # pragma: no cover - optional dependency
        raise SystemExit("huggingface_hub is not installed; copy the model directory by hand") from exc
    print(snapshot_download(repo_id=args.repo_id, local_dir=args.out))


if __name__ == "__main__":
    main()
