"""Worker of the tensor-parallel serving test: every rank builds the same small decoder, the scheduler cuts it over the
ranks and runs in lockstep; the first rank submits prompts (streaming callbacks, a cancelled request, a synchronous
``run_batch``) and writes what it got next to what one process generates alone.  Runs on gloo ranks (CPU) or NCCL ranks
(GPU); launched by torchrun."""

import argparse
import json
import os
import sys
import threading

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402


class Tok:
    stop_ids = [1]

    def encode(self, text):
        return [ord(c) % 200 + 3 for c in text]

    def decode(self, ids, skip_special_tokens=True):
        return "".join(f"<{i}>" for i in ids)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--moe", action="store_true")
    args = ap.parse_args()

    from astrai_b200.config import AutoRegressiveLMConfig
    from astrai_b200.inference import InferenceEngine, InferenceScheduler
    from astrai_b200.inference.task import STOP
    from astrai_b200.models import AutoRegressiveLM
    from astrai_b200.parallel.setup import setup_parallel

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    cuda = args.device == "cuda"
    dtype = torch.bfloat16 if cuda else torch.float32
    extra = dict(ffn_type="moe", n_routed_experts=4, n_shared_experts=1, n_activated_experts=2, moe_intermediate_size=128) if args.moe else {}
    cfg = AutoRegressiveLMConfig(vocab_size=512, hidden_size=256 if cuda else 64, num_hidden_layers=2, rms_norm_eps=1e-6,
                                 intermediate_size=512 if cuda else 128, tie_word_embeddings=True, max_position_embeddings=256,
                                 rope_theta=10000.0, num_attention_heads=4, num_key_value_heads=2, **extra)
    prompts = [[10 + 3 * i + j for j in range(4 + 5 * i)] for i in range(5)]
    with setup_parallel(rank, world, local, "nccl" if cuda else "gloo", os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"],
                        "cuda" if cuda else "cpu"):
        dev = torch.device("cuda", local) if cuda else torch.device("cpu")

        def build():
            torch.manual_seed(5)
            return AutoRegressiveLM(cfg).to(dev, dtype).eval()

        alone = None
        if rank == 0:  # the single-process answer, before any sharding
            solo = InferenceScheduler(build(), Tok(), max_batch_size=8, max_seq_len=128, enable_cuda_graph=False, page_size=4)
            alone = solo.run_batch(prompts, max_tokens=10, temperature=0.0)
        eng = InferenceEngine(build(), Tok(), max_batch_size=8, max_seq_len=128, enable_cuda_graph=cuda, page_size=4, tp_size=world)
        heads = eng.scheduler._executor.model.layers[0].attention.n_heads
        pool_heads = eng.scheduler.cache.storage.k_buffer.shape[2]
        if rank != 0:
            eng.follow()
            return
        streams = {i: [] for i in range(len(prompts))}
        done = {i: threading.Event() for i in range(len(prompts))}

        def cb(i):
            def f(piece):
                if piece is STOP:
                    done[i].set()
                else:
                    streams[i].append(piece)
            return f

        ids = [eng.scheduler.add_task(p, max_tokens=10, temperature=0.0, stream_callback=cb(i)) for i, p in enumerate(prompts)]
        cancelled = eng.scheduler.add_task([7] * 6, max_tokens=100, temperature=0.0, stream_callback=lambda piece: None)
        eng.scheduler.remove_task(cancelled)
        ok = all(ev.wait(timeout=120) for ev in done.values())
        sampled = eng.generate("hello tensor parallel", max_tokens=6, temperature=0.9, top_k=20)
        import time

        for _ in range(200):  # the finished request leaves the active list at the start of the next loop iteration
            stats = eng.get_stats()
            if stats["active_tasks"] == 0:
                break
            time.sleep(0.01)
        eng.shutdown()
        got = ["".join(streams[i]) for i in range(len(prompts))]
        want = ["".join(f"<{t}>" for t in toks) for toks in alone]
        with open(args.out, "w") as fh:
            json.dump({"finished": ok, "got": got, "want": want, "local_heads": heads, "pool_heads": pool_heads,
                       "sampled_pieces": sampled.count("<"), "active": stats["active_tasks"], "n_ids": len(set(ids))}, fh)


if __name__ == "__main__":
    main()
