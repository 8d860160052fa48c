"""Spectral statistics of a checkpoint's weight matrices (reference: ``scripts/eval/analyze_weights.py``).

For every 2-D weight: effective rank ``exp(H(p))`` with ``p = s / sum(s)`` over the singular values, stable rank
``||W||_F^2 / ||W||_2^2``, the fraction of singular values that carries 90 % of the energy, mean and std.
"""

from __future__ import annotations

import argparse
from typing import Dict

import torch

from astrai_b200.eval.common import save_json


def effective_rank_metrics(w: torch.Tensor, device: str = "cpu") -> Dict[str, float]:
    m = w.detach().to(device=device, dtype=torch.float32)
    s = torch.linalg.svdvals(m)
    p = s / s.sum().clamp_min(1e-30)
    entropy = -(p * torch.log(p.clamp_min(1e-30))).sum()
    energy = torch.cumsum(s * s, 0) / (s * s).sum().clamp_min(1e-30)
    k90 = int((energy < 0.9).sum().item()) + 1
    return {"shape": list(w.shape), "effective_rank": float(torch.exp(entropy)), "stable_rank": float((s * s).sum() / (s[0] * s[0]).clamp_min(1e-30)),
            "rank90_fraction": k90 / s.numel(), "max_rank": int(s.numel()), "mean": float(m.mean()), "std": float(m.std()),
            "spectral_norm": float(s[0])}


def analyze(state_dict: Dict[str, torch.Tensor], device: str = "cpu", name_filter: str = "") -> Dict[str, Dict]:
    return {k: effective_rank_metrics(v, device) for k, v in state_dict.items() if v.dim() == 2 and name_filter in k}


def main(argv=None):
    ap = argparse.ArgumentParser(description="Effective-rank analysis of a model directory")
    ap.add_argument("--param_path", required=True)
    ap.add_argument("--filter", default="", help="substring a parameter name must contain")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--output", default=None)
    a = ap.parse_args(argv)
    from astrai_b200.serialization import load_model_weights

    res = analyze(load_model_weights(a.param_path), a.device, a.filter)
    for name, m in res.items():
        print(f"{name:60s} {str(m['shape']):16s} eff_rank {m['effective_rank']:8.1f} / {m['max_rank']:5d}  stable {m['stable_rank']:7.1f}  r90 {m['rank90_fraction']:.2f}")
    save_json(a.output, res)
    return res


if __name__ == "__main__":
    main()
