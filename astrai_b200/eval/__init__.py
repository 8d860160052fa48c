"""Evaluation entry points: ``python -m astrai_b200.eval.{ppl,mmlu,humaneval,ifeval,ifd,rouge,analyze_weights}``.

Counterparts of the reference's ``scripts/eval/*.py``.  Scoring runs through the training forward of the model
(causal, no cache) with fused log-prob extraction; generation-based evals go through :class:`InferenceEngine`.
Datasets are read from local files only.
"""
