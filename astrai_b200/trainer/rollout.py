"""Online rollouts for RL training (``online_grpo`` / ``online_dpo``).

Three pieces, matching the roles in the reference (``astrai/trainer/rollout.py:26-421``):

* :class:`RolloutGenerator` turns a prompt batch into ``group_size`` sampled responses per prompt by handing tokenised
  prompts to the inference scheduler's synchronous :meth:`run_batch` (paged KV cache, CUDA-graphed decode, the policy
  model itself as the generator) and packs the results into left-padded prompt / right-padded response tensors;
* :class:`BaseRewardModel` scores decoded text;
* :class:`RolloutRunner` caches the scored rollout per prompt batch and refreshes it every ``rollout_interval``
  optimizer steps; calling it returns ``(result, is_fresh)``.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass, field
from typing import Any, Dict, Hashable, List, Optional, Sequence, Tuple

import torch
from torch import Tensor

PAD_ID = 0  # the strategies treat token id 0 as padding


@dataclass(kw_only=True)
class RawRollout:
    """Sampled responses before scoring.  Shapes: prompts ``[B,P]`` (left padded), responses ``[B,G,R]``."""

    prompts: Tensor
    prompt_mask: Tensor
    responses: Tensor
    response_mask: Tensor
    logprobs_old: Tensor
    prompt_texts: List[str] = field(default_factory=list)
    response_texts: List[List[str]] = field(default_factory=list)


@dataclass(kw_only=True)
class RolloutResult(RawRollout):
    """A :class:`RawRollout` plus one reward per response, ``[B,G]``."""

    rewards: Tensor


class BaseRewardModel(ABC):
    """Maps ``(prompts[B], responses[B][G])`` to a float tensor ``[B,G]``: a learned model, a rule or a remote call."""

    @abstractmethod
    def score(self, prompts: List[str], responses: List[List[str]]) -> Tensor:
        ...


def messages_from_fields(instruction: str = "", user_input: str = "", output: str = "") -> List[Dict[str, str]]:
    """``instruction`` -> system, ``input`` -> user, ``output`` -> assistant; empty fields are dropped."""
    pairs = (("system", instruction), ("user", user_input), ("assistant", output))
    return [{"role": role, "content": text} for role, text in pairs if text]


class RolloutGenerator:
    def __init__(self, scheduler, tokenizer, max_tokens: int = 1024, group_size: int = 8, temperature: float = 1.0,
                 top_k: int = 0, top_p: float = 1.0, frequency_penalty: float = 0.0, rep_window: int = 64):
        self.scheduler, self.tokenizer = scheduler, tokenizer
        self.max_tokens, self.group_size = max_tokens, group_size
        self.sampling = dict(temperature=temperature, top_k=top_k, top_p=top_p, frequency_penalty=frequency_penalty,
                             rep_window=rep_window)

    # -- prompts ---------------------------------------------------------------------------------------------------
    def _conversations(self, batch: Dict[str, Any]) -> List[List[Dict[str, str]]]:
        if "messages" in batch:
            return list(batch["messages"])
        if "instruction" in batch:
            n = len(batch["instruction"])
            inputs = batch.get("input") or [""] * n
            outputs = batch.get("output") or [""] * n
            return [messages_from_fields(i, u, o) for i, u, o in zip(batch["instruction"], inputs, outputs)]
        raise ValueError("a rollout batch needs 'messages' or 'instruction' (with optional 'input' / 'output'); "
                         f"got keys {sorted(batch.keys())}")

    def _render(self, conversations) -> Tuple[List[str], List[List[int]]]:
        """Chat-template every conversation with the generation prompt appended; batched when the tokenizer can."""
        tk = self.tokenizer
        try:
            texts = tk.apply_chat_template(conversations, tokenize=False, add_generation_prompt=True)
            if not (isinstance(texts, list) and len(texts) == len(conversations) and all(isinstance(t, str) for t in texts)):
                raise TypeError("no batched chat template")
            ids = tk.encode(texts)
            if not (len(ids) == len(texts) and all(isinstance(row, list) for row in ids)):
                raise TypeError("no batched encode")
            return texts, [list(row) for row in ids]
        except (TypeError, IndexError, KeyError):
            texts, ids = [], []
            for conv in conversations:
                texts.append(tk.apply_chat_template(conv, tokenize=False, add_generation_prompt=True))
                ids.append(list(tk.apply_chat_template(conv, tokenize=True, add_generation_prompt=True)))
            return texts, ids

    # -- generation ------------------------------------------------------------------------------------------------
    def _policy(self):
        ex = getattr(self.scheduler, "_executor", None)
        return getattr(ex, "model", None)

    @torch.no_grad()
    def generate(self, batch: Dict[str, Any]) -> RawRollout:
        model = self._policy()
        was_training = bool(model.training) if model is not None else False
        if model is not None:
            model.eval()
        try:
            return self._generate(batch)
        finally:
            if model is not None:
                model.train(was_training)

    def _generate(self, batch) -> RawRollout:
        texts, prompt_ids = self._render(self._conversations(batch))
        b, g = len(texts), self.group_size
        requests = [list(ids) for ids in prompt_ids for _ in range(g)]
        results = self.scheduler.run_batch(requests, max_tokens=self.max_tokens, return_logprobs=True, **self.sampling)
        if len(results) != b * g:
            raise RuntimeError(f"the scheduler returned {len(results)} generations for {b * g} requests")
        if any(len(toks) != len(lps) for toks, lps in results):
            raise RuntimeError("token ids and log-probabilities of a generation differ in length")
        dev = self.scheduler.device
        p_len = max(len(ids) for ids in prompt_ids)
        r_len = max(1, max(len(toks) for toks, _ in results))
        prompts = torch.full((b, p_len), PAD_ID, dtype=torch.long)
        prompt_mask = torch.zeros((b, p_len), dtype=torch.bool)
        responses = torch.full((b, g, r_len), PAD_ID, dtype=torch.long)
        response_mask = torch.zeros((b, g, r_len), dtype=torch.bool)
        logprobs = torch.zeros((b, g, r_len), dtype=torch.float32)
        decoded: List[List[str]] = []
        for i, ids in enumerate(prompt_ids):  # prompts are left padded so that responses start at one column
            prompts[i, p_len - len(ids):] = torch.tensor(ids, dtype=torch.long)
            prompt_mask[i, p_len - len(ids):] = True
            row = []
            for j in range(g):
                toks, lps = results[i * g + j]
                n = len(toks)
                if n:
                    responses[i, j, :n] = torch.tensor(toks, dtype=torch.long)
                    response_mask[i, j, :n] = True
                    logprobs[i, j, :n] = torch.tensor(lps, dtype=torch.float32)
                row.append(self.tokenizer.decode(list(toks), skip_special_tokens=True))
            decoded.append(row)
        return RawRollout(prompts=prompts.to(dev), prompt_mask=prompt_mask.to(dev), responses=responses.to(dev),
                          response_mask=response_mask.to(dev), logprobs_old=logprobs.to(dev), prompt_texts=texts,
                          response_texts=decoded)


def _freeze(value) -> Hashable:
    if isinstance(value, dict):
        return tuple(sorted((k, _freeze(v)) for k, v in value.items()))
    if isinstance(value, (list, tuple)):
        return tuple(_freeze(v) for v in value)
    if isinstance(value, Tensor):
        return ("tensor", tuple(value.shape), tuple(value.reshape(-1).tolist()))
    return value


class RolloutRunner:
    """Generation + scoring with a per-batch cache.

    A cached result is reused while the same prompt batch comes back and fewer than ``rollout_interval`` optimizer
    steps (:meth:`step`) have passed since it was generated.
    """

    def __init__(self, generator: RolloutGenerator, reward_model: BaseRewardModel, rollout_interval: int = 512):
        self.generator, self.reward_model = generator, reward_model
        self.rollout_interval = max(int(rollout_interval), 1)
        self._cached: Optional[RolloutResult] = None
        self._key: Optional[Hashable] = None
        self._age = 0

    def step(self):
        self._age += 1

    def clear_cache(self):
        self._cached, self._key = None, None

    def _score(self, raw: RawRollout) -> RolloutResult:
        rewards = self.reward_model.score(raw.prompt_texts, raw.response_texts)
        rewards = torch.as_tensor(rewards, dtype=torch.float32).to(raw.responses.device)
        want = tuple(raw.responses.shape[:2])
        if tuple(rewards.shape) != want:
            raise ValueError(f"the reward model returned shape {tuple(rewards.shape)}, expected {want}")
        return RolloutResult(rewards=rewards, **{f: getattr(raw, f) for f in RawRollout.__dataclass_fields__})

    def __call__(self, batch: Dict[str, Any]) -> Tuple[RolloutResult, bool]:
        key = _freeze(batch)
        stale = self._cached is None or key != self._key or self._age >= self.rollout_interval
        if not stale:
            return self._cached, False
        self._cached = self._score(self.generator.generate(batch))
        self._key, self._age = key, 0
        return self._cached, True
