"""Sampling rules on the CPU path (the plain-PyTorch pipeline is also the oracle of the fused GPU sampler)."""

import math

import pytest
import torch

from astrai_b200.inference.runtime.sample import (
    FrequencyPenaltyStrategy, SamplingPipeline, TemperatureStrategy, TopKStrategy, TopPStrategy, sample,
)

NEG = -float("inf")


def _logits(rows=3, vocab=12, seed=0):
    return torch.randn(rows, vocab, generator=torch.Generator().manual_seed(seed))


def test_temperature_divides_and_clamps():
    x = _logits()
    assert torch.equal(TemperatureStrategy(1.0).apply(x), x)
    assert torch.allclose(TemperatureStrategy(2.0).apply(x), x / 2)
    assert torch.isfinite(TemperatureStrategy(0.0).apply(x)).all()  # clamped to 1e-8, not a division by zero
    per_row = TemperatureStrategy(torch.tensor([1.0, 2.0, 4.0])).apply(x)
    assert torch.allclose(per_row[2], x[2] / 4) and torch.allclose(per_row[0], x[0])


@pytest.mark.parametrize("k", [1, 3, 12, 50])
def test_top_k_keeps_exactly_the_k_largest(k):
    x = _logits()
    out = TopKStrategy(k).apply(x)
    kept = (out > NEG).sum(-1)
    assert torch.equal(kept, torch.full((3,), min(k, 12)))
    top = x.topk(min(k, 12), dim=-1).indices
    assert torch.isfinite(out.gather(1, top)).all()


def test_top_k_zero_or_negative_disables():
    x = _logits()
    assert torch.equal(TopKStrategy(0).apply(x), x) and torch.equal(TopKStrategy(-3).apply(x), x)


def test_top_k_per_row_and_ties_stay():
    x = torch.tensor([[3.0, 3.0, 1.0, 0.0], [4.0, 2.0, 1.0, 0.0]])
    out = TopKStrategy(torch.tensor([1, 2])).apply(x)
    assert (out[0] > NEG).tolist() == [True, True, False, False]  # both maxima tie with the threshold: neither is removed
    assert (out[1] > NEG).tolist() == [True, True, False, False]
    mixed = TopKStrategy(torch.tensor([0, 1])).apply(x)          # k = 0 disables the filter for that row only
    assert (mixed[0] > NEG).all() and (mixed[1] > NEG).sum() == 1


def test_top_p_keeps_the_first_token_that_crosses():
    probs = torch.tensor([[0.5, 0.3, 0.15, 0.05]])
    x = probs.log()
    assert (TopPStrategy(0.6).apply(x) > NEG).tolist() == [[True, True, False, False]]   # 0.5 < 0.6: the crossing token stays
    assert (TopPStrategy(0.5).apply(x) > NEG).tolist() == [[True, True, False, False]]   # mass before token 2 is 0.5, not above p
    assert (TopPStrategy(0.45).apply(x) > NEG).tolist() == [[True, False, False, False]]
    assert (TopPStrategy(1.0).apply(x) > NEG).all()


def test_top_p_per_row_values():
    x = torch.tensor([[0.5, 0.3, 0.15, 0.05], [0.5, 0.3, 0.15, 0.05]]).log()
    out = TopPStrategy(torch.tensor([0.45, 0.9])).apply(x)
    assert (out[0] > NEG).sum() == 1 and (out[1] > NEG).sum() == 3


def test_top_p_is_order_independent():
    x = torch.tensor([[0.05, 0.5, 0.15, 0.3]]).log()
    assert (TopPStrategy(0.6).apply(x) > NEG).tolist() == [[False, True, False, True]]


def test_frequency_penalty_counts_occurrences():
    x = torch.zeros(1, 6)
    hist = torch.tensor([[2, 2, 5, 0]])
    mask = torch.tensor([[1, 1, 1, 0]]).bool()   # the trailing 0 is padding, not token 0
    out = FrequencyPenaltyStrategy(0.5).apply(x, input_ids=hist, input_mask=mask)
    assert out.tolist() == [[0.0, 0.0, -1.0, 0.0, 0.0, -0.5]]
    assert torch.equal(FrequencyPenaltyStrategy(0.0).apply(x, input_ids=hist, input_mask=mask), x)


def test_all_zero_temperature_is_argmax_of_the_raw_logits():
    x = _logits(4, 20, seed=3)
    got = sample(x, temperature=0.0, top_k=1, top_p=0.1)
    assert torch.equal(got.view(-1), x.argmax(-1))
    tok, logp = sample(x, temperature=torch.zeros(4), return_logprobs=True)
    assert torch.equal(tok.view(-1), x.argmax(-1)) and logp.shape[0] == 4


def test_top_k_one_is_deterministic_at_any_temperature():
    x = _logits(5, 30, seed=4)
    g = torch.Generator().manual_seed(0)
    assert torch.equal(sample(x, temperature=1.7, top_k=1, generator=g).view(-1), x.argmax(-1))


def test_sampled_tokens_respect_the_filters():
    x = _logits(64, 50, seed=5)
    g = torch.Generator().manual_seed(1)
    tok = sample(x, temperature=1.0, top_k=5, top_p=0.9, generator=g).view(-1)
    top5 = x.topk(5, dim=-1).indices
    assert all(int(t) in top5[i].tolist() for i, t in enumerate(tok))


def test_logprob_is_taken_from_the_filtered_distribution():
    x = torch.tensor([[2.0, 1.0, 0.0, -1.0]])
    g = torch.Generator().manual_seed(0)
    tok, logp = sample(x, temperature=1.0, top_k=2, return_logprobs=True, generator=g)
    kept = torch.log_softmax(torch.tensor([2.0, 1.0]), dim=-1)
    assert math.isclose(float(logp.view(-1)[0]), float(kept[int(tok.view(-1)[0])]), rel_tol=1e-5)


def test_same_generator_seed_same_draws():
    x = _logits(8, 100, seed=6)
    a = sample(x, temperature=1.0, top_k=20, generator=torch.Generator().manual_seed(7))
    b = sample(x, temperature=1.0, top_k=20, generator=torch.Generator().manual_seed(7))
    assert torch.equal(a, b)


def test_empirical_distribution_matches_softmax():
    x = torch.tensor([[1.0, 0.0, -1.0, -2.0]]).repeat(4000, 1)
    tok = sample(x, temperature=1.0, top_k=0, top_p=1.0, generator=torch.Generator().manual_seed(11)).view(-1)
    freq = torch.bincount(tok, minlength=4).float() / tok.numel()
    assert torch.allclose(freq, torch.softmax(x[0], -1), atol=0.03)


def test_pipeline_order_is_temperature_then_k_then_p():
    x = torch.tensor([[4.0, 3.0, 2.0, 1.0]])
    pipe = SamplingPipeline([TemperatureStrategy(0.5), TopKStrategy(3), TopPStrategy(0.99)])
    out = pipe.apply(x)
    assert (out > NEG).tolist() == [[True, True, True, False]] and torch.allclose(out[0, :3], x[0, :3] * 2)


def test_hints_avoid_device_reads_but_do_not_change_results():
    x = _logits(6, 40, seed=8)
    ks = torch.full((6,), 7)
    a = sample(x, 0.9, ks, 0.8, generator=torch.Generator().manual_seed(2))
    b = sample(x, 0.9, ks, 0.8, generator=torch.Generator().manual_seed(2),
               hints={"max_k": 7, "top_p_active": True, "has_freq": False, "greedy": False})
    assert torch.equal(a, b)


def test_custom_filter_value():
    x = _logits(2, 8, seed=9)
    out = TopKStrategy(2).apply(x, filter_value=-1e4)
    assert (out == -1e4).sum() == 12 and torch.isfinite(out).all()


# ---- edges of the individual rules --------------------------------------------------------------------------------------
def test_rules_that_are_switched_off_return_their_input_untouched():
    x = _logits()
    assert TemperatureStrategy(1.0).apply(x) is x
    assert TopKStrategy(0).apply(x) is x
    assert TopPStrategy(1.0).apply(x) is x
    assert TopPStrategy(torch.ones(3)).apply(x) is x
    assert FrequencyPenaltyStrategy(0.0).apply(x, input_ids=torch.zeros(3, 2, dtype=torch.long)) is x
    assert FrequencyPenaltyStrategy(1.5).apply(x) is x  # nothing was generated yet


def test_top_p_zero_keeps_only_the_most_likely_token():
    x = _logits(rows=4, vocab=9, seed=3)
    out = TopPStrategy(0.0).apply(x)
    kept = torch.isfinite(out)
    assert kept.sum(-1).tolist() == [1, 1, 1, 1] and torch.equal(out.argmax(-1), x.argmax(-1))


def test_top_k_larger_than_the_vocabulary_keeps_everything():
    x = _logits(vocab=5)
    assert torch.equal(TopKStrategy(50).apply(x), x)
    assert torch.equal(TopKStrategy(torch.tensor([50, 50, 50])).apply(x), x)


def test_frequency_penalty_ignores_padded_history_and_follows_the_sign():
    x = torch.zeros(2, 6)
    history = torch.tensor([[1, 1, 4, 0], [2, 0, 0, 0]])
    valid = torch.tensor([[1, 1, 1, 0], [1, 0, 0, 0]], dtype=torch.bool)
    out = FrequencyPenaltyStrategy(0.5).apply(x, input_ids=history, input_mask=valid)
    assert out[0].tolist() == [0.0, -1.0, 0.0, 0.0, -0.5, 0.0]  # token 1 twice, token 4 once; the padding zero is not counted
    assert out[1].tolist() == [0.0, 0.0, -0.5, 0.0, 0.0, 0.0]
    unmasked = FrequencyPenaltyStrategy(0.5).apply(x, input_ids=history)
    assert unmasked[0, 0].item() == -0.5 and unmasked[1, 0].item() == -1.5  # without a mask every entry counts
    boosted = FrequencyPenaltyStrategy(-1.0).apply(x, input_ids=history, input_mask=valid)
    assert boosted[0, 1].item() == 2.0 and boosted[0, 4].item() == 1.0  # a negative penalty favours repeats
    per_row = FrequencyPenaltyStrategy(torch.tensor([1.0, 0.0])).apply(x, input_ids=history, input_mask=valid)
    assert per_row[0, 1].item() == -2.0 and per_row[1].abs().sum().item() == 0.0


def test_penalty_in_the_pipeline_changes_what_greedy_like_sampling_picks():
    x = torch.tensor([[2.0, 1.9, 0.0, 0.0]])
    history = torch.tensor([[0, 0, 0]])
    plain = sample(x, temperature=1.0, top_k=1)
    penalised = sample(x, temperature=1.0, top_k=0, top_p=1.0, frequency_penalty=100.0, input_ids=history,
                       generator=torch.Generator().manual_seed(0))
    assert plain.item() == 0 and penalised.item() != 0
    # top-k runs BEFORE the penalty: with k = 1 the only survivor is token 0, whatever its penalty
    assert sample(x, temperature=1.0, top_k=1, frequency_penalty=100.0, input_ids=history).item() == 0


def test_logprobs_are_log_probabilities_of_the_returned_tokens():
    x = _logits(rows=5, vocab=20, seed=9)
    g = torch.Generator().manual_seed(4)
    tokens, logp = sample(x, temperature=0.7, top_k=6, top_p=0.9, return_logprobs=True, generator=g)
    assert tokens.shape == logp.shape == (5,) and (logp <= 0).all() and torch.isfinite(logp).all()
    filtered = SamplingPipeline([TemperatureStrategy(0.7), TopKStrategy(6), TopPStrategy(0.9)]).apply(x.float())
    assert torch.allclose(logp, torch.log_softmax(filtered, -1).gather(-1, tokens[:, None])[:, 0], atol=1e-6)
    greedy_tokens, greedy_logp = sample(x, temperature=0.0, return_logprobs=True)
    assert torch.equal(greedy_tokens, x.argmax(-1))
    assert torch.allclose(greedy_logp, torch.log_softmax(x, -1).max(-1).values, atol=1e-6)  # of the RAW distribution


def test_mixed_zero_and_positive_temperatures_are_not_the_greedy_shortcut():
    x = torch.tensor([[0.0, 5.0, 1.0], [0.0, 5.0, 1.0]])
    out = sample(x, temperature=torch.tensor([0.0, 1.0]), generator=torch.Generator().manual_seed(0))
    assert out[0].item() == 1  # a zero temperature is clamped to 1e-8: that row is as good as argmax
