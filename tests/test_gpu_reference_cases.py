"""The reference's own sampler tests (crates/llm-core/src/generate.rs:443-480, :550-583,
:629-692), run against the CUDA path through the one-row host entry points that mirror
`sample_with` / `sample`."""
import numpy as np
import pytest

import scriptonait_b200 as sb
from scriptonait_b200 import Rng, SamplingConfig

pytestmark = pytest.mark.gpu


def test_top_k_restricts_the_choice_to_the_k_best(sampler):
    logits = [0.0, 5.0, 0.0, 9.0, 0.0]
    cfg = SamplingConfig(temperature=5.0, top_k=2, top_p=1.0, repetition_penalty=1.0)
    seen = set()
    for seed in range(50):
        picked = sampler.sample_with(logits, cfg, [], Rng.seed_from_u64(seed))
        assert picked in (3, 1), f"top_k leaked token {picked}"
        seen.add(picked)
    assert seen == {1, 3}


def test_top_p_keeps_the_nucleus(sampler):
    cfg = SamplingConfig(temperature=1.0, top_k=0, top_p=0.9, repetition_penalty=1.0)
    for seed in range(20):
        assert sampler.sample_with([20.0, 0.0, 0.0, 0.0], cfg, [], Rng.seed_from_u64(seed)) == 0


def test_repetition_penalty_pushes_recent_tokens_down(sampler):
    greedy = SamplingConfig(temperature=0.0, repetition_penalty=1.5)
    rng = Rng.seed_from_u64(1)
    assert sampler.sample_with([2.0, 1.9, 0.0], greedy, [], rng) == 0
    assert sampler.sample_with([2.0, 1.9, 0.0], greedy, [0], rng) == 1
    assert rng.state == 1


def test_min_p_cuts_the_tail_of_a_confident_step(sampler):
    cfg = SamplingConfig(temperature=1.0, top_k=0, top_p=1.0, min_p=0.1, repetition_penalty=1.0)
    rng = Rng.seed_from_u64(1)
    for _ in range(64):
        assert sampler.sample_with([6.0] + [0.0] * 7, cfg, [], rng) == 0


def test_min_p_keeps_the_field_when_the_model_is_unsure(sampler):
    cfg = SamplingConfig(temperature=1.0, top_k=0, top_p=1.0, min_p=0.1, repetition_penalty=1.0)
    rng = Rng.seed_from_u64(2)
    seen = [False] * 5
    for _ in range(500):
        seen[sampler.sample_with([0.10, 0.05, 0.0, -0.05, -0.10], cfg, [], rng)] = True
    assert all(seen)


def test_min_p_always_leaves_a_candidate(sampler):
    cfg = SamplingConfig(temperature=1.0, top_k=0, top_p=1.0, min_p=5.0, repetition_penalty=1.0)
    assert sampler.sample_with([1.0, 0.9, 0.8], cfg, [], Rng.seed_from_u64(3)) == 0


def test_defaults_match_the_reference():
    d = SamplingConfig()
    assert (d.temperature, d.top_k, d.top_p, d.min_p, d.repetition_penalty, d.repetition_window, d.seed, d.allowed) == \
        (0.9, 40, 0.95, 0.0, 1.1, 128, 0, None)
    import ctypes
    c = sb.native.SamplingConfigC()
    sb.native.load().llm_cuda_sampling_config_default(ctypes.byref(c))
    assert (round(c.temperature, 6), c.top_k, round(c.top_p, 6), c.min_p, round(c.repetition_penalty, 6),
            c.repetition_window, c.seed, c.allowed) == (0.9, 40, 0.95, 0.0, 1.1, 128, 0, None)


def test_deterministic_given_same_seed_and_greedy_ignores_the_seed(sampler):
    g = np.random.default_rng(0)
    logits = g.normal(0, 2, 700).astype(np.float32)
    cfg = SamplingConfig(temperature=0.8)
    a = [sampler.sample_with(logits, cfg, [1, 2, 3], Rng(123)) for _ in range(3)]
    assert len(set(a)) == 1
    greedy = SamplingConfig(temperature=0.0, repetition_penalty=1.0)
    assert sampler.sample_with(logits, greedy, [], Rng(1)) == sampler.sample_with(logits, greedy, [], Rng(999)) == int(np.argmax(logits))


def test_plain_sample_matches_sample_with_everything_off(sampler):
    import oracle
    g = np.random.default_rng(2)
    logits = g.normal(0, 2, 400).astype(np.float32)
    for seed in range(10):
        r1, r2, r3 = Rng(seed), Rng(seed), oracle.Rng(seed)
        a = sampler.sample(logits, 0.7, r1)
        b = sampler.sample_with(logits, SamplingConfig(temperature=0.7, top_k=0, top_p=1.0, min_p=0.0, repetition_penalty=1.0), [], r2)
        c = oracle.sample(logits, 0.7, r3, exp_mode=oracle.EXP_CR)
        assert a == b == c and r1.state == r2.state == r3.state


def test_module_level_sample_with_uses_the_default_sampler():
    assert sb.sample_with([0.0, 9.0, 1.0], SamplingConfig(temperature=0.0, repetition_penalty=1.0), [], Rng(0)) == 1


def test_host_rng_mirror_matches_the_oracle_stream():
    import oracle
    a, b = Rng(1234), oracle.Rng(1234)
    for _ in range(100):
        assert a.next_u64() == b.next_u64()
    assert Rng(5).next_f32() == oracle.Rng(5).next_f32()
