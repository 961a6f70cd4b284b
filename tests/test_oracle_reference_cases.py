"""The reference's own sampler, RNG and bf16 tests, restated against the oracle.

Each test names the reference test it restates (crates/llm-core/src/generate.rs,
rng.rs, bf16.rs). These are what pins the oracle; both exp definitions must pass.
"""
import numpy as np
import pytest

import oracle
from oracle import Rng, SamplingConfig, sample_with

EXP_MODES = [oracle.EXP_LIBM, oracle.EXP_CR]


@pytest.mark.parametrize("exp_mode", EXP_MODES)
def test_top_k_restricts_the_choice_to_the_k_best(exp_mode):
    # generate.rs:550-561
    logits = np.array([0.0, 5.0, 0.0, 9.0, 0.0], np.float32)
    cfg = SamplingConfig(temperature=5.0, top_k=2, top_p=1.0, repetition_penalty=1.0)
    seen = set()
    for seed in range(50):
        picked = sample_with(logits, cfg, [], Rng.seed_from_u64(seed), exp_mode)
        assert picked in (3, 1), f"top_k leaked token {picked}"
        seen.add(picked)
    assert seen == {1, 3}


@pytest.mark.parametrize("exp_mode", EXP_MODES)
def test_top_p_keeps_the_nucleus(exp_mode):
    # generate.rs:563-573
    logits = np.array([20.0, 0.0, 0.0, 0.0], np.float32)
    cfg = SamplingConfig(temperature=1.0, top_k=0, top_p=0.9, repetition_penalty=1.0)
    for seed in range(20):
        assert sample_with(logits, cfg, [], Rng.seed_from_u64(seed), exp_mode) == 0


def test_repetition_penalty_pushes_recent_tokens_down():
    # generate.rs:575-583
    logits = np.array([2.0, 1.9, 0.0], np.float32)
    greedy = SamplingConfig(temperature=0.0, repetition_penalty=1.5)
    rng = Rng.seed_from_u64(1)
    assert sample_with(logits, greedy, [], rng) == 0
    assert sample_with(logits, greedy, [0], rng) == 1
    assert rng.state == 1, "greedy decoding consumes no RNG output"


@pytest.mark.parametrize("exp_mode", EXP_MODES)
def test_min_p_cuts_the_tail_of_a_confident_step(exp_mode):
    # generate.rs:631-648
    logits = np.array([6.0] + [0.0] * 7, np.float32)
    cfg = SamplingConfig(temperature=1.0, top_k=0, top_p=1.0, min_p=0.1, repetition_penalty=1.0)
    rng = Rng.seed_from_u64(1)
    for _ in range(64):
        assert sample_with(logits, cfg, [], rng, exp_mode) == 0


@pytest.mark.parametrize("exp_mode", EXP_MODES)
def test_min_p_keeps_the_field_when_the_model_is_unsure(exp_mode):
    # generate.rs:652-669
    logits = np.array([0.10, 0.05, 0.0, -0.05, -0.10], np.float32)
    cfg = SamplingConfig(temperature=1.0, top_k=0, top_p=1.0, min_p=0.1, repetition_penalty=1.0)
    rng = Rng.seed_from_u64(2)
    seen = [False] * 5
    for _ in range(500):
        seen[sample_with(logits, cfg, [], rng, exp_mode)] = True
    assert all(seen)


@pytest.mark.parametrize("exp_mode", EXP_MODES)
def test_min_p_always_leaves_a_candidate(exp_mode):
    # generate.rs:672-685
    logits = np.array([1.0, 0.9, 0.8], np.float32)
    cfg = SamplingConfig(temperature=1.0, top_k=0, top_p=1.0, min_p=5.0, repetition_penalty=1.0)
    assert sample_with(logits, cfg, [], Rng.seed_from_u64(3), exp_mode) == 0


def test_min_p_is_off_unless_asked_for():
    # generate.rs:689-692, and the rest of Default (generate.rs:82-95)
    d = SamplingConfig()
    assert d.min_p == 0.0
    assert (d.temperature, d.top_k, d.top_p, d.repetition_penalty, d.repetition_window, d.seed, d.allowed) == \
        (0.9, 40, 0.95, 1.1, 128, 0, None)


def test_sampling_is_deterministic_given_same_seed():
    # generate.rs:443-451 restated at sampler level
    g = np.random.default_rng(0)
    logits = g.normal(0, 2, 512).astype(np.float32)
    cfg = SamplingConfig(temperature=0.8)
    a = [sample_with(logits, cfg, [1, 2, 3], Rng.seed_from_u64(123)) for _ in range(3)]
    assert len(set(a)) == 1
    ra, rb = Rng.seed_from_u64(123), Rng.seed_from_u64(123)
    assert [sample_with(logits, cfg, [], ra) for _ in range(10)] == [sample_with(logits, cfg, [], rb) for _ in range(10)]


def test_temperature_zero_is_deterministic_across_seeds():
    # generate.rs:472-480 restated at sampler level
    g = np.random.default_rng(1)
    logits = g.normal(0, 2, 300).astype(np.float32)
    cfg = SamplingConfig(temperature=0.0, repetition_penalty=1.0)
    assert sample_with(logits, cfg, [], Rng.seed_from_u64(1)) == sample_with(logits, cfg, [], Rng.seed_from_u64(999))
    assert sample_with(logits, cfg, [], Rng.seed_from_u64(1)) == int(np.argmax(logits))


def test_plain_sample_is_temperature_only():
    # generate.rs:423-433
    g = np.random.default_rng(2)
    logits = g.normal(0, 2, 200).astype(np.float32)
    cfg = SamplingConfig(temperature=0.7, top_k=0, top_p=1.0, min_p=0.0, repetition_penalty=1.0)
    for seed in range(10):
        assert oracle.sample(logits, 0.7, Rng(seed)) == sample_with(logits, cfg, [], Rng(seed))


# ---- rng.rs:48-80 -----------------------------------------------------------
def test_rng_same_seed_same_stream_and_seeds_differ():
    a, b, c = Rng(1), Rng(1), Rng(2)
    sa = [a.next_u64() for _ in range(16)]
    assert sa == [b.next_u64() for _ in range(16)]
    assert sa != [c.next_u64() for _ in range(16)]


def test_rng_next_f32_in_unit_interval_on_the_24_bit_grid():
    r = Rng(7)
    for _ in range(2000):
        u = r.next_f32()
        assert 0.0 <= u < 1.0
        assert (u * 2 ** 24) == int(u * 2 ** 24)


def _splitmix_reference(seed, n):
    """rng.rs:16-22 evaluated with Python big integers (independent of the C++)."""
    m = (1 << 64) - 1
    s, out = seed, []
    for _ in range(n):
        s = (s + 0x9E3779B97F4A7C15) & m
        z = s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
        out.append(z ^ (z >> 31))
    return out


@pytest.mark.parametrize("seed", [0, 1, 1234, 2 ** 53 - 1, 2 ** 64 - 1])
def test_rng_matches_big_integer_evaluation(seed):
    r = Rng(seed)
    assert [r.next_u64() for _ in range(64)] == _splitmix_reference(seed, 64)


def test_rng_derived_check_values():
    assert _splitmix_reference(0, 3) == [0xe220a8397b1dcdaf, 0x6e789e6aa1b965f4, 0x06c45d188009454f]
    assert _splitmix_reference(1234, 3) == [0xbb0cf61b2f181cdb, 0x97c7a1364df06524, 0x33befae49bc025da]
    r = Rng(1234)
    assert [r.next_f32() * 2 ** 24 for _ in range(3)] == [12258550.0, 9947041.0, 3391226.0]


# ---- bf16.rs:31-43 ----------------------------------------------------------
def test_bf16_round_trips_within_its_precision():
    vals = np.array([0.0, 1.0, -1.0, 0.5, -0.017, 3.4e30, -2.1e-30, np.finfo(np.float32).tiny], np.float32)
    back = oracle.from_bf16(oracle.to_bf16(vals))
    assert np.all(np.abs(back - vals) <= np.abs(vals) * 0.01 + 1e-38)
    assert np.isnan(oracle.from_bf16(oracle.to_bf16(np.array([np.nan], np.float32)))[0])
    assert oracle.from_bf16(oracle.to_bf16(np.array([np.inf], np.float32)))[0] == np.inf


def test_bf16_narrowing_is_round_to_nearest_even():
    from scriptonait_b200 import workloads
    g = np.random.default_rng(3)
    x = np.concatenate([g.normal(0, 5, 20000).astype(np.float32),
                        np.array([1.00390625, 1.01171875, -1.00390625, 0.0, -0.0, np.inf, -np.inf], np.float32)])
    assert np.array_equal(oracle.to_bf16(x), workloads.narrow_bf16(x))
    assert np.array_equal(oracle.from_bf16(oracle.to_bf16(x)), workloads.widen_bf16(workloads.narrow_bf16(x)))
    # ties: 1 + 2^-8 is halfway between bf16 neighbours 1.0 (even) and 1 + 2^-7 (odd)
    assert oracle.to_bf16(np.array([1.00390625], np.float32))[0] == 0x3F80
    assert oracle.to_bf16(np.array([1.01171875], np.float32))[0] == 0x3F82
