"""Oracle behaviour the reference's tests do not pin, checked against the source lines
(crates/llm-core/src/generate.rs:325-420) and against the independent restatement in
tests/pyref.py."""
import numpy as np
import pytest

import oracle
import pyref
from oracle import Rng, SamplingConfig, sample_with

INF = np.float32(np.inf)


def test_allowed_mask_blocks_ids_but_never_eos_and_ids_past_the_slice_stay_allowed():
    # generate.rs:333-341
    V = 300
    logits = np.zeros(V, np.float32)
    logits[5] = 9.0      # blocked -> must never win
    logits[258] = 8.0    # EOS: blocked in the slice but exempt
    logits[299] = 7.0    # past the slice (len 280): allowed
    allowed = np.ones(280, bool)
    allowed[5] = False
    allowed[258] = False
    cfg = SamplingConfig(temperature=0.0, repetition_penalty=1.0, allowed=allowed)
    assert sample_with(logits, cfg, [], Rng(0)) == 258
    allowed2 = allowed.copy()
    logits2 = logits.copy()
    logits2[258] = -1.0
    assert sample_with(logits2, SamplingConfig(temperature=0.0, repetition_penalty=1.0, allowed=allowed2), [], Rng(0)) == 299


def test_argmax_first_occurrence_and_all_neg_inf_and_nan():
    # ops/loss.rs:6-16
    assert oracle.argmax(np.array([1, 3, 3, 2], np.float32)) == 1
    assert oracle.argmax(np.array([-INF, -INF], np.float32)) == 0
    assert oracle.argmax(np.array([np.nan, 1.0, np.nan], np.float32)) == 1
    assert oracle.argmax(np.array([0.0, -0.0], np.float32)) == 0


def test_duplicate_history_entries_compound_and_out_of_range_ids_are_skipped():
    # generate.rs:343-352: once per entry, each step rounded to f32
    logits = np.array([3.0, -2.0, 0.0, 1.0], np.float32)
    cfg = SamplingConfig(repetition_penalty=1.3)
    out = oracle.penalized_at_history(logits, cfg, [0, 0, 0, 1, 1, 2, 99, 4])
    p = np.float32(1.3)
    a = np.float32(3.0)
    for _ in range(3):
        a = np.float32(a / p)
    b = np.float32(-2.0)
    for _ in range(2):
        b = np.float32(b * p)
    assert out[0] == a and out[1] == a and out[3] == b
    assert out[5] == np.float32(0.0)          # zero takes the multiply branch and stays zero
    assert np.isnan(out[6]) and np.isnan(out[7])  # ids >= vocab are skipped


def test_ties_at_the_top_k_edge_go_to_the_lower_index():
    # generate.rs:364-370
    logits = np.array([1.0, 5.0, 5.0, 5.0, 0.0], np.float32)
    cfg = SamplingConfig(temperature=1.0, top_k=2, top_p=1.0, repetition_penalty=1.0)
    seen = {sample_with(logits, cfg, [], Rng(s)) for s in range(200)}
    assert seen == {1, 2}
    tr = sample_with(logits, cfg, [], Rng(0), trace=True)
    assert list(tr.kept_ids) == [1, 2]
    # +0.0 and -0.0 compare equal: index decides
    z = np.array([-0.0, 0.0, -1.0], np.float32)
    tr = sample_with(z, SamplingConfig(temperature=1.0, top_k=1, top_p=1.0, repetition_penalty=1.0), [], Rng(0), trace=True)
    assert list(tr.kept_ids) == [0]


def test_degenerate_sum_returns_first_of_the_ordering_without_drawing():
    # generate.rs:375-377
    cfg = SamplingConfig(temperature=1.0, top_k=0, top_p=1.0, repetition_penalty=1.0)
    rng = Rng(5)
    tr = sample_with(np.full(7, -INF, np.float32), cfg, [], rng, trace=True)
    assert tr.token == 0 and tr.flags & oracle.FLAG_DEGENERATE and rng.state == 5
    tr = sample_with(np.array([0.0, INF, 1.0, INF], np.float32), cfg, [], rng, trace=True)
    assert tr.token == 1 and tr.flags & oracle.FLAG_DEGENERATE and rng.state == 5


def test_exactly_one_rng_output_per_draw():
    # generate.rs:412
    rng = Rng(11)
    cfg = SamplingConfig()
    logits = np.random.default_rng(0).normal(0, 2, 100).astype(np.float32)
    for i in range(5):
        sample_with(logits, cfg, [], rng)
        assert rng.state == (11 + (i + 1) * oracle.GOLDEN_GAMMA) & oracle.MASK64


@pytest.mark.parametrize("case", range(60))
def test_cpp_oracle_agrees_with_the_independent_python_restatement(case):
    g = np.random.default_rng(1000 + case)
    V = int(g.integers(1, 400))
    style = case % 4
    if style == 0:
        logits = g.normal(0, 2, V).astype(np.float32)
    elif style == 1:
        logits = np.round(g.normal(0, 1.5, V)).astype(np.float32)  # many exact ties
    elif style == 2:
        logits = g.normal(0, 0.2, V).astype(np.float32)             # near-flat
    else:
        logits = g.normal(0, 3, V).astype(np.float32)
        logits[g.random(V) < 0.2] = -INF
    temperature = float(g.choice([0.0, 0.5, 0.8, 1.0, 1.3, 5.0]))
    top_k = int(g.choice([0, 1, 2, 7, 40, 1000]))
    top_p = float(g.choice([1.0, 0.95, 0.9, 0.5, 0.05]))
    min_p = float(g.choice([0.0, 0.05, 0.5, 5.0]))
    penalty = float(g.choice([1.0, 1.1, 1.5, 0.8]))
    recent = g.integers(0, V + 3, size=int(g.integers(0, 40))).astype(np.uint32)
    allowed = None
    if case % 5 == 0:
        allowed = g.random(int(g.integers(1, V + 10))) < 0.7
    seed = int(g.integers(0, 2 ** 63))
    cfg = SamplingConfig(temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p, repetition_penalty=penalty,
                         allowed=allowed)
    rng = Rng(seed)
    state = seed
    for _ in range(3):
        tr = sample_with(logits, cfg, recent, rng, exp_mode=oracle.EXP_CR, trace=True)
        tok, state, ids, probs = pyref.sample_with(logits, temperature, top_k, top_p, min_p, penalty, list(recent), state, allowed)
        assert tr.token == tok
        assert rng.state == state
        assert list(tr.kept_ids) == list(ids)
        assert [float(p) for p in tr.kept_probs] == [float(p) for p in probs]
