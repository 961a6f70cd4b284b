"""llm_cuda_sample_batch_static - the sampler for callers that may not allocate.

Some callers of this library cannot call cudaMalloc at all: a serving loop whose device
memory was carved up once at start-up, a framework that owns the allocator, a plugin that
only receives device pointers and a stream. For them the library carries the scratch that
rows split over several CTAs need in a fixed array inside its own image, and offers one
entry point that uses it and never allocates. This file checks that entry point, called
through the C ABI, against the ordinary handle-based entry point on the same inputs: token
ids, kept sets, probabilities and stage statistics must be identical (the bar every GPU
test here uses: bit-exact), on two calls in a row, because the array is shared by all calls
and keeps what the previous call left in it.

Collected last on purpose (file name): if it fails, every other test has already run.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _inputs(seed, batch, vocab, hist_len):
    import torch
    g = np.random.default_rng(seed)
    logits = torch.from_numpy(g.normal(0, 2.5, (batch, vocab)).astype(np.float32)).to("cuda:0")
    history = g.integers(0, vocab, size=(batch, hist_len), dtype=np.uint32)
    seeds = np.arange(batch, dtype=np.uint64) + np.uint64(1000 + seed)
    return logits, history, seeds


def _to_numpy(res):
    import torch
    torch.cuda.synchronize()
    u32 = lambda t: t.cpu().numpy().view(np.uint32)
    return (u32(res.tokens), u32(res.row_flags), u32(res.kept_count), u32(res.kept_ids), res.kept_probs.cpu().numpy(),
            res.row_stats.cpu().numpy())


def test_static_scratch_entry_point_matches_the_handle_based_one_twice_in_a_row(sampler):
    from scriptonait_b200 import native as N
    lib = N.load()
    for call_no, (seed, batch, vocab, split) in enumerate([(1, 48, 40000, 4), (2, 64, 33001, 3)]):
        logits, history, seeds = _inputs(seed, batch, vocab, 200)
        kw = dict(temperature=0.85, top_k=50, top_p=0.9, min_p=0.01, repetition_penalty=1.15, history=history,
                  seeds=seeds, split=split, trace=True, kept_capacity=64)
        want = _to_numpy(sampler.sample_batch(logits, **kw))
        assert sampler.last_launch_info()[1] == split, "the comparison must exercise rows split over several CTAs"
        prepared = sampler.sample_batch(logits, prepare_only=True, **kw)  # marshals the same arguments, launches nothing
        rc = lib.llm_cuda_sample_batch_static(0, C.byref(prepared.args))
        assert rc == N.OK, lib.llm_cuda_static_last_error().decode()
        got = _to_numpy(prepared.result)
        for name, a, b in zip(("tokens", "row_flags", "kept_count", "kept_ids", "kept_probs", "row_stats"), want, got):
            assert np.array_equal(a, b), f"call {call_no}: {name} differs between the two entry points"
        assert (want[1] & N.ROW_DRAW_CONSUMED).all()


def test_static_scratch_entry_point_states_its_limits(sampler):
    from scriptonait_b200 import native as N
    lib = N.load()
    logits, history, seeds = _inputs(3, 8, 5000, 16)
    base = dict(temperature=1.0, top_p=1.0, seeds=seeds, trace=True)
    too_wide = sampler.sample_batch(logits, top_k=N.STATIC_MAX_TOP_K + 1, prepare_only=True, **base)
    assert lib.llm_cuda_sample_batch_static(0, C.byref(too_wide.args)) == N.ERR_CAPACITY
    assert b"top_k" in lib.llm_cuda_static_last_error()
    window = sampler.sample_batch(logits, top_k=0, prepare_only=True, **base)
    assert lib.llm_cuda_sample_batch_static(0, C.byref(window.args)) == N.ERR_CAPACITY
    big_logits, _, big_seeds = _inputs(4, N.STATIC_MAX_BATCH + 1, 1000, 4)
    too_many = sampler.sample_batch(big_logits, top_k=8, temperature=1.0, seeds=big_seeds, prepare_only=True)
    assert lib.llm_cuda_sample_batch_static(0, C.byref(too_many.args)) == N.ERR_CAPACITY
    assert b"batch" in lib.llm_cuda_static_last_error()
    # greedy rows are always within the limits
    greedy = sampler.sample_batch(logits, temperature=0.0, repetition_penalty=1.3, history=history, trace=True,
                                  prepare_only=True)
    assert lib.llm_cuda_sample_batch_static(0, C.byref(greedy.args)) == N.OK
    want = _to_numpy(sampler.sample_batch(logits, temperature=0.0, repetition_penalty=1.3, history=history, trace=True))
    assert np.array_equal(_to_numpy(greedy.result)[0], want[0])
