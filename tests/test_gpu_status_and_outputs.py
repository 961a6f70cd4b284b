"""The device status word, the post-penalty output and the C++ header, on the GPU.

* A bounded wait inside a kernel that runs out must surface as an error code, never as a hang or a
  guessed token (the reference turns device failure into an Err: crates/llm-gpu/src/buffers.rs:58-86).
  The wait is made to run out in the one safe way: the host marks every full-ordering scratch slot
  taken and shortens the slot wait, so rows that need the full ordering give up after a few
  milliseconds. Nothing faults, traps or waits without a limit.
* penalized_out: the value of every history id after mask and repetition penalty
  (generate.rs:333-352) against the oracle, within 1e-6 relative (it is bit-exact in practice).
* include/llm_cuda.hpp: compiled with g++, linked against the library and run.
"""
import os
import subprocess

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_slot_wait_that_runs_out_reports_timeout_and_invalid_rows(sampler):
    import torch
    import scriptonait_b200 as sb
    from scriptonait_b200 import native as N
    g = np.random.default_rng(5)
    x = torch.from_numpy(g.normal(0, 0.2, (6, 9000)).astype(np.float32)).to("cuda:0")
    kw = dict(temperature=1.0, top_k=0, top_p=0.9, seeds=np.arange(6, dtype=np.uint64), trace=True)
    assert sampler.device_status() == 0
    good = sampler.sample_batch(x, force_full_sort=True, **kw)
    torch.cuda.synchronize()
    assert (good.row_flags.cpu().numpy() & N.ROW_FULL_SORT).all()
    sampler.hold_full_sort_slots(True, wait_rounds=200)
    try:
        res = sampler.sample_batch(x, force_full_sort=True, **kw)
        with pytest.raises(sb.LlmCudaError) as e:
            sampler.device_status()
        assert e.value.code == N.ERR_TIMEOUT and "slot" in str(e.value)
        flags = res.row_flags.cpu().numpy().view(np.uint32)
        assert (flags == N.ROW_INVALID).all() and (res.tokens.cpu().numpy() == 0).all()
        assert sampler.device_status() == 0, "reading the word clears it"
    finally:
        sampler.hold_full_sort_slots(False, wait_rounds=0)
    again = sampler.sample_batch(x, force_full_sort=True, **kw)
    assert sampler.device_status() == 0
    assert torch.equal(again.tokens, good.tokens)


def test_host_entry_point_returns_the_timeout_code(sampler):
    import scriptonait_b200 as sb
    from scriptonait_b200 import native as N
    g = np.random.default_rng(6)
    row = g.normal(0, 0.2, 5000).astype(np.float32)
    rng = sb.Rng(3)
    before = rng.state
    want = sampler.sample(row, 1.0, sb.Rng(3))  # flat row, no rank cut: resolved by the full ordering
    sampler.hold_full_sort_slots(True, wait_rounds=100)
    try:
        with pytest.raises(sb.LlmCudaError) as e:
            sampler.sample(row, 1.0, rng)
        assert e.value.code == N.ERR_TIMEOUT
    finally:
        sampler.hold_full_sort_slots(False, wait_rounds=0)
    assert rng.state == before, "a failed call consumes no draw"
    assert sampler.sample(row, 1.0, rng) == want


@pytest.mark.parametrize("split", [1, 3])
@pytest.mark.parametrize("with_mask", [False, True])
def test_post_penalty_values_match_the_oracle(sampler, split, with_mask):
    import torch
    g = np.random.default_rng(31 + split)
    B, V, H = 5, 30000, 300
    x = g.normal(0, 2, (B, V)).astype(np.float32)
    hist = g.integers(0, V + 50, size=(B, H), dtype=np.uint32)      # some ids past the vocabulary
    hist[0, :40] = hist[0, 0]                                        # compounding
    hist[1, :] = np.argsort(-x[1])[:H]                               # the leaders
    allowed = None
    bits = alen = None
    if with_mask:
        allowed = g.random(V) < 0.7
        bits, alen = sampler.pack_allowed(allowed)
    res = sampler.sample_batch(torch.from_numpy(x).to("cuda:0"), temperature=0.8, top_k=40, top_p=0.9,
                               repetition_penalty=1.3, history=hist, allowed_bits=bits, allowed_len=alen,
                               seeds=np.arange(B, dtype=np.uint64), split=split, want_penalized=True)
    torch.cuda.synchronize()
    got = res.penalized.cpu().numpy()
    cfg = oracle.SamplingConfig(temperature=0.8, top_k=40, top_p=0.9, repetition_penalty=1.3, allowed=allowed)
    for r in range(B):
        want = oracle.penalized_at_history(x[r], cfg, hist[r])
        nan = np.isnan(want)
        assert np.array_equal(np.isnan(got[r]), nan)
        inf = np.isinf(want)
        assert np.array_equal(got[r][inf], want[inf])
        ok = ~nan & ~inf
        rel = np.abs(got[r][ok] - want[ok]) / np.maximum(np.abs(want[ok]), 1e-30)
        assert rel.max(initial=0.0) <= 1e-6          # the tolerance the path's specification states for f32
        assert np.array_equal(got[r][ok], want[ok])  # and in fact identical: the same rounded operations


def test_cpp_header_compiles_links_and_samples(sampler, tmp_path):
    """include/llm_cuda.hpp through g++: the reference's own small cases (generate.rs:550-583)."""
    from scriptonait_b200 import native
    src = tmp_path / "hpp_check.cpp"
    src.write_text(r'''
#include <cstdio>
#include "llm_cuda.hpp"
int main() {
    try {
        llm_cuda::Sampler s(0, 8, 4096, 64, 64);
        llm_cuda::SamplingConfig cfg;            // generate.rs:82-95
        if (cfg.top_k != 40 || cfg.repetition_window != 128) return 3;
        cfg.temperature = 5.0f; cfg.top_k = 2; cfg.top_p = 1.0f; cfg.repetition_penalty = 1.0f;
        for (uint64_t seed = 0; seed < 20; ++seed) {   // generate.rs:550-561
            auto rng = llm_cuda::Rng::seed_from_u64(seed);
            std::printf("%u ", s.sample_with({0.f, 5.f, 0.f, 9.f, 0.f}, cfg, {}, rng));
        }
        llm_cuda::SamplingConfig greedy;               // generate.rs:575-583
        greedy.temperature = 0.0f; greedy.repetition_penalty = 1.5f;
        auto rng = llm_cuda::Rng::seed_from_u64(0);
        std::printf("| %u %u ", s.sample_with({2.0f, 1.9f, 0.0f}, greedy, {}, rng), s.sample_with({2.0f, 1.9f, 0.0f}, greedy, {0}, rng));
        std::printf("| %u\n", s.sample({20.f, 0.f, 0.f, 0.f}, 0.01f, rng));
    } catch (const llm_cuda::Error& e) { std::printf("error %d %s\n", e.code, e.what()); return 2; }
    return 0;
}
''')
    exe = tmp_path / "hpp_check"
    libdir = os.path.dirname(native.library_path())
    subprocess.run(["g++", "-std=c++17", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe), "-L", libdir,
                    "-lllm_cuda", f"-Wl,-rpath,{libdir}"], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    first, second, third = out.stdout.split("|")
    cfg = oracle.SamplingConfig(temperature=5.0, top_k=2, top_p=1.0, repetition_penalty=1.0)
    want = [oracle.sample_with(np.array([0, 5, 0, 9, 0], np.float32), cfg, [], oracle.Rng(seed), exp_mode=oracle.EXP_CR)
            for seed in range(20)]
    assert [int(t) for t in first.split()] == want and set(want) <= {1, 3}
    assert [int(t) for t in second.split()] == [0, 1]
    assert int(third) == 0
