"""Fused tied LM head -> sampler (llm_cuda_lm_head_sample): final RMSNorm, hidden x vocab contraction on the
tensor cores, selection epilogue, merge + ordered tail, with the logits never written in the product path.

Two bars, as the path's specification asks:
* the contraction against a float64 `y @ W^T` on the host, y = rmsnorm(x) narrowed to bf16 as the device
  does (crates/llm-core/src/ops/activation.rs:5-19; linear.wgsl): the products of bf16 values are exact in
  f32, so only the order of the f32 accumulation differs: |error| <= 2e-5 * sum|y_i w_i| per logit (stated
  tolerance; 512..4096 terms of relative 2^-24 each) - and for rows normalised on the device, a second,
  looser bar (1e-2 of the row's logit spread) that allows the rare bf16 flip from the norm's own rounding;
* every sampler stage bit-exact on the logits the tensor cores produced (read back through the testing
  aid `logits_out`): tokens, kept sets, probabilities and stage statistics equal the CPU oracle's on those
  logits, with the same seeded uniform stream.
"""
import numpy as np
import pytest

import oracle
from scriptonait_b200 import native as N
from scriptonait_b200.workloads import narrow_bf16, widen_bf16

pytestmark = pytest.mark.gpu


def _case(seed, B, H, V, scale=2.0):
    g = np.random.default_rng(seed)
    x = g.normal(0, 1.5, (B, H)).astype(np.float32)
    gain = g.uniform(0.5, 1.5, H).astype(np.float32)
    w = narrow_bf16((g.normal(0, 1, (V, H)) * (scale / np.sqrt(H))).astype(np.float32))   # logits ~ N(0, scale^2)
    return x, gain, w


def _to_dev(x, gain, w):
    import torch
    xd = torch.from_numpy(x).to("cuda:0")
    gd = torch.from_numpy(gain).to("cuda:0")
    wd = torch.from_numpy(w.view(np.int16)).to("cuda:0").view(torch.bfloat16)
    return xd, gd, wd


def _host_norm_bf16(x, gain, eps):
    ms = (x.astype(np.float32) ** 2).sum(axis=1, dtype=np.float32) / np.float32(x.shape[1])
    n = (np.float32(1.0) / np.sqrt(ms + np.float32(eps))).astype(np.float32)
    y = (x * n[:, None]).astype(np.float32) * gain[None, :]
    return widen_bf16(narrow_bf16(y.astype(np.float32)))


def _check_sampler_exact(res, logits, seeds, **params):
    import torch
    torch.cuda.synchronize()
    u32 = lambda t: t.cpu().numpy().view(np.uint32)
    flags = u32(res.row_flags)
    undecided = int((flags == N.ROW_INVALID).sum())
    ref = oracle.sample_batch(logits, seeds=seeds, exp_mode=oracle.EXP_CR, kept_capacity=res.kept_ids.shape[1], **params)
    ok = flags != N.ROW_INVALID
    assert np.array_equal(u32(res.tokens)[ok], ref.tokens[ok])
    assert np.array_equal(u32(res.kept_count)[ok], ref.kept_count[ok])
    kid, kpr = u32(res.kept_ids), res.kept_probs.cpu().numpy()
    for r in np.flatnonzero(ok):
        n = min(int(ref.kept_count[r]), kid.shape[1])
        assert np.array_equal(kid[r, :n], ref.kept_ids[r, :n]) and np.array_equal(kpr[r, :n], ref.kept_probs[r, :n])
    assert np.array_equal(res.row_stats.cpu().numpy()[ok], ref.stats[ok])
    return undecided


@pytest.mark.parametrize("B,H,V,top_k", [(48, 512, 8997, 40), (16, 256, 1000, 8), (200, 1024, 32768, 64), (256, 2048, 50257, 256)])
def test_fused_lm_head_matches_host_contraction_and_oracle_sampler(sampler, B, H, V, top_k):
    x, gain, w = _case(B + V, B, H, V)
    xd, gd, wd = _to_dev(x, gain, w)
    seeds = np.arange(B, dtype=np.uint64) + np.uint64(99)
    params = dict(temperature=0.8, top_k=top_k, top_p=0.95, min_p=0.01)
    res = sampler.lm_head_sample(xd, wd, norm_gain=gd, norm_eps=1e-5, seeds=seeds, trace=True, kept_capacity=64,
                                 want_logits=True, **params)
    assert sampler.device_status() == 0
    logits = res.logits.cpu().numpy()
    # (1) the contraction: device-normalised rows against the host's float64 product of bf16 inputs
    y = _host_norm_bf16(x, gain, 1e-5)
    wf = widen_bf16(w)
    want = y.astype(np.float64) @ wf.astype(np.float64).T
    spread = want.std(axis=1, keepdims=True)
    assert np.abs(logits - want).max() <= 1e-2 * spread.max()
    # (2) the sampler on the logits the tensor cores produced: bit-exact
    undecided = _check_sampler_exact(res, logits, seeds, repetition_penalty=1.0, **params)
    assert undecided == 0, f"{undecided} rows were left undecided by the threshold estimate"


def test_accumulation_error_bound_with_exact_inputs(sampler):
    """No norm on the device: hidden is narrowed to bf16 exactly, products are exact in f32, and only the
    accumulation order differs from the host's: |error| <= 2e-5 * sum |y_i w_i| per logit."""
    B, H, V = 32, 1024, 128 * 65
    x, _, w = _case(7, B, H, V)
    y = widen_bf16(narrow_bf16(x))
    xd, _, wd = _to_dev(y, np.ones(H, np.float32), w)
    seeds = np.arange(B, dtype=np.uint64)
    res = sampler.lm_head_sample(xd, wd, norm_gain=None, seeds=seeds, trace=True, want_logits=True, temperature=1.0,
                                 top_k=50, top_p=0.9)
    logits = res.logits.cpu().numpy()
    wf = widen_bf16(w).astype(np.float64)
    want = y.astype(np.float64) @ wf.T
    bound = 2e-5 * (np.abs(y).astype(np.float64) @ np.abs(wf).T)
    assert (np.abs(logits - want) <= bound).all()
    assert _check_sampler_exact(res, logits, seeds, temperature=1.0, top_k=50, top_p=0.9, min_p=0.0, repetition_penalty=1.0) == 0


def test_greedy_and_product_path_without_logits(sampler):
    import torch
    B, H, V = 64, 512, 128 * 80
    x, gain, w = _case(11, B, H, V)
    xd, gd, wd = _to_dev(x, gain, w)
    with_logits = sampler.lm_head_sample(xd, wd, norm_gain=gd, temperature=0.0, trace=True, want_logits=True)
    torch.cuda.synchronize()
    logits = with_logits.logits.cpu().numpy()
    assert np.array_equal(with_logits.tokens.cpu().numpy().view(np.uint32), logits.argmax(axis=1).astype(np.uint32))
    # the product path (no logits written anywhere) returns the same tokens
    seeds = np.arange(B, dtype=np.uint64) + np.uint64(5)
    a = sampler.lm_head_sample(xd, wd, norm_gain=gd, temperature=0.9, top_k=32, top_p=0.9, seeds=seeds, want_logits=True)
    b = sampler.lm_head_sample(xd, wd, norm_gain=gd, temperature=0.9, top_k=32, top_p=0.9, seeds=seeds)
    torch.cuda.synchronize()
    assert torch.equal(a.tokens, b.tokens)
    assert sampler.device_status() == 0


def test_limits_are_stated(sampler):
    import torch
    import scriptonait_b200 as sb
    x = torch.zeros((4, 64), dtype=torch.float32, device="cuda:0")
    w = torch.zeros((300, 64), dtype=torch.bfloat16, device="cuda:0")
    with pytest.raises(sb.LlmCudaError) as e:
        sampler.lm_head_sample(x, w, top_k=0)
    assert e.value.code == N.ERR_UNSUPPORTED
    with pytest.raises(sb.LlmCudaError) as e:
        sampler.lm_head_sample(x, w, top_k=300)
    assert e.value.code == N.ERR_UNSUPPORTED
