"""Launches that overlap their predecessor (overlap_previous: programmatic dependent launch).

A chain of independent calls, each with its own inputs and outputs, is issued back to back on one
stream with the flag set; every call must leave exactly what the same call leaves in strict stream
order. The chain mixes the row kinds whose later phases write shared scratch: window rows, exact
selection with several CTAs per row (scratch lists and tickets), and rows that take the full
ordering (scratch slots)."""
import numpy as np
import pytest

from scriptonait_b200 import workloads

pytestmark = pytest.mark.gpu


def _variants():
    g = np.random.default_rng(77)
    out = []
    # window rows (min-p only), bf16
    for v in range(3):
        w = workloads.c3(batch=96, vocab=32000, row0=1000 * v, variant=v)
        out.append((w, dict(split=0)))
    # exact selection, penalty, several CTAs per row
    w = workloads.c2(batch=48, vocab=32768, hist_len=128)
    out.append((w, dict(split=4)))
    # near-flat rows without a rank cut: the window cannot hold them, every row takes the full ordering
    flat = g.normal(0.0, 0.05, (6, 5000)).astype(np.float32)
    out.append((workloads.Workload("flat", flat, temperature=1.0, top_k=0, top_p=0.9, min_p=0.0,
                                   seeds=np.arange(6, dtype=np.uint64) + np.uint64(5), batch=6), dict(split=0)))
    return out


def _prepare(sampler, w, extra, overlap):
    import torch
    t = torch.from_numpy(w.logits.view(np.int16) if w.is_bf16 else w.logits).to("cuda:0")
    lg = t.view(torch.bfloat16) if w.is_bf16 else t
    call = sampler.sample_batch(lg, history=w.history, seeds=w.seeds, draw_index=w.draw_index, batch=w.batch,
                                trace=True, prepare_only=True, overlap_previous=overlap, **extra, **w.params())
    return call


def _snapshot(call):
    r = call.result
    return [x.clone() for x in (r.tokens, r.row_flags, r.kept_count, r.kept_ids, r.kept_probs)]


def test_overlapped_chain_equals_strict_order(sampler):
    import torch
    from scriptonait_b200 import native as N
    cases = _variants()
    strict = []
    for w, extra in cases:
        c = _prepare(sampler, w, extra, overlap=False)
        c.launch()
        torch.cuda.synchronize()
        strict.append(_snapshot(c))
    assert (strict[-1][1].cpu().numpy() & N.ROW_FULL_SORT).all(), "the flat rows are meant to take the full ordering"

    calls = [_prepare(sampler, w, extra, overlap=True) for w, extra in cases]
    order = [0, 1, 2, 3, 4, 3, 0, 4, 1, 3, 2, 0, 3, 4, 1]
    for rep in range(3):
        for c in calls:  # wipe the outputs so a launch that wrote nothing cannot pass
            c.result.tokens.fill_(-1)
            c.result.kept_count.fill_(-1)
        torch.cuda.synchronize()
        for i in order:
            calls[i].launch()
        torch.cuda.synchronize()
        for i, c in enumerate(calls):
            got = _snapshot(c)
            for a, b, name in zip(got, strict[i], ("tokens", "row_flags", "kept_count", "kept_ids", "kept_probs")):
                assert torch.equal(a, b), f"case {i} ({cases[i][0].name}) {name} differs in repetition {rep}"


def test_overlap_flag_after_other_work_on_the_stream(sampler):
    """The flag only changes anything behind another sampler launch; behind a copy or another
    kernel the launch waits for it like any other."""
    import torch
    w = workloads.c3(batch=32, vocab=32000)
    base = torch.from_numpy(w.logits.view(np.int16)).to("cuda:0")
    c0 = _prepare(sampler, w, dict(split=0), overlap=False)
    c0.launch()
    torch.cuda.synchronize()
    want = c0.result.tokens.clone()
    staged = torch.zeros_like(base)
    lg = staged.view(torch.bfloat16)
    call = sampler.sample_batch(lg, seeds=w.seeds, batch=w.batch, prepare_only=True, overlap_previous=True, **w.params())
    for _ in range(5):
        staged.zero_()
        staged.copy_(base)       # the logits are produced on the stream right before the launch
        call.launch()
    torch.cuda.synchronize()
    assert torch.equal(call.result.tokens, want)
