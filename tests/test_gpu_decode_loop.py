"""Device-side decode-loop glue (Generator::step / recent_tokens,
crates/llm-core/src/generate.rs:157-182): sampling, history-window append, EOS stop and
draw counting stay on the GPU across steps, and reproduce a host loop that calls the
oracle's sample_with with the last `window` tokens each step."""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("early_launch", [0, 2])
def test_batched_decode_loop_matches_a_host_loop_of_sample_with(sampler, early_launch):
    """`early_launch` = 2 launches every sampling step with overlap_previous = 2 right behind
    llm_cuda_advance_rows, which writes the step's history and draw counters: the grid may be set up
    early but reads nothing before that kernel has completed, so the results must not change."""
    import torch
    g = np.random.default_rng(21)
    B, V, steps, window = 12, 600, 40, 16
    table = g.normal(0, 2, (steps, B, V)).astype(np.float32)  # stand-in for the LM head's output per step
    table[:, :, 258] += 2.5  # make EOS reachable
    prompt = g.integers(0, V, size=(B, 5), dtype=np.uint32)
    cfg = oracle.SamplingConfig(temperature=0.9, top_k=20, top_p=0.95, min_p=0.0, repetition_penalty=1.3)
    # host reference loop
    expect, expect_recent = [], []
    for r in range(B):
        rng = oracle.Rng(1000 + r)
        toks = list(prompt[r])
        out = []
        for t in range(steps):
            nxt = oracle.sample_with(table[t, r], cfg, toks[-window:], rng, exp_mode=oracle.EXP_CR)
            if nxt == 258:
                out.append(None)
                break
            toks.append(nxt)
            out.append(nxt)
        expect.append(out)
        expect_recent.append(sorted(int(x) for x in toks[-window:]))  # recent_tokens (generate.rs:176-182)
    # device loop
    dev = "cuda:0"
    hist = torch.zeros((B, window), dtype=torch.int32, device=dev)
    hist[:, :5] = torch.from_numpy(prompt.view(np.int32)).to(dev)
    hlen = torch.full((B,), 5, dtype=torch.int32, device=dev)
    hpos = torch.full((B,), 5, dtype=torch.int32, device=dev)
    draws = torch.zeros(B, dtype=torch.int64, device=dev)
    finished = torch.zeros(B, dtype=torch.uint8, device=dev)
    seeds = torch.arange(1000, 1000 + B, dtype=torch.int64, device=dev)
    got = [[] for _ in range(B)]
    tbl = torch.from_numpy(table).to(dev)
    for t in range(steps):
        res = sampler.sample_batch(tbl[t], temperature=0.9, top_k=20, top_p=0.95, repetition_penalty=1.3, history=hist,
                                   history_len=hlen, seeds=seeds, draw_index=draws, trace=True,
                                   overlap_previous=early_launch)
        was_finished = finished.clone()
        sampler.advance_rows(res.tokens, res.row_flags, history=hist, window=window, history_len=hlen, history_pos=hpos,
                             draw_index=draws, finished=finished)
        torch.cuda.synchronize()
        tk, wf, nf = res.tokens.cpu().numpy().view(np.uint32), was_finished.cpu().numpy(), finished.cpu().numpy()
        for r in range(B):
            if wf[r]:
                continue
            got[r].append(None if nf[r] else int(tk[r]))
    assert got == expect
    # well past the window (5 + 40 tokens through a ring of 16): the ring holds exactly the last
    # `window` tokens of every row, the set the next step's penalty would run over
    hl, hh = hlen.cpu().numpy(), hist.cpu().numpy().view(np.uint32)
    assert [sorted(int(x) for x in hh[r, :hl[r]]) for r in range(B)] == expect_recent


def test_advance_rows_needs_a_write_position_for_the_ring(sampler):
    import torch
    import scriptonait_b200 as sb
    from scriptonait_b200 import native as N
    dev = "cuda:0"
    tokens = torch.zeros(4, dtype=torch.int32, device=dev)
    hist = torch.zeros((4, 8), dtype=torch.int32, device=dev)
    hlen = torch.zeros(4, dtype=torch.int32, device=dev)
    with pytest.raises(sb.LlmCudaError) as e:
        sampler.advance_rows(tokens, None, history=hist, window=8, history_len=hlen, history_pos=None)
    assert e.value.code == N.ERR_BAD_ARGUMENT
