"""Vocabulary sharding (c5): per-shard candidate lists + merge, emulated on one GPU by
calling shard_select once per column range, against the oracle on the whole row."""
import numpy as np
import pytest

import oracle
import parity
from scriptonait_b200 import native as N
from scriptonait_b200 import workloads
from scriptonait_b200.sharding import vocab_shard_ranges

pytestmark = pytest.mark.gpu


def _sharded(sampler, w, n_shards, cand_stride, hist=None, **kw):
    import torch
    lg = parity.device_logits(w)
    V = w.vocab
    vals = torch.zeros((n_shards, w.batch, cand_stride), dtype=torch.float32, device="cuda:0")
    ids = torch.zeros((n_shards, w.batch, cand_stride), dtype=torch.int32, device="cuda:0")
    cnt = torch.zeros((n_shards, w.batch), dtype=torch.int32, device="cuda:0")
    for s, (lo, hi) in enumerate(vocab_shard_ranges(V, n_shards)):
        sampler.shard_select(lg[:, lo:hi], column_offset=lo, vocab_global=V, cand_stride=cand_stride,
                             temperature=w.temperature, top_k=w.top_k, repetition_penalty=w.repetition_penalty,
                             history=hist, out=(vals[s], ids[s], cnt[s]))
    res = sampler.merge_draw(vals, ids, cnt, vocab_global=V, temperature=w.temperature, top_k=w.top_k, top_p=w.top_p,
                             min_p=w.min_p, seeds=w.seeds, trace=True, kept_capacity=64, **kw)
    torch.cuda.synchronize()
    u32 = lambda t: t.cpu().numpy().view(np.uint32)
    return parity.GpuOut(u32(res.tokens), u32(res.row_flags), u32(res.kept_count), u32(res.kept_ids),
                         res.kept_probs.cpu().numpy(), res.row_stats.cpu().numpy()), (vals, ids, cnt)


@pytest.mark.parametrize("n_shards", [2, 4, 8])
def test_c5_vocab_sharded_matches_the_unsharded_reference(sampler, n_shards):
    w = workloads.c5()
    gpu, (vals, ids, cnt) = _sharded(sampler, w, n_shards, 64)
    rep = parity.compare(parity.run_oracle(w, oracle.EXP_CR), gpu, w, exact=True)
    print(rep.summary())
    parity.assert_exact(rep)
    # every list is ordered (value descending, id ascending) and ids lie in the shard's range
    v, i, c = vals.cpu().numpy(), ids.cpu().numpy().view(np.uint32), cnt.cpu().numpy()
    for s, (lo, hi) in enumerate(vocab_shard_ranges(w.vocab, n_shards)):
        assert (c[s] == 64).all()
        assert ((i[s] >= lo) & (i[s] < hi)).all()
        assert (np.diff(v[s], axis=1) <= 0).all()


def test_vocab_sharding_with_penalty_and_greedy(sampler):
    g = np.random.default_rng(11)
    B, V = 6, 40000
    x = g.normal(0, 2, (B, V)).astype(np.float32)
    hist = g.integers(0, V, size=(B, 100), dtype=np.uint32)
    w = workloads.Workload("vs", x, temperature=0.9, top_k=32, top_p=0.9, repetition_penalty=1.4, history=hist,
                           seeds=np.arange(B, dtype=np.uint64), batch=B)
    gpu, _ = _sharded(sampler, w, 4, 32, hist=hist)
    parity.assert_exact(parity.compare(parity.run_oracle(w, oracle.EXP_CR), gpu, w, exact=True))
    wg = workloads.Workload("vsg", x, temperature=0.0, repetition_penalty=1.4, history=hist,
                            seeds=np.arange(B, dtype=np.uint64), batch=B)
    gpu, _ = _sharded(sampler, wg, 4, 8, hist=hist)
    parity.assert_exact(parity.compare(parity.run_oracle(wg, oracle.EXP_CR), gpu, wg, exact=True))


def test_vocab_sharding_rejects_top_k_zero(sampler):
    import torch
    import scriptonait_b200 as sb
    x = torch.zeros((2, 1000), dtype=torch.float32, device="cuda:0")
    with pytest.raises(sb.LlmCudaError) as e:
        sampler.shard_select(x, column_offset=0, vocab_global=2000, cand_stride=64, top_k=0)
    assert e.value.code == N.ERR_UNSUPPORTED


def _sharded_packed(sampler, w, n_shards, cand_stride, **kw):
    """The single-buffer form: every shard writes one packed block, the blocks are laid end to end as
    one all-gather would leave them, and the merge reads that buffer."""
    import torch
    from scriptonait_b200 import sharding
    lg = parity.device_logits(w)
    words = sharding.packed_words(w.batch, cand_stride)
    gathered = torch.zeros((n_shards, words), dtype=torch.int32, device="cuda:0")
    for s, (lo, hi) in enumerate(vocab_shard_ranges(w.vocab, n_shards)):
        sampler.shard_select_packed(lg[:, lo:hi], column_offset=lo, vocab_global=w.vocab, cand_stride=cand_stride,
                                    temperature=w.temperature, top_k=w.top_k, repetition_penalty=w.repetition_penalty,
                                    history=w.history, out=gathered[s])
    res = sampler.merge_draw_packed(gathered, batch=w.batch, cand_stride=cand_stride, vocab_global=w.vocab,
                                    temperature=w.temperature, top_k=w.top_k, top_p=w.top_p, min_p=w.min_p, seeds=w.seeds,
                                    trace=True, kept_capacity=64, **kw)
    torch.cuda.synchronize()
    u32 = lambda t: t.cpu().numpy().view(np.uint32)
    return parity.GpuOut(u32(res.tokens), u32(res.row_flags), u32(res.kept_count), u32(res.kept_ids),
                         res.kept_probs.cpu().numpy(), res.row_stats.cpu().numpy()), gathered


@pytest.mark.parametrize("n_shards", [2, 8])
def test_c5_packed_blocks_match_the_unsharded_reference(sampler, n_shards):
    from scriptonait_b200 import sharding
    w = workloads.c5()
    gpu, gathered = _sharded_packed(sampler, w, n_shards, 64)
    parity.assert_exact(parity.compare(parity.run_oracle(w, oracle.EXP_CR), gpu, w, exact=True))
    _, _, cnt = sharding.unpack_candidates(gathered, w.batch, 64)
    assert (cnt.cpu().numpy() == 64).all()


def test_packed_blocks_with_empty_shards_and_a_penalty(sampler):
    """Vocabulary 300 over 8 shards of 64-aligned columns: the last three shards own nothing and send
    empty lists; the merge still returns what one sample_with per row returns."""
    g = np.random.default_rng(17)
    B, V = 7, 300
    x = g.normal(0, 2, (B, V)).astype(np.float32)
    hist = g.integers(0, V, size=(B, 40), dtype=np.uint32)
    w = workloads.Workload("tiny", x, temperature=0.9, top_k=24, top_p=0.9, repetition_penalty=1.25, history=hist,
                           seeds=np.arange(B, dtype=np.uint64), batch=B)
    assert sum(1 for lo, hi in vocab_shard_ranges(V, 8) if hi == lo) == 3
    gpu, _ = _sharded_packed(sampler, w, 8, 24)
    parity.assert_exact(parity.compare(parity.run_oracle(w, oracle.EXP_CR), gpu, w, exact=True))
