"""Host-side logic of the multi-GPU paths on CPU, world_size 2 over gloo: row partition +
token gather, and vocabulary partition + candidate all-gather layout. The per-rank
compute is stood in by the CPU oracle / numpy (test infrastructure); what is under test
is the partitioning, the gather layout and that the partitioned result equals the
unpartitioned reference."""
import os
import socket

import numpy as np
import pytest

import oracle
from scriptonait_b200 import sharding, workloads


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_row_ranges_partition_every_batch():
    for batch in (0, 1, 7, 256, 1024, 1025):
        for world in (1, 2, 3, 4, 8):
            ranges = [sharding.row_shard_range(batch, world, r) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == batch
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            sizes = [hi - lo for lo, hi in ranges]
            assert max(sizes) - min(sizes) <= 1


def test_vocab_ranges_partition_every_vocabulary():
    for vocab in (1, 63, 64, 65, 50257, 128256, 262144):
        for n in (1, 2, 4, 8):
            ranges = sharding.vocab_shard_ranges(vocab, n)
            assert ranges[0][0] == 0 and ranges[-1][1] == vocab
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            assert all(lo % 64 == 0 for lo, hi in ranges if hi > lo)


def _row_worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    w = workloads.c2(batch=13, vocab=2048, hist_len=32)
    lo, hi = sharding.row_shard_range(w.batch, world, rank)
    mine = workloads.row_slice(w, lo, hi)
    res = oracle.sample_batch(mine.logits, history=mine.history, seeds=mine.seeds, threads=1, **mine.params())
    local = torch.from_numpy(res.tokens.astype(np.int64))
    full = sharding.gather_rows(local, w.batch)
    q.put((rank, full.numpy().tolist()))
    dist.destroy_process_group()


def _vocab_worker(rank, world, port, q, V=1000):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = np.random.default_rng(5)
    B, K = 5, 16
    x = g.normal(0, 2, (B, V)).astype(np.float32)
    lo, hi = sharding.vocab_shard_ranges(V, world)[rank]   # may be empty: a tiny vocabulary leaves trailing ranks without columns
    vals = np.full((B, K), -np.inf, np.float32)
    ids = np.zeros((B, K), np.int32)
    cnt = np.zeros(B, np.int32)
    for b in range(B):
        order = sorted(range(lo, hi), key=lambda i: (-float(x[b, i]), i))[:K]
        vals[b, :len(order)] = x[b, order]
        ids[b, :len(order)] = order
        cnt[b] = len(order)
    # one packed block per rank (values, ids, counts), one all-gather
    packed = torch.from_numpy(np.concatenate([vals.view(np.int32).ravel(), ids.ravel(), cnt]))
    assert packed.numel() == sharding.packed_words(B, K)
    gathered = sharding.all_gather_packed(packed)
    gv, gi, gc = sharding.unpack_candidates(gathered, B, K)
    assert tuple(gv.shape) == (world, B, K) and tuple(gi.shape) == (world, B, K) and tuple(gc.shape) == (world, B)
    merged = []
    for b in range(B):
        cand = [(float(gv[s, b, i]), int(gi[s, b, i])) for s in range(world) for i in range(int(gc[s, b]))]
        cand.sort(key=lambda t: (-t[0], t[1]))
        merged.append([i for _, i in cand[:K]])
    q.put((rank, merged))
    dist.destroy_process_group()


def _tiny_vocab_worker(rank, world, port, q):
    _vocab_worker(rank, world, port, q, V=40)   # align 64: rank 1's shard is empty


def _spawn(worker, world=2):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return out


@pytest.mark.timeout(300)
def test_row_sharded_run_equals_the_unsharded_reference_world_size_2():
    out = _spawn(_row_worker)
    w = workloads.c2(batch=13, vocab=2048, hist_len=32)
    ref = oracle.sample_batch(w.logits, history=w.history, seeds=w.seeds, threads=1, **w.params())
    assert out[0] == out[1] == ref.tokens.astype(np.int64).tolist()


@pytest.mark.timeout(300)
def test_vocab_sharded_candidate_merge_equals_global_top_k_world_size_2():
    out = _spawn(_vocab_worker)
    g = np.random.default_rng(5)
    x = g.normal(0, 2, (5, 1000)).astype(np.float32)
    for b in range(5):
        tr = oracle.sample_with(x[b], oracle.SamplingConfig(temperature=1.0, top_k=16, top_p=1.0, repetition_penalty=1.0),
                                [], oracle.Rng(0), trace=True)
        assert out[0][b] == out[1][b] == list(tr.kept_ids)


@pytest.mark.timeout(300)
def test_empty_shard_still_reaches_the_exchange_world_size_2():
    """Vocabulary 40 over 2 ranks with 64-column alignment: rank 1 owns no columns, contributes empty
    lists, and both ranks still complete the all-gather with the global top-k."""
    assert sharding.vocab_shard_ranges(40, 2)[1] == (40, 40)
    out = _spawn(_tiny_vocab_worker)
    g = np.random.default_rng(5)
    x = g.normal(0, 2, (5, 40)).astype(np.float32)
    for b in range(5):
        want = sorted(range(40), key=lambda i: (-float(x[b, i]), i))[:16]
        assert out[0][b] == out[1][b] == want
