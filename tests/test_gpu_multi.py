"""Two-GPU runs of the partitioned paths, one process per GPU over NCCL: rows sharded with
no data-path collective, and the vocabulary sharded with the one all-gather of candidate
lists. Both must return exactly what the unpartitioned reference returns. Skipped on a
single-GPU box (the CPU twin of these tests is tests/test_sharding_gloo.py)."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    import scriptonait_b200 as sb
    from scriptonait_b200 import sharding, workloads
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device(f"cuda:{rank}")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    sampler = sb.Sampler(device=rank, max_batch=256, max_vocab=262144, max_history=512, max_top_k=256)
    out = {}
    # ---- rows sharded: rank g samples its rows; the gather is control plane only
    w = workloads.c2()
    lo, hi = sharding.row_shard_range(w.batch, world, rank)
    mine = workloads.row_slice(w, lo, hi)
    res = sampler.sample_batch(torch.from_numpy(mine.logits).to(dev), history=mine.history, seeds=mine.seeds, **mine.params())
    out["rows"] = sharding.gather_rows(res.tokens, w.batch).cpu().numpy().view(np.uint32).tolist()
    # ---- vocabulary sharded (c5): select on local columns, all-gather, merge + draw on every rank
    w5 = workloads.c5()
    clo, chi = sharding.vocab_shard_ranges(w5.vocab, world)[rank]
    local = torch.from_numpy(np.ascontiguousarray(w5.logits[:, clo:chi])).to(dev)
    res5 = sharding.sample_vocab_sharded(sampler, local, column_offset=clo, vocab_global=w5.vocab, top_k=w5.top_k,
                                         temperature=w5.temperature, top_p=w5.top_p, min_p=w5.min_p, seeds=w5.seeds,
                                         cand_stride=64, trace=True)
    torch.cuda.synchronize()
    out["vocab_tokens"] = res5.tokens.cpu().numpy().view(np.uint32).tolist()
    out["vocab_kept"] = res5.kept_count.cpu().numpy().view(np.uint32).tolist()
    q.put((rank, out))
    dist.barrier()
    dist.destroy_process_group()
    sampler.close()


@pytest.mark.timeout(600)
def test_row_and_vocab_sharding_over_two_gpus_match_the_reference():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    import oracle
    import parity
    from scriptonait_b200 import workloads
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=500) for _ in range(2))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    w = workloads.c2()
    ref = parity.run_oracle(w, oracle.EXP_CR)
    assert got[0]["rows"] == got[1]["rows"] == ref.tokens.tolist()
    w5 = workloads.c5()
    ref5 = parity.run_oracle(w5, oracle.EXP_CR)
    assert got[0]["vocab_tokens"] == got[1]["vocab_tokens"] == ref5.tokens.tolist()
    assert got[0]["vocab_kept"] == ref5.kept_count.tolist()
