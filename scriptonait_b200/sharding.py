"""Multi-GPU partitioning of the sampling path: one process per GPU.

The reference is single-device (it has no collective anywhere), so there is no reference
interface to mirror here; what must hold is that a partitioned run returns exactly what
one `sample_with` per row returns (crates/llm-core/src/generate.rs:325-420).

* Row sharding: `sample_with` is a pure function of one row, its parameters, its history
  and its own RNG, so rank g takes rows [lo, hi) with their parameters and seeds and no
  data-path collective exists. Concatenating the ranks' tokens is the result.
* Vocabulary sharding: rank g holds columns [lo, hi) of every row. Each rank selects its
  best top_k candidates per row (step 1), one all-gather moves the fixed-size lists
  (NCCL over NVLink when the process group is NCCL), and every rank merges and draws
  (step 2) - all ranks obtain the same tokens. Exact because the global top-k is a
  subset of the union of per-shard top-k lists and the softmax runs over the kept k only
  (generate.rs:368-380). top_k == 0 is rejected (it would need a second exchange).
"""
from __future__ import annotations

from typing import List, Optional, Tuple


def row_shard_range(batch: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Rows [lo, hi) of rank `rank`: contiguous, sizes differ by at most one, every row
    owned exactly once."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError("bad rank / world_size")
    base, extra = divmod(batch, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def vocab_shard_ranges(vocab: int, n_shards: int, align: int = 64) -> List[Tuple[int, int]]:
    """Column ranges of the shards: contiguous, `align`-column multiples except the last,
    covering [0, vocab) exactly once. Shards past the end of a tiny vocabulary are empty."""
    if n_shards <= 0:
        raise ValueError("n_shards must be positive")
    per = -(-vocab // n_shards)
    per = -(-per // align) * align
    out = []
    for s in range(n_shards):
        lo = min(s * per, vocab)
        out.append((lo, min(lo + per, vocab)))
    return out


def gather_rows(local_tokens, batch: int, group=None):
    """Concatenates the ranks' token slices of a row-sharded batch on every rank (control
    plane only: the sampling itself needed no exchange). `local_tokens` is a torch tensor;
    works on NCCL (CUDA tensors) and on gloo (CPU tensors)."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    sizes = [row_shard_range(batch, world, r) for r in range(world)]
    width = max(hi - lo for lo, hi in sizes)
    padded = torch.zeros(width, dtype=local_tokens.dtype, device=local_tokens.device)
    padded[:local_tokens.numel()] = local_tokens
    gathered = torch.empty(world * width, dtype=local_tokens.dtype, device=local_tokens.device)
    dist.all_gather_into_tensor(gathered, padded, group=group)
    parts = [gathered[r * width:r * width + (hi - lo)] for r, (lo, hi) in enumerate(sizes)]
    return torch.cat(parts)


def all_gather_candidates(values, ids, counts, group=None):
    """The one exchange of vocabulary sharding: fixed-size candidate lists [B, S] (+ counts
    [B]) of every rank -> [G, B, S] / [G, B] on every rank. Three all-gathers of
    B*S*4, B*S*4 and B*4 bytes per rank."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    gv = torch.empty((world,) + tuple(values.shape), dtype=values.dtype, device=values.device)
    gi = torch.empty((world,) + tuple(ids.shape), dtype=ids.dtype, device=ids.device)
    gc = torch.empty((world,) + tuple(counts.shape), dtype=counts.dtype, device=counts.device)
    # flat views: both NCCL and gloo accept "output = concatenation of the ranks' inputs"
    dist.all_gather_into_tensor(gv.view(-1), values.contiguous().view(-1), group=group)
    dist.all_gather_into_tensor(gi.view(-1), ids.contiguous().view(-1), group=group)
    dist.all_gather_into_tensor(gc.view(-1), counts.contiguous().view(-1), group=group)
    return gv, gi, gc


def sample_vocab_sharded(sampler, local_logits, *, column_offset: int, vocab_global: int, top_k: int,
                         temperature=1.0, top_p=1.0, min_p=0.0, repetition_penalty=1.0, history=None, seeds=None,
                         draw_index=None, seed_base: int = 0, cand_stride: Optional[int] = None, group=None,
                         trace: bool = False):
    """Vocabulary-sharded `sample_with` for a batch: select on this rank's columns,
    all-gather the lists, merge and draw. Returns the merge's SampleResult (same tokens on
    every rank)."""
    stride = int(cand_stride or max(top_k, 1))
    vals, ids, cnt = sampler.shard_select(local_logits, column_offset=column_offset, vocab_global=vocab_global,
                                          cand_stride=stride, temperature=temperature, top_k=top_k,
                                          repetition_penalty=repetition_penalty, history=history)
    gv, gi, gc = all_gather_candidates(vals, ids, cnt, group=group)
    return sampler.merge_draw(gv, gi, gc, vocab_global=vocab_global, temperature=temperature, top_k=top_k, top_p=top_p,
                              min_p=min_p, seeds=seeds, draw_index=draw_index, seed_base=seed_base, trace=trace)
