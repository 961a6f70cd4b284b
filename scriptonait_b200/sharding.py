"""Multi-GPU partitioning of the sampling path: one process per GPU.

The reference is single-device (it has no collective anywhere), so there is no reference
interface to mirror here; what must hold is that a partitioned run returns exactly what
one `sample_with` per row returns (crates/llm-core/src/generate.rs:325-420).

* Row sharding: `sample_with` is a pure function of one row, its parameters, its history
  and its own RNG, so rank g takes rows [lo, hi) with their parameters and seeds and no
  data-path collective exists. Concatenating the ranks' tokens is the result.
* Vocabulary sharding: rank g holds columns [lo, hi) of every row. Each rank selects its
  best top_k candidates per row (step 1) into one packed block, ONE all-gather moves the blocks
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


def packed_words(batch: int, cand_stride: int) -> int:
    """32-bit words of one rank's packed candidate block: values [B, S] f32, ids [B, S] u32, counts [B] u32."""
    return 2 * batch * cand_stride + batch


def unpack_candidates(packed_all, batch: int, cand_stride: int):
    """Views of an all-gathered [G, packed_words] int32 buffer: values [G, B, S] (f32), ids [G, B, S], counts [G, B]."""
    import torch
    G = packed_all.shape[0]
    bs = batch * cand_stride
    vals = packed_all[:, :bs].view(torch.float32).view(G, batch, cand_stride)
    ids = packed_all[:, bs:2 * bs].view(G, batch, cand_stride)
    cnt = packed_all[:, 2 * bs:]
    return vals, ids, cnt


def all_gather_packed(packed, group=None, out=None):
    """The one exchange of vocabulary sharding: every rank's packed candidate block (a flat int32 tensor
    of `packed_words` words, 16.5 KB for 32 rows of 64 candidates) -> [G, packed_words] on every rank, in
    ONE all-gather (NCCL over NVLink for CUDA tensors, gloo for CPU tensors)."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if out is None:
        out = torch.empty((world, packed.numel()), dtype=packed.dtype, device=packed.device)
    dist.all_gather_into_tensor(out.view(-1), packed.view(-1), group=group)
    return out


def sample_vocab_sharded(sampler, local_logits, *, column_offset: int, vocab_global: int, top_k: int,
                         temperature=1.0, top_p=1.0, min_p=0.0, repetition_penalty=1.0, history=None, seeds=None,
                         draw_index=None, seed_base: int = 0, cand_stride: Optional[int] = None, group=None,
                         trace: bool = False):
    """Vocabulary-sharded `sample_with` for a batch: select on this rank's columns,
    all-gather the lists, merge and draw. Returns the merge's SampleResult (same tokens on
    every rank)."""
    stride = int(cand_stride or max(top_k, 1))
    packed = sampler.shard_select_packed(local_logits, column_offset=column_offset, vocab_global=vocab_global,
                                         cand_stride=stride, temperature=temperature, top_k=top_k,
                                         repetition_penalty=repetition_penalty, history=history)
    gathered = all_gather_packed(packed, group=group)
    return sampler.merge_draw_packed(gathered, batch=int(local_logits.shape[0]), cand_stride=stride,
                                     vocab_global=vocab_global, temperature=temperature, top_k=top_k, top_p=top_p,
                                     min_p=min_p, seeds=seeds, draw_index=draw_index, seed_base=seed_base, trace=trace)
