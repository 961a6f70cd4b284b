"""Seeded synthetic inputs for the five sampling workloads (c1..c5).

The reference quotes no dataset for its sampler; these generators stand in for
"a logits matrix out of the LM head" with the shapes, dtypes and value
distributions the workloads name. Everything comes from numpy's PCG64 with
`data_seed = 20260 + workload index`, so the CUDA path, the CPU oracle and the
golden fixtures all see the same bytes. Sampler seeds are `1234 + row`.

bf16 logits are produced by computing in f32 and narrowing with round to
nearest even, NaN kept quiet (crates/llm-core/src/bf16.rs:11-20); they are
carried as uint16 bit patterns.
"""
from __future__ import annotations

import dataclasses
from typing import Optional, Union

import numpy as np

SEED0 = 1234
Scalar = Union[float, int]


@dataclasses.dataclass
class Workload:
    name: str
    logits: np.ndarray                 # [B, V] float32, or uint16 holding bf16 bit patterns
    temperature: Union[float, np.ndarray] = 1.0
    top_k: Union[int, np.ndarray] = 0
    top_p: Union[float, np.ndarray] = 1.0
    min_p: Union[float, np.ndarray] = 0.0
    repetition_penalty: Union[float, np.ndarray] = 1.0
    history: Optional[np.ndarray] = None   # [B, H] uint32
    seeds: Optional[np.ndarray] = None     # [B] uint64
    draw_index: Optional[np.ndarray] = None
    broadcast_row: bool = False            # c1: B draws from one row (row stride 0)
    batch: int = 0

    @property
    def vocab(self) -> int:
        return int(self.logits.shape[-1])

    @property
    def is_bf16(self) -> bool:
        return self.logits.dtype == np.uint16

    @property
    def history_len(self) -> int:
        return 0 if self.history is None else int(self.history.shape[1])

    def algorithmic_bytes(self) -> int:
        """One read of each logits row, one read of its history, one token id written."""
        elem = 2 if self.is_bf16 else 4
        return self.batch * (self.vocab * elem + self.history_len * 4 + 4)

    def params(self) -> dict:
        return dict(temperature=self.temperature, top_k=self.top_k, top_p=self.top_p, min_p=self.min_p,
                    repetition_penalty=self.repetition_penalty)


def narrow_bf16(x: np.ndarray) -> np.ndarray:
    """f32 -> bf16 bit patterns, round to nearest even, NaN stays a quiet NaN."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32)
    lsb = (bits >> np.uint32(16)) & np.uint32(1)
    rounded = ((bits + np.uint32(0x7FFF) + lsb) >> np.uint32(16)).astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        rounded[nan] = ((bits[nan] >> np.uint32(16)) | np.uint32(0x0040)).astype(np.uint16)
    return rounded


def widen_bf16(h: np.ndarray) -> np.ndarray:
    """bf16 bit patterns -> f32, exact."""
    return (np.ascontiguousarray(h, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def _gen(index: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(20260 + index))


def _seeds(batch: int, row0: int = 0) -> np.ndarray:
    return (np.arange(batch, dtype=np.uint64) + np.uint64(SEED0 + row0))


def c1(draws: int = 1000) -> Workload:
    """batch 1, vocab 8192 f32 ~ N(0, 2.0), 5 random indices boosted by +6; T 0.8, top_k 40,
    top_p 0.95, min_p 0.05, penalty 1.1 over a fixed 64-token history; one Rng(1234),
    `draws` sequential draws (draw n uses output n of the stream)."""
    g = _gen(1)
    V = 8192
    row = g.normal(0.0, 2.0, V).astype(np.float32)
    boost = g.choice(V, size=5, replace=False)
    row[boost] += np.float32(6.0)
    hist = g.integers(0, V, size=64, dtype=np.uint32)
    return Workload("c1", row[None, :], temperature=0.8, top_k=40, top_p=0.95, min_p=0.05,
                    repetition_penalty=1.1, history=np.broadcast_to(hist, (draws, 64)).copy(),
                    seeds=np.full(draws, SEED0, np.uint64), draw_index=np.arange(draws, dtype=np.uint64),
                    broadcast_row=True, batch=draws)


def c2(batch: int = 64, vocab: int = 32768, hist_len: int = 256) -> Workload:
    """batch 64, vocab 32768 f32 ~ N(0, 3.0); per-row T ~ U[0.5, 1.2]; top_k 50, top_p 0.9,
    min_p 0; penalty 1.15 over a 256-token per-row history."""
    g = _gen(2)
    logits = g.normal(0.0, 3.0, (batch, vocab)).astype(np.float32)
    temps = g.uniform(0.5, 1.2, batch).astype(np.float32)
    hist = g.integers(0, vocab, size=(batch, hist_len), dtype=np.uint32)
    return Workload("c2", logits, temperature=temps, top_k=50, top_p=0.9, min_p=0.0,
                    repetition_penalty=1.15, history=hist, seeds=_seeds(batch), batch=batch)


def c3(batch: int = 256, vocab: int = 128256, row0: int = 0, variant: int = 0) -> Workload:
    """batch 256, vocab 128256 bf16 = Gumbel(0,1) + 4*ln(1/(rank+1)) placed through a random
    permutation per row; min_p 0.05 only (T 1.0, no top-k, no top-p, no penalty). `row0`
    offsets the sampler seeds (row-sharded ranks pass their first global row); `variant`
    gives an independent batch of the same distribution (rotating bench buffers)."""
    g = np.random.Generator(np.random.PCG64([20263, variant, row0]))
    bias = (4.0 * np.log(1.0 / (np.arange(vocab, dtype=np.float64) + 1.0))).astype(np.float32)
    out = np.empty((batch, vocab), np.uint16)
    for b in range(batch):
        vals = g.gumbel(0.0, 1.0, vocab).astype(np.float32) + bias
        perm = g.permutation(vocab)
        row = np.empty(vocab, np.float32)
        row[perm] = vals
        out[b] = narrow_bf16(row)
    return Workload("c3", out, temperature=1.0, top_k=0, top_p=1.0, min_p=0.05, repetition_penalty=1.0,
                    seeds=_seeds(batch, row0), batch=batch)


def c4(top_k: int, batch: int = 1024, vocab: int = 50257, hist_len: int = 512) -> Workload:
    """batch 1024, vocab 50257 f32 near-flat ~ N(0, 0.3); top_p 0.99, top_k from the sweep
    {1, 8, 64, 256, 1024}; penalty 1.3 over a 512-token history. The workload names no
    temperature or min_p: T 1.0 and min_p 0 are assumed."""
    g = _gen(4)
    logits = g.normal(0.0, 0.3, (batch, vocab)).astype(np.float32)
    hist = g.integers(0, vocab, size=(batch, hist_len), dtype=np.uint32)
    return Workload(f"c4-k{top_k}", logits, temperature=1.0, top_k=top_k, top_p=0.99, min_p=0.0,
                    repetition_penalty=1.3, history=hist, seeds=_seeds(batch), batch=batch)


def c5(batch: int = 32, vocab: int = 262144) -> Workload:
    """batch 32, vocab 262144 f32 ~ N(0, 2.5) with 1% of entries set to -inf; T 0.7, top_k 64,
    top_p 0.95; meant to be split by vocabulary columns over 2/4/8 GPUs."""
    g = _gen(5)
    logits = g.normal(0.0, 2.5, (batch, vocab)).astype(np.float32)
    logits[g.random((batch, vocab)) < 0.01] = -np.inf
    return Workload("c5", logits, temperature=0.7, top_k=64, top_p=0.95, min_p=0.0, repetition_penalty=1.0,
                    seeds=_seeds(batch), batch=batch)


def row_slice(w: Workload, lo: int, hi: int) -> Workload:
    """Rows [lo, hi) of a workload with their parameters, history and seeds (row sharding)."""
    def cut(x):
        return x[lo:hi] if isinstance(x, np.ndarray) else x
    return dataclasses.replace(
        w, logits=w.logits if w.broadcast_row else w.logits[lo:hi], temperature=cut(w.temperature),
        top_k=cut(w.top_k), top_p=cut(w.top_p), min_p=cut(w.min_p), repetition_penalty=cut(w.repetition_penalty),
        history=cut(w.history), seeds=cut(w.seeds), draw_index=cut(w.draw_index), batch=hi - lo)
