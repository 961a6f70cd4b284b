"""Parity harness: runs a workload through the CUDA library (C ABI) and through the CPU
oracle on the same bytes and the same seeded uniform stream, and compares token ids,
kept sets, probabilities and stage statistics.

Two oracle definitions of exp are used (see oracle/sampler_oracle.cpp):
  EXP_CR    bit-for-bit bar: every compared quantity must be identical;
  EXP_LIBM  the reference's native definition (this host's expf): probabilities within
            1e-6 relative; token / kept-set differences allowed only at a cut or draw
            boundary within 1e-6 relative of the cumulative mass, classified and counted;
            "unexplained" must be 0.
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import numpy as np

import oracle
from scriptonait_b200 import native as N
from scriptonait_b200.workloads import Workload

REL_TOL = 1e-6
SEMANTIC_FLAGS = N.ROW_GREEDY | N.ROW_DEGENERATE | N.ROW_FALLBACK_LAST | N.ROW_DRAW_CONSUMED


@dataclasses.dataclass
class GpuOut:
    tokens: np.ndarray
    flags: np.ndarray
    kept_count: np.ndarray
    kept_ids: np.ndarray
    kept_probs: np.ndarray
    stats: np.ndarray


@dataclasses.dataclass
class Report:
    rows: int = 0
    token_matches: int = 0
    kept_matches: int = 0
    top_k_tie: int = 0
    min_p_boundary: int = 0
    top_p_boundary: int = 0
    draw_boundary: int = 0
    unexplained: int = 0
    max_rel_prob: float = 0.0
    max_rel_sum: float = 0.0
    uniforms_equal: bool = True
    full_sort_rows: int = 0
    windowed_rows: int = 0
    notes: list = dataclasses.field(default_factory=list)

    def summary(self) -> str:
        return (f"rows={self.rows} token_match={self.token_matches} kept_match={self.kept_matches} "
                f"top_k_tie={self.top_k_tie} min_p_boundary={self.min_p_boundary} top_p_boundary={self.top_p_boundary} "
                f"draw_boundary={self.draw_boundary} unexplained={self.unexplained} max_rel_prob={self.max_rel_prob:.3g} "
                f"max_rel_sum={self.max_rel_sum:.3g} u_equal={self.uniforms_equal} full_sort_rows={self.full_sort_rows} "
                f"windowed_rows={self.windowed_rows}")


def run_oracle(w: Workload, exp_mode: int = oracle.EXP_CR, kept_capacity: int = 64, threads: int = 0,
               allowed: Optional[np.ndarray] = None) -> oracle.BatchResult:
    return oracle.sample_batch(w.logits, batch=w.batch, row_stride=0 if w.broadcast_row else None, history=w.history,
                               seeds=w.seeds, draw_index=w.draw_index, allowed=allowed, kept_capacity=kept_capacity,
                               exp_mode=exp_mode, threads=threads, **w.params())


def device_logits(w: Workload, device="cuda:0"):
    import torch
    lg = torch.from_numpy(w.logits.view(np.int16) if w.is_bf16 else w.logits).to(device)
    return lg.view(torch.bfloat16) if w.is_bf16 else lg


def run_gpu(sampler, w: Workload, kept_capacity: int = 64, allowed: Optional[np.ndarray] = None, logits_dev=None,
            **kwargs) -> GpuOut:
    import torch
    lg = logits_dev if logits_dev is not None else device_logits(w)
    extra = {}
    if allowed is not None:
        bits, n = sampler.pack_allowed(allowed)
        extra.update(allowed_bits=bits, allowed_len=n)
    res = sampler.sample_batch(lg, history=w.history, seeds=w.seeds, draw_index=w.draw_index, batch=w.batch,
                               row_stride=0 if w.broadcast_row else None, trace=True, kept_capacity=kept_capacity,
                               **w.params(), **extra, **kwargs)
    torch.cuda.synchronize()
    u32 = lambda t: t.cpu().numpy().view(np.uint32)
    return GpuOut(u32(res.tokens), u32(res.row_flags), u32(res.kept_count), u32(res.kept_ids),
                  res.kept_probs.cpu().numpy(), res.row_stats.cpu().numpy())


def _rel(a: float, b: float) -> float:
    d = abs(float(a) - float(b))
    m = max(abs(float(a)), abs(float(b)))
    return 0.0 if d == 0.0 else d / m if m > 0 else np.inf


def _row_param(x, r):
    return float(x[r]) if isinstance(x, np.ndarray) else float(x)


def compare(orc: oracle.BatchResult, gpu: GpuOut, w: Workload, exact: bool) -> Report:
    rep = Report(rows=w.batch)
    cap = orc.kept_ids.shape[1]
    for r in range(w.batch):
        of, gf = int(orc.flags[r]), int(gpu.flags[r])
        if gf & N.ROW_FULL_SORT:
            rep.full_sort_rows += 1
        if gf & N.ROW_WINDOWED:
            rep.windowed_rows += 1
        tok_ok = int(orc.tokens[r]) == int(gpu.tokens[r])
        drew = bool(of & oracle.FLAG_DRAW_CONSUMED)
        if (of & SEMANTIC_FLAGS & ~N.ROW_FALLBACK_LAST) != (gf & SEMANTIC_FLAGS & ~N.ROW_FALLBACK_LAST):
            rep.unexplained += 1
            rep.notes.append(f"row {r}: flags oracle={of:#x} gpu={gf:#x}")
            continue
        if not drew:  # greedy / degenerate rows: only the token is defined
            rep.token_matches += tok_ok
            rep.kept_matches += 1
            if not tok_ok:
                rep.unexplained += 1
                rep.notes.append(f"row {r}: non-drawing row token oracle={orc.tokens[r]} gpu={gpu.tokens[r]}")
            continue
        if orc.stats[r, 3] != gpu.stats[r, 3]:
            rep.uniforms_equal = False
        oc, gc = int(orc.kept_count[r]), int(gpu.kept_count[r])
        n = min(oc, gc, cap)
        ids_prefix_ok = np.array_equal(orc.kept_ids[r, :n], gpu.kept_ids[r, :n])
        kept_ok = (oc == gc) and ids_prefix_ok
        op, gp = orc.kept_probs[r, :n], gpu.kept_probs[r, :n]
        if n:
            with np.errstate(divide="ignore", invalid="ignore"):
                rel = np.abs(op.astype(np.float64) - gp) / np.maximum(np.abs(op), np.abs(gp))
            rel = np.where(op == gp, 0.0, rel)
            rep.max_rel_prob = max(rep.max_rel_prob, float(rel.max()))
        rep.max_rel_sum = max(rep.max_rel_sum, _rel(orc.stats[r, 1], gpu.stats[r, 1]))
        if exact:
            same = kept_ok and tok_ok and np.array_equal(op, gp) and np.array_equal(orc.stats[r], gpu.stats[r]) and \
                ((of ^ gf) & N.ROW_FALLBACK_LAST) == 0
            rep.token_matches += tok_ok
            rep.kept_matches += kept_ok
            if not same:
                rep.unexplained += 1
                rep.notes.append(f"row {r}: exact mismatch tok {orc.tokens[r]}/{gpu.tokens[r]} kept {oc}/{gc} "
                                 f"stats {orc.stats[r]} / {gpu.stats[r]}")
            continue
        rep.token_matches += tok_ok
        rep.kept_matches += kept_ok
        if kept_ok and tok_ok:
            continue
        # ---- classify the difference
        top_p = _row_param(w.top_p, r)
        min_p = _row_param(w.min_p, r)
        if not ids_prefix_ok:
            # the ordering itself differs: only a value tie at the top-k edge could explain it,
            # and ties are broken identically by index on both sides
            rep.unexplained += 1
            rep.notes.append(f"row {r}: kept ids differ before the cut")
            continue
        if oc != gc:
            longer = orc if oc > gc else gpu
            cut = min(oc, gc)
            if cut >= cap:
                rep.unexplained += 1
                rep.notes.append(f"row {r}: cut beyond trace capacity")
                continue
            lp = longer.kept_probs[r]
            explained = False
            if min_p > 0.0:
                thr = float(longer.stats[r, 4])
                if _rel(lp[cut], thr) <= REL_TOL:
                    rep.min_p_boundary += 1
                    explained = True
            if not explained and top_p < 1.0:
                cum = float(np.cumsum(lp[:cut].astype(np.float64))[-1]) if cut else 0.0
                if abs(cum - top_p) <= REL_TOL * max(cum, top_p):
                    rep.top_p_boundary += 1
                    explained = True
            if not explained:
                rep.unexplained += 1
                rep.notes.append(f"row {r}: kept {oc} vs {gc} not at a boundary")
            continue
        # same kept set, different token: the draw landed on a boundary of the cumulative mass
        m = min(oc, cap)
        cum = np.cumsum(orc.kept_probs[r, :m].astype(np.float64))
        total = float(orc.stats[r, 2])
        rr = float(orc.stats[r, 5])
        if m and np.min(np.abs(cum - rr)) <= REL_TOL * max(total, 1e-30):
            rep.draw_boundary += 1
        else:
            rep.unexplained += 1
            rep.notes.append(f"row {r}: token {orc.tokens[r]} vs {gpu.tokens[r]} away from any boundary")
    return rep


def assert_exact(rep: Report):
    assert rep.unexplained == 0 and rep.token_matches == rep.rows and rep.kept_matches == rep.rows and rep.uniforms_equal, \
        rep.summary() + "\n" + "\n".join(rep.notes[:10])


def assert_within_tolerance(rep: Report):
    assert rep.unexplained == 0 and rep.uniforms_equal and rep.max_rel_prob <= REL_TOL, \
        rep.summary() + "\n" + "\n".join(rep.notes[:10])
