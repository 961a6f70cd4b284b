"""Generates tests/golden/sampler_cases.npz: small seeded inputs of the sampling path with the
CPU oracle's outputs (token ids, kept sets, probabilities, stage statistics, flags).

The reference itself (Rust) cannot be run where this repository is built, so these are not
outputs of the reference binary; they freeze the oracle's restatement of
crates/llm-core/src/generate.rs:325-420 on the machine that generated them, under both exp
definitions (EXP_CR: double exp rounded to f32, EXP_LIBM: that host's expf), so that a later
change of the oracle, of the C library or of the CUDA path shows up as a diff.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle  # noqa: E402
from scriptonait_b200 import workloads  # noqa: E402

KEPT = 64


def cases():
    """name -> Workload; small enough to commit, varied enough to touch every stage."""
    g = np.random.Generator(np.random.PCG64(777))
    out = {}
    out["c1_first_32_draws"] = workloads.c1(32)
    out["c2_16x4096"] = workloads.c2(batch=16, vocab=4096, hist_len=64)
    out["c3_8x8192_bf16"] = workloads.c3(batch=8, vocab=8192)
    out["c4_k64_12x5003"] = workloads.c4(64, batch=12, vocab=5003, hist_len=96)
    out["c5_6x16384"] = workloads.c5(batch=6, vocab=16384)
    x = g.normal(0, 2, (10, 1000)).astype(np.float32)
    x[3, :] = -np.inf
    x[4, 7] = np.inf
    out["mixed_modes"] = workloads.Workload(
        "mixed", x, temperature=np.array([0.0, 0.7, 1.0, 1.0, 1.0, 1.3, 0.0, 0.9, 1.0, 2.0], np.float32),
        top_k=np.array([0, 1, 5, 0, 10, 40, 3, 1000, 0, 50], np.uint32),
        top_p=np.array([1, .9, .5, 1, 1, .95, 1, .99, 1, .3], np.float32),
        min_p=np.array([0, 0, .05, 0, 0, .1, 0, 0, 2.0, 0], np.float32),
        repetition_penalty=np.array([1.5, 1.0, 1.2, 1.0, 1.0, 1.1, 1.3, 0.8, 1.0, 1.0], np.float32),
        history=g.integers(0, 1100, size=(10, 24), dtype=np.uint32), seeds=np.arange(10, dtype=np.uint64) + np.uint64(5),
        batch=10)
    return out


def main():
    blob = {}
    for name, w in cases().items():
        blob[f"{name}/logits"] = w.logits
        for key in ("temperature", "top_k", "top_p", "min_p", "repetition_penalty"):
            blob[f"{name}/{key}"] = np.asarray(getattr(w, key))
        if w.history is not None:
            blob[f"{name}/history"] = w.history
        blob[f"{name}/seeds"] = w.seeds
        if w.draw_index is not None:
            blob[f"{name}/draw_index"] = w.draw_index
        blob[f"{name}/meta"] = np.array([w.batch, int(w.broadcast_row)], np.int64)
        for tag, mode in (("cr", oracle.EXP_CR), ("libm", oracle.EXP_LIBM)):
            r = oracle.sample_batch(w.logits, batch=w.batch, row_stride=0 if w.broadcast_row else None, history=w.history,
                                    seeds=w.seeds, draw_index=w.draw_index, kept_capacity=KEPT, exp_mode=mode, threads=1,
                                    **w.params())
            blob[f"{name}/{tag}/tokens"] = r.tokens
            blob[f"{name}/{tag}/flags"] = r.flags
            blob[f"{name}/{tag}/kept_count"] = r.kept_count
            blob[f"{name}/{tag}/kept_ids"] = r.kept_ids
            blob[f"{name}/{tag}/kept_probs"] = r.kept_probs
            blob[f"{name}/{tag}/stats"] = r.stats
    path = os.path.join(HERE, "sampler_cases.npz")
    np.savez_compressed(path, **blob)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
