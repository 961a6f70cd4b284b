"""Times the sampler on the named synthetic workloads (c1..c5), one JSON line per workload.

    python -m scriptonait_b200.timing c4-k64 c5 --steps 200

`ce` times `llm_cuda_cross_entropy` (loss + gradient) over 256 x 128256 f32 logits instead.

Logits are resident on the GPU; a step is one `llm_cuda_sample_batch` call over the whole batch.
Inputs rotate over enough copies of the batch to exceed the 126 MB L2 (a copy holds the same values
at another address, so every step misses L2 the same way). Timed with CUDA events on the launching
stream after warm-up. `--overlap` lets consecutive steps overlap (independent outputs per copy).
The fraction is algorithmic bytes (one read of each logits row and history, one token written)
per second over the measured HBM copy rate passed as `--peak-gbs`.
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from . import workloads
from .sampler import Sampler

L2_BYTES = 126e6


def make(name: str) -> workloads.Workload:
    if name == "c1":
        return workloads.c1(1000)
    if name == "c2":
        return workloads.c2()
    if name == "c3":
        return workloads.c3()
    if name.startswith("c4-k"):
        return workloads.c4(int(name[4:]))
    if name == "c5":
        return workloads.c5()
    raise SystemExit(f"unknown workload {name!r}: c1 c2 c3 c4-k<K> c5")


def time_workload(sampler: Sampler, w: workloads.Workload, steps: int, warmup: int, overlap: bool) -> dict:
    import torch
    copies = int(max(1, min(8, L2_BYTES * 1.5 // max(w.logits.nbytes, 1) + 1)))
    calls = []
    for _ in range(copies):
        t = torch.from_numpy(w.logits.view(np.int16) if w.is_bf16 else w.logits).to("cuda")
        lg = t.view(torch.bfloat16) if w.is_bf16 else t
        calls.append(sampler.sample_batch(lg, history=w.history, seeds=w.seeds, draw_index=w.draw_index, batch=w.batch,
                                          row_stride=0 if w.broadcast_row else None, prepare_only=True,
                                          overlap_previous=overlap, **w.params()))
    for i in range(max(warmup, 3)):
        calls[i % copies].launch()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        calls[i % copies].launch()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / steps * 1e3
    kernels, split = sampler.last_launch_info()
    return {"workload": w.name, "rows": w.batch, "vocab": w.vocab, "logits_dtype": "bf16" if w.is_bf16 else "f32",
            "us_per_step": us, "rows_per_s": w.batch / (us * 1e-6), "algorithmic_gbs": w.algorithmic_bytes() / us / 1e3,
            "kernels_per_step": kernels, "ctas_per_row": split, "copies": copies, "overlap": overlap, "steps": steps}


def time_cross_entropy(sampler: Sampler, steps: int, warmup: int) -> dict:
    import torch
    rows, vocab = 256, 128256
    gen = torch.Generator(device="cuda")
    gen.manual_seed(77)
    xs = [torch.randn((rows, vocab), generator=gen, device="cuda") * 2.0 for _ in range(3)]  # 394 MB against 126 MB of L2
    tg = torch.randint(0, vocab, (rows,), generator=gen, device="cuda", dtype=torch.int32)
    for i in range(max(warmup, 3)):
        sampler.cross_entropy(xs[i % 3], tg)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        sampler.cross_entropy(xs[i % 3], tg)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / steps * 1e3
    return {"workload": "ce", "rows": rows, "vocab": vocab, "logits_dtype": "f32", "us_per_step": us,
            "algorithmic_gbs": rows * vocab * 8 / us / 1e3, "kernels_per_step": 1, "copies": 3, "steps": steps}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("workloads", nargs="*", default=["c3", "c2", "c4-k1", "c4-k64", "c4-k1024", "c5", "c1"])
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--overlap", action="store_true")
    ap.add_argument("--peak-gbs", type=float, default=0.0, help="measured HBM copy rate, for the fraction")
    args = ap.parse_args()
    sampler = Sampler(device=0, max_batch=1024, max_vocab=262144, max_history=512, max_top_k=1024)
    try:
        for name in args.workloads:
            line = (time_cross_entropy(sampler, args.steps, args.warmup) if name == "ce"
                    else time_workload(sampler, make(name), args.steps, args.warmup, args.overlap))
            if args.peak_gbs > 0:
                line["frac_of_peak"] = line["algorithmic_gbs"] / args.peak_gbs
            print(json.dumps(line), flush=True)
    finally:
        sampler.close()


if __name__ == "__main__":
    main()
