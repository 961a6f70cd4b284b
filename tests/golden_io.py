"""Loads tests/golden/sampler_cases.npz back into Workload objects + the frozen oracle outputs."""
import os

import numpy as np

import oracle
from scriptonait_b200.workloads import Workload

PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "sampler_cases.npz")


def _param(a):
    return a.item() if a.ndim == 0 else a


def load():
    z = np.load(PATH)
    names = sorted({k.split("/")[0] for k in z.files})
    out = {}
    for n in names:
        batch, broadcast = (int(v) for v in z[f"{n}/meta"])
        w = Workload(n, z[f"{n}/logits"], temperature=_param(z[f"{n}/temperature"]), top_k=_param(z[f"{n}/top_k"]),
                     top_p=_param(z[f"{n}/top_p"]), min_p=_param(z[f"{n}/min_p"]),
                     repetition_penalty=_param(z[f"{n}/repetition_penalty"]),
                     history=z[f"{n}/history"] if f"{n}/history" in z.files else None, seeds=z[f"{n}/seeds"],
                     draw_index=z[f"{n}/draw_index"] if f"{n}/draw_index" in z.files else None,
                     broadcast_row=bool(broadcast), batch=batch)
        frozen = {}
        for tag in ("cr", "libm"):
            frozen[tag] = oracle.BatchResult(z[f"{n}/{tag}/tokens"], z[f"{n}/{tag}/flags"], z[f"{n}/{tag}/kept_count"],
                                             z[f"{n}/{tag}/kept_ids"], z[f"{n}/{tag}/kept_probs"], z[f"{n}/{tag}/stats"])
        out[n] = (w, frozen)
    return out
