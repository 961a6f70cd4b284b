"""ctypes binding of the CPU oracle (oracle/sampler_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
bench's CPU-baseline and reference arms. The product package never imports it.

The oracle restates the reference sampler (crates/llm-core/src/generate.rs:325-420,
rng.rs:10-34, ops/loss.rs:6-16, bf16.rs:11-25); see the header of the C++ file
for what pins it and what remains unpinned.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import os
from typing import Optional, Sequence

import numpy as np

from . import build as _build

EXP_LIBM = 0  # this host's expf: what a native build of the reference computes here
EXP_CR = 1    # correctly rounded exp (double exp rounded to float)

FLAG_GREEDY = 1
FLAG_DEGENERATE = 2
FLAG_FALLBACK_LAST = 4
FLAG_DRAW_CONSUMED = 8
FLAG_NAN_INPUT = 32

EOS = 258  # crates/llm-core/src/tokenizer.rs:38
GOLDEN_GAMMA = 0x9E3779B97F4A7C15
MASK64 = (1 << 64) - 1


class _Config(C.Structure):
    _fields_ = [
        ("temperature", C.c_float), ("top_k", C.c_uint32), ("top_p", C.c_float), ("min_p", C.c_float),
        ("repetition_penalty", C.c_float), ("allowed", C.c_void_p), ("allowed_len", C.c_uint32),
        ("eos_id", C.c_uint32), ("exp_mode", C.c_uint32),
    ]


class _Trace(C.Structure):
    _fields_ = [
        ("kept_count", C.c_void_p), ("kept_ids", C.c_void_p), ("kept_probs", C.c_void_p),
        ("kept_capacity", C.c_uint32), ("stats", C.c_void_p), ("flags", C.c_void_p), ("work", C.c_void_p),
    ]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        path = _build.build()
        L = C.CDLL(path)
        L.oracle_rng_next_u64.restype = C.c_uint64
        L.oracle_rng_next_u64.argtypes = [C.POINTER(C.c_uint64)]
        L.oracle_rng_next_f32.restype = C.c_float
        L.oracle_rng_next_f32.argtypes = [C.POINTER(C.c_uint64)]
        L.oracle_argmax.restype = C.c_uint32
        L.oracle_argmax.argtypes = [C.c_void_p, C.c_uint32]
        L.oracle_to_bf16.restype = C.c_uint16
        L.oracle_to_bf16.argtypes = [C.c_float]
        L.oracle_from_bf16.restype = C.c_float
        L.oracle_from_bf16.argtypes = [C.c_uint16]
        L.oracle_widen_bf16.restype = None
        L.oracle_widen_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]
        L.oracle_narrow_bf16.restype = None
        L.oracle_narrow_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]
        L.oracle_sample_with.restype = C.c_uint32
        L.oracle_sample_with.argtypes = [C.c_void_p, C.c_uint32, C.POINTER(_Config), C.c_void_p, C.c_uint32,
                                         C.POINTER(C.c_uint64), C.POINTER(_Trace)]
        L.oracle_sample.restype = C.c_uint32
        L.oracle_sample.argtypes = [C.c_void_p, C.c_uint32, C.c_float, C.c_uint32, C.POINTER(C.c_uint64)]
        L.oracle_sample_batch.restype = None
        L.oracle_sample_batch.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint64,
                                          C.POINTER(_Config)] + [C.c_void_p] * 6 + [C.c_uint32] + \
                                         [C.c_void_p] * 7 + [C.c_uint32, C.c_void_p, C.c_void_p, C.c_uint32]
        L.oracle_penalized_at_history.restype = None
        L.oracle_penalized_at_history.argtypes = [C.c_void_p, C.c_uint32, C.POINTER(_Config), C.c_void_p,
                                                  C.c_uint32, C.c_void_p]
        L.oracle_hardware_threads.restype = C.c_uint32
        _lib = L
    return _lib


def _ptr(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


@dataclasses.dataclass
class SamplingConfig:
    """Field-for-field mirror of the reference's SamplingConfig with its defaults
    (crates/llm-core/src/generate.rs:24-95)."""
    temperature: float = 0.9
    top_k: int = 40
    top_p: float = 0.95
    min_p: float = 0.0
    repetition_penalty: float = 1.1
    repetition_window: int = 128
    seed: int = 0
    allowed: Optional[np.ndarray] = None  # bool per id, or None


class Rng:
    """SplitMix64 (crates/llm-core/src/rng.rs:10-34); the state lives in a C uint64."""

    def __init__(self, seed: int):
        self._state = C.c_uint64(seed & MASK64)

    @classmethod
    def seed_from_u64(cls, seed: int) -> "Rng":
        return cls(seed)

    @property
    def state(self) -> int:
        return self._state.value

    def next_u64(self) -> int:
        return lib().oracle_rng_next_u64(C.byref(self._state))

    def next_f32(self) -> float:
        return lib().oracle_rng_next_f32(C.byref(self._state))


@dataclasses.dataclass
class Trace:
    token: int
    flags: int
    kept_count: int
    kept_ids: np.ndarray
    kept_probs: np.ndarray
    stats: np.ndarray  # max, sum, total, u, min-p threshold, r
    work: Optional[np.ndarray] = None


def _config_struct(cfg: SamplingConfig, exp_mode: int, keepalive: list) -> _Config:
    s = _Config()
    s.temperature = cfg.temperature
    s.top_k = int(cfg.top_k)
    s.top_p = cfg.top_p
    s.min_p = cfg.min_p
    s.repetition_penalty = cfg.repetition_penalty
    if cfg.allowed is not None:
        a = np.ascontiguousarray(np.asarray(cfg.allowed).astype(np.uint8))
        keepalive.append(a)
        s.allowed = a.ctypes.data
        s.allowed_len = a.size
    else:
        s.allowed = None
        s.allowed_len = 0
    s.eos_id = EOS
    s.exp_mode = exp_mode
    return s


def sample_with(logits: np.ndarray, cfg: SamplingConfig, recent: Sequence[int], rng: Rng,
                exp_mode: int = EXP_LIBM, trace: bool = False, kept_capacity: int = 0, want_work: bool = False):
    """sample_with(logits, sampling, recent, rng) of generate.rs:325-330. Returns the
    token id, or a Trace when `trace` is set."""
    row = np.ascontiguousarray(logits, dtype=np.float32)
    rec = np.ascontiguousarray(np.asarray(recent, dtype=np.uint32))
    keep: list = []
    cs = _config_struct(cfg, exp_mode, keep)
    if not trace:
        return int(lib().oracle_sample_with(_ptr(row), row.size, C.byref(cs), _ptr(rec), rec.size,
                                            C.byref(rng._state), None))
    cap = kept_capacity or row.size
    kc = np.zeros(1, np.uint32)
    ids = np.zeros(cap, np.uint32)
    pr = np.zeros(cap, np.float32)
    st = np.zeros(6, np.float32)
    fl = np.zeros(1, np.uint32)
    wk = np.zeros(row.size, np.float32) if want_work else None
    tr = _Trace(kc.ctypes.data, ids.ctypes.data, pr.ctypes.data, cap, st.ctypes.data, fl.ctypes.data,
                wk.ctypes.data if wk is not None else None)
    tok = int(lib().oracle_sample_with(_ptr(row), row.size, C.byref(cs), _ptr(rec), rec.size,
                                       C.byref(rng._state), C.byref(tr)))
    n = min(int(kc[0]), cap)
    return Trace(tok, int(fl[0]), int(kc[0]), ids[:n].copy(), pr[:n].copy(), st, wk)


def sample(logits: np.ndarray, temperature: float, rng: Rng, exp_mode: int = EXP_LIBM) -> int:
    """sample(logits, temperature, rng) of generate.rs:423-433."""
    row = np.ascontiguousarray(logits, dtype=np.float32)
    return int(lib().oracle_sample(_ptr(row), row.size, temperature, exp_mode, C.byref(rng._state)))


def argmax(row: np.ndarray) -> int:
    r = np.ascontiguousarray(row, dtype=np.float32)
    return int(lib().oracle_argmax(_ptr(r), r.size))


def to_bf16(x: np.ndarray) -> np.ndarray:
    src = np.ascontiguousarray(x, dtype=np.float32)
    dst = np.empty(src.shape, np.uint16)
    lib().oracle_narrow_bf16(_ptr(src), _ptr(dst), src.size)
    return dst


def from_bf16(h: np.ndarray) -> np.ndarray:
    src = np.ascontiguousarray(h, dtype=np.uint16)
    dst = np.empty(src.shape, np.float32)
    lib().oracle_widen_bf16(_ptr(src), _ptr(dst), src.size)
    return dst


@dataclasses.dataclass
class BatchResult:
    tokens: np.ndarray
    flags: np.ndarray
    kept_count: np.ndarray
    kept_ids: np.ndarray
    kept_probs: np.ndarray
    stats: np.ndarray


def _rows(x, batch, dtype):
    if x is None or np.isscalar(x):
        return None
    a = np.ascontiguousarray(np.asarray(x, dtype=dtype))
    assert a.shape == (batch,)
    return a


def sample_batch(logits: np.ndarray, *, temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, repetition_penalty=1.0,
                 history: Optional[np.ndarray] = None, history_len: Optional[np.ndarray] = None,
                 seeds: Optional[np.ndarray] = None, draw_index: Optional[np.ndarray] = None,
                 allowed: Optional[np.ndarray] = None, kept_capacity: int = 64, exp_mode: int = EXP_LIBM,
                 threads: int = 0, row_stride: Optional[int] = None, batch: Optional[int] = None) -> BatchResult:
    """Row r = one independent sample_with call. `logits` is [B, V] float32, or uint16
    holding bf16 bit patterns (widened exactly before the call). Scalars or [B] arrays
    for the five parameters. `row_stride=0` with `batch=N` draws N times from one row."""
    lg = np.ascontiguousarray(logits)
    if lg.ndim == 1:
        lg = lg[None, :]
    B = int(batch if batch is not None else lg.shape[0])
    V = int(lg.shape[1])
    stride = int(V if row_stride is None else row_stride)
    is_bf16 = lg.dtype == np.uint16
    if not is_bf16:
        lg = np.ascontiguousarray(lg, dtype=np.float32)
    keep: list = []
    scal = SamplingConfig(
        temperature=float(temperature) if np.isscalar(temperature) else 1.0,
        top_k=int(top_k) if np.isscalar(top_k) else 0,
        top_p=float(top_p) if np.isscalar(top_p) else 1.0,
        min_p=float(min_p) if np.isscalar(min_p) else 0.0,
        repetition_penalty=float(repetition_penalty) if np.isscalar(repetition_penalty) else 1.0,
        allowed=allowed)
    cs = _config_struct(scal, exp_mode, keep)
    t_rows = _rows(temperature, B, np.float32)
    k_rows = _rows(top_k, B, np.uint32)
    p_rows = _rows(top_p, B, np.float32)
    m_rows = _rows(min_p, B, np.float32)
    r_rows = _rows(repetition_penalty, B, np.float32)
    hist = None
    hstride = 0
    hlen = None
    if history is not None:
        hist = np.ascontiguousarray(history, dtype=np.uint32)
        assert hist.ndim == 2 and hist.shape[0] == B
        hstride = hist.shape[1]
        if history_len is not None:
            hlen = np.ascontiguousarray(history_len, dtype=np.uint32)
    sd = np.ascontiguousarray(seeds if seeds is not None else np.zeros(B), dtype=np.uint64)
    di = None if draw_index is None else np.ascontiguousarray(draw_index, dtype=np.uint64)
    tokens = np.zeros(B, np.uint32)
    kc = np.zeros(B, np.uint32)
    ids = np.zeros((B, kept_capacity), np.uint32)
    pr = np.zeros((B, kept_capacity), np.float32)
    st = np.zeros((B, 6), np.float32)
    fl = np.zeros(B, np.uint32)
    nthreads = threads or int(lib().oracle_hardware_threads())
    lib().oracle_sample_batch(None if is_bf16 else _ptr(lg), _ptr(lg) if is_bf16 else None, B, V, stride,
                              C.byref(cs), _ptr(t_rows), _ptr(k_rows), _ptr(p_rows), _ptr(m_rows), _ptr(r_rows),
                              _ptr(hist), hstride, _ptr(hlen), _ptr(sd), _ptr(di), _ptr(tokens), _ptr(kc),
                              _ptr(ids), _ptr(pr), kept_capacity, _ptr(st), _ptr(fl), nthreads)
    return BatchResult(tokens, fl, kc, ids, pr, st)


def penalized_at_history(logits: np.ndarray, cfg: SamplingConfig, recent: Sequence[int]) -> np.ndarray:
    row = np.ascontiguousarray(logits, dtype=np.float32)
    rec = np.ascontiguousarray(np.asarray(recent, dtype=np.uint32))
    keep: list = []
    cs = _config_struct(cfg, EXP_LIBM, keep)
    out = np.zeros(rec.size, np.float32)
    lib().oracle_penalized_at_history(_ptr(row), row.size, C.byref(cs), _ptr(rec), rec.size, _ptr(out))
    return out


def cross_entropy(logits: np.ndarray, targets: Sequence[int], want_grad: bool = True):
    """llm_core::ops::cross_entropy (ops/loss.rs:20-45): (mean loss, d_logits [T, V] or None, per-row loss terms)."""
    x = np.ascontiguousarray(logits, dtype=np.float32)
    t_len, vocab = x.shape
    tg = np.ascontiguousarray(np.asarray(targets, dtype=np.uint32))
    assert tg.size == t_len and (tg < vocab).all()
    d = np.zeros_like(x) if want_grad else None
    rl = np.zeros(t_len, np.float32)
    L = lib()
    L.oracle_cross_entropy.restype = C.c_float
    L.oracle_cross_entropy.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p]
    mean = float(L.oracle_cross_entropy(_ptr(x), _ptr(tg), t_len, vocab, _ptr(d), _ptr(rl)))
    return mean, d, rl


def hardware_threads() -> int:
    return int(lib().oracle_hardware_threads())
