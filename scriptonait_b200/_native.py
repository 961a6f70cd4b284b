"""ctypes view of libllm_cuda.so (include/llm_cuda.h).

Loading fails loudly: there is no Python or CPU stand-in for the CUDA library.
"""
from __future__ import annotations

import ctypes as C
import os

from . import _build

ABI_VERSION = 2

OK = 0
ERR_BAD_ARGUMENT = -1
ERR_CAPACITY = -2
ERR_CUDA = -3
ERR_UNSUPPORTED = -4
ERR_NO_DEVICE = -5
ERR_TIMEOUT = -6

STATUS_COPY_TIMEOUT = 1
STATUS_SLOT_TIMEOUT = 2
STATUS_CHECK_FAILED = 4

DTYPE_F32 = 0
DTYPE_BF16 = 1

ROW_GREEDY = 1
ROW_DEGENERATE = 2
ROW_FALLBACK_LAST = 4
ROW_DRAW_CONSUMED = 8
ROW_FULL_SORT = 16
ROW_INVALID = 64
ROW_WINDOWED = 128

EOS_DEFAULT = 258
ROW_STATS = 6

EXPORTS = [
    "llm_cuda_abi_version", "llm_cuda_sampling_config_default", "llm_cuda_sampler_create", "llm_cuda_sampler_destroy",
    "llm_cuda_last_error", "llm_cuda_sample_batch", "llm_cuda_sample_batch_host", "llm_cuda_sample_with",
    "llm_cuda_sample", "llm_cuda_shard_select", "llm_cuda_merge_draw", "llm_cuda_advance_rows",
    "llm_cuda_pack_allowed", "llm_cuda_last_launch_info", "llm_cuda_sample_batch_static", "llm_cuda_static_last_error",
    "llm_cuda_device_status", "llm_cuda_test_hold_full_sort_slots", "llm_cuda_packed_candidates_bytes",
    "llm_cuda_shard_select_packed", "llm_cuda_merge_draw_packed", "llm_cuda_lm_head_sample", "llm_cuda_cross_entropy",
]
STATIC_MAX_BATCH, STATIC_MAX_TOP_K, STATIC_MAX_HISTORY = 64, 256, 512


class SamplingConfigC(C.Structure):
    _fields_ = [
        ("temperature", C.c_float), ("top_k", C.c_uint32), ("top_p", C.c_float), ("min_p", C.c_float),
        ("repetition_penalty", C.c_float), ("repetition_window", C.c_uint32), ("seed", C.c_uint64),
        ("allowed", C.c_void_p), ("allowed_len", C.c_uint32),
    ]


class SampleArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("logits_dtype", C.c_uint32), ("logits", C.c_void_p),
        ("batch", C.c_uint32), ("vocab", C.c_uint32), ("row_stride_elems", C.c_uint64),
        ("temperature", C.c_float), ("top_k", C.c_uint32), ("top_p", C.c_float), ("min_p", C.c_float),
        ("repetition_penalty", C.c_float), ("overlap_previous", C.c_uint32),
        ("temperature_rows", C.c_void_p), ("top_k_rows", C.c_void_p), ("top_p_rows", C.c_void_p),
        ("min_p_rows", C.c_void_p), ("repetition_penalty_rows", C.c_void_p),
        ("history", C.c_void_p), ("history_stride", C.c_uint32), ("history_len", C.c_uint32),
        ("history_len_rows", C.c_void_p),
        ("allowed_bits", C.c_void_p), ("allowed_len", C.c_uint32), ("eos_id", C.c_uint32),
        ("seeds", C.c_void_p), ("draw_index", C.c_void_p), ("seed_base", C.c_uint64), ("uniforms", C.c_void_p),
        ("tokens", C.c_void_p),
        ("row_flags", C.c_void_p), ("kept_count", C.c_void_p), ("kept_ids", C.c_void_p), ("kept_probs", C.c_void_p),
        ("kept_capacity", C.c_uint32), ("reserved1", C.c_uint32), ("row_stats", C.c_void_p),
        ("column_offset", C.c_uint32), ("vocab_global", C.c_uint32),
        ("split", C.c_uint32), ("force_full_sort", C.c_uint32), ("stream", C.c_void_p),
        ("penalized_out", C.c_void_p),
    ]


class LmHeadArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("batch", C.c_uint32), ("hidden", C.c_void_p), ("norm_gain", C.c_void_p),
        ("norm_eps", C.c_float), ("hidden_dim", C.c_uint32), ("embed", C.c_void_p), ("vocab", C.c_uint32),
        ("temperature", C.c_float), ("top_k", C.c_uint32), ("top_p", C.c_float), ("min_p", C.c_float),
        ("reserved0", C.c_uint32), ("seeds", C.c_void_p), ("draw_index", C.c_void_p), ("seed_base", C.c_uint64),
        ("uniforms", C.c_void_p), ("tokens", C.c_void_p), ("row_flags", C.c_void_p), ("kept_count", C.c_void_p),
        ("kept_ids", C.c_void_p), ("kept_probs", C.c_void_p), ("kept_capacity", C.c_uint32), ("reserved1", C.c_uint32),
        ("row_stats", C.c_void_p), ("logits_out", C.c_void_p), ("stream", C.c_void_p),
    ]


_libs: dict = {}


def library_path() -> str:
    return _build.LIBRARY


def load(checked: bool = False) -> C.CDLL:
    """Builds (when stale and nvcc is present) and loads the CUDA library - the product build, or with
    `checked` the bounds-checked build of the same sources. Raises if it cannot be produced or loaded;
    nothing else can stand in for it."""
    if checked in _libs:
        return _libs[checked]
    path = _build.CHECKED_LIBRARY if checked else _build.LIBRARY
    if _build.is_stale(path):
        try:
            _build.build(checked=checked)
        except Exception as exc:  # keep a prebuilt library if the toolchain is missing
            if not os.path.exists(path):
                raise RuntimeError(f"{os.path.basename(path)} is missing and could not be built: {exc}") from exc
    L = C.CDLL(path)
    vp, u32, i32 = C.c_void_p, C.c_uint32, C.c_int32
    L.llm_cuda_abi_version.restype = u32
    L.llm_cuda_abi_version.argtypes = []
    L.llm_cuda_sampling_config_default.restype = None
    L.llm_cuda_sampling_config_default.argtypes = [C.POINTER(SamplingConfigC)]
    L.llm_cuda_sampler_create.restype = i32
    L.llm_cuda_sampler_create.argtypes = [i32, u32, u32, u32, u32, C.POINTER(vp)]
    L.llm_cuda_sampler_destroy.restype = i32
    L.llm_cuda_sampler_destroy.argtypes = [vp]
    L.llm_cuda_last_error.restype = C.c_char_p
    L.llm_cuda_last_error.argtypes = [vp]
    L.llm_cuda_sample_batch.restype = i32
    L.llm_cuda_sample_batch.argtypes = [vp, C.POINTER(SampleArgs)]
    L.llm_cuda_sample_batch_host.restype = i32
    L.llm_cuda_sample_batch_host.argtypes = [vp, C.POINTER(SampleArgs)]
    L.llm_cuda_sample_with.restype = i32
    L.llm_cuda_sample_with.argtypes = [vp, vp, u32, C.POINTER(SamplingConfigC), vp, u32, C.POINTER(C.c_uint64),
                                       C.POINTER(u32)]
    L.llm_cuda_sample.restype = i32
    L.llm_cuda_sample.argtypes = [vp, vp, u32, C.c_float, C.POINTER(C.c_uint64), C.POINTER(u32)]
    L.llm_cuda_shard_select.restype = i32
    L.llm_cuda_shard_select.argtypes = [vp, C.POINTER(SampleArgs), vp, vp, vp, u32]
    L.llm_cuda_merge_draw.restype = i32
    L.llm_cuda_merge_draw.argtypes = [vp, C.POINTER(SampleArgs), vp, vp, vp, u32, u32]
    L.llm_cuda_advance_rows.restype = i32
    L.llm_cuda_advance_rows.argtypes = [vp, u32, vp, vp, vp, u32, u32, vp, vp, vp, vp, u32, vp]
    L.llm_cuda_pack_allowed.restype = i32
    L.llm_cuda_pack_allowed.argtypes = [vp, vp, u32, vp, vp]
    L.llm_cuda_last_launch_info.restype = i32
    L.llm_cuda_last_launch_info.argtypes = [vp, C.POINTER(u32), C.POINTER(u32)]
    L.llm_cuda_cross_entropy.restype = i32
    L.llm_cuda_cross_entropy.argtypes = [vp, vp, u32, u32, u32, vp, vp, vp, vp]
    L.llm_cuda_packed_candidates_bytes.restype = C.c_size_t
    L.llm_cuda_packed_candidates_bytes.argtypes = [u32, u32]
    L.llm_cuda_shard_select_packed.restype = i32
    L.llm_cuda_shard_select_packed.argtypes = [vp, C.POINTER(SampleArgs), vp, u32]
    L.llm_cuda_merge_draw_packed.restype = i32
    L.llm_cuda_merge_draw_packed.argtypes = [vp, C.POINTER(SampleArgs), vp, u32, u32]
    L.llm_cuda_lm_head_sample.restype = i32
    L.llm_cuda_lm_head_sample.argtypes = [vp, C.POINTER(LmHeadArgs)]
    L.llm_cuda_device_status.restype = i32
    L.llm_cuda_device_status.argtypes = [vp, vp, C.POINTER(u32)]
    L.llm_cuda_test_hold_full_sort_slots.restype = i32
    L.llm_cuda_test_hold_full_sort_slots.argtypes = [vp, u32, u32, vp]
    L.llm_cuda_sample_batch_static.restype = i32
    L.llm_cuda_sample_batch_static.argtypes = [i32, C.POINTER(SampleArgs)]
    L.llm_cuda_static_last_error.restype = C.c_char_p
    L.llm_cuda_static_last_error.argtypes = []
    if L.llm_cuda_abi_version() != ABI_VERSION:
        raise RuntimeError("libllm_cuda.so ABI version mismatch")
    _libs[checked] = L
    return L
