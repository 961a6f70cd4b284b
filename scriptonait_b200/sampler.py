"""Host-side mirror of the reference's sampler interface over the CUDA library.

Names, argument meaning and error behaviour follow crates/llm-core/src/generate.rs:
`SamplingConfig` (:24-95), `sample_with(logits, sampling, recent, rng)` (:325-330),
`sample(logits, temperature, rng)` (:423-433) and `Rng` (crates/llm-core/src/rng.rs:6-34).
`Sampler.sample_batch` is the batched, device-resident form a GPU decode loop uses in
place of the per-token logits read-back + CPU `sample_with` call of
crates/wasm-app/src/inference.rs:325-347.

PyTorch appears here only as the owner of device memory and streams. Every call goes
through the C ABI of include/llm_cuda.h; there is no Python or CPU implementation of
the sampling arithmetic in this package.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
from typing import Optional, Sequence, Union

import numpy as np

from . import _native as N

MASK64 = (1 << 64) - 1
GOLDEN_GAMMA = 0x9E3779B97F4A7C15
EOS = N.EOS_DEFAULT


class LlmCudaError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"llm_cuda error {code}: {message}")
        self.code = code


@dataclasses.dataclass
class SamplingConfig:
    """How a token is picked from a row of logits (generate.rs:24-95, same defaults)."""
    temperature: float = 0.9      # <= 0 means greedy
    top_k: int = 40               # 0 disables
    top_p: float = 0.95           # 1.0 disables; applied after top_k and min_p
    min_p: float = 0.0            # 0.0 disables; applied after top_k, before top_p
    repetition_penalty: float = 1.1  # 1.0 disables
    repetition_window: int = 128
    seed: int = 0
    allowed: Optional[np.ndarray] = None  # one bool per id; None allows everything


class Rng:
    """SplitMix64 (rng.rs:6-34). Only the state word and the integer stream live on the
    host; the uniform a draw uses is recomputed on the GPU from (state, output number)."""

    def __init__(self, seed: int):
        self.state = seed & MASK64

    @classmethod
    def seed_from_u64(cls, seed: int) -> "Rng":
        return cls(seed)

    def next_u64(self) -> int:
        self.state = (self.state + GOLDEN_GAMMA) & MASK64
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
        return z ^ (z >> 31)

    def next_f32(self) -> float:
        return float(np.float32(self.next_u64() >> 40) / np.float32(1 << 24))


@dataclasses.dataclass
class SampleResult:
    tokens: "object"                  # torch uint32-as-int32 tensor on the device, [B]
    row_flags: Optional["object"] = None
    kept_count: Optional["object"] = None
    kept_ids: Optional["object"] = None
    kept_probs: Optional["object"] = None
    row_stats: Optional["object"] = None
    penalized: Optional["object"] = None   # [B, H] post-mask, post-penalty, pre-temperature value at each history position
    logits: Optional["object"] = None      # fused LM head only, on request: the logits the tensor cores produced


class PreparedCall:
    """A fully marshalled llm_cuda_sample_batch call over fixed device buffers."""

    def __init__(self, sampler: "Sampler", args: "N.SampleArgs", result: SampleResult):
        self.sampler, self.args, self.result = sampler, args, result
        self._fn = sampler._lib.llm_cuda_sample_batch
        self._ref = C.byref(args)

    def launch(self) -> SampleResult:
        rc = self._fn(self.sampler._h, self._ref)
        if rc != N.OK:
            self.sampler._check(rc)
        return self.result


def _torch():
    import torch  # deferred: importing the package must not require a GPU
    return torch


ParamT = Union[float, int, "object"]


class Sampler:
    """Owns one llm_cuda_sampler handle (one GPU, one stream at a time)."""

    def __init__(self, device: int = 0, max_batch: int = 1024, max_vocab: int = 262144, max_history: int = 1024,
                 max_top_k: int = 1024, checked: bool = False):
        """`checked`: use the bounds-checked build of the library (slower; for tests)."""
        self._lib = N.load(checked)
        self._h = C.c_void_p()
        self.device = device
        self.max_batch, self.max_vocab, self.max_history, self.max_top_k = max_batch, max_vocab, max_history, max_top_k
        rc = self._lib.llm_cuda_sampler_create(device, max_batch, max_vocab, max_history, max_top_k, C.byref(self._h))
        if rc != N.OK:
            msg = self._lib.llm_cuda_last_error(None).decode()
            self._h = C.c_void_p()
            raise LlmCudaError(rc, msg)

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h:
            self._lib.llm_cuda_sampler_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int) -> None:
        if rc != N.OK:
            raise LlmCudaError(rc, self._lib.llm_cuda_last_error(self._h).decode())

    def device_status(self, stream=None) -> int:
        """Synchronises the stream, then reads and clears the device status word. Raises LlmCudaError
        (ERR_TIMEOUT) when a bounded wait inside a kernel ran out; returns 0 otherwise."""
        torch = _torch()
        st = stream if stream is not None else torch.cuda.current_stream(torch.device(f"cuda:{self.device}")).cuda_stream
        bits = C.c_uint32()
        self._check(self._lib.llm_cuda_device_status(self._h, st, C.byref(bits)))
        return bits.value

    def hold_full_sort_slots(self, hold: bool, wait_rounds: int = 0, stream=None) -> None:
        """Testing aid: marks every full-ordering scratch slot taken (or frees them) and shortens the
        slot wait of later launches to `wait_rounds` polls (0 = default)."""
        torch = _torch()
        st = stream if stream is not None else torch.cuda.current_stream(torch.device(f"cuda:{self.device}")).cuda_stream
        self._check(self._lib.llm_cuda_test_hold_full_sort_slots(self._h, 1 if hold else 0, wait_rounds, st))

    def last_launch_info(self) -> tuple[int, int]:
        k, s = C.c_uint32(), C.c_uint32()
        self._lib.llm_cuda_last_launch_info(self._h, C.byref(k), C.byref(s))
        return k.value, s.value

    # ------------------------------------------------------------------ device path
    def _fill_args(self, *, logits, batch, vocab, row_stride, dtype, temperature, top_k, top_p, min_p,
                   repetition_penalty, history, history_len, allowed_bits, allowed_len, eos_id, seeds, draw_index,
                   seed_base, uniforms, split, force_full_sort, stream, keep) -> N.SampleArgs:
        torch = _torch()
        a = N.SampleArgs()
        a.struct_size = C.sizeof(N.SampleArgs)
        a.logits_dtype = dtype
        a.logits = logits
        a.batch = batch
        a.vocab = vocab
        a.row_stride_elems = row_stride

        def param(value, scalar_field, rows_field, tdtype, default):
            if value is None:
                setattr(a, scalar_field, default)
            elif isinstance(value, (int, float, np.floating, np.integer)):
                setattr(a, scalar_field, value)
            else:
                t = value if isinstance(value, torch.Tensor) else torch.as_tensor(_as_signed(np.asarray(value)))
                t = t.to(device=f"cuda:{self.device}", dtype=tdtype).contiguous()
                assert t.numel() == batch, f"{rows_field}: expected {batch} values"
                keep.append(t)
                setattr(a, scalar_field, default)
                setattr(a, rows_field, t.data_ptr())

        param(temperature, "temperature", "temperature_rows", torch.float32, 1.0)
        param(top_k, "top_k", "top_k_rows", torch.int32, 0)
        param(top_p, "top_p", "top_p_rows", torch.float32, 1.0)
        param(min_p, "min_p", "min_p_rows", torch.float32, 0.0)
        param(repetition_penalty, "repetition_penalty", "repetition_penalty_rows", torch.float32, 1.0)

        def dev(value, tdtype):
            if value is None:
                return None
            t = value if isinstance(value, torch.Tensor) else torch.as_tensor(_as_signed(np.asarray(value)))
            if t.dtype in (torch.uint32, torch.uint64):  # reinterpret, torch cannot cast these on every build
                t = t.view(torch.int32 if t.dtype == torch.uint32 else torch.int64)
            t = t.to(device=f"cuda:{self.device}", dtype=tdtype).contiguous()
            keep.append(t)
            return t

        if history is not None:
            h = dev(_as_signed(history), torch.int32)
            assert h.dim() == 2 and h.shape[0] == batch
            a.history = h.data_ptr()
            a.history_stride = h.shape[1]
            if history_len is None:
                a.history_len = h.shape[1]
            elif isinstance(history_len, (int, np.integer)):
                a.history_len = int(history_len)
            else:
                hl = dev(_as_signed(history_len), torch.int32)
                a.history_len_rows = hl.data_ptr()
        if allowed_bits is not None:
            ab = dev(_as_signed(allowed_bits), torch.int32)
            a.allowed_bits = ab.data_ptr()
            a.allowed_len = int(allowed_len if allowed_len is not None else ab.numel() * 32)
        a.eos_id = eos_id
        if seeds is not None:
            sd = dev(_as_signed(seeds), torch.int64)
            assert sd.numel() == batch
            a.seeds = sd.data_ptr()
        if draw_index is not None:
            di = dev(_as_signed(draw_index), torch.int64)
            assert di.numel() == batch
            a.draw_index = di.data_ptr()
        a.seed_base = seed_base & MASK64
        if uniforms is not None:
            un = dev(uniforms, torch.float32)
            a.uniforms = un.data_ptr()
        a.split = split
        a.force_full_sort = 1 if force_full_sort else 0
        a.stream = stream
        return a

    def sample_batch(self, logits, *, temperature: ParamT = 1.0, top_k: ParamT = 0, top_p: ParamT = 1.0,
                     min_p: ParamT = 0.0, repetition_penalty: ParamT = 1.0, history=None, history_len=None,
                     allowed_bits=None, allowed_len: Optional[int] = None, eos_id: int = EOS, seeds=None,
                     draw_index=None, seed_base: int = 0, uniforms=None, batch: Optional[int] = None,
                     row_stride: Optional[int] = None, trace: bool = False, kept_capacity: int = 64, split: int = 0,
                     force_full_sort: bool = False, out_tokens=None, stream=None, prepare_only: bool = False,
                     overlap_previous: bool = False, want_penalized: bool = False):
        """Row r of `logits` ([B, V] CUDA tensor, float32 / bfloat16 / uint16 bf16 bits) is one
        `sample_with` call with Rng::seed_from_u64(seeds[r]) advanced by draw_index[r] outputs.
        Parameters are scalars or per-row arrays. Asynchronous on the current (or given) stream.
        With `prepare_only` nothing is launched: the returned PreparedCall re-issues the same call
        (same buffers, same stream) with one C-ABI call per `launch()`, which is what a decode
        loop over fixed buffers wants. `overlap_previous` lets the launch begin reading its inputs
        before the operation that precedes it on the stream has completed (outputs keep stream
        order); only for calls none of whose inputs that operation writes."""
        torch = _torch()
        assert logits.is_cuda and logits.dim() == 2 and logits.stride(1) == 1, "logits: [B, V] CUDA tensor, unit column stride"
        if logits.dtype == torch.float32:
            dtype = N.DTYPE_F32
        elif logits.dtype in (torch.bfloat16, torch.uint16, torch.int16):
            dtype = N.DTYPE_BF16
        else:
            raise TypeError(f"unsupported logits dtype {logits.dtype}")
        B = int(batch if batch is not None else logits.shape[0])
        V = int(logits.shape[1])
        stride = int(row_stride if row_stride is not None else logits.stride(0))
        st = stream if stream is not None else torch.cuda.current_stream(logits.device).cuda_stream
        keep: list = [logits]
        a = self._fill_args(logits=logits.data_ptr(), batch=B, vocab=V, row_stride=stride, dtype=dtype,
                            temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p,
                            repetition_penalty=repetition_penalty, history=history, history_len=history_len,
                            allowed_bits=allowed_bits, allowed_len=allowed_len, eos_id=eos_id, seeds=seeds,
                            draw_index=draw_index, seed_base=seed_base, uniforms=uniforms, split=split,
                            force_full_sort=force_full_sort, stream=st, keep=keep)
        a.overlap_previous = int(overlap_previous)  # False/True, or 2 = early launch with strict data order
        res = self._outputs(a, B, trace, kept_capacity, out_tokens, logits.device)
        if want_penalized and a.history:
            res.penalized = torch.full((B, int(a.history_stride)), float("nan"), dtype=torch.float32, device=logits.device)
            a.penalized_out = res.penalized.data_ptr()
        res._keepalive = keep  # inputs must outlive the asynchronous launch
        call = PreparedCall(self, a, res)
        if prepare_only:
            return call
        call.launch()
        return res

    def _outputs(self, a: N.SampleArgs, B: int, trace: bool, kept_capacity: int, out_tokens, device) -> SampleResult:
        torch = _torch()
        tokens = out_tokens if out_tokens is not None else torch.empty(B, dtype=torch.int32, device=device)
        a.tokens = tokens.data_ptr()
        res = SampleResult(tokens)
        if trace:
            res.row_flags = torch.zeros(B, dtype=torch.int32, device=device)
            res.kept_count = torch.zeros(B, dtype=torch.int32, device=device)
            res.kept_ids = torch.zeros((B, kept_capacity), dtype=torch.int32, device=device)
            res.kept_probs = torch.zeros((B, kept_capacity), dtype=torch.float32, device=device)
            res.row_stats = torch.zeros((B, N.ROW_STATS), dtype=torch.float32, device=device)
            a.row_flags = res.row_flags.data_ptr()
            a.kept_count = res.kept_count.data_ptr()
            a.kept_ids = res.kept_ids.data_ptr()
            a.kept_probs = res.kept_probs.data_ptr()
            a.kept_capacity = kept_capacity
            a.row_stats = res.row_stats.data_ptr()
        return res

    # ------------------------------------------------------------------ vocabulary sharding
    def shard_select(self, logits, *, column_offset: int, vocab_global: int, cand_stride: int, temperature: ParamT = 1.0,
                     top_k: int = 0, repetition_penalty: ParamT = 1.0, history=None, history_len=None,
                     allowed_bits=None, allowed_len: Optional[int] = None, eos_id: int = EOS, split: int = 0,
                     out=None, stream=None):
        """Step 1 of vocabulary sharding: this GPU's columns -> per-row ordered candidate lists
        (values [B, cand_stride] f32, global ids [B, cand_stride], counts [B])."""
        torch = _torch()
        assert logits.is_cuda and logits.dim() == 2 and logits.stride(1) == 1
        dtype = N.DTYPE_F32 if logits.dtype == torch.float32 else N.DTYPE_BF16
        B, V = int(logits.shape[0]), int(logits.shape[1])
        st = stream if stream is not None else torch.cuda.current_stream(logits.device).cuda_stream
        keep: list = [logits]
        a = self._fill_args(logits=logits.data_ptr(), batch=B, vocab=V, row_stride=int(logits.stride(0)), dtype=dtype,
                            temperature=temperature, top_k=top_k, top_p=1.0, min_p=0.0,
                            repetition_penalty=repetition_penalty, history=history, history_len=history_len,
                            allowed_bits=allowed_bits, allowed_len=allowed_len, eos_id=eos_id, seeds=None,
                            draw_index=None, seed_base=0, uniforms=None, split=split, force_full_sort=False,
                            stream=st, keep=keep)
        a.column_offset = column_offset
        a.vocab_global = vocab_global
        if out is None:
            vals = torch.zeros((B, cand_stride), dtype=torch.float32, device=logits.device)
            ids = torch.zeros((B, cand_stride), dtype=torch.int32, device=logits.device)
            cnt = torch.zeros(B, dtype=torch.int32, device=logits.device)
        else:
            vals, ids, cnt = out
        self._check(self._lib.llm_cuda_shard_select(self._h, C.byref(a), vals.data_ptr(), ids.data_ptr(), cnt.data_ptr(),
                                                    cand_stride))
        self._keepalive = keep
        return vals, ids, cnt

    def shard_select_packed(self, logits, *, column_offset: int, vocab_global: int, cand_stride: int,
                            temperature: ParamT = 1.0, top_k: int = 0, repetition_penalty: ParamT = 1.0, history=None,
                            history_len=None, allowed_bits=None, allowed_len: Optional[int] = None, eos_id: int = EOS,
                            split: int = 0, out=None, stream=None, prepare_only: bool = False):
        """Step 1 into ONE packed block (values, ids, counts; llm_cuda_shard_select_packed): a flat int32
        tensor of 2*B*cand_stride + B words, ready for a single all-gather. `logits` may have zero columns
        (a shard past the end of a small vocabulary): the block then holds empty lists."""
        torch = _torch()
        assert logits.is_cuda and logits.dim() == 2 and (logits.shape[1] == 0 or logits.stride(1) == 1)
        dtype = N.DTYPE_F32 if logits.dtype == torch.float32 else N.DTYPE_BF16
        B, V = int(logits.shape[0]), int(logits.shape[1])
        st = stream if stream is not None else torch.cuda.current_stream(logits.device).cuda_stream
        keep: list = [logits]
        a = self._fill_args(logits=logits.data_ptr() if V else None, batch=B, vocab=V,
                            row_stride=int(logits.stride(0)) if V else 0, dtype=dtype,
                            temperature=temperature, top_k=top_k, top_p=1.0, min_p=0.0,
                            repetition_penalty=repetition_penalty, history=history, history_len=history_len,
                            allowed_bits=allowed_bits, allowed_len=allowed_len, eos_id=eos_id, seeds=None,
                            draw_index=None, seed_base=0, uniforms=None, split=split, force_full_sort=False,
                            stream=st, keep=keep)
        a.column_offset = column_offset
        a.vocab_global = vocab_global
        words = 2 * B * cand_stride + B
        packed = out if out is not None else torch.zeros(words, dtype=torch.int32, device=logits.device)
        assert packed.numel() == words and packed.is_contiguous()
        keep.append(packed)
        fn, h, ref, ptr = self._lib.llm_cuda_shard_select_packed, self._h, C.byref(a), packed.data_ptr()

        def launch():
            rc = fn(h, ref, ptr, cand_stride)
            if rc != N.OK:
                self._check(rc)
            return packed

        launch._keepalive = (a, keep)
        if prepare_only:
            return launch
        self._keepalive = keep
        return launch()

    def merge_draw_packed(self, packed_all, *, batch: int, cand_stride: int, vocab_global: int,
                          temperature: ParamT = 1.0, top_k: int = 0, top_p: ParamT = 1.0, min_p: ParamT = 0.0,
                          seeds=None, draw_index=None, seed_base: int = 0, uniforms=None, trace: bool = False,
                          kept_capacity: int = 64, stream=None, prepare_only: bool = False):
        """Step 2 over the all-gathered packed blocks [G, 2*B*cand_stride + B] (llm_cuda_merge_draw_packed)."""
        torch = _torch()
        G = int(packed_all.shape[0])
        assert packed_all.is_contiguous() and packed_all.numel() == G * (2 * batch * cand_stride + batch)
        st = stream if stream is not None else torch.cuda.current_stream(packed_all.device).cuda_stream
        keep: list = [packed_all]
        a = self._fill_args(logits=None, batch=batch, vocab=0, row_stride=0, dtype=N.DTYPE_F32, temperature=temperature,
                            top_k=top_k, top_p=top_p, min_p=min_p, repetition_penalty=1.0, history=None,
                            history_len=None, allowed_bits=None, allowed_len=None, eos_id=EOS, seeds=seeds,
                            draw_index=draw_index, seed_base=seed_base, uniforms=uniforms, split=0,
                            force_full_sort=False, stream=st, keep=keep)
        a.vocab_global = vocab_global
        res = self._outputs(a, batch, trace, kept_capacity, None, packed_all.device)
        res._keepalive = keep
        fn, h, ref, ptr = self._lib.llm_cuda_merge_draw_packed, self._h, C.byref(a), packed_all.data_ptr()

        def launch():
            rc = fn(h, ref, ptr, G, cand_stride)
            if rc != N.OK:
                self._check(rc)
            return res

        launch._keepalive = (a, keep)
        if prepare_only:
            return launch
        return launch()

    def merge_draw(self, cand_values, cand_ids, cand_count, *, vocab_global: int, temperature: ParamT = 1.0,
                   top_k: int = 0, top_p: ParamT = 1.0, min_p: ParamT = 0.0, seeds=None, draw_index=None,
                   seed_base: int = 0, uniforms=None, trace: bool = False, kept_capacity: int = 64,
                   stream=None) -> SampleResult:
        """Step 2: gathered lists [G, B, cand_stride] (+ counts [G, B]) -> tokens."""
        torch = _torch()
        G, B, S = (int(x) for x in cand_values.shape)
        assert cand_values.is_contiguous() and cand_ids.is_contiguous() and cand_count.is_contiguous()
        st = stream if stream is not None else torch.cuda.current_stream(cand_values.device).cuda_stream
        keep: list = [cand_values, cand_ids, cand_count]
        a = self._fill_args(logits=None, batch=B, vocab=0, row_stride=0, dtype=N.DTYPE_F32, temperature=temperature,
                            top_k=top_k, top_p=top_p, min_p=min_p, repetition_penalty=1.0, history=None,
                            history_len=None, allowed_bits=None, allowed_len=None, eos_id=EOS, seeds=seeds,
                            draw_index=draw_index, seed_base=seed_base, uniforms=uniforms, split=0,
                            force_full_sort=False, stream=st, keep=keep)
        a.vocab_global = vocab_global
        res = self._outputs(a, B, trace, kept_capacity, None, cand_values.device)
        self._check(self._lib.llm_cuda_merge_draw(self._h, C.byref(a), cand_values.data_ptr(), cand_ids.data_ptr(),
                                                  cand_count.data_ptr(), G, S))
        res._keepalive = keep
        return res

    # ------------------------------------------------------------------ fused LM head -> sampler
    def lm_head_sample(self, hidden, embed, *, norm_gain=None, norm_eps: float = 1e-5, temperature: float = 1.0,
                       top_k: int = 40, top_p: float = 1.0, min_p: float = 0.0, seeds=None, draw_index=None,
                       seed_base: int = 0, uniforms=None, trace: bool = False, kept_capacity: int = 64,
                       want_logits: bool = False, stream=None, prepare_only: bool = False):
        """Final RMSNorm + tied LM head + sampling for a decode batch without materialising the logits
        (llm_cuda_lm_head_sample; replaces crates/llm-gpu/src/model.rs:481-490 and the sample_with call that
        follows). `hidden` [B, H] float32 CUDA tensor, `embed` [V, H] bfloat16 CUDA tensor (row-major),
        `norm_gain` [H] float32 or None when `hidden` is already normalised. With `want_logits` the
        logits the tensor cores produced are also written (testing aid) and returned as `.logits`."""
        torch = _torch()
        assert hidden.is_cuda and hidden.dtype == torch.float32 and hidden.dim() == 2 and hidden.is_contiguous()
        assert embed.is_cuda and embed.dtype == torch.bfloat16 and embed.dim() == 2 and embed.is_contiguous()
        B, H = int(hidden.shape[0]), int(hidden.shape[1])
        V = int(embed.shape[0])
        assert int(embed.shape[1]) == H
        st = stream if stream is not None else torch.cuda.current_stream(hidden.device).cuda_stream
        a = N.LmHeadArgs()
        a.struct_size = C.sizeof(N.LmHeadArgs)
        a.batch, a.hidden_dim, a.vocab = B, H, V
        a.hidden, a.embed = hidden.data_ptr(), embed.data_ptr()
        keep: list = [hidden, embed]
        if norm_gain is not None:
            g = norm_gain.to(device=hidden.device, dtype=torch.float32).contiguous()
            keep.append(g)
            a.norm_gain = g.data_ptr()
        a.norm_eps = norm_eps
        a.temperature, a.top_k, a.top_p, a.min_p = temperature, top_k, top_p, min_p

        def dev64(value):
            t = value if isinstance(value, torch.Tensor) else torch.as_tensor(_as_signed(np.asarray(value)))
            t = t.to(device=hidden.device, dtype=torch.int64).contiguous()
            keep.append(t)
            return t.data_ptr()

        if seeds is not None:
            a.seeds = dev64(seeds)
        if draw_index is not None:
            a.draw_index = dev64(draw_index)
        a.seed_base = seed_base & MASK64
        if uniforms is not None:
            un = torch.as_tensor(uniforms).to(device=hidden.device, dtype=torch.float32).contiguous()
            keep.append(un)
            a.uniforms = un.data_ptr()
        a.stream = st
        sa = N.SampleArgs()  # only to reuse the per-stage output allocation
        res = self._outputs(sa, B, trace, kept_capacity, None, hidden.device)
        a.tokens = res.tokens.data_ptr()
        if trace:
            a.row_flags, a.kept_count = res.row_flags.data_ptr(), res.kept_count.data_ptr()
            a.kept_ids, a.kept_probs = res.kept_ids.data_ptr(), res.kept_probs.data_ptr()
            a.kept_capacity, a.row_stats = kept_capacity, res.row_stats.data_ptr()
        res.logits = None
        if want_logits:
            res.logits = torch.empty((B, V), dtype=torch.float32, device=hidden.device)
            a.logits_out = res.logits.data_ptr()
        res._keepalive = keep
        fn, h, ref = self._lib.llm_cuda_lm_head_sample, self._h, C.byref(a)

        def launch():
            rc = fn(h, ref)
            if rc != N.OK:
                self._check(rc)
            return res

        launch._keepalive = (a, keep)
        if prepare_only:
            return launch
        return launch()

    # ------------------------------------------------------------------ decode-loop glue
    def advance_rows(self, tokens, row_flags, *, history=None, window: int = 128, history_len=None, history_pos=None,
                     draw_index=None, finished=None, eos_id: int = EOS, stream=None) -> None:
        """Generator::step's bookkeeping on the device (generate.rs:157-182)."""
        torch = _torch()
        st = stream if stream is not None else torch.cuda.current_stream(tokens.device).cuda_stream
        ptr = lambda t: None if t is None else t.data_ptr()
        stride = 0 if history is None else int(history.stride(0))
        self._check(self._lib.llm_cuda_advance_rows(self._h, int(tokens.numel()), tokens.data_ptr(), ptr(row_flags),
                                                    ptr(history), stride, window, ptr(history_len), ptr(history_pos),
                                                    ptr(draw_index), ptr(finished), eos_id, st))

    def pack_allowed(self, allowed: np.ndarray):
        """bool-per-id (Corpus::seen_tokens, corpus.rs:236-246) -> device bit mask + its length."""
        torch = _torch()
        a = np.ascontiguousarray(np.asarray(allowed).astype(np.uint8))
        bits = torch.zeros((a.size + 31) // 32, dtype=torch.int32, device=f"cuda:{self.device}")
        st = torch.cuda.current_stream(bits.device).cuda_stream
        self._check(self._lib.llm_cuda_pack_allowed(self._h, a.ctypes.data, a.size, bits.data_ptr(), st))
        return bits, int(a.size)

    def cross_entropy(self, logits, targets, want_grad: bool = True):
        """llm_core::ops::cross_entropy (ops/loss.rs:20-45; shaders/cross_entropy.wgsl) over device tensors: `logits`
        [T, V] float32, `targets` [T] int32. Returns (row_loss [T], d_logits [T, V] or None); the loss is
        row_loss.mean(), the gradient is already divided by T."""
        torch = _torch()
        if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
            raise ValueError("logits must be a [T, V] float32 tensor with contiguous rows")
        t_len, vocab = int(logits.shape[0]), int(logits.shape[1])
        if targets.dtype != torch.int32 or targets.numel() != t_len or not targets.is_contiguous():
            raise ValueError("targets must be a contiguous int32 tensor with one entry per row")
        row_loss = torch.empty(t_len, dtype=torch.float32, device=logits.device)
        grad = None
        if want_grad:
            # same strides, and the same offset from a 16-byte boundary: the kernel splits both rows alike
            span = (t_len - 1) * int(logits.stride(0)) + vocab
            lead = (logits.data_ptr() % 16) // 4
            grad = torch.empty(span + 4, dtype=torch.float32, device=logits.device)[lead:lead + span].as_strided(
                tuple(logits.shape), tuple(logits.stride()))
        st = torch.cuda.current_stream(logits.device).cuda_stream
        self._check(self._lib.llm_cuda_cross_entropy(self._h, logits.data_ptr(), t_len, vocab, int(logits.stride(0)), targets.data_ptr(),
                                                     row_loss.data_ptr(), grad.data_ptr() if want_grad else None, st))
        return row_loss, grad

    # ------------------------------------------------------------------ host-buffer path
    def sample_batch_host(self, logits: np.ndarray, *, temperature=1.0, top_k=0, top_p=1.0, min_p=0.0,
                          repetition_penalty=1.0, history: Optional[np.ndarray] = None,
                          allowed: Optional[np.ndarray] = None, seeds: Optional[np.ndarray] = None,
                          draw_index: Optional[np.ndarray] = None, seed_base: int = 0, batch: Optional[int] = None,
                          row_stride: Optional[int] = None, out_tokens: Optional[np.ndarray] = None,
                          want_flags: bool = False):
        """Same call with every array in host memory (numpy): copies in, samples, copies the
        tokens back, synchronises. `logits` float32, or uint16 holding bf16 bit patterns."""
        lg = logits if logits.flags.c_contiguous else np.ascontiguousarray(logits)
        if lg.ndim == 1:
            lg = lg[None, :]
        B = int(batch if batch is not None else lg.shape[0])
        V = int(lg.shape[1])
        a = N.SampleArgs()
        a.struct_size = C.sizeof(N.SampleArgs)
        if lg.dtype == np.float32:
            a.logits_dtype = N.DTYPE_F32
        elif lg.dtype == np.uint16:
            a.logits_dtype = N.DTYPE_BF16
        else:
            raise TypeError("logits must be float32 or uint16 (bf16 bits)")
        a.logits = lg.ctypes.data
        a.batch, a.vocab = B, V
        a.row_stride_elems = int(V if row_stride is None else row_stride)
        keep = [lg]

        def param(value, scalar_field, rows_field, npdtype, default):
            if np.isscalar(value):
                setattr(a, scalar_field, value)
            else:
                arr = np.ascontiguousarray(np.asarray(value, dtype=npdtype))
                assert arr.shape == (B,)
                keep.append(arr)
                setattr(a, scalar_field, default)
                setattr(a, rows_field, arr.ctypes.data)

        param(temperature, "temperature", "temperature_rows", np.float32, 1.0)
        param(top_k, "top_k", "top_k_rows", np.uint32, 0)
        param(top_p, "top_p", "top_p_rows", np.float32, 1.0)
        param(min_p, "min_p", "min_p_rows", np.float32, 0.0)
        param(repetition_penalty, "repetition_penalty", "repetition_penalty_rows", np.float32, 1.0)
        if history is not None:
            h = np.ascontiguousarray(history, dtype=np.uint32)
            keep.append(h)
            a.history = h.ctypes.data
            a.history_stride = a.history_len = h.shape[1]
        if allowed is not None:
            al = np.asarray(allowed).astype(bool)
            padded = np.ones(((al.size + 31) // 32) * 32, dtype=bool)
            padded[:al.size] = al
            bits = np.packbits(padded, bitorder="little").view(np.uint32).copy()
            keep.append(bits)
            a.allowed_bits = bits.ctypes.data
            a.allowed_len = al.size
        a.eos_id = EOS
        if seeds is not None:
            sd = np.ascontiguousarray(seeds, dtype=np.uint64)
            keep.append(sd)
            a.seeds = sd.ctypes.data
        if draw_index is not None:
            di = np.ascontiguousarray(draw_index, dtype=np.uint64)
            keep.append(di)
            a.draw_index = di.ctypes.data
        a.seed_base = seed_base & MASK64
        tokens = out_tokens if out_tokens is not None else np.zeros(B, np.uint32)
        a.tokens = tokens.ctypes.data
        flags = np.zeros(B, np.uint32) if want_flags else None
        if flags is not None:
            a.row_flags = flags.ctypes.data
        self._check(self._lib.llm_cuda_sample_batch_host(self._h, C.byref(a)))
        return (tokens, flags) if want_flags else tokens

    def sample_with(self, logits, sampling: SamplingConfig, recent: Sequence[int], rng: Rng) -> int:
        """sample_with(logits, sampling, recent, rng) -> token id (generate.rs:325-330). The RNG
        advances by one output exactly when the reference would draw."""
        row = np.ascontiguousarray(logits, dtype=np.float32)
        rec = np.ascontiguousarray(np.asarray(recent, dtype=np.uint32))
        cfg = N.SamplingConfigC()
        cfg.temperature = sampling.temperature
        cfg.top_k = int(sampling.top_k)
        cfg.top_p = sampling.top_p
        cfg.min_p = sampling.min_p
        cfg.repetition_penalty = sampling.repetition_penalty
        cfg.repetition_window = int(sampling.repetition_window)
        cfg.seed = sampling.seed & MASK64
        al = None
        if sampling.allowed is not None:
            al = np.ascontiguousarray(np.asarray(sampling.allowed).astype(np.uint8))
            cfg.allowed = al.ctypes.data
            cfg.allowed_len = al.size
        state = C.c_uint64(rng.state)
        tok = C.c_uint32()
        self._check(self._lib.llm_cuda_sample_with(self._h, row.ctypes.data, row.size, C.byref(cfg),
                                                   rec.ctypes.data if rec.size else None, rec.size, C.byref(state),
                                                   C.byref(tok)))
        rng.state = state.value
        return int(tok.value)

    def sample(self, logits, temperature: float, rng: Rng) -> int:
        """sample(logits, temperature, rng) (generate.rs:423-433): temperature only."""
        row = np.ascontiguousarray(logits, dtype=np.float32)
        state = C.c_uint64(rng.state)
        tok = C.c_uint32()
        self._check(self._lib.llm_cuda_sample(self._h, row.ctypes.data, row.size, temperature, C.byref(state),
                                              C.byref(tok)))
        rng.state = state.value
        return int(tok.value)


def _as_signed(x):
    """numpy uint32/uint64 arrays -> same bits as int32/int64 (torch has no full unsigned support)."""
    if isinstance(x, np.ndarray):
        if x.dtype == np.uint32:
            return x.view(np.int32)
        if x.dtype == np.uint64:
            return x.view(np.int64)
    return x


_default: Optional[Sampler] = None


def default_sampler() -> Sampler:
    global _default
    if _default is None:
        _default = Sampler()
    return _default


def sample_with(logits, sampling: SamplingConfig, recent: Sequence[int], rng: Rng) -> int:
    """Module-level `sample_with`, same shape as the reference's free function."""
    return default_sampler().sample_with(logits, sampling, recent, rng)


def sample(logits, temperature: float, rng: Rng) -> int:
    return default_sampler().sample(logits, temperature, rng)
