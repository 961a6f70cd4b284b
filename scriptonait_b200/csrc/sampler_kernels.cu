// Kernels of the B200 token sampler (sm_100a) and their launch plans.
//
// stream_select_kernel   one pass over the logits of a row (or of a column
//                        shard of it): allowed mask, repetition penalty and the
//                        selection filter are applied while the row streams
//                        through registers with 128-bit loads; only the few
//                        values that can still reach the kept set are staged
//                        in shared memory, radix-selected, sorted and pushed
//                        through the exact ordered tail of sample_with.
// merge_draw_kernel      the ordered tail over candidate lists gathered from
//                        several GPUs (vocabulary sharding).
// full_sort_row          (device function of the streaming kernel) literal full
//                        ordering of a row in global scratch, for the rare rows
//                        whose kept set or draw reaches past the window.
// advance_rows_kernel    decode-loop glue (history ring, EOS, draw counter).
// pack_allowed_kernel    bool-per-id -> bit mask.
//
// Reference: crates/llm-core/src/generate.rs:325-420 (sample_with),
// :157-182 (Generator::step / recent_tokens).
#include "sampler_kernels.h"

#include <stdio.h>

#include <cuda_bf16.h>

#include "sampler_device.cuh"

namespace llmc {

template <typename ElemT>
struct Traits;
template <>
struct Traits<float> {
    static constexpr int VEC = 4;  // elements per 16-byte vector
    static constexpr uint32_t NAN4 = 0x7fc00000u;
};
template <>
struct Traits<uint16_t> {
    static constexpr int VEC = 8;
    static constexpr uint32_t NAN4 = 0x7fc07fc0u;
};

template <typename ElemT>
__device__ __forceinline__ void unpack(const uint4& v, float (&x)[Traits<ElemT>::VEC]);
template <>
__device__ __forceinline__ void unpack<float>(const uint4& v, float (&x)[4]) {
    x[0] = __uint_as_float(v.x);
    x[1] = __uint_as_float(v.y);
    x[2] = __uint_as_float(v.z);
    x[3] = __uint_as_float(v.w);
}
template <>
__device__ __forceinline__ void unpack<uint16_t>(const uint4& v, float (&x)[8]) {
    // bf16 -> f32 is a 16-bit shift (crates/llm-core/src/bf16.rs:22-25); the lower address is the low half
    x[0] = __uint_as_float(v.x << 16);
    x[1] = __uint_as_float(v.x & 0xffff0000u);
    x[2] = __uint_as_float(v.y << 16);
    x[3] = __uint_as_float(v.y & 0xffff0000u);
    x[4] = __uint_as_float(v.z << 16);
    x[5] = __uint_as_float(v.z & 0xffff0000u);
    x[6] = __uint_as_float(v.w << 16);
    x[7] = __uint_as_float(v.w & 0xffff0000u);
}

// Maximum of the elements of one 16-byte vector, NaN elements ignored.
template <typename ElemT>
__device__ __forceinline__ float vector_max(const uint4& v);
template <>
__device__ __forceinline__ float vector_max<float>(const uint4& v) {
    return fmaxf(fmaxf(__uint_as_float(v.x), __uint_as_float(v.y)), fmaxf(__uint_as_float(v.z), __uint_as_float(v.w)));
}
template <>
__device__ __forceinline__ float vector_max<uint16_t>(const uint4& v) {
    // packed bf16 maxima: three 2-wide maxima, one across the halves, then the exact widening shift
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&v.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
    const __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162*>(&v.z);
    const __nv_bfloat162 d = *reinterpret_cast<const __nv_bfloat162*>(&v.w);
    const __nv_bfloat162 m2 = __hmax2(__hmax2(a, b), __hmax2(c, d));
    const __nv_bfloat16 m = __hmax(__low2bfloat16(m2), __high2bfloat16(m2));
    return __uint_as_float((uint32_t)__bfloat16_as_ushort(m) << 16);
}

__device__ __forceinline__ uint32_t vol_load(const uint32_t* p) { return *(const volatile uint32_t*)p; }

// ---- bulk-copy (TMA) ring: global -> shared, completion on an mbarrier -------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// One elected thread: `bytes` (multiple of 16) from 16-byte aligned global memory to
// 16-byte aligned shared memory of this CTA.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}
// One poll with a suspend-time hint: the thread sleeps in hardware until the phase completes or
// the hint (nanoseconds) runs out, so waiting warps do not flood the shared-memory pipeline with
// polls that every other warp's loads, stores and atomics would queue behind.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity), "r"(20000u)
        : "memory");
    return ok != 0u;
}
// Bounded wait: gives up after WAIT_LIMIT polls (each poll blocks for up to 20 us, about a
// second in all), records it, and lets the CTA run to its end.
constexpr uint32_t WAIT_LIMIT = 1u << 16;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(64);
    }
    return false;
}

// A row that needs the full ordering where no full-sort scratch exists (the allocation-free
// entry point, candidate lists gathered from other GPUs): reported, not guessed.
__device__ __forceinline__ void report_unresolved(const KParams& P, uint32_t b) {
    if (P.out_q) {
        P.out_cnt[b] = 0u;
        return;
    }
    P.tokens[b] = 0u;
    if (P.row_flags) P.row_flags[b] = LLM_CUDA_ROW_INVALID;
    if (P.kept_count) P.kept_count[b] = 0u;
}

// Streaming threshold of window mode for a given maximum (both in the post-temperature domain).
__device__ __forceinline__ float window_stream_bound(float qmax) {
    return __fsub_rn(__fsub_rn(qmax, WINDOW_STREAM), __fmul_rn(fabsf(qmax), 2.384185791015625e-07f));
}
__device__ __forceinline__ float temper(float x, float T) { return (T == 1.0f) ? x : __fdiv_rn(x, T); }  // generate.rs:357-359

// The r-th largest of the 32 lanes' keys (1 <= r <= 32), returned to every lane. Keys are ordered
// keys of floats, all above 0, so 0 serves as "taken".
__device__ __forceinline__ uint32_t warp_rth_largest(uint32_t key, uint32_t r, unsigned lane) {
    if (r <= 8u) {
        uint32_t cur = key, res = 0u;
        for (uint32_t i = 0; i < r; ++i) {
            res = __reduce_max_sync(FULL_MASK, cur);
            const unsigned who = __ballot_sync(FULL_MASK, cur == res);
            if ((int)lane == __ffs(who) - 1) cur = 0u;  // take one holder of the maximum out
        }
        return res;
    }
    uint32_t rank = 0u;
#pragma unroll 4
    for (int o = 1; o < 32; ++o) {
        const unsigned src = (lane + o) & 31u;
        const uint32_t other = __shfl_sync(FULL_MASK, key, src);
        rank += (other > key || (other == key && src < lane)) ? 1u : 0u;
    }
    const unsigned holder = __ballot_sync(FULL_MASK, rank == r - 1u);
    return __shfl_sync(FULL_MASK, key, __ffs(holder) - 1);
}

// After all candidates of a row are in cand[0..n): final selection, ordering
// and either the ordered tail (token out) or the candidate list out. `scratch`
// is EPILOGUE_SCRATCH bytes of shared memory nothing else uses any more.
// `need_k`: the candidates came from a sampled threshold, and only decide the row if at least k_eff of them exist.
static __device__ int finish_row(const KParams& P, uint32_t b, const RowCfg& rc, uint32_t n, bool overflow, float qmax, Shared& S,
                           float* cand_q, uint32_t* cand_i, unsigned char* scratch, bool window_filtered = false,
                           bool need_k = false) {
    float* probs = reinterpret_cast<float*>(scratch);                               // up to MAX_SORT floats
    uint64_t* rank_keys = reinterpret_cast<uint64_t*>(scratch + RANK_KEYS_OFF);     // THREADS 64-bit words, past probs[THREADS)
    uint64_t* net_keys = reinterpret_cast<uint64_t*>(scratch);                      // 2048 keys, before any probability exists
    if (!rc.windowed) {
        if (need_k && !overflow && n < rc.k_eff) return 2;  // the sampled threshold was too high for this row
        // a set the rank sort below takes in one go needs no selection first: it is cut after sorting
        if (n > (uint32_t)THREADS) n = keep_top_k(n, rc.k_eff, S, cand_q, cand_i);
    } else if (!overflow) {
        // exact window: exactly the terms the reference's f32 sums can see
        if (!window_filtered)
            n = compact_inplace(
                n, [=](float q, uint32_t) { return (__fsub_rn(q, qmax) >= WINDOW_EXACT) || (q == qmax); }, S, cand_q, cand_i);
        uint32_t m = 1u;  // the sort pads to a power of two inside the buffer
        while (m < n) m <<= 1;
        if (m > P.ccap || n > MAX_SORT) overflow = true;
    }
    // ids blocked by the allowed mask are skipped by the stream. They only matter when the ordering
    // runs out of other values (fewer unmasked values than the rank cut, or nothing finite at all):
    // then the -inf entries belong to the kept set, and the full ordering of the row produces them.
    if (P.allowed_bits && !P.out_q && !overflow) {
        if (!rc.windowed && n < rc.k_eff) return 2;
        if (rc.windowed && qmax == neg_inf()) return 2;
    }
    if (overflow) return 1;  // the candidates did not fit: the window tier in global memory can still take the row
    PHASE(3);
    // sets of up to THREADS entries are ranked directly, the exponentials computed alongside
    const bool small = n <= (uint32_t)THREADS;
    const bool small_tail = small && !P.out_q && !rc.greedy;
    if (small)
        sort_small(n, S, cand_q, cand_i, rank_keys, S.hist[0], probs, small_tail);
    else if (n <= 2048u)
        sort_keys64(n, cand_q, cand_i, net_keys);
    else
        sort_candidates(n, cand_q, cand_i);
    PHASE(4);
    const uint32_t n_use = min(n, rc.k_eff);
    const bool truncated = rc.windowed && (n_use < rc.k_eff);
    if (P.out_q) {  // vocabulary sharding, step 1: the ordered list is the result
        grid_dependency_wait();
        for (uint32_t i = threadIdx.x; i < min(n_use, P.out_stride); i += THREADS) {
            P.out_q[(size_t)b * P.out_stride + i] = cand_q[i];
            P.out_i[(size_t)b * P.out_stride + i] = cand_i[i];
        }
        if (threadIdx.x == 0) P.out_cnt[b] = min(n_use, P.out_stride);
        return 0;
    }
    if (rc.greedy || n_use == 0u) {
        if (threadIdx.x == 0) {
            S.token = n_use ? cand_i[0] : 0u;  // ops/loss.rs:6-16: first index of the maximum; 0 when nothing compares greater than -inf
            if (n_use && cand_q[0] == neg_inf()) S.token = 0u;
            S.out_flags = rc.greedy ? LLM_CUDA_ROW_GREEDY : LLM_CUDA_ROW_DEGENERATE;
            S.kept_n = 0u;
            S.f_sum = S.f_total = S.f_u = S.f_thr = S.f_r = 0.f;
        }
        cta_sync();
        write_row_outputs(P, b, 0u, S, n_use ? cand_q[0] : 0.f, cand_i, probs, 0u);
        return 0;
    }
    const uint32_t wflag = rc.windowed ? LLM_CUDA_ROW_WINDOWED : 0u;
    ordered_tail(P, b, rc, n_use, truncated, rc.k_eff, S, cand_q, cand_i, probs, small_tail);
    PHASE(5);
    if (S.out_flags & ROW_NEEDS_FULL) return 2;  // the kept set or the walk leaves the window: the whole row is needed
    write_row_outputs(P, b, wflag, S, cand_q[0], cand_i, probs, S.keep);
    PHASE(6);
    PHASE(11);
    return 0;
}

// Pulls the candidate lists of `nsh` shards of row b into cand[] (compacting
// whenever the next list would not fit) and returns the count; `overflow` and
// `qmax` as finish_row expects them.
constexpr uint32_t LIST_SORTED = 0x40000000u;  // flag in a list's count: entries are in the reference order
constexpr uint32_t LIST_COUNT = 0x3fffffffu;

static __device__ uint32_t merge_lists(const KParams& P, uint32_t b, const RowCfg& rc, uint32_t nsh, Shared& S, float* cand_q,
                                uint32_t* cand_i, bool& overflow, float& qmax, bool all_sorted = false) {
    const uint32_t LOWEST = 0x007fffffu;  // okey(-inf)
    if (threadIdx.x == 0) {
        S.count = 0u;
        S.max_key = LOWEST;
        S.keep = 0u;      // overflow marker seen
        S.newcount = 0u;  // entries of all lists together
        S.tau_key = LOWEST;      // largest k-th entry of a sorted list
        S.minkey = 0xffffffffu;  // smallest r-th entry over the lists, r = ceil(k / lists)
    }
    cta_sync();
    // Rank-cut rows: two lower bounds of the k-th largest value come for free from sorted lists. A
    // list's k-th entry has k entries at or above it; and with r = ceil(k / lists), every list has r
    // entries at or above its own r-th entry, so the smallest of those has lists * r >= k. Entries
    // below the better of the two cannot be among the best k and are not copied at all.
    const uint32_t k = rc.k_eff;
    const uint32_t r = (k + nsh - 1u) / nsh;
    for (uint32_t s = threadIdx.x; s < nsh; s += THREADS) {
        const size_t at = (size_t)s * P.sc_cnt_shard + b;
        if (P.sc_maxkey) atomicMax(&S.max_key, __ldcg(&P.sc_maxkey[at]));
        const uint32_t raw = __ldcg(&P.sc_cnt[at]);
        if (raw == 0xffffffffu || (P.sc_need && (raw > P.sc_stride || raw < P.sc_need))) {
            S.keep = 1u;
        } else {
            const uint32_t cnt = min(raw & LIST_COUNT, P.sc_stride);
            atomicAdd(&S.newcount, cnt);
            if (!rc.windowed) {
                const bool sorted = all_sorted || (raw & LIST_SORTED);
                const float* sq = P.sc_q + (size_t)s * P.sc_shard_words + (size_t)b * P.sc_stride;
                if (sorted && cnt >= k) atomicMax(&S.tau_key, okey(__ldcg(&sq[k - 1u])));
                atomicMin(&S.minkey, (sorted && cnt >= r) ? okey(__ldcg(&sq[r - 1u])) : LOWEST);
            }
        }
    }
    cta_sync();
    overflow = S.keep != 0u;
    qmax = okey_to_float(S.max_key);
    const float tq = window_stream_bound(qmax);
    if (!overflow && S.newcount <= P.ccap) {
        // everything fits at once: each warp copies whole lists, all lists in flight together
        const uint32_t thr = rc.windowed ? LOWEST : max(S.tau_key, S.minkey == 0xffffffffu ? LOWEST : S.minkey);
        const uint32_t lane = threadIdx.x & 31u;
        for (uint32_t s = threadIdx.x >> 5; s < nsh; s += WARPS) {
            const uint32_t raw = __ldcg(&P.sc_cnt[(size_t)s * P.sc_cnt_shard + b]);
            const uint32_t cnt = min(raw & LIST_COUNT, P.sc_stride);
            const bool sorted = all_sorted || (raw & LIST_SORTED);
            const float* sq = P.sc_q + (size_t)s * P.sc_shard_words + (size_t)b * P.sc_stride;
            const uint32_t* si = P.sc_i + (size_t)s * P.sc_shard_words + (size_t)b * P.sc_stride;
            for (uint32_t i0 = 0; i0 < cnt; i0 += 32u) {
                const uint32_t i = i0 + lane;
                const float q = i < cnt ? __ldcg(&sq[i]) : 0.0f;
                const bool pass = i < cnt && okey(q) >= thr;
                const unsigned m = __ballot_sync(FULL_MASK, pass);
                if (m == 0u) {
                    if (sorted && !rc.windowed) break;  // everything further down the list is smaller still
                    continue;
                }
                uint32_t base = 0u;
                if (lane == 0) base = atomicAdd(&S.count, (uint32_t)__popc(m));
                base = __shfl_sync(FULL_MASK, base, 0);
                if (pass) {
                    const uint32_t slot = base + (uint32_t)__popc(m & ((1u << lane) - 1u));
                    cand_q[slot] = q;
                    cand_i[slot] = __ldcg(&si[i]);
                }
            }
        }
        cta_sync();
        return S.count;
    }
    for (uint32_t s = 0; s < nsh && !overflow; ++s) {
        const uint32_t cnt = min(__ldcg(&P.sc_cnt[(size_t)s * P.sc_cnt_shard + b]) & LIST_COUNT, P.sc_stride);
        uint32_t n = S.count;
        if (n + cnt > P.ccap) {
            if (!rc.windowed) {
                n = keep_top_k(n, rc.k_eff, S, cand_q, cand_i);
            } else {
                n = compact_inplace(
                    n, [=](float q, uint32_t) { return q >= tq; }, S, cand_q, cand_i);
            }
            if (n + cnt > P.ccap) overflow = true;
        }
        if (overflow) break;
        const float* sq = P.sc_q + (size_t)s * P.sc_shard_words + (size_t)b * P.sc_stride;
        const uint32_t* si = P.sc_i + (size_t)s * P.sc_shard_words + (size_t)b * P.sc_stride;
        for (uint32_t i = threadIdx.x; i < cnt; i += THREADS) {
            const float q = __ldcg(&sq[i]);
            cand_q[n + i] = q;
            cand_i[n + i] = __ldcg(&si[i]);
        }
        cta_sync();
        if (threadIdx.x == 0) S.count = n + cnt;
        cta_sync();
    }
    return S.count;
}

// ---------------------------------------------------------------------------
// The hot kernel. Grid (split, batch); one CTA streams the columns
// [shard*shard_cols, ...) of one row through a ring of RING_STAGES shared-memory
// stages (12 KB or 16 KB each, the launch plan's choice) filled by bulk copies, so up to
// 36 or 48 KB are in flight per CTA whatever the occupancy.
// MODE trims the code to what a launch can need (the hot loop must stay small enough for the
// instruction cache): 0 = rows of either kind, 1 = every row runs in window mode, 2 = no row does.
constexpr int STREAM_THREADS = THREADS + 32;  // THREADS consumers + one warp that only issues the bulk copies
// ---------------------------------------------------------------------------
// Full ordering of a row in global scratch (stable radix sort of 32-bit keys with
// the column index as payload, L2-resident), then the ordered tail exactly as the
// reference walks it. Much slower than the streaming path and rarely needed:
// rows whose window overflowed or whose kept set / walk left the window. Run by
// the 256 consumer threads of the CTA that found the row undecided, in one of
// P.full_nslots scratch slots; `hkeys/hcnt` is the CTA's id->count table
// (P.hash_slots entries, rebuilt here for the whole vocabulary).
struct FullShared {
    RowCfg rc;
    uint32_t nvalid, keep, token, flags, kept_n, slot;
    float sum, total, u, r, thr, mx;
};


// Claims a free scratch slot. Every holder is a running CTA of this same grid that releases its
// slot without waiting for anyone, so a bounded poll is enough; 0xffffffff when the bound runs out.
static __device__ uint32_t acquire_full_slot(const KParams& P) {
    const uint32_t n = P.full_nslots;
    if (!P.full_slots || n == 0u) return 0xffffffffu;
    uint32_t i = (blockIdx.y * gridDim.x + blockIdx.x) % n;
    for (uint32_t round = 0; round < P.full_slot_rounds; ++round) {
        for (uint32_t k = 0; k < n; ++k) {
            if (atomicCAS(&P.full_slots[i], 0u, 1u) == 0u) return i;
            i = (i + 1u == n) ? 0u : i + 1u;
        }
        __nanosleep(4000);
    }
    return 0xffffffffu;
}

// Shared-memory words of the full ordering's working area (`work`): the radix sort's tables (the chains
// use the per-warp totals' words).
constexpr uint32_t WORK_HIST = 0u;      // [2][256] digit histograms: this pass's, and the next pass's while keys are moved
constexpr uint32_t WORK_BASE = 512u;    // [256] where the next key of every digit goes
constexpr uint32_t WORK_WTOT = 768u;    // [2][32] per-warp totals (two sets)
constexpr uint32_t WORK_DELTA = 832u;   // [256] per digit: position in the output minus position in the reordered tile
constexpr uint32_t WORK_WRUN = 1088u;   // [2][WARPS][256] per-warp digit counts of a tile (two sets, used alternately)
constexpr uint32_t WORK_TILE = WORK_WRUN + 2u * (uint32_t)WARPS * 256u;  // [2][1024] a tile's keys and columns, ordered by digit
constexpr uint32_t WORK_WORDS = WORK_TILE + 2048u;
static_assert(2u * 32u >= CHAIN_WORDS, "the chains' shared words are the per-warp totals' two sets");
static_assert(512u + WORK_WORDS * 4u <= RING_STAGES * STAGE_BYTES, "the full ordering's working area lives in the ring");

// What the full ordering needs to read one row the way the reference edits it. Held by value in the
// functions that stream the row: fields of the launch parameters, reached through a reference, would
// have to be read again after every store to scratch.
struct RowSource {
    const void* row;               // first logit of the row
    const uint32_t* allowed_bits;  // or NULL
    const uint32_t* hkeys;         // id -> occurrences table of the row's history
    const uint32_t* hcnt;
    uint32_t bf16, vocab, col_offset, eos_id, allowed_len, hash_slots, has_pen;
    float pen, T;
};

__device__ __forceinline__ RowSource row_source(const KParams& P, uint32_t b, const RowCfg& rc, const uint32_t* hkeys, const uint32_t* hcnt) {
    RowSource R;
    R.bf16 = P.dtype == LLM_CUDA_DTYPE_BF16 ? 1u : 0u;
    R.row = R.bf16 ? static_cast<const void*>(reinterpret_cast<const uint16_t*>(P.logits) + (size_t)b * P.row_stride)
                   : static_cast<const void*>(reinterpret_cast<const float*>(P.logits) + (size_t)b * P.row_stride);
    R.allowed_bits = P.allowed_bits;
    R.hkeys = hkeys;
    R.hcnt = hcnt;
    R.vocab = P.vocab;
    R.col_offset = P.col_offset;
    R.eos_id = P.eos_id;
    R.allowed_len = P.allowed_len;
    R.hash_slots = P.hash_slots;
    R.has_pen = rc.has_pen;
    R.pen = rc.pen;
    R.T = rc.T;
    return R;
}

__device__ __forceinline__ float source_load(const RowSource& R, uint32_t c) {
    if (R.bf16) return load_logit(reinterpret_cast<const uint16_t*>(R.row) + c);
    return load_logit(reinterpret_cast<const float*>(R.row) + c);
}

// One logit as the reference orders it: allowed mask (generate.rs:333-341), penalty, temperature.
__device__ __forceinline__ float source_edit(const RowSource& R, uint32_t c, float x) {
    const uint32_t gid = R.col_offset + c;
    if (R.allowed_bits && gid != R.eos_id && gid < R.allowed_len && ((__ldg(&R.allowed_bits[gid >> 5]) >> (gid & 31u)) & 1u) == 0u)
        x = neg_inf();
    if (R.has_pen) x = penalize(x, R.pen, hash_count(R.hkeys, R.hcnt, R.hash_slots, gid));
    return temper(x, R.T);
}

// Every column of the row as a (key, column) pair in column order; returns this thread's count of
// values that are not NaN. ~(ordered bits) ascending == value descending; a stable sort from column
// order gives index ascending among equal values, which is the reference's order. Eight columns per
// thread and round, their loads travelling together; the loop is kept small enough to need no spill
// (the streaming kernel runs with almost no L1, and a spilled value costs a trip to L2).
template <bool EDITS>
__device__ __forceinline__ uint32_t build_all_keys_t(const RowSource& R, uint32_t* __restrict__ sk, uint32_t* __restrict__ si) {
    const uint32_t V = R.vocab;
    const float T = R.T;
    uint32_t valid = 0u;
    for (uint32_t c0 = threadIdx.x; c0 < V; c0 += 8u * THREADS) {
        float x[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t c = c0 + (uint32_t)u * THREADS;
            x[u] = c < V ? source_load(R, c) : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t c = c0 + (uint32_t)u * THREADS;
            if (c >= V) continue;
            const float q = EDITS ? source_edit(R, c, x[u]) : temper(x[u], T);
            uint32_t key = 0xffffffffu;  // NaN: behind everything (no value maps here: ~okey(-inf) is 0xff800000)
            if (q == q) {
                key = ~okey(q);
                ++valid;
            }
            __stcg(&sk[c], key);
            __stcg(&si[c], c);
        }
    }
    return valid;
}

static __device__ __noinline__ uint32_t build_all_keys(const RowSource R, uint32_t* __restrict__ sk, uint32_t* __restrict__ si) {
    if (R.allowed_bits || R.has_pen) return build_all_keys_t<true>(R, sk, si);
    return build_all_keys_t<false>(R, sk, si);
}

// The members of a row's significance window, as (key, column) pairs compacted in column order into
// sk / si (`cap` entries each); returns their number (the same in every thread). Rounds of 2048
// columns: warp w takes columns [256 w, 256 w + 256) of the round, 32 consecutive columns per step, so
// (warp, step, lane) order is column order; ballots place a member inside its warp, warp totals (one
// barrier per round, two sets of totals used alternately) place the warp.
template <bool EDITS>
__device__ __forceinline__ uint32_t build_window_keys_t(const KParams& P, const RowSource& R, float win_qmax, uint32_t* __restrict__ sk,
                                                        uint32_t* __restrict__ si, uint32_t cap, uint32_t* work) {
    const uint32_t tid = threadIdx.x;
    const unsigned lane = tid & 31u, warp = tid >> 5;
    const unsigned below = (1u << lane) - 1u;
    const uint32_t V = R.vocab;
    constexpr int STEPS = 8;
    const float T = R.T;
    uint32_t run_base = 0u;  // the same in every thread
    uint32_t it = 0u;
    for (uint32_t chunk = 0; chunk < V; chunk += (uint32_t)STEPS * THREADS, ++it) {
        const uint32_t c0 = chunk + warp * (uint32_t)STEPS * 32u + lane;
        float q[STEPS];
#pragma unroll
        for (int e = 0; e < STEPS; ++e) {
            const uint32_t c = c0 + (uint32_t)e * 32u;
            q[e] = c < V ? source_load(R, c) : 0.0f;
        }
        uint32_t mine = 0u, wcount = 0u;
#pragma unroll
        for (int e = 0; e < STEPS; ++e) {
            const uint32_t c = c0 + (uint32_t)e * 32u;
            bool in = false;
            if (c < V) {
                q[e] = EDITS ? source_edit(R, c, q[e]) : temper(q[e], T);
                in = (__fsub_rn(q[e], win_qmax) >= WINDOW_EXACT) || (q[e] == win_qmax);  // false for NaN
            }
            if (in) mine |= 1u << e;
            wcount += (uint32_t)__popc(__ballot_sync(FULL_MASK, in));
        }
        uint32_t* wtot = work + WORK_WTOT + (it & 1u) * 32u;
        if (lane == 0) wtot[warp] = wcount;
        cta_sync();
        uint32_t off = run_base, total = 0u;
#pragma unroll
        for (uint32_t w = 0; w < (uint32_t)WARPS; ++w) {
            const uint32_t t = wtot[w];
            if (w < warp) off += t;
            total += t;
        }
#pragma unroll
        for (int e = 0; e < STEPS; ++e) {
            const bool in = (mine >> e) & 1u;
            const unsigned m = __ballot_sync(FULL_MASK, in);
            const uint32_t at = off + (uint32_t)__popc(m & below);
            off += (uint32_t)__popc(m);
            if (in && IN_BOUNDS(at, cap)) {
                __stcg(&sk[at], ~okey(q[e]));
                __stcg(&si[at], c0 + (uint32_t)e * 32u);
            }
        }
        run_base += total;
    }
    cta_sync();
    return run_base;
}

static __device__ __noinline__ uint32_t build_window_keys(const KParams& P, const RowSource R, float win_qmax, uint32_t* __restrict__ sk,
                                                   uint32_t* __restrict__ si, uint32_t cap, uint32_t* work) {
    if (R.allowed_bits || R.has_pen) return build_window_keys_t<true>(P, R, win_qmax, sk, si, cap, work);
    return build_window_keys_t<false>(P, R, win_qmax, sk, si, cap, work);
}

// The lanes of the warp that hold the same 8-bit digit as this one, from one vote per bit (`match_any`
// takes a step per distinct value, about a thousand cycles for 32 different digits). Lanes without a
// key (`have` false) match nobody and are matched by nobody.
__device__ __forceinline__ unsigned digit_peers(uint32_t d, bool have) {
    unsigned peers = __ballot_sync(FULL_MASK, have);
#pragma unroll
    for (int bit = 0; bit < 8; ++bit) {
        const bool set = (d >> bit) & 1u;
        const unsigned m = __ballot_sync(FULL_MASK, set);
        peers &= set ? m : ~m;
    }
    return peers;
}

// One key's digit into a shared-memory histogram: plain additions, except that a digit common to the
// whole warp (equal keys, key bits that are zero in every value) is added once.
__device__ __forceinline__ void count_digit(uint32_t* hist, uint32_t d, bool have) {
    const uint32_t d0 = __shfl_sync(FULL_MASK, d, 0);
    if (__all_sync(FULL_MASK, have && d == d0)) {
        if ((threadIdx.x & 31u) == 0u) atomicAdd(&hist[d0], 32u);
    } else if (have) {
        atomicAdd(&hist[d], 1u);
    }
}

// Least-significant-digit radix sort, 8 bits per pass, by this CTA alone. Per pass: the digit
// histogram (counted while the previous pass moved the keys, or by a pass of its own), an exclusive
// scan, then a stable scatter in tiles of 1024 keys - warp w takes keys [128 w, 128 w + 128) of the
// tile, 32 consecutive keys per step, so (warp, step, lane) order is the order the keys are in. A key's
// place inside its tile is the tile's keys of smaller digits + the same-digit keys of earlier warps +
// those earlier in its own warp (one vote per digit bit finds the lanes that share a digit, a returning
// shared-memory addition counts the earlier steps). The tile is put in that order in shared memory
// first and written out from there, so that consecutive threads store to consecutive addresses within
// a digit: scattered 4-byte stores, one memory transaction each, cost more than everything else in
// the pass together. The next tile's keys are already on their way while this tile is placed.
// Sorts n_all (key, column) pairs; the pointers are exchanged so that sk / si hold the result.
static __device__ __noinline__ void radix_sort_row(const KParams& P, uint32_t n_all, uint32_t*& sk_io, uint32_t*& si_io, uint32_t*& dk_io, uint32_t*& di_io,
                                            uint32_t* work) {
    const uint32_t tid = threadIdx.x;
    const unsigned lane = tid & 31u, warp = tid >> 5;
    const unsigned below = (1u << lane) - 1u;
    // local copies: the stores below must not be taken for stores to the caller's pointer variables
    uint32_t* __restrict__ sk = sk_io;
    uint32_t* __restrict__ si = si_io;
    uint32_t* __restrict__ dk = dk_io;
    uint32_t* __restrict__ di = di_io;
    constexpr int KEYS = 4;
    constexpr uint32_t TILE = KEYS * (uint32_t)THREADS, WSPAN = KEYS * 32u;
    uint32_t* gbase = work + WORK_BASE;
    uint32_t* wtot = work + WORK_WTOT;
    uint32_t* wtot_tile = work + WORK_WTOT + 32u;
    uint32_t* delta = work + WORK_DELTA;
    uint32_t* tk = work + WORK_TILE;
    uint32_t* ti = tk + TILE;
    uint32_t cur = 0u;        // which histogram belongs to this pass
    bool counted = false;     // ... and whether the previous pass filled it
    for (uint32_t shift = 0; shift < 32u; shift += 8u) {
        uint32_t* hist = work + WORK_HIST + cur * 256u;
        uint32_t* hist_next = work + WORK_HIST + (cur ^ 1u) * 256u;
        if (!counted) {
            hist[tid] = 0u;
            cta_sync();
            for (uint32_t i0 = 0; i0 < n_all; i0 += 8u * THREADS) {
                uint32_t kk[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const uint32_t i = i0 + (uint32_t)u * THREADS + tid;
                    kk[u] = i < n_all ? __ldcg(&sk[i]) : 0u;
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) count_digit(hist, (kk[u] >> shift) & 255u, i0 + (uint32_t)u * THREADS + tid < n_all);
            }
            cta_sync();
        }
        const uint32_t mine = hist[tid];
        hist_next[tid] = 0u;
        counted = false;
        if (cta_sync_or(mine == n_all ? 1 : 0)) continue;  // every key has the same digit: nothing moves
        uint32_t incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t y = __shfl_up_sync(FULL_MASK, incl, o);
            if (lane >= (unsigned)o) incl += y;
        }
        if (lane == 31) wtot[warp] = incl;
        {   // the first tile's per-warp counts start from zero
            uint32_t* w0 = work + WORK_WRUN;
#pragma unroll
            for (uint32_t w = 0; w < (uint32_t)WARPS; ++w) w0[w * 256u + tid] = 0u;
        }
        cta_sync();
        uint32_t pre = 0u;
        for (uint32_t w = 0; w < warp; ++w) pre += wtot[w];
        gbase[tid] = pre + incl - mine;
        const bool count_next = shift < 24u;
        uint32_t kn[KEYS];
#pragma unroll
        for (int e = 0; e < KEYS; ++e) {
            const uint32_t i = warp * WSPAN + (uint32_t)e * 32u + lane;
            kn[e] = i < n_all ? __ldcg(&sk[i]) : 0u;
        }
        cta_sync();
        uint32_t t = 0u;
        for (uint32_t tile = 0; tile < n_all; tile += TILE, ++t) {
            uint32_t* wr = work + WORK_WRUN + (t & 1u) * (uint32_t)WARPS * 256u;
            uint32_t* wr_other = work + WORK_WRUN + ((t + 1u) & 1u) * (uint32_t)WARPS * 256u;
            uint32_t k[KEYS], id[KEYS], pos[KEYS];
            const uint32_t i_first = tile + warp * WSPAN + lane;
#pragma unroll
            for (int e = 0; e < KEYS; ++e) k[e] = kn[e];
#pragma unroll
            for (int e = 0; e < KEYS; ++e) {
                const uint32_t i = i_first + TILE + (uint32_t)e * 32u;
                kn[e] = i < n_all ? __ldcg(&sk[i]) : 0u;
            }
#pragma unroll
            for (int e = 0; e < KEYS; ++e) {  // place among the warp's keys of the same digit
                const bool have = i_first + (uint32_t)e * 32u < n_all;
                const uint32_t d = (k[e] >> shift) & 255u;
                const unsigned peers = digit_peers(d, have);
                const uint32_t lower = (uint32_t)__popc(peers & below);
                uint32_t old = 0u;
                if (have && lower == 0u) old = atomicAdd(&wr[warp * 256u + d], (uint32_t)__popc(peers));  // the earlier steps' count
                old = __shfl_sync(FULL_MASK, old, have ? __ffs(peers) - 1 : (int)lane);
                pos[e] = old + lower;
            }
            if (count_next) {
#pragma unroll
                for (int e = 0; e < KEYS; ++e) count_digit(hist_next, (k[e] >> (shift + 8u)) & 255u, i_first + (uint32_t)e * 32u < n_all);
            }
            cta_sync();
#pragma unroll
            for (int e = 0; e < KEYS; ++e) {  // the columns: needed two barriers from here
                const uint32_t i = i_first + (uint32_t)e * 32u;
                id[e] = i < n_all ? __ldcg(&si[i]) : 0u;
            }
            // digit `tid`: its keys in this tile; the other table is cleared for the next tile
            uint32_t c = 0u;
#pragma unroll
            for (uint32_t w = 0; w < (uint32_t)WARPS; ++w) {
                c += wr[w * 256u + tid];
                wr_other[w * 256u + tid] = 0u;
            }
            uint32_t before = c;  // becomes the tile's keys of digits up to this one
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t y = __shfl_up_sync(FULL_MASK, before, o);
                if (lane >= (unsigned)o) before += y;
            }
            if (lane == 31) wtot_tile[warp] = before;
            cta_sync();
            {
                uint32_t start = before - c;  // where the digit begins in the reordered tile
                for (uint32_t w = 0; w < warp; ++w) start += wtot_tile[w];
                const uint32_t g = gbase[tid];
                delta[tid] = g - start;
                gbase[tid] = g + c;
#pragma unroll
                for (uint32_t w = 0; w < (uint32_t)WARPS; ++w) {  // the warps' counts become the warps' first positions
                    const uint32_t cw = wr[w * 256u + tid];
                    wr[w * 256u + tid] = start;
                    start += cw;
                }
            }
            cta_sync();
#pragma unroll
            for (int e = 0; e < KEYS; ++e) {
                if (i_first + (uint32_t)e * 32u < n_all) {
                    const uint32_t at = wr[warp * 256u + ((k[e] >> shift) & 255u)] + pos[e];
                    if (!IN_BOUNDS(at, TILE)) continue;
                    tk[at] = k[e];
                    ti[at] = id[e];
                }
            }
            cta_sync();
            const uint32_t m = min(TILE, n_all - tile);
#pragma unroll
            for (int e = 0; e < KEYS; ++e) {
                const uint32_t j = (uint32_t)e * THREADS + tid;
                if (j < m) {
                    const uint32_t kk = tk[j];
                    const uint32_t out = delta[(kk >> shift) & 255u] + j;
                    if (!IN_BOUNDS(out, n_all)) continue;
                    __stcg(&dk[out], kk);
                    __stcg(&di[out], ti[j]);
                }
            }
        }
        cta_sync();  // the moved keys and the next pass's histogram are complete
        counted = count_next;
        cur ^= 1u;
        uint32_t* tmp = sk; sk = dk; dk = tmp;
        tmp = si; si = di; di = tmp;
    }
    sk_io = sk;
    si_io = si;
    dk_io = dk;
    di_io = di;
}

// `try_window` (window rows whose candidates did not fit in shared memory, `win_qmax` their exact
// maximum after temperature): first only the row's significance window is ordered - usually a few
// thousand values instead of the whole row - with the same rules about what such a truncated ordering
// can and cannot decide as the shared-memory path; the whole row follows only if it cannot.
static __device__ __noinline__ void full_sort_row(const KParams& P, uint32_t b, FullShared& F, uint32_t* work, uint32_t* hkeys,
                                           uint32_t* hcnt, bool try_window = false, float win_qmax = 0.0f) {
    const uint32_t tid = threadIdx.x;
    const uint32_t V = P.vocab;
    grid_dependency_wait();  // the scratch slots are shared with the previous launch
    if (!P.full_keys) {
        if (tid == 0) report_unresolved(P, b);
        return;
    }
    cta_sync();  // whatever used this shared memory before is finished
    if (tid == 0) {
        resolve_row(P, b, F.rc);
        F.slot = acquire_full_slot(P);
        F.nvalid = 0u;
        F.keep = 0u;
        F.flags = 0u;
        F.kept_n = 0u;
        F.token = 0u;
        F.sum = F.total = F.u = F.r = F.thr = F.mx = 0.f;
    }
    for (uint32_t i = tid; i < P.hash_slots; i += THREADS) {
        hkeys[i] = EMPTY_KEY;
        hcnt[i] = 0u;
    }
    cta_sync();
    const RowCfg rc = F.rc;
    if (F.slot == 0xffffffffu) {  // no scratch slot came free within the bound: reported, not guessed
        if (tid == 0) {
            report_unresolved(P, b);
            if (P.device_errors) atomicOr(P.device_errors, 2u);
        }
        return;
    }
    // a slot: two (key, index) array pairs for the radix passes to alternate between, and the probabilities
    uint32_t* slot_base = reinterpret_cast<uint32_t*>(P.full_keys) + (size_t)F.slot * 4u * P.full_vpad;
    uint32_t* sk = slot_base;                      // keys in
    uint32_t* si = slot_base + P.full_vpad;        // column indices in
    uint32_t* dk = slot_base + 2u * P.full_vpad;   // keys out
    uint32_t* di = slot_base + 3u * P.full_vpad;   // column indices out
    float* vals = P.full_vals + (size_t)F.slot * P.full_vpad;
    if (rc.has_pen) {
        const uint32_t* hist = P.history + (size_t)b * P.hist_stride;
        for (uint32_t j = tid; j < rc.hlen; j += THREADS) {
            const uint32_t id = __ldg(&hist[j]);
            if (id >= P.col_offset && id - P.col_offset < V) hash_insert(hkeys, hcnt, P.hash_slots, id);
        }
    }
    cta_sync();
    bool filter = try_window;  // this attempt orders the significance window only
    PHASE(14);
    for (;;) {
    uint32_t n_all = V;        // keys to sort
    // ---- keys: ~(ordered bits) ascending == value descending; a stable sort from column order gives
    //      index ascending among equal values, which is the reference's order
    uint32_t myvalid = 0u;
    const RowSource R = row_source(P, b, rc, hkeys, hcnt);
    if (filter) {
        n_all = build_window_keys(P, R, win_qmax, sk, si, P.full_vpad, work);
        if (tid == 0) myvalid = n_all;
    } else {
        myvalid = build_all_keys(R, sk, si);
    }
    if (myvalid) atomicAdd(&F.nvalid, myvalid);
    cta_sync();
    PHASE(3);
    radix_sort_row(P, n_all, sk, si, dk, di, work);
    PHASE(4);
    const uint32_t n = min(F.nvalid, rc.k_eff);
    // window attempt: the reference's ordering continues past these n entries with values outside the
    // significance window; what that leaves undecided is handled as in the shared-memory path
    const bool truncated = filter && n < rc.k_eff;
    auto q_at = [&](uint32_t i) { return okey_to_float(~__ldcg(&sk[i])); };
    auto id_at = [&](uint32_t i) { return P.col_offset + __ldcg(&si[i]); };
    float mx = 0.f;
    bool done = false;
    if (rc.greedy || n == 0u) {
        if (tid == 0) {
            F.token = n ? id_at(0) : 0u;
            if (n && q_at(0) == neg_inf()) F.token = 0u;
            F.flags = rc.greedy ? LLM_CUDA_ROW_GREEDY : LLM_CUDA_ROW_DEGENERATE;
        }
        done = true;
    }
    if (!done) {
        mx = q_at(0);
        if (tid == 0) F.mx = mx;
        for (uint32_t i0 = tid; i0 < n; i0 += 8u * THREADS) {
            float q8[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint32_t i = i0 + (uint32_t)u * THREADS;
                q8[u] = i < n ? q_at(i) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint32_t i = i0 + (uint32_t)u * THREADS;
                if (i < n) __stcg(&vals[i], exp_f32(__fsub_rn(q8[u], mx)));
            }
        }
        cta_sync();
        PHASE(8);
        {   // the sum of the exponentials (generate.rs:386-389), by the whole CTA
            float s = 0.0f;
            cta_chain<true>(vals, n, CHAIN_SUM, 0.0f, &s, work + WORK_WTOT);
            if (tid == 0) {
                F.sum = s;
                F.keep = n;
            }
        }
        cta_sync();
        PHASE(9);
        const float sum = F.sum;
        if ((sum <= 0.0f) || !(fabsf(sum) <= 3.402823466e38f)) {
            if (tid == 0) {
                F.token = id_at(0);
                F.flags = LLM_CUDA_ROW_DEGENERATE;
            }
            done = true;
        }
        if (!done) {
            for (uint32_t i0 = tid; i0 < n; i0 += 8u * THREADS) {
                float e8[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const uint32_t i = i0 + (uint32_t)u * THREADS;
                    e8[u] = i < n ? __ldcg(&vals[i]) : 0.0f;
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const uint32_t i = i0 + (uint32_t)u * THREADS;
                    if (i < n) __stcg(&vals[i], __fdiv_rn(e8[u], sum));
                }
            }
            cta_sync();
            if (rc.min_p > 0.0f) {
                const float thr = __fmul_rn(rc.min_p, __ldcg(&vals[0]));
                uint32_t first_fail = n;
                for (uint32_t i = tid; i < n; i += THREADS) {
                    if (!(__ldcg(&vals[i]) >= thr)) {
                        first_fail = i;
                        break;
                    }
                }
                if (first_fail < n) atomicMin(&F.keep, first_fail);
                cta_sync();
                if (tid == 0) {
                    F.thr = thr;
                    if (F.keep < 1u) F.keep = 1u;
                }
                cta_sync();
            }
            // every window entry passed min-p and more entries follow: whether those pass is only
            // certain when the threshold is at least 2^-24 of the leader
            const bool unknown_tail = truncated && rc.min_p > 0.0f && F.keep == n && rc.min_p < 5.9604644775390625e-08f;
            const bool open_tail = truncated && F.keep == n && !(rc.min_p > 0.0f);  // the kept set continues past the window
            PHASE(10);
            {   // cumulative probability and the draw's walk (generate.rs:396-417), by the whole CTA, every thread alike
                const uint32_t keep_minp = F.keep;
                uint32_t keep = keep_minp;
                float total = 0.0f;
                bool reached = false;
                {
                    const uint32_t at = cta_chain<true>(vals, keep_minp, rc.top_p < 1.0f ? CHAIN_CUMULATIVE : CHAIN_SUM, rc.top_p, &total,
                                                        work + WORK_WTOT);
                    if (rc.top_p < 1.0f && at < keep_minp) {
                        keep = at + 1u;  // the first index whose running sum reaches top_p
                        reached = true;
                    }
                }
                const float u = row_uniform(P, b);
                float rr = __fmul_rn(u, total);
                const float r0 = rr;
                uint32_t flags = LLM_CUDA_ROW_DRAW_CONSUMED;
                const uint32_t at = cta_chain<true>(vals, keep, CHAIN_WALK, 0.0f, &rr, work + WORK_WTOT);
                const bool found = at < keep;
                // entries past the window add less than half an ulp to the running sums, so `total` is final
                const bool tail_kept = open_tail && !reached;
                uint32_t token = 0u;
                if (found) {
                    token = id_at(at);
                    if (unknown_tail) flags = ROW_NEEDS_FULL;
                } else if (tail_kept || unknown_tail) {
                    flags = ROW_NEEDS_FULL;  // the walk continues into entries the window dropped
                } else {
                    token = id_at(keep - 1u);
                    flags |= LLM_CUDA_ROW_FALLBACK_LAST;
                }
                cta_sync();  // everyone has read F.keep
                if (tid == 0) {
                    F.total = total;
                    F.u = u;
                    F.r = r0;
                    F.token = token;
                    F.flags = flags;
                    F.keep = keep;
                    F.kept_n = tail_kept ? rc.k_eff : keep;
                }
            }
        }
    }
    cta_sync();
    PHASE(5);
    if (filter && (F.flags & ROW_NEEDS_FULL)) {
        // the window could not settle the row: once more over the whole row
        cta_sync();  // everyone has seen the flags
        if (tid == 0) {
            F.nvalid = 0u;
            F.keep = 0u;
            F.flags = 0u;
            F.kept_n = 0u;
            F.token = 0u;
            F.sum = F.total = F.u = F.r = F.thr = F.mx = 0.f;
        }
        cta_sync();
        filter = false;
        continue;
    }
    break;
    }  // attempts
    const float mx = F.mx;
    auto id_at = [&](uint32_t i) { return P.col_offset + __ldcg(&si[i]); };
    const uint32_t flags = F.flags | LLM_CUDA_ROW_FULL_SORT;
    if (tid == 0) {
        P.tokens[b] = F.token;
        if (P.row_flags) P.row_flags[b] = flags;
        if (P.kept_count) P.kept_count[b] = F.kept_n;
        if (P.row_stats) {
            float* st = P.row_stats + (size_t)b * LLM_CUDA_ROW_STATS;
            st[0] = mx;
            st[1] = F.sum;
            st[2] = F.total;
            st[3] = F.u;
            st[4] = F.thr;
            st[5] = F.r;
        }
    }
    if (P.kept_cap && (flags & LLM_CUDA_ROW_DRAW_CONSUMED)) {
        const uint32_t lim = min(F.keep, P.kept_cap);
        for (uint32_t i = tid; i < lim; i += THREADS) {
            if (P.kept_ids) P.kept_ids[(size_t)b * P.kept_cap + i] = id_at(i);
            if (P.kept_probs) P.kept_probs[(size_t)b * P.kept_cap + i] = __ldcg(&vals[i]);
        }
    }
    cta_sync();
    PHASE(6);
    PHASE(11);
    if (tid == 0) {
        __threadfence();
        atomicExch(&P.full_slots[F.slot], 0u);
    }
}

// Optional per-stage output: the edited value (allowed mask, every penalty application; before temperature)
// at each history position whose id lies in this CTA's columns [gid0, gid0 + ncols); NaN for ids outside
// the matrix. `table`: the id -> edited value table exists (penalty rows of kernels built with tables).
// Not inlined: rarely asked for, and kept out of the streaming kernel's register allocation.
template <typename ElemT>
__device__ __noinline__ void write_penalized(const KParams& P, uint32_t b, uint32_t hlen, uint32_t gid0, uint32_t ncols, bool shard0,
                                             bool table, const uint32_t* hkeys, const uint32_t* hcnt) {
    const uint32_t* hist = P.history + (size_t)b * P.hist_stride;
    float* out = P.penalized_out + (size_t)b * P.hist_stride;
    const ElemT* row = reinterpret_cast<const ElemT*>(P.logits) + (size_t)b * P.row_stride;
    for (uint32_t j = threadIdx.x; j < hlen; j += THREADS) {
        const uint32_t id = __ldg(&hist[j]);
        if (id >= gid0 && id - gid0 < ncols) {
            float v;
            if (table) {
                v = __uint_as_float(0x7fc00000u);
                const uint32_t mask = P.hash_slots - 1u;
                uint32_t h = hash_slot(id, mask);
                for (uint32_t probe = 0; probe < P.hash_slots; ++probe) {
                    if (hkeys[h] == id) {
                        v = __uint_as_float(hcnt[h]);
                        break;
                    }
                    h = (h + 1u) & mask;
                }
            } else {
                v = load_logit(row + (id - P.col_offset));
                if (id_blocked(P, id)) v = neg_inf();
            }
            out[j] = v;
        } else if (shard0 && !(id >= P.col_offset && id - P.col_offset < P.vocab)) {
            out[j] = __uint_as_float(0x7fc00000u);
        }
    }
}

template <typename ElemT, bool BITS, int MODE, int U>
__global__ void __launch_bounds__(STREAM_THREADS, 4) stream_select_kernel(const __grid_constant__ KParams P) {
    constexpr int VEC = Traits<ElemT>::VEC;
    constexpr uint32_t VPS = (uint32_t)U * THREADS;  // 16-byte vectors per stage: U per consumer thread
    constexpr uint32_t STAGE = VPS * 16u;            // bytes per ring stage (12 KB or 16 KB, the launch plan's choice)
    extern __shared__ __align__(128) unsigned char dyn[];
    __shared__ Shared S;
    __shared__ __align__(8) uint64_t full_bar[RING_STAGES];   // a stage's bytes have landed
    __shared__ __align__(8) uint64_t empty_bar[RING_STAGES];  // all consumer warps are done with a stage
    unsigned char* ring = dyn;
    // The candidate buffer and the epilogue scratch are only used after the sweep; when they fit they
    // share the ring's memory (the launch plan decides and passes the offsets).
    float* cand_q = reinterpret_cast<float*>(dyn + P.cand_off);
    uint32_t* cand_i = reinterpret_cast<uint32_t*>(cand_q + P.ccap);
    unsigned char* scratch = dyn + P.scratch_off;  // list of flagged vectors during the revisit, then finish_row's sort keys / probabilities
    uint32_t* bitmap = reinterpret_cast<uint32_t*>(dyn + P.tables_off);
    uint32_t* hkeys = bitmap + P.bitmap_words;
    uint32_t* hcnt = hkeys + P.hash_slots;
    float* lane_top = reinterpret_cast<float*>(hcnt + P.hash_slots);  // rank cuts above 256: every lane's best values
    uint32_t* grp_max = reinterpret_cast<uint32_t*>(lane_top + P.lane_top_words);  // one flag word per 32 vectors

    const uint32_t b = blockIdx.y, shard = blockIdx.x, tid = threadIdx.x;
    const unsigned lane = tid & 31u, warp = tid >> 5;
    const uint32_t LOWEST = 0x007fffffu;  // okey(-inf)
    // overlap_previous = 2: the grid was set up while its predecessor was still running (its CTAs are resident,
    // the launch latency is paid), but it touches no global memory before that kernel has completed
    if (P.wait_first) grid_dependency_wait();
    // A launch that asked to overlap its predecessor is released by the producer lane of every CTA
    // once three eighths of the CTA's row have been requested (measured best: released at the very
    // start, three launches stream at once and then order at once). That launch reads its inputs and
    // writes shared memory only until it has passed grid_dependency_wait(): that comes right before a
    // row's outputs are written, before the split-row scratch and before the full-ordering scratch.
    // ---- this CTA's columns and their 16-byte alignment (independent of the row's parameters)
    const uint32_t c0 = shard * P.shard_cols;
    const uint32_t c1 = min(c0 + P.shard_cols, P.vocab);
    const uint32_t ncols = c1 - c0;
    const ElemT* row = reinterpret_cast<const ElemT*>(P.logits) + (size_t)b * P.row_stride;
    const uint32_t mis = (uint32_t)((reinterpret_cast<uintptr_t>(row + c0) & 15u) / sizeof(ElemT));
    const uint32_t head = min(mis ? (uint32_t)VEC - mis : 0u, ncols);  // leading elements before the first aligned vector
    const uint32_t lead = mis;                                        // bitmap coordinate of column c0
    const uint32_t nvi = (ncols - head) / VEC;                        // whole aligned vectors
    const uint32_t tail0 = head + nvi * VEC;                          // first trailing element (relative to c0)
    const uint32_t ntail = ncols - tail0;
    const uint32_t gid0 = P.col_offset + c0;                          // global id of column c0
    const unsigned char* vbase = reinterpret_cast<const unsigned char*>(row + c0 + head);  // 16-byte aligned
    const uint32_t vtiles = (nvi + VPS - 1u) / VPS;
    const uint32_t first_stages = min((uint32_t)RING_STAGES, vtiles);
    // the stage whose request releases a launch that asked to overlap this one (see below)
    const uint32_t release_at = (vtiles * 3u) / 8u;

    auto issue = [&](uint32_t tt) {  // the producer lane only
        const uint32_t first = tt * VPS;
        const uint32_t nv = min(VPS, nvi - first);
        uint64_t* bar = &full_bar[tt % RING_STAGES];
        mbar_expect_tx(bar, nv * 16u);
        bulk_load(ring + (size_t)(tt % RING_STAGES) * STAGE, vbase + (size_t)first * 16u, nv * 16u, bar);
    };
    // ---- the ring starts before anything else: the producer lane sets up the barriers and requests the
    //      first stages while thread 0 still reads the row's parameters
    if (tid == (uint32_t)THREADS) {
#pragma unroll
        for (int i = 0; i < RING_STAGES; ++i) {
            mbar_init(&full_bar[i], 1u);
            mbar_init(&empty_bar[i], (uint32_t)WARPS);
        }
        mbar_fence_init();
        for (uint32_t tt = 0; tt < first_stages; ++tt) issue(tt);
        if (release_at < first_stages) grid_launch_dependents();  // a short row: released at once
    }
    // the draw's uniform is an input: one thread requests its ingredients now and finishes it after the
    // tables are built, so that the latency hides behind the sweep
    const bool fetch_u = (tid == 32u) && !P.out_q;
    uint64_t u_seed = 0ull, u_done = 0ull;
    float u_given = 0.0f;
    if (fetch_u) {
        if (P.uniforms) {
            u_given = P.uniforms[b];
        } else {
            u_seed = P.seeds ? P.seeds[b] : P.seed_base + (uint64_t)b;
            u_done = P.draw_index ? P.draw_index[b] : 0ull;
        }
    }
    if (tid == 0) {
        resolve_row(P, b, S.rc);
        S.u_pre_valid = 0u;
        S.count = 0u;
        S.tau_key = LOWEST;
        S.max_key = LOWEST;
        S.error = 0u;
        S.last = 0u;
        S.sortmax = 0u;
        S.keep = 0u;
    }
    __syncthreads();  // the one barrier all STREAM_THREADS threads share
    RowCfg rc = S.rc;
    if (MODE == 1) rc.windowed = 1u;  // lets the compiler drop the exact-selection code
    if (MODE >= 2) rc.windowed = 0u;  // ... or the window code
    PHASE(0);
    PHASE(12);
    if (rc.invalid || P.force_full) {
        // the stages already requested must have landed before this CTA's shared memory is given up
        for (uint32_t tt = 0; tt < first_stages; ++tt) (void)mbar_wait_bounded(&full_bar[tt], 0u);
        grid_dependency_wait();
        if (rc.invalid) {
            if (shard == 0 && tid == 0) {
                if (P.out_q) {
                    P.out_cnt[b] = 0u;
                } else {
                    P.tokens[b] = 0u;
                    if (P.row_flags) P.row_flags[b] = LLM_CUDA_ROW_INVALID;
                    if (P.kept_count) P.kept_count[b] = 0u;
                }
            }
            return;
        }
        __syncthreads();  // every thread has seen its stages land: the ring may be reused
        if (warp < (unsigned)WARPS && shard == 0) full_sort_row(P, b, *reinterpret_cast<FullShared*>(ring), reinterpret_cast<uint32_t*>(ring + 512), hkeys, hcnt);
        return;
    }
    const float T = rc.T;

    if (warp == (unsigned)WARPS) {
        // the producer warp: keeps the ring full, refilling a stage as soon as every consumer warp
        // has released it; it takes no part in the consumers' barriers and leaves when all is issued
        if (lane == 0) {
            for (uint32_t tt = first_stages; tt < vtiles; ++tt) {
                if (!mbar_wait_bounded(&empty_bar[tt % RING_STAGES], ((tt / RING_STAGES) - 1u) & 1u)) {
                    atomicOr(&S.error, 4u);  // consumers will time out on the stage as well and report it
                    break;
                }
                issue(tt);
                if (tt == release_at) grid_launch_dependents();
            }
        }
        return;
    }

    // ---- mask / penalty side tables
    float pre_x[2] = {0.0f, 0.0f};                       // logits of this thread's first two history ids ...
    uint32_t pre_slot[2] = {EMPTY_KEY, EMPTY_KEY};       // ... and their table slots, where this thread created them
    if (BITS) {
        // the first 512 history ids are fetched while the tables are cleared
        const uint32_t* hist = P.history + (size_t)b * P.hist_stride;
        uint32_t pre_id[2] = {0u, 0u};
        if (rc.has_pen) {
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const uint32_t j = (uint32_t)k * THREADS + tid;
                if (j < rc.hlen) pre_id[k] = __ldg(&hist[j]);
            }
            // ... and so are their logits: the scattered loads travel while the tables are cleared and
            // filled, instead of costing a trip to memory of their own afterwards
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const uint32_t j = (uint32_t)k * THREADS + tid;
                if (j < rc.hlen && pre_id[k] >= gid0 && pre_id[k] - gid0 < ncols) pre_x[k] = load_logit(row + (pre_id[k] - P.col_offset));
            }
        }
        for (uint32_t w = tid; w < P.bitmap_words; w += THREADS) bitmap[w] = 0u;
        for (uint32_t i = tid; i < P.hash_slots; i += THREADS) {
            hkeys[i] = EMPTY_KEY;
            hcnt[i] = 0u;
        }
        cta_sync();
        if (rc.has_pen) {
            auto note = [&](uint32_t id) -> uint32_t {  // the table slot, if this occurrence of the id created it
                uint32_t created = EMPTY_KEY;
                if (id >= gid0 && id - gid0 < ncols) {  // ids outside the vocabulary are skipped (generate.rs:345)
                    created = hash_insert_owner(hkeys, hcnt, P.hash_slots, id);
                    const uint32_t j2 = id - gid0 + lead;
                    if (IN_BOUNDS(j2 >> 5, P.bitmap_words)) atomicOr(&bitmap[j2 >> 5], 1u << (j2 & 31u));
                }
                return created;
            };
#pragma unroll
            for (int k = 0; k < 2; ++k)
                if ((uint32_t)k * THREADS + tid < rc.hlen) pre_slot[k] = note(pre_id[k]);
            for (uint32_t j = 2u * THREADS + tid; j < rc.hlen; j += THREADS) (void)note(__ldg(&hist[j]));
        }
        if (P.allowed_bits) {
            // bit jb of bitmap word w stands for global id gid0 - lead + 32*w + jb
            const uint32_t nwords_mask = (P.allowed_len + 31u) >> 5;
            for (uint32_t w = tid; w * 32u < ncols + lead; w += THREADS) {
                const long long g0 = (long long)gid0 - (long long)lead + 32ll * (long long)w;
                const long long q0 = g0 >> 5;  // floor
                const uint32_t r0 = (uint32_t)(g0 & 31ll);
                const uint32_t lo = (q0 >= 0 && q0 < (long long)nwords_mask) ? __ldg(&P.allowed_bits[q0]) : 0xffffffffu;
                const uint32_t hi = (q0 + 1 >= 0 && q0 + 1 < (long long)nwords_mask) ? __ldg(&P.allowed_bits[q0 + 1]) : 0xffffffffu;
                uint32_t blocked = ~__funnelshift_r(lo, hi, r0);
                if (blocked) {
                    uint32_t valid = 0u;  // bits that are real columns, inside the mask, and not EOS
                    for (uint32_t jb = 0; jb < 32u; ++jb) {
                        const long long g = g0 + (long long)jb;
                        const uint32_t j2 = w * 32u + jb;
                        if (j2 >= lead && j2 < lead + ncols && g >= 0 && g < (long long)P.allowed_len && (uint32_t)g != P.eos_id)
                            valid |= 1u << jb;
                    }
                    blocked &= valid;
                    if (blocked && IN_BOUNDS(w, P.bitmap_words)) atomicOr(&bitmap[w], blocked);
                }
            }
        }
        cta_sync();
    }

    uint32_t end = 0u;  // highest candidate slot handed out, as seen by this warp
    float tmax = neg_inf();  // largest value of the edited row this thread has seen
    PHASE(1);
    if (fetch_u) {  // read by thread 0 after several more barriers
        S.u_pre = P.uniforms ? u_given : u24_to_f32(splitmix_output(u_seed, u_done + 1ull));  // rng.rs:31-34
        S.u_pre_valid = 1u;
    }

    // ---- ids with a penalty: the stream never edits values. Every distinct history id of this
    //      CTA's columns is read once here, masked and penalised; the value replaces the id's count
    //      in the table and becomes a candidate after the sweep, if it can still matter then. The
    //      stream skips all flagged ids (penalised or blocked by the mask).
    if (BITS && rc.has_pen && rc.hlen <= 2u * (uint32_t)THREADS) {
        // every id's first occurrence was inserted by the thread that already holds its logit
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            if (pre_slot[k] != EMPTY_KEY) {
                float x = pre_x[k];
                if (id_blocked(P, hkeys[pre_slot[k]])) x = neg_inf();
                x = penalize(x, rc.pen, hcnt[pre_slot[k]]);
                tmax = fmaxf(tmax, x);
                hcnt[pre_slot[k]] = __float_as_uint(x);  // only this thread touches the slot
            }
        }
    } else if (BITS) {
        // four table slots per thread and round, so that the scattered loads of a round are in flight together
        for (uint32_t base = 0; base < P.hash_slots; base += 4u * THREADS) {
            uint32_t id[4], cnt[4];
            float x[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t slot = base + (uint32_t)k * THREADS + tid;
                id[k] = slot < P.hash_slots ? hkeys[slot] : EMPTY_KEY;
                cnt[k] = slot < P.hash_slots ? hcnt[slot] : 0u;
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                x[k] = __uint_as_float(0x7fc00000u);
                if (id[k] != EMPTY_KEY) x[k] = load_logit(row + (id[k] - P.col_offset));
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (id[k] != EMPTY_KEY) {
                    if (id_blocked(P, id[k])) x[k] = neg_inf();
                    x[k] = penalize(x[k], rc.pen, cnt[k]);
                    tmax = fmaxf(tmax, x[k]);
                    hcnt[base + (uint32_t)k * THREADS + tid] = __float_as_uint(x[k]);  // only this thread touches the slot
                }
            }
        }
    }

    // ---- leading / trailing elements that are not part of a whole aligned vector (warp 0, one per lane)
    float ht_x = __uint_as_float(0x7fc00000u);
    uint32_t ht_rel = 0u;
    if (warp == 0) {
        bool valid = false;
        if (lane < head) {
            ht_rel = lane;
            valid = true;
        } else if (lane >= 16u && lane - 16u < ntail) {
            ht_rel = tail0 + (lane - 16u);
            valid = true;
        }
        if (valid) {
            ht_x = load_logit(row + c0 + ht_rel);
            if (BITS) {
                const uint32_t j2 = ht_rel + lead;
                if ((bitmap[j2 >> 5] >> (j2 & 31u)) & 1u) ht_x = __uint_as_float(0x7fc00000u);  // handled above / blocked
            }
            tmax = fmaxf(tmax, ht_x);
        }
    }

    // ---- the stream: one sweep without CTA barriers (after the first stage) that only takes maxima
    //      and flags. Every lane takes the maximum of each of its 16-byte vectors (packed bf16
    //      arithmetic for bf16 rows); one ballot word per warp step (32 vectors, 512 bytes) records
    //      which vectors reach the running threshold - a superset of those that reach the final one,
    //      because the threshold only rises. Afterwards only the flagged vectors (a few per cent of
    //      the row) are read again, from L2, against the final threshold.
    //      Window rows: threshold = running maximum - 17.5 (exact once the sweep has seen the row).
    //      Exact-selection rows: a running lower bound of the k-th largest value. The lanes' elements
    //      are disjoint, so each lane's m best vector maxima are m distinct elements of the edited row:
    //        k <= 256 (m = 1): the r-th largest lane maximum of a warp has >= r elements at or above
    //          it, and the minimum over the warps of those (r = ceil(k/8)) has >= k;
    //        k  > 256 (m = ceil(k/256) <= 8, kept sorted in shared memory): the minimum over all
    //          lanes of the lane's m-th best has >= 256*m >= k elements at or above it.
    //      Lane values only rise, so a warp combines its fresh value with whatever the other warps
    //      published last: no barrier. The bound is refreshed at stages 0-4, 6, 8, 12, 16, ... (the
    //      gain of a refresh falls off as 1/stage).
    bool wait_failed = false;
    const bool sweep_k = !rc.windowed;
    const uint32_t m_lane = sweep_k ? (rc.k_eff + (uint32_t)THREADS - 1u) / (uint32_t)THREADS : 1u;  // 1..8
    uint32_t tau_k = LOWEST;  // this warp's view of the running lower bound (ordered key, pre-temperature domain)
    // The bound is a pre-temperature value, the reference ranks by x / T (generate.rs:357-367): with T != 1
    // neighbouring floats can round to the same quotient, and one of them with a lower index then comes
    // before the bound's own element. Filters therefore use the bound lowered by four floats (no more
    // than two or three values share a quotient); the exact selection afterwards works on the quotients.
    const uint32_t tau_slack = (T == 1.0f) ? 0u : 4u;
    auto lowered = [&](uint32_t key) { return key > LOWEST + tau_slack ? key - tau_slack : LOWEST; };
    // Rank cuts above 64 on rows this CTA holds whole: the lanes' maxima bound the k-th largest value only
    // loosely then (thousands of vectors get flagged), so the threshold is SAMPLED instead - the r-th
    // largest of the 256 threads' maxima over the first stage, r chosen so that about 1.6 k values of the
    // row are expected at or above it - and kept for the whole sweep. Exactness does not rest on the
    // estimate: every value at or above the threshold is captured, so if at least k are, the k largest are
    // among them; a row where fewer are is ordered in full instead (an order that rises along the row). r: with
    // S values in the first stage, r0 = k S / V of the k largest are expected among them, and the r-th
    // largest sampled value has about r (1 - 1/sqrt(r)) V/S ... r (1 + 1/sqrt(r)) V/S row values at or above
    // it: r = (2.5 + sqrt(6.25 + r0))^2 leaves five standard deviations of room above k.
    // MODE 3 (chosen by the launch plan: a scalar rank cut above 64 and at most an eighth of the row, rows
    // not split, tokens wanted): every non-greedy row of the launch is sampled this way.
    const bool sampled = (MODE == 3) && rc.k_eff > 1u;
    float lmin = neg_inf();   // m_lane > 1: the lane's m-th best so far
    if (m_lane > 1u && !sampled)
        for (uint32_t i = 0; i < m_lane; ++i)
            if (IN_BOUNDS(i * THREADS + tid, P.lane_top_words)) lane_top[i * THREADS + tid] = neg_inf();
    // the lane's m best, descending, in lane_top[i*THREADS + tid]; returns the new m-th best
    auto lane_insert = [&](float v) {
        for (uint32_t i = 0; i < m_lane; ++i) {
            const float cur = lane_top[i * THREADS + tid];
            if (v > cur) {
                if (IN_BOUNDS(i * THREADS + tid, P.lane_top_words)) lane_top[i * THREADS + tid] = v;
                v = cur;
            }
        }
        return lane_top[(m_lane - 1u) * THREADS + tid];
    };
    // this warp's share of the bound, from the lanes' current values
    auto warp_bound = [&]() -> uint32_t {
        if (m_lane > 1u) return __reduce_min_sync(FULL_MASK, okey(lmin));
        return warp_rth_largest(okey(tmax), (rc.k_eff + WARPS - 1u) / WARPS, lane);
    };
    for (uint32_t tt = 0; tt < vtiles; ++tt) {
        const uint32_t t = tt;
        const uint32_t stage = tt % RING_STAGES;
        if (!mbar_wait_bounded(&full_bar[stage], (tt / RING_STAGES) & 1u)) wait_failed = true;
        const uint4* sv = reinterpret_cast<const uint4*>(ring + (size_t)stage * STAGE);
        float vm[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t j = u * THREADS + tid;
            const uint32_t v = t * VPS + j;
            float m = __uint_as_float(0x7fc00000u);  // NaN: an absent vector never passes and never raises a maximum
            if (v < nvi && !wait_failed) m = vector_max<ElemT>(sv[j]);
            vm[u] = m;  // of the raw values; NaN elements are ignored by the maxima
            if (!BITS && m_lane == 1u) tmax = fmaxf(tmax, m);
        }
        if ((BITS || m_lane > 1u) && !sampled) {
            // A value of the edited row is wanted: flagged ids (penalised, blocked) must not count.
            // Only a vector that would change the lane's state is looked up in the bitmap (a lane's
            // best values change O(m log n) times over a row); vm[u] stays the raw maximum, which
            // keeps every test against a threshold below a superset test.
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (vm[u] > ((m_lane > 1u) ? lmin : tmax)) {
                    float m = vm[u];
                    if (BITS) {
                        const uint32_t j = u * THREADS + tid;
                        const uint32_t v = t * VPS + j;
                        const uint32_t j2 = head + v * VEC + lead;
                        const uint32_t nib = (bitmap[j2 >> 5] >> (j2 & 31u)) & ((1u << VEC) - 1u);
                        if (nib) {
                            float x[VEC];
                            unpack<ElemT>(sv[j], x);
                            m = neg_inf();
#pragma unroll
                            for (int e = 0; e < VEC; ++e)
                                if (!((nib >> e) & 1u)) m = fmaxf(m, x[e]);
                        }
                    }
                    if (m_lane > 1u) {
                        if (m > lmin) lmin = lane_insert(m);
                    } else {
                        tmax = fmaxf(tmax, m);
                    }
                }
            }
        }
        float tau_run;
        if (!sweep_k) {
            // window rows: the running maximum gives the running threshold
            const uint32_t wk = __reduce_max_sync(FULL_MASK, okey(tmax));
            if (tt == 0) {
                if (lane == 0) atomicMax(&S.max_key, wk);
                cta_sync();
                if (tid == 0) {
                    const float qmax0 = temper(okey_to_float(S.max_key), T);
                    S.tau_key = raw_threshold_key(window_stream_bound(qmax0), T);
                }
                cta_sync();
            } else if (lane == 0 && wk > vol_load(&S.max_key)) {
                // the maximum rose: this warp tightens the shared threshold itself (monotone, so
                // warps that still read the old value only keep a superset)
                const uint32_t prev = atomicMax(&S.max_key, wk);
                const float qmax1 = temper(okey_to_float(max(prev, wk)), T);
                atomicMax(&S.tau_key, raw_threshold_key(window_stream_bound(qmax1), T));
            }
            tau_run = okey_to_float(vol_load(&S.tau_key));
        } else if (sampled) {
            if (tt == 0) {
                const float n_sample = (float)min(nvi * (uint32_t)VEC, VPS * (uint32_t)VEC);
                const float r0 = (float)rc.k_eff * n_sample / (float)max(ncols, 1u);
                const float rr = 2.5f + sqrtf(6.25f + r0);
                const float p_elem = fminf(1.0f, rr * rr / fmaxf(n_sample, 1.0f));
                // a thread's maximum over its U * VEC sampled values reaches the threshold with probability q
                const float q_thread = 1.0f - __powf(1.0f - p_elem, (float)(U * VEC));
                const uint32_t sample_rank = min(250u, max(1u, (uint32_t)(q_thread * (float)THREADS + 0.5f)));
                // the sample_rank-th largest of the threads' first-stage maxima (absent vectors rank last)
                float m0 = neg_inf();
#pragma unroll
                for (int u = 0; u < U; ++u) m0 = fmaxf(m0, vm[u]);
                const uint32_t mine = okey(m0);
                S.hist[0][tid] = mine;
                cta_sync();
                uint32_t above = 0u;
                for (uint32_t j = 0; j < (uint32_t)THREADS; ++j) {
                    const uint32_t o = S.hist[0][j];
                    above += (o > mine || (o == mine && j < tid)) ? 1u : 0u;
                }
                if (above == sample_rank - 1u) S.tau_key = max(mine, LOWEST);
                cta_sync();
                tau_k = S.tau_key;
            }
            tau_run = okey_to_float(lowered(tau_k));
        } else {
            const uint32_t h3 = tt / 3u;
            const bool refresh = tt < 4u || (tt & (tt - 1u)) == 0u || (tt == 3u * h3 && (h3 & (h3 - 1u)) == 0u);
            if (refresh) {
                const uint32_t kth = warp_bound();
                if (lane == 0) *(volatile uint32_t*)&S.wkth[warp] = kth;
                if (tt == 0) cta_sync();  // every warp has published once
                else __syncwarp();
                const uint32_t lo = __reduce_min_sync(FULL_MASK, vol_load(&S.wkth[lane & (WARPS - 1u)]));
                tau_k = max(tau_k, max(lo, LOWEST));
            }
            tau_run = okey_to_float(lowered(tau_k));
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const unsigned gm = __ballot_sync(FULL_MASK, vm[u] >= tau_run);
            if (lane == 0 && IN_BOUNDS((t * U + u) * WARPS + warp, P.groups)) grp_max[(t * U + u) * WARPS + warp] = gm;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);  // this warp is done with the stage
    }
    if (rc.windowed) {
        // covers rows too short for a whole vector: only the leading / trailing elements exist
        const uint32_t wk = __reduce_max_sync(FULL_MASK, okey(tmax));
        if (lane == 0) atomicMax(&S.max_key, wk);
    } else if (!sampled) {
        // every lane's final values go into its warp's bound (a warp still sweeping that reads it early
        // only sees a bound that is valid already)
        const uint32_t kth = warp_bound();
        if (lane == 0) *(volatile uint32_t*)&S.wkth[warp] = kth;
    }
    cta_sync();
    bool window_filtered = false;  // the candidates already are exactly the window
    PHASE(7);
    if (P.penalized_out && P.history) {
        grid_dependency_wait();
        write_penalized<ElemT>(P, b, rc.hlen, gid0, ncols, shard == 0u, BITS && rc.has_pen, hkeys, hcnt);
    }
    {
        // the sweep fixed the threshold: the penalised ids, the leading / trailing elements and the
        // vectors flagged during the sweep (read again, from L2) are tested exactly and appended
        // every thread derives the final threshold itself: from the row's maximum (window rows), or
        // as the minimum of the warps' bounds (a lower bound of the k-th largest value)
        const float qmaxf = temper(okey_to_float(S.max_key), T);
        float tau;
        if (sampled) {
            tau = okey_to_float(lowered(vtiles ? S.tau_key : LOWEST));  // a row too short for one vector was never sampled
        } else if (sweep_k) {
            uint32_t lo = S.wkth[0];
#pragma unroll
            for (int w = 1; w < WARPS; ++w) lo = min(lo, S.wkth[w]);
            tau = okey_to_float(lowered(max(lo, LOWEST)));
        } else {
            tau = okey_to_float(raw_threshold_key(window_stream_bound(qmaxf), T));
        }
        // Exact-selection rows check the buffer after every round (at most ROUND*VEC = 1024 new
        // entries, which the buffer has room for beyond `limit`) and keep the best k when it fills;
        // `tau` then rises to the k-th value, in every thread alike. Window rows that overflow are
        // ordered in full instead.
        bool can_overflow = true;  // set below from what is still to come: most rows can skip every check
        auto settle = [&]() {
            if (!sweep_k || !can_overflow) return;
            const int over = cta_sync_or(vol_load(&S.count) > P.limit ? 1 : 0);
            if (!over) return;
            uint32_t n2 = min(S.count, P.ccap);
            cta_sync();
            if (n2 > rc.k_eff) {
                n2 = keep_top_k(n2, rc.k_eff, S, cand_q, cand_i);
                if (tid == 0) S.count = n2;
                cta_sync();
                tau = fmaxf(tau, okey_to_float(raw_threshold_key(okey_to_float(S.minkey), T)));
            }
            cta_sync();
        };
        // does a value of the edited row (pre-temperature x, post-temperature q) still matter?
        auto matters = [&](float x, float q) {
            if (sweep_k) return x >= tau;
            return (__fsub_rn(q, qmaxf) >= WINDOW_EXACT) || (q == qmaxf);  // exactly the terms the reference's sums can see
        };
        // (1) penalised ids: their edited values wait in the table (at most half the table is in use)
        can_overflow = P.hash_slots / 2u + 64u > P.ccap;
        if (BITS) {
            for (uint32_t base = 0; base < P.hash_slots; base += THREADS) {
                const uint32_t slot = base + tid;
                const uint32_t id = slot < P.hash_slots ? hkeys[slot] : EMPTY_KEY;
                const bool have = id != EMPTY_KEY;
                const float x = have ? __uint_as_float(hcnt[slot]) : __uint_as_float(0x7fc00000u);
                const float q = temper(x, T);
                warp_append(have && x >= neg_inf() && matters(x, q), q, id, S, cand_q, cand_i, P.ccap, end);
                settle();
            }
        }
        // (2) leading / trailing elements
        if (warp == 0) {
            const float q = temper(ht_x, T);
            warp_append(ht_x >= neg_inf() && matters(ht_x, q), q, gid0 + ht_rel, S, cand_q, cand_i, P.ccap, end);
        }
        // (3) the flagged vectors
        const uint32_t ngroups = (nvi + 31u) / 32u;
        const uint4* gv = reinterpret_cast<const uint4*>(vbase);
        const uint4 nothing = make_uint4(0u, 0u, 0u, 0u);
        uint32_t* vlist = reinterpret_cast<uint32_t*>(scratch);
        const uint32_t VLIST_CAP = P.vlist_cap;
        // list them: one shared-memory atomic per warp step (prefix sums inside the warp)
        for (uint32_t g0 = 0; g0 < ngroups; g0 += THREADS) {
            const uint32_t g = g0 + tid;
            unsigned m = g < ngroups ? grp_max[g] : 0u;
            const uint32_t c = (uint32_t)__popc(m);
            uint32_t incl = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t y = __shfl_up_sync(FULL_MASK, incl, o);
                if (lane >= (unsigned)o) incl += y;
            }
            const uint32_t total = __shfl_sync(FULL_MASK, incl, 31);
            if (total == 0u) continue;
            uint32_t base = 0u;
            if (lane == 31) base = atomicAdd(&S.keep, total);
            base = __shfl_sync(FULL_MASK, base, 31);
            uint32_t at = base + incl - c;
            while (m) {
                const uint32_t bit = (uint32_t)__ffs(m) - 1u;
                m &= m - 1u;
                if (at < VLIST_CAP) vlist[at] = g * 32u + bit;
                ++at;
            }
        }
        cta_sync();
        PHASE(13);
        const uint32_t nq = S.keep;
        // a round of an exact-selection row appends at most 1024 entries: 1024/VEC vectors
        const uint32_t ROUND = sweep_k ? 1024u / (uint32_t)VEC : (uint32_t)THREADS;
        // the rounds take their vectors from the list, or straight from the flag words when the list
        // could not hold them all
        const bool listed = nq <= VLIST_CAP;
        const uint32_t rounds = listed ? (nq + ROUND - 1u) / ROUND : (ngroups + ROUND / 32u - 1u) / (ROUND / 32u);
        // everything appended so far (at most half the table's slots and one warp's worth of leading /
        // trailing elements) plus every element of every flagged vector: if even that fits, the buffer
        // cannot fill up and the final selection sees it all at once
        can_overflow = (uint64_t)(BITS ? P.hash_slots / 2u : 0u) + 32u + (uint64_t)nq * (uint32_t)VEC > (uint64_t)P.ccap;
        // read a flagged vector again (L2) and append the elements that matter; the appends of a
        // warp step share one atomic
        auto examine = [&](bool have, uint32_t v, const uint4& data) {
            float x[VEC];
            uint32_t em = 0u;
            const uint32_t rel0 = head + v * VEC;
            if (have) {
                unpack<ElemT>(data, x);
                uint32_t nib = 0u;
                if (BITS) {
                    const uint32_t j2 = rel0 + lead;
                    nib = (bitmap[j2 >> 5] >> (j2 & 31u)) & ((1u << VEC) - 1u);  // flagged: handled before the stream
                }
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    if (x[e] >= tau && !((nib >> e) & 1u)) {
                        const float q = temper(x[e], T);
                        if (matters(x[e], q)) em |= 1u << e;
                        x[e] = q;
                    }
                }
            }
            const uint32_t c = (uint32_t)__popc(em);
            uint32_t incl = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t y = __shfl_up_sync(FULL_MASK, incl, o);
                if (lane >= (unsigned)o) incl += y;
            }
            const uint32_t total = __shfl_sync(FULL_MASK, incl, 31);
            if (total == 0u) return;
            uint32_t base = 0u;
            if (lane == 31) base = atomicAdd(&S.count, total);
            base = __shfl_sync(FULL_MASK, base, 31);
            uint32_t slot = base + incl - c;
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                if ((em >> e) & 1u) {
                    if (slot < P.ccap) {
                        cand_q[slot] = x[e];
                        cand_i[slot] = gid0 + rel0 + e;
                    } else {
                        S.error = 1u;
                    }
                    ++slot;
                }
            }
        };
        // the vector of round r for this thread; the load of the next round is issued before the current
        // round is examined, so a row pays one trip to L2 (or to memory: the vector may have left L2)
        auto fetch = [&](uint32_t r, uint32_t& v, uint4& d) {
            bool have;
            if (listed) {
                const uint32_t i = r * ROUND + tid;
                v = (r < rounds && tid < ROUND && i < nq) ? vlist[i] : 0xffffffffu;
                have = v < nvi;
            } else {
                const uint32_t wr = ROUND / 32u;  // warps taking part in a round
                const uint32_t g = r * wr + warp;
                const unsigned m = (r < rounds && warp < wr && g < ngroups) ? grp_max[g] : 0u;  // same word for the whole warp
                v = g * 32u + lane;
                have = ((m >> lane) & 1u) && v < nvi;
                if (!have) v = 0xffffffffu;
            }
            d = have ? __ldg(gv + v) : nothing;
        };
        uint32_t v_next;
        uint4 d_next;
        uint32_t r_done = rounds;
        fetch(0u, v_next, d_next);
#pragma unroll 1
        for (uint32_t r = 0; r < rounds; ++r) {
            const uint32_t v = v_next;
            const uint4 d = d_next;
            fetch(r + 1u, v_next, d_next);
            examine(v < nvi, v, d);
            settle();
            // a window that has already outgrown the buffer is ordered in global scratch: stop collecting it
            if (!sweep_k && __any_sync(FULL_MASK, (vol_load(&S.error) & 1u) != 0u)) {
                r_done = r + 1u;
                break;
            }
        }
        if (tid == 0) {
            S.ex_done = r_done;
            S.ex_all = rounds;
        }
        cta_sync();
        window_filtered = rc.windowed && P.split == 1u;
    }
    PHASE(2);
    if (wait_failed) atomicOr(&S.error, 4u);
    cta_sync();

    // every value that passed the exact test was counted, whether or not it still fitted; where the collection
    // stopped early, the count is scaled to the whole list (it only chooses which ordering is tried first)
    uint32_t found_total = S.count;
    if (S.ex_done < S.ex_all) found_total = (uint32_t)min((uint64_t)found_total * S.ex_all / max(S.ex_done, 1u), (uint64_t)ncols);
    uint32_t n = min(S.count, P.ccap);
    bool overflow = (S.error & 3u) != 0u;  // window too large, or an append fell off the buffer
    float qmax = temper(okey_to_float(S.max_key), T);
    if (S.error & 4u) {  // a bulk copy never completed: report, do not guess
        if (tid == 0 && P.device_errors) atomicOr(P.device_errors, 1u);
        overflow = true;
    }

    if (P.split == 1u) {
        const int undecided = finish_row(P, b, rc, n, overflow, qmax, S, cand_q, cand_i, scratch, window_filtered, sampled);
        if (undecided)
            // the window alone is tried first, unless it is most of the row anyway
            full_sort_row(P, b, *reinterpret_cast<FullShared*>(ring), reinterpret_cast<uint32_t*>(ring + 512), hkeys, hcnt,
                          undecided == 1 && rc.windowed && !(S.error & 4u) && qmax > neg_inf() && found_total < ncols / 2u, qmax);
        return;
    }

    // ---- several CTAs share the row: leave this shard's survivors in scratch;
    //      the CTA that arrives last merges them (no CTA ever waits for another)
    grid_dependency_wait();  // the scratch lists and tickets are shared with the previous launch
    bool list_sorted = false;
    if (!rc.windowed) {
        if (n > (uint32_t)THREADS) n = keep_top_k(n, rc.k_eff, S, cand_q, cand_i);
        if (n <= (uint32_t)THREADS) {
            // small enough for the rank sort: ordered (and cut at k) in two barriers; the merging CTA
            // uses the order to leave most of the list behind
            sort_small(n, S, cand_q, cand_i, reinterpret_cast<uint64_t*>(scratch), S.hist[0], nullptr, false);
            n = min(n, rc.k_eff);
            list_sorted = true;
        }
    } else if (!overflow) {
        n = compact_inplace(
            n, [=](float q, uint32_t) { return (__fsub_rn(q, qmax) >= WINDOW_EXACT) || (q == qmax); }, S, cand_q, cand_i);
        if (n > P.sc_stride) overflow = true;
    }
    {
        const size_t at = (size_t)shard * P.sc_rows + b;
        float* sq = P.sc_q + at * P.sc_stride;
        uint32_t* si = P.sc_i + at * P.sc_stride;
        if (!overflow) {
            for (uint32_t i = tid; i < n; i += THREADS) {
                if (!IN_BOUNDS(i, P.sc_stride)) continue;
                __stcg(&sq[i], cand_q[i]);
                __stcg(&si[i], cand_i[i]);
            }
        }
        if (tid == 0) {
            __stcg(&P.sc_cnt[at], overflow ? 0xffffffffu : (n | (list_sorted ? LIST_SORTED : 0u)));
            __stcg(&P.sc_maxkey[at], okey(qmax));
        }
    }
    __threadfence();
    cta_sync();
    if (tid == 0) {
        const uint32_t ticket = atomicAdd(&P.sc_ticket[b], 1u);
        S.last = (ticket == P.split - 1u) ? 1u : 0u;
    }
    cta_sync();
    if (!S.last) return;
    if (tid == 0) P.sc_ticket[b] = 0u;  // re-armed for the next launch on this stream
    __threadfence();
    n = merge_lists(P, b, rc, P.split, S, cand_q, cand_i, overflow, qmax);
    const int undecided = finish_row(P, b, rc, n, overflow, qmax, S, cand_q, cand_i, scratch);
    if (undecided)
        full_sort_row(P, b, *reinterpret_cast<FullShared*>(ring), reinterpret_cast<uint32_t*>(ring + 512), hkeys, hcnt,
                      undecided == 1 && rc.windowed && !(S.error & 4u) && qmax > neg_inf(), qmax);
}

// ---------------------------------------------------------------------------
// The streaming kernel's 32 variants are compiled in four translation units of eight (one per element type
// and with / without the mask and penalty tables), each of which includes this file with
// LLMC_STREAM_ELEM / LLMC_STREAM_BITS / LLMC_STREAM_TAG defined and exports two host functions:
// configure_stream_<tag> and launch_stream_<tag>. The units compile side by side, and every build gives the
// same binary (nvcc's own splitting of one unit does not: its output, and its speed, varied from build to build).
#ifdef LLMC_STREAM_ELEM
template <typename ElemT, bool BITS, int MODE, int U>
static cudaError_t configure_one(int v) {
    cudaError_t e = cudaFuncSetAttribute(stream_select_kernel<ElemT, BITS, MODE, U>, cudaFuncAttributeMaxDynamicSharedMemorySize, v);
    if (e != cudaSuccess) return e;
    // four CTAs of ~55 KB each only fit when the SM's L1/shared split favours shared memory
    return cudaFuncSetAttribute(stream_select_kernel<ElemT, BITS, MODE, U>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                (int)cudaSharedmemCarveoutMaxShared);
}

template <typename ElemT, bool BITS>
static cudaError_t configure_stream(int v) {
    cudaError_t e;
    if ((e = configure_one<ElemT, BITS, 0, 3>(v)) != cudaSuccess) return e;
    if ((e = configure_one<ElemT, BITS, 1, 3>(v)) != cudaSuccess) return e;
    if ((e = configure_one<ElemT, BITS, 2, 3>(v)) != cudaSuccess) return e;
    if ((e = configure_one<ElemT, BITS, 3, 3>(v)) != cudaSuccess) return e;
    if ((e = configure_one<ElemT, BITS, 0, 4>(v)) != cudaSuccess) return e;
    if ((e = configure_one<ElemT, BITS, 1, 4>(v)) != cudaSuccess) return e;
    if ((e = configure_one<ElemT, BITS, 2, 4>(v)) != cudaSuccess) return e;
    return configure_one<ElemT, BITS, 3, 4>(v);
}

template <typename ElemT, bool BITS, int MODE, int U>
static cudaError_t launch_stream_t(const KParams& P, const LaunchPlan& plan, cudaStream_t stream, bool overlap) {
    auto kern = stream_select_kernel<ElemT, BITS, MODE, U>;
    dim3 grid(plan.split, P.batch, 1);
    if (!overlap) {
        kern<<<grid, STREAM_THREADS, plan.smem, stream>>>(P);
        return cudaGetLastError();
    }
    // programmatic dependent launch: the grid may start while the previous kernel of the stream is
    // still running, if that kernel allows it (this kernel does, at its first instruction); it reads
    // only its inputs until its dependency wait, which returns once the previous grid has finished
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(STREAM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = plan.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, P);
}

template <typename ElemT, bool BITS, int MODE>
static cudaError_t launch_stream_u(const KParams& P, const LaunchPlan& plan, cudaStream_t stream, bool overlap) {
    if (plan.stage_u == 4u) return launch_stream_t<ElemT, BITS, MODE, 4>(P, plan, stream, overlap);
    return launch_stream_t<ElemT, BITS, MODE, 3>(P, plan, stream, overlap);
}

template <typename ElemT, bool BITS>
static cudaError_t launch_stream_m(const KParams& P, const LaunchPlan& plan, cudaStream_t stream, bool overlap) {
    if (plan.mode == 1) return launch_stream_u<ElemT, BITS, 1>(P, plan, stream, overlap);
    if (plan.mode == 2) return launch_stream_u<ElemT, BITS, 2>(P, plan, stream, overlap);
    if (plan.mode == 3) return launch_stream_u<ElemT, BITS, 3>(P, plan, stream, overlap);
    return launch_stream_u<ElemT, BITS, 0>(P, plan, stream, overlap);
}

#define LLMC_CAT2(a, b) a##b
#define LLMC_CAT(a, b) LLMC_CAT2(a, b)
cudaError_t LLMC_CAT(configure_stream_, LLMC_STREAM_TAG)(int max_dyn_smem) {
    return configure_stream<LLMC_STREAM_ELEM, LLMC_STREAM_BITS>(max_dyn_smem);
}
cudaError_t LLMC_CAT(launch_stream_, LLMC_STREAM_TAG)(const KParams& P, const LaunchPlan& plan, cudaStream_t stream, bool overlap) {
    return launch_stream_m<LLMC_STREAM_ELEM, LLMC_STREAM_BITS>(P, plan, stream, overlap);
}
#endif  // LLMC_STREAM_ELEM

#ifndef LLMC_KERNELS_ONLY  // a translation unit that only wants the streaming kernel's variants stops here
// Ordered tail over gathered candidate lists: one CTA per row.
__global__ void __launch_bounds__(THREADS) merge_draw_kernel(const __grid_constant__ KParams P) {
    extern __shared__ __align__(128) unsigned char dyn[];
    __shared__ Shared S;
    unsigned char* scratch = dyn;  // epilogue scratch where the streaming kernel has its ring
    float* cand_q = reinterpret_cast<float*>(dyn + RING_STAGES * STAGE_BYTES);
    uint32_t* cand_i = reinterpret_cast<uint32_t*>(cand_q + P.ccap);
    const uint32_t b = blockIdx.x;
    if (threadIdx.x == 0) {
        resolve_row(P, b, S.rc);
        S.error = 0u;
        S.u_pre_valid = 0u;
        S.sortmax = 0u;
    }
    cta_sync();
    const RowCfg rc = S.rc;
    if (rc.invalid) {
        if (threadIdx.x == 0) {
            P.tokens[b] = 0u;
            if (P.row_flags) P.row_flags[b] = LLM_CUDA_ROW_INVALID;
            if (P.kept_count) P.kept_count[b] = 0u;
        }
        return;
    }
    bool overflow;
    float qmax;
    // lists gathered from other GPUs were written in order by finish_row there; the fused LM head's are not ordered
    const uint32_t n = merge_lists(P, b, rc, P.split, S, cand_q, cand_i, overflow, qmax, /*all_sorted=*/P.sc_sorted != 0u);
    // the logits of a gathered row live on other GPUs: a row its lists cannot decide is reported
    if (finish_row(P, b, rc, n, overflow, qmax, S, cand_q, cand_i, scratch) && threadIdx.x == 0) report_unresolved(P, b);
}

// ---------------------------------------------------------------------------
// Generator::step's bookkeeping (generate.rs:157-182), one thread per row.
__global__ void advance_rows_kernel(uint32_t batch, const uint32_t* tokens, const uint32_t* row_flags, uint32_t* history,
                                    uint32_t history_stride, uint32_t window, uint32_t* history_len, uint32_t* history_pos,
                                    uint64_t* draw_index, uint8_t* finished, uint32_t eos_id) {
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= batch) return;
    if (finished && finished[r]) return;
    if (draw_index && row_flags && (row_flags[r] & LLM_CUDA_ROW_DRAW_CONSUMED)) draw_index[r] += 1ull;
    const uint32_t tok = tokens[r];
    if (tok == eos_id) {  // step() returns None and does not advance
        if (finished) finished[r] = 1;
        return;
    }
    if (history && history_stride) {
        const uint32_t cap = min(window, history_stride);
        if (cap == 0u) return;
        const uint32_t len = history_len[r];
        if (len < cap) {  // still filling: keep chronological order in [0, len)
            history[(size_t)r * history_stride + len] = tok;
            history_len[r] = len + 1u;
            history_pos[r] = (len + 1u) % cap;
        } else {  // ring: overwrite the oldest entry (the penalty does not depend on the order)
            const uint32_t pos = history_pos[r] % cap;
            history[(size_t)r * history_stride + pos] = tok;
            history_pos[r] = (pos + 1u) % cap;
        }
    }
}

__global__ void pack_allowed_kernel(const uint8_t* allowed, uint32_t n, uint32_t* bits) {
    const uint32_t w = blockIdx.x * blockDim.x + threadIdx.x;
    if (w * 32u >= n) return;
    uint32_t word = 0u;
    for (uint32_t j = 0; j < 32u; ++j) {
        const uint32_t id = w * 32u + j;
        if (id >= n || allowed[id]) word |= 1u << j;  // ids past the slice count as allowed
    }
    bits[w] = word;
}

// ---------------------------------------------------------------------------
// host side: launch plans
#ifdef LLMC_DEV
static int g_dev_stage_u = 0;
#endif
static uint32_t pow2_ceil(uint32_t x) {
    uint32_t p = 1u;
    while (p < x) p <<= 1;
    return p;
}

int plan_launch(const DeviceInfo& dev, const KParams& base, bool top_k_known, uint32_t top_k_hint, uint32_t max_top_k,
                uint32_t max_history, uint32_t requested_split, uint32_t max_lists, LaunchPlan* plan) {
    const uint32_t tile = STAGE_BYTES / (base.dtype == LLM_CUDA_DTYPE_BF16 ? 2u : 4u);  // logits per ring stage
    // candidate capacity
    uint32_t kcap;
    bool window_only = false;  // every non-greedy row is known to run in window mode
    if (top_k_known) {
        const uint32_t k = (top_k_hint == 0u || top_k_hint >= base.vocab_global) ? base.vocab_global : top_k_hint;
        if (k <= MAX_KCAP) {
            kcap = pow2_ceil(k < 64u ? 64u : k);
        } else {
            kcap = 64u;  // only greedy rows (k = 1) are selected exactly in such a launch
            window_only = true;
        }
    } else {
        kcap = pow2_ceil(max_top_k < 64u ? 64u : (max_top_k > MAX_KCAP ? MAX_KCAP : max_top_k));
    }
    plan->kcap = kcap;
    // 1: every row is known to run in window mode (scalar temperature > 0, so no greedy row either);
    // 2: no row can; 0: decided per row in the kernel
    const bool may_be_greedy = base.t_rows != nullptr || base.temperature <= 0.0f;
    plan->mode = (window_only && !may_be_greedy) ? 1 : ((top_k_known && !window_only) ? 2 : 0);
    plan->sample_threshold = false;  // decided below, once the split is known
    if (window_only) {
        // an append that falls off the buffer sends the row to the full ordering
        plan->ccap = WINDOW_CAP;
        plan->limit = WINDOW_CAP / 2u;
    } else {
        // candidates are appended after the sweep in rounds of at most 1024 entries, each followed by a
        // check of the buffer against the compaction trigger
        plan->limit = 2u * kcap > 1024u ? 2u * kcap : 1024u;
        plan->ccap = plan->limit + 32u + 1024u;
        if (plan->ccap < WINDOW_CAP && !top_k_known) plan->ccap = WINDOW_CAP;  // rows with top_k 0 may be mixed in
    }
    plan->bits = (base.allowed_bits != nullptr) || (base.history != nullptr && (base.r_rows != nullptr || base.penalty != 1.0f) &&
                                                    (base.hist_len_rows != nullptr || base.hist_len > 0u));
    // split: fill the machine when the batch is small, keep shards long enough to stream
    uint32_t split = requested_split;
    if (split == 0u && window_only) {
        // a window is measured from the row's maximum; a CTA that sees only part of the row
        // would measure it from its own, lower maximum and keep far too much
        split = 1u;
    }
    // a scalar rank cut above 64 is cheapest with the threshold sampled from the row's first stage (kernel MODE 3),
    // which needs the row in one CTA: with a few dozen rows or more that beats filling the machine with shards
    const bool sampled_fits = plan->mode == 2 && base.out_q == nullptr && base.full_keys_wanted && top_k_hint > 64u &&
                              (uint64_t)top_k_hint * 8u <= base.vocab;
    if (split == 0u && sampled_fits && (uint64_t)base.batch * 8u >= dev.sm_count) split = 1u;
    if (split == 0u) {
        const uint32_t target = 4u * dev.sm_count;
        split = target / (base.batch ? base.batch : 1u);
        const uint32_t by_len = base.vocab / (4u * tile);
        if (split > by_len) split = by_len;
    }
    if (split < 1u) split = 1u;
    if (split > 64u) split = 64u;
    if ((uint64_t)split * base.batch > max_lists) split = max_lists / base.batch;
    if (split < 1u) split = 1u;
    uint32_t shard_cols = (base.vocab + split - 1u) / split;
    shard_cols = (shard_cols + 63u) & ~63u;
    if (shard_cols == 0u) shard_cols = 64u;
    split = (base.vocab + shard_cols - 1u) / shard_cols;
    if (split < 1u) split = 1u;
    plan->split = split;
    plan->shard_cols = shard_cols;
    // exact-selection launches with a scalar rank cut above 64 (and at most an eighth of the row) whose rows are
    // not split and that draw tokens: the threshold is sampled from the first stage (kernel MODE 3)
    if (sampled_fits && split == 1u) {
        plan->mode = 3;
        plan->sample_threshold = true;
    }
    if (plan->bits) {
        plan->bitmap_words = (shard_cols + 8u + 31u) / 32u + 1u;
        // sized for this launch's longest history (the handle's maximum when rows bring their own lengths)
        uint32_t hmax = max_history ? max_history : 1u;
        if (base.history != nullptr) {
            const uint32_t hl = base.hist_len_rows ? base.hist_stride : base.hist_len;
            if (hl > 0u && hl < hmax) hmax = hl;
        }
        plan->hash_slots = pow2_ceil(2u * hmax);
        if (plan->hash_slots < 64u) plan->hash_slots = 64u;
    } else {
        plan->bitmap_words = 0u;
        plan->hash_slots = 0u;
    }
    // one flag word per group of 32 vectors of the shard
    const uint32_t vec_elems = 16u / (base.dtype == LLM_CUDA_DTYPE_BF16 ? 2u : 4u);
    plan->groups = (shard_cols / vec_elems + 31u) / 32u + WARPS * 4u;  // + one stage of slack at the larger stage size
    // rank cuts above 256 keep ceil(k/256) best values per lane
    plan->lane_top_words = (!window_only && kcap > (uint32_t)THREADS) ? kcap : 0u;
    // The candidate buffer and the epilogue scratch (sort keys + probabilities) are used only after the
    // sweep: when both fit into the ring they live there, which is what lets four CTAs share an SM.
    const size_t cand_bytes = (size_t)plan->ccap * 8u;
    const size_t tables_bytes = (size_t)plan->bitmap_words * 4u + (size_t)plan->hash_slots * 8u +
                                (size_t)plan->lane_top_words * 4u + (size_t)plan->groups * 4u;
    // Stage size: 16 KB stages (48 KB in flight per CTA) unless that costs a resident CTA; an SM has
    // 228 KB of shared memory, and each CTA takes 1 KB of it plus the kernel's static share.
    auto layout = [&](uint32_t u, size_t* smem, bool* aliased) {
        const size_t ring_bytes = (size_t)RING_STAGES * u * THREADS * 16u;
        *aliased = cand_bytes + EPILOGUE_SCRATCH <= ring_bytes;
        *smem = ring_bytes + tables_bytes + (*aliased ? 0u : cand_bytes);
    };
    auto resident = [&](size_t smem) {
        const size_t per_cta = smem + 1024u + 2304u;
        const size_t n = 233472u / per_cta;
        return n > 4u ? (size_t)4u : n;
    };
    size_t smem3, smem4;
    bool alias3, alias4;
    layout(3u, &smem3, &alias3);
    layout(4u, &smem4, &alias4);
    bool big = smem4 <= dev.max_dyn_smem && resident(smem4) >= resident(smem3);
#ifdef LLMC_DEV
    if (g_dev_stage_u == 3) big = false;
    if (g_dev_stage_u == 4 && smem4 <= dev.max_dyn_smem) big = true;
#endif
    plan->stage_u = big ? 4u : 3u;
    const bool aliased = big ? alias4 : alias3;
    const size_t ring_bytes = (size_t)RING_STAGES * plan->stage_u * THREADS * 16u;
    const size_t smem_total = ring_bytes + tables_bytes + (aliased ? 0u : cand_bytes);
    if (smem_total > dev.max_dyn_smem) return -1;
    if (aliased) {
        size_t cb = cand_bytes;
        // window launches: twice the candidates where the ring has the room anyway (16 KB stages), so that rows
        // with 2049..4096 significant values are still ordered in shared memory
        if (window_only && (size_t)WINDOW_CAP_WIDE * 8u + EPILOGUE_SCRATCH <= ring_bytes) {
            plan->ccap = WINDOW_CAP_WIDE;
            cb = (size_t)WINDOW_CAP_WIDE * 8u;
        }
        plan->cand_off = 0u;
        plan->scratch_off = (uint32_t)cb;
        plan->tables_off = (uint32_t)ring_bytes;
        plan->vlist_cap = (uint32_t)((ring_bytes - cb) / 4u);
    } else {
        plan->cand_off = (uint32_t)ring_bytes;
        plan->scratch_off = 0u;
        plan->tables_off = (uint32_t)(ring_bytes + cand_bytes);
        plan->vlist_cap = (uint32_t)(ring_bytes / 4u);
    }
    plan->smem = smem_total;
    return 0;
}

void apply_plan(const LaunchPlan& plan, KParams* P) {
    P->split = plan.split;
    P->shard_cols = plan.shard_cols;
    P->kcap = plan.kcap;
    P->ccap = plan.ccap;
    P->limit = plan.limit;
    P->hash_slots = plan.hash_slots;
    P->bitmap_words = plan.bitmap_words;
    P->groups = plan.groups;
    P->lane_top_words = plan.lane_top_words;
    P->cand_off = plan.cand_off;
    P->scratch_off = plan.scratch_off;
    P->tables_off = plan.tables_off;
    P->vlist_cap = plan.vlist_cap;
}

#ifdef LLMC_DEV
void dev_override(int key, int value) {
    if (key == 0) g_dev_stage_u = value;
}
#endif

cudaError_t configure_kernels(size_t max_dyn_smem) {
    const int v = (int)max_dyn_smem;
    cudaError_t e;
    if ((e = configure_stream_f32(v)) != cudaSuccess) return e;
    if ((e = configure_stream_f32_tables(v)) != cudaSuccess) return e;
    if ((e = configure_stream_bf16(v)) != cudaSuccess) return e;
    if ((e = configure_stream_bf16_tables(v)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(merge_draw_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, v)) != cudaSuccess) return e;
    return cudaSuccess;
}

cudaError_t launch_stream_select(const KParams& P, const LaunchPlan& plan, cudaStream_t stream, bool overlap) {
    if (P.dtype == LLM_CUDA_DTYPE_BF16)
        return plan.bits ? launch_stream_bf16_tables(P, plan, stream, overlap) : launch_stream_bf16(P, plan, stream, overlap);
    return plan.bits ? launch_stream_f32_tables(P, plan, stream, overlap) : launch_stream_f32(P, plan, stream, overlap);
}

cudaError_t launch_merge_draw(const KParams& P, const LaunchPlan& plan, cudaStream_t stream) {
    const size_t smem = (size_t)RING_STAGES * STAGE_BYTES + (size_t)plan.ccap * 8u;
    merge_draw_kernel<<<P.batch, THREADS, smem, stream>>>(P);
    return cudaGetLastError();
}

cudaError_t launch_advance_rows(uint32_t batch, const uint32_t* tokens, const uint32_t* row_flags, uint32_t* history,
                                uint32_t history_stride, uint32_t window, uint32_t* history_len, uint32_t* history_pos,
                                uint64_t* draw_index, uint8_t* finished, uint32_t eos_id, cudaStream_t stream) {
    if (batch == 0u) return cudaSuccess;
    advance_rows_kernel<<<(batch + 127u) / 128u, 128, 0, stream>>>(batch, tokens, row_flags, history, history_stride, window,
                                                                  history_len, history_pos, draw_index, finished, eos_id);
    return cudaGetLastError();
}

cudaError_t launch_pack_allowed(const uint8_t* allowed_dev, uint32_t n, uint32_t* bits, cudaStream_t stream) {
    const uint32_t words = (n + 31u) / 32u;
    if (words == 0u) return cudaSuccess;
    pack_allowed_kernel<<<(words + 127u) / 128u, 128, 0, stream>>>(allowed_dev, n, bits);
    return cudaGetLastError();
}

#endif  // LLMC_KERNELS_ONLY

}  // namespace llmc
