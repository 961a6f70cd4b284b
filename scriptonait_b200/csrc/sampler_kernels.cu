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
// full_sort_kernel       literal full ordering of a row, for the rare rows
//                        whose kept set or draw reaches past the window.
// advance_rows_kernel    decode-loop glue (history ring, EOS, draw counter).
// pack_allowed_kernel    bool-per-id -> bit mask.
//
// Reference: crates/llm-core/src/generate.rs:325-420 (sample_with),
// :157-182 (Generator::step / recent_tokens).
#include "sampler_kernels.h"

#include <stdio.h>

#include "sampler_device.cuh"

namespace llmc {

template <typename ElemT>
struct Traits;
template <>
struct Traits<float> {
    static constexpr int VEC = 4;  // elements per 16-byte load
    static constexpr int U = 4;    // 16-byte loads per thread per tile
    static constexpr uint32_t NAN4 = 0x7fc00000u;
};
template <>
struct Traits<uint16_t> {
    static constexpr int VEC = 8;
    static constexpr int U = 2;
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

__device__ __forceinline__ uint32_t vol_load(const uint32_t* p) { return *(const volatile uint32_t*)p; }

__device__ __forceinline__ void push_full(const KParams& P, uint32_t b) {
    const uint32_t pos = atomicAdd(P.full_count, 1u);
    P.full_list[pos] = b;
}

// Streaming threshold (pre-temperature ordered key) of window mode for a given maximum.
__device__ __forceinline__ float window_stream_bound(float qmax) {
    return __fsub_rn(__fsub_rn(qmax, WINDOW_STREAM), __fmul_rn(fabsf(qmax), 2.384185791015625e-07f));
}
__device__ __forceinline__ float temper(float x, float T) { return (T == 1.0f) ? x : __fdiv_rn(x, T); }  // generate.rs:357-359

// Mask and penalty for one element whose bitmap bit is set (generate.rs:333-352).
__device__ __forceinline__ float edit_value(const KParams& P, const RowCfg& rc, float x, uint32_t gid, const uint32_t* hkeys,
                                            const uint32_t* hcnt) {
    if (id_blocked(P, gid)) x = neg_inf();
    if (rc.has_pen) x = penalize(x, rc.pen, hash_count(hkeys, hcnt, P.hash_slots, gid));
    return x;
}

// After all candidates of a row are in cand[0..n): final selection, ordering
// and either the ordered tail (token out) or the candidate list out.
__device__ void finish_row(const KParams& P, uint32_t b, const RowCfg& rc, uint32_t n, bool overflow, float qmax, Shared& S,
                           float* cand_q, uint32_t* cand_i) {
    const uint32_t limit = 2u * P.kcap;
    if (!rc.windowed) {
        n = keep_top_k(n, rc.k_eff, S, cand_q, cand_i);
    } else if (!overflow) {
        // exact window: exactly the terms the reference's f32 sums can see
        n = compact_inplace(
            n, [=](float q, uint32_t) { return (__fsub_rn(q, qmax) >= WINDOW_EXACT) || (q == qmax); }, S, cand_q, cand_i);
        if (n > limit) overflow = true;
    }
    if (overflow) {
        if (threadIdx.x == 0) push_full(P, b);
        return;
    }
    sort_candidates(n, cand_q, cand_i);
    const uint32_t n_use = min(n, rc.k_eff);
    const bool truncated = rc.windowed && (n_use < rc.k_eff);
    if (P.out_q) {  // vocabulary sharding, step 1: the ordered list is the result
        for (uint32_t i = threadIdx.x; i < min(n_use, P.out_stride); i += THREADS) {
            P.out_q[(size_t)b * P.out_stride + i] = cand_q[i];
            P.out_i[(size_t)b * P.out_stride + i] = cand_i[i];
        }
        if (threadIdx.x == 0) P.out_cnt[b] = min(n_use, P.out_stride);
        return;
    }
    float* probs = cand_q + limit;
    if (rc.greedy || n_use == 0u) {
        if (threadIdx.x == 0) {
            S.token = n_use ? cand_i[0] : 0u;  // ops/loss.rs:6-16: first index of the maximum; 0 when nothing compares greater than -inf
            if (n_use && cand_q[0] == neg_inf()) S.token = 0u;
            S.out_flags = rc.greedy ? LLM_CUDA_ROW_GREEDY : LLM_CUDA_ROW_DEGENERATE;
            S.kept_n = 0u;
            S.f_sum = S.f_total = S.f_u = S.f_thr = S.f_r = 0.f;
        }
        __syncthreads();
        write_row_outputs(P, b, 0u, S, n_use ? cand_q[0] : 0.f, cand_i, probs, 0u);
        return;
    }
    ordered_tail(P, b, rc, n_use, truncated, rc.k_eff, S, cand_q, cand_i, probs);
    if (S.out_flags & ROW_NEEDS_FULL) {
        if (threadIdx.x == 0) push_full(P, b);
        return;
    }
    write_row_outputs(P, b, rc.windowed ? LLM_CUDA_ROW_WINDOWED : 0u, S, cand_q[0], cand_i, probs, S.keep);
}

// Pulls the candidate lists of `nsh` shards of row b into cand[] (compacting
// whenever the next list would not fit) and returns the count; `overflow` and
// `qmax` as finish_row expects them.
__device__ uint32_t merge_lists(const KParams& P, uint32_t b, const RowCfg& rc, uint32_t nsh, Shared& S, float* cand_q,
                                uint32_t* cand_i, bool& overflow, float& qmax) {
    const uint32_t limit = 2u * P.kcap;
    if (threadIdx.x == 0) {
        S.count = 0u;
        S.max_key = 0x007fffffu;
        S.keep = 0u;  // overflow marker seen
    }
    __syncthreads();
    for (uint32_t s = threadIdx.x; s < nsh; s += THREADS) {
        const size_t at = (size_t)s * P.sc_rows + b;
        if (P.sc_maxkey) atomicMax(&S.max_key, __ldcg(&P.sc_maxkey[at]));
        if (__ldcg(&P.sc_cnt[at]) == 0xffffffffu) S.keep = 1u;
    }
    __syncthreads();
    overflow = S.keep != 0u;
    qmax = okey_to_float(S.max_key);
    const float tq = window_stream_bound(qmax);
    for (uint32_t s = 0; s < nsh && !overflow; ++s) {
        const size_t at = (size_t)s * P.sc_rows + b;
        const uint32_t cnt = min(__ldcg(&P.sc_cnt[at]), P.sc_stride);
        uint32_t n = S.count;
        if (n + cnt > P.ccap) {
            if (!rc.windowed) {
                n = keep_top_k(n, rc.k_eff, S, cand_q, cand_i);
            } else {
                n = compact_inplace(
                    n, [=](float q, uint32_t) { return q >= tq; }, S, cand_q, cand_i);
                if (n > limit) overflow = true;
            }
            if (n + cnt > P.ccap) overflow = true;
        }
        if (overflow) break;
        const float* sq = P.sc_q + at * P.sc_stride;
        const uint32_t* si = P.sc_i + at * P.sc_stride;
        for (uint32_t i = threadIdx.x; i < cnt; i += THREADS) {
            cand_q[n + i] = __ldcg(&sq[i]);
            cand_i[n + i] = __ldcg(&si[i]);
        }
        __syncthreads();
        if (threadIdx.x == 0) S.count = n + cnt;
        __syncthreads();
    }
    return S.count;
}

template <typename ElemT, bool BITS>
__global__ void __launch_bounds__(THREADS) stream_select_kernel(const __grid_constant__ KParams P) {
    constexpr int VEC = Traits<ElemT>::VEC;
    constexpr int U = Traits<ElemT>::U;
    static_assert(THREADS * U * VEC == (int)TILE_ELEMS, "tile geometry");
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ Shared S;
    float* cand_q = reinterpret_cast<float*>(dyn);
    uint32_t* cand_i = reinterpret_cast<uint32_t*>(cand_q + P.ccap);
    uint32_t* bitmap = cand_i + P.ccap;
    uint32_t* hkeys = bitmap + P.bitmap_words;
    uint32_t* hcnt = hkeys + P.hash_slots;

    const uint32_t b = blockIdx.y, shard = blockIdx.x, tid = threadIdx.x;
    const unsigned lane = tid & 31u, warp = tid >> 5;
    const uint32_t LOWEST = 0x007fffffu;  // okey(-inf)
    if (tid == 0) {
        resolve_row(P, b, S.rc);
        S.count = 0u;
        S.tau_key = LOWEST;
        S.max_key = LOWEST;
        S.error = 0u;
        S.last = 0u;
    }
    __syncthreads();
    const RowCfg rc = S.rc;
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
    if (P.force_full) {
        if (shard == 0 && tid == 0) push_full(P, b);
        return;
    }

    // ---- this CTA's columns and their 16-byte alignment
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
    const uint4* vbase = reinterpret_cast<const uint4*>(row + c0 + head);
    const float T = rc.T;
    const uint32_t limit = 2u * P.kcap;  // compaction trigger; ccap - limit = TILE_ELEMS of headroom

    // ---- mask / penalty side tables
    if (BITS) {
        for (uint32_t w = tid; w < P.bitmap_words; w += THREADS) bitmap[w] = 0u;
        for (uint32_t i = tid; i < P.hash_slots; i += THREADS) {
            hkeys[i] = EMPTY_KEY;
            hcnt[i] = 0u;
        }
        __syncthreads();
        if (rc.has_pen) {
            const uint32_t* hist = P.history + (size_t)b * P.hist_stride;
            for (uint32_t j = tid; j < rc.hlen; j += THREADS) {
                const uint32_t id = __ldg(&hist[j]);
                if (id >= gid0 && id - gid0 < ncols) {  // ids outside the vocabulary are skipped (generate.rs:345)
                    hash_insert(hkeys, hcnt, P.hash_slots, id);
                    const uint32_t j2 = id - gid0 + lead;
                    atomicOr(&bitmap[j2 >> 5], 1u << (j2 & 31u));
                }
            }
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
                uint32_t allowed = __funnelshift_r(lo, hi, r0);
                uint32_t blocked = ~allowed;
                uint32_t valid = 0u;  // bits that are real columns, inside the mask, and not EOS
                for (uint32_t jb = 0; jb < 32u; ++jb) {
                    const long long g = g0 + (long long)jb;
                    const uint32_t j2 = w * 32u + jb;
                    if (j2 >= lead && j2 < lead + ncols && g >= 0 && g < (long long)P.allowed_len && (uint32_t)g != P.eos_id)
                        valid |= 1u << jb;
                }
                blocked &= valid;
                if (blocked) atomicOr(&bitmap[w], blocked);
            }
        }
        __syncthreads();
    }

    uint32_t end = 0u;  // highest candidate slot handed out, as seen by this warp
    float tmax = neg_inf();

    // ---- leading / trailing elements that are not part of a whole aligned vector (warp 0)
    if (warp == 0) {
        bool valid = false;
        uint32_t rel = 0u;
        if (lane < head) {
            rel = lane;
            valid = true;
        } else if (lane >= 16u && lane - 16u < ntail) {
            rel = tail0 + (lane - 16u);
            valid = true;
        }
        float x = __uint_as_float(0x7fc00000u);
        if (valid) {
            x = load_logit(row + c0 + rel);
            if (BITS) {
                const uint32_t j2 = rel + lead;
                if ((bitmap[j2 >> 5] >> (j2 & 31u)) & 1u) x = edit_value(P, rc, x, gid0 + rel, hkeys, hcnt);
            }
            tmax = fmaxf(tmax, x);
        }
        warp_append(valid && x >= neg_inf(), temper(x, T), gid0 + rel, S, cand_q, cand_i, P.ccap, end);
    }

    // ---- the stream: tile t = vectors [t*THREADS*U, (t+1)*THREADS*U), prefetched one tile ahead
    const uint32_t ntiles = (nvi + THREADS * U - 1) / (THREADS * U);
    uint4 cur[U], nxt[U];
    auto load_tile = [&](uint4(&dst)[U], uint32_t t) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t v = (t * U + u) * THREADS + tid;
            if (v < nvi) {
                dst[u] = __ldcs(vbase + v);
            } else {
                dst[u] = make_uint4(Traits<ElemT>::NAN4, Traits<ElemT>::NAN4, Traits<ElemT>::NAN4, Traits<ElemT>::NAN4);
            }
        }
    };
    if (ntiles) load_tile(cur, 0);
    uint32_t seen_max_key = LOWEST;
    for (uint32_t t = 0; t <= ntiles; ++t) {
        // iteration t == ntiles only publishes the maximum and settles the buffer
        if (t < ntiles) {
            if (t + 1 < ntiles) load_tile(nxt, t + 1);
            const float tau = okey_to_float(vol_load(&S.tau_key));
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint32_t v = (t * U + u) * THREADS + tid;
                float x[VEC];
                unpack<ElemT>(cur[u], x);
                const uint32_t rel0 = head + v * VEC;  // column (relative to c0) of x[0]
                if (BITS) {
                    if (v < nvi) {
                        const uint32_t j2 = rel0 + lead;  // multiple of VEC: the VEC bits sit in one word
                        uint32_t nib = (bitmap[j2 >> 5] >> (j2 & 31u)) & ((1u << VEC) - 1u);
                        if (nib) {
#pragma unroll
                            for (int e = 0; e < VEC; ++e)
                                if ((nib >> e) & 1u) x[e] = edit_value(P, rc, x[e], gid0 + rel0 + e, hkeys, hcnt);
                        }
                    }
                }
                float vm = x[0];
#pragma unroll
                for (int e = 1; e < VEC; ++e) vm = fmaxf(vm, x[e]);
                tmax = fmaxf(tmax, vm);
                if (__any_sync(FULL_MASK, vm >= tau)) {
#pragma unroll
                    for (int e = 0; e < VEC; ++e)
                        warp_append(x[e] >= tau, temper(x[e], T), gid0 + rel0 + e, S, cand_q, cand_i, P.ccap, end);
                }
            }
        }
        if (rc.windowed) {
            const uint32_t mk = okey(tmax);
            if (mk > seen_max_key) {
                atomicMax(&S.max_key, mk);
                seen_max_key = mk;
            }
        }
        const int over = __syncthreads_or(end > limit);
        if (over) {
            uint32_t n = min(S.count, P.ccap);
            __syncthreads();
            if (!rc.windowed) {
                if (n > rc.k_eff) {
                    n = keep_top_k(n, rc.k_eff, S, cand_q, cand_i);
                    if (tid == 0) {
                        S.count = n;
                        S.tau_key = max(S.tau_key, raw_threshold_key(okey_to_float(S.minkey), T));
                    }
                }
            } else {
                const float qmax = temper(okey_to_float(S.max_key), T);
                const float tq = window_stream_bound(qmax);
                n = compact_inplace(
                    n, [=](float q, uint32_t) { return q >= tq; }, S, cand_q, cand_i);
                if (tid == 0) {
                    if (n > limit) {  // the window does not fit: the full-sort kernel takes the row
                        S.count = 0u;
                        S.tau_key = 0xff800000u;  // okey(+inf)
                        S.error |= 2u;
                    } else {
                        S.count = n;
                        S.tau_key = max(S.tau_key, raw_threshold_key(tq, T));
                    }
                }
            }
            __syncthreads();
            end = S.count;
        } else if (rc.windowed && tid == 0) {
            const float qmax = temper(okey_to_float(S.max_key), T);
            const uint32_t tk = raw_threshold_key(window_stream_bound(qmax), T);
            if (tk > S.tau_key) S.tau_key = tk;
        }
        if (t < ntiles) {
#pragma unroll
            for (int u = 0; u < U; ++u) cur[u] = nxt[u];
        }
    }
    __syncthreads();

    uint32_t n = min(S.count, P.ccap);
    bool overflow = (S.error & 2u) != 0u;
    float qmax = temper(okey_to_float(S.max_key), T);

    if (P.split == 1u) {
        finish_row(P, b, rc, n, overflow, qmax, S, cand_q, cand_i);
        return;
    }

    // ---- several CTAs share the row: leave this shard's survivors in scratch;
    //      the CTA that arrives last merges them (no CTA ever waits for another)
    if (!rc.windowed) {
        n = keep_top_k(n, rc.k_eff, S, cand_q, cand_i);
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
                __stcg(&sq[i], cand_q[i]);
                __stcg(&si[i], cand_i[i]);
            }
        }
        if (tid == 0) {
            __stcg(&P.sc_cnt[at], overflow ? 0xffffffffu : n);
            __stcg(&P.sc_maxkey[at], okey(qmax));
        }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const uint32_t ticket = atomicAdd(&P.sc_ticket[b], 1u);
        S.last = (ticket == P.split - 1u) ? 1u : 0u;
    }
    __syncthreads();
    if (!S.last) return;
    if (tid == 0) P.sc_ticket[b] = 0u;  // re-armed for the next launch on this stream
    __threadfence();
    n = merge_lists(P, b, rc, P.split, S, cand_q, cand_i, overflow, qmax);
    finish_row(P, b, rc, n, overflow, qmax, S, cand_q, cand_i);
}

// Ordered tail over gathered candidate lists: one CTA per row.
__global__ void __launch_bounds__(THREADS) merge_draw_kernel(const __grid_constant__ KParams P) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ Shared S;
    float* cand_q = reinterpret_cast<float*>(dyn);
    uint32_t* cand_i = reinterpret_cast<uint32_t*>(cand_q + P.ccap);
    const uint32_t b = blockIdx.x;
    if (threadIdx.x == 0) {
        resolve_row(P, b, S.rc);
        S.error = 0u;
    }
    __syncthreads();
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
    const uint32_t n = merge_lists(P, b, rc, P.split, S, cand_q, cand_i, overflow, qmax);
    finish_row(P, b, rc, n, overflow, qmax, S, cand_q, cand_i);
}

// ---------------------------------------------------------------------------
// Full ordering of a row in global scratch (bitonic sort of 64-bit keys), then
// the ordered tail exactly as the reference walks it. Slow and rarely needed:
// rows whose window overflowed or whose kept set / walk left the window.
constexpr int FULL_THREADS = 1024;

struct FullShared {
    RowCfg rc;
    uint32_t nvalid, keep, token, flags, kept_n;
    float sum, total, u, r, thr;
};

__global__ void __launch_bounds__(FULL_THREADS) full_sort_kernel(const __grid_constant__ KParams P, uint64_t* keys_all,
                                                                 float* vals_all, uint32_t vpad, uint32_t* ticket) {
    extern __shared__ __align__(16) unsigned char dynf[];
    __shared__ FullShared F;
    uint32_t* hkeys = reinterpret_cast<uint32_t*>(dynf);
    uint32_t* hcnt = hkeys + P.hash_slots;
    const uint32_t tid = threadIdx.x;
    const uint32_t count = *(volatile uint32_t*)P.full_count;
    uint64_t* keys = keys_all + (size_t)blockIdx.x * vpad;
    float* vals = vals_all + (size_t)blockIdx.x * vpad;
    const uint32_t V = P.vocab;
    uint32_t m = 1u;
    while (m < V) m <<= 1;

    for (uint32_t r = blockIdx.x; r < count; r += gridDim.x) {
        const uint32_t b = __ldcg(&P.full_list[r]);
        if (tid == 0) {
            resolve_row(P, b, F.rc);
            F.nvalid = 0u;
            F.keep = 0u;
            F.flags = 0u;
            F.kept_n = 0u;
            F.token = 0u;
            F.sum = F.total = F.u = F.r = F.thr = 0.f;
        }
        for (uint32_t i = tid; i < P.hash_slots; i += FULL_THREADS) {
            hkeys[i] = EMPTY_KEY;
            hcnt[i] = 0u;
        }
        __syncthreads();
        const RowCfg rc = F.rc;
        if (rc.has_pen) {
            const uint32_t* hist = P.history + (size_t)b * P.hist_stride;
            for (uint32_t j = tid; j < rc.hlen; j += FULL_THREADS) {
                const uint32_t id = __ldg(&hist[j]);
                if (id >= P.col_offset && id - P.col_offset < V) hash_insert(hkeys, hcnt, P.hash_slots, id);
            }
        }
        __syncthreads();
        // ---- keys: ascending u64 order == value descending, index ascending
        uint32_t myvalid = 0u;
        for (uint32_t c = tid; c < m; c += FULL_THREADS) {
            uint64_t key = ~0ull;
            if (c < V) {
                float x;
                if (P.dtype == LLM_CUDA_DTYPE_BF16)
                    x = load_logit(reinterpret_cast<const uint16_t*>(P.logits) + (size_t)b * P.row_stride + c);
                else
                    x = load_logit(reinterpret_cast<const float*>(P.logits) + (size_t)b * P.row_stride + c);
                const uint32_t gid = P.col_offset + c;
                if (id_blocked(P, gid)) x = neg_inf();
                if (rc.has_pen) x = penalize(x, rc.pen, hash_count(hkeys, hcnt, P.hash_slots, gid));
                const float q = temper(x, rc.T);
                if (q == q) {
                    key = ((uint64_t)(~okey(q)) << 32) | (uint64_t)c;
                    ++myvalid;
                }
            }
            __stcg(&keys[c], key);
        }
        if (myvalid) atomicAdd(&F.nvalid, myvalid);
        __syncthreads();
        for (uint32_t size = 2u; size <= m; size <<= 1) {
            for (uint32_t stride = size >> 1; stride > 0u; stride >>= 1) {
                for (uint32_t t = tid; t < (m >> 1); t += FULL_THREADS) {
                    const uint32_t lo = ((t & ~(stride - 1u)) << 1) | (t & (stride - 1u));
                    const uint32_t hi = lo + stride;
                    const uint64_t a = __ldcg(&keys[lo]), c = __ldcg(&keys[hi]);
                    const bool ascending = ((lo & size) == 0u);
                    if ((a > c) == ascending) {
                        __stcg(&keys[lo], c);
                        __stcg(&keys[hi], a);
                    }
                }
                __syncthreads();
            }
        }
        const uint32_t n = min(F.nvalid, rc.k_eff);
        auto q_at = [&](uint32_t i) { return okey_to_float(~(uint32_t)(__ldcg(&keys[i]) >> 32)); };
        auto id_at = [&](uint32_t i) { return P.col_offset + (uint32_t)(__ldcg(&keys[i]) & 0xffffffffull); };
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
            for (uint32_t i = tid; i < n; i += FULL_THREADS) __stcg(&vals[i], exp_f32(__fsub_rn(q_at(i), mx)));
            __syncthreads();
            if (tid == 0) {
                float s = 0.0f;
                for (uint32_t i = 0; i < n; ++i) {
                    const float e = __ldcg(&vals[i]);
                    if (e < 5.9604644775390625e-08f && s >= 1.0f) break;
                    s = __fadd_rn(s, e);
                }
                F.sum = s;
                F.keep = n;
            }
            __syncthreads();
            const float sum = F.sum;
            if ((sum <= 0.0f) || !(fabsf(sum) <= 3.402823466e38f)) {
                if (tid == 0) {
                    F.token = id_at(0);
                    F.flags = LLM_CUDA_ROW_DEGENERATE;
                }
                done = true;
            }
            if (!done) {
                for (uint32_t i = tid; i < n; i += FULL_THREADS) __stcg(&vals[i], __fdiv_rn(__ldcg(&vals[i]), sum));
                __syncthreads();
                if (rc.min_p > 0.0f) {
                    const float thr = __fmul_rn(rc.min_p, __ldcg(&vals[0]));
                    uint32_t first_fail = n;
                    for (uint32_t i = tid; i < n; i += FULL_THREADS) {
                        if (!(__ldcg(&vals[i]) >= thr)) {
                            first_fail = i;
                            break;
                        }
                    }
                    if (first_fail < n) atomicMin(&F.keep, first_fail);
                    __syncthreads();
                    if (tid == 0) {
                        F.thr = thr;
                        if (F.keep < 1u) F.keep = 1u;
                    }
                    __syncthreads();
                }
                if (tid == 0) {
                    const uint32_t keep_minp = F.keep;
                    uint32_t keep = keep_minp;
                    float total = 0.0f;
                    const float p0 = __ldcg(&vals[0]);
                    const float tiny = __fmul_rn(p0, 1.4901161193847656e-08f);  // 2^-26 of the leader: below half an ulp of any running sum
                    if (rc.top_p < 1.0f) {
                        float cum = 0.0f;
                        for (uint32_t i = 0; i < keep_minp; ++i) {
                            const float p = __ldcg(&vals[i]);
                            if (p < tiny) break;  // this and all later terms leave cum unchanged: top_p is never reached
                            cum = __fadd_rn(cum, p);
                            if (cum >= rc.top_p) {
                                keep = i + 1u;
                                break;
                            }
                        }
                        total = cum;
                    } else {
                        for (uint32_t i = 0; i < keep_minp; ++i) {
                            const float p = __ldcg(&vals[i]);
                            if (p < tiny) break;
                            total = __fadd_rn(total, p);
                        }
                    }
                    float u;
                    if (P.uniforms) {
                        u = P.uniforms[b];
                    } else {
                        const uint64_t seed = P.seeds ? P.seeds[b] : P.seed_base + (uint64_t)b;
                        const uint64_t dn = P.draw_index ? P.draw_index[b] : 0ull;
                        u = u24_to_f32(splitmix_output(seed, dn + 1ull));
                    }
                    float rr = __fmul_rn(u, total);
                    F.total = total;
                    F.u = u;
                    F.r = rr;
                    uint32_t flags = LLM_CUDA_ROW_DRAW_CONSUMED;
                    uint32_t token = 0u;
                    bool found = false;
                    for (uint32_t i = 0; i < keep; ++i) {
                        const float p = __ldcg(&vals[i]);
                        if (rr < p) {
                            token = id_at(i);
                            found = true;
                            break;
                        }
                        rr = __fsub_rn(rr, p);
                    }
                    if (!found) {
                        token = id_at(keep - 1u);
                        flags |= LLM_CUDA_ROW_FALLBACK_LAST;
                    }
                    F.token = token;
                    F.flags = flags;
                    F.keep = keep;
                    F.kept_n = keep;
                }
            }
        }
        __syncthreads();
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
            for (uint32_t i = tid; i < lim; i += FULL_THREADS) {
                if (P.kept_ids) P.kept_ids[(size_t)b * P.kept_cap + i] = id_at(i);
                if (P.kept_probs) P.kept_probs[(size_t)b * P.kept_cap + i] = __ldcg(&vals[i]);
            }
        }
        __syncthreads();
    }
    // the last CTA to leave re-arms the row list for the next launch
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const uint32_t t = atomicAdd(ticket, 1u);
        if (t == gridDim.x - 1u) {
            *P.full_count = 0u;
            *ticket = 0u;
            __threadfence();
        }
    }
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
            if (history_pos) history_pos[r] = (len + 1u) % cap;
        } else {  // ring: overwrite the oldest entry (the penalty does not depend on the order)
            const uint32_t pos = history_pos ? history_pos[r] % cap : 0u;
            history[(size_t)r * history_stride + pos] = tok;
            if (history_pos) history_pos[r] = (pos + 1u) % cap;
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
static uint32_t pow2_ceil(uint32_t x) {
    uint32_t p = 1u;
    while (p < x) p <<= 1;
    return p;
}

int plan_launch(const DeviceInfo& dev, const KParams& base, bool top_k_known, uint32_t top_k_hint, uint32_t max_top_k,
                uint32_t max_history, uint32_t requested_split, uint32_t max_lists, LaunchPlan* plan) {
    // candidate capacity
    uint32_t kcap;
    if (top_k_known) {
        const uint32_t k = (top_k_hint == 0u || top_k_hint >= base.vocab_global) ? base.vocab_global : top_k_hint;
        kcap = (k <= MAX_KCAP) ? pow2_ceil(k < 256u ? 256u : k) : 1024u;
    } else {
        kcap = pow2_ceil(max_top_k < 256u ? 256u : (max_top_k > MAX_KCAP ? MAX_KCAP : max_top_k));
    }
    plan->kcap = kcap;
    plan->ccap = 2u * kcap + TILE_ELEMS;
    plan->bits = (base.allowed_bits != nullptr) || (base.history != nullptr && (base.r_rows != nullptr || base.penalty != 1.0f) &&
                                                    (base.hist_len_rows != nullptr || base.hist_len > 0u));
    // split: fill the machine when the batch is small, keep shards long enough to stream
    uint32_t split = requested_split;
    if (split == 0u) {
        const uint32_t target = 4u * dev.sm_count;
        split = target / (base.batch ? base.batch : 1u);
        const uint32_t by_len = base.vocab / 8192u;
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
    if (plan->bits) {
        plan->bitmap_words = (shard_cols + 8u + 31u) / 32u + 1u;
        plan->hash_slots = pow2_ceil(2u * (max_history ? max_history : 1u));
        if (plan->hash_slots < 64u) plan->hash_slots = 64u;
    } else {
        plan->bitmap_words = 0u;
        plan->hash_slots = 0u;
    }
    plan->smem = (size_t)plan->ccap * 8u + (size_t)plan->bitmap_words * 4u + (size_t)plan->hash_slots * 8u;
    if (plan->smem > dev.max_dyn_smem) return -1;
    return 0;
}

cudaError_t configure_kernels(size_t max_dyn_smem) {
    const int v = (int)max_dyn_smem;
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(stream_select_kernel<float, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, v)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(stream_select_kernel<float, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, v)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(stream_select_kernel<uint16_t, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, v)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(stream_select_kernel<uint16_t, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, v)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(merge_draw_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, v)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(full_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, v)) != cudaSuccess) return e;
    return cudaSuccess;
}

template <typename ElemT, bool BITS>
static cudaError_t launch_stream_t(const KParams& P, const LaunchPlan& plan, cudaStream_t stream) {
    auto kern = stream_select_kernel<ElemT, BITS>;
    dim3 grid(plan.split, P.batch, 1);
    kern<<<grid, THREADS, plan.smem, stream>>>(P);
    return cudaGetLastError();
}

cudaError_t launch_stream_select(const KParams& P, const LaunchPlan& plan, cudaStream_t stream) {
    if (P.dtype == LLM_CUDA_DTYPE_BF16) {
        return plan.bits ? launch_stream_t<uint16_t, true>(P, plan, stream) : launch_stream_t<uint16_t, false>(P, plan, stream);
    }
    return plan.bits ? launch_stream_t<float, true>(P, plan, stream) : launch_stream_t<float, false>(P, plan, stream);
}

cudaError_t launch_merge_draw(const KParams& P, const LaunchPlan& plan, cudaStream_t stream) {
    const size_t smem = (size_t)plan.ccap * 8u;
    merge_draw_kernel<<<P.batch, THREADS, smem, stream>>>(P);
    return cudaGetLastError();
}

cudaError_t launch_full_sort(const KParams& P, uint32_t hash_slots, uint32_t nslots, uint64_t* keys, float* vals, uint32_t vpad,
                             uint32_t* ticket, cudaStream_t stream) {
    KParams Q = P;
    Q.hash_slots = hash_slots;
    const size_t smem = (size_t)hash_slots * 8u;
    full_sort_kernel<<<nslots, FULL_THREADS, smem, stream>>>(Q, keys, vals, vpad, ticket);
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

}  // namespace llmc
