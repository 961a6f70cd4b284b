// Device-side building blocks of the B200 token sampler (sm_100a).
//
// Everything here reproduces, per row, the arithmetic of the reference's
// `sample_with` (crates/llm-core/src/generate.rs:325-420): each f32 operation
// of the reference is one explicitly rounded operation here (__fadd_rn,
// __fmul_rn, __fdiv_rn, ...), in the same order, so no multiply-add is fused and
// no sum is reassociated.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/llm_cuda.h"
#include "sampler_kernels.h"

namespace llmc {

// Development builds only (-DLLMC_DEV; the product build never sets it): per-CTA phase marks, 16 per
// CTA: slots 0 and 11 hold the global timer (the CTA's start and end), the others the SM's cycle counter.
#ifdef LLMC_DEV
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define PHASE(slot)                                                                                              \
    do {                                                                                                         \
        if (P.phase_ns && threadIdx.x == 0)                                                                      \
            P.phase_ns[((size_t)blockIdx.y * gridDim.x + blockIdx.x) * 16u + (slot)] =                            \
                ((slot) == 0 || (slot) == 11) ? global_ns() : (unsigned long long)clock64();                                       \
    } while (0)
#else
#define PHASE(slot) do { } while (0)
#endif

// Checked builds (-DLLM_CUDA_CHECKED, a second library the tests run the small and odd shapes against): every
// store at a computed offset into the kernels' shared-memory regions or into scratch is compared with
// the region's size first. An offset out of bounds sets LLM_CUDA_STATUS_CHECK_FAILED in the device status
// word and the store is skipped - nothing traps. The product build compiles the test away.
#ifdef LLM_CUDA_CHECKED
#define IN_BOUNDS(idx, bound) llmc::in_bounds_or_report(P, (uint32_t)(idx), (uint32_t)(bound))
#else
#define IN_BOUNDS(idx, bound) true
#endif

constexpr int THREADS = 256;             // threads per CTA of the streaming kernel
constexpr int WARPS = THREADS / 32;
constexpr uint32_t STAGE_BYTES = 12288;  // the smaller of the two ring stage sizes (12 KB / 16 KB, chosen per launch)
constexpr int RING_STAGES = 3;           // bulk copies in flight per CTA: up to RING_STAGES stages
constexpr uint32_t WINDOW_CAP = 2048;    // candidate buffer of launches whose rows all run in window mode
constexpr uint32_t MAX_SORT = 4096;      // most candidates the ordered tail takes (its scratch lives in the ring's memory after the sweep)
constexpr uint32_t WINDOW_CAP_WIDE = 4096; // the same, where the ring leaves room for it without costing a resident CTA
// Probabilities of up to MAX_SORT candidates. The sort keys share it: a rank sort (at most THREADS entries)
// keeps its keys in the last THREADS * 8 bytes, which its own probabilities never reach; the key-only
// network (at most 2048 entries) takes the whole block before any probability exists.
constexpr uint32_t EPILOGUE_SCRATCH = MAX_SORT * 4u;
constexpr uint32_t RANK_KEYS_OFF = EPILOGUE_SCRATCH - (uint32_t)THREADS * 8u;
static_assert((size_t)THREADS * 8u + (size_t)MAX_SORT * 4u <= (size_t)RING_STAGES * STAGE_BYTES, "epilogue scratch");
constexpr unsigned FULL_MASK = 0xffffffffu;
constexpr uint32_t EMPTY_KEY = 0xffffffffu;
constexpr uint32_t MAX_KCAP = 2048;      // largest top_k handled by exact selection; above: window mode

// Window mode (top_k == 0 or beyond MAX_KCAP): the reference's left-to-right
// f32 sums over the descending ordering stop changing once exp(q - max) < 2^-25
// (the running sum is >= 1 after the leader, so such a term is below half an
// ulp), so only values with fl(q - max) >= WINDOW_EXACT can influence any sum,
// cut or probability. The streaming filter uses the wider WINDOW_STREAM bound.
constexpr float WINDOW_EXACT = -17.4f;
constexpr float WINDOW_STREAM = 17.5f;

// Internal row flag: the candidate window could not decide the row; the
// row is then ordered in full by its own CTA. Never visible to the caller.
constexpr uint32_t ROW_NEEDS_FULL = 0x80000000u;


// Barrier over the THREADS consumer threads of a CTA (named barrier 1). The streaming kernel
// runs one extra warp that only issues bulk copies and never joins these barriers.
__device__ __forceinline__ void cta_sync() { asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory"); }
__device__ __forceinline__ int cta_sync_or(int pred) {
    int r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.s32 p, %1, 0;\n\tbar.red.or.pred q, 1, %2, p;\n\tselp.s32 %0, 1, 0, q;\n\t}"
        : "=r"(r)
        : "r"(pred), "n"(THREADS)
        : "memory");
    return r;
}

#ifdef LLM_CUDA_CHECKED
__device__ __forceinline__ bool in_bounds_or_report(const KParams& P, uint32_t idx, uint32_t bound) {
    if (idx < bound) return true;
    if (P.device_errors) atomicOr(P.device_errors, LLM_CUDA_STATUS_CHECK_FAILED);
    return false;
}
#endif

struct RowCfg {
    float T, top_p, min_p, pen;
    uint32_t k_eff;     // rank cut: min(top_k, vocab), vocab when top_k == 0, 1 when greedy
    uint32_t hlen;
    uint32_t greedy, windowed, invalid, has_pen;
};

// ---------------------------------------------------------------------------
// ordered keys: u32 keys whose unsigned order is the numeric order of the
// floats, with -0.0 folded onto +0.0 (the reference compares numerically,
// generate.rs:366, so the two zeros tie and the lower index wins).
__device__ __forceinline__ uint32_t okey(float x) {
    x = __fadd_rn(x, 0.0f);
    uint32_t b = __float_as_uint(x);
    return b ^ ((uint32_t)((int32_t)b >> 31) | 0x80000000u);
}
__device__ __forceinline__ float okey_to_float(uint32_t k) {
    uint32_t b = (k & 0x80000000u) ? (k ^ 0x80000000u) : ~k;
    return __uint_as_float(b);
}
// composite ordering key: larger = earlier in the reference's ordering
// (value descending, index ascending).
__device__ __forceinline__ uint64_t composite(float q, uint32_t idx) {
    return ((uint64_t)okey(q) << 32) | (uint64_t)(~idx);
}
// true when (qa, ia) comes before (qb, ib) in the reference's ordering
__device__ __forceinline__ bool before(float qa, uint32_t ia, float qb, uint32_t ib) {
    return composite(qa, ia) > composite(qb, ib);
}

__device__ __forceinline__ float neg_inf() { return __uint_as_float(0xff800000u); }
__device__ __forceinline__ float pos_inf() { return __uint_as_float(0x7f800000u); }

// SplitMix64 output number n (1-based) of Rng::seed_from_u64(seed)
// (crates/llm-core/src/rng.rs:16-22): the state after n steps is seed + n*gamma.
__device__ __forceinline__ uint64_t splitmix_output(uint64_t seed, uint64_t n) {
    uint64_t z = seed + n * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
// next_f32 (rng.rs:31-34): top 24 bits over 2^24, exact in f32.
__device__ __forceinline__ float u24_to_f32(uint64_t out) {
    return __fmul_rn((float)(uint32_t)(out >> 40), 1.0f / 16777216.0f);
}

// exp as the reference sees it (generate.rs:373): the double-precision exp
// rounded once to f32, i.e. the correctly rounded f32 exp except when the double
// result lies within a double ulp of a rounding boundary.
__device__ __forceinline__ float exp_f32(float x) { return __double2float_rn(exp((double)x)); }

__device__ __forceinline__ float penalize(float x, float pen, uint32_t times) {
    // generate.rs:343-352: once per history occurrence, each step rounded.
    for (uint32_t i = 0; i < times; ++i) x = (x > 0.0f) ? __fdiv_rn(x, pen) : __fmul_rn(x, pen);
    return x;
}

__device__ __forceinline__ float load_logit(const float* p) { return *p; }
__device__ __forceinline__ float load_logit(const uint16_t* p) {
    return __uint_as_float((uint32_t)(*p) << 16);  // bf16.rs:22-25
}

// ---------------------------------------------------------------------------
__device__ __forceinline__ void resolve_row(const KParams& P, uint32_t b, RowCfg& rc) {
    float T = P.t_rows ? P.t_rows[b] : P.temperature;
    uint32_t k = P.k_rows ? P.k_rows[b] : P.top_k;
    rc.top_p = P.p_rows ? P.p_rows[b] : P.top_p;
    rc.min_p = P.m_rows ? P.m_rows[b] : P.min_p;
    rc.pen = P.r_rows ? P.r_rows[b] : P.penalty;
    rc.hlen = P.history ? (P.hist_len_rows ? min(P.hist_len_rows[b], P.hist_stride) : P.hist_len) : 0u;
    rc.invalid = (T != T) || (rc.pen != rc.pen);
    rc.greedy = (!rc.invalid && T <= 0.0f) ? 1u : 0u;           // generate.rs:354
    rc.T = rc.greedy ? 1.0f : T;
    const uint32_t vg = P.vocab_global;
    rc.k_eff = rc.greedy ? 1u : ((k == 0u || k >= vg) ? vg : k);  // generate.rs:368-370
    rc.windowed = (!rc.greedy && rc.k_eff > P.kcap) ? 1u : 0u;
    rc.has_pen = (rc.pen != 1.0f && rc.hlen > 0u) ? 1u : 0u;      // generate.rs:343
}

// Lower bound, in the pre-temperature domain, for "x / T >= tq": fl(tq * T)
// lowered by four floats. A superset filter; exact selection happens on q.
__device__ __forceinline__ uint32_t raw_threshold_key(float tq, float T) {
    float tx = (T == 1.0f) ? tq : __fmul_rn(tq, T);
    const uint32_t lowest = 0x007fffffu;  // okey(-inf); smaller keys would decode to NaN
    if (tx != tx) return lowest;          // NaN (0 * inf): filter nothing
    const uint32_t k = okey(tx);
    return k > lowest + 4u ? k - 4u : lowest;
}

// ---------------------------------------------------------------------------
// shared-memory hash of the history ids that fall into this CTA's columns:
// id -> number of occurrences.
__device__ __forceinline__ uint32_t hash_slot(uint32_t id, uint32_t mask) { return ((id * 0x9E3779B1u) >> 11) & mask; }

__device__ __forceinline__ void hash_insert(uint32_t* hkeys, uint32_t* hcnt, uint32_t slots, uint32_t id) {
    const uint32_t mask = slots - 1u;
    uint32_t h = hash_slot(id, mask);
    for (uint32_t probe = 0; probe < slots; ++probe) {
        uint32_t prev = atomicCAS(&hkeys[h], EMPTY_KEY, id);
        if (prev == EMPTY_KEY || prev == id) {
            atomicAdd(&hcnt[h], 1u);
            return;
        }
        h = (h + 1u) & mask;
    }
}
// Same insertion; returns the slot when this call created it (the first occurrence of the id), else EMPTY_KEY.
__device__ __forceinline__ uint32_t hash_insert_owner(uint32_t* hkeys, uint32_t* hcnt, uint32_t slots, uint32_t id) {
    const uint32_t mask = slots - 1u;
    uint32_t h = hash_slot(id, mask);
    for (uint32_t probe = 0; probe < slots; ++probe) {
        uint32_t prev = atomicCAS(&hkeys[h], EMPTY_KEY, id);
        if (prev == EMPTY_KEY || prev == id) {
            atomicAdd(&hcnt[h], 1u);
            return prev == EMPTY_KEY ? h : EMPTY_KEY;
        }
        h = (h + 1u) & mask;
    }
    return EMPTY_KEY;
}
__device__ __forceinline__ uint32_t hash_count(const uint32_t* hkeys, const uint32_t* hcnt, uint32_t slots, uint32_t id) {
    const uint32_t mask = slots - 1u;
    uint32_t h = hash_slot(id, mask);
    for (uint32_t probe = 0; probe < slots; ++probe) {
        uint32_t k = hkeys[h];
        if (k == id) return hcnt[h];
        if (k == EMPTY_KEY) return 0u;
        h = (h + 1u) & mask;
    }
    return 0u;
}

// allowed(id) of generate.rs:333-341: EOS always, ids past the mask always.
__device__ __forceinline__ bool id_blocked(const KParams& P, uint32_t gid) {
    if (!P.allowed_bits || gid == P.eos_id || gid >= P.allowed_len) return false;
    return ((__ldg(&P.allowed_bits[gid >> 5]) >> (gid & 31u)) & 1u) == 0u;
}

// ---------------------------------------------------------------------------
// Block-wide state of one row's candidate buffer.
struct Shared {
    RowCfg rc;
    uint32_t count;        // candidates in the buffer
    uint32_t tau_key;      // ordered key of the streaming threshold (pre-temperature domain)
    uint32_t max_key;      // ordered key of the largest pre-temperature value seen
    uint32_t newcount;
    uint32_t minkey;
    uint32_t sel_digit, sel_need, sel_bucket;
    uint32_t keep;
    uint32_t error;        // internal consistency failures (buffer overrun guard)
    uint32_t last;         // this CTA merges the row
    uint32_t sortmax;      // ordered key of the largest candidate, found while the small sort stages its keys
    uint32_t wkth[WARPS];   // per-warp lower bounds for the first tile's threshold
    float u_pre;              // the row's uniform, fetched early by kernels that can (u_pre_valid != 0)
    uint32_t u_pre_valid;
    uint32_t hist[2][256];  // radix-select histograms, alternated between passes
    float f_sum, f_total, f_u, f_r, f_thr;
    uint32_t token, out_flags, kept_n, walk_end;
    uint32_t ex_done, ex_all;  // rounds of the flagged-vector examination that ran / that the list holds
};

// Warp-collective append of passing lanes to the candidate buffer. `end` tracks
// the highest slot handed out so far as seen by this warp.
__device__ __forceinline__ void warp_append(bool pass, float q, uint32_t idx, Shared& S, float* cand_q, uint32_t* cand_i,
                                            uint32_t ccap, uint32_t& end) {
    const unsigned m = __ballot_sync(FULL_MASK, pass);
    if (m == 0u) return;
    const unsigned lane = threadIdx.x & 31u;
    const int leader = __ffs(m) - 1;
    uint32_t base = 0;
    if ((int)lane == leader) base = atomicAdd(&S.count, (uint32_t)__popc(m));
    base = __shfl_sync(FULL_MASK, base, leader);
    if (pass) {
        const uint32_t slot = base + (uint32_t)__popc(m & ((1u << lane) - 1u));
        if (slot < ccap) {
            cand_q[slot] = q;
            cand_i[slot] = idx;
        } else {
            S.error = 1u;
        }
    }
    end = max(end, base + (uint32_t)__popc(m));
}

// In-place compaction of cand[0..n) to the entries `keep` accepts; returns the
// new count (order not preserved) and leaves the smallest kept ordered key in
// S.minkey. Round r reads slots [r*THREADS, (r+1)*THREADS) and, after a
// barrier, writes below the number kept so far, which never exceeds the slots
// already read.
template <class Pred>
__device__ __forceinline__ uint32_t compact_inplace(uint32_t n, Pred keep, Shared& S, float* cand_q, uint32_t* cand_i) {
    if (threadIdx.x == 0) {
        S.newcount = 0u;
        S.minkey = 0xffffffffu;
    }
    cta_sync();
    const unsigned lane = threadIdx.x & 31u;
    for (uint32_t base = 0; base < n; base += THREADS) {
        const uint32_t i = base + threadIdx.x;
        bool k = false;
        float q = 0.f;
        uint32_t id = 0u;
        if (i < n) {
            q = cand_q[i];
            id = cand_i[i];
            k = keep(q, id);
        }
        cta_sync();
        const unsigned m = __ballot_sync(FULL_MASK, k);
        if (m) {
            const int leader = __ffs(m) - 1;
            const uint32_t mk = __reduce_min_sync(FULL_MASK, k ? okey(q) : 0xffffffffu);
            uint32_t dst = 0;
            if ((int)lane == leader) {
                dst = atomicAdd(&S.newcount, (uint32_t)__popc(m));
                atomicMin(&S.minkey, mk);
            }
            dst = __shfl_sync(FULL_MASK, dst, leader);
            if (k) {
                const uint32_t slot = dst + (uint32_t)__popc(m & ((1u << lane) - 1u));
                cand_q[slot] = q;
                cand_i[slot] = id;
            }
        }
    }
    cta_sync();
    return S.newcount;
}

// Radix select over the 64-bit composite keys of cand[0..n): finds (shift, thr)
// such that exactly k entries satisfy (composite >> shift) >= thr. Requires
// 1 <= k < n. Eight bits per pass from the top; stops as soon as the bucket that
// holds the k-th entry is wanted whole. A warp whose active lanes all hit the same
// bin adds once (the top bytes of float keys are nearly constant, and a plain
// histogram would serialise on one address); otherwise every lane adds for itself
// (`match_any` takes a step per distinct digit, far more than the few conflicts of
// mixed digits cost). The 256-bin scan is done redundantly by every warp, so a pass
// costs two barriers.
__device__ __forceinline__ void radix_select(uint32_t n, uint32_t k, Shared& S, const float* cand_q, const uint32_t* cand_i,
                                             uint64_t& thr, int& shift) {
    uint64_t prefix = 0ull;
    uint32_t need = k;
    const unsigned lane = threadIdx.x & 31u;
    S.hist[0][threadIdx.x] = 0u;  // THREADS == 256 bins
    cta_sync();
    const uint32_t n_up = (n + 31u) & ~31u;  // whole warps iterate together
    for (int p = 0; p < 8; ++p) {
        const int sh = 56 - 8 * p;
        uint32_t* H = S.hist[p & 1];
        for (uint32_t i = threadIdx.x; i < n_up; i += THREADS) {
            bool act = false;
            uint32_t digit = 0u;
            if (i < n) {
                const uint64_t c = composite(cand_q[i], cand_i[i]);
                act = (p == 0) || ((c >> (sh + 8)) == prefix);
                digit = (uint32_t)(c >> sh) & 255u;
            }
            const unsigned am = __ballot_sync(FULL_MASK, act);
            if (am) {
                const int src = __ffs(am) - 1;
                const uint32_t d0 = __shfl_sync(FULL_MASK, digit, src);
                if (__all_sync(FULL_MASK, !act || digit == d0)) {
                    if ((int)lane == src) atomicAdd(&H[d0], (uint32_t)__popc(am));
                } else if (act) {
                    atomicAdd(&H[digit], 1u);
                }
            }
        }
        S.hist[(p + 1) & 1][threadIdx.x] = 0u;  // last read two barriers ago
        cta_sync();
        // every warp scans the 256 bins: lane l owns bins [8l, 8l+8)
        uint32_t bins[8];
        uint32_t mine = 0u;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            bins[j] = H[lane * 8u + j];
            mine += bins[j];
        }
        uint32_t x = mine;  // becomes the number of entries in bins of lanes >= lane
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t y = __shfl_down_sync(FULL_MASK, x, o);
            if (lane + o < 32u) x += y;
        }
        const uint32_t above_lane = x - mine;
        const bool owner = (above_lane < need) && (need <= x);
        uint32_t digit = 0u, newneed = 0u, bucket = 0u;
        if (owner) {
            uint32_t above = above_lane;
#pragma unroll
            for (int j = 7; j >= 0; --j) {
                if (above < need && need <= above + bins[j]) {
                    digit = lane * 8u + j;
                    newneed = need - above;
                    bucket = bins[j];
                }
                above += bins[j];
            }
        }
        const unsigned om = __ballot_sync(FULL_MASK, owner);
        const int src = om ? __ffs(om) - 1 : 0;
        digit = __shfl_sync(FULL_MASK, digit, src);
        newneed = __shfl_sync(FULL_MASK, newneed, src);
        bucket = __shfl_sync(FULL_MASK, bucket, src);
        prefix = (prefix << 8) | (uint64_t)digit;
        need = newneed;
        if (bucket == need || p == 7 || om == 0u) {
            shift = sh;
            thr = prefix;
            cta_sync();  // histograms are free again
            return;
        }
        cta_sync();
    }
}

// Keeps the best k entries of cand[0..n) (reference ordering); returns the new count.
__device__ __forceinline__ uint32_t keep_top_k(uint32_t n, uint32_t k, Shared& S, float* cand_q, uint32_t* cand_i) {
    if (n <= k) return n;
    uint64_t thr;
    int shift;
    radix_select(n, k, S, cand_q, cand_i, thr, shift);
    return compact_inplace(
        n, [=](float q, uint32_t id) { return (composite(q, id) >> shift) >= thr; }, S, cand_q, cand_i);
}

// Sorts cand[0..n), n <= THREADS, into the reference ordering by ranking: an entry's place is the
// number of entries that come before it. With n <= 128 the comparisons of one entry are split over
// 2, 4 or 8 threads (partial ranks meet in `rank_acc`, THREADS words of scratch). With `want_exp`, probs[rank] = exp(q - max) is computed alongside (the maximum
// is found while the keys are staged; S.sortmax must be 0 on entry), which is generate.rs:372-373
// for the sorted set: the double-precision exp runs while the ranks are counted.
__device__ __forceinline__ void sort_small(uint32_t n, Shared& S, float* cand_q, uint32_t* cand_i, uint64_t* keys64,
                                           uint32_t* rank_acc, float* probs, bool want_exp) {
    const uint32_t tid = threadIdx.x;
    const unsigned lane = tid & 31u;
    float q = 0.f;
    uint32_t id = 0u;
    const bool have = tid < n;
    if (have) {
        q = cand_q[tid];
        id = cand_i[tid];
        keys64[tid] = composite(q, id);
    }
    uint32_t parts = 1u;
    while (parts < 8u && n * 2u * parts <= (uint32_t)THREADS) parts <<= 1;
    if (parts > 1u) rank_acc[tid] = 0u;
    if (want_exp) {
        const uint32_t wk = __reduce_max_sync(FULL_MASK, have ? okey(q) : 0u);
        if (lane == 0 && wk) atomicMax(&S.sortmax, wk);
    }
    cta_sync();
    const uint32_t npad = (uint32_t)THREADS / parts;
    const uint32_t elem = tid & (npad - 1u), part = tid / npad;
    uint32_t rank = 0u;
    if (elem < n) {
        const uint64_t mine = keys64[elem];
        const uint32_t chunk = (n + parts - 1u) / parts;
        const uint32_t j0 = part * chunk, j1 = min(n, j0 + chunk);
#pragma unroll 4
        for (uint32_t j = j0; j < j1; ++j) rank += (keys64[j] > mine) ? 1u : 0u;  // keys are distinct
        if (parts > 1u && part > 0u && rank) atomicAdd(&rank_acc[elem], rank);
    }
    float e = 0.f;
    if (want_exp && have) e = exp_f32(__fsub_rn(q, okey_to_float(S.sortmax)));
    if (parts > 1u) cta_sync();
    if (have) {
        if (parts > 1u) rank += rank_acc[tid];  // tid < n <= npad: this thread is part 0 of its own entry
        cand_q[rank] = q;
        cand_i[rank] = id;
        if (want_exp) probs[rank] = e;
    }
    cta_sync();
}

// Sorts cand[0..n), THREADS < n <= 2048, into the reference ordering: a bitonic network over the 64-bit
// composite keys alone (one 8-byte word per entry in `keys`, room for the next power of two; padding keys
// are 0 and sort last), from which values and ids are read back afterwards (a value's ordered key is
// exact except that -0.0 comes back as +0.0, which no later stage can tell apart).
// Every thread holds E consecutive keys in registers: compare-exchange steps whose partners lie in the same
// thread need nothing, those inside a warp take one shuffle per key, and only the strides that cross warps
// (six steps of the whole network) go through shared memory and a barrier.
template <int E>
__device__ __forceinline__ void sort_keys64_regs(uint32_t n, float* cand_q, uint32_t* cand_i, uint64_t* keys) {
    const uint32_t t = threadIdx.x;
    constexpr uint32_t M = (uint32_t)E * (uint32_t)THREADS;
    uint64_t k[E];
#pragma unroll
    for (int e = 0; e < E; ++e) {
        const uint32_t i = t * E + e;
        k[e] = i < n ? composite(cand_q[i], cand_i[i]) : 0ull;
    }
#pragma unroll
    for (uint32_t size = 2u; size <= M; size <<= 1) {
#pragma unroll
        for (uint32_t stride = size >> 1; stride > 0u; stride >>= 1) {
            if (stride < (uint32_t)E) {
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    if ((e & stride) == 0u) {
                        const bool larger_first = (((t * E + e) & size) == 0u);  // first-in-order (largest key) at the low slot
                        const uint64_t lo = k[e], hi = k[e + stride];
                        if ((hi > lo) == larger_first) {
                            k[e] = hi;
                            k[e + stride] = lo;
                        }
                    }
                }
            } else if (stride < 32u * (uint32_t)E) {
                const uint32_t d = stride / (uint32_t)E;
                const bool am_low = (t & d) == 0u;
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    const uint64_t other = __shfl_xor_sync(FULL_MASK, k[e], (int)d);
                    const bool larger_first = (((t * E + e) & size) == 0u);
                    const bool keep_larger = (am_low == larger_first);
                    k[e] = keep_larger ? (other > k[e] ? other : k[e]) : (other < k[e] ? other : k[e]);
                }
            } else {
                cta_sync();  // the previous exchange's reads are done
#pragma unroll
                for (int e = 0; e < E; ++e) keys[t * E + e] = k[e];
                cta_sync();
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    const uint32_t i = t * E + e;
                    const uint64_t other = keys[i ^ stride];
                    const bool larger_first = ((i & size) == 0u);
                    const bool keep_larger = (((i & stride) == 0u) == larger_first);
                    k[e] = keep_larger ? (other > k[e] ? other : k[e]) : (other < k[e] ? other : k[e]);
                }
            }
        }
    }
    cta_sync();  // cand_q / cand_i were read by everyone long ago; the keys' last exchange is read
#pragma unroll
    for (int e = 0; e < E; ++e) {
        const uint32_t i = t * E + e;
        if (i < n) {
            cand_q[i] = okey_to_float((uint32_t)(k[e] >> 32));
            cand_i[i] = ~(uint32_t)k[e];
        }
    }
    cta_sync();
}

// Not inlined: the network's registers stay out of the streaming kernel's own allocation.
static __device__ __noinline__ void sort_keys64(uint32_t n, float* cand_q, uint32_t* cand_i, uint64_t* keys) {
    if (n <= 2u * THREADS)
        sort_keys64_regs<2>(n, cand_q, cand_i, keys);
    else if (n <= 4u * THREADS)
        sort_keys64_regs<4>(n, cand_q, cand_i, keys);
    else
        sort_keys64_regs<8>(n, cand_q, cand_i, keys);
}

// Sorts cand[0..n), n > THREADS, into the reference ordering with a bitonic network; slots [n, m)
// (m the next power of two) are filled with entries that sort last.
__device__ __forceinline__ void sort_candidates(uint32_t n, float* cand_q, uint32_t* cand_i) {
    uint32_t m = 1u;
    while (m < n) m <<= 1;
    for (uint32_t i = n + threadIdx.x; i < m; i += THREADS) {
        cand_q[i] = neg_inf();
        cand_i[i] = 0xffffffffu;
    }
    cta_sync();
    for (uint32_t size = 2u; size <= m; size <<= 1) {
        for (uint32_t stride = size >> 1; stride > 0u; stride >>= 1) {
            for (uint32_t t = threadIdx.x; t < (m >> 1); t += THREADS) {
                const uint32_t lo = ((t & ~(stride - 1u)) << 1) | (t & (stride - 1u));
                const uint32_t hi = lo + stride;
                const bool descending_block = ((lo & size) == 0u);  // first-in-order at the low slot
                const float ql = cand_q[lo], qh = cand_q[hi];
                const uint32_t il = cand_i[lo], ih = cand_i[hi];
                const bool hi_first = before(qh, ih, ql, il);
                if (hi_first == descending_block) {
                    cand_q[lo] = qh;
                    cand_i[lo] = ih;
                    cand_q[hi] = ql;
                    cand_i[hi] = il;
                }
            }
            cta_sync();
        }
    }
}

// ---------------------------------------------------------------------------
// The ordered tail of sample_with (generate.rs:372-419) over the sorted
// candidates cand[0..n). `probs` is scratch for n floats. `truncated` says that
// the reference's ordering continues past these n entries with values outside
// the significance window (window mode only). Thread 0 owns the sequential
// chains; everything else is data parallel. Returns through S: token, flags,
// kept_n and the stage statistics.
// A chain of dependent rounded f32 operations acc = op(acc, v[i]) over v[0..n) in shared memory (16-byte
// aligned), strictly in order, run by the calling thread alone. Whole blocks of 64 are walked eight values
// at a time, the next eight already loaded, with no test or branch inside the block (a test and a branch on
// the running value cost about fifty cycles, ten additions' worth); what is left, and a block that holds
// a hit, is walked in groups of eight with the test per element and one branch per group (keeping the
// first hit by selects instead makes a second, longer dependent chain: measured slower).
//   hit(before, after, x)  the chain stops at the first element where it holds: its index is returned and
//                          acc is left as it was after that element.
//   any_hit(after)         asked after a block with the value acc has then: true iff hit held for one of its
//                          elements (the callers' chains are monotone, so the last value tells); only then
//                          is the block walked again.
//   rest_is_noop(x0, acc)  asked before a block with its first value: true means no later element can change
//                          acc or hit (values are in descending order), so stop.
// MIN_BLOCKS: the block walk is used while that many blocks are left; a chain that can hit passes 2 (a rest
// of under 128 values is cheaper walked once, with the tests, than twice), one that cannot passes 1.
// Returns n when nothing hit.
template <uint32_t MIN_BLOCKS, class Op, class Hit, class AnyHit, class Noop>
__device__ __forceinline__ uint32_t thread_chain(const float* v, uint32_t n, float& acc_io, Op op, Hit hit, AnyHit any_hit,
                                                 Noop rest_is_noop) {
    float acc = acc_io;
    uint32_t j = 0u;
    uint32_t result = n;
    const float4* v4 = reinterpret_cast<const float4*>(v);
    // [from, to) in groups of eight with the hit test per element but one branch per group: the first hit, if any
    // (acc and result set, true returned); otherwise acc is the value after element to - 1
    auto walk = [&](uint32_t from, uint32_t to, float start) {
        float a = start;
#pragma unroll 1
        for (uint32_t i = from; i < to; i += 8u) {
            float x[8], c[8];
            if (i + 8u <= to) {
                const float4 lo = v4[i >> 2], hi = v4[(i >> 2) + 1u];
                x[0] = lo.x; x[1] = lo.y; x[2] = lo.z; x[3] = lo.w;
                x[4] = hi.x; x[5] = hi.y; x[6] = hi.z; x[7] = hi.w;
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) x[e] = (i + (uint32_t)e < to) ? v[i + e] : 0.0f;
            }
            uint32_t h = 0u;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float was = a;
                a = op(a, x[e]);
                c[e] = a;
                if (i + (uint32_t)e < to && hit(was, a, x[e])) h |= 1u << e;
            }
            if (h) {
                const uint32_t e0 = (uint32_t)__ffs(h) - 1u;
                float at = c[0];
#pragma unroll
                for (int e = 1; e < 8; ++e) at = (e0 == (uint32_t)e) ? c[e] : at;
                acc = at;
                result = i + e0;
                return true;
            }
        }
        acc = a;
        return false;
    };
    bool done = false;
#pragma unroll 1
    for (; j + MIN_BLOCKS * 64u <= n; j += 64u) {
        if (rest_is_noop(v[j], acc)) {
            done = true;
            break;
        }
        const float before = acc;
        float4 p = v4[j >> 2], q = v4[(j >> 2) + 1u];
#pragma unroll
        for (uint32_t s8 = 0; s8 < 8u; ++s8) {
            float4 p2 = p, q2 = q;
            if (s8 < 7u) {
                p2 = v4[(j >> 2) + 2u * s8 + 2u];
                q2 = v4[(j >> 2) + 2u * s8 + 3u];
            }
            acc = op(acc, p.x); acc = op(acc, p.y); acc = op(acc, p.z); acc = op(acc, p.w);
            acc = op(acc, q.x); acc = op(acc, q.y); acc = op(acc, q.z); acc = op(acc, q.w);
            p = p2;
            q = q2;
        }
        if (any_hit(acc) && walk(j, j + 64u, before)) {
            done = true;
            break;
        }
    }
    if (!done && j < n && !rest_is_noop(v[j], acc)) (void)walk(j, n, acc);
    acc_io = acc;
    return result;
}

// ---------------------------------------------------------------------------
// Long chains, exactly, by the whole CTA. The reference's sums are sequences of dependent rounded f32
// additions (or subtractions); a thread can only walk them one term after the other. But while the
// running value s stays inside one binade, s = A * u with u = ulp(s) and A an integer in
// [2^23, 2^24), and round-to-nearest-even of s + x is A + floor(x/u) + c, where c depends on the
// fraction of x/u alone (above / below one half) except for an exact half, where it depends on the
// parity of A. So every term is a little machine with two states (the parity of A before it) that
// adds an integer and leaves a parity, machines compose associatively, and a chunk of 2048 terms is
// evaluated with a prefix scan over the CTA instead of 2048 dependent additions. Whatever the
// integers cannot express is an "event", found as the first term where A would cross a bound: the
// value leaving its binade (the next binade rounds on a different grid), a term larger than the
// value, the cumulative sum reaching top_p, the walk's r falling below its term. The term of an
// event is evaluated with real f32 arithmetic from the exact value before it, so are a few terms
// after it (events come in clusters where value and terms are of similar size), and the scan starts
// again behind them. The result is bit for bit that of the sequential chain
// (tests/test_gpu_full_ordering.py and the flat-row parity tests run through it).
constexpr uint32_t CHAIN_SAT = 1u << 30;
struct ChainMachine {
    uint32_t inc0, inc1;  // what the terms add to A for parity 0 / 1 of A before them (saturating)
    uint32_t par;         // bit p: the parity they leave for parity p before them
};
__device__ __forceinline__ ChainMachine chain_then(const ChainMachine& f, const ChainMachine& g) {  // f's terms, then g's
    ChainMachine h;
    const uint32_t f0 = f.par & 1u, f1 = (f.par >> 1) & 1u;
    h.inc0 = min(f.inc0 + (f0 ? g.inc1 : g.inc0), CHAIN_SAT);
    h.inc1 = min(f.inc1 + (f1 ? g.inc1 : g.inc0), CHAIN_SAT);
    h.par = ((g.par >> f0) & 1u) | (((g.par >> f1) & 1u) << 1);
    return h;
}
// One term against a value whose unbiased exponent is es: floor(x/u), whether the fraction is above one
// half / exactly one half / not zero, and whether the term lies above the value's binade.
struct ChainTerm {
    uint32_t fl;
    uint32_t bits;  // 1: fraction > 1/2, 2: fraction == 1/2, 4: fraction != 0, 8: term above the binade
};
__device__ __forceinline__ ChainTerm chain_term(float x, int es) {
    const uint32_t b = __float_as_uint(x);
    const uint32_t ex = (b >> 23) & 0xffu;
    const uint32_t m = b & 0x7fffffu;
    const uint32_t M = ex ? (m | 0x800000u) : m;
    const int E = ex ? (int)ex - 127 : -126;
    const int shift = es - E;
    ChainTerm t;
    if (shift < 0) {
        t.fl = 0u;
        t.bits = 8u;
    } else if (shift >= 32) {
        t.fl = 0u;
        t.bits = M ? 4u : 0u;
    } else {
        t.fl = M >> shift;
        const uint32_t rem = M & ((1u << shift) - 1u);
        const uint32_t half = shift ? (1u << (shift - 1)) : 0xffffffffu;
        t.bits = (rem > half ? 1u : 0u) | (rem == half ? 2u : 0u) | (rem ? 4u : 0u);
    }
    return t;
}
__device__ __forceinline__ uint32_t chain_step(const ChainTerm& t, uint32_t parity) {  // what the term adds to / takes from A
    return t.fl + ((t.bits & 2u) ? ((parity + t.fl) & 1u) : (t.bits & 1u));
}

enum { CHAIN_SUM = 0, CHAIN_CUMULATIVE = 1, CHAIN_WALK = 2 };
constexpr uint32_t CHAIN_EPT = 8;                                  // terms per thread and chunk
constexpr uint32_t CHAIN_SPAN = CHAIN_EPT * (uint32_t)THREADS;     // terms per chunk
constexpr uint32_t CHAIN_WORDS = 3u * WARPS + 2u;                  // shared words the function needs

// Called by all THREADS threads of the CTA with the same arguments; v[0..n) in global (GLOBAL: read past L1,
// other threads of the CTA have just written it) or shared memory, descending (that is only used to stop
// early), finite, not negative. `sh`: CHAIN_WORDS words of shared memory.
//   CHAIN_SUM         acc = fl(acc + v[i]) over all i; returns n
//   CHAIN_CUMULATIVE  the same, stopping at the first i with acc >= bound (returned, acc as after it); n if none
//   CHAIN_WALK        stops at the first i with acc < v[i] (returned, acc as before it), else acc = fl(acc - v[i]); n if none
// Every thread returns the same result.
template <bool GLOBAL>
__device__ __noinline__ uint32_t cta_chain(const float* v, uint32_t n, int kind, float bound, float* acc_io, uint32_t* sh) {
    const uint32_t tid = threadIdx.x;
    const unsigned lane = tid & 31u, warp = tid >> 5;
    uint32_t* w_inc0 = sh;
    uint32_t* w_inc1 = sh + WARPS;
    uint32_t* w_par = sh + 2 * WARPS;
    uint32_t* sh_event = sh + 3 * WARPS;
    uint32_t* sh_before = sh + 3 * WARPS + 1;
    float s = *acc_io;
    uint32_t pos = 0u;
    uint32_t result = n;
    const bool sub = kind == CHAIN_WALK;
    auto at = [&](uint32_t i) { return GLOBAL ? __ldcg(v + i) : v[i]; };
    // one term with real arithmetic, by every thread alike; true when the chain ends at it
    auto real_step = [&](uint32_t i) {
        const float x = at(i);
        if (sub) {
            if (s < x) {
                result = i;
                return true;
            }
            s = __fsub_rn(s, x);
            return false;
        }
        s = __fadd_rn(s, x);
        if (kind == CHAIN_CUMULATIVE && s >= bound) {
            result = i;
            return true;
        }
        return false;
    };
    while (pos < n) {
        const uint32_t sb = __float_as_uint(s);
        const uint32_t sex = (sb >> 23) & 0xffu;
        if (sex == 0u || sex == 0xffu || (sb >> 31) || (pos & 7u)) {  // zero, subnormal, not finite or negative: no integer form
            if (real_step(pos)) break;
            ++pos;
            continue;
        }
        const int es = (int)sex - 127;
        const uint32_t A0 = (sb & 0x7fffffu) | 0x800000u;
        if (!sub) {
            // a term under half an ulp changes nothing, and the terms only get smaller
            const ChainTerm t0 = chain_term(at(pos), es);
            if (t0.fl == 0u && (t0.bits & 11u) == 0u) break;
        }
        // the bound on A that ends the scan: the binade's end, or where the value reaches `bound`
        uint32_t B = 1u << 24;
        if (kind == CHAIN_CUMULATIVE) {
            const uint32_t bb = __float_as_uint(bound);
            const uint32_t bex = (bb >> 23) & 0xffu;
            const int eb = bex ? (int)bex - 127 : -126;
            if ((bb >> 31) || bb == 0u || eb < es)
                B = 0u;  // every value qualifies
            else if (eb == es)
                B = min(B, (bb & 0x7fffffu) | 0x800000u);
        }
        if (tid == 0) *sh_event = 0xffffffffu;
        // this thread's terms (chunks start at multiples of eight: two 16-byte loads), and their machine
        float x[CHAIN_EPT];
        const uint32_t first = pos + tid * CHAIN_EPT;
        if (first + CHAIN_EPT <= n) {
            const float4* v4 = reinterpret_cast<const float4*>(v + first);
            const float4 lo = GLOBAL ? __ldcg(v4) : v4[0];
            const float4 hi = GLOBAL ? __ldcg(v4 + 1) : v4[1];
            x[0] = lo.x; x[1] = lo.y; x[2] = lo.z; x[3] = lo.w;
            x[4] = hi.x; x[5] = hi.y; x[6] = hi.z; x[7] = hi.w;
        } else {
#pragma unroll
            for (uint32_t k = 0; k < CHAIN_EPT; ++k) x[k] = first + k < n ? at(first + k) : 0.0f;
        }
        ChainMachine mine;
        mine.inc0 = mine.inc1 = 0u;
        mine.par = 2u;
        {
            uint32_t p0 = 0u, p1 = 1u;
#pragma unroll
            for (uint32_t k = 0; k < CHAIN_EPT; ++k) {
                const ChainTerm t = chain_term(x[k], es);
                const uint32_t d0 = chain_step(t, p0), d1 = chain_step(t, p1);
                mine.inc0 = min(mine.inc0 + d0, CHAIN_SAT);
                mine.inc1 = min(mine.inc1 + d1, CHAIN_SAT);
                p0 = (p0 + d0) & 1u;
                p1 = (p1 + d1) & 1u;
            }
            mine.par = p0 | (p1 << 1);
        }
        // inclusive scan over the warp, then over the warps
        ChainMachine incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            ChainMachine prev;
            prev.inc0 = __shfl_up_sync(FULL_MASK, incl.inc0, o);
            prev.inc1 = __shfl_up_sync(FULL_MASK, incl.inc1, o);
            prev.par = __shfl_up_sync(FULL_MASK, incl.par, o);
            if (lane >= (unsigned)o) incl = chain_then(prev, incl);
        }
        if (lane == 31) {
            w_inc0[warp] = incl.inc0;
            w_inc1[warp] = incl.inc1;
            w_par[warp] = incl.par;
        }
        ChainMachine excl;  // the terms of this warp before this thread's
        excl.inc0 = __shfl_up_sync(FULL_MASK, incl.inc0, 1);
        excl.inc1 = __shfl_up_sync(FULL_MASK, incl.inc1, 1);
        excl.par = __shfl_up_sync(FULL_MASK, incl.par, 1);
        if (lane == 0) {
            excl.inc0 = excl.inc1 = 0u;
            excl.par = 2u;
        }
        cta_sync();
        ChainMachine before;  // everything before this thread's terms
        before.inc0 = before.inc1 = 0u;
        before.par = 2u;
        ChainMachine whole = before;  // the whole chunk
#pragma unroll
        for (uint32_t w = 0; w < (uint32_t)WARPS; ++w) {
            ChainMachine m;
            m.inc0 = w_inc0[w];
            m.inc1 = w_inc1[w];
            m.par = w_par[w];
            if (w < warp) before = chain_then(before, m);
            whole = chain_then(whole, m);
        }
        before = chain_then(before, excl);
        const uint32_t par0 = A0 & 1u;
        const uint32_t moved = par0 ? before.inc1 : before.inc0;
        uint32_t A = sub ? A0 - min(moved, A0) : A0 + moved;
        uint32_t my_event = 0xffffffffu, my_before = 0u;
#pragma unroll
        for (uint32_t k = 0; k < CHAIN_EPT; ++k) {
            const ChainTerm t = chain_term(x[k], es);
            const uint32_t d = chain_step(t, A & 1u);
            bool ev;
            if (sub)
                ev = (t.bits & 8u) || A < t.fl + ((t.bits >> 2) & 1u) + (1u << 23);
            else
                ev = (t.bits & 8u) || A + d >= B;
            if (ev && my_event == 0xffffffffu && first + k < n) {
                my_event = first + k;
                my_before = A;
            }
            A = sub ? A - d : A + d;
        }
        if (my_event != 0xffffffffu) atomicMin(sh_event, my_event);
        cta_sync();
        const uint32_t ev = *sh_event;
        if (ev == 0xffffffffu) {
            const uint32_t all = par0 ? whole.inc1 : whole.inc0;
            const uint32_t A_end = sub ? A0 - all : A0 + all;
            s = __uint_as_float((sb & 0xff800000u) | (A_end & 0x7fffffu));  // same binade: A_end in [2^23, 2^24)
            pos = min(pos + CHAIN_SPAN, n);
            cta_sync();  // everyone has read the event word before the next chunk resets it
            continue;
        }
        if (my_event == ev) *sh_before = my_before;
        cta_sync();
        const uint32_t A_before = *sh_before;
        s = __uint_as_float((sb & 0xff800000u) | (A_before & 0x7fffffu));
        // the event's term and the terms up to the next multiple of eight (at least eight of them), one by one
        bool ended = false;
        uint32_t i = ev;
        const uint32_t until = min(n, (ev + 16u) & ~7u);
        for (; i < until; ++i) {
            if (real_step(i)) {
                ended = true;
                break;
            }
        }
        if (ended) break;
        pos = i;
    }
    *acc_io = s;
    return result;
}

// The ordered tail's three chains as functions of their own: inlined, their registers would be taken out of
// the streaming kernel's allocation, and whatever that spills costs a trip to L2 (the kernel runs with
// almost no L1).
//   generate.rs:374, the left-to-right f32 sum. Once the sum is >= 1 a term below 2^-24 is under half an
//   ulp and leaves it unchanged, and the terms only get smaller.
static __device__ __noinline__ float tail_sum(const float* probs, uint32_t n) {
    float s = 0.0f;
    thread_chain<1>(
        probs, n, s, [](float acc, float e) { return __fadd_rn(acc, e); }, [](float, float, float) { return false; },
        [](float) { return false; }, [](float e0, float acc) { return e0 < 5.9604644775390625e-08f && acc >= 1.0f; });
    return s;
}
//   generate.rs:397-409; the later re-summation of the kept prefix (:411) repeats the same additions. The
//   running sum never falls: it has reached top_p inside a block iff it is there at the block's end.
//   Returns the first index that reaches top_p (n if none, or if top_p is 1); the sum so far in *total.
static __device__ __noinline__ uint32_t tail_cumulative(const float* probs, uint32_t n, float top_p, float* total) {
    float acc = 0.0f;
    auto add = [](float a, float p) { return __fadd_rn(a, p); };
    auto never = [](float, float) { return false; };
    uint32_t at;
    if (top_p < 1.0f)
        at = thread_chain<2>(probs, n, acc, add, [=](float, float after, float) { return after >= top_p; },
                          [=](float after) { return after >= top_p; }, never);
    else
        at = thread_chain<1>(probs, n, acc, add, [](float, float, float) { return false; }, [](float) { return false; }, never);
    *total = acc;
    return at;
}
//   generate.rs:413-418 stops at the first entry with r < p. r starts at u * total >= 0, and r - p rounds to
//   a negative number exactly when r < p; from there on it only falls: a block holds that entry iff r is
//   negative at the block's end. Returns that entry's index (n if there is none).
static __device__ __noinline__ uint32_t tail_walk(const float* probs, uint32_t n, float r) {
    return thread_chain<2>(
        probs, n, r, [](float acc, float p) { return __fsub_rn(acc, p); }, [](float before, float, float p) { return before < p; },
        [](float after) { return after < 0.0f; }, [](float, float) { return false; });
}

// The uniform the row's draw consumes: output `draw_index + 1` of its SplitMix64 stream
// (rng.rs:31-34), or the caller's pinned value.
__device__ __forceinline__ float row_uniform(const KParams& P, uint32_t b) {
    if (P.uniforms) return P.uniforms[b];
    const uint64_t seed = P.seeds ? P.seeds[b] : P.seed_base + (uint64_t)b;
    const uint64_t done = P.draw_index ? P.draw_index[b] : 0ull;
    return u24_to_f32(splitmix_output(seed, done + 1ull));
}

// `probs_ready`: probs[i] already holds exp(q_i - max) (the small sort computes it alongside the ranks).
// The chains of thread 0 run through thread_chain: the additions stay strictly sequential, only loads
// and comparisons leave the dependent chain.
__device__ __forceinline__ void ordered_tail(const KParams& P, uint32_t b, const RowCfg& rc, uint32_t n, bool truncated,
                                             uint32_t k_total, Shared& S, const float* cand_q, const uint32_t* cand_i,
                                             float* probs, bool probs_ready = false) {
    const float mx = cand_q[0];  // generate.rs:372 (the ordering is NaN-free, so the fold is its first element)
    if (!probs_ready)
        for (uint32_t i = threadIdx.x; i < n; i += THREADS) probs[i] = exp_f32(__fsub_rn(cand_q[i], mx));  // :373
    if (threadIdx.x == 0) {
        S.keep = n;
        S.out_flags = 0u;
        S.f_thr = 0.f;
        S.f_total = 0.f;
        S.f_u = 0.f;
        S.f_r = 0.f;
        S.kept_n = 0u;
    }
    cta_sync();
    PHASE(8);
    if (threadIdx.x == 0) {
        S.f_sum = tail_sum(probs, n);
    }
    const float e_first = probs[0];  // read before anyone normalises it (the barrier below comes first)
    cta_sync();
    PHASE(9);
    const float sum = S.f_sum;
    const bool degenerate = (sum <= 0.0f) || !(fabsf(sum) <= 3.402823466e38f);  // :375 (catches NaN and inf)
    if (degenerate) {
        if (threadIdx.x == 0) {
            S.token = cand_i[0];
            S.out_flags = LLM_CUDA_ROW_DEGENERATE;
        }
        cta_sync();
        return;
    }
    // :378-380 normalise, and :384-395 min-p in the same sweep: the leading run with p >= min_p * p[0],
    // never empty. Every thread derives p[0] itself, so no barrier separates the two.
    const float thr = __fmul_rn(rc.min_p, __fdiv_rn(e_first, sum));
    {
        uint32_t first_fail = n;
        for (uint32_t i = threadIdx.x; i < n; i += THREADS) {
            const float pi = __fdiv_rn(probs[i], sum);
            probs[i] = pi;
            if (rc.min_p > 0.0f && !(pi >= thr) && first_fail == n) first_fail = i;
        }
        if (first_fail < n) atomicMin(&S.keep, first_fail);
    }
    cta_sync();
    PHASE(10);
    if (threadIdx.x == 0) {
        const uint32_t keep_minp = max(S.keep, 1u);
        // every window entry passed min-p and more entries follow: whether those pass is only certain
        // when the threshold is at least 2^-24 of the leader
        const bool unknown_tail = rc.min_p > 0.0f && truncated && keep_minp == n && rc.min_p < 5.9604644775390625e-08f;
        const bool open_tail = truncated && keep_minp == n && !(rc.min_p > 0.0f);  // kept set continues past the window
        if (rc.min_p > 0.0f) S.f_thr = thr;
        uint32_t keep = keep_minp;
        float total = 0.0f;
        bool reached = false;
        {
            const uint32_t at = tail_cumulative(probs, keep_minp, rc.top_p, &total);
            if (rc.top_p < 1.0f && at < keep_minp) {
                keep = at + 1u;  // the first index that reaches top_p
                reached = true;
            }
        }
        // entries past the window add less than half an ulp to `cum`/`total`, so both are final
        const bool tail_kept = open_tail && !reached;
        const float u = S.u_pre_valid ? S.u_pre : row_uniform(P, b);
        float r = __fmul_rn(u, total);  // :412
        S.f_total = total;
        S.f_u = u;
        S.f_r = r;
        uint32_t flags = LLM_CUDA_ROW_DRAW_CONSUMED;
        uint32_t token = 0u;
        const uint32_t at = tail_walk(probs, keep, r);
        const bool found = at < keep;
        if (found) token = cand_i[at];
        if (!found) {
            if (tail_kept || unknown_tail) {
                flags = ROW_NEEDS_FULL;  // the walk continues into entries the window dropped
            } else {
                token = cand_i[keep - 1u];  // :419
                flags |= LLM_CUDA_ROW_FALLBACK_LAST;
            }
        } else if (unknown_tail) {
            flags = ROW_NEEDS_FULL;
        }
        S.token = token;
        S.out_flags = flags;
        S.keep = keep;
        S.kept_n = tail_kept ? k_total : keep;
    }
    cta_sync();
}

// Programmatic dependent launch. Both are no-ops for a grid launched the ordinary way. A grid that
// was allowed to start before its predecessor on the stream finished must pass the wait before it
// writes global memory or touches scratch the two grids share.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Writes the row's results. `listed` = how many kept entries cand/probs hold.
__device__ __forceinline__ void write_row_outputs(const KParams& P, uint32_t b, uint32_t extra_flags, const Shared& S,
                                                  float mx, const uint32_t* cand_i, const float* probs, uint32_t listed) {
    const uint32_t flags = S.out_flags | extra_flags;
    grid_dependency_wait();
    if (threadIdx.x == 0) {
        P.tokens[b] = S.token;
        if (P.row_flags) P.row_flags[b] = flags;
        if (P.kept_count) P.kept_count[b] = S.kept_n;
        if (P.row_stats) {
            float* st = P.row_stats + (size_t)b * LLM_CUDA_ROW_STATS;
            st[0] = mx;
            st[1] = S.f_sum;
            st[2] = S.f_total;
            st[3] = S.f_u;
            st[4] = S.f_thr;
            st[5] = S.f_r;
        }
    }
    if (P.kept_cap && (flags & LLM_CUDA_ROW_DRAW_CONSUMED)) {
        const uint32_t m = min(listed, P.kept_cap);
        for (uint32_t i = threadIdx.x; i < m; i += THREADS) {
            if (P.kept_ids) P.kept_ids[(size_t)b * P.kept_cap + i] = cand_i[i];
            if (P.kept_probs) P.kept_probs[(size_t)b * P.kept_cap + i] = probs[i];
        }
    }
}

}  // namespace llmc
