// Fused tied LM head -> sampler for a decode batch (sm_100a): final RMSNorm, the hidden x vocab
// contraction on the 5th-generation tensor cores, and a selection epilogue that keeps only the logits
// that can reach the top-k - the [batch, vocab] logits matrix is never written.
//
// What it replaces in the reference: the last three dispatches of GpuModel::decode_step
// (crates/llm-gpu/src/model.rs:481-490: dispatch_rmsnorm, dispatch_linear(..., vocab) over the tied
// embedding, and the copy + read_back of vocab*4 bytes per token), the WGSL linear kernel
// (crates/llm-gpu/src/shaders/linear.wgsl) and the CPU sample_with call that follows
// (crates/wasm-app/src/inference.rs:325-347).
//
// Pipeline (one stream, no host round trip):
//   rmsnorm_bf16_kernel       y = x * rsqrt(mean(x^2) + eps) * gain (ops/activation.rs:5-19), narrowed to bf16
//   lm_head_kernel, probe     every PROBE_EVERY-th tile of 128 vocabulary rows: logits of that eighth of the
//                             vocabulary go to a small probe buffer
//   probe_threshold_kernel    per row: the r-th largest probe logit becomes the row's threshold (r chosen so
//                             that about 3-4 k logits of the whole row reach it); probe logits at or above
//                             it become candidates
//   lm_head_kernel, main      the other tiles: the epilogue reads the accumulators out of tensor memory and
//                             appends (logit / T, vocabulary id) for every logit at or above the threshold
//   merge_draw_kernel         the sampler's own merge + ordered tail over the candidate lists; a row whose
//                             candidates number fewer than top_k (threshold too high) or more than the list
//                             holds is undecided - it is reported, never guessed
// Exact by construction: every logit >= threshold is captured, so when at least top_k were captured the
// top_k largest are among them, whatever the threshold was.
//
// lm_head_kernel: 192 threads. Warp 0 issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of a
// 128 x 64 tile of the embedding and the batch x 64 tile of the hidden states into a ring of 4-8 stages; warp 1
// issues tcgen05.mma (M = 128 vocabulary rows, N = padded batch, K = 16 per instruction) into one of two
// accumulators in tensor memory and commits to mbarriers; warps 2-5 are the epilogue (tcgen05.ld). Every
// wait is bounded: a wait that runs out sets LLM_CUDA_STATUS_COPY_TIMEOUT, all roles leave their loops,
// tensor memory is freed and the kernel returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/llm_cuda.h"
#include "lm_head.h"

namespace llmc {

namespace {

constexpr int LM_THREADS = 192;
constexpr int TILE_M = 128;            // vocabulary rows per tile = lanes of tensor memory
constexpr int KCHUNK = 64;             // bf16 elements per 128-byte swizzled shared-memory row
constexpr int LM_MAX_STAGES = 8;      // ring stages: as many as fit in shared memory, up to this
constexpr uint32_t A_STAGE_BYTES = TILE_M * KCHUNK * 2;  // 16 KB
constexpr uint32_t LM_WAIT_LIMIT = 1u << 16;

__device__ __forceinline__ uint32_t saddr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(saddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(saddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(saddr(bar)) : "memory");
}
__device__ __forceinline__ bool bar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(saddr(bar)), "r"(parity), "r"(20000u)
        : "memory");
    return ok != 0u;
}
// Bounded wait that also gives up as soon as another role has raised `abort`.
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort) {
    for (uint32_t i = 0; i < LM_WAIT_LIMIT; ++i) {
        if (bar_try_wait(bar, parity)) return true;
        if (*abort) return false;
        __nanosleep(32);
    }
    *abort = 1u;
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int32_t c0, int32_t c1, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     saddr(smem_dst)),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(saddr(bar))
                 : "memory");
}
// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzle: start
// address and strides in 16-byte units, 1024 bytes between groups of eight rows, descriptor version 1.
__device__ __forceinline__ uint64_t umma_desc_k128(uint32_t smem_byte_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_byte_addr >> 4) & 0x3fffu);  // start address
    d |= (uint64_t)1u << 16;                           // leading byte offset (not used by swizzled K-major layouts)
    d |= (uint64_t)(1024u >> 4) << 32;                 // stride byte offset: eight rows of 128 bytes
    d |= (uint64_t)1u << 46;                           // descriptor version (Blackwell)
    d |= (uint64_t)2u << 61;                           // layout type: 128-byte swizzle
    return d;
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(saddr(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// 32 consecutive accumulator columns of this thread's lane of tensor memory.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, "
        "%18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// generate.rs:357-359: a true IEEE division per element; T == 1 is the identity
__device__ __forceinline__ float temper_lm(float x, float T) { return (T == 1.0f) ? x : __fdiv_rn(x, T); }

// The vocabulary tile the i-th work item of a phase stands for.
__device__ __forceinline__ uint32_t tile_of(uint32_t phase, uint32_t i, uint32_t probe_every) {
    if (phase == LM_PHASE_PROBE) return i * probe_every;
    if (phase == LM_PHASE_MAIN) return i + i / (probe_every - 1u) + 1u;  // the tiles the probe skipped
    return i;
}

}  // namespace

// Programmatic dependent launch (no-ops for a grid launched the ordinary way). The step's kernels are launched
// so that each may start while its predecessor is still running; a kernel executes the wait before it first
// touches anything its predecessor writes, and allows its own successor to start only after that wait, so
// that when a kernel starts early, everything two or more launches back is complete.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__global__ void __launch_bounds__(LM_THREADS, 2)
lm_head_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const LmParams P) {
    extern __shared__ unsigned char lm_dyn[];
    __shared__ __align__(8) uint64_t full_bar[LM_MAX_STAGES], empty_bar[LM_MAX_STAGES], acc_full[2], acc_empty[2], drain_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile uint32_t abort_flag;
    __shared__ float thr_s[256];

    // 1024-byte alignment: the swizzle pattern repeats every eight 128-byte rows
    unsigned char* base = lm_dyn + ((1024u - (saddr(lm_dyn) & 1023u)) & 1023u);
    const uint32_t n_pad = P.n_pad;
    const uint32_t b_stage_bytes = n_pad * KCHUNK * 2u;
    unsigned char* a_tiles = base;
    const uint32_t LM_STAGES = P.stages;
    unsigned char* b_tiles = base + (size_t)LM_STAGES * A_STAGE_BYTES;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t n_items = P.n_items;
    const uint32_t k_chunks = P.k_chunks;

    if (tid == 0) {
        for (uint32_t s = 0; s < LM_STAGES; ++s) {
            bar_init(&full_bar[s], 1u);
            bar_init(&empty_bar[s], 1u);
        }
        for (int j = 0; j < 2; ++j) {
            bar_init(&acc_full[j], 1u);
            bar_init(&acc_empty[j], 4u);  // one arrival per epilogue warp
        }
        bar_init(&drain_bar, 1u);
        abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // tensor memory: both accumulators, allocated by one whole warp, which also frees it
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(&tmem_base_slot)), "r"(P.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        // ---- TMA producer
        if (lane == 0) {
            // the probe pass follows the kernel that writes the normalised hidden states; the main pass follows the
            // threshold kernel, which its loads and tensor-core work do not depend on: they start at once
            if (P.phase != LM_PHASE_MAIN) pdl_wait();
            uint32_t g = 0;  // chunks issued
            for (uint32_t i = blockIdx.x; i < n_items && !abort_flag; i += gridDim.x) {
                const uint32_t tile = tile_of(P.phase, i, P.probe_every);
                for (uint32_t kc = 0; kc < k_chunks; ++kc, ++g) {
                    const uint32_t s = g % LM_STAGES;
                    if (g >= LM_STAGES && !bar_wait(&empty_bar[s], ((g / LM_STAGES) - 1u) & 1u, &abort_flag)) break;
                    bar_expect_tx(&full_bar[s], A_STAGE_BYTES + b_stage_bytes);
                    tma_load_2d(a_tiles + (size_t)s * A_STAGE_BYTES, &map_w, (int32_t)(kc * KCHUNK), (int32_t)(tile * TILE_M), &full_bar[s]);
                    tma_load_2d(b_tiles + (size_t)s * b_stage_bytes, &map_x, (int32_t)(kc * KCHUNK), 0, &full_bar[s]);
                }
            }
        }
        __syncwarp();  // the warp is whole again before the CTA-wide barrier below
    } else if (warp == 1) {
        // ---- MMA issuer
        if (lane == 0) {
            // instruction descriptor: f32 accumulate, bf16 x bf16, both operands K-major, N = n_pad, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((n_pad >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);
            uint32_t g = 0, it = 0;
            for (uint32_t i = blockIdx.x; i < n_items && !abort_flag; i += gridDim.x, ++it) {
                const uint32_t j = it & 1u;
                if (it >= 2u && !bar_wait(&acc_empty[j], ((it >> 1) - 1u) & 1u, &abort_flag)) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + j * (P.tmem_cols >> 1);
                bool ok = true;
                for (uint32_t kc = 0; kc < k_chunks; ++kc, ++g) {
                    const uint32_t s = g % LM_STAGES;
                    if (!bar_wait(&full_bar[s], (g / LM_STAGES) & 1u, &abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = saddr(a_tiles + (size_t)s * A_STAGE_BYTES);
                    const uint32_t b_addr = saddr(b_tiles + (size_t)s * b_stage_bytes);
#pragma unroll
                    for (uint32_t k = 0; k < (uint32_t)KCHUNK / 16u; ++k)  // 16 bf16 = 32 bytes per instruction along K
                        umma_bf16(tmem_d, umma_desc_k128(a_addr + k * 32u), umma_desc_k128(b_addr + k * 32u), idesc, (kc | k) ? 1u : 0u);
                    umma_commit(&empty_bar[s]);  // the stage is free once these instructions have read it
                }
                if (!ok) break;
                umma_commit(&acc_full[j]);  // the accumulator is complete once they have all retired
            }
            // nothing of this CTA's may still be running on the tensor cores when tensor memory is freed
            umma_commit(&drain_bar);
            (void)bar_wait(&drain_bar, 0u, &abort_flag);
        }
        __syncwarp();
    } else {
        // ---- epilogue: warp w reads lanes 32 * (w % 4) .. + 31 of tensor memory (its quarter)
        const uint32_t quarter = warp & 3u;
        const uint32_t row_in_tile = quarter * 32u + lane;
        // the thresholds (main pass) come from the preceding kernel, and what this one writes may still be read by it
        pdl_wait();
        for (uint32_t i = tid - 64u; i < 256u; i += 128u) thr_s[i] = (P.thr && i < P.batch) ? P.thr[i] : __uint_as_float(0x7f800000u);
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
        if (tid == 64u) pdl_launch_dependents();
        uint32_t it = 0;
        for (uint32_t i = blockIdx.x; i < n_items && !abort_flag; i += gridDim.x, ++it) {
            const uint32_t j = it & 1u;
            const uint32_t tile = tile_of(P.phase, i, P.probe_every);
            if (!bar_wait(&acc_full[j], (it >> 1) & 1u, &abort_flag)) break;
            tc_fence_after();
            const uint32_t v = tile * TILE_M + row_in_tile;  // vocabulary id of this thread's accumulator row
            const bool v_ok = v < P.vocab;
            for (uint32_t c0 = 0; c0 < n_pad; c0 += 32u) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((quarter * 32u) << 16) + j * (P.tmem_cols >> 1) + c0, r);
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const uint32_t b = c0 + (uint32_t)c;
                    if (b >= P.batch) continue;
                    const float x = __uint_as_float(r[c]);
                    if (P.logits_out && v_ok) P.logits_out[(size_t)b * P.vocab + v] = x;
                    if (P.phase == LM_PHASE_PROBE) {
                        P.probe_out[(size_t)b * P.probe_cols + (size_t)i * TILE_M + row_in_tile] = v_ok ? x : __uint_as_float(0xff800000u);
                    } else if (P.phase == LM_PHASE_MAIN && v_ok && x >= thr_s[b]) {
                        const uint32_t slot = atomicAdd(&P.cand_count[b], 1u);
                        if (slot < P.cand_cap) {
                            P.cand_q[(size_t)b * P.cand_cap + slot] = temper_lm(x, P.temperature);
                            P.cand_i[(size_t)b * P.cand_cap + slot] = v;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) bar_arrive(&acc_empty[j]);
        }
    }
    __syncthreads();
    if (tid == 0 && abort_flag && P.device_errors) atomicOr(P.device_errors, LLM_CUDA_STATUS_COPY_TIMEOUT);
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(P.tmem_cols) : "memory");
    }
}

// y[b, :] = bf16(x[b, :] * rsqrt(mean(x[b, :]^2) + eps) * gain) (crates/llm-core/src/ops/activation.rs:5-19), or
// bf16(x) when gain is NULL; rows batch .. n_pad - 1 of y are zero. One CTA per row of y.
__global__ void rmsnorm_bf16_kernel(const float* x, const float* gain, float eps, uint32_t batch, uint32_t dim, __nv_bfloat16* y,
                                    uint32_t* cand_count) {
    const uint32_t b = blockIdx.x;
    pdl_launch_dependents();  // launched the ordinary way itself: whatever precedes it is complete
    if (threadIdx.x == 0 && cand_count) cand_count[b] = 0u;  // the step's candidate lists start empty
    __shared__ float part[32];
    __shared__ float inv_s;
    if (b >= batch) {
        for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) y[(size_t)b * dim + i] = __float2bfloat16(0.0f);
        return;
    }
    const float* row = x + (size_t)b * dim;
    const uint32_t dim4 = dim / 4u;  // dim is a multiple of 8: whole 16-byte vectors
    const float4* row4 = reinterpret_cast<const float4*>(row);
    float inv = 1.0f;
    if (gain) {
        float ss = 0.0f;
#pragma unroll 4
        for (uint32_t i = threadIdx.x; i < dim4; i += blockDim.x) {
            const float4 v = __ldg(&row4[i]);
            ss = fmaf(v.x, v.x, ss);
            ss = fmaf(v.y, v.y, ss);
            ss = fmaf(v.z, v.z, ss);
            ss = fmaf(v.w, v.w, ss);
        }
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if ((threadIdx.x & 31u) == 0) part[threadIdx.x >> 5] = ss;
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = 0.0f;
            for (uint32_t w = 0; w < (blockDim.x + 31u) / 32u; ++w) t += part[w];
            inv_s = 1.0f / sqrtf(t / (float)dim + eps);
        }
        __syncthreads();
        inv = inv_s;
    }
    const float4* gain4 = reinterpret_cast<const float4*>(gain);
    uint2* y2 = reinterpret_cast<uint2*>(y + (size_t)b * dim);
#pragma unroll 4
    for (uint32_t i = threadIdx.x; i < dim4; i += blockDim.x) {
        float4 v = __ldg(&row4[i]);
        if (gain) {
            const float4 g = __ldg(&gain4[i]);
            v.x = v.x * inv * g.x;
            v.y = v.y * inv * g.y;
            v.z = v.z * inv * g.z;
            v.w = v.w * inv * g.w;
        }
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        y2[i] = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    }
}

namespace {
__device__ __forceinline__ uint32_t lm_okey(float x) {
    x = __fadd_rn(x, 0.0f);
    const uint32_t b = __float_as_uint(x);
    return b ^ ((uint32_t)((int32_t)b >> 31) | 0x80000000u);
}
__device__ __forceinline__ float lm_okey_to_float(uint32_t k) {
    const uint32_t b = (k & 0x80000000u) ? (k ^ 0x80000000u) : ~k;
    return __uint_as_float(b);
}
}  // namespace

// Per row: a threshold near the `rank`-th largest of the row's probe logits - lowered by four floats when
// T != 1, since neighbouring floats can share a quotient x / T - and the probe logits at or above it become
// the row's first candidates. Any threshold keeps the result exact (the merge step checks that enough
// logits reached it); it only has to land where a few times top_k logits of the row pass. `exact` (small
// vocabularies, probed whole): a radix select over ordered keys, 8 bits a pass. Otherwise 256 groups of
// four threads each take the maximum of their share of the probe, and the rank-th largest of those 256
// maxima is used: at least `rank` probe logits reach it and, the top values nearly always sitting with
// different groups, hardly more. One CTA of 1024 threads per row.
__global__ void __launch_bounds__(1024) probe_threshold_kernel(const LmParams P, uint32_t rank, uint32_t exact) {
    const uint32_t b = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;  // 1024 threads: a row's probe is one round of 16-byte loads
    pdl_wait();               // the probe pass's logits
    pdl_launch_dependents();  // the main pass may set itself up and start its contraction meanwhile
    __shared__ uint32_t hist[256];
    __shared__ uint32_t sel_digit, sel_need;
    const float* row = P.probe_out + (size_t)b * P.probe_cols;
    const float4* row4 = reinterpret_cast<const float4*>(row);  // probe rows are whole tiles of 128 floats
    const uint32_t n = P.probe_cols;
    uint32_t need = rank < 1u ? 1u : rank;
    uint32_t prefix = 0u;
    if (!exact) {
        // 256 groups of four threads: the rank-th largest of the groups' maxima
        uint32_t best = 0u;  // below every ordered key of a float
#pragma unroll 4
        for (uint32_t i = tid; i < n / 4u; i += nt) {
            const float4 v = __ldg(&row4[i]);
            if (v.x == v.x) best = max(best, lm_okey(v.x));
            if (v.y == v.y) best = max(best, lm_okey(v.y));
            if (v.z == v.z) best = max(best, lm_okey(v.z));
            if (v.w == v.w) best = max(best, lm_okey(v.w));
        }
        best = max(best, __shfl_xor_sync(0xffffffffu, best, 1));
        best = max(best, __shfl_xor_sync(0xffffffffu, best, 2));
        if ((tid & 3u) == 0u) hist[tid >> 2] = best;
        __syncthreads();
        if (tid < 256u) {
            const uint32_t mine = hist[tid];
            uint32_t above = 0u;  // maxima that come before this group's (ties broken by group number)
            for (uint32_t j = 0; j < 256u; ++j) {
                const uint32_t o = hist[j];
                above += (o > mine || (o == mine && j < tid)) ? 1u : 0u;
            }
            if (above == min(need, 256u) - 1u) sel_digit = mine;
        }
        __syncthreads();
        prefix = sel_digit;
    } else
    for (int pass = 0; pass < 4; ++pass) {
        const int sh = 24 - 8 * pass;
        if (tid < 256u) hist[tid] = 0u;
        __syncthreads();
        for (uint32_t i = tid; i < n; i += nt) {
            const float x = row[i];
            if (x != x) continue;
            const uint32_t key = lm_okey(x);
            if (pass == 0 || (key >> (sh + 8)) == prefix) atomicAdd(&hist[(key >> sh) & 255u], 1u);
        }
        __syncthreads();
        if (tid == 0) {
            uint32_t above = 0u, d = 255u;
            for (;; --d) {
                if (above + hist[d] >= need || d == 0u) break;
                above += hist[d];
            }
            sel_digit = d;
            sel_need = need > above ? need - above : 1u;
        }
        __syncthreads();
        prefix = (prefix << 8) | sel_digit;
        need = sel_need;
        __syncthreads();
    }
    uint32_t key = prefix;  // ordered key of (about) the rank-th largest probe logit
    const uint32_t lowest = 0x007fffffu;  // ordered key of -inf
    if (P.temperature != 1.0f) key = key > lowest + 4u ? key - 4u : lowest;
    if (key < lowest) key = lowest;
    const float thr = lm_okey_to_float(key);
    if (tid == 0) P.thr[b] = thr;
#pragma unroll 4
    for (uint32_t i4 = tid; i4 < n / 4u; i4 += nt) {
        const float4 q = __ldg(&row4[i4]);
        const float xs[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const uint32_t i = i4 * 4u + (uint32_t)e;
            const uint32_t v = (i / TILE_M) * P.probe_every * TILE_M + (i % TILE_M);
            if (v < P.vocab && xs[e] >= thr) {
                const uint32_t slot = atomicAdd(&P.cand_count[b], 1u);
                if (slot < P.cand_cap) {
                    P.cand_q[(size_t)b * P.cand_cap + slot] = temper_lm(xs[e], P.temperature);
                    P.cand_i[(size_t)b * P.cand_cap + slot] = v;
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// A [rows, cols] row-major bf16 matrix as a TMA tensor map whose box is box_rows x 64 elements
// (128 bytes per row, 128-byte swizzle); reads past the matrix give zeros.
static int make_map(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return -1;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2u};
    const cuuint32_t box[2] = {(cuuint32_t)KCHUNK, box_rows};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2u, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -2;
}

uint32_t lm_head_stages(uint32_t n_pad, size_t max_dyn_smem) {
    const size_t per_stage = A_STAGE_BYTES + (size_t)n_pad * KCHUNK * 2u;
    size_t n = (max_dyn_smem - 1024u) / per_stage;
    if (n > (size_t)LM_MAX_STAGES) n = LM_MAX_STAGES;
    return (uint32_t)n;
}

size_t lm_head_smem_bytes(uint32_t n_pad, uint32_t stages) { return (size_t)stages * (A_STAGE_BYTES + (size_t)n_pad * KCHUNK * 2u) + 1024u; }

// A launch that may start before its predecessor on the stream has finished (programmatic stream serialization);
// the kernels place their own waits.
template <class... Params, class... Args>
static cudaError_t launch_after(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, Params(args)...);
}

cudaError_t lm_head_configure(size_t max_dyn_smem) {
    return cudaFuncSetAttribute(lm_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)max_dyn_smem);
}

cudaError_t launch_rmsnorm_bf16(const float* x, const float* gain, float eps, uint32_t batch, uint32_t n_pad, uint32_t dim, void* y,
                                uint32_t* cand_count, cudaStream_t stream) {
    rmsnorm_bf16_kernel<<<n_pad, 256, 0, stream>>>(x, gain, eps, batch, dim, static_cast<__nv_bfloat16*>(y), cand_count);
    return cudaGetLastError();
}

int launch_lm_head(const LmParams& P, const void* embed, const void* x_norm, uint32_t hidden, uint32_t sm_count, cudaStream_t stream,
                   cudaError_t* cuda_error) {
    *cuda_error = cudaSuccess;
    if (P.n_items == 0u) return 0;
    CUtensorMap map_w, map_x;
    if (make_map(&map_w, embed, P.vocab, hidden, TILE_M) != 0) return -1;
    if (make_map(&map_x, x_norm, P.n_pad, hidden, P.n_pad) != 0) return -1;
    // small batches leave room for two CTAs per SM (each with half of tensor memory): more loads in flight
    const uint32_t slots = sm_count * P.ctas_per_sm;
    const uint32_t grid = P.n_items < slots ? P.n_items : slots;
    *cuda_error = launch_after(lm_head_kernel, dim3(grid), dim3(LM_THREADS), lm_head_smem_bytes(P.n_pad, P.stages), stream, map_w, map_x, P);
    return *cuda_error == cudaSuccess ? 0 : -3;
}

cudaError_t launch_probe_threshold(const LmParams& P, uint32_t rank, bool exact, cudaStream_t stream) {
    return launch_after(probe_threshold_kernel, dim3(P.batch), dim3(1024), 0, stream, P, rank, exact ? 1u : 0u);
}

}  // namespace llmc
