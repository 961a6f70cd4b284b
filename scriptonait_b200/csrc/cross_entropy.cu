// Cross-entropy over the rows of a logits matrix, with the gradient with respect to the logits: the row
// reduction that the training step shares with the sampler's softmax. Replaces
// crates/llm-gpu/src/shaders/cross_entropy.wgsl:29-88 (one workgroup per row: maximum, sum of exponentials,
// loss, gradient) and is checked against the CPU statement of the same arithmetic,
// crates/llm-core/src/ops/loss.rs:20-45.
//
// One CTA of 512 threads per row. HBM-bound: a row is read once from memory (maximum and sum of
// exponentials in the same sweep: every thread keeps a running maximum and rescales its sum when the
// maximum rises), read once more from L2 for the gradient, and the gradient is written once: 8 bytes per
// logit of algorithmic traffic. Loads and stores are 16 bytes per thread, eight loads in flight in the first sweep.
#include "cross_entropy.h"

#include <math.h>
#include <stdint.h>

namespace llmc {

namespace {

constexpr int CE_THREADS = 512;

// (m1, s1) and (m2, s2): maximum and sum of exp(x - maximum) of two sets; the pair of their union
__device__ __forceinline__ void ce_merge(float& m, float& s, float m2, float s2) {
    const float mm = fmaxf(m, m2);
    // exp(-inf - -inf) would be NaN: a set that has seen nothing has sum 0 and is skipped
    const float a = (s > 0.0f) ? s * expf(m - mm) : 0.0f;
    const float b = (s2 > 0.0f) ? s2 * expf(m2 - mm) : 0.0f;
    m = mm;
    s = a + b;
}

__device__ __forceinline__ void ce_take(float& m, float& s, float x) {
    if (x > m) {
        s = (s > 0.0f ? s * expf(m - x) : 0.0f) + 1.0f;
        m = x;
    } else if (x > -INFINITY) {  // -inf adds nothing (and -inf minus a maximum of -inf would be NaN)
        s += expf(x - m);
    }
}

__global__ void __launch_bounds__(CE_THREADS) cross_entropy_rows_kernel(const float* __restrict__ logits, uint32_t rows, uint32_t vocab,
                                                                        size_t row_stride, const uint32_t* __restrict__ targets,
                                                                        float* __restrict__ row_loss, float* __restrict__ d_logits,
                                                                        float inv_rows) {
    const uint32_t t = blockIdx.x, tid = threadIdx.x;
    const unsigned lane = tid & 31u, warp = tid >> 5;
    const float* row = logits + (size_t)t * row_stride;
    __shared__ float sh_m[CE_THREADS / 32], sh_s[CE_THREADS / 32];
    __shared__ float sh_max, sh_sum;
    // leading elements up to the first 16-byte boundary, whole vectors, trailing elements
    const uint32_t mis = (uint32_t)((reinterpret_cast<uintptr_t>(row) & 15u) / 4u);
    const uint32_t head = mis ? min(4u - mis, vocab) : 0u;
    const uint32_t nvec = (vocab - head) / 4u;
    const uint32_t tail0 = head + nvec * 4u;
    const float4* rv = reinterpret_cast<const float4*>(row + head);

    float m = -INFINITY, s = 0.0f;
    if (tid < head) ce_take(m, s, row[tid]);
    if (tid < vocab - tail0) ce_take(m, s, row[tail0 + tid]);
    for (uint32_t i0 = tid; i0 < nvec; i0 += 8u * CE_THREADS) {
        float4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t i = i0 + (uint32_t)u * CE_THREADS;
            v[u] = i < nvec ? __ldg(&rv[i]) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            // the vector's own maximum first: one rescaling of the running sum per vector at most
            const float vm = fmaxf(fmaxf(v[u].x, v[u].y), fmaxf(v[u].z, v[u].w));
            if (vm > m) {
                s = (s > 0.0f) ? s * expf(m - vm) : 0.0f;
                m = vm;
            }
            if (vm > -INFINITY) s += expf(v[u].x - m) + expf(v[u].y - m) + expf(v[u].z - m) + expf(v[u].w - m);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
        ce_merge(m, s, m2, s2);
    }
    if (lane == 0) {
        sh_m[warp] = m;
        sh_s[warp] = s;
    }
    __syncthreads();
    if (warp == 0) {
        m = lane < CE_THREADS / 32 ? sh_m[lane] : -INFINITY;
        s = lane < CE_THREADS / 32 ? sh_s[lane] : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
            ce_merge(m, s, m2, s2);
        }
        if (lane == 0) {
            sh_max = m;
            sh_sum = s;
        }
    }
    __syncthreads();
    const float maxv = sh_max, sum = sh_sum;
    const uint32_t tgt = targets[t];
    // loss.rs:33-35; a target outside the vocabulary (the reference panics on it) gives NaN instead of a stray read
    if (tid == 0) row_loss[t] = tgt < vocab ? logf(sum) + maxv - row[tgt] : __uint_as_float(0x7fc00000u);
    if (!d_logits) return;
    // loss.rs:36-40: (softmax - one-hot) / rows; the row comes from L2 this time
    float* drow = d_logits + (size_t)t * row_stride;
    auto grad = [&](float x, uint32_t v) { return (expf(x - maxv) / sum - (v == tgt ? 1.0f : 0.0f)) * inv_rows; };
    if (tid < head) drow[tid] = grad(row[tid], tid);
    if (tid < vocab - tail0) drow[tail0 + tid] = grad(row[tail0 + tid], tail0 + tid);
    float4* dv = reinterpret_cast<float4*>(drow + head);  // same stride and base alignment as the logits: checked by the host
    for (uint32_t i0 = tid; i0 < nvec; i0 += 4u * CE_THREADS) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint32_t i = i0 + (uint32_t)u * CE_THREADS;
            if (i < nvec) v[u] = __ldcg(&rv[i]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint32_t i = i0 + (uint32_t)u * CE_THREADS;
            if (i < nvec) {
                const uint32_t c = head + i * 4u;
                __stcs(&dv[i], make_float4(grad(v[u].x, c), grad(v[u].y, c + 1u), grad(v[u].z, c + 2u), grad(v[u].w, c + 3u)));
            }
        }
    }
}

}  // namespace

cudaError_t launch_cross_entropy_rows(const float* logits, uint32_t rows, uint32_t vocab, size_t row_stride, const uint32_t* targets,
                                      float* row_loss, float* d_logits, cudaStream_t stream) {
    if (rows == 0u) return cudaSuccess;
    cross_entropy_rows_kernel<<<rows, CE_THREADS, 0, stream>>>(logits, rows, vocab, row_stride, targets, row_loss, d_logits,
                                                               1.0f / (float)rows);
    return cudaGetLastError();
}

}  // namespace llmc
