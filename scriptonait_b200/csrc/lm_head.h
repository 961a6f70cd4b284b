// Host-visible declarations of the fused LM head -> sampler kernels (lm_head.cu).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace llmc {

constexpr uint32_t LM_PHASE_PROBE = 0u;  // every probe_every-th vocabulary tile; logits go to the probe buffer
constexpr uint32_t LM_PHASE_MAIN = 1u;   // the other tiles; logits at or above the row's threshold become candidates
constexpr uint32_t LM_PHASE_ALL = 2u;    // every tile, nothing selected (only useful with logits_out)

struct LmParams {
    uint32_t vocab, batch, n_pad;    // n_pad: batch rounded up to a multiple of 16 (the N of the tensor-core instruction)
    uint32_t k_chunks;               // hidden_dim / 64, rounded up
    uint32_t phase, probe_every;
    uint32_t n_items;                // vocabulary tiles this launch works through
    uint32_t stages;                 // ring stages (as many as shared memory holds, up to 8)
    uint32_t tmem_cols;              // tensor-memory columns this CTA allocates: two accumulators of tmem_cols / 2
    uint32_t ctas_per_sm;            // 2 when two CTAs' shared memory and tensor memory fit on an SM, else 1
    float temperature;
    float* thr;                      // [batch] per-row threshold (written by the probe step, read by the main step)
    float* probe_out;                // [batch, probe_cols]
    uint32_t probe_cols;
    float* cand_q;                   // [batch, cand_cap] logit / T
    uint32_t* cand_i;                // [batch, cand_cap] vocabulary id
    uint32_t* cand_count;            // [batch]
    uint32_t cand_cap;
    float* logits_out;               // optional [batch, vocab]: testing aid, the logits themselves
    uint32_t* device_errors;
};

uint32_t lm_head_stages(uint32_t n_pad, size_t max_dyn_smem);
size_t lm_head_smem_bytes(uint32_t n_pad, uint32_t stages);
cudaError_t lm_head_configure(size_t max_dyn_smem);
// also zeroes cand_count[0 .. n_pad) (NULL to skip)
cudaError_t launch_rmsnorm_bf16(const float* x, const float* gain, float eps, uint32_t batch, uint32_t n_pad, uint32_t dim, void* y,
                                uint32_t* cand_count, cudaStream_t stream);
// 0, -1 (no tensor-map encoder / encoding failed) or -3 (launch failed, *cuda_error says why)
int launch_lm_head(const LmParams& P, const void* embed, const void* x_norm, uint32_t hidden, uint32_t sm_count, cudaStream_t stream,
                   cudaError_t* cuda_error);
cudaError_t launch_probe_threshold(const LmParams& P, uint32_t rank, bool exact, cudaStream_t stream);

}  // namespace llmc
