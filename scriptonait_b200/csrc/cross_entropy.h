// Cross-entropy row kernel (launch wrapper); see cross_entropy.cu.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace llmc {

// row_loss[t] = log(sum_v exp(x[t, v] - max_t)) + max_t - x[t, targets[t]];
// d_logits[t, v] (optional) = (softmax(x[t, :])[v] - (v == targets[t])) / rows. Device pointers; d_logits has the
// logits' row stride, and its base the logits' alignment modulo 16 bytes.
cudaError_t launch_cross_entropy_rows(const float* logits, uint32_t rows, uint32_t vocab, size_t row_stride, const uint32_t* targets,
                                      float* row_loss, float* d_logits, cudaStream_t stream);

}  // namespace llmc
