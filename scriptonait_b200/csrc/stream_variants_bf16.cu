// stream_select_kernel: the eight variants for bf16 logits, no mask / penalty tables (four row modes x two ring stage sizes), with
// their configure / launch functions. One of four such translation units, compiled side by side.
#define LLMC_KERNELS_ONLY
#define LLMC_STREAM_ELEM uint16_t
#define LLMC_STREAM_BITS false
#define LLMC_STREAM_TAG bf16
#include "sampler_kernels.cu"
