// stream_select_kernel: the eight variants for bf16 logits, mask / penalty tables (four row modes x two ring stage sizes), with
// their configure / launch functions. One of four such translation units, compiled side by side.
#define LLMC_KERNELS_ONLY
#define LLMC_STREAM_ELEM uint16_t
#define LLMC_STREAM_BITS true
#define LLMC_STREAM_TAG bf16_tables
#include "sampler_kernels.cu"
