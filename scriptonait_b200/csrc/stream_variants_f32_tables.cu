// stream_select_kernel: the eight variants for f32 logits, mask / penalty tables (four row modes x two ring stage sizes), with
// their configure / launch functions. One of four such translation units, compiled side by side.
#define LLMC_KERNELS_ONLY
#define LLMC_STREAM_ELEM float
#define LLMC_STREAM_BITS true
#define LLMC_STREAM_TAG f32_tables
#include "sampler_kernels.cu"
