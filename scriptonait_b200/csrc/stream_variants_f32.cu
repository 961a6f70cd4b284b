// stream_select_kernel: the eight variants for f32 logits, no mask / penalty tables (four row modes x two ring stage sizes), with
// their configure / launch functions. One of four such translation units, compiled side by side.
#define LLMC_KERNELS_ONLY
#define LLMC_STREAM_ELEM float
#define LLMC_STREAM_BITS false
#define LLMC_STREAM_TAG f32
#include "sampler_kernels.cu"
