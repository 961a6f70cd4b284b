"""scriptonait_b200: the B200-native token sampler behind scriptonait's sampler interface.

One path of biffjezos/scriptonait - `sample_with` (crates/llm-core/src/generate.rs:325-420) -
as hand-written sm_100a CUDA kernels behind the C ABI of include/llm_cuda.h, with this
package as the host-side mirror of the reference's `SamplingConfig` / `sample_with` /
`sample` / `Rng`. Importing the package needs no GPU; creating a `Sampler` does, and
fails loudly without one (there is no CPU fallback).
"""
from .sampler import (EOS, LlmCudaError, Rng, SampleResult, Sampler, SamplingConfig, default_sampler, sample,
                      sample_with)
from . import _native as native

__all__ = ["EOS", "LlmCudaError", "Rng", "SampleResult", "Sampler", "SamplingConfig", "default_sampler", "sample",
           "sample_with", "native"]
