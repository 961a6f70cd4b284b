// llm_cuda.hpp - C++ host-side mirror of the reference's sampler interface over the C ABI
// of llm_cuda.h. Header only; link against libllm_cuda.so.
//
// The reference is Rust and no Rust toolchain was available where this was written, so the
// host layer above the C ABI is C++ with the reference's names, argument meaning and error
// behaviour:
//   SamplingConfig   crates/llm-core/src/generate.rs:24-95 (same fields, same defaults)
//   Rng              crates/llm-core/src/rng.rs:6-34 (SplitMix64; state word only)
//   sample_with      crates/llm-core/src/generate.rs:325-330
//   sample           crates/llm-core/src/generate.rs:423-433
// Like the reference's functions these never throw for data reasons (degenerate rows return
// a token, generate.rs:375-377,419); a failing CUDA call or a capacity violation raises
// llm_cuda::Error, the one failure mode the CPU reference does not have.
#ifndef LLM_CUDA_HPP
#define LLM_CUDA_HPP

#include <cstdint>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

#include "llm_cuda.h"

namespace llm_cuda {

struct Error : std::runtime_error {
    int32_t code;
    Error(int32_t c, const std::string& what) : std::runtime_error(what), code(c) {}
};

// How a token is picked from a row of logits (generate.rs:24-95).
struct SamplingConfig {
    float temperature = 0.9f;         // <= 0.0 means greedy
    std::size_t top_k = 40;           // 0 disables
    float top_p = 0.95f;              // 1.0 disables; applied after top_k and min_p
    float min_p = 0.0f;               // 0.0 disables; applied after top_k, before top_p
    float repetition_penalty = 1.1f;  // 1.0 disables
    std::size_t repetition_window = 128;
    uint64_t seed = 0;
    std::optional<std::vector<bool>> allowed;  // one flag per id; nullopt allows everything
};

// SplitMix64 (rng.rs:6-34).
class Rng {
  public:
    static Rng seed_from_u64(uint64_t seed) { return Rng(seed); }
    uint64_t next_u64() {
        state_ += 0x9E3779B97F4A7C15ull;
        uint64_t z = state_;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    }
    float next_f32() { return static_cast<float>(next_u64() >> 40) / static_cast<float>(1u << 24); }
    uint64_t& state() { return state_; }

  private:
    explicit Rng(uint64_t s) : state_(s) {}
    uint64_t state_;
};

// Owns one llm_cuda_sampler handle (one GPU, one stream at a time).
class Sampler {
  public:
    explicit Sampler(int device = 0, uint32_t max_batch = 1024, uint32_t max_vocab = 262144, uint32_t max_history = 1024,
                     uint32_t max_top_k = 1024) {
        const int32_t rc = llm_cuda_sampler_create(device, max_batch, max_vocab, max_history, max_top_k, &h_);
        if (rc != LLM_CUDA_OK) throw Error(rc, llm_cuda_last_error(nullptr));
    }
    ~Sampler() { llm_cuda_sampler_destroy(h_); }
    Sampler(const Sampler&) = delete;
    Sampler& operator=(const Sampler&) = delete;

    llm_cuda_sampler* handle() { return h_; }

    // sample_with(logits, sampling, recent, rng) -> token id (generate.rs:325-330).
    uint32_t sample_with(const std::vector<float>& logits, const SamplingConfig& sampling, const std::vector<uint32_t>& recent,
                         Rng& rng) {
        llm_cuda_sampling_config c;
        llm_cuda_sampling_config_default(&c);
        c.temperature = sampling.temperature;
        c.top_k = static_cast<uint32_t>(sampling.top_k);
        c.top_p = sampling.top_p;
        c.min_p = sampling.min_p;
        c.repetition_penalty = sampling.repetition_penalty;
        c.repetition_window = static_cast<uint32_t>(sampling.repetition_window);
        c.seed = sampling.seed;
        std::vector<uint8_t> mask;
        if (sampling.allowed) {
            mask.assign(sampling.allowed->begin(), sampling.allowed->end());
            c.allowed = mask.data();
            c.allowed_len = static_cast<uint32_t>(mask.size());
        }
        uint32_t token = 0;
        check(llm_cuda_sample_with(h_, logits.data(), static_cast<uint32_t>(logits.size()), &c,
                                   recent.empty() ? nullptr : recent.data(), static_cast<uint32_t>(recent.size()),
                                   &rng.state(), &token));
        return token;
    }

    // sample(logits, temperature, rng) (generate.rs:423-433).
    uint32_t sample(const std::vector<float>& logits, float temperature, Rng& rng) {
        uint32_t token = 0;
        check(llm_cuda_sample(h_, logits.data(), static_cast<uint32_t>(logits.size()), temperature, &rng.state(), &token));
        return token;
    }

    // Batched, device-resident call; see llm_cuda_sample_args.
    void sample_batch(llm_cuda_sample_args& args) {
        args.struct_size = sizeof(args);
        check(llm_cuda_sample_batch(h_, &args));
    }

    // llm_core::ops::cross_entropy over device pointers (crates/llm-core/src/ops/loss.rs:20-45): per-row loss terms
    // and, unless d_logits is null, the gradient already divided by `rows`; see llm_cuda_cross_entropy.
    void cross_entropy(const float* logits, uint32_t rows, uint32_t vocab, const uint32_t* targets, float* row_loss,
                       float* d_logits = nullptr, uint32_t row_stride_elems = 0, void* stream = nullptr) {
        check(llm_cuda_cross_entropy(h_, logits, rows, vocab, row_stride_elems, targets, row_loss, d_logits, stream));
    }

  private:
    void check(int32_t rc) {
        if (rc != LLM_CUDA_OK) throw Error(rc, llm_cuda_last_error(h_));
    }
    llm_cuda_sampler* h_ = nullptr;
};

}  // namespace llm_cuda

#endif  // LLM_CUDA_HPP
