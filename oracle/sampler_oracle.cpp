// CPU oracle for the token-sampling path of biffjezos/scriptonait.
//
// THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE. Only the test suite, the
// smoke check and the bench's CPU-baseline / reference arms may load it; the
// shipped library never links, imports or calls anything in this file.
//
// It is a line-by-line restatement, in C++17, of the reference's Rust:
//   sample_with        crates/llm-core/src/generate.rs:325-420
//   sample             crates/llm-core/src/generate.rs:423-433
//   SamplingConfig     crates/llm-core/src/generate.rs:24-95 (defaults :82-95)
//   Rng (SplitMix64)   crates/llm-core/src/rng.rs:10-34
//   argmax             crates/llm-core/src/ops/loss.rs:6-16
//   to_bf16/from_bf16  crates/llm-core/src/bf16.rs:11-25
//   EOS = 258          crates/llm-core/src/tokenizer.rs:38
//
// The reference is Rust and no Rust toolchain exists where this was written,
// so the reference itself was never executed against this file. Pinning:
//   * pinned by the reference's own known-answer sampler tests
//     (generate.rs:550-583, :629-692) and RNG/bf16 property tests
//     (rng.rs:48-80, bf16.rs:31-43), restated in tests/test_oracle_reference_cases.py;
//   * PARITY UNPINNED for what those tests do not cover: exact RNG output
//     values (the reference holds no golden values; the constants are checked
//     against an independent big-integer evaluation of rng.rs:16-22), the
//     `allowed` branch, argmax tie/NaN behaviour, duplicate-history
//     compounding, index tie-breaking at the top-k edge, the degenerate-sum
//     return and the post-walk fallback. For those the source lines above are
//     the only authority.
//
// Floating point: every f32 operation of the reference is one rounded `float`
// operation here, in the same order. Build with -ffp-contract=off and without
// -ffast-math so no multiply-add is fused and no sum is reassociated.
//
// exp: the reference calls f32::exp, i.e. the platform libm's expf. Two
// definitions are offered (ORACLE_EXP_*): LIBM calls this host's expf (what a
// native build of the reference would do on this machine); CR rounds the
// double-precision exp to float, which is the correctly rounded result except
// when the double result falls within one double ulp of a float rounding
// boundary. glibc's expf differs from CR by one float ulp in a small fraction
// of arguments, which is why parity against LIBM is stated with a tolerance
// while parity against CR is bit-for-bit.

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <numeric>
#include <thread>
#include <vector>

extern "C" {

enum { ORACLE_EXP_LIBM = 0, ORACLE_EXP_CR = 1 };

// Row flags reported beside the token (same bit meanings as the CUDA library).
enum {
    ORACLE_FLAG_GREEDY = 1u,         // temperature <= 0: argmax returned, no draw consumed
    ORACLE_FLAG_DEGENERATE = 2u,     // sum <= 0 or not finite: order[0] returned, no draw consumed
    ORACLE_FLAG_FALLBACK_LAST = 4u,  // the walk ran off the kept set: last kept id returned
    ORACLE_FLAG_DRAW_CONSUMED = 8u,  // exactly one next_u64 was taken from the RNG
    ORACLE_FLAG_NAN_INPUT = 32u,     // a NaN reached the ordering step (unsupported input)
};

// Mirrors SamplingConfig (generate.rs:24-80) without seed/window, which the
// caller turns into an RNG state and a history slice before sample_with.
typedef struct oracle_sampling_config {
    float temperature;         // <= 0 means greedy
    uint32_t top_k;            // 0 disables
    float top_p;               // 1.0 disables
    float min_p;               // 0.0 disables
    float repetition_penalty;  // 1.0 disables
    const uint8_t* allowed;    // one byte per id (0 = blocked), or NULL for "allow all"
    uint32_t allowed_len;      // ids >= allowed_len count as allowed
    uint32_t eos_id;           // exempt from the allowed mask (258 in the reference)
    uint32_t exp_mode;         // ORACLE_EXP_*
} oracle_sampling_config;

// Per-stage outputs parity is judged on. Any pointer may be NULL.
typedef struct oracle_trace {
    uint32_t* kept_count;  // size of the kept set after top-k, min-p and top-p
    uint32_t* kept_ids;    // first kept_capacity kept ids, most likely first
    float* kept_probs;     // their normalised probabilities (p_i / sum)
    uint32_t kept_capacity;
    float* stats;          // [0]=max [1]=sum [2]=total [3]=u [4]=min-p threshold [5]=r=u*total
    uint32_t* flags;       // ORACLE_FLAG_*
    float* work;           // vocab floats: the row after mask, penalty and temperature
} oracle_trace;

// ---- rng.rs:10-34 -------------------------------------------------------
uint64_t oracle_rng_next_u64(uint64_t* state) {
    *state += 0x9E3779B97F4A7C15ull;  // wrapping add
    uint64_t z = *state;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

float oracle_rng_next_f32(uint64_t* state) {
    // top 24 bits, exact in f32, divided by 2^24 (exact)
    return (float)(oracle_rng_next_u64(state) >> 40) / (float)(1u << 24);
}

// ---- ops/loss.rs:6-16 ---------------------------------------------------
uint32_t oracle_argmax(const float* row, uint32_t n) {
    uint32_t best = 0;
    float best_val = -std::numeric_limits<float>::infinity();
    for (uint32_t i = 0; i < n; ++i) {
        if (row[i] > best_val) {
            best_val = row[i];
            best = i;
        }
    }
    return best;
}

// ---- bf16.rs:11-25 ------------------------------------------------------
uint16_t oracle_to_bf16(float x) {
    uint32_t bits;
    std::memcpy(&bits, &x, 4);
    if (x != x) return (uint16_t)((bits >> 16) | 0x0040u);
    uint32_t lsb = (bits >> 16) & 1u;
    return (uint16_t)((bits + 0x7fffu + lsb) >> 16);
}

float oracle_from_bf16(uint16_t h) {
    uint32_t bits = (uint32_t)h << 16;
    float x;
    std::memcpy(&x, &bits, 4);
    return x;
}

void oracle_widen_bf16(const uint16_t* src, float* dst, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) dst[i] = oracle_from_bf16(src[i]);
}

void oracle_narrow_bf16(const float* src, uint16_t* dst, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) dst[i] = oracle_to_bf16(src[i]);
}

}  // extern "C"

namespace {

inline float oracle_exp(float x, uint32_t mode) {
    if (mode == ORACLE_EXP_CR) return (float)std::exp((double)x);
    return expf(x);
}

// Rust's f32::max: if one argument is NaN the other is returned.
inline float rust_f32_max(float a, float b) {
    if (a != a) return b;
    if (b != b) return a;
    return a > b ? a : b;
}

// generate.rs:325-420, statement by statement.
uint32_t sample_with_impl(const float* logits, uint32_t vocab, const oracle_sampling_config& cfg,
                          const uint32_t* recent, uint32_t n_recent, uint64_t* rng_state,
                          const oracle_trace* tr) {
    uint32_t flags = 0;
    float st_max = 0.f, st_sum = 0.f, st_total = 0.f, st_u = 0.f, st_thr = 0.f, st_r = 0.f;
    uint32_t kept_n = 0;
    auto finish = [&](uint32_t token, const std::vector<uint32_t>* order, const std::vector<float>* probs) {
        if (tr) {
            if (tr->flags) *tr->flags = flags;
            if (tr->kept_count) *tr->kept_count = kept_n;
            if (tr->stats) {
                tr->stats[0] = st_max; tr->stats[1] = st_sum; tr->stats[2] = st_total;
                tr->stats[3] = st_u; tr->stats[4] = st_thr; tr->stats[5] = st_r;
            }
            if (order && probs) {
                uint32_t n = std::min<uint32_t>(kept_n, tr->kept_capacity);
                for (uint32_t i = 0; i < n; ++i) {
                    if (tr->kept_ids) tr->kept_ids[i] = (*order)[i];
                    if (tr->kept_probs) tr->kept_probs[i] = (*probs)[i];
                }
            }
        }
        return token;
    };

    // :331  work on a copy
    std::vector<float> work(logits, logits + vocab);

    // :333-341  allowed mask, EOS exempt, ids past the slice allowed
    if (cfg.allowed) {
        for (uint32_t id = 0; id < vocab; ++id) {
            bool ok = id < cfg.allowed_len ? cfg.allowed[id] != 0 : true;
            if (id != cfg.eos_id && !ok) work[id] = -std::numeric_limits<float>::infinity();
        }
    }

    // :343-352  repetition penalty, once per history entry, compounding
    if (cfg.repetition_penalty != 1.0f) {
        for (uint32_t j = 0; j < n_recent; ++j) {
            uint32_t id = recent[j];
            if (id < vocab) {
                float l = work[id];
                work[id] = l > 0.0f ? l / cfg.repetition_penalty : l * cfg.repetition_penalty;
            }
        }
    }

    // :354-356  greedy
    if (cfg.temperature <= 0.0f) {
        flags |= ORACLE_FLAG_GREEDY;
        if (tr && tr->work) std::memcpy(tr->work, work.data(), sizeof(float) * vocab);
        return finish(oracle_argmax(work.data(), vocab), nullptr, nullptr);
    }
    // :357-359  temperature: a true division per element
    for (uint32_t i = 0; i < vocab; ++i) work[i] = work[i] / cfg.temperature;
    if (tr && tr->work) std::memcpy(tr->work, work.data(), sizeof(float) * vocab);

    // :364-367  all indices, value descending, index ascending on ties.
    // On NaN-free input this comparator is a strict total order, so every
    // correct sort returns the reference's permutation. A NaN makes the
    // reference's comparator inconsistent (result unspecified); here NaN is
    // ordered after everything and the row is flagged.
    bool has_nan = false;
    for (uint32_t i = 0; i < vocab; ++i) has_nan |= (work[i] != work[i]);
    if (has_nan) flags |= ORACLE_FLAG_NAN_INPUT;
    std::vector<uint32_t> order(vocab);
    std::iota(order.begin(), order.end(), 0u);
    const float* w = work.data();
    if (!has_nan) {
        std::sort(order.begin(), order.end(), [w](uint32_t a, uint32_t b) {
            if (w[b] < w[a]) return true;   // a has the larger value: a first
            if (w[a] < w[b]) return false;
            return a < b;                   // numeric tie (incl. +0 == -0): lower index first
        });
    } else {
        std::sort(order.begin(), order.end(), [w](uint32_t a, uint32_t b) {
            bool na = w[a] != w[a], nb = w[b] != w[b];
            if (na != nb) return nb;
            if (!na) {
                if (w[b] < w[a]) return true;
                if (w[a] < w[b]) return false;
            }
            return a < b;
        });
    }
    // :368-370  top-k
    if (cfg.top_k > 0 && cfg.top_k < order.size()) order.resize(cfg.top_k);

    // :372  max over the kept values, folded from -inf with f32::max
    float mx = -std::numeric_limits<float>::infinity();
    for (uint32_t i : order) mx = rust_f32_max(mx, work[i]);
    st_max = mx;
    // :373  probs = exp(work - max)
    std::vector<float> probs(order.size());
    for (size_t i = 0; i < order.size(); ++i) probs[i] = oracle_exp(work[order[i]] - mx, cfg.exp_mode);
    // :374  sequential left-to-right f32 sum in sorted order
    float sum = 0.0f;
    for (float p : probs) sum = sum + p;
    st_sum = sum;
    // :375-377  degenerate
    if (sum <= 0.0f || !std::isfinite(sum)) {
        flags |= ORACLE_FLAG_DEGENERATE;
        return finish(order.empty() ? 0u : order[0], nullptr, nullptr);
    }
    // :378-380  normalise
    for (float& p : probs) p = p / sum;

    // :384-395  min-p: leading run with p >= min_p * probs[0], at least one
    if (cfg.min_p > 0.0f) {
        float threshold = cfg.min_p * (probs.empty() ? 0.0f : probs[0]);
        st_thr = threshold;
        size_t keep = 0;
        while (keep < probs.size() && probs[keep] >= threshold) ++keep;
        keep = std::max<size_t>(keep, 1);
        keep = std::min(keep, probs.size());  // Vec::truncate is a no-op past the end
        probs.resize(keep);
        order.resize(keep);
    }

    // :397-409  top-p
    if (cfg.top_p < 1.0f) {
        float cumulative = 0.0f;
        size_t keep = probs.size();
        for (size_t i = 0; i < probs.size(); ++i) {
            cumulative = cumulative + probs[i];
            if (cumulative >= cfg.top_p) {
                keep = i + 1;
                break;
            }
        }
        probs.resize(keep);
        order.resize(keep);
    }
    kept_n = (uint32_t)order.size();

    // :411-418  draw
    float total = 0.0f;
    for (float p : probs) total = total + p;
    st_total = total;
    float u = oracle_rng_next_f32(rng_state);
    flags |= ORACLE_FLAG_DRAW_CONSUMED;
    st_u = u;
    float r = u * total;
    st_r = r;
    for (size_t i = 0; i < probs.size(); ++i) {
        if (r < probs[i]) return finish(order[i], &order, &probs);
        r = r - probs[i];
    }
    // :419  rounding left r >= 0 after the walk
    flags |= ORACLE_FLAG_FALLBACK_LAST;
    return finish(order.empty() ? 0u : order.back(), &order, &probs);
}

}  // namespace

extern "C" {

// One call of sample_with (generate.rs:325-330). `rng_state` is the Rng's
// state word, advanced exactly as the reference advances it.
uint32_t oracle_sample_with(const float* logits, uint32_t vocab, const oracle_sampling_config* cfg,
                            const uint32_t* recent, uint32_t n_recent, uint64_t* rng_state,
                            const oracle_trace* trace) {
    return sample_with_impl(logits, vocab, *cfg, recent, n_recent, rng_state, trace);
}

// sample() (generate.rs:423-433): temperature only, everything else off.
uint32_t oracle_sample(const float* logits, uint32_t vocab, float temperature, uint32_t exp_mode,
                       uint64_t* rng_state) {
    oracle_sampling_config cfg{};
    cfg.temperature = temperature;
    cfg.top_k = 0;
    cfg.top_p = 1.0f;
    cfg.min_p = 0.0f;
    cfg.repetition_penalty = 1.0f;
    cfg.allowed = nullptr;
    cfg.eos_id = 258;
    cfg.exp_mode = exp_mode;
    return sample_with_impl(logits, vocab, cfg, nullptr, 0, rng_state, nullptr);
}

// Batched driver used for parity runs and for the timed CPU baseline: row r
// is an independent sample_with call. Rows are spread over `n_threads`
// std::threads (dynamic row claiming). Per-row parameter arrays may be NULL,
// in which case the scalar in `cfg` applies. bf16 rows (logits_bf16 != NULL)
// are widened exactly (bf16.rs:22-25) before the call, as the reference would
// have to. Row r draws with Rng::seed_from_u64(seeds[r]) advanced by
// draw_index[r] outputs first. Trace arrays are [batch] / [batch, kept_capacity]
// / [batch, 6]; any may be NULL.
void oracle_sample_batch(const float* logits_f32, const uint16_t* logits_bf16, uint32_t batch, uint32_t vocab,
                         uint64_t row_stride, const oracle_sampling_config* cfg, const float* temperature_rows,
                         const uint32_t* top_k_rows, const float* top_p_rows, const float* min_p_rows,
                         const float* penalty_rows, const uint32_t* history, uint32_t history_stride,
                         const uint32_t* history_len, const uint64_t* seeds, const uint64_t* draw_index,
                         uint32_t* tokens, uint32_t* kept_count, uint32_t* kept_ids, float* kept_probs,
                         uint32_t kept_capacity, float* stats, uint32_t* flags, uint32_t n_threads) {
    if (n_threads == 0) n_threads = 1;
    std::atomic<uint32_t> next{0};
    auto worker = [&]() {
        std::vector<float> widened;
        for (;;) {
            uint32_t r = next.fetch_add(1);
            if (r >= batch) break;
            const float* row;
            if (logits_bf16) {
                widened.resize(vocab);
                oracle_widen_bf16(logits_bf16 + (uint64_t)r * row_stride, widened.data(), vocab);
                row = widened.data();
            } else {
                row = logits_f32 + (uint64_t)r * row_stride;
            }
            oracle_sampling_config c = *cfg;
            if (temperature_rows) c.temperature = temperature_rows[r];
            if (top_k_rows) c.top_k = top_k_rows[r];
            if (top_p_rows) c.top_p = top_p_rows[r];
            if (min_p_rows) c.min_p = min_p_rows[r];
            if (penalty_rows) c.repetition_penalty = penalty_rows[r];
            uint64_t state = seeds ? seeds[r] : 0;
            if (draw_index) state += draw_index[r] * 0x9E3779B97F4A7C15ull;
            oracle_trace tr{};
            tr.kept_count = kept_count ? kept_count + r : nullptr;
            tr.kept_ids = kept_ids ? kept_ids + (uint64_t)r * kept_capacity : nullptr;
            tr.kept_probs = kept_probs ? kept_probs + (uint64_t)r * kept_capacity : nullptr;
            tr.kept_capacity = kept_capacity;
            tr.stats = stats ? stats + (uint64_t)r * 6 : nullptr;
            tr.flags = flags ? flags + r : nullptr;
            tr.work = nullptr;
            const uint32_t* hist = history ? history + (uint64_t)r * history_stride : nullptr;
            uint32_t hl = history ? (history_len ? history_len[r] : history_stride) : 0;
            tokens[r] = sample_with_impl(row, vocab, c, hist, hl, &state, &tr);
        }
    };
    if (n_threads == 1) {
        worker();
    } else {
        std::vector<std::thread> pool;
        for (uint32_t t = 0; t < n_threads; ++t) pool.emplace_back(worker);
        for (auto& t : pool) t.join();
    }
}

// Post-penalty values at the history positions (the quantity the
// "post-penalty within 1e-6" check compares): out[j] is work[recent[j]] after
// the mask and all penalty applications, before temperature; ids >= vocab
// give NaN.
void oracle_penalized_at_history(const float* logits, uint32_t vocab, const oracle_sampling_config* cfg,
                                 const uint32_t* recent, uint32_t n_recent, float* out) {
    std::vector<float> work(logits, logits + vocab);
    if (cfg->allowed) {
        for (uint32_t id = 0; id < vocab; ++id) {
            bool ok = id < cfg->allowed_len ? cfg->allowed[id] != 0 : true;
            if (id != cfg->eos_id && !ok) work[id] = -std::numeric_limits<float>::infinity();
        }
    }
    if (cfg->repetition_penalty != 1.0f) {
        for (uint32_t j = 0; j < n_recent; ++j) {
            uint32_t id = recent[j];
            if (id < vocab) {
                float l = work[id];
                work[id] = l > 0.0f ? l / cfg->repetition_penalty : l * cfg->repetition_penalty;
            }
        }
    }
    for (uint32_t j = 0; j < n_recent; ++j)
        out[j] = recent[j] < vocab ? work[recent[j]] : std::numeric_limits<float>::quiet_NaN();
}

// llm_core::ops::cross_entropy (crates/llm-core/src/ops/loss.rs:20-45), statement by statement: per row the
// maximum (fold from -inf, :26), the exponentials and their left-to-right f32 sum (:27-32), the row's loss
// ln(sum) + max - row[target] added to a running f32 total (:33-35), the gradient (exp / sum - one-hot) / T
// (:36-40); returns total / T (:42). `row_loss` (optional) receives each row's own term, which is what
// crates/llm-gpu/src/shaders/cross_entropy.wgsl:72-74 writes per row.
float oracle_cross_entropy(const float* logits, const uint32_t* targets, uint32_t t_len, uint32_t vocab, float* d_logits,
                           float* row_loss) {
    float total_loss = 0.0f;
    std::vector<float> exps(vocab);
    for (uint32_t t = 0; t < t_len; ++t) {
        const float* row = logits + (size_t)t * vocab;
        float max = -std::numeric_limits<float>::infinity();
        for (uint32_t i = 0; i < vocab; ++i) max = std::fmax(max, row[i]);
        float sum = 0.0f;
        for (uint32_t i = 0; i < vocab; ++i) {
            const float e = std::exp(row[i] - max);
            exps[i] = e;
            sum += e;
        }
        const uint32_t target = targets[t];
        const float log_z = std::log(sum) + max;
        const float term = log_z - row[target];
        total_loss += term;
        if (row_loss) row_loss[t] = term;
        if (d_logits) {
            float* d_row = d_logits + (size_t)t * vocab;
            for (uint32_t i = 0; i < vocab; ++i) {
                const float p = exps[i] / sum;
                d_row[i] = (p - (i == target ? 1.0f : 0.0f)) / (float)t_len;
            }
        }
    }
    return total_loss / (float)t_len;
}

uint32_t oracle_hardware_threads(void) {
    unsigned n = std::thread::hardware_concurrency();
    return n ? n : 1;
}

}  // extern "C"
