/* llm_cuda.h - C ABI of the B200 token sampler.
 *
 * One path of biffjezos/scriptonait behind a plain C boundary: the per-row
 * sampler `sample_with` (crates/llm-core/src/generate.rs:325-420) - allowed
 * mask, repetition penalty over a token history, temperature, top-k, min-p,
 * top-p and a seeded categorical draw - batched over the rows of a logits
 * matrix that already lives in GPU memory. The parameter surface is the
 * reference's (`temperature, top_k, top_p, min_p, repetition_penalty, seed`,
 * crates/llm-core/src/generate.rs:24-95; crates/wasm-app/src/inference.rs:90-108).
 *
 * Conventions
 *  - every function returns an int32_t status (LLM_CUDA_OK or a negative
 *    LLM_CUDA_ERR_*); nothing throws or aborts across this boundary;
 *  - "device pointer" = memory of the handle's GPU; the caller owns all
 *    buffers and the stream; the library owns only the handle's scratch;
 *  - calls that take device pointers are asynchronous on `stream`;
 *  - a handle is used from one host thread and one stream at a time;
 *  - there is no CPU fallback: without a usable GPU every call fails.
 */
#ifndef LLM_CUDA_H
#define LLM_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LLM_CUDA_ABI_VERSION 2u

/* status codes */
#define LLM_CUDA_OK 0
#define LLM_CUDA_ERR_BAD_ARGUMENT (-1)  /* NULL where a pointer is required, wrong struct_size, bad dtype, ... */
#define LLM_CUDA_ERR_CAPACITY (-2)      /* batch / vocab / history / top_k beyond what the handle was created for */
#define LLM_CUDA_ERR_CUDA (-3)          /* a CUDA runtime call failed; see llm_cuda_last_error */
#define LLM_CUDA_ERR_UNSUPPORTED (-4)   /* e.g. vocabulary sharding with top_k == 0 */
#define LLM_CUDA_ERR_NO_DEVICE (-5)     /* no CUDA device / wrong architecture */
#define LLM_CUDA_ERR_TIMEOUT (-6)       /* a bounded wait inside a kernel ran out (llm_cuda_device_status); the rows it hit carry LLM_CUDA_ROW_INVALID */

/* bits of the device status word (llm_cuda_device_status) */
#define LLM_CUDA_STATUS_COPY_TIMEOUT 1u /* a bulk copy into shared memory did not complete within its wait limit */
#define LLM_CUDA_STATUS_SLOT_TIMEOUT 2u /* no full-ordering scratch slot came free within the wait limit */
#define LLM_CUDA_STATUS_CHECK_FAILED 4u /* checked builds only: a computed shared-memory or scratch index left its bounds (the access was skipped) */

/* logits element types */
#define LLM_CUDA_DTYPE_F32 0u
#define LLM_CUDA_DTYPE_BF16 1u /* widened exactly to f32 (crates/llm-core/src/bf16.rs:22-25) before any arithmetic */

/* per-row flags written to `row_flags` */
#define LLM_CUDA_ROW_GREEDY 1u         /* temperature <= 0: argmax after mask+penalty, no draw consumed (generate.rs:354-356) */
#define LLM_CUDA_ROW_DEGENERATE 2u     /* softmax sum <= 0 or not finite: first id of the ordering returned, no draw consumed (generate.rs:375-377) */
#define LLM_CUDA_ROW_FALLBACK_LAST 4u  /* the walk ran past the kept set: last kept id returned (generate.rs:419) */
#define LLM_CUDA_ROW_DRAW_CONSUMED 8u  /* exactly one RNG output was used: the caller advances draw_index by one */
#define LLM_CUDA_ROW_FULL_SORT 16u     /* the row was resolved by ordering the whole row (candidate window too small) */
#define LLM_CUDA_ROW_INVALID 64u       /* a per-row parameter was NaN; token 0 returned */
#define LLM_CUDA_ROW_WINDOWED 128u     /* ordering ran on the significant-value window, not on a top-k list */

/* The end-of-text id the allowed mask never blocks (crates/llm-core/src/tokenizer.rs:38). */
#define LLM_CUDA_EOS_DEFAULT 258u

/* Number of floats per row in `row_stats`: max, sum, total, u, min-p threshold, r = u*total. */
#define LLM_CUDA_ROW_STATS 6u

typedef struct llm_cuda_sampler llm_cuda_sampler; /* opaque */

/* Mirrors `SamplingConfig` (crates/llm-core/src/generate.rs:24-95) for the one-row
 * host wrapper. `llm_cuda_sampling_config_default` fills the reference's defaults
 * (generate.rs:82-95): 0.9 / 40 / 0.95 / 0.0 / 1.1 / 128 / 0 / no mask. */
typedef struct llm_cuda_sampling_config {
    float temperature;          /* <= 0 means greedy */
    uint32_t top_k;             /* 0 disables */
    float top_p;                /* 1.0 disables */
    float min_p;                /* 0.0 disables */
    float repetition_penalty;   /* 1.0 disables */
    uint32_t repetition_window; /* how many trailing history tokens the caller passes as `recent` */
    uint64_t seed;
    const uint8_t* allowed;     /* host, one byte per id (0 = blocked), or NULL = allow everything */
    uint32_t allowed_len;       /* ids >= allowed_len count as allowed */
} llm_cuda_sampling_config;

/* Batched call: row r of `logits` is one independent `sample_with`.
 * Scalars apply to every row unless the matching *_rows device array is given. */
typedef struct llm_cuda_sample_args {
    uint32_t struct_size;       /* = sizeof(llm_cuda_sample_args) */
    uint32_t logits_dtype;      /* LLM_CUDA_DTYPE_* */
    const void* logits;         /* device, [batch, row_stride_elems]; read only, never modified (generate.rs:331) */
    uint32_t batch;
    uint32_t vocab;             /* columns of this matrix */
    uint64_t row_stride_elems;  /* elements between rows; 0 = every row reads row 0 */

    float temperature;
    uint32_t top_k;
    float top_p;
    float min_p;
    float repetition_penalty;
    uint32_t overlap_previous;  /* nonzero: this launch may begin reading its INPUTS (logits, history, seeds,
                                 * draw_index, uniforms, every *_rows array, allowed_bits) before the operation
                                 * that precedes it on the stream has completed; its writes still come after.
                                 * Set it only when none of those arrays is written by that preceding
                                 * operation - e.g. consecutive llm_cuda_sample_batch calls over independent
                                 * batches. Not behind the kernel that produced the logits, and not behind
                                 * llm_cuda_advance_rows (it writes draw_index and history). 0 = strict stream
                                 * order. 2 = early launch only: the grid is set up while the preceding kernel
                                 * is finishing (if that kernel allows it, as this library's do) but reads and
                                 * writes nothing before it has completed - data order is strict, safe behind any
                                 * operation; it only takes the launch latency off the critical path.
                                 * llm_cuda_sample_batch_static ignores the flag (always strict). */
    const float* temperature_rows;        /* device [batch] or NULL */
    const uint32_t* top_k_rows;           /* device [batch] or NULL */
    const float* top_p_rows;              /* device [batch] or NULL */
    const float* min_p_rows;              /* device [batch] or NULL */
    const float* repetition_penalty_rows; /* device [batch] or NULL */

    const uint32_t* history;     /* device [batch, history_stride] token ids (any value, repeats allowed), or NULL */
    uint32_t history_stride;
    uint32_t history_len;        /* used when history_len_rows is NULL; <= history_stride */
    const uint32_t* history_len_rows; /* device [batch] or NULL */

    const uint32_t* allowed_bits; /* device, bit i of word i/32 set = id i allowed; NULL = allow everything */
    uint32_t allowed_len;         /* ids >= allowed_len count as allowed */
    uint32_t eos_id;              /* never blocked by the mask */

    const uint64_t* seeds;       /* device [batch]: Rng::seed_from_u64(seeds[r]); NULL = seed_base + r */
    const uint64_t* draw_index;  /* device [batch]: outputs already consumed from that Rng; NULL = 0 */
    uint64_t seed_base;
    const float* uniforms;       /* device [batch] or NULL: replaces rng.next_f32() (pins the uniform stream) */

    uint32_t* tokens;            /* device [batch], out */

    /* optional per-stage outputs (NULL to skip) */
    uint32_t* row_flags;         /* device [batch] LLM_CUDA_ROW_* */
    uint32_t* kept_count;        /* device [batch]: size of the kept set */
    uint32_t* kept_ids;          /* device [batch, kept_capacity]: kept ids, most likely first */
    float* kept_probs;           /* device [batch, kept_capacity]: their probabilities p_i / sum */
    uint32_t kept_capacity;
    uint32_t reserved1;
    float* row_stats;            /* device [batch, LLM_CUDA_ROW_STATS] */

    /* vocabulary sharding (llm_cuda_shard_select only; 0 / vocab otherwise) */
    uint32_t column_offset;      /* global id of column 0 of this matrix */
    uint32_t vocab_global;       /* 0 = vocab */

    uint32_t split;              /* CTAs per row; 0 = choose */
    uint32_t force_full_sort;    /* testing aid: resolve every row by ordering the whole row */
    void* stream;                /* cudaStream_t */

    float* penalized_out;        /* optional, device [batch, history_stride]: entry (r, j), j < history length of row r, receives
                                  * the value of logit history[r, j] after the allowed mask and every penalty application and
                                  * before temperature (generate.rs:333-352); NaN for ids outside this matrix's columns.
                                  * Written for rows the streaming path samples (not for NaN-parameter or force_full_sort rows) */
} llm_cuda_sample_args;

/* Reference defaults (generate.rs:82-95). */
void llm_cuda_sampling_config_default(llm_cuda_sampling_config* out);

/* Creates a sampler bound to `device` with scratch sized for the given maxima.
 * Replaces nothing in the reference (it allocates two Vecs per call,
 * generate.rs:331,364); this is where the device scratch those become lives.
 * max_batch <= 65535 (LLM_CUDA_ERR_CAPACITY beyond). */
int32_t llm_cuda_sampler_create(int32_t device, uint32_t max_batch, uint32_t max_vocab, uint32_t max_history,
                                uint32_t max_top_k, llm_cuda_sampler** out);
int32_t llm_cuda_sampler_destroy(llm_cuda_sampler* s);

/* Text of the last error on this handle (or of the last failed create when s is NULL). */
const char* llm_cuda_last_error(const llm_cuda_sampler* s);

/* Batched `sample_with` over device buffers - the hot path.
 * Replaces the sampling call of the GPU generation loop
 * (crates/wasm-app/src/inference.rs:326-327) and of Generator::step
 * (crates/llm-core/src/generate.rs:157-165), without the per-token logits
 * read-back (crates/llm-gpu/src/model.rs:483-490,520-550). */
int32_t llm_cuda_sample_batch(llm_cuda_sampler* s, const llm_cuda_sample_args* args);

/* Same call with every array in HOST memory: copies inputs to the device, runs
 * llm_cuda_sample_batch, copies `tokens` (and any requested per-stage outputs)
 * back and synchronises. Pointers in `args` are host pointers here. This is the
 * path a caller takes whose logits were produced on the host, as the reference's
 * CPU generation loop does (crates/llm-core/src/generate.rs:157-165). */
int32_t llm_cuda_sample_batch_host(llm_cuda_sampler* s, const llm_cuda_sample_args* host_args);

/* One row, host buffers, the reference's own signature:
 * sample_with(logits, sampling, recent, rng) -> token (generate.rs:325-330).
 * `rng_state` is the SplitMix64 state word (crates/llm-core/src/rng.rs:6-22); it
 * is advanced by one output exactly when the reference would draw. */
int32_t llm_cuda_sample_with(llm_cuda_sampler* s, const float* logits, uint32_t vocab,
                             const llm_cuda_sampling_config* sampling, const uint32_t* recent, uint32_t n_recent,
                             uint64_t* rng_state, uint32_t* token_out);

/* sample(logits, temperature, rng) (generate.rs:423-433): temperature only. */
int32_t llm_cuda_sample(llm_cuda_sampler* s, const float* logits, uint32_t vocab, float temperature,
                        uint64_t* rng_state, uint32_t* token_out);

/* Vocabulary sharding, step 1 of 2: this GPU holds columns
 * [column_offset, column_offset + vocab) of every row. Applies mask, penalty
 * and temperature to its columns and writes, per row, its best
 * min(top_k, vocab) candidates in order (value descending, global id ascending)
 * - the ordering of generate.rs:364-367 - into
 * cand_values[batch, cand_stride] / cand_ids[batch, cand_stride], with the
 * number written in cand_count[batch]. Requires 0 < top_k <= cand_stride; greedy
 * rows (temperature <= 0) send one candidate. A shard with vocab == 0 (past the end of
 * a small vocabulary) is legal and writes empty lists. No reference counterpart (the
 * reference is single-device); exact because the global top-k is a subset of
 * the union of per-shard top-k lists and the softmax runs over the kept k only
 * (generate.rs:368-380). */
int32_t llm_cuda_shard_select(llm_cuda_sampler* s, const llm_cuda_sample_args* args, float* cand_values,
                              uint32_t* cand_ids, uint32_t* cand_count, uint32_t cand_stride);

/* Vocabulary sharding, step 2 of 2: after the candidate lists of all `n_shards`
 * have been gathered as [n_shards, batch, cand_stride] (+ counts
 * [n_shards, batch]), merges them per row with the same comparator and runs
 * softmax, min-p, top-p and the draw (generate.rs:368-419). The lists must be
 * as llm_cuda_shard_select wrote them (each in the reference order, best first):
 * the merge relies on that order to skip entries that cannot reach the kept set.
 * `args` supplies the parameters, RNG and outputs; its logits/history fields are
 * ignored. Every rank that calls this with the same inputs gets the same tokens. */
int32_t llm_cuda_merge_draw(llm_cuda_sampler* s, const llm_cuda_sample_args* args, const float* cand_values,
                            const uint32_t* cand_ids, const uint32_t* cand_count, uint32_t n_shards,
                            uint32_t cand_stride);

/* The same two steps with ONE buffer per rank, so that the exchange between them is a single
 * all-gather: a packed block holds, for `batch` rows, the values [batch, cand_stride] (f32), then the
 * global ids [batch, cand_stride] (u32), then the counts [batch] (u32) -
 * llm_cuda_packed_candidates_bytes(batch, cand_stride) bytes (16.5 KB for 32 rows of 64 candidates).
 * llm_cuda_shard_select_packed writes this GPU's block; llm_cuda_merge_draw_packed reads `n_shards`
 * such blocks laid end to end, which is exactly what an all-gather of the ranks' blocks produces
 * (ncclAllGather over NVLink). Same requirements, results and errors as the three-pointer forms.
 * No reference counterpart (the reference is single-device). */
size_t llm_cuda_packed_candidates_bytes(uint32_t batch, uint32_t cand_stride);
int32_t llm_cuda_shard_select_packed(llm_cuda_sampler* s, const llm_cuda_sample_args* args, void* packed_out,
                                     uint32_t cand_stride);
int32_t llm_cuda_merge_draw_packed(llm_cuda_sampler* s, const llm_cuda_sample_args* args, const void* packed_all,
                                   uint32_t n_shards, uint32_t cand_stride);

/* Fused tied LM head -> sampler for a decode batch: final RMSNorm, the hidden x vocab contraction over the
 * tied embedding on the tensor cores, and sampling, without ever writing the [batch, vocab] logits.
 * Replaces the last three dispatches of GpuModel::decode_step (crates/llm-gpu/src/model.rs:481-490:
 * dispatch_rmsnorm, dispatch_linear over self.embed, the vocab*4-byte copy + read_back), the linear kernel
 * crates/llm-gpu/src/shaders/linear.wgsl and the sample_with call on the host that follows
 * (crates/wasm-app/src/inference.rs:325-347). The hidden states are narrowed to bf16 after the norm and the
 * products accumulate in f32 on the tensor cores, so the logits differ from the reference's f32 contraction
 * by bf16 input rounding; given those logits every sampler stage is exact (logits_out exposes them).
 * Limits: batch <= 256, hidden_dim a multiple of 8, 0 < top_k <= 256 or greedy; no repetition penalty and
 * no allowed mask on this path (use llm_cuda_sample_batch on materialised logits for those). A row whose
 * threshold estimate left fewer than top_k candidates, or more than the 2048 a list holds, is reported
 * with LLM_CUDA_ROW_INVALID (token 0), not guessed. */
typedef struct llm_cuda_lm_head_args {
    uint32_t struct_size;        /* = sizeof(llm_cuda_lm_head_args) */
    uint32_t batch;              /* rows of `hidden` (decode batch), <= 256 */
    const float* hidden;         /* device [batch, hidden_dim] f32: the last layer's output, before the final norm */
    const float* norm_gain;      /* device [hidden_dim] final RMSNorm gain, or NULL when `hidden` is already normalised */
    float norm_eps;
    uint32_t hidden_dim;
    const void* embed;           /* device [vocab, hidden_dim] bf16, row-major: the tied embedding / LM head weight */
    uint32_t vocab;
    float temperature;           /* <= 0: greedy */
    uint32_t top_k;
    float top_p;
    float min_p;
    uint32_t reserved0;
    const uint64_t* seeds;       /* as in llm_cuda_sample_args */
    const uint64_t* draw_index;
    uint64_t seed_base;
    const float* uniforms;
    uint32_t* tokens;            /* device [batch], out */
    uint32_t* row_flags;         /* optional per-stage outputs, as in llm_cuda_sample_args */
    uint32_t* kept_count;
    uint32_t* kept_ids;
    float* kept_probs;
    uint32_t kept_capacity;
    uint32_t reserved1;
    float* row_stats;
    float* logits_out;           /* optional device [batch, vocab] f32, testing aid: also write the logits themselves */
    void* stream;
} llm_cuda_lm_head_args;
int32_t llm_cuda_lm_head_sample(llm_cuda_sampler* s, const llm_cuda_lm_head_args* args);

/* Device-side decode-loop glue (Generator::step / recent_tokens,
 * crates/llm-core/src/generate.rs:157-182; the EOS test of
 * crates/wasm-app/src/inference.rs:326-333): for each row that is not finished,
 * appends tokens[r] to its history ring, which holds the last cap = min(window, history_stride)
 * tokens of the row in history[r, 0 .. cap): while history_len[r] < cap the token goes to slot
 * history_len[r]; once the ring is full it replaces the oldest entry, at slot history_pos[r] % cap
 * (history_pos is required whenever history is given: LLM_CUDA_ERR_BAD_ARGUMENT without it).
 * Adds one to draw_index[r] when row_flags[r] has DRAW_CONSUMED, and sets finished[r] when the
 * token is eos_id (the token is then not appended, as step() returns None).
 * All pointers are device pointers; asynchronous on `stream`. */
int32_t llm_cuda_advance_rows(llm_cuda_sampler* s, uint32_t batch, const uint32_t* tokens, const uint32_t* row_flags,
                              uint32_t* history, uint32_t history_stride, uint32_t window, uint32_t* history_len,
                              uint32_t* history_pos, uint64_t* draw_index, uint8_t* finished, uint32_t eos_id,
                              void* stream);

/* Packs a host bool-per-id slice (Corpus::seen_tokens, crates/llm-core/src/corpus.rs:236-246;
 * SamplingConfig::allowed, generate.rs:67-80) into the device bit mask
 * `allowed_bits` expects: ceil(n/32) words. `bits_out` is a device pointer. */
int32_t llm_cuda_pack_allowed(llm_cuda_sampler* s, const uint8_t* allowed_host, uint32_t n, uint32_t* bits_out,
                              void* stream);

/* Cross-entropy over the rows of a [rows, vocab] f32 logits matrix and its gradient with respect to the
 * logits: the training-side row reduction next to the sampler's softmax. Replaces
 * crates/llm-gpu/src/shaders/cross_entropy.wgsl:29-88 / llm_core::ops::cross_entropy
 * (crates/llm-core/src/ops/loss.rs:20-45):
 *   row_loss[t]    = ln(sum_v exp(x[t,v] - max_t)) + max_t - x[t, targets[t]]      (the mean over t is the loss)
 *   d_logits[t, v] = (softmax(x[t,:])[v] - (v == targets[t])) / rows                (optional: may be NULL)
 * All pointers are device pointers; `d_logits` uses the logits' row stride and must share the logits' base
 * alignment modulo 16 bytes (a tensor of the same shape does). A target outside [0, vocab) gives that row a
 * NaN loss (the reference panics). Asynchronous on `stream`. */
int32_t llm_cuda_cross_entropy(llm_cuda_sampler* s, const float* logits, uint32_t rows, uint32_t vocab,
                               uint32_t row_stride_elems, const uint32_t* targets, float* row_loss, float* d_logits,
                               void* stream);

/* Reads and clears the handle's device status word after `stream` has drained (this call synchronises
 * the stream). The kernels never wait without a limit: a wait that runs out gives the row up
 * (LLM_CUDA_ROW_INVALID, token 0) and sets a LLM_CUDA_STATUS_* bit here instead of hanging or guessing.
 * Returns LLM_CUDA_OK when the word is 0 and LLM_CUDA_ERR_TIMEOUT when a wait ran out; `bits_out` (optional)
 * receives the word either way. The reference's analogue turns a lost device into an Err
 * (crates/llm-gpu/src/buffers.rs:58-86, consumed at crates/wasm-app/src/inference.rs:203-214).
 * llm_cuda_sample_batch_host, llm_cuda_sample_with and llm_cuda_sample check it themselves before they return. */
int32_t llm_cuda_device_status(llm_cuda_sampler* s, void* stream, uint32_t* bits_out);

/* Testing aid for the status path, safe by construction: `hold` != 0 marks every full-ordering scratch slot
 * as taken (0 releases them), and `wait_rounds` != 0 shortens the slot wait of later launches to that many
 * polls of about 4 us (0 restores the default). A launch whose rows need the full ordering then finds no
 * slot, gives those rows up after the shortened wait and reports LLM_CUDA_STATUS_SLOT_TIMEOUT; nothing
 * faults, traps or waits without a limit. Synchronises `stream`. No reference counterpart. */
int32_t llm_cuda_test_hold_full_sort_slots(llm_cuda_sampler* s, uint32_t hold, uint32_t wait_rounds, void* stream);

/* Launch statistics of the last call on this handle (for benchmarks): how many
 * kernels it launched and the CTAs-per-row split it chose. */
int32_t llm_cuda_last_launch_info(const llm_cuda_sampler* s, uint32_t* kernels_launched, uint32_t* split_used);

/* Limits of llm_cuda_sample_batch_static (the size of its fixed scratch follows from them:
 * 256 candidate lists of 2*256 entries, about 1 MiB per GPU that loads the library). */
#define LLM_CUDA_STATIC_MAX_BATCH 64u
#define LLM_CUDA_STATIC_MAX_TOP_K 256u
#define LLM_CUDA_STATIC_MAX_HISTORY 512u

/* llm_cuda_sample_batch without a handle and without any allocation. It has no counterpart
 * in the reference (whose sampler allocates two Vecs per call, generate.rs:331,364); it exists
 * for callers that are not allowed to call cudaMalloc / cudaFree at all - a serving loop whose
 * device memory is partitioned once and then frozen, a host framework that owns the allocator,
 * a plugin that only ever receives device pointers and a stream. The scratch that rows split
 * over several CTAs need lives in a fixed array inside the library image (every GPU that loads
 * the library holds it until the process exits), so:
 *   - sizes are capped: batch <= 64, 0 < top_k <= 256 (or greedy), history <= 512; no per-row
 *     top_k / temperature arrays, no allowed mask, no vocabulary sharding - anything that could
 *     need the window or full-sort stages returns LLM_CUDA_ERR_UNSUPPORTED / _CAPACITY;
 *   - all calls share the one array: calls that overlap on the GPU race; serialise them
 *     (one stream, or events between streams);
 *   - the first call on a device looks up the array's device address and raises the kernels'
 *     shared-memory limit; make that first call before any stream capture begins.
 * Same arguments and results as llm_cuda_sample_batch otherwise (asynchronous on args->stream;
 * overlap_previous is ignored: every launch keeps strict stream order).
 * Errors: llm_cuda_static_last_error(). */
int32_t llm_cuda_sample_batch_static(int32_t device, const llm_cuda_sample_args* args);
const char* llm_cuda_static_last_error(void);

uint32_t llm_cuda_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* LLM_CUDA_H */
