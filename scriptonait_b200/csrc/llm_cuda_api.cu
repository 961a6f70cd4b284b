// C ABI of the B200 token sampler: argument checking, scratch ownership and
// kernel launches. Declarations and the reference interfaces each entry point
// stands in for are in include/llm_cuda.h. There is no CPU path in this file:
// every entry point either launches the CUDA kernels or returns an error.
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>
#include <stdlib.h>

#include <new>
#include <vector>

#include "../../include/llm_cuda.h"
#include "sampler_kernels.h"
#include "cross_entropy.h"
#include "lm_head.h"

using namespace llmc;

namespace {

constexpr uint32_t kMaxKcap = 2048;           // must match MAX_KCAP
constexpr uint64_t kScratchEntries = 1u << 22;  // candidate entries shared by the CTAs of split rows (32 MiB)
constexpr uint64_t kGamma = 0x9E3779B97F4A7C15ull;
constexpr uint32_t kLmCandCap = 2048;   // candidates per row the fused LM head keeps
constexpr uint32_t kLmProbeEvery = 8;   // one vocabulary tile in eight is probed for the thresholds
constexpr uint32_t kSlotRounds = 1u << 16;  // a quarter of a second of polling: thousands of rows can queue for the slots of a launch

char g_create_error[512] = "";

uint32_t pow2_ceil_u32(uint32_t x) {
    uint32_t p = 1u;
    while (p < x) p <<= 1;
    return p;
}

}  // namespace

namespace llmc {

int validate_sample_args(const llm_cuda_sample_args* a, bool needs_logits, char* err, size_t err_len) {
    auto bad = [&](const char* fmt, unsigned long long x = 0, unsigned long long y = 0) {
        snprintf(err, err_len, fmt, x, y);
        return LLM_CUDA_ERR_BAD_ARGUMENT;
    };
    if (!a) return bad("args is NULL");
    if (a->struct_size != sizeof(llm_cuda_sample_args))
        return bad("struct_size %llu, expected %llu", a->struct_size, sizeof(llm_cuda_sample_args));
    if (a->logits_dtype != LLM_CUDA_DTYPE_F32 && a->logits_dtype != LLM_CUDA_DTYPE_BF16)
        return bad("unknown logits_dtype %llu", a->logits_dtype);
    if (needs_logits) {
        if (a->batch && !a->logits) return bad("logits is NULL");
        if (a->vocab == 0) return bad("vocab is 0");
        if (a->row_stride_elems != 0 && a->row_stride_elems < a->vocab)
            return bad("row_stride_elems %llu < vocab %llu", a->row_stride_elems, a->vocab);
        // rows are read as 16-byte vectors from the first 16-byte boundary on, element by element before
        // it: that only works out when the matrix starts on an element boundary
        const uintptr_t esz = a->logits_dtype == LLM_CUDA_DTYPE_BF16 ? 2 : 4;
        if (reinterpret_cast<uintptr_t>(a->logits) % esz) return bad("logits pointer not element aligned");
        if (a->history && a->history_len > a->history_stride)
            return bad("history_len %llu > history_stride %llu", a->history_len, a->history_stride);
    }
    if (a->temperature_rows == nullptr && a->temperature != a->temperature) return bad("temperature is NaN");
    if (a->repetition_penalty_rows == nullptr && a->repetition_penalty != a->repetition_penalty)
        return bad("repetition_penalty is NaN");
    if ((a->kept_ids || a->kept_probs) && a->kept_capacity == 0) return bad("kept_ids/kept_probs given with kept_capacity 0");
    return LLM_CUDA_OK;
}

}  // namespace llmc

struct llm_cuda_sampler {
    int device = 0;
    uint32_t max_batch = 0, max_vocab = 0, max_history = 0, max_top_k = 0;
    DeviceInfo dev{};
    // split-row scratch
    float* sc_q = nullptr;
    uint32_t* sc_i = nullptr;
    uint32_t* sc_cnt = nullptr;
    uint32_t* sc_maxkey = nullptr;
    uint32_t* sc_ticket = nullptr;
    uint32_t sc_lists = 0;  // capacity of sc_cnt / sc_maxkey
    // full-sort scratch
    uint32_t* full_slots = nullptr;
    uint64_t* full_keys = nullptr;
    float* full_vals = nullptr;
    uint32_t vpad = 0, nslots = 0;
    uint32_t* device_errors = nullptr;  // LLM_CUDA_STATUS_* bits set by kernels whose bounded waits ran out
    uint32_t slot_rounds = kSlotRounds;
#ifdef LLMC_DEV
    unsigned long long* phase_ns = nullptr;  // development builds only: per-CTA phase timestamps
#endif
    // scratch of the fused LM head path (allocated on its first use, grown on demand)
    void* lm_xnorm = nullptr;       // [n_pad, hidden] bf16
    float* lm_probe = nullptr;      // [batch, probe_cols]
    float* lm_thr = nullptr;        // [256]
    float* lm_cand_q = nullptr;     // [256, kLmCandCap]
    uint32_t* lm_cand_i = nullptr;
    uint32_t* lm_cand_count = nullptr;
    size_t lm_xnorm_bytes = 0, lm_probe_bytes = 0;
    bool lm_configured = false;
    // staging for the host-buffer entry points (grown on demand)
    unsigned char* arena = nullptr;
    size_t arena_bytes = 0;
    uint32_t last_kernels = 0, last_split = 0;
    char err[512] = "";
};

namespace {

int32_t fail(llm_cuda_sampler* s, int32_t code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(s ? s->err : g_create_error, 512, fmt, ap);
    va_end(ap);
    return code;
}

#define CUDA_TRY(s, call)                                                                                  \
    do {                                                                                                   \
        cudaError_t e_ = (call);                                                                           \
        if (e_ != cudaSuccess) return fail((s), LLM_CUDA_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

void free_all(llm_cuda_sampler* s) {
    cudaFree(s->sc_q);
    cudaFree(s->sc_i);
    cudaFree(s->sc_cnt);
    cudaFree(s->sc_maxkey);
    cudaFree(s->sc_ticket);
    cudaFree(s->full_slots);
    cudaFree(s->full_keys);
    cudaFree(s->full_vals);
    cudaFree(s->device_errors);
    cudaFree(s->lm_xnorm);
    cudaFree(s->lm_probe);
    cudaFree(s->lm_thr);
    cudaFree(s->lm_cand_q);
    cudaFree(s->lm_cand_i);
    cudaFree(s->lm_cand_count);
    cudaFree(s->arena);
}

// Shared validation + parameter block for the three device-buffer entry points.
int32_t fill_params(llm_cuda_sampler* s, const llm_cuda_sample_args* a, bool needs_logits, KParams* P) {
    if (!s) return fail(nullptr, LLM_CUDA_ERR_BAD_ARGUMENT, "sampler handle is NULL");
    {
        const int32_t rc = validate_sample_args(a, needs_logits, s->err, sizeof(s->err));
        if (rc != LLM_CUDA_OK) return rc;
    }
    if (a->batch > s->max_batch) return fail(s, LLM_CUDA_ERR_CAPACITY, "batch %u > max_batch %u", a->batch, s->max_batch);
    if (needs_logits) {
        if (a->vocab > s->max_vocab) return fail(s, LLM_CUDA_ERR_CAPACITY, "vocab %u > max_vocab %u", a->vocab, s->max_vocab);
        if (a->history) {
            const uint32_t hmax = a->history_len_rows ? a->history_stride : a->history_len;
            if (hmax > s->max_history) return fail(s, LLM_CUDA_ERR_CAPACITY, "history %u > max_history %u", hmax, s->max_history);
        }
    }

    memset(P, 0, sizeof(*P));
    P->logits = a->logits;
    P->row_stride = a->row_stride_elems;
    P->batch = a->batch;
    P->vocab = a->vocab;
    P->dtype = a->logits_dtype;
    P->temperature = a->temperature;
    P->top_p = a->top_p;
    P->min_p = a->min_p;
    P->penalty = a->repetition_penalty;
    P->top_k = a->top_k;
    P->t_rows = a->temperature_rows;
    P->k_rows = a->top_k_rows;
    P->p_rows = a->top_p_rows;
    P->m_rows = a->min_p_rows;
    P->r_rows = a->repetition_penalty_rows;
    P->history = a->history;
    P->hist_stride = a->history_stride;
    P->hist_len = a->history_len;
    P->hist_len_rows = a->history_len_rows;
    P->allowed_bits = a->allowed_bits;
    P->allowed_len = a->allowed_len;
    P->eos_id = a->eos_id;
    P->seeds = a->seeds;
    P->draw_index = a->draw_index;
    P->seed_base = a->seed_base;
    P->uniforms = a->uniforms;
    P->tokens = a->tokens;
    P->row_flags = a->row_flags;
    P->kept_count = a->kept_count;
    P->kept_ids = a->kept_ids;
    P->kept_probs = a->kept_probs;
    P->kept_cap = (a->kept_ids || a->kept_probs) ? a->kept_capacity : 0u;
    P->row_stats = a->row_stats;
    P->col_offset = a->column_offset;
    P->vocab_global = a->vocab_global ? a->vocab_global : a->vocab;
    P->force_full = a->force_full_sort;
    P->device_errors = s->device_errors;
    P->full_slot_rounds = s->slot_rounds;
    P->penalized_out = a->penalized_out;
#ifdef LLMC_DEV
    P->phase_ns = s->phase_ns;
#endif
    return LLM_CUDA_OK;
}

bool scalar_greedy(const llm_cuda_sample_args* a) { return a->temperature_rows == nullptr && a->temperature <= 0.0f; }

// Plans and launches the streaming kernel (rows it cannot decide are ordered in full by their own CTA).
int32_t run_select(llm_cuda_sampler* s, const llm_cuda_sample_args* a, KParams& P) {
    LaunchPlan plan{};
    P.full_keys_wanted = 1u;  // this handle owns full-ordering scratch: rows a sampled threshold cannot decide have somewhere to go
    const bool k_known = (a->top_k_rows == nullptr);
    const uint32_t k_hint = scalar_greedy(a) ? 1u : a->top_k;
    // lists the split scratch can hold at this launch's list length
    uint32_t list_len;
    {
        LaunchPlan probe{};
        if (plan_launch(s->dev, P, k_known, k_hint, s->max_top_k, s->max_history, 1u, 1u, &probe) != 0)
            return fail(s, LLM_CUDA_ERR_CAPACITY, "shared-memory layout does not fit (history %u)", s->max_history);
        list_len = probe.limit;
    }
    uint64_t max_lists = kScratchEntries / list_len;
    if (max_lists > s->sc_lists) max_lists = s->sc_lists;
    if (plan_launch(s->dev, P, k_known, k_hint, s->max_top_k, s->max_history, a->split, (uint32_t)max_lists, &plan) != 0)
        return fail(s, LLM_CUDA_ERR_CAPACITY, "shared-memory layout does not fit (vocab %u, history %u)", a->vocab, s->max_history);
    apply_plan(plan, &P);
    P.sc_q = s->sc_q;
    P.sc_i = s->sc_i;
    P.sc_cnt = s->sc_cnt;
    P.sc_maxkey = s->sc_maxkey;
    P.sc_ticket = s->sc_ticket;
    P.sc_stride = plan.limit;
    P.sc_rows = P.batch;
    P.sc_shard_words = P.sc_rows * P.sc_stride;
    P.sc_cnt_shard = P.sc_rows;
    cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
    s->last_kernels = 0;
    s->last_split = plan.split;
    if (P.batch == 0) return LLM_CUDA_OK;
    // rows the stream cannot decide are ordered in full by their own CTA, in one of these slots
    P.full_keys = reinterpret_cast<unsigned long long*>(s->full_keys);
    P.full_vals = s->full_vals;
    P.full_slots = s->full_slots;
    P.full_vpad = s->vpad;
    P.full_nslots = s->nslots;
    P.wait_first = a->overlap_previous == 2u ? 1u : 0u;
    CUDA_TRY(s, launch_stream_select(P, plan, stream, a->overlap_previous != 0u));
    s->last_kernels++;
    return LLM_CUDA_OK;
}

// Carves `bytes` (256-byte aligned) out of the staging arena.
struct Carver {
    unsigned char* base;
    size_t off = 0;
    void* take(size_t bytes) {
        void* p = base ? base + off : nullptr;
        off += (bytes + 255u) & ~size_t(255);
        return p;
    }
};

}  // namespace

extern "C" {

uint32_t llm_cuda_abi_version(void) { return LLM_CUDA_ABI_VERSION; }

void llm_cuda_sampling_config_default(llm_cuda_sampling_config* out) {
    if (!out) return;
    out->temperature = 0.9f;
    out->top_k = 40;
    out->top_p = 0.95f;
    out->min_p = 0.0f;
    out->repetition_penalty = 1.1f;
    out->repetition_window = 128;
    out->seed = 0;
    out->allowed = nullptr;
    out->allowed_len = 0;
}

const char* llm_cuda_last_error(const llm_cuda_sampler* s) { return s ? s->err : g_create_error; }

int32_t llm_cuda_sampler_create(int32_t device, uint32_t max_batch, uint32_t max_vocab, uint32_t max_history,
                                uint32_t max_top_k, llm_cuda_sampler** out) {
    if (!out) return fail(nullptr, LLM_CUDA_ERR_BAD_ARGUMENT, "out is NULL");
    *out = nullptr;
    if (max_batch == 0 || max_vocab == 0) return fail(nullptr, LLM_CUDA_ERR_BAD_ARGUMENT, "max_batch and max_vocab must be > 0");
    if (max_batch > 65535u)  // rows are the grid's y dimension
        return fail(nullptr, LLM_CUDA_ERR_CAPACITY, "max_batch %u exceeds the 65535 rows one launch can take", max_batch);
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev == 0)
        return fail(nullptr, LLM_CUDA_ERR_NO_DEVICE, "no CUDA device (%s); this library has no CPU path", cudaGetErrorString(e));
    if (device < 0 || device >= ndev) return fail(nullptr, LLM_CUDA_ERR_BAD_ARGUMENT, "device %d out of range (%d devices)", device, ndev);
    cudaDeviceProp prop{};
    e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return fail(nullptr, LLM_CUDA_ERR_CUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    if (prop.major != 10)
        return fail(nullptr, LLM_CUDA_ERR_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
    llm_cuda_sampler* s = new (std::nothrow) llm_cuda_sampler();
    if (!s) return fail(nullptr, LLM_CUDA_ERR_CUDA, "out of host memory");
    s->device = device;
    s->max_batch = max_batch;
    s->max_vocab = max_vocab;
    s->max_history = max_history;
    s->max_top_k = max_top_k ? max_top_k : 1u;
    s->dev.sm_count = (uint32_t)prop.multiProcessorCount;
    s->dev.max_dyn_smem = (size_t)prop.sharedMemPerBlockOptin - 4096u;  // room for the kernels' static shared memory
    auto bail = [&](const char* what, cudaError_t ce) {
        fail(nullptr, LLM_CUDA_ERR_CUDA, "%s: %s", what, cudaGetErrorString(ce));
        free_all(s);
        delete s;
        return LLM_CUDA_ERR_CUDA;
    };
    if ((e = cudaSetDevice(device)) != cudaSuccess) return bail("cudaSetDevice", e);
    if ((e = configure_kernels(s->dev.max_dyn_smem)) != cudaSuccess) return bail("cudaFuncSetAttribute", e);
    s->sc_lists = max_batch > 4096u ? max_batch : 4096u;
    // the arrays of a slot, and the slots, start an odd number of 256-byte lines apart: rows that are ordered
    // side by side step through their arrays together, and a power-of-two spacing would send all of their
    // traffic to the same few memory channels
    s->vpad = ((max_vocab + 1023u) & ~1023u) + 1088u;
    // two slots per SM (a batch of such rows then orders at two rows per SM instead of queueing for one): 20
    // bytes per column (two key/index array pairs and the probabilities), at most 2 GiB in all; a CTA that
    // finds every slot taken waits for one (bounded)
    s->nslots = 2u * s->dev.sm_count;
    if (s->nslots > max_batch) s->nslots = max_batch;
    while (s->nslots > s->dev.sm_count && (uint64_t)s->nslots * s->vpad * 20u > (2ull << 30)) s->nslots -= 1u;
    if ((e = cudaMalloc(&s->sc_q, kScratchEntries * 4u)) != cudaSuccess) return bail("cudaMalloc", e);
    if ((e = cudaMalloc(&s->sc_i, kScratchEntries * 4u)) != cudaSuccess) return bail("cudaMalloc", e);
    if ((e = cudaMalloc(&s->sc_cnt, (size_t)s->sc_lists * 4u)) != cudaSuccess) return bail("cudaMalloc", e);
    if ((e = cudaMalloc(&s->sc_maxkey, (size_t)s->sc_lists * 4u)) != cudaSuccess) return bail("cudaMalloc", e);
    if ((e = cudaMalloc(&s->sc_ticket, (size_t)max_batch * 4u)) != cudaSuccess) return bail("cudaMalloc", e);
    if ((e = cudaMalloc(&s->full_slots, (size_t)s->nslots * 4u)) != cudaSuccess) return bail("cudaMalloc", e);
    if ((e = cudaMalloc(&s->full_keys, (size_t)s->nslots * s->vpad * 16u)) != cudaSuccess) return bail("cudaMalloc", e);
    if ((e = cudaMalloc(&s->full_vals, (size_t)s->nslots * s->vpad * 4u)) != cudaSuccess) return bail("cudaMalloc", e);
    if ((e = cudaMemset(s->sc_ticket, 0, (size_t)max_batch * 4u)) != cudaSuccess) return bail("cudaMemset", e);
    if ((e = cudaMemset(s->full_slots, 0, (size_t)s->nslots * 4u)) != cudaSuccess) return bail("cudaMemset", e);
    if ((e = cudaMalloc(&s->device_errors, 4u)) != cudaSuccess) return bail("cudaMalloc", e);
    if ((e = cudaMemset(s->device_errors, 0, 4u)) != cudaSuccess) return bail("cudaMemset", e);
    if ((e = cudaDeviceSynchronize()) != cudaSuccess) return bail("cudaDeviceSynchronize", e);
    *out = s;
    return LLM_CUDA_OK;
}

int32_t llm_cuda_sampler_destroy(llm_cuda_sampler* s) {
    if (!s) return LLM_CUDA_OK;
    cudaSetDevice(s->device);
    cudaDeviceSynchronize();
    free_all(s);
    delete s;
    return LLM_CUDA_OK;
}

int32_t llm_cuda_device_status(llm_cuda_sampler* s, void* stream, uint32_t* bits_out) {
    if (!s) return fail(nullptr, LLM_CUDA_ERR_BAD_ARGUMENT, "sampler handle is NULL");
    CUDA_TRY(s, cudaSetDevice(s->device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint32_t bits = 0u;
    CUDA_TRY(s, cudaMemcpyAsync(&bits, s->device_errors, 4u, cudaMemcpyDeviceToHost, st));
    CUDA_TRY(s, cudaStreamSynchronize(st));
    if (bits) CUDA_TRY(s, cudaMemsetAsync(s->device_errors, 0, 4u, st));
    if (bits_out) *bits_out = bits;
    if (bits)
        return fail(s, LLM_CUDA_ERR_TIMEOUT, "device status 0x%x:%s%s%s", bits,
                    (bits & LLM_CUDA_STATUS_COPY_TIMEOUT) ? " a bulk copy did not complete within its wait limit;" : "",
                    (bits & LLM_CUDA_STATUS_SLOT_TIMEOUT) ? " no full-ordering slot came free within the wait limit;" : "",
                    (bits & LLM_CUDA_STATUS_CHECK_FAILED) ? " an index check failed;" : "");
    return LLM_CUDA_OK;
}

int32_t llm_cuda_test_hold_full_sort_slots(llm_cuda_sampler* s, uint32_t hold, uint32_t wait_rounds, void* stream) {
    if (!s) return fail(nullptr, LLM_CUDA_ERR_BAD_ARGUMENT, "sampler handle is NULL");
    CUDA_TRY(s, cudaSetDevice(s->device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    CUDA_TRY(s, cudaStreamSynchronize(st));  // no launch is using the slots
    // every byte 1 makes a word nonzero = taken; only 0 counts as free
    CUDA_TRY(s, cudaMemsetAsync(s->full_slots, hold ? 1 : 0, (size_t)s->nslots * 4u, st));
    CUDA_TRY(s, cudaStreamSynchronize(st));
    s->slot_rounds = wait_rounds ? wait_rounds : kSlotRounds;
    return LLM_CUDA_OK;
}

int32_t llm_cuda_last_launch_info(const llm_cuda_sampler* s, uint32_t* kernels_launched, uint32_t* split_used) {
    if (!s) return LLM_CUDA_ERR_BAD_ARGUMENT;
    if (kernels_launched) *kernels_launched = s->last_kernels;
    if (split_used) *split_used = s->last_split;
    return LLM_CUDA_OK;
}

#ifdef LLMC_DEV
// Development builds only (never in the product library): phase timestamps and launch-plan overrides.
int32_t llm_cuda_debug_phase_buffer(llm_cuda_sampler* s, unsigned long long* device_buffer) {
    if (!s) return LLM_CUDA_ERR_BAD_ARGUMENT;
    s->phase_ns = device_buffer;
    return LLM_CUDA_OK;
}
void llm_cuda_dev_set(int32_t key, int32_t value) { llmc::dev_override(key, value); }
#endif

int32_t llm_cuda_sample_batch(llm_cuda_sampler* s, const llm_cuda_sample_args* a) {
    KParams P;
    int32_t rc = fill_params(s, a, true, &P);
    if (rc != LLM_CUDA_OK) return rc;
    if (a->batch && !a->tokens) return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "tokens is NULL");
    if (a->column_offset != 0 || (a->vocab_global != 0 && a->vocab_global != a->vocab))
        return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "column_offset/vocab_global are for llm_cuda_shard_select");
    CUDA_TRY(s, cudaSetDevice(s->device));
    return run_select(s, a, P);
}

int32_t llm_cuda_shard_select(llm_cuda_sampler* s, const llm_cuda_sample_args* a, float* cand_values, uint32_t* cand_ids,
                              uint32_t* cand_count, uint32_t cand_stride) {
    if (s && a && a->struct_size == sizeof(llm_cuda_sample_args) && a->vocab == 0 && cand_count) {
        // a shard past the end of a small vocabulary holds no columns: it contributes empty lists, so that
        // every rank still reaches the exchange
        if (a->batch > s->max_batch) return fail(s, LLM_CUDA_ERR_CAPACITY, "batch %u > max_batch %u", a->batch, s->max_batch);
        CUDA_TRY(s, cudaSetDevice(s->device));
        if (a->batch)
            CUDA_TRY(s, cudaMemsetAsync(cand_count, 0, (size_t)a->batch * 4u, static_cast<cudaStream_t>(a->stream)));
        s->last_kernels = 0;
        return LLM_CUDA_OK;
    }
    KParams P;
    int32_t rc = fill_params(s, a, true, &P);
    if (rc != LLM_CUDA_OK) return rc;
    if (!cand_values || !cand_ids || !cand_count || cand_stride == 0)
        return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "candidate outputs are NULL or cand_stride is 0");
    if (a->top_k_rows) return fail(s, LLM_CUDA_ERR_UNSUPPORTED, "vocabulary sharding takes a scalar top_k");
    if (!scalar_greedy(a)) {
        if (a->top_k == 0) return fail(s, LLM_CUDA_ERR_UNSUPPORTED, "vocabulary sharding needs top_k > 0 (the softmax over an unbounded kept set would need a second exchange)");
        if (a->top_k > cand_stride || a->top_k > kMaxKcap)
            return fail(s, LLM_CUDA_ERR_CAPACITY, "top_k %u exceeds cand_stride %u or the selection capacity %u", a->top_k, cand_stride, kMaxKcap);
    }
    if ((uint64_t)a->column_offset + a->vocab > (uint64_t)P.vocab_global)
        return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "column_offset %u + vocab %u exceeds vocab_global %u", a->column_offset, a->vocab, P.vocab_global);
    P.out_q = cand_values;
    P.out_i = cand_ids;
    P.out_cnt = cand_count;
    P.out_stride = cand_stride;
    P.force_full = 0;
    CUDA_TRY(s, cudaSetDevice(s->device));
    return run_select(s, a, P);
}

namespace {

// The merge step over lists laid out as the two public forms describe.
int32_t run_merge(llm_cuda_sampler* s, const llm_cuda_sample_args* a, const float* cand_values, const uint32_t* cand_ids,
                  const uint32_t* cand_count, uint32_t n_shards, uint32_t cand_stride, uint64_t shard_words,
                  uint64_t cnt_shard, bool lists_sorted = true, uint32_t need = 0u) {
    KParams P;
    int32_t rc = fill_params(s, a, false, &P);
    if (rc != LLM_CUDA_OK) return rc;
    if (!cand_values || !cand_ids || !cand_count || n_shards == 0 || cand_stride == 0)
        return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "candidate inputs are NULL or empty");
    if (a->batch && !a->tokens) return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "tokens is NULL");
    if (a->top_k_rows) return fail(s, LLM_CUDA_ERR_UNSUPPORTED, "vocabulary sharding takes a scalar top_k");
    if (!scalar_greedy(a) && (a->top_k == 0 || a->top_k > kMaxKcap))
        return fail(s, LLM_CUDA_ERR_UNSUPPORTED, "vocabulary sharding needs 0 < top_k <= %u", kMaxKcap);
    if (P.vocab_global == 0) return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "vocab_global (or vocab) must be set");
    if (shard_words > 0xffffffffull || cnt_shard > 0xffffffffull)
        return fail(s, LLM_CUDA_ERR_CAPACITY, "candidate lists of one shard exceed 2^32 words");
    const uint32_t k = scalar_greedy(a) ? 1u : a->top_k;
    const uint32_t k_eff = k >= P.vocab_global ? P.vocab_global : k;
    LaunchPlan plan{};
    plan.kcap = pow2_ceil_u32(k_eff < 64u ? 64u : k_eff);
    plan.ccap = 2u * plan.kcap + 2048u;
    plan.limit = 2u * plan.kcap;
    if (cand_stride > plan.ccap - plan.kcap)
        return fail(s, LLM_CUDA_ERR_CAPACITY, "cand_stride %u too large for the merge buffer (%u)", cand_stride, plan.ccap - plan.kcap);
    P.kcap = plan.kcap;
    P.ccap = plan.ccap;
    P.limit = plan.limit;
    P.split = n_shards;
    P.sc_q = const_cast<float*>(cand_values);
    P.sc_i = const_cast<uint32_t*>(cand_ids);
    P.sc_cnt = const_cast<uint32_t*>(cand_count);
    P.sc_maxkey = nullptr;
    P.sc_stride = cand_stride;
    P.sc_rows = a->batch;
    P.sc_shard_words = (uint32_t)shard_words;
    P.sc_cnt_shard = (uint32_t)cnt_shard;
    P.sc_sorted = lists_sorted ? 1u : 0u;
    P.sc_need = need;
    P.force_full = 0;
    s->last_kernels = 0;
    s->last_split = n_shards;
    if (a->batch == 0) return LLM_CUDA_OK;
    CUDA_TRY(s, cudaSetDevice(s->device));
    CUDA_TRY(s, launch_merge_draw(P, plan, static_cast<cudaStream_t>(a->stream)));
    s->last_kernels = 1;
    return LLM_CUDA_OK;
}

}  // namespace

int32_t llm_cuda_merge_draw(llm_cuda_sampler* s, const llm_cuda_sample_args* a, const float* cand_values,
                            const uint32_t* cand_ids, const uint32_t* cand_count, uint32_t n_shards, uint32_t cand_stride) {
    const uint64_t B = a ? a->batch : 0u;
    return run_merge(s, a, cand_values, cand_ids, cand_count, n_shards, cand_stride, B * cand_stride, B);
}

size_t llm_cuda_packed_candidates_bytes(uint32_t batch, uint32_t cand_stride) {
    return ((size_t)2u * batch * cand_stride + batch) * 4u;
}

int32_t llm_cuda_shard_select_packed(llm_cuda_sampler* s, const llm_cuda_sample_args* a, void* packed_out, uint32_t cand_stride) {
    if (!s) return fail(nullptr, LLM_CUDA_ERR_BAD_ARGUMENT, "sampler handle is NULL");
    if (!a || !packed_out) return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "args or packed_out is NULL");
    float* values = static_cast<float*>(packed_out);
    uint32_t* ids = reinterpret_cast<uint32_t*>(values) + (size_t)a->batch * cand_stride;
    uint32_t* counts = ids + (size_t)a->batch * cand_stride;
    return llm_cuda_shard_select(s, a, values, ids, counts, cand_stride);
}

int32_t llm_cuda_merge_draw_packed(llm_cuda_sampler* s, const llm_cuda_sample_args* a, const void* packed_all, uint32_t n_shards,
                                   uint32_t cand_stride) {
    if (!s) return fail(nullptr, LLM_CUDA_ERR_BAD_ARGUMENT, "sampler handle is NULL");
    if (!a || !packed_all) return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "args or packed_all is NULL");
    const uint64_t B = a->batch;
    const uint64_t block = 2u * B * cand_stride + B;  // words per shard
    const float* values = static_cast<const float*>(packed_all);
    const uint32_t* ids = reinterpret_cast<const uint32_t*>(values) + B * cand_stride;
    const uint32_t* counts = ids + B * cand_stride;
    return run_merge(s, a, values, ids, counts, n_shards, cand_stride, block, block);
}

int32_t llm_cuda_lm_head_sample(llm_cuda_sampler* s, const llm_cuda_lm_head_args* a) {
    if (!s) return fail(nullptr, LLM_CUDA_ERR_BAD_ARGUMENT, "sampler handle is NULL");
    if (!a) return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "args is NULL");
    if (a->struct_size != sizeof(llm_cuda_lm_head_args))
        return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "struct_size %u, expected %zu", a->struct_size, sizeof(llm_cuda_lm_head_args));
    if (a->batch == 0) return LLM_CUDA_OK;
    if (!a->hidden || !a->embed || !a->tokens) return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "hidden, embed or tokens is NULL");
    if (a->batch > 256u || a->batch > s->max_batch)
        return fail(s, LLM_CUDA_ERR_CAPACITY, "batch %u beyond 256 (one tensor-core tile) or the handle's max_batch", a->batch);
    if (a->vocab == 0 || a->hidden_dim == 0 || a->hidden_dim % 8u)
        return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "vocab and hidden_dim must be > 0 and hidden_dim a multiple of 8 (16-byte rows for TMA)");
    if ((reinterpret_cast<uintptr_t>(a->embed) & 15u) || (reinterpret_cast<uintptr_t>(a->hidden) & 15u) ||
        (reinterpret_cast<uintptr_t>(a->norm_gain) & 15u))
        return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "embed, hidden and norm_gain must be 16-byte aligned");
    if (a->temperature != a->temperature) return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "temperature is NaN");
    const bool greedy = a->temperature <= 0.0f;
    if (!greedy && (a->top_k == 0 || a->top_k > 256u))
        return fail(s, LLM_CUDA_ERR_UNSUPPORTED, "the fused LM head samples rows with 0 < top_k <= 256 (or greedy); top_k %u needs the logits and llm_cuda_sample_batch", a->top_k);
    if ((a->kept_ids || a->kept_probs) && a->kept_capacity == 0)
        return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "kept_ids/kept_probs given with kept_capacity 0");
    CUDA_TRY(s, cudaSetDevice(s->device));
    cudaStream_t st = static_cast<cudaStream_t>(a->stream);
    const uint32_t B = a->batch, V = a->vocab, H = a->hidden_dim;
    const uint32_t n_pad = (B + 15u) & ~15u;
    const uint32_t k = greedy ? 1u : a->top_k;
    const uint32_t n_tiles = (V + 127u) / 128u;
    // small vocabularies are probed whole: the thresholds are then exact and the main step has nothing to do
    const uint32_t probe_every = n_tiles >= 64u ? kLmProbeEvery : 1u;
    const uint32_t n_probe = (n_tiles + probe_every - 1u) / probe_every;
    const uint32_t probe_cols = n_probe * 128u;
    if (!s->lm_configured) {
        CUDA_TRY(s, lm_head_configure(s->dev.max_dyn_smem));
        CUDA_TRY(s, cudaMalloc(&s->lm_thr, 256u * 4u));
        CUDA_TRY(s, cudaMalloc(&s->lm_cand_q, (size_t)256u * kLmCandCap * 4u));
        CUDA_TRY(s, cudaMalloc(&s->lm_cand_i, (size_t)256u * kLmCandCap * 4u));
        CUDA_TRY(s, cudaMalloc(&s->lm_cand_count, 256u * 4u));
        s->lm_configured = true;
    }
    const size_t xnorm_bytes = (size_t)n_pad * H * 2u, probe_bytes = (size_t)B * probe_cols * 4u;
    if (xnorm_bytes > s->lm_xnorm_bytes || probe_bytes > s->lm_probe_bytes) {
        CUDA_TRY(s, cudaStreamSynchronize(st));  // nothing may still be using the old buffers
        if (xnorm_bytes > s->lm_xnorm_bytes) {
            cudaFree(s->lm_xnorm);
            s->lm_xnorm = nullptr;
            s->lm_xnorm_bytes = 0;
            CUDA_TRY(s, cudaMalloc(&s->lm_xnorm, xnorm_bytes));
            s->lm_xnorm_bytes = xnorm_bytes;
        }
        if (probe_bytes > s->lm_probe_bytes) {
            cudaFree(s->lm_probe);
            s->lm_probe = nullptr;
            s->lm_probe_bytes = 0;
            CUDA_TRY(s, cudaMalloc(&s->lm_probe, probe_bytes));
            s->lm_probe_bytes = probe_bytes;
        }
    }
    // up to 128 rows: two CTAs per SM, each with half of the SM's shared memory and tensor memory
    const uint32_t ctas_per_sm = n_pad <= 128u ? 2u : 1u;
    const uint32_t stages = lm_head_stages(n_pad, ctas_per_sm == 2u ? (s->dev.max_dyn_smem - 8192u) / 2u : s->dev.max_dyn_smem);
    if (stages < 2u) return fail(s, LLM_CUDA_ERR_CAPACITY, "shared memory for batch %u does not fit", B);

    LmParams P;
    memset(&P, 0, sizeof(P));
    P.vocab = V;
    P.batch = B;
    P.n_pad = n_pad;
    P.k_chunks = (H + 63u) / 64u;
    P.probe_every = probe_every;
    P.stages = stages;
    P.tmem_cols = ctas_per_sm == 2u ? 256u : 512u;
    P.ctas_per_sm = ctas_per_sm;
    P.temperature = greedy ? 1.0f : a->temperature;
    P.thr = s->lm_thr;
    P.probe_out = s->lm_probe;
    P.probe_cols = probe_cols;
    P.cand_q = s->lm_cand_q;
    P.cand_i = s->lm_cand_i;
    P.cand_count = s->lm_cand_count;
    P.cand_cap = kLmCandCap;
    P.logits_out = a->logits_out;
    P.device_errors = s->device_errors;

    s->last_kernels = 0;
    CUDA_TRY(s, launch_rmsnorm_bf16(static_cast<const float*>(a->hidden), a->norm_gain, a->norm_eps, B, n_pad, H, s->lm_xnorm,
                                    s->lm_cand_count, st));
    cudaError_t ce = cudaSuccess;
    P.phase = LM_PHASE_PROBE;
    P.n_items = n_probe;
    int rc = launch_lm_head(P, a->embed, s->lm_xnorm, H, s->dev.sm_count, st, &ce);
    if (rc == -1) return fail(s, LLM_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled is unavailable or rejected the matrices");
    if (rc != 0) return fail(s, LLM_CUDA_ERR_CUDA, "lm_head_kernel (probe): %s", cudaGetErrorString(ce));
    // the r-th largest of a row's probed logits stands at about rank r * probe_every in the whole row: r is chosen
    // so that this is 2-3 times top_k plus a margin; the merge step reports the rows where it still fell short
    uint32_t rank = probe_every == 1u ? k : 2u * ((k + probe_every - 1u) / probe_every) + 8u;
    if (rank > probe_cols) rank = probe_cols;
    CUDA_TRY(s, launch_probe_threshold(P, rank, probe_every == 1u, st));
    P.phase = LM_PHASE_MAIN;
    P.n_items = n_tiles - n_probe;
    rc = launch_lm_head(P, a->embed, s->lm_xnorm, H, s->dev.sm_count, st, &ce);
    if (rc != 0) return fail(s, LLM_CUDA_ERR_CUDA, "lm_head_kernel (main): %s", cudaGetErrorString(ce));

    // the sampler's own merge + ordered tail over one unordered candidate list per row
    llm_cuda_sample_args m;
    memset(&m, 0, sizeof(m));
    m.struct_size = sizeof(m);
    m.logits_dtype = LLM_CUDA_DTYPE_F32;
    m.batch = B;
    m.vocab_global = V;
    m.temperature = a->temperature;
    m.top_k = a->top_k;
    m.top_p = a->top_p;
    m.min_p = a->min_p;
    m.repetition_penalty = 1.0f;
    m.eos_id = LLM_CUDA_EOS_DEFAULT;
    m.seeds = a->seeds;
    m.draw_index = a->draw_index;
    m.seed_base = a->seed_base;
    m.uniforms = a->uniforms;
    m.tokens = a->tokens;
    m.row_flags = a->row_flags;
    m.kept_count = a->kept_count;
    m.kept_ids = a->kept_ids;
    m.kept_probs = a->kept_probs;
    m.kept_capacity = a->kept_capacity;
    m.row_stats = a->row_stats;
    m.stream = a->stream;
    const int32_t mr = run_merge(s, &m, s->lm_cand_q, s->lm_cand_i, s->lm_cand_count, 1u, kLmCandCap, (uint64_t)B * kLmCandCap, B,
                                 /*lists_sorted=*/false, /*need=*/k < V ? k : V);
    if (mr != LLM_CUDA_OK) return mr;
    s->last_kernels = P.n_items ? 5u : 4u;
    return LLM_CUDA_OK;
}

int32_t llm_cuda_advance_rows(llm_cuda_sampler* s, uint32_t batch, const uint32_t* tokens, const uint32_t* row_flags,
                              uint32_t* history, uint32_t history_stride, uint32_t window, uint32_t* history_len,
                              uint32_t* history_pos, uint64_t* draw_index, uint8_t* finished, uint32_t eos_id, void* stream) {
    if (!s) return fail(nullptr, LLM_CUDA_ERR_BAD_ARGUMENT, "sampler handle is NULL");
    if (batch && !tokens) return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "tokens is NULL");
    if (history && !history_len) return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "history given without history_len");
    // without a write position a full ring could only ever replace one slot and the window would go stale
    if (history && !history_pos) return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "history given without history_pos");
    CUDA_TRY(s, cudaSetDevice(s->device));
    CUDA_TRY(s, launch_advance_rows(batch, tokens, row_flags, history, history_stride, window, history_len, history_pos,
                                    draw_index, finished, eos_id, static_cast<cudaStream_t>(stream)));
    return LLM_CUDA_OK;
}

int32_t llm_cuda_pack_allowed(llm_cuda_sampler* s, const uint8_t* allowed_host, uint32_t n, uint32_t* bits_out, void* stream) {
    if (!s) return fail(nullptr, LLM_CUDA_ERR_BAD_ARGUMENT, "sampler handle is NULL");
    if (n && (!allowed_host || !bits_out)) return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "allowed_host or bits_out is NULL");
    if (n == 0) return LLM_CUDA_OK;
    CUDA_TRY(s, cudaSetDevice(s->device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (s->arena_bytes < n) {
        CUDA_TRY(s, cudaStreamSynchronize(st));
        cudaFree(s->arena);
        s->arena = nullptr;
        s->arena_bytes = 0;
        CUDA_TRY(s, cudaMalloc(&s->arena, (size_t)n));
        s->arena_bytes = n;
    }
    CUDA_TRY(s, cudaMemcpyAsync(s->arena, allowed_host, n, cudaMemcpyHostToDevice, st));
    CUDA_TRY(s, launch_pack_allowed(s->arena, n, bits_out, st));
    CUDA_TRY(s, cudaStreamSynchronize(st));  // the staging buffer is reused by the next host-buffer call
    return LLM_CUDA_OK;
}

int32_t llm_cuda_cross_entropy(llm_cuda_sampler* s, const float* logits, uint32_t rows, uint32_t vocab, uint32_t row_stride_elems,
                               const uint32_t* targets, float* row_loss, float* d_logits, void* stream) {
    if (!s) return fail(nullptr, LLM_CUDA_ERR_BAD_ARGUMENT, "sampler handle is NULL");
    if (rows == 0u) return LLM_CUDA_OK;
    if (!logits || !targets || !row_loss) return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "logits, targets or row_loss is NULL");
    if (vocab == 0u) return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "vocab is 0");
    const uint32_t stride = row_stride_elems ? row_stride_elems : vocab;
    if (stride < vocab) return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "row stride %u below vocab %u", stride, vocab);
    if ((reinterpret_cast<uintptr_t>(logits) & 3u) || (d_logits && (reinterpret_cast<uintptr_t>(d_logits) & 3u)))
        return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "logits or d_logits pointer not 4-byte aligned");
    // the gradient is written with the same split into leading elements and 16-byte vectors as the row is read
    if (d_logits && ((reinterpret_cast<uintptr_t>(logits) ^ reinterpret_cast<uintptr_t>(d_logits)) & 15u))
        return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "d_logits must share the logits' alignment modulo 16 bytes");
    CUDA_TRY(s, cudaSetDevice(s->device));
    CUDA_TRY(s, llmc::launch_cross_entropy_rows(logits, rows, vocab, stride, targets, row_loss, d_logits, static_cast<cudaStream_t>(stream)));
    return LLM_CUDA_OK;
}

int32_t llm_cuda_sample_batch_host(llm_cuda_sampler* s, const llm_cuda_sample_args* h) {
    if (!s) return fail(nullptr, LLM_CUDA_ERR_BAD_ARGUMENT, "sampler handle is NULL");
    if (!h) return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "args is NULL");
    if (h->struct_size != sizeof(llm_cuda_sample_args))
        return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "struct_size %u, expected %zu", h->struct_size, sizeof(llm_cuda_sample_args));
    if (h->batch > s->max_batch) return fail(s, LLM_CUDA_ERR_CAPACITY, "batch %u > max_batch %u", h->batch, s->max_batch);
    if (h->vocab == 0 || h->vocab > s->max_vocab) return fail(s, LLM_CUDA_ERR_CAPACITY, "vocab %u outside 1..%u", h->vocab, s->max_vocab);
    if (h->batch == 0) return LLM_CUDA_OK;
    if (!h->logits || !h->tokens) return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "logits or tokens is NULL");
    if (h->row_stride_elems != 0 && h->row_stride_elems < h->vocab) return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "row_stride_elems < vocab");
    CUDA_TRY(s, cudaSetDevice(s->device));
    cudaStream_t st = static_cast<cudaStream_t>(h->stream);
    const size_t B = h->batch;
    const size_t esz = h->logits_dtype == LLM_CUDA_DTYPE_BF16 ? 2 : 4;
    const size_t logits_rows = h->row_stride_elems == 0 ? 1 : B;
    const size_t logits_bytes = (logits_rows - 1) * h->row_stride_elems * esz + (size_t)h->vocab * esz;
    const size_t hist_bytes = h->history ? B * h->history_stride * 4u : 0;
    const size_t mask_bytes = h->allowed_bits ? ((size_t)(h->allowed_len + 31u) / 32u) * 4u : 0;
    const size_t kept_elems = (h->kept_ids || h->kept_probs) ? B * h->kept_capacity : 0;
    // two passes over the same carving: measure, then assign
    llm_cuda_sample_args d = *h;
    for (int pass = 0; pass < 2; ++pass) {
        Carver c{pass ? s->arena : nullptr};
        d.logits = c.take(logits_bytes);
        d.temperature_rows = h->temperature_rows ? (const float*)c.take(B * 4) : nullptr;
        d.top_k_rows = h->top_k_rows ? (const uint32_t*)c.take(B * 4) : nullptr;
        d.top_p_rows = h->top_p_rows ? (const float*)c.take(B * 4) : nullptr;
        d.min_p_rows = h->min_p_rows ? (const float*)c.take(B * 4) : nullptr;
        d.repetition_penalty_rows = h->repetition_penalty_rows ? (const float*)c.take(B * 4) : nullptr;
        d.history = h->history ? (const uint32_t*)c.take(hist_bytes) : nullptr;
        d.history_len_rows = h->history_len_rows ? (const uint32_t*)c.take(B * 4) : nullptr;
        d.allowed_bits = h->allowed_bits ? (const uint32_t*)c.take(mask_bytes) : nullptr;
        d.seeds = h->seeds ? (const uint64_t*)c.take(B * 8) : nullptr;
        d.draw_index = h->draw_index ? (const uint64_t*)c.take(B * 8) : nullptr;
        d.uniforms = h->uniforms ? (const float*)c.take(B * 4) : nullptr;
        d.tokens = (uint32_t*)c.take(B * 4);
        d.row_flags = h->row_flags ? (uint32_t*)c.take(B * 4) : nullptr;
        d.kept_count = h->kept_count ? (uint32_t*)c.take(B * 4) : nullptr;
        d.kept_ids = h->kept_ids ? (uint32_t*)c.take(kept_elems * 4) : nullptr;
        d.kept_probs = h->kept_probs ? (float*)c.take(kept_elems * 4) : nullptr;
        d.row_stats = h->row_stats ? (float*)c.take(B * LLM_CUDA_ROW_STATS * 4) : nullptr;
        d.penalized_out = (h->penalized_out && h->history) ? (float*)c.take(hist_bytes) : nullptr;
        if (pass == 0 && c.off > s->arena_bytes) {
            CUDA_TRY(s, cudaStreamSynchronize(st));
            cudaFree(s->arena);
            s->arena = nullptr;
            s->arena_bytes = 0;
            CUDA_TRY(s, cudaMalloc(&s->arena, c.off));
            s->arena_bytes = c.off;
        }
    }
    auto up = [&](const void* dst, const void* src, size_t bytes) -> cudaError_t {
        if (!src || bytes == 0) return cudaSuccess;
        return cudaMemcpyAsync(const_cast<void*>(dst), src, bytes, cudaMemcpyHostToDevice, st);
    };
    CUDA_TRY(s, up(d.logits, h->logits, logits_bytes));
    CUDA_TRY(s, up(d.temperature_rows, h->temperature_rows, B * 4));
    CUDA_TRY(s, up(d.top_k_rows, h->top_k_rows, B * 4));
    CUDA_TRY(s, up(d.top_p_rows, h->top_p_rows, B * 4));
    CUDA_TRY(s, up(d.min_p_rows, h->min_p_rows, B * 4));
    CUDA_TRY(s, up(d.repetition_penalty_rows, h->repetition_penalty_rows, B * 4));
    CUDA_TRY(s, up(d.history, h->history, hist_bytes));
    CUDA_TRY(s, up(d.history_len_rows, h->history_len_rows, B * 4));
    CUDA_TRY(s, up(d.allowed_bits, h->allowed_bits, mask_bytes));
    CUDA_TRY(s, up(d.seeds, h->seeds, B * 8));
    CUDA_TRY(s, up(d.draw_index, h->draw_index, B * 8));
    CUDA_TRY(s, up(d.uniforms, h->uniforms, B * 4));
    int32_t rc = llm_cuda_sample_batch(s, &d);
    if (rc != LLM_CUDA_OK) return rc;
    auto down = [&](void* dst, const void* src, size_t bytes) -> cudaError_t {
        if (!dst || !src || bytes == 0) return cudaSuccess;
        return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, st);
    };
    CUDA_TRY(s, down(h->tokens, d.tokens, B * 4));
    CUDA_TRY(s, down(h->row_flags, d.row_flags, B * 4));
    CUDA_TRY(s, down(h->kept_count, d.kept_count, B * 4));
    CUDA_TRY(s, down(h->kept_ids, d.kept_ids, kept_elems * 4));
    CUDA_TRY(s, down(h->kept_probs, d.kept_probs, kept_elems * 4));
    CUDA_TRY(s, down(h->row_stats, d.row_stats, B * LLM_CUDA_ROW_STATS * 4));
    CUDA_TRY(s, down(h->penalized_out, d.penalized_out, hist_bytes));
    // synchronises the stream; a bounded wait that ran out inside the kernel becomes LLM_CUDA_ERR_TIMEOUT
    return llm_cuda_device_status(s, h->stream, nullptr);
}

int32_t llm_cuda_sample_with(llm_cuda_sampler* s, const float* logits, uint32_t vocab, const llm_cuda_sampling_config* cfg,
                             const uint32_t* recent, uint32_t n_recent, uint64_t* rng_state, uint32_t* token_out) {
    if (!s) return fail(nullptr, LLM_CUDA_ERR_BAD_ARGUMENT, "sampler handle is NULL");
    if (!logits || !cfg || !rng_state || !token_out) return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "NULL argument");
    if (n_recent && !recent) return fail(s, LLM_CUDA_ERR_BAD_ARGUMENT, "recent is NULL with n_recent > 0");
    if (n_recent > s->max_history) return fail(s, LLM_CUDA_ERR_CAPACITY, "history %u > max_history %u", n_recent, s->max_history);
    std::vector<uint32_t> bits;
    llm_cuda_sample_args a;
    memset(&a, 0, sizeof(a));
    a.struct_size = sizeof(a);
    a.logits_dtype = LLM_CUDA_DTYPE_F32;
    a.logits = logits;
    a.batch = 1;
    a.vocab = vocab;
    a.row_stride_elems = vocab;
    a.temperature = cfg->temperature;
    a.top_k = cfg->top_k;
    a.top_p = cfg->top_p;
    a.min_p = cfg->min_p;
    a.repetition_penalty = cfg->repetition_penalty;
    if (n_recent) {
        a.history = recent;
        a.history_stride = n_recent;
        a.history_len = n_recent;
    }
    if (cfg->allowed) {
        const uint32_t n = cfg->allowed_len;
        bits.assign((n + 31u) / 32u, 0u);
        for (uint32_t i = 0; i < n; ++i)
            if (cfg->allowed[i]) bits[i >> 5] |= 1u << (i & 31u);
        for (uint32_t i = n; i < (uint32_t)bits.size() * 32u; ++i) bits[i >> 5] |= 1u << (i & 31u);
        if (!bits.empty()) {
            a.allowed_bits = bits.data();
            a.allowed_len = n;
        }
    }
    a.eos_id = LLM_CUDA_EOS_DEFAULT;
    a.seed_base = *rng_state;  // row 0 draws output 1 of an Rng whose state is *rng_state
    uint32_t flags = 0;
    a.tokens = token_out;
    a.row_flags = &flags;
    int32_t rc = llm_cuda_sample_batch_host(s, &a);
    if (rc != LLM_CUDA_OK) return rc;
    if (flags & LLM_CUDA_ROW_DRAW_CONSUMED) *rng_state += kGamma;  // rng.rs:17
    return LLM_CUDA_OK;
}

int32_t llm_cuda_sample(llm_cuda_sampler* s, const float* logits, uint32_t vocab, float temperature, uint64_t* rng_state,
                        uint32_t* token_out) {
    llm_cuda_sampling_config cfg;
    llm_cuda_sampling_config_default(&cfg);
    cfg.temperature = temperature;  // generate.rs:423-433: everything else off
    cfg.top_k = 0;
    cfg.top_p = 1.0f;
    cfg.min_p = 0.0f;
    cfg.repetition_penalty = 1.0f;
    return llm_cuda_sample_with(s, logits, vocab, &cfg, nullptr, 0, rng_state, token_out);
}

}  // extern "C"
