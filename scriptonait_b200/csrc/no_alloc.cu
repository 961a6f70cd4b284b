// llm_cuda_sample_batch_static: the batched sampler for callers that must not allocate.
//
// Who that is: code running where cudaMalloc / cudaFree are off limits - inside a serving
// loop whose memory is carved up once at start-up and then frozen, under a framework that
// owns the allocator and forbids side allocations, or in a plugin that is handed device
// pointers and a stream and nothing else. llm_cuda_sampler_create sizes and allocates the
// scratch the streaming kernel needs when several CTAs share one row (their candidate
// lists, counts, maxima and one ticket per row); this entry point takes no handle and keeps
// that scratch in a fixed array inside the library image instead.
//
// The price: the array has a fixed, modest size (see the limits below), every GPU that
// loads the library carries it until the process exits, and every call shares it - two
// calls that overlap on the GPU (different streams, different host threads) would race on
// it, so calls must be serialised by the caller (one stream, or events between streams).
// The array keeps whatever the previous call left; the only part that must start at zero,
// the per-row tickets, is cleared on the stream at the start of every call.
//
// The first call on a device sets that device up (the address of the array is looked up with
// cudaGetSymbolAddress while the device is current, and the kernels' shared-memory limit is
// raised). It does this once per device; make that first call before starting any stream
// capture.
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include "../../include/llm_cuda.h"
#include "sampler_kernels.h"

using namespace llmc;

namespace {

constexpr uint32_t kMaxBatch = LLM_CUDA_STATIC_MAX_BATCH;       // rows per call
constexpr uint32_t kMaxTopK = LLM_CUDA_STATIC_MAX_TOP_K;        // exact-selection rows only
constexpr uint32_t kMaxHistory = LLM_CUDA_STATIC_MAX_HISTORY;   // history entries per row
constexpr uint32_t kListLen = 2u * kMaxTopK;                    // entries per candidate list
constexpr uint32_t kMaxLists = 256u;                            // lists (= CTAs of split rows) per call
constexpr size_t kOffValues = 0;
constexpr size_t kOffIds = kOffValues + (size_t)kMaxLists * kListLen * 4u;
constexpr size_t kOffCounts = kOffIds + (size_t)kMaxLists * kListLen * 4u;
constexpr size_t kOffMaxima = kOffCounts + (size_t)kMaxLists * 4u;
constexpr size_t kOffTickets = kOffMaxima + (size_t)kMaxLists * 4u;
constexpr size_t kScratchBytes = kOffTickets + (size_t)kMaxBatch * 4u;  // 1 050 880 bytes

// The scratch itself. In host code this name is only a stand-in for the symbol - it is not
// a device address and must never be handed to a kernel; device_scratch() below asks the
// runtime for the real address, per device.
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
struct PerDevice {
    bool ready = false;
    unsigned char* scratch = nullptr;
    DeviceInfo info{};
};
PerDevice g_devices[kMaxDevices];
char g_static_error[512] = "";

int32_t fail(int32_t code, const char* fmt, const char* a = "", unsigned long long x = 0, unsigned long long y = 0) {
    snprintf(g_static_error, sizeof(g_static_error), fmt, a, x, y);
    return code;
}

// Once per device, with that device current: the device address of the static array.
int32_t device_scratch(int device, PerDevice** out) {
    if (device < 0 || device >= kMaxDevices) return fail(LLM_CUDA_ERR_BAD_ARGUMENT, "device %s%llu out of range", "", (unsigned long long)device);
    PerDevice& d = g_devices[device];
    if (!d.ready) {
        cudaError_t e = cudaSetDevice(device);
        if (e != cudaSuccess) return fail(LLM_CUDA_ERR_NO_DEVICE, "cudaSetDevice: %s", cudaGetErrorString(e));
        cudaDeviceProp prop{};
        e = cudaGetDeviceProperties(&prop, device);
        if (e != cudaSuccess) return fail(LLM_CUDA_ERR_CUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
        if (prop.major != 10) return fail(LLM_CUDA_ERR_NO_DEVICE, "device is not sm_100%s", "");
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || p == nullptr) return fail(LLM_CUDA_ERR_CUDA, "cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        d.scratch = static_cast<unsigned char*>(p);
        d.info.sm_count = (uint32_t)prop.multiProcessorCount;
        d.info.max_dyn_smem = (size_t)prop.sharedMemPerBlockOptin - 4096u;
        e = configure_kernels(d.info.max_dyn_smem);
        if (e != cudaSuccess) return fail(LLM_CUDA_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        d.ready = true;
    }
    *out = &d;
    return LLM_CUDA_OK;
}

}  // namespace

extern "C" {

const char* llm_cuda_static_last_error(void) { return g_static_error; }

int32_t llm_cuda_sample_batch_static(int32_t device, const llm_cuda_sample_args* a) {
    {   // the checks the handle-based entry point makes too: pointers and their alignment, strides, NaN scalars
        const int32_t rc = validate_sample_args(a, true, g_static_error, sizeof(g_static_error));
        if (rc != LLM_CUDA_OK) return rc;
    }
    if (a->batch == 0) return LLM_CUDA_OK;
    if (!a->tokens) return fail(LLM_CUDA_ERR_BAD_ARGUMENT, "tokens is NULL%s");
    // ---- the limits of the fixed scratch, stated in the header
    if (a->batch > kMaxBatch)
        return fail(LLM_CUDA_ERR_CAPACITY, "batch %s%llu exceeds the static limit %llu", "", a->batch, kMaxBatch);
    if (a->top_k_rows || a->temperature_rows)
        return fail(LLM_CUDA_ERR_UNSUPPORTED, "per-row top_k / temperature arrays are not available without a handle%s");
    const bool greedy = a->temperature <= 0.0f;
    if (!greedy && (a->top_k == 0 || a->top_k > kMaxTopK))
        return fail(LLM_CUDA_ERR_CAPACITY, "top_k %s%llu outside 1..%llu: rows that need the window or the full-sort stage need a handle", "",
                    a->top_k, kMaxTopK);
    if (a->allowed_bits) return fail(LLM_CUDA_ERR_UNSUPPORTED, "the allowed mask can need the full-sort stage, which needs a handle%s");
    if (a->force_full_sort || a->column_offset || (a->vocab_global && a->vocab_global != a->vocab))
        return fail(LLM_CUDA_ERR_UNSUPPORTED, "full-sort and vocabulary sharding need a handle%s");
    uint32_t hist = 0;
    if (a->history) {
        hist = a->history_len_rows ? a->history_stride : a->history_len;
        if (hist > kMaxHistory) return fail(LLM_CUDA_ERR_CAPACITY, "history %s%llu exceeds the static limit %llu", "", hist, kMaxHistory);
    }

    PerDevice* d = nullptr;
    int32_t rc = device_scratch(device, &d);
    if (rc != LLM_CUDA_OK) return rc;
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return fail(LLM_CUDA_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(e));

    KParams P;
    memset(&P, 0, sizeof(P));
    P.logits = a->logits;
    P.row_stride = a->row_stride_elems;
    P.batch = a->batch;
    P.vocab = a->vocab;
    P.dtype = a->logits_dtype;
    P.temperature = a->temperature;
    P.top_p = a->top_p;
    P.min_p = a->min_p;
    P.penalty = a->repetition_penalty;
    P.top_k = a->top_k;
    P.p_rows = a->top_p_rows;
    P.m_rows = a->min_p_rows;
    P.r_rows = a->repetition_penalty_rows;
    P.history = a->history;
    P.hist_stride = a->history_stride;
    P.hist_len = a->history_len;
    P.hist_len_rows = a->history_len_rows;
    P.eos_id = a->eos_id;
    P.seeds = a->seeds;
    P.draw_index = a->draw_index;
    P.seed_base = a->seed_base;
    P.uniforms = a->uniforms;
    P.tokens = a->tokens;
    P.row_flags = a->row_flags;
    P.kept_count = a->kept_count;
    P.kept_ids = a->kept_ids;
    P.kept_probs = a->kept_probs;
    P.kept_cap = (a->kept_ids || a->kept_probs) ? a->kept_capacity : 0u;
    P.row_stats = a->row_stats;
    P.vocab_global = a->vocab;
    // no full-sort stage here: full_keys stays NULL and such a row would be flagged, but the
    // checks above leave only rows that exact selection always resolves

    LaunchPlan plan{};
    const uint32_t k_hint = greedy ? 1u : a->top_k;
    const uint32_t max_lists = kMaxLists;
    if (plan_launch(d->info, P, true, k_hint, kMaxTopK, kMaxHistory, a->split, max_lists, &plan) != 0)
        return fail(LLM_CUDA_ERR_CAPACITY, "shared-memory layout does not fit%s");
    // the fixed lists are shorter than the handle's; a lower compaction trigger is always valid
    // as long as it leaves room for the kept set
    const uint32_t limit = plan.limit < kListLen ? plan.limit : kListLen;
    if (limit < 2u * plan.kcap) return fail(LLM_CUDA_ERR_CAPACITY, "candidate lists exceed the static scratch%s");
    apply_plan(plan, &P);
    P.limit = limit;
    P.sc_q = reinterpret_cast<float*>(d->scratch + kOffValues);
    P.sc_i = reinterpret_cast<uint32_t*>(d->scratch + kOffIds);
    P.sc_cnt = reinterpret_cast<uint32_t*>(d->scratch + kOffCounts);
    P.sc_maxkey = reinterpret_cast<uint32_t*>(d->scratch + kOffMaxima);
    P.sc_ticket = reinterpret_cast<uint32_t*>(d->scratch + kOffTickets);
    P.sc_stride = limit;
    P.sc_rows = P.batch;
    P.sc_shard_words = P.sc_rows * P.sc_stride;
    P.sc_cnt_shard = P.sc_rows;
    cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
    // the tickets are the one part of the shared array that must start at zero
    e = cudaMemsetAsync(P.sc_ticket, 0, (size_t)kMaxBatch * 4u, stream);
    if (e != cudaSuccess) return fail(LLM_CUDA_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
    e = launch_stream_select(P, plan, stream);
    if (e != cudaSuccess) return fail(LLM_CUDA_ERR_CUDA, "kernel launch: %s", cudaGetErrorString(e));
    return LLM_CUDA_OK;
}

}  // extern "C"
