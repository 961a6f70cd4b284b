// Host-visible declarations of the sampler kernels: the parameter block every
// kernel receives, the launch plan, and the launchers the C ABI calls.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

struct llm_cuda_sample_args;

namespace llmc {

// Argument checks every entry point that takes a device-pointer argument block shares: block size,
// dtype, pointers and their alignment, strides, history bounds, NaN scalars. Returns 0, or a negative
// LLM_CUDA_ERR_* with its text in `err`. Limits that depend on who owns the scratch (batch, vocabulary,
// history, rank cut) are checked by the callers.
int validate_sample_args(const llm_cuda_sample_args* a, bool needs_logits, char* err, size_t err_len);

struct KParams {
    const void* logits;
    uint64_t row_stride;
    uint32_t batch, vocab, dtype;
    float temperature, top_p, min_p, penalty;
    uint32_t top_k;
    const float* t_rows;
    const uint32_t* k_rows;
    const float* p_rows;
    const float* m_rows;
    const float* r_rows;
    const uint32_t* history;
    uint32_t hist_stride, hist_len;
    const uint32_t* hist_len_rows;
    const uint32_t* allowed_bits;
    uint32_t allowed_len, eos_id;
    const uint64_t* seeds;
    const uint64_t* draw_index;
    uint64_t seed_base;
    const float* uniforms;
    uint32_t* tokens;
    uint32_t* row_flags;
    uint32_t* kept_count;
    uint32_t* kept_ids;
    float* kept_probs;
    uint32_t kept_cap;
    float* row_stats;
    uint32_t col_offset, vocab_global;
    // launch geometry
    uint32_t split, shard_cols;
    uint32_t kcap, ccap, limit;     // kcap: exact-selection capacity; ccap: buffer entries; limit: compaction trigger
    uint32_t hash_slots, bitmap_words, groups;   // groups: flag words (one per 32 vectors) the layout holds
    uint32_t cand_off, scratch_off, tables_off;  // byte offsets into the kernel's dynamic shared memory
    uint32_t vlist_cap;             // flagged vectors the revisit list can hold
    uint32_t lane_top_words;        // floats of shared memory for the lanes' best values (rank cuts above 256), else 0
    // scratch shared by the CTAs of one row when split > 1 (also the input of merge_draw)
    float* sc_q;                    // [shard][row][sc_stride]   (element (s, b, i) at (s*sc_rows + b)*sc_stride + i)
    uint32_t* sc_i;
    uint32_t* sc_cnt;               // [shard][row]
    uint32_t* sc_maxkey;            // [shard][row] ordered key of the shard's maximum q
    uint32_t* sc_ticket;            // [row]
    uint32_t sc_stride, sc_rows;
    // where shard s keeps its lists: values / ids of row b at sc_q / sc_i + s*sc_shard_words + b*sc_stride, its
    // count at sc_cnt[s*sc_cnt_shard + b] (sc_rows*sc_stride and sc_rows for separate arrays; one packed block per
    // shard - values, ids, counts - has the block's length in both)
    uint32_t sc_shard_words, sc_cnt_shard;
    uint32_t sc_sorted;             // merge_draw: every gathered list is in the reference order (best first)
    uint32_t sc_need;               // merge_draw: nonzero = a list with fewer entries than this, or more than sc_stride, cannot decide its row
    // candidate lists out (vocabulary sharding step 1); NULL = draw a token
    float* out_q;
    uint32_t* out_i;
    uint32_t* out_cnt;
    uint32_t out_stride;
    uint32_t force_full;
    uint32_t full_keys_wanted;      // host only: the launch will have full-ordering scratch (the plan may pick variants that need it)
    uint32_t wait_first;            // launched early (programmatic dependent launch) but must read nothing before the preceding kernel has completed
    // full ordering of the rare rows the stream cannot decide: scratch slots claimed by the row's own CTA
    unsigned long long* full_keys;  // [full_nslots][4][full_vpad] 32-bit words (keys in/out, column indices in/out), or NULL = no such stage
    float* full_vals;               // [full_nslots][full_vpad]
    uint32_t* full_slots;           // [full_nslots] 0 = free, 1 = taken; all zero between launches
    uint32_t full_vpad, full_nslots;
    uint32_t full_slot_rounds;      // polls (about 4 us each) a CTA spends looking for a free slot before it gives the row up
    uint32_t* device_errors;        // bit 0: a bulk copy did not complete within the wait limit; bit 1: no full-sort slot came free
    float* penalized_out;           // optional [batch][hist_stride]: post-mask, post-penalty, pre-temperature value at each history position
#ifdef LLMC_DEV
    unsigned long long* phase_ns;   // development builds only: optional [CTAs][8] phase timestamps, or NULL
#endif
};

struct DeviceInfo {
    uint32_t sm_count;
    size_t max_dyn_smem;  // opt-in dynamic shared memory per CTA
};

struct LaunchPlan {
    uint32_t split, shard_cols, kcap, ccap, limit, hash_slots, bitmap_words, groups, lane_top_words,
        cand_off, scratch_off, tables_off, vlist_cap, stage_u;  // stage_u: 16-byte vectors per consumer thread and ring stage (3 or 4)
    size_t smem;
    bool bits;  // mask or penalty tables needed
    bool sample_threshold;
    int mode;   // kernel variant: 0 rows of either kind, 1 window-mode rows only, 2 exact-selection rows only,
                // 3 exact-selection rows whose threshold is sampled from the first stage (rank cuts above 64)
};

// Raises the dynamic shared-memory limit of every kernel; once per device.
cudaError_t configure_kernels(size_t max_dyn_smem);
// the four translation units of the streaming kernel's variants (stream_variants_*.cu)
cudaError_t configure_stream_f32(int max_dyn_smem);
cudaError_t configure_stream_f32_tables(int max_dyn_smem);
cudaError_t configure_stream_bf16(int max_dyn_smem);
cudaError_t configure_stream_bf16_tables(int max_dyn_smem);
cudaError_t launch_stream_f32(const KParams& P, const LaunchPlan& plan, cudaStream_t stream, bool overlap);
cudaError_t launch_stream_f32_tables(const KParams& P, const LaunchPlan& plan, cudaStream_t stream, bool overlap);
cudaError_t launch_stream_bf16(const KParams& P, const LaunchPlan& plan, cudaStream_t stream, bool overlap);
cudaError_t launch_stream_bf16_tables(const KParams& P, const LaunchPlan& plan, cudaStream_t stream, bool overlap);

// Chooses candidate capacity, CTAs per row and shared-memory layout. Returns 0, or -1
// when the layout does not fit in shared memory.
int plan_launch(const DeviceInfo& dev, const KParams& base, bool top_k_known, uint32_t top_k_hint, uint32_t max_top_k,
                uint32_t max_history, uint32_t requested_split, uint32_t max_lists, LaunchPlan* plan);

// `overlap`: launch with programmatic stream serialization, so the grid may begin reading its inputs
// while the previous kernel of the stream (if it is this kernel too) is still finishing.
cudaError_t launch_stream_select(const KParams& P, const LaunchPlan& plan, cudaStream_t stream, bool overlap = false);
// Copies the plan's geometry (split, capacities, shared-memory offsets) into the parameter block.
void apply_plan(const LaunchPlan& plan, KParams* P);
#ifdef LLMC_DEV
void dev_override(int key, int value);  // development builds only: 0 = ring stage size (3 / 4 / 0 auto)
#endif
cudaError_t launch_merge_draw(const KParams& P, const LaunchPlan& plan, cudaStream_t stream);
cudaError_t launch_advance_rows(uint32_t batch, const uint32_t* tokens, const uint32_t* row_flags, uint32_t* history,
                                uint32_t history_stride, uint32_t window, uint32_t* history_len, uint32_t* history_pos,
                                uint64_t* draw_index, uint8_t* finished, uint32_t eos_id, cudaStream_t stream);
cudaError_t launch_pack_allowed(const uint8_t* allowed_dev, uint32_t n, uint32_t* bits, cudaStream_t stream);

}  // namespace llmc
