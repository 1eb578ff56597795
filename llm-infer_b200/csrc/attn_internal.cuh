// Declarations shared by the translation units of libllm_infer_attn.so.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <utility>
#include <cstdint>

#include "../../include/llm_infer_attn.h"

namespace b200 {

// ----------------------------------------------------------------------------
// Split-KV decode: how the KV rows are divided.
//
// A "segment" is one (sequence, kv-head group) pair; a head group is HPC
// consecutive kv heads that one CTA streams together (their slices of a cache
// row are contiguous, so one bulk copy fetches them all). A segment is cut
// into tiles of TT = 16 * (8 / HPC) rows. All tiles of all segments form one
// flat list of NT tiles; CTA c of A active CTAs owns tiles
// [c*NT/A, (c+1)*NT/A). For every segment it touches, each of its 8 warps
// writes one partial (normalised O, LSE) into slot (c + s) * TS + ts, where s
// is the segment index and ts the warp's row sub-tile. Because both c and s
// only grow along the flat list, c + s is unique per (CTA, segment) pair and
// the slots of one segment are consecutive, which is what the merge pass reads.
// ----------------------------------------------------------------------------
struct DecodeParams {
    const void* q;
    const uint16_t* k;
    const uint16_t* v;
    float* part_o;         // [slots*TS][HPC][G][D]
    float* part_lse;       // [slots*TS][HPC][G]
    uint32_t* seg_prefix;  // [nseg+1] tile prefix written by CTA 0 when lengths are ragged
    const uint32_t* kv_len;
    uint32_t kv_len_uniform;
    uint32_t batch;
    uint32_t n_heads;
    uint32_t n_kv_heads;
    uint32_t group;        // G = n_heads / n_kv_heads
    uint32_t head_groups;  // n_kv_heads / HPC
    uint64_t kv_row_stride;
    uint64_t kv_batch_stride;
    float scale_log2;  // softmax scale * log2(e)
    int32_t q_dtype;
    uint32_t max_ctas;
    uint32_t min_tiles_per_cta;
    uint32_t nstages;
    uint32_t kv_early;     // AttnDecodeArgs.kv_early
    uint32_t kv_capacity;  // rows a sequence's caches hold, 0 = not stated (lengths beyond it are clamped and reported)
#ifdef ATTN_BOUNDS_CHECK
    uint64_t part_rows;    // rows of part_o / entries of part_lse that exist
    uint64_t group_slots;  // group records / group counters that exist (single-launch mode)
#endif
    uint32_t* status;
    // single-launch (fused merge) mode only: final output and per-segment arrival counters
    void* o;
    float* lse;
    int32_t o_dtype;
    uint32_t* counters;  // [nseg], zero before the first launch; the kernel leaves them zero
    // two-level merge of the single-launch mode (segments shared by many CTAs): first-level groups of CTAs merge
    // their partials into group records, the last group to finish merges the records. nullptr = one level only.
    uint32_t* group_counters;  // [grid + nseg], zero before the first launch; the kernel leaves them zero
    float* group_o;            // [(grid + nseg) * hpc * group][head_dim]
    float* group_lse;          // [(grid + nseg) * hpc * group]
#ifdef ATTN_TRACE
    unsigned long long* trace;  // [grid][8] time stamps, or null
#endif
};

struct MergeParams {
    void* o;
    float* lse;
    const float* part_o;
    const float* part_lse;
    uint64_t o_part_stride;
    uint64_t lse_part_stride;
    uint32_t n_parts;
    uint32_t rows;
    uint32_t head_dim;
    int32_t o_dtype;
    // decode-internal mode (split_grid != 0): partial ranges are derived per row
    uint32_t split_grid;
    uint32_t hpc;
    uint32_t ts;
    uint32_t tile_rows;
    uint32_t n_heads;
    uint32_t group;
    uint32_t head_groups;
    uint32_t batch;
    const uint32_t* kv_len;
    uint32_t kv_len_uniform;
    uint32_t kv_capacity;
    uint32_t max_ctas;
    uint32_t min_tiles_per_cta;
    const uint32_t* seg_prefix;
#ifdef ATTN_BOUNDS_CHECK
    uint64_t part_rows;
#endif
    // cross-GPU exchange (xchg_world > 0): every CTA stores its locally merged slice of a row (and the row's LSE) into
    // every rank's exchange buffer over NVLink as 64-bit words {value, step}, then collects the xchg_world records of
    // its own slice from this GPU's buffer, waiting (bounded) until each word carries the current step, and merges
    // them. Buffer layout: see exchange_words().
    unsigned long long* xchg_peers[ATTN_MAX_PEERS];
    uint32_t xchg_world;
    uint32_t xchg_rank;
    uint32_t xchg_step;
    uint32_t xchg_poll_limit;
    uint32_t* status;
#ifdef ATTN_TRACE
    unsigned long long* trace;  // [grid][8] time stamps, or null
#endif
};

// Floats of head_dim that one CTA of the merge pass owns. Few output rows (one long sequence: 32 rows, each with a
// partial per split-pass CTA) are cut into 32- or 64-float slices so that the pass fills the GPU and every thread
// has all of its loads in flight at once; many rows (batched decode) keep whole rows per CTA. A function of the
// shape only, so that all ranks of a sharded decode lay out their exchange buffers identically.
__host__ __device__ inline uint32_t merge_slice_floats(uint64_t rows, uint32_t head_dim) {
    constexpr uint64_t kMaxCtas = 592;  // four CTAs per SM of a 148-SM part
    if (head_dim % 32 == 0 && rows * (head_dim / 32) <= kMaxCtas) return 32;
    if (head_dim % 64 == 0 && rows * (head_dim / 64) <= kMaxCtas) return 64;
    if (head_dim % 128 == 0) return 128;
    return head_dim % 64 == 0 ? 64 : 32;
}

// Exchange buffer of the sharded decode, in 64-bit words: rec[2 (step parity)][world (source rank)][rows * nslices]
// cells of (slice + 1) words each (the slice's values, then the row's LSE), each word = value bits | step << 32;
// then two control words (steps completed, CTAs finished in the current step).
__host__ __device__ inline uint64_t exchange_cell_words(uint32_t slice) { return static_cast<uint64_t>(slice) + 1; }
__host__ __device__ inline uint64_t exchange_rank_words(uint64_t rows, uint32_t head_dim, uint32_t slice) {
    return rows * (head_dim / slice) * exchange_cell_words(slice);
}
__host__ __device__ inline uint64_t exchange_words(uint64_t rows, uint32_t head_dim, uint32_t world) {
    return 2ull * world * exchange_rank_words(rows, head_dim, merge_slice_floats(rows, head_dim)) + 2;
}

// A sequence's length as the kernels use it: clamped to the stated capacity.
__host__ __device__ inline uint32_t clamped_len(uint32_t len, uint32_t capacity) {
    return (capacity && len > capacity) ? capacity : len;
}

// Number of CTAs that actually take tiles, identical in the split and merge passes.
__host__ __device__ inline uint32_t active_ctas(uint32_t grid, uint32_t max_ctas, uint32_t min_tiles, uint64_t nt) {
    uint64_t a = grid;
    if (max_ctas && max_ctas < a) a = max_ctas;
    uint64_t by_work = nt / (min_tiles ? min_tiles : 1);
    if (by_work < 1) by_work = 1;
    if (by_work < a) a = by_work;
    return static_cast<uint32_t>(a);
}

// CTA that owns flat tile t when nt tiles are dealt to a CTAs as [c*nt/a, (c+1)*nt/a).
__host__ __device__ inline uint32_t cta_of_tile(uint64_t t, uint64_t nt, uint64_t a) {
    return static_cast<uint32_t>(((t + 1) * a - 1) / nt);
}

// ----------------------------------------------------------------------------
// host helpers (attn_api.cu)
// ----------------------------------------------------------------------------
extern thread_local int g_last_cuda_error;
extern std::atomic<uint64_t> g_launch_count;

inline int cuda_fail(cudaError_t e) {
    g_last_cuda_error = static_cast<int>(e);
    return ATTN_ERR_CUDA;
}

#define B200_CUDA_TRY(expr)                                  \
    do {                                                     \
        cudaError_t e_ = (expr);                             \
        if (e_ != cudaSuccess) return ::b200::cuda_fail(e_); \
    } while (0)

// Launch with programmatic dependent launch allowed: the grid may be scheduled while the previous grid of the stream
// is still running (its CTAs start as SMs free up), so launch latency, barrier set-up and prefetches of data that no
// kernel writes (weights) overlap the previous kernel's tail. Such a kernel must execute griddepcontrol.wait before
// it reads anything another kernel produces and before it writes global memory.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

struct DeviceInfo {
    int device;
    int sm_count;
    int cc_major;
    int max_smem_optin;
};
// Properties of the current device (cached per device; no allocation).
int current_device_info(DeviceInfo* out);

int launch_decode_split(const DecodeParams& p, uint32_t head_dim, uint32_t hpc, bool qsplit, bool kv_bf16, bool fused,
                        uint32_t grid, size_t smem_bytes, cudaStream_t stream);
int launch_merge(const MergeParams& p, cudaStream_t stream, bool dependent_launch);
// fp16-weight GEMV on the tensor cores (attn_gemv_f16mma.cu): batches and the fused forms of attn_gemv_f16.
int launch_gemv_f16_mma(const AttnGemvArgs* a, cudaStream_t stream);

// Geometry of the decode split for given dimensions.
struct DecodePlan {
    uint32_t hpc;        // kv heads per CTA (8, 4, 2 or 1)
    uint32_t ts;         // row sub-tiles per head = 8 / hpc
    uint32_t tile_rows;  // 16 * ts
    uint32_t group;
    uint32_t head_groups;
    uint32_t nseg;
    uint32_t grid;
    uint32_t nstages;
    size_t smem_bytes;
    size_t part_o_floats;
    size_t part_lse_floats;
    size_t prefix_words;
    // behind the status words: first-level records of the single-launch mode's two-level merge
    size_t group_base_words;     // offset of group_o from the start of the workspace, in 32-bit words
    size_t group_o_floats;
    size_t group_lse_floats;
    size_t group_counter_words;
    size_t workspace_bytes;         // what attn_decode needs
    size_t symbol_workspace_bytes;  // what the kernel symbol needs (workspace_bytes + the group records)
};
int make_decode_plan(uint32_t batch, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, const DeviceInfo& dev,
                     DecodePlan* plan);

}  // namespace b200
