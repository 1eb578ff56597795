// C-ABI entry points (include/llm_infer_attn.h): argument validation, planning
// and kernel launches. Nothing here allocates, frees or synchronises.
#include <cmath>
#include <cstdlib>
#include <cstring>

#include "attn_internal.cuh"

namespace b200 {

thread_local int g_last_cuda_error = 0;
std::atomic<uint64_t> g_launch_count{0};

namespace {
constexpr int kMaxDevices = 64;
struct DevCache {
    std::atomic<int> ready{0};
    DeviceInfo info{};
};
DevCache g_dev[kMaxDevices];
}  // namespace

int current_device_info(DeviceInfo* out) {
    int dev = 0;
    B200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return ATTN_ERR_DEVICE;
    DevCache& c = g_dev[dev];
    if (c.ready.load(std::memory_order_acquire) != 2) {
        DeviceInfo info{};
        info.device = dev;
        B200_CUDA_TRY(cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, dev));
        B200_CUDA_TRY(cudaDeviceGetAttribute(&info.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
        B200_CUDA_TRY(cudaDeviceGetAttribute(&info.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        int expected = 0;
        if (c.ready.compare_exchange_strong(expected, 1, std::memory_order_acq_rel)) {
            c.info = info;
            c.ready.store(2, std::memory_order_release);
        } else {
            // another thread is filling the slot, or already has: the values are identical
            *out = info;
            return ATTN_OK;
        }
    }
    *out = c.info;
    return ATTN_OK;
}

namespace {

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

bool valid_dtype(int32_t d) { return d == ATTN_DTYPE_F32 || d == ATTN_DTYPE_F16 || d == ATTN_DTYPE_BF16; }
bool valid_out_dtype(int32_t d) { return valid_dtype(d) || d == ATTN_DTYPE_SPLIT16; }

// Rows each CTA should own at least before another CTA is brought in: below
// this the per-CTA fixed cost (Q load, partial write, merge work) outweighs the
// extra memory parallelism. (One sequence of 4096 rows: 19.5 us with 64, 17.3 us with 32, 17.4 us with 16.)
constexpr uint32_t kMinRowsPerCta = 32;

// Largest number of partials per segment for which attn_decode runs as one launch whose last-arriving CTAs merge
// (the form the engine's kernel symbol always uses). 0 = never: at every shape measured the two-launch chain, whose
// merge pass is already resident when the split pass ends, was faster (17.4 against 28.8 us for one sequence of 4096 rows).
constexpr uint32_t kFusedMaxParts = 0;

#ifdef ATTN_TRACE
unsigned long long* g_trace_split = nullptr;
unsigned long long* g_trace_merge = nullptr;
#endif

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

size_t attn_decode_workspace_bytes(uint32_t batch, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim) {
    DeviceInfo dev{};
    if (current_device_info(&dev) != ATTN_OK) return 0;
    DecodePlan plan{};
    if (make_decode_plan(batch, n_heads, n_kv_heads, head_dim, dev, &plan) != ATTN_OK) return 0;
    return plan.workspace_bytes;
}

}  // extern "C"

namespace {
struct Exchange {
    const AttnDecodeShardedArgs* s;
};

int decode_impl(const AttnDecodeArgs* a, void* stream_v, const Exchange* xchg) {
    if (!a || !a->o || !a->q || !a->k || !a->v) return ATTN_ERR_INVALID_ARG;
    if (!valid_out_dtype(a->o_dtype) || !valid_dtype(a->q_dtype)) return ATTN_ERR_INVALID_ARG;
    if (a->o_dtype == ATTN_DTYPE_SPLIT16 && (a->n_heads * a->head_dim) % 4 != 0) return ATTN_ERR_UNSUPPORTED;
    if (a->kv_dtype != ATTN_DTYPE_F16 && a->kv_dtype != ATTN_DTYPE_BF16) return ATTN_ERR_UNSUPPORTED;
    if (a->batch == 0 || a->n_heads == 0 || a->n_kv_heads == 0 || a->head_dim == 0) return ATTN_ERR_INVALID_ARG;
    if (a->n_heads % a->n_kv_heads != 0) return ATTN_ERR_INVALID_ARG;
    if (a->batch > 1 && a->kv_batch_stride == 0) return ATTN_ERR_INVALID_ARG;

    DeviceInfo dev{};
    int rc = current_device_info(&dev);
    if (rc != ATTN_OK) return rc;
    if (dev.cc_major != 10) return ATTN_ERR_DEVICE;
    DecodePlan plan{};
    rc = make_decode_plan(a->batch, a->n_heads, a->n_kv_heads, a->head_dim, dev, &plan);
    if (rc != ATTN_OK) return rc;

    const uint64_t row_stride = a->kv_row_stride ? a->kv_row_stride : static_cast<uint64_t>(a->n_kv_heads) * a->head_dim;
    if (row_stride < static_cast<uint64_t>(a->n_kv_heads) * a->head_dim) return ATTN_ERR_INVALID_ARG;
    // bulk copies need 16-byte aligned sources: 8 elements of 16 bits
    if (!aligned16(a->k) || !aligned16(a->v) || !aligned16(a->q) || row_stride % 8 != 0 || a->kv_batch_stride % 8 != 0)
        return ATTN_ERR_ALIGNMENT;
    if (!a->workspace || a->workspace_bytes < plan.workspace_bytes) return ATTN_ERR_WORKSPACE;
    if (!aligned16(a->workspace)) return ATTN_ERR_ALIGNMENT;

    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    float* ws = static_cast<float*>(a->workspace);

    DecodeParams p{};
    p.q = a->q;
    p.k = static_cast<const uint16_t*>(a->k);
    p.v = static_cast<const uint16_t*>(a->v);
    p.part_o = ws;
    p.part_lse = ws + plan.part_o_floats;
    p.seg_prefix = reinterpret_cast<uint32_t*>(ws + plan.part_o_floats + plan.part_lse_floats);
    p.kv_len = a->kv_len;
    p.kv_len_uniform = a->kv_len_uniform;
    p.batch = a->batch;
    p.n_heads = a->n_heads;
    p.n_kv_heads = a->n_kv_heads;
    p.group = plan.group;
    p.head_groups = plan.head_groups;
    p.kv_row_stride = row_stride;
    p.kv_batch_stride = a->kv_batch_stride;
    const float scale = a->scale != 0.f ? a->scale : 1.0f / sqrtf(static_cast<float>(a->head_dim));
    p.scale_log2 = scale * 1.4426950408889634f;
    p.q_dtype = a->q_dtype;
    p.max_ctas = a->max_ctas;
    uint32_t min_rows = kMinRowsPerCta;
#ifdef ATTN_TRACE
    if (const char* e = getenv("ATTN_TRACE_MIN_ROWS")) min_rows = static_cast<uint32_t>(atoi(e));  // profiling knob
#endif
    p.min_tiles_per_cta = (min_rows + plan.tile_rows - 1) / plan.tile_rows;
    p.nstages = plan.nstages;
    p.kv_early = a->kv_early ? 1u : 0u;
    p.kv_capacity = a->kv_capacity;
#ifdef ATTN_BOUNDS_CHECK
    p.part_rows = plan.part_o_floats / a->head_dim;
#endif
    p.status = a->status;
#ifdef ATTN_TRACE
    p.trace = g_trace_split;
#endif

    const bool kv_bf16 = a->kv_dtype == ATTN_DTYPE_BF16;
    const bool qsplit = a->q_dtype != ATTN_DTYPE_F16;
    // Single-launch mode: when every segment is shared by only a few CTAs (batched decode), the CTA that delivers a
    // segment's last partial merges it and there is no merge pass. With many partials per segment (one long
    // sequence) that one CTA would be slow, and the parallel merge pass is used instead.
    const uint32_t parts_per_segment = (plan.grid + plan.nseg - 1) / plan.nseg + 1;
    const bool fused = !xchg && !kv_bf16 && a->kv_len == nullptr && parts_per_segment <= kFusedMaxParts;
    if (fused) {
        p.o = a->o;
        p.lse = a->lse;
        p.o_dtype = a->o_dtype;
        p.counters = p.seg_prefix + plan.prefix_words;
        B200_CUDA_TRY(cudaMemsetAsync(p.counters, 0, static_cast<size_t>(plan.nseg) * 4, stream));
    }
    rc = launch_decode_split(p, a->head_dim, plan.hpc, qsplit, kv_bf16, fused, plan.grid, plan.smem_bytes, stream);
    if (rc != ATTN_OK || fused) return rc;

    MergeParams m{};
    m.o = a->o;
    m.lse = a->lse;
    m.part_o = p.part_o;
    m.part_lse = p.part_lse;
    m.rows = a->batch * a->n_heads;
    m.head_dim = a->head_dim;
    m.o_dtype = a->o_dtype;
    m.split_grid = plan.grid;
    m.hpc = plan.hpc;
    m.ts = plan.ts;
    m.tile_rows = plan.tile_rows;
    m.n_heads = a->n_heads;
    m.group = plan.group;
    m.head_groups = plan.head_groups;
    m.batch = a->batch;
    m.kv_len = a->kv_len;
    m.kv_len_uniform = a->kv_len_uniform;
    m.kv_capacity = a->kv_capacity;
#ifdef ATTN_BOUNDS_CHECK
    m.part_rows = plan.part_o_floats / a->head_dim;
#endif
    m.max_ctas = p.max_ctas;
    m.min_tiles_per_cta = p.min_tiles_per_cta;
    m.seg_prefix = p.seg_prefix;
    m.status = a->status;
#ifdef ATTN_TRACE
    m.trace = g_trace_merge;
#endif
    if (xchg) {
        const AttnDecodeShardedArgs* s = xchg->s;
        m.xchg_world = s->world_size;
        m.xchg_rank = s->rank;
        m.xchg_step = s->step;
        m.xchg_poll_limit = s->poll_limit ? s->poll_limit : (1u << 21);
        for (uint32_t r = 0; r < s->world_size; ++r)
            m.xchg_peers[r] = static_cast<unsigned long long*>(s->peer_buffers[r]);
    }
    return launch_merge(m, stream, /*dependent_launch=*/true);
}
}  // namespace

extern "C" {

int attn_decode(const AttnDecodeArgs* a, void* stream_v) { return decode_impl(a, stream_v, nullptr); }

size_t attn_decode_sharded_exchange_bytes(uint32_t batch, uint32_t n_heads, uint32_t head_dim, uint32_t world_size) {
    if (world_size == 0 || world_size > ATTN_MAX_PEERS) return 0;
    if (batch == 0 || n_heads == 0 || head_dim == 0 || head_dim % 32 != 0) return 0;
    return exchange_words(static_cast<uint64_t>(batch) * n_heads, head_dim, world_size) * 8;  // records + 2 control words
}

uint32_t attn_decode_sharded_cell_floats(uint32_t batch, uint32_t n_heads, uint32_t head_dim) {
    if (batch == 0 || n_heads == 0 || head_dim == 0 || head_dim % 32 != 0) return 0;
    return merge_slice_floats(static_cast<uint64_t>(batch) * n_heads, head_dim);
}

int attn_decode_sharded(const AttnDecodeShardedArgs* s, void* stream_v) {
    if (!s) return ATTN_ERR_INVALID_ARG;
    if (s->world_size == 0 || s->world_size > ATTN_MAX_PEERS || s->rank >= s->world_size) return ATTN_ERR_INVALID_ARG;
    for (uint32_t r = 0; r < s->world_size; ++r) {
        if (!s->peer_buffers[r]) return ATTN_ERR_INVALID_ARG;
        if (reinterpret_cast<uintptr_t>(s->peer_buffers[r]) & 15u) return ATTN_ERR_ALIGNMENT;
    }
    Exchange x{s};
    return decode_impl(&s->decode, stream_v, &x);
}

int attn_merge(const AttnMergeArgs* a, void* stream_v) {
    if (!a || !a->o || !a->part_o || !a->part_lse) return ATTN_ERR_INVALID_ARG;
    if (!valid_out_dtype(a->o_dtype)) return ATTN_ERR_INVALID_ARG;
    if (a->n_parts == 0 || a->rows == 0) return ATTN_ERR_INVALID_ARG;
    if (a->head_dim != 32 && a->head_dim != 64 && a->head_dim != 128 && a->head_dim != 256) return ATTN_ERR_UNSUPPORTED;
    if (!aligned16(a->part_o) || a->o_part_stride % 4 != 0) return ATTN_ERR_ALIGNMENT;
    MergeParams m{};
    m.o = a->o;
    m.lse = a->lse;
    m.part_o = a->part_o;
    m.part_lse = a->part_lse;
    m.o_part_stride = a->o_part_stride;
    m.lse_part_stride = a->lse_part_stride;
    m.n_parts = a->n_parts;
    m.rows = a->rows;
    m.head_dim = a->head_dim;
    m.o_dtype = a->o_dtype;
    m.split_grid = 0;
    return launch_merge(m, static_cast<cudaStream_t>(stream_v), /*dependent_launch=*/false);
}

const char* attn_status_string(int code) {
    switch (code) {
        case ATTN_OK: return "ok";
        case ATTN_ERR_INVALID_ARG: return "invalid argument";
        case ATTN_ERR_UNSUPPORTED: return "unsupported shape or dtype";
        case ATTN_ERR_ALIGNMENT: return "pointer or stride not 16-byte aligned";
        case ATTN_ERR_WORKSPACE: return "workspace missing or too small";
        case ATTN_ERR_CUDA: return "CUDA runtime call failed";
        case ATTN_ERR_DEVICE: return "device is not sm_100";
        default: return "unknown status";
    }
}

int attn_last_cuda_error(void) { return g_last_cuda_error; }

#ifdef ATTN_TRACE
// Profiling build only: device buffers that receive eight time stamps per CTA of the split pass and of the merge
// pass of every following attn_decode / attn_decode_sharded call (null = off).
void attn_trace_set_buffers(unsigned long long* split_pass, unsigned long long* merge_pass) {
    g_trace_split = split_pass;
    g_trace_merge = merge_pass;
}
#endif

uint64_t attn_kernel_launch_count(void) { return g_launch_count.load(std::memory_order_relaxed); }

size_t attn_abi_struct_size(int which) {
    switch (which) {
        case 0: return sizeof(AttnDecodeArgs);
        case 1: return sizeof(AttnDecodeShardedArgs);
        case 2: return sizeof(AttnPrefillArgs);
        case 3: return sizeof(AttnRopeInsertArgs);
        case 4: return sizeof(AttnGemvArgs);
        case 5: return sizeof(AttnMergeArgs);
        case 6: return sizeof(AttnGemmArgs);
        case 7: return sizeof(AttnRopePromptArgs);
        default: return 0;
    }
}

}  // extern "C"
