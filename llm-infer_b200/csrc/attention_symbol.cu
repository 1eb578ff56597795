// The engine's own kernel symbol, include/kernels.cuh:26, defined for sm_100a:
// fp32 q/o, fp16 K/V, one sequence, all model dimensions taken from device
// constant memory (set by attention_configure). One launch = split-KV pass +
// merge by the last-arriving CTAs (in two levels), so it fits a single CUDA-graph kernel node
// whose grid is frozen (include/model/device.hpp:219-237): the grid is always
// one CTA per SM and CTAs without rows exit at once.
#include "../../include/kernels_b200.cuh"
#include "decode_body.cuh"

namespace b200 {
namespace {

struct AttentionSymbolConfig {
    uint32_t configured;
    uint32_t n_heads;
    uint32_t n_kv_heads;
    uint32_t head_dim;
    uint32_t hpc;
    uint32_t group;
    uint32_t head_groups;
    uint32_t nstages;
    uint32_t min_tiles_per_cta;
    float scale_log2;
    float* part_o;
    float* part_lse;
    uint32_t* counters;
    uint32_t* group_counters;
    float* group_o;
    float* group_lse;
    uint32_t* status;     // one word of the workspace: ATTN_STATUS_* bits
    uint32_t smem_bytes;  // dynamic shared memory the node must be launched with
#ifdef ATTN_BOUNDS_CHECK
    uint64_t part_rows;    // what the checking build compares its workspace indices with
    uint64_t group_slots;
#endif
};

__constant__ AttentionSymbolConfig g_cfg;

// host mirror of what was last configured on each device
struct HostCfg {
    bool ok = false;
    uint32_t grid = 0, smem = 0;
    uint32_t* status = nullptr;
};
HostCfg g_host_cfg[64];

// Two forms per shape: up to eight query heads per kv head (rows 8-15 of the MMAs dropped: no spills in the
// 168 registers of this nine-warp CTA), and the general one.
template <int D, int HPC>
__device__ __forceinline__ void run(const DecodeParams& p, unsigned char* smem) {
    if (p.group <= 8) {
        decode_detail::decode_split_body<D, HPC, /*QSPLIT=*/true, /*BF16=*/false, /*FUSED=*/true, /*LOW8=*/true>(p, smem);
    } else {
        decode_detail::decode_split_body<D, HPC, /*QSPLIT=*/true, /*BF16=*/false, /*FUSED=*/true, /*LOW8=*/false>(p, smem);
    }
}

}  // namespace
}  // namespace b200

__global__ void __launch_bounds__(b200::decode_detail::kThreads, 1)
attention(float* o, const float* q, const half* k, const half* v, uint32_t kv_tokens) {
    using namespace b200;
    extern __shared__ __align__(128) unsigned char smem[];
    const AttentionSymbolConfig& c = g_cfg;
    // The body needs exactly this block size (8 consumer warps + the producer warp, named barriers over 256 threads)
    // and the configured amount of dynamic shared memory (barriers and the K/V ring). A node added with the engine's
    // old geometry (128 threads, no shared memory, src/model/block.cu:214-224) is refused here instead of touching
    // shared memory it does not own: nothing is written except the status bit.
    if (c.configured && (blockDim.x != static_cast<unsigned>(decode_detail::kThreads) || blockDim.y != 1 ||
                         blockDim.z != 1 || gridDim.y != 1 || gridDim.z != 1 || dynamic_smem_bytes() < c.smem_bytes)) {
        if (threadIdx.x == 0 && blockIdx.x == 0 && c.status) atomicOr(c.status, ATTN_STATUS_BAD_SHAPE);
        return;
    }
    if (!c.configured || kv_tokens == 0) {
        // kv_tokens == 0 cannot happen in the engine (kv_len >= 1); an unconfigured device is a host bug.
        if (kv_tokens == 0 && c.configured) {
            for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < c.n_heads * c.head_dim;
                 i += gridDim.x * blockDim.x)
                o[i] = 0.f;
        }
        return;
    }
    DecodeParams p{};
    p.q = q;
    p.k = reinterpret_cast<const uint16_t*>(k);
    p.v = reinterpret_cast<const uint16_t*>(v);
    p.part_o = c.part_o;
    p.part_lse = c.part_lse;
    p.seg_prefix = nullptr;
    p.kv_len = nullptr;
    p.kv_len_uniform = kv_tokens;
    p.batch = 1;
    p.n_heads = c.n_heads;
    p.n_kv_heads = c.n_kv_heads;
    p.group = c.group;
    p.head_groups = c.head_groups;
    p.kv_row_stride = static_cast<uint64_t>(c.n_kv_heads) * c.head_dim;
    p.kv_batch_stride = 0;
    p.scale_log2 = c.scale_log2;
    p.q_dtype = ATTN_DTYPE_F32;
    p.max_ctas = 0;
    p.min_tiles_per_cta = c.min_tiles_per_cta;
    p.nstages = c.nstages;
    p.status = c.status;
    p.o = o;
    p.lse = nullptr;
    p.o_dtype = ATTN_DTYPE_F32;
    p.counters = c.counters;
    p.group_counters = c.group_counters;
    p.group_o = c.group_o;
    p.group_lse = c.group_lse;
#ifdef ATTN_BOUNDS_CHECK
    p.part_rows = c.part_rows;
    p.group_slots = c.group_slots;
#endif
    if (c.head_dim == 128) {
        switch (c.hpc) {
            case 8: run<128, 8>(p, smem); break;
            case 4: run<128, 4>(p, smem); break;
            case 2: run<128, 2>(p, smem); break;
            default: run<128, 1>(p, smem); break;
        }
    } else {
        switch (c.hpc) {
            case 8: run<64, 8>(p, smem); break;
            case 4: run<64, 4>(p, smem); break;
            case 2: run<64, 2>(p, smem); break;
            default: run<64, 1>(p, smem); break;
        }
    }
}

using namespace b200;

namespace {
// Rows per CTA below which a further CTA is not worth its share of the merge in the single-launch kernel.
constexpr uint32_t kSymbolMinRowsPerCta = 64;

int plan_for(uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, DecodePlan* plan) {
    DeviceInfo dev{};
    int rc = current_device_info(&dev);
    if (rc != ATTN_OK) return rc;
    return make_decode_plan(1, n_heads, n_kv_heads, head_dim, dev, plan);
}
}  // namespace

extern "C" {

size_t attention_workspace_bytes(uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim) {
    DecodePlan plan{};
    if (plan_for(n_heads, n_kv_heads, head_dim, &plan) != ATTN_OK) return 0;
    return plan.symbol_workspace_bytes;
}

int attention_configure(uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, float scale, void* workspace,
                        size_t workspace_bytes, void* stream_v) {
    DecodePlan plan{};
    int rc = plan_for(n_heads, n_kv_heads, head_dim, &plan);
    if (rc != ATTN_OK) return rc;
    if (!workspace || workspace_bytes < attention_workspace_bytes(n_heads, n_kv_heads, head_dim))
        return ATTN_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(workspace) & 15u) return ATTN_ERR_ALIGNMENT;
    int dev = 0;
    B200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return ATTN_ERR_DEVICE;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

    AttentionSymbolConfig c{};
    c.configured = 1;
    c.n_heads = n_heads;
    c.n_kv_heads = n_kv_heads;
    c.head_dim = head_dim;
    c.hpc = plan.hpc;
    c.group = plan.group;
    c.head_groups = plan.head_groups;
    c.nstages = plan.nstages;
    c.min_tiles_per_cta = (kSymbolMinRowsPerCta + plan.tile_rows - 1) / plan.tile_rows;
    const float s = scale != 0.f ? scale : 1.0f / sqrtf(static_cast<float>(head_dim));
    c.scale_log2 = s * 1.4426950408889634f;
    float* ws = static_cast<float*>(workspace);
    c.part_o = ws;
    c.part_lse = ws + plan.part_o_floats;
    c.counters = reinterpret_cast<uint32_t*>(ws + plan.part_o_floats + plan.part_lse_floats) + plan.prefix_words;
    c.status = c.counters + ((static_cast<size_t>(plan.nseg) + 3) & ~3ull);
    c.group_o = ws + plan.group_base_words;
    c.group_lse = c.group_o + plan.group_o_floats;
    c.group_counters = reinterpret_cast<uint32_t*>(c.group_lse + plan.group_lse_floats);
    c.smem_bytes = static_cast<uint32_t>(plan.smem_bytes);
#ifdef ATTN_BOUNDS_CHECK
    c.part_rows = plan.part_o_floats / head_dim;
    c.group_slots = static_cast<uint64_t>(plan.grid) + plan.nseg;
#endif
    // counters (rounded up to four words), the status word behind them and the group counters start at zero
    B200_CUDA_TRY(cudaMemsetAsync(c.counters, 0, (((static_cast<size_t>(plan.nseg) + 3) & ~3ull) + 4) * 4, stream));
    B200_CUDA_TRY(cudaMemsetAsync(c.group_counters, 0, plan.group_counter_words * 4, stream));
    B200_CUDA_TRY(cudaMemcpyToSymbolAsync(g_cfg, &c, sizeof(c), 0, cudaMemcpyHostToDevice, stream));
    B200_CUDA_TRY(cudaStreamSynchronize(stream));  // c lives on this stack frame
    B200_CUDA_TRY(cudaFuncSetAttribute(attention, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(plan.smem_bytes)));
    g_host_cfg[dev].ok = true;
    g_host_cfg[dev].grid = plan.grid;
    g_host_cfg[dev].smem = static_cast<uint32_t>(plan.smem_bytes);
    g_host_cfg[dev].status = c.status;
    return ATTN_OK;
}

int attention_status(uint32_t* bits, int clear, void* stream_v) {
    int dev = 0;
    B200_CUDA_TRY(cudaGetDevice(&dev));
    if (!bits || dev < 0 || dev >= 64 || !g_host_cfg[dev].ok) return ATTN_ERR_INVALID_ARG;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    B200_CUDA_TRY(cudaMemcpyAsync(bits, g_host_cfg[dev].status, 4, cudaMemcpyDeviceToHost, stream));
    if (clear) B200_CUDA_TRY(cudaMemsetAsync(g_host_cfg[dev].status, 0, 4, stream));
    B200_CUDA_TRY(cudaStreamSynchronize(stream));
    return ATTN_OK;
}

int attention_launch_dims(uint32_t* grid, uint32_t* block, uint32_t* shared_mem_bytes) {
    int dev = 0;
    B200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !g_host_cfg[dev].ok) return ATTN_ERR_INVALID_ARG;
    if (grid) *grid = g_host_cfg[dev].grid;
    if (block) *block = decode_detail::kThreads;
    if (shared_mem_bytes) *shared_mem_bytes = g_host_cfg[dev].smem;
    return ATTN_OK;
}

const void* attention_kernel_function(void) { return reinterpret_cast<const void*>(attention); }

static int fill_node_params(cudaKernelNodeParams* np, void** argv) {
    uint32_t grid = 0, block = 0, smem = 0;
    int rc = attention_launch_dims(&grid, &block, &smem);
    if (rc != ATTN_OK) return rc;
    memset(np, 0, sizeof(*np));
    np->func = reinterpret_cast<void*>(attention);
    np->gridDim = dim3(grid);
    np->blockDim = dim3(block);
    np->sharedMemBytes = smem;
    np->kernelParams = argv;
    np->extra = nullptr;
    return ATTN_OK;
}

int attention_graph_add_node(void* graph, void* node_out, const void* deps, size_t n_deps, float* o, const float* q,
                             const void* k, const void* v, uint32_t kv_tokens) {
    if (!graph || !node_out) return ATTN_ERR_INVALID_ARG;
    void* argv[5] = {&o, &q, &k, &v, &kv_tokens};
    cudaKernelNodeParams np;
    int rc = fill_node_params(&np, argv);
    if (rc != ATTN_OK) return rc;
    B200_CUDA_TRY(cudaGraphAddKernelNode(static_cast<cudaGraphNode_t*>(node_out), static_cast<cudaGraph_t>(graph),
                                         static_cast<const cudaGraphNode_t*>(deps), n_deps, &np));
    return ATTN_OK;
}

int attention_graph_exec_update(void* graph_exec, void* node, float* o, const float* q, const void* k, const void* v,
                                uint32_t kv_tokens) {
    if (!graph_exec || !node) return ATTN_ERR_INVALID_ARG;
    void* argv[5] = {&o, &q, &k, &v, &kv_tokens};
    cudaKernelNodeParams np;
    int rc = fill_node_params(&np, argv);
    if (rc != ATTN_OK) return rc;
    B200_CUDA_TRY(cudaGraphExecKernelNodeSetParams(static_cast<cudaGraphExec_t>(graph_exec),
                                                   static_cast<cudaGraphNode_t>(node), &np));
    return ATTN_OK;
}

int attention_launch(float* o, const float* q, const void* k, const void* v, uint32_t kv_tokens, void* stream_v) {
    uint32_t grid = 0, block = 0, smem = 0;
    int rc = attention_launch_dims(&grid, &block, &smem);
    if (rc != ATTN_OK) return rc;
    attention<<<grid, block, smem, static_cast<cudaStream_t>(stream_v)>>>(
        o, q, static_cast<const half*>(k), static_cast<const half*>(v), kv_tokens);
    B200_CUDA_TRY(cudaGetLastError());
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return ATTN_OK;
}

}  // extern "C"
