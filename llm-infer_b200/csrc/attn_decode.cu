// Launchers of the split-KV decode pass (kernel body: decode_body.cuh) and the
// planning of its shared memory, grid and workspace.
#include "decode_body.cuh"

namespace b200 {

namespace {

using decode_detail::kConsumerWarps;
using decode_detail::kThreads;

// FUSED = the CTA that delivers a segment's last partial also merges it (single launch, no merge pass).
template <int D, int HPC, bool QSPLIT, bool BF16, bool FUSED>
__global__ void __launch_bounds__(kThreads, 1) decode_split_kernel(const __grid_constant__ DecodeParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    decode_detail::decode_split_body<D, HPC, QSPLIT, BF16, FUSED>(p, smem);
}

template <int D, int HPC, bool QSPLIT, bool BF16, bool FUSED>
int launch_one(const DecodeParams& p, uint32_t grid, size_t smem_bytes, cudaStream_t stream) {
    auto kernel = decode_split_kernel<D, HPC, QSPLIT, BF16, FUSED>;
    B200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem_bytes)));
    // launched as a programmatic dependent: the launch overlaps the previous kernel's tail; the kernel waits for that
    // kernel before it reads anything
    B200_CUDA_TRY(launch_dependent(kernel, dim3(grid), dim3(kThreads), smem_bytes, stream, p));
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return ATTN_OK;
}

template <int D, bool QSPLIT, bool BF16, bool FUSED>
int launch_hpc(const DecodeParams& p, uint32_t hpc, uint32_t grid, size_t smem_bytes, cudaStream_t stream) {
    switch (hpc) {
        case 8: return launch_one<D, 8, QSPLIT, BF16, FUSED>(p, grid, smem_bytes, stream);
        case 4: return launch_one<D, 4, QSPLIT, BF16, FUSED>(p, grid, smem_bytes, stream);
        case 2: return launch_one<D, 2, QSPLIT, BF16, FUSED>(p, grid, smem_bytes, stream);
        case 1: return launch_one<D, 1, QSPLIT, BF16, FUSED>(p, grid, smem_bytes, stream);
        default: return ATTN_ERR_UNSUPPORTED;
    }
}

template <int D>
int launch_d(const DecodeParams& p, uint32_t hpc, bool qsplit, bool kv_bf16, bool fused, uint32_t grid,
             size_t smem_bytes, cudaStream_t stream) {
    if (kv_bf16) {
        // bf16 MMA operands: Q and P always carry a residual term (8-bit significand otherwise); two-pass only
        return launch_hpc<D, true, true, false>(p, hpc, grid, smem_bytes, stream);
    }
    if (fused) {
        return qsplit ? launch_hpc<D, true, false, true>(p, hpc, grid, smem_bytes, stream)
                      : launch_hpc<D, false, false, true>(p, hpc, grid, smem_bytes, stream);
    }
    return qsplit ? launch_hpc<D, true, false, false>(p, hpc, grid, smem_bytes, stream)
                  : launch_hpc<D, false, false, false>(p, hpc, grid, smem_bytes, stream);
}

}  // namespace

int launch_decode_split(const DecodeParams& p, uint32_t head_dim, uint32_t hpc, bool qsplit, bool kv_bf16, bool fused,
                        uint32_t grid, size_t smem_bytes, cudaStream_t stream) {
    switch (head_dim) {
        case 128: return launch_d<128>(p, hpc, qsplit, kv_bf16, fused, grid, smem_bytes, stream);
        case 64: return launch_d<64>(p, hpc, qsplit, kv_bf16, fused, grid, smem_bytes, stream);
        default: return ATTN_ERR_UNSUPPORTED;
    }
}

int make_decode_plan(uint32_t batch, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, const DeviceInfo& dev,
                     DecodePlan* plan) {
    if (batch == 0 || n_heads == 0 || n_kv_heads == 0 || n_heads % n_kv_heads != 0) return ATTN_ERR_INVALID_ARG;
    if (head_dim != 64 && head_dim != 128) return ATTN_ERR_UNSUPPORTED;
    DecodePlan pl{};
    pl.group = n_heads / n_kv_heads;
    if (pl.group > 16) return ATTN_ERR_UNSUPPORTED;
    pl.hpc = (n_kv_heads % 8 == 0) ? 8 : (n_kv_heads % 4 == 0) ? 4 : (n_kv_heads % 2 == 0) ? 2 : 1;
    pl.ts = kConsumerWarps / pl.hpc;
    pl.tile_rows = 16 * pl.ts;
    pl.head_groups = n_kv_heads / pl.hpc;
    uint64_t nseg = static_cast<uint64_t>(batch) * pl.head_groups;
    if (nseg > 32768) return ATTN_ERR_UNSUPPORTED;
    pl.nseg = static_cast<uint32_t>(nseg);
    pl.grid = static_cast<uint32_t>(dev.sm_count);
    const size_t tile_bytes = static_cast<size_t>(pl.tile_rows) * (static_cast<size_t>(pl.hpc) * head_dim * 2 + 16);
    // behind the ring: two more barriers, the query rows of one segment (fp32 at most), the tile prefix, two words
    const size_t fixed = 16 + static_cast<size_t>(pl.hpc) * pl.group * head_dim * 4 + static_cast<size_t>(pl.nseg + 1) * 4 + 128;
    size_t budget = static_cast<size_t>(dev.max_smem_optin);
    if (budget < fixed + 2 * (2 * tile_bytes + 24)) return ATTN_ERR_UNSUPPORTED;
    size_t nst = (budget - fixed) / (2 * tile_bytes + 24);
    if (nst > 8) nst = 8;
    pl.nstages = static_cast<uint32_t>(nst);
    pl.smem_bytes = nst * (2 * tile_bytes + 24) + fixed;
    const size_t slots = static_cast<size_t>(pl.grid) + pl.nseg;
    const size_t rows = slots * pl.ts * pl.hpc * pl.group;
    pl.part_o_floats = rows * head_dim;
    pl.part_lse_floats = (rows + 3) & ~static_cast<size_t>(3);
    // partials, LSEs, tile prefix [nseg+1], arrival counters [nseg] of the single-launch mode, four words of which
    // the first is the status word of the engine's kernel symbol
    pl.prefix_words = (static_cast<size_t>(pl.nseg) + 1 + 3) & ~3ull;
    pl.workspace_bytes =
        (pl.part_o_floats + pl.part_lse_floats + pl.prefix_words + ((static_cast<size_t>(pl.nseg) + 3) & ~3ull) + 4) * 4;
    // the engine's single-launch kernel symbol also keeps first-level group records behind that
    pl.group_base_words = pl.workspace_bytes / 4;
    const size_t group_rows = slots * pl.hpc * pl.group;
    pl.group_o_floats = group_rows * head_dim;
    pl.group_lse_floats = (group_rows + 3) & ~static_cast<size_t>(3);
    pl.group_counter_words = (slots + 3) & ~static_cast<size_t>(3);
    pl.symbol_workspace_bytes = (pl.group_base_words + pl.group_o_floats + pl.group_lse_floats + pl.group_counter_words) * 4;
    *plan = pl;
    return ATTN_OK;
}

}  // namespace b200
