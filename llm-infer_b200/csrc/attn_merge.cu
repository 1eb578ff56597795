// Merge pass: combines partial (O, LSE) results of one query head with the
// engine's online-softmax state merge (src/attention.cu:41-65) written in
// log-sum-exp form. With lse_i = m_i + ln z_i the reference's pairwise rule
//     o_c = o_a (z_a/z_c) e^{m_a-m_c} + o_b (z_b/z_c) e^{m_b-m_c}
// becomes, for n partials at once,
//     out = sum_i o_i * exp(lse_i - L) / sum_j exp(lse_j - L),  L = max_i lse_i,
// and an all-empty row (every lse_i = -inf, where the reference computes 0/0)
// yields zeros.
//
// One warp per output row (batch x head); lanes split head_dim. Two users:
//   * the decode split pass (partials of consecutive slots, located per row),
//   * attn_merge(): partials stacked with a constant stride, e.g. the all-gather
//     buffer of the KV-sharded multi-GPU decode.
#include "attn_internal.cuh"
#include "merge_device.cuh"
#include "ptx_sm100.cuh"

namespace b200 {

namespace {

constexpr int kMergeWarps = 4;

template <int VEC>
__global__ void __launch_bounds__(kMergeWarps * 32) merge_kernel(const __grid_constant__ MergeParams p) {
    const int lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * kMergeWarps + (threadIdx.x >> 5);
    // Wait for the grid that produced the partials (no-op without a programmatic dependency).
    grid_dep_wait();
    if (row >= p.rows) return;

    const float* po;
    const float* pl;
    uint64_t o_stride, l_stride;
    uint32_t n;
    if (p.split_grid) {
        // locate the consecutive slots the split pass wrote for this row's segment
        const uint32_t b = row / p.n_heads;
        const uint32_t h = row - b * p.n_heads;
        const uint32_t kvh = h / p.group;
        const uint32_t g = h - kvh * p.group;
        const uint32_t hg = kvh / p.hpc;
        const uint32_t hh = kvh - hg * p.hpc;
        const uint32_t nseg = p.batch * p.head_groups;
        const uint32_t seg = b * p.head_groups + hg;
        uint64_t nt, tile0, tile_end;
        if (p.kv_len) {
            nt = p.seg_prefix[nseg];
            tile0 = p.seg_prefix[seg];
            tile_end = p.seg_prefix[seg + 1];
        } else {
            const uint64_t tu = (p.kv_len_uniform + p.tile_rows - 1) / p.tile_rows;
            nt = tu * nseg;
            tile0 = tu * seg;
            tile_end = tile0 + tu;
        }
        if (tile_end == tile0) {
            n = 0;
            po = nullptr;
            pl = nullptr;
            o_stride = l_stride = 0;
        } else {
            const uint32_t a = active_ctas(p.split_grid, p.max_ctas, p.min_tiles_per_cta, nt);
            const uint32_t c_first = cta_of_tile(tile0, nt, a);
            const uint32_t c_last = cta_of_tile(tile_end - 1, nt, a);
            n = (c_last - c_first + 1) * p.ts;
            const uint64_t first_slot = (static_cast<uint64_t>(c_first) + seg) * p.ts;
            const uint64_t row0 = (first_slot * p.hpc + hh) * p.group + g;
            l_stride = static_cast<uint64_t>(p.hpc) * p.group;
            o_stride = l_stride * p.head_dim;
            po = p.part_o + row0 * p.head_dim;
            pl = p.part_lse + row0;
        }
    } else {
        n = p.n_parts;
        o_stride = p.o_part_stride;
        l_stride = p.lse_part_stride;
        po = p.part_o + static_cast<uint64_t>(row) * p.head_dim;
        pl = p.part_lse + row;
    }

    if (p.head_dim == 64 * VEC) {
        warp_merge_row<VEC, 2>(po, pl, o_stride, l_stride, n, p.o, p.o_dtype, p.lse, row, lane);
    } else {
        warp_merge_row<VEC, 1>(po, pl, o_stride, l_stride, n, p.o, p.o_dtype, p.lse, row, lane);
    }
}

template <int VEC>
int launch_merge_vec(const MergeParams& p, cudaStream_t stream, bool dependent_launch) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((p.rows + kMergeWarps - 1) / kMergeWarps);
    cfg.blockDim = dim3(kMergeWarps * 32);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (dependent_launch) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, merge_kernel<VEC>, p));
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return ATTN_OK;
}

}  // namespace

int launch_merge(const MergeParams& p, cudaStream_t stream, bool dependent_launch) {
    if (p.rows == 0) return ATTN_OK;
    const uint32_t d = p.head_dim;
    // lanes own VEC consecutive floats of each 32*VEC chunk; head_dim is 1 or 2 chunks
    if (d == 128 || d == 256) return launch_merge_vec<4>(p, stream, dependent_launch);
    if (d == 64) return launch_merge_vec<2>(p, stream, dependent_launch);
    if (d == 32) return launch_merge_vec<1>(p, stream, dependent_launch);
    return ATTN_ERR_UNSUPPORTED;
}

}  // namespace b200
