// Merge pass: combines partial (O, LSE) results of one query head with the
// engine's online-softmax state merge (src/attention.cu:41-65) written in
// log-sum-exp form. With lse_i = m_i + ln z_i the reference's pairwise rule
//     o_c = o_a (z_a/z_c) e^{m_a-m_c} + o_b (z_b/z_c) e^{m_b-m_c}
// becomes, for n partials at once,
//     out = sum_i o_i * exp(lse_i - L) / sum_j exp(lse_j - L),  L = max_i lse_i,
// and an all-empty row (every lse_i = -inf, where the reference computes 0/0)
// yields zeros.
//
// One CTA per output row (batch x head); warps split the partials, lanes split head_dim. Two users:
//   * the decode split pass (partials of consecutive slots, located per row),
//   * attn_merge(): partials stacked with a constant stride, e.g. the all-gather
//     buffer of the KV-sharded multi-GPU decode.
#include "attn_internal.cuh"
#include "merge_device.cuh"
#include "ptx_sm100.cuh"

namespace b200 {

namespace {

constexpr int kMergeWarps = 4;
constexpr int kMergeThreads = kMergeWarps * 32;

// One CTA per output row. The four warps take every fourth partial each (so that up to a few hundred
// partials of a long single sequence are fetched with many loads in flight) and combine through shared memory.
template <int VEC, int CHUNKS>
__global__ void __launch_bounds__(kMergeThreads) merge_kernel(const __grid_constant__ MergeParams p) {
    using V = typename MergeVec<VEC>::type;
    constexpr int HEAD_DIM = CHUNKS * 32 * VEC;
    __shared__ float s_red[2][kMergeWarps];
    __shared__ float s_acc[kMergeWarps][HEAD_DIM];
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const uint32_t row = blockIdx.x;
    // Wait for the grid that produced the partials (no-op without a programmatic dependency).
    grid_dep_wait();

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

    // pass 1: L = max lse, Z = sum exp(lse - L) over all partials (L2-only loads: the producer grid may still
    // have been running when this CTA started)
    float mx = -INFINITY;
    for (uint32_t i = tid; i < n; i += kMergeThreads) mx = fmaxf(mx, __ldcg(pl + i * l_stride));
#pragma unroll
    for (int off = 16; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    if (lane == 0) s_red[0][warp] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(s_red[0][0], s_red[0][1]), fmaxf(s_red[0][2], s_red[0][3]));
    float z = 0.f;
    if (mx != -INFINITY) {
        for (uint32_t i = tid; i < n; i += kMergeThreads) z += __expf(__ldcg(pl + i * l_stride) - mx);
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) z += __shfl_xor_sync(0xffffffffu, z, off);
    if (lane == 0) s_red[1][warp] = z;
    __syncthreads();
    z = s_red[1][0] + s_red[1][1] + s_red[1][2] + s_red[1][3];
    const float inv_z = z > 0.f ? 1.f / z : 0.f;

    // pass 2: warp w accumulates partials w, w + 4, ...
    float acc[CHUNKS][VEC];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[c][e] = 0.f;
    if (mx != -INFINITY) {
#pragma unroll 8
        for (uint32_t i = warp; i < n; i += kMergeWarps) {
            const float w = __expf(__ldcg(pl + i * l_stride) - mx) * inv_z;
            const float* src = po + i * o_stride + lane * VEC;
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c) {
                V x = __ldcg(reinterpret_cast<const V*>(src + c * 32 * VEC));
                const float* xs = reinterpret_cast<const float*>(&x);
#pragma unroll
                for (int e = 0; e < VEC; ++e) acc[c][e] = fmaf(w, xs[e], acc[c][e]);
            }
        }
    }
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
        for (int e = 0; e < VEC; ++e) s_acc[warp][c * 32 * VEC + lane * VEC + e] = acc[c][e];
    __syncthreads();
    for (int d = tid; d < HEAD_DIM; d += kMergeThreads) {
        const float x = (s_acc[0][d] + s_acc[1][d]) + (s_acc[2][d] + s_acc[3][d]);
        store_out(p.o, p.o_dtype, static_cast<size_t>(row) * HEAD_DIM + d, x);
    }
    if (p.lse && tid == 0) p.lse[row] = z > 0.f ? mx + logf(z) : -INFINITY;
}

template <int VEC, int CHUNKS>
int launch_merge_vec(const MergeParams& p, cudaStream_t stream, bool dependent_launch) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(p.rows);
    cfg.blockDim = dim3(kMergeThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (dependent_launch) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, merge_kernel<VEC, CHUNKS>, p));
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return ATTN_OK;
}

}  // namespace

int launch_merge(const MergeParams& p, cudaStream_t stream, bool dependent_launch) {
    if (p.rows == 0) return ATTN_OK;
    const uint32_t d = p.head_dim;
    // lanes own VEC consecutive floats of each 32*VEC chunk; head_dim is 1 or 2 chunks
    if (d == 256) return launch_merge_vec<4, 2>(p, stream, dependent_launch);
    if (d == 128) return launch_merge_vec<4, 1>(p, stream, dependent_launch);
    if (d == 64) return launch_merge_vec<2, 1>(p, stream, dependent_launch);
    if (d == 32) return launch_merge_vec<1, 1>(p, stream, dependent_launch);
    return ATTN_ERR_UNSUPPORTED;
}

}  // namespace b200
