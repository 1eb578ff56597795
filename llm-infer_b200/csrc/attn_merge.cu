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
// With an exchange descriptor (attn_decode_sharded) the same kernel also carries the collective of the multi-GPU
// path: peer stores of the merged row, per-row flags, bounded wait, merge of the arrived records.
#include "attn_internal.cuh"
#include "merge_device.cuh"
#include "ptx_sm100.cuh"

namespace b200 {

namespace {

constexpr int kMergeWarps = 8;
constexpr int kMergeThreads = kMergeWarps * 32;

// One CTA per output row. The eight warps take every eighth partial each (so that up to a few hundred
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
    // Let the next kernel of the stream be scheduled (a weight GEMV starts prefetching), then wait for the grid that
    // produced the partials (no-op without a programmatic dependency).
    grid_dep_launch_dependents();
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
    mx = s_red[0][0];
#pragma unroll
    for (int w = 1; w < kMergeWarps; ++w) mx = fmaxf(mx, s_red[0][w]);
    float z = 0.f;
    if (mx != -INFINITY) {
        for (uint32_t i = tid; i < n; i += kMergeThreads) z += __expf(__ldcg(pl + i * l_stride) - mx);
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) z += __shfl_xor_sync(0xffffffffu, z, off);
    if (lane == 0) s_red[1][warp] = z;
    __syncthreads();
    z = 0.f;
#pragma unroll
    for (int w = 0; w < kMergeWarps; ++w) z += s_red[1][w];
    const float inv_z = z > 0.f ? 1.f / z : 0.f;

    // pass 2: warp w accumulates partials w, w + 8, ...
    float acc[CHUNKS][VEC];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[c][e] = 0.f;
    if (mx != -INFINITY) {
        // four partials per round, all eight loads (LSE and O) issued before any is used: with up to a few hundred
        // partials per row (one long sequence) this loop is bound by L2 latency, not bandwidth
        constexpr int kBatch = 4;
        for (uint32_t i0 = warp; i0 < n; i0 += kMergeWarps * kBatch) {
            float lw[kBatch];
            V x[kBatch][CHUNKS];
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
                const uint32_t i = i0 + b * kMergeWarps;
                const bool valid = i < n;
                lw[b] = valid ? __ldcg(pl + i * l_stride) : -INFINITY;
                const float* src = po + (valid ? i : 0) * o_stride + lane * VEC;
#pragma unroll
                for (int c = 0; c < CHUNKS; ++c) x[b][c] = __ldcg(reinterpret_cast<const V*>(src + c * 32 * VEC));
            }
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
                const float w = __expf(lw[b] - mx) * inv_z;  // 0 for the padding of the last round
#pragma unroll
                for (int c = 0; c < CHUNKS; ++c) {
                    const float* xs = reinterpret_cast<const float*>(&x[b][c]);
#pragma unroll
                    for (int e = 0; e < VEC; ++e) acc[c][e] = fmaf(w, xs[e], acc[c][e]);
                }
            }
        }
    }
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
        for (int e = 0; e < VEC; ++e) s_acc[warp][c * 32 * VEC + lane * VEC + e] = acc[c][e];
    __syncthreads();
    const float lse_local = z > 0.f ? mx + logf(z) : -INFINITY;
    if (p.xchg_world == 0) {
        for (int d = tid; d < HEAD_DIM; d += kMergeThreads) {
            float x = 0.f;
#pragma unroll
            for (int w = 0; w < kMergeWarps; ++w) x += s_acc[w][d];
            store_out(p.o, p.o_dtype, static_cast<size_t>(row) * HEAD_DIM + d, x);
        }
        if (p.lse && tid == 0) p.lse[row] = lse_local;
        return;
    }

    // ---- cross-GPU part: compute step followed by its collective, in the same kernel -------------------------
    // 1. store this rank's merged row into every rank's exchange buffer (plain stores to peer memory over NVLink),
    // 2. system-scope fence, then raise this (rank, row)'s flag on every rank with a release store,
    // 3. wait (bounded) until every rank's flag for this row shows the current step in the local buffer,
    // 4. merge the records that arrived locally. Rows are independent, so a CTA waits for its own row only.
    __shared__ uint32_t s_fail;
    __shared__ uint32_t s_step;
    const uint32_t world = p.xchg_world, me = p.xchg_rank, rows = p.rows;
    const size_t rec_floats = static_cast<size_t>(rows) * (HEAD_DIM + 1);
    const size_t flags_off = 2 * static_cast<size_t>(world) * rec_floats;
    // control words behind the flags of the local buffer: [0] = steps completed so far, [1] = rows finished in this step
    uint32_t* ctl = reinterpret_cast<uint32_t*>(p.xchg_peers[me] + flags_off) + static_cast<size_t>(world) * rows;
    if (tid == 0) {
        s_fail = 0;
        // step 0 in the arguments = count steps on the device (keeps the launch arguments constant, e.g. for graph replay)
        s_step = p.xchg_step ? p.xchg_step : *reinterpret_cast<volatile uint32_t*>(ctl) + 1u;
    }
    __syncthreads();
    const uint32_t step = s_step;
    const size_t rec_me = ((step & 1u) * world + me) * rec_floats;
    // Every CTA of this launch has read the step by now or will before it finishes its own row, and the counter only
    // advances after all rows have finished, so all rows of one launch agree on the step.
    auto finish_row = [&]() {
        if (p.xchg_step == 0 && tid == 0) {
            __threadfence();
            if (atomicAdd(ctl + 1, 1u) == rows - 1) {
                ctl[1] = 0;
                __threadfence();
                atomicAdd(ctl, 1u);
            }
        }
    };
    for (int d = tid; d < HEAD_DIM; d += kMergeThreads) {
        float x = 0.f;
#pragma unroll
            for (int w = 0; w < kMergeWarps; ++w) x += s_acc[w][d];
        for (uint32_t r = 0; r < world; ++r) p.xchg_peers[r][rec_me + static_cast<size_t>(row) * HEAD_DIM + d] = x;
    }
    if (tid == 0) {
        for (uint32_t r = 0; r < world; ++r) p.xchg_peers[r][rec_me + static_cast<size_t>(rows) * HEAD_DIM + row] = lse_local;
    }
    __threadfence_system();
    __syncthreads();
    if (tid < static_cast<int>(world)) {
        uint32_t* remote = reinterpret_cast<uint32_t*>(p.xchg_peers[tid] + flags_off) + static_cast<size_t>(me) * rows + row;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(step) : "memory");
        const uint32_t* local = reinterpret_cast<const uint32_t*>(p.xchg_peers[me] + flags_off) + static_cast<size_t>(tid) * rows + row;
        bool seen = false;
        for (uint32_t it = 0; it < p.xchg_poll_limit; ++it) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(local) : "memory");
            if (v == step) { seen = true; break; }
            __nanosleep(64);
        }
        if (!seen) {
            // a peer never delivered this row: report it and leave the output row untouched
            if (p.status) atomicOr(p.status, ATTN_STATUS_WAIT_TIMEOUT);
            atomicExch(&s_fail, 1u);
        }
    }
    __syncthreads();
    if (s_fail) {
        finish_row();
        return;
    }
    const float* mine = p.xchg_peers[me] + (step & 1u) * world * rec_floats;
    float gmx = -INFINITY;
    for (uint32_t r = 0; r < world; ++r) gmx = fmaxf(gmx, __ldcg(mine + r * rec_floats + static_cast<size_t>(rows) * HEAD_DIM + row));
    float gz = 0.f;
    if (gmx != -INFINITY) {
        for (uint32_t r = 0; r < world; ++r) gz += __expf(__ldcg(mine + r * rec_floats + static_cast<size_t>(rows) * HEAD_DIM + row) - gmx);
    }
    const float inv_gz = gz > 0.f ? 1.f / gz : 0.f;
    for (int d = tid; d < HEAD_DIM; d += kMergeThreads) {
        float acc_d = 0.f;
        if (gmx != -INFINITY) {
            for (uint32_t r = 0; r < world; ++r) {
                const float w = __expf(__ldcg(mine + r * rec_floats + static_cast<size_t>(rows) * HEAD_DIM + row) - gmx) * inv_gz;
                acc_d = fmaf(w, __ldcg(mine + r * rec_floats + static_cast<size_t>(row) * HEAD_DIM + d), acc_d);
            }
        }
        store_out(p.o, p.o_dtype, static_cast<size_t>(row) * HEAD_DIM + d, acc_d);
    }
    if (p.lse && tid == 0) p.lse[row] = gz > 0.f ? gmx + logf(gz) : -INFINITY;
    finish_row();
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
