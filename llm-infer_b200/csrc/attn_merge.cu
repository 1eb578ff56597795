// Merge pass: combines partial (O, LSE) results of one query head with the
// engine's online-softmax state merge (src/attention.cu:41-65) written in
// log-sum-exp form. With lse_i = m_i + ln z_i the reference's pairwise rule
//     o_c = o_a (z_a/z_c) e^{m_a-m_c} + o_b (z_b/z_c) e^{m_b-m_c}
// becomes, for n partials at once,
//     out = sum_i o_i * exp(lse_i - L) / sum_j exp(lse_j - L),  L = max_i lse_i,
// and an all-empty row (every lse_i = -inf, where the reference computes 0/0)
// yields zeros.
//
// One CTA per (output row, slice of head_dim). A thread owns four floats of the slice and every P-th partial; it
// folds its partials into a running (m, z, acc) state exactly as the reference folds tiles, with the loads of up to
// six partials (LSE and O together) in flight before the first is used, so a row with a partial per split-pass CTA
// (one long sequence) costs one or two L2 round trips instead of a chain of them. Warps reduce with shuffles, the
// eight warps through shared memory with one barrier. Two users:
//   * the decode split pass (partials of consecutive slots, located per row),
//   * attn_merge(): partials stacked with a constant stride, e.g. the all-gather
//     buffer of the KV-sharded multi-GPU decode.
// With an exchange descriptor (attn_decode_sharded) the same kernel also carries the collective of the multi-GPU
// path: peer stores of the merged slice as self-validating 64-bit words, bounded wait for the other ranks' words,
// merge of the arrived records.
#include "attn_internal.cuh"
#include "merge_device.cuh"
#include "ptx_sm100.cuh"

namespace b200 {

namespace {

constexpr int kMergeWarps = merge_detail::kWarps;
constexpr int kMergeThreads = merge_detail::kThreads;

#ifdef ATTN_TRACE
#define MTRACE(k) ATTN_TRACE_AT((p.trace && threadIdx.x == 0) ? p.trace + static_cast<size_t>(blockIdx.x) * 8 : nullptr, k)
#else
#define MTRACE(k) \
    do {          \
    } while (0)
#endif

// Many output rows with few partials each (batched decode: a row's segment is shared by a handful of split-pass
// CTAs): two WARPS per row (even and odd partials), lanes over head_dim, the loads of up to six partials per warp in
// flight - a dozen partials cost one L2 round trip - and one small exchange through shared memory. Registers and
// shared memory are kept low enough that every CTA of this pass fits next to a split-pass CTA (which leaves about
// 17 K registers and 13 KB of shared memory per SM) and is already waiting on its SM when that pass ends.
constexpr int kRowsPerCta = kMergeWarps / 2;

template <int VEC, int CHUNKS>
__global__ void __launch_bounds__(kMergeThreads, 4) merge_rows_kernel(const __grid_constant__ MergeParams p) {
    using V = typename MergeVec<VEC>::type;
    constexpr int kInFlight = CHUNKS == 1 ? 6 : 3;
    constexpr int HEAD_DIM = CHUNKS * 32 * VEC;
    __shared__ float s_mz[kRowsPerCta][2];
    __shared__ __align__(16) float s_acc[kRowsPerCta][HEAD_DIM];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int sub = warp & 1;  // this warp folds partials sub, sub + 2, ...
    const int rl = warp >> 1;
    const uint32_t row = blockIdx.x * kRowsPerCta + rl;
    const bool live = row < p.rows;
    MTRACE(0);
    grid_dep_launch_dependents();
    const float* po = nullptr;
    const float* pl = nullptr;
    uint64_t o_stride = 0, l_stride = 0;
    uint32_t n = 0;
    if (live) locate_partials(p, row, po, pl, o_stride, l_stride, n);
    grid_dep_wait();
    MTRACE(1);
    float m = -INFINITY, z = 0.f;
    float acc[CHUNKS][VEC];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[c][e] = 0.f;
    for (uint32_t i0 = sub; i0 < n; i0 += 2 * kInFlight) {
        float lw[kInFlight];
        V x[kInFlight][CHUNKS];
#pragma unroll
        for (int b = 0; b < kInFlight; ++b) {
            const uint32_t i = i0 + 2 * b;
            lw[b] = -INFINITY;
            if (i < n) {
                lw[b] = __ldcg(pl + i * l_stride);
                const float* src = po + i * o_stride + lane * VEC;
#pragma unroll
                for (int c = 0; c < CHUNKS; ++c) x[b][c] = __ldcg(reinterpret_cast<const V*>(src + c * 32 * VEC));
            }
        }
        float bm = lw[0];
#pragma unroll
        for (int b = 1; b < kInFlight; ++b) bm = fmaxf(bm, lw[b]);
        if (bm > m) {
            const float s = __expf(m - bm);  // 0 when nothing was folded yet
            z *= s;
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
                for (int e = 0; e < VEC; ++e) acc[c][e] *= s;
            m = bm;
        }
        if (m != -INFINITY) {
#pragma unroll
            for (int b = 0; b < kInFlight; ++b) {
                if (i0 + 2 * b < n) {
                    const float w = __expf(lw[b] - m);  // 0 for an empty partial
                    z += w;
#pragma unroll
                    for (int c = 0; c < CHUNKS; ++c) {
                        const float* xs = reinterpret_cast<const float*>(&x[b][c]);
#pragma unroll
                        for (int e = 0; e < VEC; ++e) acc[c][e] = fmaf(w, xs[e], acc[c][e]);
                    }
                }
            }
        }
    }
    MTRACE(2);
    // the odd warp hands its state (m, z, acc) to the even warp of the row, which merges the two and stores
    if (sub == 1) {
        if (lane == 0) {
            s_mz[rl][0] = m;
            s_mz[rl][1] = z;
        }
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
            for (int e = 0; e < VEC; ++e) s_acc[rl][c * 32 * VEC + lane * VEC + e] = acc[c][e];
    }
    __syncthreads();
    if (sub == 1 || !live) return;
    const float m1 = s_mz[rl][0], z1 = s_mz[rl][1];
    const float mx = fmaxf(m, m1);
    const float e0 = m == -INFINITY ? 0.f : __expf(m - mx), e1 = m1 == -INFINITY ? 0.f : __expf(m1 - mx);
    const float zt = z * e0 + z1 * e1;
    const float inv_z = zt > 0.f ? 1.f / zt : 0.f;
    const size_t obase = static_cast<size_t>(row) * p.head_dim + lane * VEC;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            const float v = acc[c][e] * e0 + s_acc[rl][c * 32 * VEC + lane * VEC + e] * e1;
            store_out(p.o, p.o_dtype, obase + c * 32 * VEC + e, v * inv_z);
        }
    if (p.lse && lane == 0) p.lse[row] = zt > 0.f ? mx + logf(zt) : -INFINITY;
    MTRACE(3);
}

// XCHG: the launch carries the cross-GPU exchange (its record buffer is only reserved then, so that the plain
// pass keeps a small shared-memory footprint and fits next to a split-pass CTA).
template <int SLICE, bool XCHG>
__global__ void __launch_bounds__(kMergeThreads) merge_kernel(const __grid_constant__ MergeParams p) {
    constexpr int LP = SLICE / 4;             // lanes that share one partial (a float4 each)
    __shared__ MergeScratch<SLICE> s_scratch;
    __shared__ float s_out[SLICE + 1];
    const int tid = threadIdx.x;
    const int dl = tid % LP;  // which four floats of the slice
    const uint32_t nslices = p.head_dim / SLICE;
    const uint32_t row = blockIdx.x / nslices;
    const uint32_t slice = blockIdx.x - row * nslices;
    MTRACE(0);
    // Let the next kernel of the stream be scheduled (a weight GEMV starts prefetching), then wait for the grid that
    // produced the partials (no-op without a programmatic dependency).
    grid_dep_launch_dependents();
    const float* po;
    const float* pl;
    uint64_t o_stride, l_stride;
    uint32_t n;
    locate_partials(p, row, po, pl, o_stride, l_stride, n);
    if (po) po += slice * SLICE + dl * 4;
    grid_dep_wait();
    MTRACE(1);
    // The exchange's step number (step 0 in the arguments = count steps on the device, which keeps the launch
    // arguments constant, e.g. for graph replay) is fetched here, together with the partials, not when it is needed.
    // Not earlier: this grid may be resident while the previous exchange launch, which advances the counter with its
    // last cell, is still running; the wait above orders the two (this pass waits for its split pass, which waited
    // for that launch).
    uint32_t step_early = 0;
    if (XCHG && tid == 0 && p.xchg_world) {
        const unsigned long long* ctl0 =
            p.xchg_peers[p.xchg_rank] + 2ull * p.xchg_world * exchange_rank_words(p.rows, p.head_dim, SLICE);
        step_early = p.xchg_step ? p.xchg_step : static_cast<uint32_t>(*reinterpret_cast<const volatile unsigned long long*>(ctl0)) + 1u;
    }

    float x_out, lse_local;
    merge_cell<SLICE>(po, pl, o_stride, l_stride, n, tid, s_scratch, [] { __syncthreads(); }, x_out, lse_local);
    MTRACE(2);
    const size_t out_idx = static_cast<size_t>(row) * p.head_dim + slice * SLICE + tid;
    if (!XCHG || p.xchg_world == 0) {
        if (tid < SLICE) store_out(p.o, p.o_dtype, out_idx, x_out);
        if (p.lse && slice == 0 && tid == 0) p.lse[row] = lse_local;
        MTRACE(3);
        return;
    }

    // ---- cross-GPU part: compute step followed by its collective, in the same kernel -------------------------
    // 1. store this rank's merged slice and LSE into every rank's exchange buffer: plain 64-bit stores to peer
    //    memory over NVLink, each word = value | step << 32, so a word is its own arrival flag (no fence, no
    //    separate flag write);
    // 2. collect the world records of this (row, slice) cell from the local buffer, polling (bounded) each word until
    //    it carries the current step;
    // 3. merge the records. Cells are independent, so a CTA waits for its own cell only.
    // Records are double-buffered by step parity: a peer can be at most one step ahead (it needs this rank's
    // record of step s+1 to finish s+1), so the cell of parity s is never overwritten before it was read.
    __shared__ uint32_t s_fail;
    __shared__ uint32_t s_step;
    __shared__ float s_rec[XCHG ? ATTN_MAX_PEERS : 1][SLICE + 1];
    const uint32_t world = p.xchg_world, me = p.xchg_rank;
    const uint64_t rank_words = exchange_rank_words(p.rows, p.head_dim, SLICE);
    constexpr uint32_t kCell = SLICE + 1;
    // control words behind the records of the local buffer: [0] = steps completed so far, [1] = CTAs finished in this step
    unsigned long long* ctl = p.xchg_peers[me] + 2ull * world * rank_words;
    if (tid == 0) {
        s_fail = 0;
        s_step = step_early;
    }
    if (tid < SLICE) s_out[tid] = x_out;
    if (tid == 0) s_out[SLICE] = lse_local;
    __syncthreads();
    const uint32_t step = s_step;
    // Every CTA of this launch has read the step by now or will before it finishes its own cell, and the counter only
    // advances after all CTAs have finished, so all cells of one launch agree on the step.
    auto finish_cell = [&]() {
        if (p.xchg_step == 0 && tid == 0) {
            __threadfence();
            if (atomicAdd(ctl + 1, 1ull) == gridDim.x - 1) {
                ctl[1] = 0;
                __threadfence();
                atomicAdd(ctl, 1ull);
            }
        }
    };
    const uint64_t cell_off = (static_cast<uint64_t>(step & 1u) * world) * rank_words +
                              static_cast<uint64_t>(blockIdx.x) * kCell;  // + source rank * rank_words
    const unsigned long long tag = static_cast<unsigned long long>(step) << 32;
    for (uint32_t idx = tid; idx < world * kCell; idx += kMergeThreads) {
        const uint32_t r = idx / kCell, w = idx - r * kCell;
        st_sys_u64(p.xchg_peers[r] + cell_off + me * rank_words + w, tag | __float_as_uint(s_out[w]));
    }
    MTRACE(3);
    for (uint32_t idx = tid; idx < world * kCell; idx += kMergeThreads) {
        const uint32_t r = idx / kCell, w = idx - r * kCell;
        const unsigned long long* src = p.xchg_peers[me] + cell_off + r * rank_words + w;
        bool seen = false;
        for (uint32_t it = 0; it < p.xchg_poll_limit; ++it) {
            const unsigned long long v = ld_sys_u64(src);
            if (static_cast<uint32_t>(v >> 32) == step) {
                s_rec[r][w] = __uint_as_float(static_cast<uint32_t>(v));
                seen = true;
                break;
            }
            if (it > 8) __nanosleep(40);
        }
        if (!seen) {
            // a peer never delivered this cell: report it and leave the output untouched
            if (p.status) atomicOr(p.status, ATTN_STATUS_WAIT_TIMEOUT);
            atomicExch(&s_fail, 1u);
        }
    }
    __syncthreads();
    MTRACE(4);
    if (s_fail) {
        finish_cell();
        return;
    }
    float gmx = -INFINITY;
    for (uint32_t r = 0; r < world; ++r) gmx = fmaxf(gmx, s_rec[r][SLICE]);
    float gz = 0.f, acc_d = 0.f;
    if (gmx != -INFINITY) {
        for (uint32_t r = 0; r < world; ++r) {
            const float w = __expf(s_rec[r][SLICE] - gmx);  // 0 for a rank whose shard was empty
            gz += w;
            if (tid < SLICE) acc_d = fmaf(w, s_rec[r][tid], acc_d);
        }
    }
    if (tid < SLICE) store_out(p.o, p.o_dtype, out_idx, gz > 0.f ? acc_d / gz : 0.f);
    if (p.lse && slice == 0 && tid == 0) p.lse[row] = gz > 0.f ? gmx + logf(gz) : -INFINITY;
    finish_cell();
    MTRACE(5);
}

template <int SLICE>
int launch_merge_slice(const MergeParams& p, cudaStream_t stream, bool dependent_launch) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(p.rows * (p.head_dim / SLICE));
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
    if (p.xchg_world) B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, merge_kernel<SLICE, true>, p));
    else B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, merge_kernel<SLICE, false>, p));
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return ATTN_OK;
}

template <int VEC, int CHUNKS>
int launch_merge_rows(const MergeParams& p, cudaStream_t stream, bool dependent_launch) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((p.rows + kRowsPerCta - 1) / kRowsPerCta);
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
    B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, merge_rows_kernel<VEC, CHUNKS>, p));
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return ATTN_OK;
}

}  // namespace

int launch_merge(const MergeParams& p, cudaStream_t stream, bool dependent_launch) {
    if (p.rows == 0) return ATTN_OK;
    if (p.head_dim % 32 != 0) return ATTN_ERR_UNSUPPORTED;
    // Many rows: the split pass's CTAs are shared out over many segments, so a row has few partials (on average
    // (CTAs + segments) / segments of them) and a warp folds them alone; likewise a caller's short stack of partials.
    const bool few_parts = p.split_grid ? p.rows >= 256 : (p.rows >= 256 && p.n_parts <= 16);
    if (few_parts && p.xchg_world == 0) {
        switch (p.head_dim) {
            case 32: return launch_merge_rows<1, 1>(p, stream, dependent_launch);
            case 64: return launch_merge_rows<2, 1>(p, stream, dependent_launch);
            case 128: return launch_merge_rows<4, 1>(p, stream, dependent_launch);
            case 256: return launch_merge_rows<4, 2>(p, stream, dependent_launch);
            default: break;
        }
    }
    switch (merge_slice_floats(p.rows, p.head_dim)) {
        case 32: return launch_merge_slice<32>(p, stream, dependent_launch);
        case 64: return launch_merge_slice<64>(p, stream, dependent_launch);
        case 128: return launch_merge_slice<128>(p, stream, dependent_launch);
        default: return ATTN_ERR_UNSUPPORTED;
    }
}

}  // namespace b200
