// Device routines shared by the stand-alone merge kernels and the single-launch decode kernel.
#pragma once

#include "attn_internal.cuh"
#include "ptx_sm100.cuh"

namespace b200 {

template <int VEC>
struct MergeVec;
template <>
struct MergeVec<1> { using type = float; };
template <>
struct MergeVec<2> { using type = float2; };
template <>
struct MergeVec<4> { using type = float4; };

// One element of a vector in the prepared-activation form (ATTN_DTYPE_SPLIT16): element idx = 4r + e lives in the
// 16-bit half (e & 1) of word 4r + (e >> 1) (fp16 value) and of word 4r + 2 + (e >> 1) (fp16 residual).
__device__ __forceinline__ void store_split16(void* o, size_t idx, float x) {
    x = fminf(fmaxf(x, -65504.f), 65504.f);
    const __half hi = __float2half_rn(x);
    const __half lo = __float2half_rn(x - __half2float(hi));
    __half* words = reinterpret_cast<__half*>(o) + (idx & ~static_cast<size_t>(3)) * 2;  // 8 halves per group of 4
    const size_t e = idx & 3;
    words[(e >> 1) * 2 + (e & 1)] = hi;
    words[4 + (e >> 1) * 2 + (e & 1)] = lo;
}

__device__ __forceinline__ void store_out(void* o, int32_t dtype, size_t idx, float x) {
    if (dtype == ATTN_DTYPE_F32) reinterpret_cast<float*>(o)[idx] = x;
    else if (dtype == ATTN_DTYPE_F16) reinterpret_cast<__half*>(o)[idx] = __float2half_rn(x);
    else if (dtype == ATTN_DTYPE_SPLIT16) store_split16(o, idx, x);
    else reinterpret_cast<__nv_bfloat16*>(o)[idx] = __float2bfloat16_rn(x);
}

// out[row] = sum_i w_i * po[i*o_stride + :], w_i = exp(pl[i*l_stride] - L) / Z   (log-sum-exp form of
// the state merge in src/attention.cu:41-65; an all-empty row gives zeros). Partials are read with
// L2-only loads: the grid that wrote them may still have been running when this CTA started.
// CHUNKS * 32 * VEC == head_dim.
template <int VEC, int CHUNKS>
__device__ __forceinline__ void warp_merge_row(const float* po, const float* pl, uint64_t o_stride, uint64_t l_stride,
                                               uint32_t n, void* o, int32_t o_dtype, float* lse_out, size_t row,
                                               int lane) {
    using V = typename MergeVec<VEC>::type;
    constexpr int HEAD_DIM = CHUNKS * 32 * VEC;
    float mx = -INFINITY;
    for (uint32_t i = lane; i < n; i += 32) mx = fmaxf(mx, __ldcg(pl + i * l_stride));
#pragma unroll
    for (int off = 16; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    float z = 0.f;
    if (mx != -INFINITY) {
        for (uint32_t i = lane; i < n; i += 32) z += __expf(__ldcg(pl + i * l_stride) - mx);
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) z += __shfl_xor_sync(0xffffffffu, z, off);
    const float inv_z = z > 0.f ? 1.f / z : 0.f;

    float acc[CHUNKS][VEC];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[c][i] = 0.f;
    if (mx != -INFINITY) {
#pragma unroll 4
        for (uint32_t i = 0; i < n; ++i) {
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
    const size_t obase = row * HEAD_DIM + lane * VEC;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
        for (int e = 0; e < VEC; ++e) store_out(o, o_dtype, obase + c * 32 * VEC + e, acc[c][e]);
    if (lse_out && lane == 0) lse_out[row] = z > 0.f ? mx + logf(z) : -INFINITY;
}


// Where the partials of output row `row` are: n of them, partial i at po + i * o_stride (head_dim floats) with its
// LSE at pl + i * l_stride. For the decode split pass these are the consecutive slots the pass wrote for the row's
// segment; with ragged lengths the tile prefix is read, which that pass writes: the wait for it happens in here.
__device__ __forceinline__ void locate_partials(const MergeParams& p, uint32_t row, const float*& po, const float*& pl,
                                                uint64_t& o_stride, uint64_t& l_stride, uint32_t& n) {
    if (p.split_grid) {
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
            grid_dep_wait();  // the tile prefix is written by the split pass
            nt = p.seg_prefix[nseg];
            tile0 = p.seg_prefix[seg];
            tile_end = p.seg_prefix[seg + 1];
        } else {
            const uint64_t tu = (clamped_len(p.kv_len_uniform, p.kv_capacity) + p.tile_rows - 1) / p.tile_rows;
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
#ifdef ATTN_BOUNDS_CHECK
            if (row0 + static_cast<uint64_t>(n - 1) * l_stride >= p.part_rows) {  // would read past the partials
                if (p.status) atomicOr(p.status, ATTN_STATUS_BAD_INDEX);
                n = 0;
            }
#endif
        }
    } else {
        n = p.n_parts;
        o_stride = p.o_part_stride;
        l_stride = p.lse_part_stride;
        po = p.part_o + static_cast<uint64_t>(row) * p.head_dim;
        pl = p.part_lse + row;
    }
}

// 256 threads merge n partial records of `rows` consecutive output rows each: partial i of row r at
// po + i * o_stride + r * D (D floats) with its LSE at pl + i * l_stride + r. A thread owns four floats of one row over
// all partials and folds them into a running (m, z, acc) state as the reference folds tiles
// (src/attention.cu:41-65), eight partials' loads (LSE and values, L2-only) in flight at a time; no thread needs
// another's result. store(r, f, value, lse) receives the normalised float4 number f of row r and the row's
// log-sum-exp (zeros and -inf for an all-empty row). (Inlined on purpose: as a call, the variables that `store`
// captures by reference had to live in local memory for the whole calling kernel, which slowed its streaming loop.)
template <int D, typename Store>
__device__ __forceinline__ void cta_merge_rows(const float* po, const float* pl, uint64_t o_stride, uint64_t l_stride,
                                               uint32_t n, uint32_t rows, int tid, Store store) {
    constexpr int F4 = D / 4;
    constexpr int kInFlight = 8;
    for (uint32_t it = tid; it < rows * F4; it += 256) {
        const uint32_t r = it / F4, f = it - r * F4;
        const float* o0 = po + static_cast<size_t>(r) * D + f * 4;
        const float* l0 = pl + r;
        float m = -INFINITY, z = 0.f;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (uint32_t i0 = 0; i0 < n; i0 += kInFlight) {
            float lw[kInFlight];
            float4 x[kInFlight];
#pragma unroll
            for (int b = 0; b < kInFlight; ++b) {
                const uint32_t i = i0 + b;
                lw[b] = -INFINITY;
                x[b] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (i < n) {
                    lw[b] = __ldcg(l0 + i * l_stride);
                    x[b] = __ldcg(reinterpret_cast<const float4*>(o0 + i * o_stride));
                }
            }
            float bm = lw[0];
#pragma unroll
            for (int b = 1; b < kInFlight; ++b) bm = fmaxf(bm, lw[b]);
            if (bm > m) {
                const float sc = __expf(m - bm);  // 0 when nothing was folded yet
                z *= sc;
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[e] *= sc;
                m = bm;
            }
            if (m != -INFINITY) {
#pragma unroll
                for (int b = 0; b < kInFlight; ++b) {
                    const float w = __expf(lw[b] - m);  // 0 for empty partials and for the padding of the last round
                    z += w;
                    acc[0] = fmaf(w, x[b].x, acc[0]);
                    acc[1] = fmaf(w, x[b].y, acc[1]);
                    acc[2] = fmaf(w, x[b].z, acc[2]);
                    acc[3] = fmaf(w, x[b].w, acc[3]);
                }
            }
        }
        const float inv = z > 0.f ? 1.f / z : 0.f;
        store(r, f, make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv), z > 0.f ? m + logf(z) : -INFINITY);
    }
}

namespace merge_detail {
constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kLoadsInFlight = 6;
}  // namespace merge_detail

// Shared-memory scratch of merge_cell().
template <int SLICE>
struct MergeScratch {
    float m[merge_detail::kWarps];
    float z[merge_detail::kWarps];
    alignas(16) float acc[merge_detail::kWarps][SLICE];
};

// 256 threads merge the n partials of one cell = (output row, SLICE floats of head_dim). Thread tid owns four floats of
// the slice (tid % (SLICE/4)) and every P-th partial (P = 256 / (SLICE/4)); it folds its partials into a running
// (m, z, acc) state exactly as the reference folds tiles (src/attention.cu:41-65), with the loads of up to six
// partials (LSE and O together, L2-only: the grid that wrote them may still have been running when this CTA started)
// in flight before the first is used. Warps reduce with shuffles, the eight warps through `s` with one barrier
// (`sync` is that barrier over exactly these 256 threads). po already points at this thread's four floats of partial
// 0. On return x_out holds the merged, normalised value of element tid of the slice (threads tid < SLICE) and lse
// the row's log-sum-exp (every thread); an all-empty row gives zeros and -inf.
template <int SLICE, typename Sync>
__device__ __forceinline__ void merge_cell(const float* po, const float* pl, uint64_t o_stride, uint64_t l_stride,
                                           uint32_t n, int tid, MergeScratch<SLICE>& s, Sync sync, float& x_out,
                                           float& lse) {
    using namespace merge_detail;
    constexpr int LP = SLICE / 4;
    constexpr int P = kThreads / LP;
    const int lane = tid & 31, warp = tid >> 5;
    const int pg = tid / LP, dl = tid % LP;
    float m_t = -INFINITY, z_t = 0.f;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (uint32_t i0 = pg; i0 < n; i0 += P * kLoadsInFlight) {
        float lw[kLoadsInFlight];
        float4 x[kLoadsInFlight];
#pragma unroll
        for (int b = 0; b < kLoadsInFlight; ++b) {
            const uint32_t i = i0 + b * P;
            lw[b] = -INFINITY;
            x[b] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < n) {  // no load for the padding of the last round
                lw[b] = __ldcg(pl + i * l_stride);
                x[b] = __ldcg(reinterpret_cast<const float4*>(po + i * o_stride));
            }
        }
        float bm = lw[0];
#pragma unroll
        for (int b = 1; b < kLoadsInFlight; ++b) bm = fmaxf(bm, lw[b]);
        if (bm > m_t) {
            const float sc = __expf(m_t - bm);  // 0 when nothing was folded yet (m_t = -inf)
            z_t *= sc;
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[e] *= sc;
            m_t = bm;
        }
        if (m_t != -INFINITY) {
#pragma unroll
            for (int b = 0; b < kLoadsInFlight; ++b) {
                const float w = __expf(lw[b] - m_t);  // 0 for empty partials and for the padding of the last round
                z_t += w;
                acc[0] = fmaf(w, x[b].x, acc[0]);
                acc[1] = fmaf(w, x[b].y, acc[1]);
                acc[2] = fmaf(w, x[b].z, acc[2]);
                acc[3] = fmaf(w, x[b].w, acc[3]);
            }
        }
    }
    // warp: common maximum, then sums over the partial groups of the warp
    float m_w = m_t;
#pragma unroll
    for (int off = 16; off; off >>= 1) m_w = fmaxf(m_w, __shfl_xor_sync(0xffffffffu, m_w, off));
    const float sc = m_t == -INFINITY ? 0.f : __expf(m_t - m_w);
    float z_w = dl == 0 ? z_t * sc : 0.f;  // z_t is replicated over the LP lanes of a partial group
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[e] *= sc;
#pragma unroll
    for (int off = 16; off; off >>= 1) z_w += __shfl_xor_sync(0xffffffffu, z_w, off);
#pragma unroll
    for (int off = LP; off < 32; off <<= 1) {
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], off);
    }
    if (lane < LP) *reinterpret_cast<float4*>(&s.acc[warp][lane * 4]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    if (lane == 0) {
        s.m[warp] = m_w;
        s.z[warp] = z_w;
    }
    sync();
    // CTA: the eight warp states merged by every thread that owns an output element
    float mx = s.m[0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) mx = fmaxf(mx, s.m[w]);
    float z = 0.f;
    x_out = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
        const float e = s.m[w] == -INFINITY ? 0.f : __expf(s.m[w] - mx);
        z = fmaf(s.z[w], e, z);
        if (tid < SLICE) x_out = fmaf(s.acc[w][tid], e, x_out);
    }
    x_out *= z > 0.f ? 1.f / z : 0.f;
    lse = z > 0.f ? mx + logf(z) : -INFINITY;
}

}  // namespace b200
