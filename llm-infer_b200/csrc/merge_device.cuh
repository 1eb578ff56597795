// Device routine shared by the stand-alone merge kernel and the fused
// (single-launch) decode kernel: one warp merges n partials of one output row.
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

}  // namespace b200
