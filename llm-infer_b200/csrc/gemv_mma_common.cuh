// Pieces shared by the tensor-core weight GEMVs (attn_gemv_q8.cu: Q8_0 blocks, attn_gemv_f16mma.cu: fp16 weights):
// the launch parameters, the m16n8k16 MMA wrappers, the TMA tile load of 16 weight rows, the fixed-order reduction of
// the warps' partial sums with its epilogue (row segments, SwiGLU, clamp, accumulate, split-k partials, slices carried
// in shared memory), and the host-side filling of the parameters that do not depend on the weight format.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>

#include "attn_internal.cuh"
#include "merge_device.cuh"
#include "ptx_sm100.cuh"
#include "tma_tile.cuh"

namespace b200 {
namespace gemv_mma {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr uint32_t kRows = 16;  // rows of a group = M of the MMA

struct Params {
    void* out0;               // rows [0, seg_end0)
    void* out1;               // rows [seg_end0, seg_end1)
    void* out2;               // rows [seg_end1, d)
    uint64_t out_stride0, out_stride1, out_stride2;  // elements between sequences of each output
    const float* x;
    uint32_t* status;
    uint64_t x_batch_stride;  // elements between sequences of x
    uint32_t seg_end0, seg_end1;
    uint32_t slice_units;     // units (Q8_0: 32-element blocks; fp16: 64-element chunks) of the inner dimension staged at a time
    uint32_t n_slices;        // slice_units * n_slices = units per row
    uint32_t d, batch;        // output rows; with swiglu W has 2 d rows: gate rows, then up rows
    uint32_t stages;
    uint32_t x_col_pitch;     // 32-bit words between sequences of the staged activations
    uint32_t acc_groups;      // row groups per CTA whose partial sums are carried across slices (0 when n_slices == 1)
    uint32_t swiglu;
    uint32_t k_split;         // > 1: the grid is k_split sets of CTAs, set s computes slice s only and stores its partial sums
    uint64_t partial_stride;  // elements between the partial outputs of consecutive slices
    float clip;
    int32_t out_dtype;
    int32_t accumulate;
    int32_t x_split;          // x holds prepared activations (ATTN_DTYPE_SPLIT16 words) instead of fp32
    const uint8_t* w_tiles;   // Q8_0 weights in the tiled layout (attn_repack_q8_0_tiled), else unused
    uint32_t row_chunks;      // tiles per row group in that layout (n / 256)
};

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The first MMA of a block: accumulates onto zero (constant inputs, no registers to clear).
__device__ __forceinline__ void mma_f16_first(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// Tile load through the TMA engine: 16 rows of W in one request (rows beyond the tensor read as zeros).
__device__ __forceinline__ void tma_load_rows(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y,
                                              uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "l"(policy)
        : "memory");
}

// One fp32 activation quadruple as a B-fragment group {hi(x0,x1), hi(x2,x3), lo(x0,x1), lo(x2,x3)}: fp16 value plus fp16
// residual (~ 22 significant bits), |x| clamped to the fp16 range.
__device__ __forceinline__ uint4 split_activations(float x0, float x1, float x2, float x3) {
    x0 = fminf(fmaxf(x0, -65504.f), 65504.f);
    x1 = fminf(fmaxf(x1, -65504.f), 65504.f);
    x2 = fminf(fmaxf(x2, -65504.f), 65504.f);
    x3 = fminf(fmaxf(x3, -65504.f), 65504.f);
    const __half2 h01 = __floats2half2_rn(x0, x1), h23 = __floats2half2_rn(x2, x3);
    const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
    const __half2 l01 = __floats2half2_rn(x0 - f01.x, x1 - f01.y), l23 = __floats2half2_rn(x2 - f23.x, x3 - f23.y);
    uint4 o;
    o.x = *reinterpret_cast<const uint32_t*>(&h01);
    o.y = *reinterpret_cast<const uint32_t*>(&h23);
    o.z = *reinterpret_cast<const uint32_t*>(&l01);
    o.w = *reinterpret_cast<const uint32_t*>(&l23);
    return o;
}

// This warp's four partial sums of a row group (rows g, g + 8; columns 2t, 2t + 1) into the reduction buffer.
template <int WARPS = kWarps>
__device__ __forceinline__ void store_partial(float* red, uint32_t part, uint32_t warp, uint32_t g, uint32_t t,
                                              const float (&tot)[4]) {
    float* mine = red + (part * WARPS + warp) * 128;
    mine[g * 8 + 2 * t] = tot[0];
    mine[g * 8 + 2 * t + 1] = tot[1];
    mine[(g + 8) * 8 + 2 * t] = tot[2];
    mine[(g + 8) * 8 + 2 * t + 1] = tot[3];
}

// After the block-wide barrier that follows store_partial: threads 0..127 add the warps' partial sums of one row
// group in a fixed order, carry them across slices in shared memory, and on the last slice apply the epilogue (SwiGLU
// over the gate / up parts, clamp, row segment, accumulate or split-k partial output).
template <int WARPS = kWarps>
__device__ __forceinline__ void reduce_and_store(const Params& p, const float* red, float* s_acc, uint32_t tid,
                                                 uint32_t parts, uint32_t gi, uint32_t rg, uint32_t slice,
                                                 uint32_t slice_begin, uint32_t slice_end) {
    if (tid >= 128) return;
    float y[2] = {0.f, 0.f};
    for (uint32_t part = 0; part < parts; ++part) {
        const float* src = red + part * WARPS * 128 + tid;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) v += src[w * 128];
        if (slice_end - slice_begin > 1) {
            float* carry = s_acc + (gi * 2 + part) * 128 + tid;
            if (slice > slice_begin) v += *carry;
            if (slice + 1 < slice_end) *carry = v;
        }
        y[part] = v;
    }
    const uint32_t row = rg * kRows + (tid >> 3), c = tid & 7;
    if (slice + 1 != slice_end || row >= p.d || c >= p.batch) return;
    float v = y[0];
    if (p.swiglu) v = __fdiv_rn(v, 1.0f + expf(-v)) * y[1];  // silu(gate) * up, src/model/block.cpp:206-210
    if (p.clip > 0.f) v = fminf(fmaxf(v, -p.clip), p.clip);
    void* out = p.out0;
    uint64_t stride = p.out_stride0;
    uint32_t r0 = 0;
    if (row >= p.seg_end1) {
        out = p.out2, stride = p.out_stride2, r0 = p.seg_end1;
    } else if (row >= p.seg_end0) {
        out = p.out1, stride = p.out_stride1, r0 = p.seg_end0;
    }
    const size_t o = static_cast<size_t>(c) * stride + (row - r0) + (p.k_split > 1 ? slice_begin * p.partial_stride : 0);
    if (p.out_dtype == ATTN_DTYPE_F32) {
        float* dst = reinterpret_cast<float*>(out) + o;
        *dst = p.accumulate ? *dst + v : v;
    } else if (p.out_dtype == ATTN_DTYPE_SPLIT16) {
        // a sequence's segment is a vector of its own: the group of four is counted from the segment's first row
        store_split16(reinterpret_cast<uint32_t*>(out) + static_cast<size_t>(c) * stride, row - r0, v);
    } else {
        reinterpret_cast<__half*>(out)[o] = __float2half_rn(v);
    }
}

// Argument checks common to both weight formats (after the caller's pointer checks).
inline int check_fused_args(const AttnGemvArgs* a, uint32_t* k_split_out) {
    if (a->batch > 8) return ATTN_ERR_UNSUPPORTED;
    if (a->accumulate && a->out_dtype != ATTN_DTYPE_F32) return ATTN_ERR_UNSUPPORTED;
    if (a->x_format != ATTN_DTYPE_F32 && a->x_format != ATTN_DTYPE_SPLIT16) return ATTN_ERR_INVALID_ARG;
    if (a->out_dtype == ATTN_DTYPE_SPLIT16 && (a->d % 4 || a->split1 % 4 || a->split2 % 4 || a->k_split > 1)) return ATTN_ERR_UNSUPPORTED;
    if (a->swiglu && (a->d % kRows != 0 || a->split1 || a->split2)) return ATTN_ERR_UNSUPPORTED;
    const uint32_t k_split = a->k_split > 1 ? a->k_split : 1;
    if (k_split > 1 && (a->swiglu || a->split1 || a->accumulate || a->clip > 0.f || a->out_dtype != ATTN_DTYPE_F32))
        return ATTN_ERR_UNSUPPORTED;
    if ((a->split1 && (!a->out2 || a->split1 >= a->d)) || (a->split2 && (!a->out3 || a->split2 <= a->split1 || a->split2 >= a->d)))
        return ATTN_ERR_INVALID_ARG;
    *k_split_out = k_split;
    return ATTN_OK;
}

// The parameters that do not depend on the weight format.
inline void fill_common(Params& p, const AttnGemvArgs* a, uint32_t k_split) {
    const uint64_t stride0 = a->out_batch_stride ? a->out_batch_stride : (a->split1 ? a->split1 : a->d);
    p.out0 = a->out;
    p.out_stride0 = stride0;
    p.seg_end0 = a->split1 ? a->split1 : a->d;
    p.out1 = a->out2;
    p.out_stride1 = a->out2_batch_stride ? a->out2_batch_stride : ((a->split2 ? a->split2 : a->d) - p.seg_end0);
    p.seg_end1 = a->split2 ? a->split2 : a->d;
    p.out2 = a->out3;
    p.out_stride2 = a->out3_batch_stride ? a->out3_batch_stride : (a->d - p.seg_end1);
    p.x = a->x;
    p.status = a->status;
    p.x_batch_stride = a->n;
    p.d = a->d;
    p.batch = a->batch;
    p.k_split = k_split;
    p.partial_stride = static_cast<uint64_t>(a->batch) * stride0;
    p.swiglu = a->swiglu ? 1u : 0u;
    p.clip = a->clip;
    p.out_dtype = a->out_dtype;
    p.accumulate = a->accumulate;
    p.x_split = a->x_format == ATTN_DTYPE_SPLIT16;
}

}  // namespace gemv_mma
}  // namespace b200
