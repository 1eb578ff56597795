// Weight GEMV for the projections around attention (Q/K/V, output, FFN, classifier): out[b][j] = sum_i x[b][i] *
// W[j][i] with fp16 weights stored [d][n] (n fastest) and fp32 activations, fp32 accumulation, optional symmetric
// clamp, fp32 or fp16 result (the fp16 form writes V straight into its KV-cache row), optionally added to what the
// fp32 output already holds (the residual connections of src/model/block.cpp:169-172,219-222).
//
// Replaces the engine's warp-per-row kernels fused_gemv_clip / fused_gemv_clip_f2h (src/kernels.cu:117-136,229-239,
// scalar 2-byte loads) and matches its CPU matmul() (include/kernels_cpu.hpp:69-80) with the clamp of
// src/model/block.cpp:130-138 (both sides; the engine's GPU kernel clamps only from above, src/kernels.cu:218-227,
// which the CPU path - the model of record - does not).
//
// This file holds the kernel for ONE sequence with a plain output; batches and the fused forms (row segments, SwiGLU,
// k_split) run on the tensor cores (attn_gemv_f16mma.cu). HBM-bound: every weight byte is read exactly once per call.
// One persistent CTA per SM, 16 warps; the activations are staged once in shared memory (fp32); each warp owns
// output rows j, j + #warps, ... and streams a row with 256-bit loads, eight in flight per lane (128 KB in flight per
// SM), streaming (no-allocate) cache policy. Algorithmic bytes per call = d*n*2 + batch*(n*4 + d*sizeof(out)).
#include "attn_internal.cuh"
#include "ptx_sm100.cuh"

namespace b200 {
namespace {

constexpr int kGemvWarps = 16;
constexpr int kGemvThreads = kGemvWarps * 32;
constexpr int kUnroll = 8;  // 32-byte loads in flight per lane (a whole 8 KB row per warp and round)

struct GemvParams {
    void* out;
    const float* x;
    const uint16_t* w;
    uint64_t out_batch_stride;
    uint64_t w_row_stride;    // elements between rows of W (>= n: a launch may cover a column slice)
    uint64_t x_batch_stride;  // elements between sequences of x
    uint32_t n, d;
    float clip;
    int32_t out_dtype;
    int32_t accumulate;
};

struct alignas(32) U8 {
    uint32_t v[8];
};

// 256-bit streaming load (sm_100): read-only path, no L1 allocation, evict-first in L2.
__device__ __forceinline__ U8 ld_stream32(const void* p) {
    U8 r;
    asm volatile("ld.global.nc.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]), "=r"(r.v[5]), "=r"(r.v[6]), "=r"(r.v[7])
                 : "l"(p));
    return r;
}

template <int BATCH>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_f16_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ __align__(16) float s_x[];  // [BATCH][n]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    grid_dep_launch_dependents();  // the next kernel of the stream may be scheduled as SMs free up
    grid_dep_wait();               // x (and out, when accumulating) come from the previous kernel
    // Activations are staged permuted: inside every span of 512 elements, the four elements (16L + 4q .. +3) that
    // lane L multiplies with the q-th quarter of its 32-byte weight chunk are stored at q*128 + 4L, so that the 32
    // lanes of a warp read 512 consecutive bytes (no bank conflicts) although each lane owns 16 consecutive weights.
    for (uint32_t i = tid * 4; i < BATCH * p.n; i += kGemvThreads * 4) {
        const uint32_t b = i / p.n, col = i - b * p.n;
        const uint32_t r = col & 511u;
        const uint32_t dst = (i - r) + ((r & 15u) >> 2) * 128u + (r >> 4) * 4u;
        *reinterpret_cast<float4*>(s_x + dst) = *reinterpret_cast<const float4*>(p.x + b * p.x_batch_stride + col);
    }
    __syncthreads();
    const uint32_t chunks = p.n / 16;  // 32-byte chunks (16 weights) per row
    for (uint32_t j = blockIdx.x * kGemvWarps + warp; j < p.d; j += gridDim.x * kGemvWarps) {
        const uint16_t* row = p.w + static_cast<size_t>(j) * p.w_row_stride;
        float acc[BATCH];
#pragma unroll
        for (int b = 0; b < BATCH; ++b) acc[b] = 0.f;
        for (uint32_t c0 = lane; c0 < chunks; c0 += 32 * kUnroll) {
            U8 wv[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const uint32_t c = c0 + u * 32;
                if (c < chunks) wv[u] = ld_stream32(row + static_cast<size_t>(c) * 16);
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const uint32_t c = c0 + u * 32;
                if (c < chunks) {
                    const __half2* h = reinterpret_cast<const __half2*>(&wv[u]);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {  // 4 weights per step
                        const float2 wa = __half22float2(h[2 * q4]), wb = __half22float2(h[2 * q4 + 1]);
#pragma unroll
                        for (int b = 0; b < BATCH; ++b) {
                            // chunk c = span (c / 32), lane (c % 32); see the permutation above
                            const float4 xv = *reinterpret_cast<const float4*>(s_x + b * p.n + (c >> 5) * 512 + q4 * 128 + (c & 31u) * 4);
                            acc[b] = fmaf(xv.x, wa.x, acc[b]);
                            acc[b] = fmaf(xv.y, wa.y, acc[b]);
                            acc[b] = fmaf(xv.z, wb.x, acc[b]);
                            acc[b] = fmaf(xv.w, wb.y, acc[b]);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int b = 0; b < BATCH; ++b) {
#pragma unroll
            for (int off = 16; off; off >>= 1) acc[b] += __shfl_xor_sync(0xffffffffu, acc[b], off);
        }
        if (lane == 0) {
#pragma unroll
            for (int b = 0; b < BATCH; ++b) {
                float y = acc[b];
                if (p.clip > 0.f) y = fminf(fmaxf(y, -p.clip), p.clip);
                const size_t o = static_cast<size_t>(b) * p.out_batch_stride + j;
                if (p.out_dtype == ATTN_DTYPE_F32) {
                    float* dst = reinterpret_cast<float*>(p.out) + o;
                    *dst = p.accumulate ? *dst + y : y;  // residual connection: x += W h (src/model/block.cpp:169-172)
                }
                else reinterpret_cast<__half*>(p.out)[o] = __float2half_rn(y);
            }
        }
    }
}

template <int BATCH>
int launch_gemv(const GemvParams& p, int sm_count, size_t smem, cudaStream_t stream) {
    auto kernel = gemv_f16_kernel<BATCH>;
    B200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    const uint32_t row_blocks = (p.d + kGemvWarps - 1) / kGemvWarps;
    const uint32_t grid = row_blocks < static_cast<uint32_t>(sm_count) ? row_blocks : static_cast<uint32_t>(sm_count);
    B200_CUDA_TRY(launch_dependent(kernel, dim3(grid), dim3(kGemvThreads), smem, stream, p));
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return ATTN_OK;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int attn_gemv_f16(const AttnGemvArgs* a, void* stream_v) {
    if (!a || !a->out || !a->x || !a->w || a->n == 0 || a->d == 0 || a->batch == 0) return ATTN_ERR_INVALID_ARG;
    if (a->out_dtype != ATTN_DTYPE_F32 && a->out_dtype != ATTN_DTYPE_F16) return ATTN_ERR_INVALID_ARG;
    if (a->accumulate && a->out_dtype != ATTN_DTYPE_F32) return ATTN_ERR_UNSUPPORTED;
    if (a->x_format != ATTN_DTYPE_F32) return ATTN_ERR_UNSUPPORTED;  // prepared activations: Q8_0 kernel only
    if ((reinterpret_cast<uintptr_t>(a->x) & 15u) || (reinterpret_cast<uintptr_t>(a->w) & 31u)) return ATTN_ERR_ALIGNMENT;
    // Batches and the fused forms (row segments, SwiGLU, k_split) run on the tensor cores; one sequence with a plain
    // output stays on the streaming kernel below (same bandwidth, no staging of fragments).
    if (a->batch > 1 || a->split1 || a->split2 || a->swiglu || a->k_split > 1) {
        return launch_gemv_f16_mma(a, static_cast<cudaStream_t>(stream_v));
    }
    if (a->n % 512 != 0) return ATTN_ERR_UNSUPPORTED;
    DeviceInfo dev{};
    int rc = current_device_info(&dev);
    if (rc != ATTN_OK) return rc;
    // The activations of one launch must fit in shared memory. A longer inner dimension (beyond ~ 58 000 elements) is
    // covered by several launches over column slices of W, each adding to the output: the sums of the slices are
    // added in a fixed order, so the result does not depend on scheduling.
    const uint32_t slice_max = static_cast<uint32_t>(static_cast<size_t>(dev.max_smem_optin) / (a->batch * sizeof(float))) & ~511u;
    if (slice_max == 0) return ATTN_ERR_UNSUPPORTED;
    const uint32_t slices = (a->n + slice_max - 1) / slice_max;
    const uint32_t slice_len = ((a->n + slices - 1) / slices + 511u) & ~511u;  // equal slices, multiples of 512
    if (slices > 1 && (a->clip > 0.f || a->out_dtype != ATTN_DTYPE_F32)) return ATTN_ERR_UNSUPPORTED;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    for (uint32_t s = 0; s < slices; ++s) {
        const uint32_t n0 = s * slice_len;
        GemvParams p{};
        p.out = a->out;
        p.x = a->x + n0;
        p.w = static_cast<const uint16_t*>(a->w) + n0;
        p.out_batch_stride = a->out_batch_stride ? a->out_batch_stride : a->d;
        p.w_row_stride = a->n;
        p.x_batch_stride = a->n;
        p.n = (a->n - n0 < slice_len) ? a->n - n0 : slice_len;
        p.d = a->d;
        p.clip = a->clip;
        p.out_dtype = a->out_dtype;
        p.accumulate = (s > 0) ? 1 : a->accumulate;
        const size_t smem = static_cast<size_t>(a->batch) * p.n * sizeof(float);
        rc = launch_gemv<1>(p, dev.sm_count, smem, stream);  // batches go to the tensor-core kernel above
        if (rc != ATTN_OK) return rc;
    }
    return ATTN_OK;
}
