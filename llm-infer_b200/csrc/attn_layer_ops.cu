// The small per-token steps of a transformer block that sit between the weight GEMVs and attention, for a batch of
// sequences per launch: embedding row copy, RMSNorm, the SwiGLU gate, greedy argmax over the logits. They restate, on
// the device, the CPU steps of the engine's forward pass (the model of record; its CUDA block stops after attention,
// src/model/block.cu:235-239, and its CUDA model has no classifier, src/model/model.cu:67-87):
//   embedding   src/model/model.cpp:101-118 (fp16 table row -> fp32 x)
//   rmsnorm     include/kernels_cpu.hpp:43-67 (x / sqrt(mean(x^2) + eps) * weight, division before the multiply)
//   swiglu      src/model/block.cpp:206-210 with silu(x) = x / (1 + expf(-x)), include/kernels_cpu.hpp:198
//   argmax      tools/infer.cpp:64-74 (first index of the maximum)
// All of them move a few KB to a few hundred KB per sequence: latency-bound, no roofline is quoted for them. They are
// launched as programmatic dependents (their launch overlaps the previous kernel's tail) and wait for it first thing.
#include <cuda_fp16.h>

#include "attn_internal.cuh"
#include "ptx_sm100.cuh"

namespace b200 {
namespace {

constexpr int kOpsThreads = 256;

__device__ __forceinline__ float block_sum(float v, float* s_red) {
#pragma unroll
    for (int off = 16; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    float t = 0.f;
    // fixed order over the warps: the result does not depend on scheduling
    for (int w = 0; w < kOpsThreads / 32; ++w) t += s_red[w];
    __syncthreads();
    return t;
}

__global__ void __launch_bounds__(kOpsThreads) embed_kernel(float* x, const __half* table, const uint32_t* tokens,
                                                            uint32_t dim, uint32_t vocab, uint32_t* status) {
    grid_dep_launch_dependents();
    grid_dep_wait();
    const uint32_t b = blockIdx.x;
    const uint32_t tok = tokens[b];
    if (tok >= vocab) {  // never read outside the table; report instead
        if (threadIdx.x == 0 && status) atomicOr(status, ATTN_STATUS_BAD_SHAPE);
        return;
    }
    const __half* row = table + static_cast<size_t>(tok) * dim;
    for (uint32_t i = threadIdx.x; i < dim; i += kOpsThreads) x[static_cast<size_t>(b) * dim + i] = __half2float(row[i]);
}

// The same row copy from a Q8_0 table (GGML blocks: fp16 scale + 32 signed bytes per 32 elements).
__global__ void __launch_bounds__(kOpsThreads) embed_q8_kernel(float* x, const uint8_t* table, const uint32_t* tokens,
                                                               uint32_t dim, uint32_t vocab, uint32_t* status) {
    grid_dep_launch_dependents();
    grid_dep_wait();
    const uint32_t b = blockIdx.x;
    const uint32_t tok = tokens[b];
    if (tok >= vocab) {
        if (threadIdx.x == 0 && status) atomicOr(status, ATTN_STATUS_BAD_SHAPE);
        return;
    }
    const uint8_t* row = table + static_cast<size_t>(tok) * (dim / 32) * 34;
    for (uint32_t i = threadIdx.x; i < dim; i += kOpsThreads) {
        const uint8_t* blk = row + static_cast<size_t>(i / 32) * 34;
        const float scale = __half2float(__ushort_as_half(static_cast<unsigned short>(blk[0] | (blk[1] << 8))));
        x[static_cast<size_t>(b) * dim + i] = scale * static_cast<float>(static_cast<int8_t>(blk[2 + (i % 32)]));
    }
}

__global__ void __launch_bounds__(kOpsThreads) rmsnorm_kernel(float* out, const float* x, const float* weight,
                                                              uint32_t dim, float eps) {
    __shared__ float s_red[kOpsThreads / 32];
    grid_dep_launch_dependents();
    grid_dep_wait();
    const size_t base = static_cast<size_t>(blockIdx.x) * dim;
    float ss = 0.f;
    for (uint32_t i = threadIdx.x; i < dim; i += kOpsThreads) {
        const float v = x[base + i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, s_red);
    const float rms = sqrtf(ss / static_cast<float>(dim) + eps);
    for (uint32_t i = threadIdx.x; i < dim; i += kOpsThreads) out[base + i] = __fdiv_rn(x[base + i], rms) * weight[i];
}

__global__ void __launch_bounds__(kOpsThreads) swiglu_kernel(float* hb, const float* hb2, size_t count) {
    grid_dep_launch_dependents();
    grid_dep_wait();
    const size_t i = static_cast<size_t>(blockIdx.x) * kOpsThreads + threadIdx.x;
    if (i < count) {
        const float a = hb[i];
        hb[i] = __fdiv_rn(a, 1.0f + expf(-a)) * hb2[i];
    }
}

__global__ void __launch_bounds__(1024) argmax_kernel(uint32_t* out, const float* logits, uint32_t vocab) {
    __shared__ float s_val[32];
    __shared__ uint32_t s_idx[32];
    grid_dep_launch_dependents();
    grid_dep_wait();
    const float* row = logits + static_cast<size_t>(blockIdx.x) * vocab;
    float best = -INFINITY;
    uint32_t best_i = 0xffffffffu;
    for (uint32_t i = threadIdx.x; i < vocab; i += 1024) {
        const float v = row[i];
        if (v > best || best_i == 0xffffffffu) {  // strictly greater: the first index of the maximum wins
            best = v;
            best_i = i;
        }
    }
    auto take = [&](float v, uint32_t i) {
        if (i != 0xffffffffu && (best_i == 0xffffffffu || v > best || (v == best && i < best_i))) {
            best = v;
            best_i = i;
        }
    };
#pragma unroll
    for (int off = 16; off; off >>= 1) {
        const float v = __shfl_xor_sync(0xffffffffu, best, off);
        const uint32_t i = __shfl_xor_sync(0xffffffffu, best_i, off);
        take(v, i);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) {
        s_val[warp] = best;
        s_idx[warp] = best_i;
    }
    __syncthreads();
    if (warp == 0) {
        best = s_val[lane];
        best_i = s_idx[lane];
#pragma unroll
        for (int off = 16; off; off >>= 1) {
            const float v = __shfl_xor_sync(0xffffffffu, best, off);
            const uint32_t i = __shfl_xor_sync(0xffffffffu, best_i, off);
            take(v, i);
        }
        if (lane == 0) out[blockIdx.x] = best_i;
    }
}

inline void count_launch() { g_launch_count.fetch_add(1, std::memory_order_relaxed); }

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int attn_embed_f16(float* x, const void* table, const uint32_t* tokens, uint32_t batch, uint32_t dim,
                              uint32_t vocab, uint32_t* status, void* stream) {
    if (!x || !table || !tokens || batch == 0 || dim == 0 || vocab == 0) return ATTN_ERR_INVALID_ARG;
    B200_CUDA_TRY(launch_dependent(embed_kernel, dim3(batch), dim3(kOpsThreads), 0, static_cast<cudaStream_t>(stream), x,
                                   static_cast<const __half*>(table), tokens, dim, vocab, status));
    count_launch();
    return ATTN_OK;
}

extern "C" int attn_embed_q8_0(float* x, const void* table, const uint32_t* tokens, uint32_t batch, uint32_t dim,
                               uint32_t vocab, uint32_t* status, void* stream) {
    if (!x || !table || !tokens || batch == 0 || dim == 0 || vocab == 0 || dim % 32 != 0) return ATTN_ERR_INVALID_ARG;
    B200_CUDA_TRY(launch_dependent(embed_q8_kernel, dim3(batch), dim3(kOpsThreads), 0, static_cast<cudaStream_t>(stream), x,
                                   static_cast<const uint8_t*>(table), tokens, dim, vocab, status));
    count_launch();
    return ATTN_OK;
}

extern "C" int attn_rmsnorm(float* out, const float* x, const float* weight, uint32_t batch, uint32_t dim, float eps,
                            void* stream) {
    if (!out || !x || !weight || batch == 0 || dim == 0) return ATTN_ERR_INVALID_ARG;
    B200_CUDA_TRY(launch_dependent(rmsnorm_kernel, dim3(batch), dim3(kOpsThreads), 0, static_cast<cudaStream_t>(stream), out, x,
                                   weight, dim, eps));
    count_launch();
    return ATTN_OK;
}

extern "C" int attn_swiglu(float* hb, const float* hb2, uint64_t count, void* stream) {
    if (!hb || !hb2 || count == 0) return ATTN_ERR_INVALID_ARG;
    const uint64_t blocks = (count + kOpsThreads - 1) / kOpsThreads;
    if (blocks > 0x7fffffffull) return ATTN_ERR_UNSUPPORTED;
    B200_CUDA_TRY(launch_dependent(swiglu_kernel, dim3(static_cast<uint32_t>(blocks)), dim3(kOpsThreads), 0,
                                   static_cast<cudaStream_t>(stream), hb, hb2, static_cast<size_t>(count)));
    count_launch();
    return ATTN_OK;
}

extern "C" int attn_argmax(uint32_t* out, const float* logits, uint32_t batch, uint32_t vocab, void* stream) {
    if (!out || !logits || batch == 0 || vocab == 0) return ATTN_ERR_INVALID_ARG;
    B200_CUDA_TRY(launch_dependent(argmax_kernel, dim3(batch), dim3(1024), 0, static_cast<cudaStream_t>(stream), out, logits, vocab));
    count_launch();
    return ATTN_OK;
}
