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
#include "gemv_mma_common.cuh"
#include "ptx_sm100.cuh"

namespace b200 {
namespace {

constexpr int kOpsThreads = 256;

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

// One CTA of 1024 threads per sequence; each thread keeps its (up to two) float4 of the row in registers, so the row
// is read once. Optionally the row is first completed with partial sums that a split-k GEMV left behind
// (x += part[0] + part[1] + ..., added in that order, the residual connection of src/model/block.cpp:219-222) and
// written back. Rows longer than 8192 or not a multiple of 4 take the plain two-pass form.
constexpr int kNormThreads = 1024;

struct NormParams {
    float* out;             // fp32 result, or null when out_split is given
    uint32_t* out_split;    // the result as prepared activations (ATTN_DTYPE_SPLIT16 words), or null
    const float* x;
    float* x_store;         // where the completed row goes (partials only); may be x
    const float* partials;  // [n_partials][batch][dim] or null
    const float* weight;
    uint64_t partial_stride;
    uint32_t n_partials, dim;
    float eps;
};

__global__ void __launch_bounds__(kNormThreads) rmsnorm_kernel(const __grid_constant__ NormParams p) {
    __shared__ float s_red[kNormThreads / 32];
    grid_dep_launch_dependents();
    grid_dep_wait();
    const size_t base = static_cast<size_t>(blockIdx.x) * p.dim;
    const uint32_t tid = threadIdx.x;
    const bool fast = (p.dim % 4 == 0) && p.dim <= 2 * 4 * kNormThreads;
    float4 v[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
    float4 wv[2] = {v[0], v[0]};  // the norm weights do not wait for the reduction: fetched with the row
    float ss = 0.f;
    auto row_value = [&](size_t i) {
        float r = p.x[i];
        for (uint32_t s = 0; s < p.n_partials; ++s) r += p.partials[s * p.partial_stride + i];
        return r;
    };
    if (fast) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const uint32_t i = (tid + j * kNormThreads) * 4;
            if (i < p.dim) {
                v[j] = *reinterpret_cast<const float4*>(p.x + base + i);
                wv[j] = *reinterpret_cast<const float4*>(p.weight + i);
                for (uint32_t s = 0; s < p.n_partials; ++s) {
                    const float4 a = *reinterpret_cast<const float4*>(p.partials + s * p.partial_stride + base + i);
                    v[j].x += a.x, v[j].y += a.y, v[j].z += a.z, v[j].w += a.w;
                }
                if (p.n_partials) *reinterpret_cast<float4*>(p.x_store + base + i) = v[j];
                ss = fmaf(v[j].x, v[j].x, ss);
                ss = fmaf(v[j].y, v[j].y, ss);
                ss = fmaf(v[j].z, v[j].z, ss);
                ss = fmaf(v[j].w, v[j].w, ss);
            }
        }
    } else {
        for (uint32_t i = tid; i < p.dim; i += kNormThreads) {
            const float r = row_value(base + i);
            ss = fmaf(r, r, ss);
        }
    }
    // block sum in a fixed order: lanes by shuffle, then the 32 warps' sums one after the other
#pragma unroll
    for (int off = 16; off; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if ((tid & 31) == 0) s_red[tid >> 5] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < kNormThreads / 32; ++w) total += s_red[w];
    const float rms = sqrtf(total / static_cast<float>(p.dim) + p.eps);
    if (fast) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const uint32_t i = (tid + j * kNormThreads) * 4;
            if (i < p.dim) {
                const float4 w = wv[j];
                float4 o;
                o.x = __fdiv_rn(v[j].x, rms) * w.x;
                o.y = __fdiv_rn(v[j].y, rms) * w.y;
                o.z = __fdiv_rn(v[j].z, rms) * w.z;
                o.w = __fdiv_rn(v[j].w, rms) * w.w;
                if (p.out_split) {
                    *reinterpret_cast<uint4*>(p.out_split + base + i) = gemv_mma::split_activations(o.x, o.y, o.z, o.w);
                } else {
                    *reinterpret_cast<float4*>(p.out + base + i) = o;
                }
            }
        }
    } else {
        for (uint32_t i = tid; i < p.dim; i += kNormThreads) {
            const float r = row_value(base + i);
            if (p.n_partials) p.x_store[base + i] = r;
            const float o = __fdiv_rn(r, rms) * p.weight[i];
            if (p.out_split) store_split16(p.out_split + base, i, o);
            else p.out[base + i] = o;
        }
    }
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

namespace {
int launch_rmsnorm(float* out, uint32_t* out_split, float* x, const float* partials, uint32_t n_partials,
                   uint64_t partial_stride, const float* weight, uint32_t batch, uint32_t dim, float eps, void* stream) {
    if ((!out && !out_split) || !x || !weight || batch == 0 || dim == 0 || (n_partials && !partials)) return ATTN_ERR_INVALID_ARG;
    if (n_partials && out == x) return ATTN_ERR_INVALID_ARG;  // the completed row and its norm are both kept
    if (out_split && dim % 4 != 0) return ATTN_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(out_split) | reinterpret_cast<uintptr_t>(x) |
         reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(partials)) & 15u)
        return ATTN_ERR_ALIGNMENT;
    if (n_partials && partial_stride % 4 != 0) return ATTN_ERR_ALIGNMENT;
    NormParams p{};
    p.out = out;
    p.out_split = out_split;
    p.x = x;
    p.x_store = x;
    p.partials = partials;
    p.weight = weight;
    p.partial_stride = partial_stride;
    p.n_partials = n_partials;
    p.dim = dim;
    p.eps = eps;
    B200_CUDA_TRY(launch_dependent(rmsnorm_kernel, dim3(batch), dim3(kNormThreads), 0, static_cast<cudaStream_t>(stream), p));
    count_launch();
    return ATTN_OK;
}
}  // namespace

extern "C" int attn_rmsnorm_residual(float* out, float* x, const float* partials, uint32_t n_partials,
                                     uint64_t partial_stride, const float* weight, uint32_t batch, uint32_t dim, float eps,
                                     void* stream) {
    return launch_rmsnorm(out, nullptr, x, partials, n_partials, partial_stride, weight, batch, dim, eps, stream);
}

extern "C" int attn_rmsnorm_residual_split(uint32_t* out_split, float* x, const float* partials, uint32_t n_partials,
                                           uint64_t partial_stride, const float* weight, uint32_t batch, uint32_t dim,
                                           float eps, void* stream) {
    return launch_rmsnorm(nullptr, out_split, x, partials, n_partials, partial_stride, weight, batch, dim, eps, stream);
}

extern "C" int attn_rmsnorm(float* out, const float* x, const float* weight, uint32_t batch, uint32_t dim, float eps,
                            void* stream) {
    return attn_rmsnorm_residual(out, const_cast<float*>(x), nullptr, 0, 0, weight, batch, dim, eps, stream);
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
