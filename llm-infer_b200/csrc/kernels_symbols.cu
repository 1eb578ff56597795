// The engine's remaining kernel symbols (include/kernels.cuh:9-24) defined for sm_100a with exactly the declared
// signatures, so that the engine's graph-building host code (src/model/block.cu:25-205, src/model/model.cu:28-86)
// links against this library unchanged when its own src/kernels.cu is left out of the build:
//
//   copy_embedding_float / copy_embedding_half   kernels.cuh:9-10    (engine: src/kernels.cu:144-167)
//   rmsnorm                                      kernels.cuh:12      (src/kernels.cu:173-212)
//   fused_gemv_clip / fused_gemv_clip_f2h        kernels.cuh:14-17   (src/kernels.cu:117-136,229-239)
//   rope_f2f / rope_f2h / rope_h2h               kernels.cuh:19-24   (src/kernels.cu:66-115,245-258)
//
// The engine fixes each node's grid and block when the node is first added (include/model/device.hpp:185-217) and
// its call sites keep their own geometry (128-thread blocks, one warp per GEMV output, one thread per rotary pair,
// one CTA for the norm). Every kernel here is therefore written over a grid-stride loop: it is correct under the
// engine's geometry and under any other one-dimensional geometry, and kernels_b200_launch_dims() names the geometry
// that suits a B200 for callers that are free to choose.
//
// Numerics follow the CPU path, the engine's only complete forward pass: the clamp is two-sided
// (src/model/block.cpp:130-138; the engine's own GPU epilogue clips only from above, src/kernels.cu:218-227), the norm
// divides before it multiplies (include/kernels_cpu.hpp:43-67), and the rotary angle is the fp32 product pos * freq
// with freq, cos and sin evaluated in double precision and rounded once (the host's powf/cosf/sinf are correctly
// rounded in practice, CUDA's single-precision ones are not, and at late positions one ulp of freq moves the angle
// visibly; include/kernels_cpu.hpp:82-120).
#include <optional>

#include "../../include/kernels_b200.cuh"
#include "attn_internal.cuh"

namespace b200 {
namespace symbols {

__device__ __forceinline__ uint32_t global_thread() { return blockIdx.x * blockDim.x + threadIdx.x; }
__device__ __forceinline__ uint32_t global_threads() { return gridDim.x * blockDim.x; }

__device__ __forceinline__ float clamp_both(float x, const std::optional<float>& clip) {
    if (clip.has_value()) {
        const float c = clip.value();
        x = fminf(fmaxf(x, -c), c);
    }
    return x;
}

__device__ __forceinline__ uint4 ld_stream_16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ float dot8(const uint4& w, const float4& x0, const float4& x1, float acc) {
    const __half2* h = reinterpret_cast<const __half2*>(&w);
    const float2 a = __half22float2(h[0]), b = __half22float2(h[1]), c = __half22float2(h[2]), d = __half22float2(h[3]);
    acc = fmaf(a.x, x0.x, acc);
    acc = fmaf(a.y, x0.y, acc);
    acc = fmaf(b.x, x0.z, acc);
    acc = fmaf(b.y, x0.w, acc);
    acc = fmaf(c.x, x1.x, acc);
    acc = fmaf(c.y, x1.y, acc);
    acc = fmaf(d.x, x1.z, acc);
    acc = fmaf(d.y, x1.w, acc);
    return acc;
}

// out[j] = clamp(sum_i x[i] * w[j*n + i]): a warp per output row, rows dealt round-robin to however many warps the
// launch has. A lane streams 16 bytes (8 weights) per load, four loads in flight, weights bypassing L1; the
// activations (n floats, shared by every row) come through L1/L2.
template <typename Out>
__device__ __forceinline__ void gemv_rows(Out* out, const float* x, const half* w, uint32_t n, uint32_t d,
                                          const std::optional<float>& clip) {
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warp = global_thread() >> 5;
    const uint32_t n_warps = global_threads() >> 5;
    const bool vec = (n % 8 == 0) && ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x)) & 15u) == 0;
    for (uint32_t j = warp; j < d; j += n_warps) {
        const half* row = w + static_cast<size_t>(j) * n;
        float acc = 0.f;
        if (vec) {
            const uint32_t chunks = n / 8;  // 16-byte chunks of the row
            uint32_t c = lane;
            for (; c + 96 < chunks; c += 128) {
                uint4 wv[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) wv[u] = ld_stream_16(row + static_cast<size_t>(c + 32 * u) * 8);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float4* xp = reinterpret_cast<const float4*>(x + static_cast<size_t>(c + 32 * u) * 8);
                    acc = dot8(wv[u], xp[0], xp[1], acc);
                }
            }
            for (; c < chunks; c += 32) {
                const uint4 wv = ld_stream_16(row + static_cast<size_t>(c) * 8);
                const float4* xp = reinterpret_cast<const float4*>(x + static_cast<size_t>(c) * 8);
                acc = dot8(wv, xp[0], xp[1], acc);
            }
        } else {
            for (uint32_t i = lane; i < n; i += 32) acc = fmaf(__half2float(row[i]), x[i], acc);
        }
#pragma unroll
        for (int off = 16; off; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
        if (lane == 0) {
            acc = clamp_both(acc, clip);
            if constexpr (sizeof(Out) == 4) out[j] = acc;
            else out[j] = __float2half_rn(acc);
        }
    }
}

// cos / sin of the rotary angle of pair index i (elements i, i + 1 of a head) at position pos.
__device__ __forceinline__ float2 rotary_cos_sin(uint32_t i, uint32_t pos, float theta, uint32_t rotary_dim) {
    const float e = static_cast<float>(i) / static_cast<float>(rotary_dim);
    const float freq = 1.0f / static_cast<float>(pow(static_cast<double>(theta), static_cast<double>(e)));
    const float deg = static_cast<float>(pos) * freq;
    return make_float2(static_cast<float>(cos(static_cast<double>(deg))), static_cast<float>(sin(static_cast<double>(deg))));
}

template <typename Out, typename In>
__device__ __forceinline__ void rope_pairs(Out* out, const In* x, uint32_t n_heads, uint32_t head_dim, uint32_t pos,
                                           float theta, uint32_t rotary_dim) {
    const uint32_t pairs = n_heads * head_dim / 2;
    for (uint32_t t = global_thread(); t < pairs; t += global_threads()) {
        const uint32_t inner = (t * 2) % head_dim;
        float2 a;
        if constexpr (sizeof(In) == 4) a = reinterpret_cast<const float2*>(x)[t];
        else a = __half22float2(reinterpret_cast<const __half2*>(x)[t]);
        if (inner + 1 < rotary_dim) {
            const float2 cs = rotary_cos_sin(inner, pos, theta, rotary_dim);
            a = make_float2(a.x * cs.x - a.y * cs.y, a.x * cs.y + a.y * cs.x);
        }
        if constexpr (sizeof(Out) == 4) reinterpret_cast<float2*>(out)[t] = a;
        else reinterpret_cast<__half2*>(out)[t] = __floats2half2_rn(a.x, a.y);
    }
}

}  // namespace symbols
}  // namespace b200

using namespace b200::symbols;

__global__ void copy_embedding_float(float* out, const float* token_embedding_table, uint32_t token, uint32_t dim) {
    const float* src = token_embedding_table + static_cast<size_t>(token) * dim;
    for (uint32_t i = global_thread(); i < dim; i += global_threads()) out[i] = src[i];
}

__global__ void copy_embedding_half(float* out, const half* token_embedding_table, uint32_t token, uint32_t dim) {
    const half* src = token_embedding_table + static_cast<size_t>(token) * dim;
    if (dim % 2 == 0 && (reinterpret_cast<uintptr_t>(src) & 3u) == 0 && (reinterpret_cast<uintptr_t>(out) & 7u) == 0) {
        for (uint32_t i = global_thread(); i < dim / 2; i += global_threads())
            reinterpret_cast<float2*>(out)[i] = __half22float2(reinterpret_cast<const __half2*>(src)[i]);
    } else {
        for (uint32_t i = global_thread(); i < dim; i += global_threads()) out[i] = __half2float(src[i]);
    }
}

// One CTA normalises the row (the engine launches exactly one, src/model/block.cu:28-34); further CTAs of a larger
// grid have nothing to do. Any block size that is a multiple of 32 up to 1024 works.
__global__ void rmsnorm(float* out, const float* x, const float* weight, uint32_t size, float eps) {
    if (blockIdx.x != 0) return;
    __shared__ float s_red[32];
    const uint32_t tid = threadIdx.x, nthr = blockDim.x;
    float ss = 0.f;
    for (uint32_t i = tid; i < size; i += nthr) {
        const float v = x[i];
        ss = fmaf(v, v, ss);
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if ((tid & 31) == 0) s_red[tid >> 5] = ss;
    __syncthreads();
    float total = 0.f;
    for (uint32_t w = 0; w < (nthr + 31) / 32; ++w) total += s_red[w];
    const float rms = sqrtf(total / static_cast<float>(size) + eps);
    for (uint32_t i = tid; i < size; i += nthr) out[i] = __fdiv_rn(x[i], rms) * weight[i];
}

__global__ void fused_gemv_clip(float* out, const float* x, const half* w, uint32_t n, uint32_t d,
                                std::optional<float> clip) {
    gemv_rows<float>(out, x, w, n, d, clip);
}

__global__ void fused_gemv_clip_f2h(half* out, const float* x, const half* w, uint32_t n, uint32_t d,
                                    std::optional<float> clip) {
    gemv_rows<half>(out, x, w, n, d, clip);
}

__global__ void rope_f2f(float* out, const float* x, uint32_t n_heads, uint32_t head_dim, uint32_t pos, float theta,
                         uint32_t rotary_dim) {
    rope_pairs<float, float>(out, x, n_heads, head_dim, pos, theta, rotary_dim);
}

__global__ void rope_f2h(half* out, const float* x, uint32_t n_heads, uint32_t head_dim, uint32_t pos, float theta,
                         uint32_t rotary_dim) {
    rope_pairs<half, float>(out, x, n_heads, head_dim, pos, theta, rotary_dim);
}

__global__ void rope_h2h(half* out, const half* x, uint32_t n_heads, uint32_t head_dim, uint32_t pos, float theta,
                         uint32_t rotary_dim) {
    rope_pairs<half, half>(out, x, n_heads, head_dim, pos, theta, rotary_dim);
}

// ---------------------------------------------------------------------------------------------------------------
// Host helpers: geometry, plain launches and graph nodes for callers (and tests) that reach the kernels through the
// C ABI instead of linking the symbols.
// ---------------------------------------------------------------------------------------------------------------
using namespace b200;

namespace {

struct OptionalFloat {  // what the kernels take by value; built here so that callers need no C++ type
    std::optional<float> v;
    OptionalFloat(int has, float x) : v(has ? std::optional<float>(x) : std::nullopt) {}
};

const void* symbol_function(int which) {
    switch (which) {
        case KERNELS_B200_COPY_EMBEDDING_FLOAT: return reinterpret_cast<const void*>(copy_embedding_float);
        case KERNELS_B200_COPY_EMBEDDING_HALF: return reinterpret_cast<const void*>(copy_embedding_half);
        case KERNELS_B200_RMSNORM: return reinterpret_cast<const void*>(rmsnorm);
        case KERNELS_B200_FUSED_GEMV_CLIP: return reinterpret_cast<const void*>(fused_gemv_clip);
        case KERNELS_B200_FUSED_GEMV_CLIP_F2H: return reinterpret_cast<const void*>(fused_gemv_clip_f2h);
        case KERNELS_B200_ROPE_F2F: return reinterpret_cast<const void*>(rope_f2f);
        case KERNELS_B200_ROPE_F2H: return reinterpret_cast<const void*>(rope_f2h);
        case KERNELS_B200_ROPE_H2H: return reinterpret_cast<const void*>(rope_h2h);
        default: return nullptr;
    }
}

int run(int which, void** argv, uint32_t grid, uint32_t block, void* graph, void* node_out, void* stream) {
    const void* fn = symbol_function(which);
    if (!fn || grid == 0 || block == 0 || block > 1024) return ATTN_ERR_INVALID_ARG;
    if (graph) {
        if (!node_out) return ATTN_ERR_INVALID_ARG;
        cudaKernelNodeParams np;
        memset(&np, 0, sizeof(np));
        np.func = const_cast<void*>(fn);
        np.gridDim = dim3(grid);
        np.blockDim = dim3(block);
        np.sharedMemBytes = 0;
        np.kernelParams = argv;
        B200_CUDA_TRY(cudaGraphAddKernelNode(static_cast<cudaGraphNode_t*>(node_out), static_cast<cudaGraph_t>(graph),
                                             nullptr, 0, &np));
        return ATTN_OK;
    }
    B200_CUDA_TRY(cudaLaunchKernel(fn, dim3(grid), dim3(block), argv, 0, static_cast<cudaStream_t>(stream)));
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return ATTN_OK;
}

}  // namespace

extern "C" {

const void* kernels_b200_function(int which) { return symbol_function(which); }

int kernels_b200_launch_dims(int which, uint32_t work, uint32_t* grid, uint32_t* block) {
    DeviceInfo dev{};
    int rc = current_device_info(&dev);
    if (rc != ATTN_OK) return rc;
    uint32_t g = 1, b = 128;
    switch (which) {
        case KERNELS_B200_RMSNORM:
            g = 1;
            b = 1024;
            break;
        case KERNELS_B200_FUSED_GEMV_CLIP:
        case KERNELS_B200_FUSED_GEMV_CLIP_F2H: {
            // persistent: eight 8-warp CTAs per SM share the rows (work = d), never more warps than rows
            b = 256;
            const uint32_t want = static_cast<uint32_t>(dev.sm_count) * 8;
            const uint32_t need = (work + 7) / 8;
            g = need < want ? (need ? need : 1) : want;
            break;
        }
        case KERNELS_B200_COPY_EMBEDDING_FLOAT:
        case KERNELS_B200_COPY_EMBEDDING_HALF:
        case KERNELS_B200_ROPE_F2F:
        case KERNELS_B200_ROPE_F2H:
        case KERNELS_B200_ROPE_H2H: {
            // work = elements; a thread per pair
            b = 128;
            const uint32_t pairs = (work + 1) / 2;
            g = (pairs + b - 1) / b;
            if (g == 0) g = 1;
            break;
        }
        default: return ATTN_ERR_INVALID_ARG;
    }
    if (grid) *grid = g;
    if (block) *block = b;
    return ATTN_OK;
}

int kernels_b200_copy_embedding(int half_table, float* out, const void* table, uint32_t token, uint32_t dim,
                                uint32_t grid, uint32_t block, void* graph, void* node_out, void* stream) {
    void* argv[4] = {&out, &table, &token, &dim};
    return run(half_table ? KERNELS_B200_COPY_EMBEDDING_HALF : KERNELS_B200_COPY_EMBEDDING_FLOAT, argv, grid, block,
               graph, node_out, stream);
}

int kernels_b200_rmsnorm(float* out, const float* x, const float* weight, uint32_t size, float eps, uint32_t grid,
                         uint32_t block, void* graph, void* node_out, void* stream) {
    if (block % 32 != 0) return ATTN_ERR_INVALID_ARG;
    void* argv[5] = {&out, &x, &weight, &size, &eps};
    return run(KERNELS_B200_RMSNORM, argv, grid, block, graph, node_out, stream);
}

int kernels_b200_fused_gemv_clip(int out_half, void* out, const float* x, const void* w, uint32_t n, uint32_t d,
                                 int has_clip, float clip, uint32_t grid, uint32_t block, void* graph, void* node_out,
                                 void* stream) {
    if (block % 32 != 0) return ATTN_ERR_INVALID_ARG;
    OptionalFloat c(has_clip, clip);
    void* argv[6] = {&out, &x, &w, &n, &d, &c.v};
    return run(out_half ? KERNELS_B200_FUSED_GEMV_CLIP_F2H : KERNELS_B200_FUSED_GEMV_CLIP, argv, grid, block, graph,
               node_out, stream);
}

int kernels_b200_rope(int which, void* out, const void* x, uint32_t n_heads, uint32_t head_dim, uint32_t pos,
                      float theta, uint32_t rotary_dim, uint32_t grid, uint32_t block, void* graph, void* node_out,
                      void* stream) {
    if (which != KERNELS_B200_ROPE_F2F && which != KERNELS_B200_ROPE_F2H && which != KERNELS_B200_ROPE_H2H)
        return ATTN_ERR_INVALID_ARG;
    if (head_dim % 2 != 0) return ATTN_ERR_INVALID_ARG;
    void* argv[7] = {&out, &x, &n_heads, &head_dim, &pos, &theta, &rotary_dim};
    return run(which, argv, grid, block, graph, node_out, stream);
}

}  // extern "C"
