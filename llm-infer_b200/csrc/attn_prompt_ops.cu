// The steps around the batched projection GEMM (attn_gemm_f16) when whole prompts are processed at once instead of
// one token per forward pass (the engine's prompt loop, tools/infer.cpp:271-274, calls Model::forward per token; the
// results per token are the same, src/model/model.cpp:60-76). Every kernel here works on rows = prompt tokens of all
// sequences, packed one after the other:
//   rmsnorm rows            -> activations as an fp16 value / fp16 residual pair of matrices (the GEMM's A operand)
//   fp32 rows               -> the same pair (attention output before the output projection)
//   stacked gate | up rows  -> silu(gate) * up as that pair (src/model/block.cpp:198-210)
//   Q8_0 weight rows        -> fp16 value / residual pair (scale x int8 has up to 18 significant bits)
//   rotary embedding of every token's q and k, fp16 insert of k and v into the token's cache row
//                              (src/model/block.cpp:140-148 per token)
//   row gather                 (the last token of every prompt continues into the classifier)
// HBM-bound elementwise passes, a few hundred MB per layer at 9 000 prompt tokens; no roofline is quoted for them.
#include <cuda_fp16.h>

#include "attn_internal.cuh"
#include "ptx_sm100.cuh"

namespace b200 {
namespace {

constexpr int kRowThreads = 256;

__device__ __forceinline__ void split_pair(float x, __half& hi, __half& lo) {
    x = fminf(fmaxf(x, -65504.f), 65504.f);
    hi = __float2half_rn(x);
    lo = __float2half_rn(x - __half2float(hi));
}

__device__ __forceinline__ void store_pair4(__half* hi, __half* lo, size_t idx, float a, float b, float c, float d) {
    __half h[4], l[4];
    split_pair(a, h[0], l[0]);
    split_pair(b, h[1], l[1]);
    split_pair(c, h[2], l[2]);
    split_pair(d, h[3], l[3]);
    *reinterpret_cast<uint2*>(hi + idx) = *reinterpret_cast<const uint2*>(h);
    *reinterpret_cast<uint2*>(lo + idx) = *reinterpret_cast<const uint2*>(l);
}

// One CTA per row: out = x / sqrt(mean(x^2) + eps) * weight (include/kernels_cpu.hpp:43-67), written as the pair.
__global__ void __launch_bounds__(kRowThreads) rmsnorm_pair_kernel(__half* hi, __half* lo, const float* x,
                                                                   const float* weight, uint32_t dim, float eps) {
    __shared__ float s_red[kRowThreads / 32];
    grid_dep_launch_dependents();
    grid_dep_wait();
    const size_t base = static_cast<size_t>(blockIdx.x) * dim;
    const uint32_t tid = threadIdx.x;
    float ss = 0.f;
    for (uint32_t i = tid * 4; i < dim; i += kRowThreads * 4) {
        const float4 v = *reinterpret_cast<const float4*>(x + base + i);
        ss = fmaf(v.x, v.x, ss);
        ss = fmaf(v.y, v.y, ss);
        ss = fmaf(v.z, v.z, ss);
        ss = fmaf(v.w, v.w, ss);
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if ((tid & 31) == 0) s_red[tid >> 5] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < kRowThreads / 32; ++w) total += s_red[w];
    const float rms = sqrtf(total / static_cast<float>(dim) + eps);
    for (uint32_t i = tid * 4; i < dim; i += kRowThreads * 4) {
        const float4 v = *reinterpret_cast<const float4*>(x + base + i);
        const float4 w = *reinterpret_cast<const float4*>(weight + i);
        store_pair4(hi, lo, base + i, __fdiv_rn(v.x, rms) * w.x, __fdiv_rn(v.y, rms) * w.y, __fdiv_rn(v.z, rms) * w.z,
                    __fdiv_rn(v.w, rms) * w.w);
    }
}

__global__ void __launch_bounds__(kRowThreads) split_pair_kernel(__half* hi, __half* lo, const float* x, size_t count4) {
    grid_dep_launch_dependents();
    grid_dep_wait();
    for (size_t i = static_cast<size_t>(blockIdx.x) * kRowThreads + threadIdx.x; i < count4;
         i += static_cast<size_t>(gridDim.x) * kRowThreads) {
        const float4 v = reinterpret_cast<const float4*>(x)[i];
        store_pair4(hi, lo, i * 4, v.x, v.y, v.z, v.w);
    }
}

// c: [rows][ldc] with the gate values in columns [0, hidden) and the up values in [hidden, 2 hidden).
__global__ void __launch_bounds__(kRowThreads) swiglu_pair_kernel(__half* hi, __half* lo, const float* c, uint32_t hidden,
                                                                  uint64_t ldc) {
    grid_dep_launch_dependents();
    grid_dep_wait();
    const float* row = c + static_cast<size_t>(blockIdx.x) * ldc;
    const size_t out = static_cast<size_t>(blockIdx.x) * hidden;
    for (uint32_t i = threadIdx.x * 4; i < hidden; i += kRowThreads * 4) {
        const float4 g = *reinterpret_cast<const float4*>(row + i);
        const float4 u = *reinterpret_cast<const float4*>(row + hidden + i);
        // silu(x) = x / (1 + expf(-x)), src/model/block.cpp:206-210
        store_pair4(hi, lo, out + i, __fdiv_rn(g.x, 1.0f + expf(-g.x)) * u.x, __fdiv_rn(g.y, 1.0f + expf(-g.y)) * u.y,
                    __fdiv_rn(g.z, 1.0f + expf(-g.z)) * u.z, __fdiv_rn(g.w, 1.0f + expf(-g.w)) * u.w);
    }
}

// Q8_0 rows (GGML blocks: fp16 scale + 32 signed bytes) -> value = fp32(scale) * q as the pair. A thread per block.
__global__ void __launch_bounds__(kRowThreads) dequant_q8_pair_kernel(__half* hi, __half* lo, const uint8_t* w,
                                                                      size_t n_blocks) {
    grid_dep_launch_dependents();
    grid_dep_wait();
    for (size_t b = static_cast<size_t>(blockIdx.x) * kRowThreads + threadIdx.x; b < n_blocks;
         b += static_cast<size_t>(gridDim.x) * kRowThreads) {
        const uint8_t* blk = w + b * 34;
        const float scale = __half2float(__ushort_as_half(static_cast<unsigned short>(blk[0] | (blk[1] << 8))));
        // the 32 values start two bytes into the block: 2-byte aligned loads
        const unsigned short* q16 = reinterpret_cast<const unsigned short*>(blk + 2);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const unsigned short a = q16[2 * i], c = q16[2 * i + 1];
            store_pair4(hi, lo, b * 32 + 4 * i, scale * static_cast<float>(static_cast<int8_t>(a & 0xff)),
                        scale * static_cast<float>(static_cast<int8_t>(a >> 8)),
                        scale * static_cast<float>(static_cast<int8_t>(c & 0xff)),
                        scale * static_cast<float>(static_cast<int8_t>(c >> 8)));
        }
    }
}

struct RopePromptParams {
    __half* q_out;          // [tokens][n_heads][head_dim]
    const float* qkv;       // [tokens][ld]: q, then k, then v of the token
    uint16_t* k_cache;
    uint16_t* v_cache;
    const float* inv_freq;  // optional [rotary_dim / 2]
    const uint32_t* token_seq;
    const uint32_t* token_pos;
    uint64_t ld, kv_row_stride, kv_batch_stride;
    uint32_t n_heads, n_kv_heads, head_dim, rotary_dim;
    float theta;
    float clip;  // > 0: q, k, v are clamped to [-clip, clip] first (src/model/block.cpp:130-138)
};

// One CTA per token. Conventions of include/kernels_cpu.hpp:82-120: adjacent pairs, freq_i = 1 / powf(theta, i / rot),
// angle = pos * freq_i in fp32; freq, cos and sin are evaluated in double precision and rounded once (see
// attn_rope.cu); fp16 stores round to nearest even.
__global__ void __launch_bounds__(kRowThreads) rope_prompt_kernel(const __grid_constant__ RopePromptParams p) {
    extern __shared__ float s_tab[];  // [2][rotary_dim / 2]
    grid_dep_launch_dependents();
    grid_dep_wait();
    const uint32_t t = blockIdx.x, tid = threadIdx.x;
    const uint32_t half = p.rotary_dim / 2;
    const uint32_t pos = p.token_pos[t], seq = p.token_seq[t];
    for (uint32_t i = tid; i < half; i += kRowThreads) {
        float freq;
        if (p.inv_freq) {
            freq = p.inv_freq[i];
        } else {
            const float e = static_cast<float>(2 * i) / static_cast<float>(p.rotary_dim);
            freq = 1.0f / static_cast<float>(pow(static_cast<double>(p.theta), static_cast<double>(e)));
        }
        const float deg = static_cast<float>(pos) * freq;
        s_tab[i] = static_cast<float>(cos(static_cast<double>(deg)));
        s_tab[half + i] = static_cast<float>(sin(static_cast<double>(deg)));
    }
    __syncthreads();
    const uint32_t D = p.head_dim, hp = D / 2;
    const float* row = p.qkv + static_cast<size_t>(t) * p.ld;
    const float lim = p.clip > 0.f ? p.clip : INFINITY;
    auto clamp2 = [&](float2 v) { return make_float2(fminf(fmaxf(v.x, -lim), lim), fminf(fmaxf(v.y, -lim), lim)); };
    const uint32_t q_dim = p.n_heads * D, kv_dim = p.n_kv_heads * D;
    for (uint32_t idx = tid; idx < p.n_heads * hp; idx += kRowThreads) {
        const uint32_t i = idx % hp;
        const float2 x = clamp2(*reinterpret_cast<const float2*>(row + 2 * idx));
        float y0 = x.x, y1 = x.y;
        if (i < half) {
            const float c = s_tab[i], s = s_tab[half + i];
            y0 = x.x * c - x.y * s;
            y1 = x.x * s + x.y * c;
        }
        *reinterpret_cast<__half2*>(p.q_out + static_cast<size_t>(t) * q_dim + 2 * idx) = __floats2half2_rn(y0, y1);
    }
    const size_t crow = static_cast<size_t>(seq) * p.kv_batch_stride + static_cast<size_t>(pos) * p.kv_row_stride;
    for (uint32_t idx = tid; idx < p.n_kv_heads * hp; idx += kRowThreads) {
        const uint32_t i = idx % hp;
        const float2 x = clamp2(*reinterpret_cast<const float2*>(row + q_dim + 2 * idx));
        float y0 = x.x, y1 = x.y;
        if (i < half) {
            const float c = s_tab[i], s = s_tab[half + i];
            y0 = x.x * c - x.y * s;
            y1 = x.x * s + x.y * c;
        }
        *reinterpret_cast<__half2*>(p.k_cache + crow + 2 * idx) = __floats2half2_rn(y0, y1);
        const float2 v = clamp2(*reinterpret_cast<const float2*>(row + q_dim + kv_dim + 2 * idx));
        *reinterpret_cast<__half2*>(p.v_cache + crow + 2 * idx) = __floats2half2_rn(v.x, v.y);
    }
}

__global__ void __launch_bounds__(kRowThreads) gather_rows_kernel(float* out, const float* x, const uint32_t* rows,
                                                                  uint32_t dim) {
    grid_dep_launch_dependents();
    grid_dep_wait();
    const float* src = x + static_cast<size_t>(rows[blockIdx.x]) * dim;
    float* dst = out + static_cast<size_t>(blockIdx.x) * dim;
    for (uint32_t i = threadIdx.x; i < dim; i += kRowThreads) dst[i] = src[i];
}

bool aligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
uint32_t stream_grid(size_t items) {
    const size_t blocks = (items + kRowThreads - 1) / kRowThreads;
    return static_cast<uint32_t>(blocks < 148 * 16 ? (blocks ? blocks : 1) : 148 * 16);
}
void count_launch() { g_launch_count.fetch_add(1, std::memory_order_relaxed); }

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int attn_rmsnorm_f16pair(void* hi, void* lo, const float* x, const float* weight, uint32_t rows, uint32_t dim, float eps,
                         void* stream) {
    if (!hi || !lo || !x || !weight || rows == 0 || dim == 0) return ATTN_ERR_INVALID_ARG;
    if (dim % 4 != 0) return ATTN_ERR_UNSUPPORTED;
    if (!aligned(hi, 8) || !aligned(lo, 8) || !aligned(x, 16) || !aligned(weight, 16)) return ATTN_ERR_ALIGNMENT;
    B200_CUDA_TRY(launch_dependent(rmsnorm_pair_kernel, dim3(rows), dim3(kRowThreads), 0, static_cast<cudaStream_t>(stream),
                                   static_cast<__half*>(hi), static_cast<__half*>(lo), x, weight, dim, eps));
    count_launch();
    return ATTN_OK;
}

int attn_split_f16pair(void* hi, void* lo, const float* x, uint64_t count, void* stream) {
    if (!hi || !lo || !x || count == 0) return ATTN_ERR_INVALID_ARG;
    if (count % 4 != 0) return ATTN_ERR_UNSUPPORTED;
    if (!aligned(hi, 8) || !aligned(lo, 8) || !aligned(x, 16)) return ATTN_ERR_ALIGNMENT;
    B200_CUDA_TRY(launch_dependent(split_pair_kernel, dim3(stream_grid(count / 4)), dim3(kRowThreads), 0,
                                   static_cast<cudaStream_t>(stream), static_cast<__half*>(hi), static_cast<__half*>(lo), x,
                                   static_cast<size_t>(count / 4)));
    count_launch();
    return ATTN_OK;
}

int attn_swiglu_f16pair(void* hi, void* lo, const float* gate_up, uint32_t rows, uint32_t hidden, uint64_t ld,
                        void* stream) {
    if (!hi || !lo || !gate_up || rows == 0 || hidden == 0) return ATTN_ERR_INVALID_ARG;
    if (ld == 0) ld = 2ull * hidden;
    if (hidden % 4 != 0 || ld % 4 != 0 || ld < 2ull * hidden) return ATTN_ERR_UNSUPPORTED;
    if (!aligned(hi, 8) || !aligned(lo, 8) || !aligned(gate_up, 16)) return ATTN_ERR_ALIGNMENT;
    B200_CUDA_TRY(launch_dependent(swiglu_pair_kernel, dim3(rows), dim3(kRowThreads), 0, static_cast<cudaStream_t>(stream),
                                   static_cast<__half*>(hi), static_cast<__half*>(lo), gate_up, hidden, ld));
    count_launch();
    return ATTN_OK;
}

int attn_dequant_q8_0_f16pair(void* hi, void* lo, const void* w, uint64_t rows, uint32_t n, void* stream) {
    if (!hi || !lo || !w || rows == 0 || n == 0) return ATTN_ERR_INVALID_ARG;
    if (n % 32 != 0) return ATTN_ERR_UNSUPPORTED;
    if (!aligned(hi, 8) || !aligned(lo, 8) || !aligned(w, 2)) return ATTN_ERR_ALIGNMENT;
    const size_t n_blocks = static_cast<size_t>(rows) * (n / 32);
    B200_CUDA_TRY(launch_dependent(dequant_q8_pair_kernel, dim3(stream_grid(n_blocks)), dim3(kRowThreads), 0,
                                   static_cast<cudaStream_t>(stream), static_cast<__half*>(hi), static_cast<__half*>(lo),
                                   static_cast<const uint8_t*>(w), n_blocks));
    count_launch();
    return ATTN_OK;
}

int attn_rope_prompt(const AttnRopePromptArgs* a, void* stream) {
    if (!a || !a->q_out || !a->qkv || !a->k_cache || !a->v_cache || !a->token_seq || !a->token_pos) return ATTN_ERR_INVALID_ARG;
    if (a->tokens == 0 || a->n_heads == 0 || a->n_kv_heads == 0 || a->head_dim == 0) return ATTN_ERR_INVALID_ARG;
    const uint32_t rot = a->rotary_dim ? a->rotary_dim : a->head_dim;
    if (a->head_dim % 2 != 0 || rot % 2 != 0 || rot > a->head_dim) return ATTN_ERR_INVALID_ARG;
    const uint64_t width = static_cast<uint64_t>(a->n_heads + 2 * a->n_kv_heads) * a->head_dim;
    const uint64_t ld = a->ld ? a->ld : width;
    const uint64_t row_stride = a->kv_row_stride ? a->kv_row_stride : static_cast<uint64_t>(a->n_kv_heads) * a->head_dim;
    if (ld < width || ld % 2 != 0 || row_stride % 2 != 0 || a->kv_batch_stride % 2 != 0) return ATTN_ERR_ALIGNMENT;
    if (!aligned(a->qkv, 8) || !aligned(a->q_out, 4) || !aligned(a->k_cache, 4) || !aligned(a->v_cache, 4))
        return ATTN_ERR_ALIGNMENT;
    RopePromptParams p{};
    p.q_out = static_cast<__half*>(a->q_out);
    p.qkv = a->qkv;
    p.k_cache = static_cast<uint16_t*>(a->k_cache);
    p.v_cache = static_cast<uint16_t*>(a->v_cache);
    p.inv_freq = a->inv_freq;
    p.token_seq = a->token_seq;
    p.token_pos = a->token_pos;
    p.ld = ld;
    p.kv_row_stride = row_stride;
    p.kv_batch_stride = a->kv_batch_stride;
    p.n_heads = a->n_heads;
    p.n_kv_heads = a->n_kv_heads;
    p.head_dim = a->head_dim;
    p.rotary_dim = rot;
    p.theta = a->theta;
    p.clip = a->qkv_clip;
    B200_CUDA_TRY(launch_dependent(rope_prompt_kernel, dim3(a->tokens), dim3(kRowThreads), static_cast<size_t>(rot) * 4,
                                   static_cast<cudaStream_t>(stream), p));
    count_launch();
    return ATTN_OK;
}

int attn_gather_rows(float* out, const float* x, const uint32_t* rows, uint32_t n_rows, uint32_t dim, void* stream) {
    if (!out || !x || !rows || n_rows == 0 || dim == 0) return ATTN_ERR_INVALID_ARG;
    B200_CUDA_TRY(launch_dependent(gather_rows_kernel, dim3(n_rows), dim3(kRowThreads), 0, static_cast<cudaStream_t>(stream),
                                   out, x, rows, dim));
    count_launch();
    return ATTN_OK;
}

}  // extern "C"
