// Rotary embedding of the current token's Q and K, fp16 insert of K and V into the KV cache, and the one-position
// re-rotation of the attention-sink rows: the step directly in front of attention, in one launch.
//
// Replaces, for a batch of sequences, what the engine does per token in src/model/block.cpp:140-155 (CPU) and as
// three graph nodes in src/model/block.cu:114-205 (rope_f2f for Q, rope_f2h for K straight into the cache,
// rope_h2h on the sink rows; kernels in src/kernels.cu:66-115,245-258), with V's fp32 -> fp16 store taken out of
// the projection kernel (src/model/block.cu:96-110). Conventions are the reference's: adjacent pairs (i, i+1),
// freq_i = 1 / powf(theta, i / rotary_dim), angle = pos * freq_i in fp32 (include/kernels_cpu.hpp:82-120),
// round-to-nearest-even fp16 stores (kernels_cpu.hpp:17), dimensions >= rotary_dim copied unrotated.
//
// The fp32 angle of a late position is sensitive to the last bit of freq_i, and the host's powf / cosf / sinf are not
// bit-identical to CUDA's. To stay within one fp16 ulp of the CPU result this kernel (i) takes the frequency
// table from the caller when given (computed with the host's powf, bit-identical to the CPU path) and otherwise
// evaluates it in double precision, and (ii) evaluates cos / sin of the fp32 angle in double precision and rounds
// once. That is head_dim / 2 double-precision evaluations per sequence and call, negligible next to the cache row
// writes. HBM traffic per call: reads Q, K, V once, writes Q, one K row and one V row per sequence (+ sink rows).
#include "attn_internal.cuh"
#include "ptx_sm100.cuh"

namespace b200 {
namespace {

struct RopeParams {
    void* q_out;
    const float* q;
    const float* k;
    const float* v;
    uint16_t* k_cache;
    uint16_t* v_cache;
    const float* inv_freq;  // optional [rotary_dim / 2]
    const uint32_t* pos;
    const uint32_t* kv_pos;
    uint64_t kv_row_stride, kv_batch_stride;
    uint32_t batch, n_heads, n_kv_heads, head_dim, rotary_dim, kv_sink;
    float theta;
    int32_t q_out_dtype;
    int32_t pos_early;
};

constexpr int kRopeThreads = 1024;

// grid = (batch); each CTA handles one sequence's token: table of cos/sin, then all pairs.
__global__ void __launch_bounds__(kRopeThreads) rope_kv_insert_kernel(const __grid_constant__ RopeParams p) {
    extern __shared__ float s_tab[];  // [2][rotary_dim/2] cos, sin at `pos`; then [2][rotary_dim/2] at position 1
    // The cos / sin table depends only on the token's position. When the caller states that the positions were in
    // place before the previous kernel of the stream was launched (pos_early), the table is computed while that kernel
    // (the Q/K/V projection) may still be running, and only q, k, v and the caches are read after the wait.
    grid_dep_launch_dependents();
    if (!p.pos_early) grid_dep_wait();
    const uint32_t b = blockIdx.x;
    const uint32_t half = p.rotary_dim / 2;
    const uint32_t pos = p.pos[b];
    const int tid = threadIdx.x;
    for (uint32_t i = tid; i < half; i += kRopeThreads) {
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
        const float deg1 = 1.0f * freq;
        s_tab[2 * half + i] = static_cast<float>(cos(static_cast<double>(deg1)));
        s_tab[3 * half + i] = static_cast<float>(sin(static_cast<double>(deg1)));
    }
    if (p.pos_early) grid_dep_wait();
    __syncthreads();

    const uint32_t D = p.head_dim, hp = D / 2;
    // ---- Q: [n_heads][D/2] pairs
    for (uint32_t idx = tid; idx < p.n_heads * hp; idx += kRopeThreads) {
        const uint32_t h = idx / hp, i = idx - h * hp;
        const size_t off = (static_cast<size_t>(b) * p.n_heads + h) * D + 2 * i;
        const float2 x = *reinterpret_cast<const float2*>(p.q + off);
        float y0 = x.x, y1 = x.y;
        if (i < half) {
            const float c = s_tab[i], s = s_tab[half + i];
            y0 = x.x * c - x.y * s;
            y1 = x.x * s + x.y * c;
        }
        if (p.q_out_dtype == ATTN_DTYPE_F32) {
            *reinterpret_cast<float2*>(reinterpret_cast<float*>(p.q_out) + off) = make_float2(y0, y1);
        } else if (p.q_out_dtype == ATTN_DTYPE_F16) {
            *reinterpret_cast<__half2*>(reinterpret_cast<__half*>(p.q_out) + off) = __floats2half2_rn(y0, y1);
        } else {
            *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(p.q_out) + off) = __floats2bfloat162_rn(y0, y1);
        }
    }
    // ---- K (rotated) and V (as is) of the current token -> fp16 cache row kv_pos
    const size_t row = static_cast<size_t>(b) * p.kv_batch_stride + static_cast<size_t>(p.kv_pos[b]) * p.kv_row_stride;
    for (uint32_t idx = tid; idx < p.n_kv_heads * hp; idx += kRopeThreads) {
        const uint32_t h = idx / hp, i = idx - h * hp;
        const size_t off = (static_cast<size_t>(b) * p.n_kv_heads + h) * D + 2 * i;
        const float2 x = *reinterpret_cast<const float2*>(p.k + off);
        float y0 = x.x, y1 = x.y;
        if (i < half) {
            const float c = s_tab[i], s = s_tab[half + i];
            y0 = x.x * c - x.y * s;
            y1 = x.x * s + x.y * c;
        }
        *reinterpret_cast<__half2*>(p.k_cache + row + h * D + 2 * i) = __floats2half2_rn(y0, y1);
        const float2 vv = *reinterpret_cast<const float2*>(p.v + off);
        *reinterpret_cast<__half2*>(p.v_cache + row + h * D + 2 * i) = __floats2half2_rn(vv.x, vv.y);
    }
    // ---- attention sinks: rows [0, kv_sink) of K move one position forward, in place on fp16 storage.
    // The reference inserts the new row first and rotates afterwards; the new row never is a sink row
    // (kv_pos >= kv_sink whenever kv_sink > 0, src/model/model.cpp:65-67), so the order does not matter here.
    for (uint32_t idx = tid; idx < p.kv_sink * p.n_kv_heads * half; idx += kRopeThreads) {
        const uint32_t i = idx % half;
        const uint32_t h = (idx / half) % p.n_kv_heads;
        const uint32_t s_row = idx / (half * p.n_kv_heads);
        __half2* ptr = reinterpret_cast<__half2*>(p.k_cache + static_cast<size_t>(b) * p.kv_batch_stride +
                                                  static_cast<size_t>(s_row) * p.kv_row_stride + h * D + 2 * i);
        const float2 x = __half22float2(*ptr);
        const float c = s_tab[2 * half + i], s = s_tab[3 * half + i];
        *ptr = __floats2half2_rn(x.x * c - x.y * s, x.x * s + x.y * c);
    }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int attn_rope_kv_insert(const AttnRopeInsertArgs* a, void* stream_v) {
    if (!a || !a->q_out || !a->q || !a->k || !a->v || !a->k_cache || !a->v_cache || !a->pos || !a->kv_pos)
        return ATTN_ERR_INVALID_ARG;
    if (a->batch == 0 || a->n_heads == 0 || a->n_kv_heads == 0 || a->head_dim == 0) return ATTN_ERR_INVALID_ARG;
    if (a->head_dim % 2 != 0 || a->rotary_dim % 2 != 0 || a->rotary_dim > a->head_dim) return ATTN_ERR_INVALID_ARG;
    if (a->q_out_dtype != ATTN_DTYPE_F32 && a->q_out_dtype != ATTN_DTYPE_F16 && a->q_out_dtype != ATTN_DTYPE_BF16)
        return ATTN_ERR_INVALID_ARG;
    if (a->batch > 1 && a->kv_batch_stride == 0) return ATTN_ERR_INVALID_ARG;
    const uint64_t row_stride = a->kv_row_stride ? a->kv_row_stride : static_cast<uint64_t>(a->n_kv_heads) * a->head_dim;
    if ((reinterpret_cast<uintptr_t>(a->q) | reinterpret_cast<uintptr_t>(a->k) | reinterpret_cast<uintptr_t>(a->v) |
         reinterpret_cast<uintptr_t>(a->q_out)) & 7u)
        return ATTN_ERR_ALIGNMENT;
    if ((reinterpret_cast<uintptr_t>(a->k_cache) | reinterpret_cast<uintptr_t>(a->v_cache)) & 3u || row_stride % 2 != 0 ||
        a->kv_batch_stride % 2 != 0)
        return ATTN_ERR_ALIGNMENT;
    RopeParams p{};
    p.q_out = a->q_out;
    p.q = a->q;
    p.k = a->k;
    p.v = a->v;
    p.k_cache = static_cast<uint16_t*>(a->k_cache);
    p.v_cache = static_cast<uint16_t*>(a->v_cache);
    p.inv_freq = a->inv_freq;
    p.pos = a->pos;
    p.kv_pos = a->kv_pos;
    p.kv_row_stride = row_stride;
    p.kv_batch_stride = a->kv_batch_stride;
    p.batch = a->batch;
    p.n_heads = a->n_heads;
    p.n_kv_heads = a->n_kv_heads;
    p.head_dim = a->head_dim;
    p.rotary_dim = a->rotary_dim ? a->rotary_dim : a->head_dim;
    p.kv_sink = a->kv_sink;
    p.theta = a->theta;
    p.q_out_dtype = a->q_out_dtype;
    const size_t smem = static_cast<size_t>(p.rotary_dim) * 2 * sizeof(float);
    p.pos_early = a->pos_early;
    B200_CUDA_TRY(launch_dependent(rope_kv_insert_kernel, dim3(a->batch), dim3(kRopeThreads), smem,
                                   static_cast<cudaStream_t>(stream_v), p));
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return ATTN_OK;
}
