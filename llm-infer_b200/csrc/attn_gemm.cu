// Projection of many tokens at once (the prompt phase) on the 5th-generation tensor cores:
//
//     C[t][j] (+)= sum_i A[t][i] * W[j][i]        t < m tokens, j < n_out, i < k
//
// where the engine multiplies one token's activations by the same matrix per call (matmul() of
// include/kernels_cpu.hpp:69-80, once per prompt token from tools/infer.cpp:271-274; on the GPU the warp-per-row
// fused_gemv_clip of src/kernels.cu:117-136). W is the engine's fp16 [n_out][k] matrix (k fastest), C is fp32.
// A arrives as two fp16 matrices, the rounded value and the rounding residual (A_hi + A_lo carries ~22 bits of the
// fp32 activation): the tensor cores multiply 16-bit operands, and one rounded operand (2^-11) would be visible in
// the greedy token stream, which has to equal the CPU path's. Two MMAs per k-step therefore (A_hi W, A_lo W); a caller
// with weights that are not exact in fp16 (Q8_0: scale x int8) passes the weights' own residual in a second call
// with a_lo = NULL and accumulate = 1.
//
// Kernel: persistent CTAs (one per SM), tile 128 tokens x 256 outputs, k in steps of 64 (128-byte swizzled rows):
//   warp 0      TMA producer: A_hi, A_lo [128][64] and W [256][64] tiles into a 3-stage ring (one mbarrier per stage)
//   warp 1      one thread issues tcgen05.mma (M 128, N 256, K 16; both operands in shared memory, K-major) into
//               one of two 256-column accumulators in tensor memory; tcgen05.commit releases the stage / hands over
//               the accumulator
//   warps 2-5   epilogue: thread = token row = tensor-memory lane; 32 columns at a time, tcgen05.ld -> (C +) -> store,
//               while the MMA warp already fills the other accumulator with the next tile
// Tiles are dealt so that CTAs running together share the W tile (2 MB) and walk down the tokens.
// FLOPs per call (useful) = 2 m n_out k; tensor work is twice that with a_lo. Every wait is bounded.
#include "attn_internal.cuh"
#include "tcgen05_sm100.cuh"
#include "tma_tile.cuh"

namespace b200 {
namespace {

using namespace tc;

constexpr int GM = 128, GN = 256, GK = 64;
constexpr int kGemmStages = 3;
constexpr int kGemmThreads = 192;
constexpr uint32_t kATile = GM * GK * 2;   // 16 KB
constexpr uint32_t kWTile = GN * GK * 2;   // 32 KB
constexpr uint32_t kStage = 2 * kATile + kWTile;
constexpr uint32_t kGemmBars = kGemmStages * kStage;
constexpr uint32_t kGemmSmem = kGemmBars + 128 + 1024;

struct GemmParams {
    float* c;
    uint64_t ldc;
    uint32_t m, n_out, k;
    uint32_t has_lo;
    int32_t accumulate;
    uint32_t* status;
};

enum { G_FULL = 0, G_EMPTY = G_FULL + kGemmStages, G_ACC_FULL = G_EMPTY + kGemmStages, G_ACC_EMPTY = G_ACC_FULL + 2,
       G_BARS = G_ACC_EMPTY + 2 };

__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_f16_kernel(const __grid_constant__ CUtensorMap tm_a_hi, const __grid_constant__ CUtensorMap tm_a_lo,
                const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ GemmParams p) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;  // swizzled tiles want 1024-byte alignment
    unsigned char* smem = smem_raw + (base - raw);
    const uint32_t bars = base + kGemmBars;
    auto bar = [&](int i) { return bars + 8u * i; };
    volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + kGemmBars + G_BARS * 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t m_tiles = (p.m + GM - 1) / GM, n_tiles = (p.n_out + GN - 1) / GN;
    const uint32_t tiles = m_tiles * n_tiles, k_steps = p.k / GK;

    if (tid == 0) {
        for (int s = 0; s < kGemmStages; ++s) {
            mbar_init(bar(G_FULL + s), 1);
            mbar_init(bar(G_EMPTY + s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar(G_ACC_FULL + a), 1);
            mbar_init(bar(G_ACC_EMPTY + a), 4);  // one arrival per epilogue warp
        }
        mbar_init_fence();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)), 512);
        tmem_relinquish();
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = *tmem_ptr_smem;

    grid_dep_launch_dependents();
    grid_dep_wait();

    if (warp == 0) {
        if (lane == 0) {
            // =============================== TMA producer ===============================
            const uint32_t bytes = (p.has_lo ? 2 * kATile : kATile) + kWTile;
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
                const int m0 = static_cast<int>((t % m_tiles) * GM), n0 = static_cast<int>((t / m_tiles) * GN);
                for (uint32_t ks = 0; ks < k_steps; ++ks, ++it) {
                    const uint32_t s = it % kGemmStages;
                    if (it >= kGemmStages && !mbar_wait(bar(G_EMPTY + s), ((it / kGemmStages) - 1) & 1)) {
                        if (p.status) atomicOr(p.status, ATTN_STATUS_WAIT_TIMEOUT);
                        ok = false;
                        break;
                    }
                    const uint32_t dst = base + s * kStage;
                    mbar_arrive_expect_tx(bar(G_FULL + s), bytes);
                    tma_load_2d(dst, &tm_a_hi, bar(G_FULL + s), static_cast<int>(ks * GK), m0);
                    if (p.has_lo) tma_load_2d(dst + kATile, &tm_a_lo, bar(G_FULL + s), static_cast<int>(ks * GK), m0);
                    tma_load_2d(dst + 2 * kATile, &tm_w, bar(G_FULL + s), static_cast<int>(ks * GK), n0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // =============================== MMA issuer ===============================
            constexpr uint32_t idesc = instr_desc(0, 0, 0, GM, GN);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++local) {
                const uint32_t a = local & 1;
                if (local >= 2 && !mbar_wait(bar(G_ACC_EMPTY + a), ((local >> 1) - 1) & 1)) {
                    if (p.status) atomicOr(p.status, ATTN_STATUS_WAIT_TIMEOUT);
                    break;
                }
                fence_after();
                const uint32_t d_tmem = tmem_base + a * GN;
                for (uint32_t ks = 0; ks < k_steps; ++ks, ++it) {
                    const uint32_t s = it % kGemmStages;
                    if (!mbar_wait(bar(G_FULL + s), (it / kGemmStages) & 1)) {
                        if (p.status) atomicOr(p.status, ATTN_STATUS_WAIT_TIMEOUT);
                        ok = false;
                        break;
                    }
                    fence_after();
                    const uint32_t a_hi = base + s * kStage, a_lo = a_hi + kATile, w = a_hi + 2 * kATile;
#pragma unroll
                    for (int kk = 0; kk < GK / 16; ++kk) {
                        // K-major operands, 128-byte swizzle: 32 bytes per k-step of 16, 8-row groups 1024 bytes apart
                        const uint64_t wd = smem_desc(w + kk * 32, 16, 1024);
                        mma_ss(d_tmem, smem_desc(a_hi + kk * 32, 16, 1024), wd, idesc, (ks | kk) != 0);
                        if (p.has_lo) mma_ss(d_tmem, smem_desc(a_lo + kk * 32, 16, 1024), wd, idesc, 1);
                    }
                    commit(bar(G_EMPTY + s));  // the stage may be refilled once these MMAs have read it
                }
                if (ok) commit(bar(G_ACC_FULL + a));
            }
        }
    } else {
        // =============================== epilogue warps ===============================
        const uint32_t quarter = warp & 3;                      // the tensor-memory lanes this warp may read
        const uint32_t row_in_tile = quarter * 32 + lane;
        const uint32_t lane_addr = (quarter * 32) << 16;
        uint32_t local = 0;
        for (uint32_t t = blockIdx.x; t < tiles; t += gridDim.x, ++local) {
            const uint32_t a = local & 1;
            const uint32_t m0 = (t % m_tiles) * GM, n0 = (t / m_tiles) * GN;
            if (!mbar_wait(bar(G_ACC_FULL + a), (local >> 1) & 1)) {
                if (lane == 0 && p.status) atomicOr(p.status, ATTN_STATUS_WAIT_TIMEOUT);
                break;
            }
            fence_after();
            const uint32_t row = m0 + row_in_tile;
            float* crow = p.c + static_cast<size_t>(row) * p.ldc + n0;
#pragma unroll 1
            for (int c = 0; c < GN / 32; ++c) {
                float v[32];
                tmem_ld32(tmem_base + a * GN + lane_addr + c * 32, v);
                tmem_wait_ld();
                if (row < p.m && n0 + c * 32 < p.n_out) {   // n_out is a multiple of 32
                    float4* dst = reinterpret_cast<float4*>(crow + c * 32);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        float4 o = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                        if (p.accumulate) {
                            const float4 old = dst[i];
                            o.x += old.x, o.y += old.y, o.z += old.z, o.w += old.w;
                        }
                        dst[i] = o;
                    }
                }
            }
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(G_ACC_EMPTY + a));
        }
    }

    // ---- common exit: everybody meets, then the allocating warp releases tensor memory ----
    fence_before();
    __syncthreads();
    if (warp == 1) {
        fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// [rows][k] fp16 matrix, k fastest; box = 64 elements (128 bytes) x box_rows rows, 128-byte swizzle.
int make_k_major_map(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t k, uint32_t box_rows) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return ATTN_ERR_CUDA;
    const cuuint64_t dims[2] = {k, rows};
    const cuuint64_t strides[1] = {k * 2};
    const cuuint32_t box[2] = {GK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        g_last_cuda_error = static_cast<int>(r);
        return ATTN_ERR_CUDA;
    }
    return ATTN_OK;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int attn_gemm_f16(const AttnGemmArgs* a, void* stream_v) {
    if (!a || !a->c || !a->a_hi || !a->w || a->m == 0 || a->n_out == 0 || a->k == 0) return ATTN_ERR_INVALID_ARG;
    if (a->k % GK != 0 || a->n_out % 32 != 0) return ATTN_ERR_UNSUPPORTED;
    const uint64_t ldc = a->ldc ? a->ldc : a->n_out;
    if (ldc < a->n_out || ldc % 4 != 0) return ATTN_ERR_INVALID_ARG;
    if ((reinterpret_cast<uintptr_t>(a->c) | reinterpret_cast<uintptr_t>(a->a_hi) | reinterpret_cast<uintptr_t>(a->a_lo) |
         reinterpret_cast<uintptr_t>(a->w)) & 15u)
        return ATTN_ERR_ALIGNMENT;
    DeviceInfo dev{};
    int rc = current_device_info(&dev);
    if (rc != ATTN_OK) return rc;
    if (dev.cc_major != 10) return ATTN_ERR_DEVICE;
    CUtensorMap tm_hi, tm_lo, tm_w;
    if ((rc = make_k_major_map(&tm_hi, a->a_hi, a->m, a->k, GM)) != ATTN_OK) return rc;
    if ((rc = make_k_major_map(&tm_lo, a->a_lo ? a->a_lo : a->a_hi, a->m, a->k, GM)) != ATTN_OK) return rc;
    if ((rc = make_k_major_map(&tm_w, a->w, a->n_out, a->k, GN)) != ATTN_OK) return rc;
    GemmParams p{};
    p.c = a->c;
    p.ldc = ldc;
    p.m = a->m;
    p.n_out = a->n_out;
    p.k = a->k;
    p.has_lo = a->a_lo ? 1u : 0u;
    p.accumulate = a->accumulate;
    p.status = a->status;
    const uint32_t tiles = ((a->m + GM - 1) / GM) * ((a->n_out + GN - 1) / GN);
    const uint32_t grid = tiles < static_cast<uint32_t>(dev.sm_count) ? tiles : static_cast<uint32_t>(dev.sm_count);
    B200_CUDA_TRY(cudaFuncSetAttribute(gemm_f16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kGemmSmem)));
    B200_CUDA_TRY(launch_dependent(gemm_f16_kernel, dim3(grid), dim3(kGemmThreads), kGemmSmem,
                                   static_cast<cudaStream_t>(stream_v), tm_hi, tm_lo, tm_w, p));
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return ATTN_OK;
}
