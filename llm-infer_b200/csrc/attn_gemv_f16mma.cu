// Weight GEMV over fp16 weights on the tensor cores, for batches: out[b][j] = clamp(sum_i x[b][i] * W[j][i]) with W
// [d][n] fp16 (n fastest) and fp32 activations of 1..8 sequences. It is the formulation of the Q8_0 kernel next to it
// applied to the engine's own weight type (matmul() of include/kernels_cpu.hpp:69-80, clamp of
// src/model/block.cpp:130-138): the streaming kernel of attn_gemv.cu multiplies every weight by every sequence's
// activation on the CUDA cores and reads those activations from shared memory once per weight (batch 8: 1.5 TB/s),
// whereas here a batch of up to 8 sequences is the N dimension of one m16n8k16 MMA and costs nothing extra.
//
// One persistent CTA per SM, 8 warps. A CTA owns groups of 16 consecutive rows; its warps split the inner dimension
// in chunks of 64 elements. Every warp runs its own ring of shared-memory stages, each filled by one TMA tile load
// (16 rows x 128 bytes, 128-byte swizzle) and refilled by the warp as soon as it has consumed it. A fragments come
// straight from the swizzled tile with ldmatrix; B = the activations as fp16 value + fp16 residual (two MMAs per
// k-step, ~ 22 significant bits; |x| is clamped to the fp16 range), fp32 accumulation in the MMA over the whole inner
// dimension. The eight warps' partial sums of a row group are added in a fixed order. Measured ceiling ~ 3.8 TB/s
// whatever the batch: the TMA engine delivers the 128-byte rows of a swizzled tile at ~ 0.1 row per clock and SM
// (272-byte rows of the Q8_0 tiles: ~ 4.9 TB/s), so one sequence with a plain output stays on the streaming kernel. Row segments, the SwiGLU
// epilogue over stacked gate / up rows, in-kernel slices of the inner dimension and k_split work as in the Q8_0 kernel.
//
// Algorithmic bytes per call = rows * n * 2 + batch * (n*4 + d*sizeof(out)).
#include <cuda.h>
#include <cuda_fp16.h>

#include "attn_internal.cuh"
#include "ptx_sm100.cuh"

namespace b200 {
namespace {

constexpr int kQ8Warps = 8;  // warps per CTA
constexpr int kQ8Threads = kQ8Warps * 32;
constexpr uint32_t kChunkElems = 64;                        // elements of one row per stage: one 128-byte swizzle row
constexpr uint32_t kRows = 16;                              // rows of a group = M of the MMA
constexpr uint32_t kStageBytes = kRows * kChunkElems * 2;   // 2048: one swizzle-128B tile of 16 rows
constexpr uint32_t kMaxStages = 6;                          // barrier slots per warp

struct MmaParams {
    void* out0;               // rows [0, seg_end0)
    void* out1;               // rows [seg_end0, seg_end1)
    void* out2;               // rows [seg_end1, d)
    uint64_t out_stride0, out_stride1, out_stride2;  // elements between sequences of each output
    const float* x;
    uint32_t* status;
    uint64_t x_batch_stride;  // elements between sequences of x
    uint32_t seg_end0, seg_end1;
    uint32_t slice_chunks;    // 64-element chunks of the inner dimension staged at a time
    uint32_t n_slices;        // slice_chunks * n_slices = chunks per row
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
};

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Four 8x8 fp16 matrices from shared memory, one row address per lane: the A fragment of one k-step.
__device__ __forceinline__ void ldmatrix_a(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

// Tile load through the TMA engine: 16 rows x 128 bytes of W in one request (rows beyond d read as zeros).
__device__ __forceinline__ void tma_load_rows(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y,
                                              uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "l"(policy)
        : "memory");
}

__global__ void __launch_bounds__(kQ8Threads, 1) gemv_f16_mma_kernel(const __grid_constant__ CUtensorMap tm_w,
                                                                     const __grid_constant__ MmaParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);  // swizzled tiles want 1024-byte alignment
    // layout: [ring: warps x stages x kStageBytes][red: 2 x 2 x warps x 128 floats][acc: acc_groups x 2 x 128 floats]
    //         [bars: warps x kMaxStages][x fragments]
    const uint32_t ring_bytes = kQ8Warps * p.stages * kStageBytes;
    float* s_red = reinterpret_cast<float*>(smem + ring_bytes);
    float* s_acc = s_red + 2 * 2 * kQ8Warps * 128;
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_acc + p.acc_groups * 2 * 128);
    uint32_t* s_x = reinterpret_cast<uint32_t*>(s_bar + kQ8Warps * kMaxStages);

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t groups = (p.d + kRows - 1) / kRows;
    const uint32_t parts = p.swiglu ? 2u : 1u;  // row groups of W per output row group (gate, up)
    // chunks of one slice of one row group that this warp owns: warp, warp + 8, ...
    const uint32_t cpw = (p.slice_chunks > warp) ? (p.slice_chunks - warp + kQ8Warps - 1) / kQ8Warps : 0;
    // split-k: the grid is k_split sets of CTAs; set s handles slice s of every row group it owns
    const uint32_t ctas = gridDim.x / p.k_split, cta = blockIdx.x % ctas;
    const uint32_t slice_begin = p.k_split > 1 ? blockIdx.x / ctas : 0;
    const uint32_t slice_end = p.k_split > 1 ? slice_begin + 1 : p.n_slices;
    const uint32_t my_groups = (groups > cta) ? (groups - cta + ctas - 1) / ctas : 0;
    const uint32_t total = (slice_end - slice_begin) * my_groups * parts * cpw;  // items: slice > group > part > chunk

    const uint32_t ring0 = smem_u32(smem) + warp * p.stages * kStageBytes;
    const uint32_t bar0 = smem_u32(s_bar) + warp * kMaxStages * 8;
    const uint64_t policy = l2_policy_evict_first();

    if (lane == 0) {
        for (uint32_t s = 0; s < p.stages; ++s) mbar_init(bar0 + 8 * s, 1);
        mbar_init_fence();
    }
    __syncwarp();

    auto issue = [&](uint32_t item) {
        const uint32_t ci = item % cpw, q = item / cpw;
        const uint32_t part = q % parts, q2 = q / parts;
        const uint32_t gi = q2 % my_groups, slice = slice_begin + q2 / my_groups;
        const uint32_t rg = cta + gi * ctas;
        const uint32_t chunk = slice * p.slice_chunks + warp + ci * kQ8Warps;
        const uint32_t stage = item % p.stages;
        const uint32_t bar = bar0 + 8 * stage;
        if (lane == 0) {
            mbar_arrive_expect_tx(bar, kStageBytes);
            // x = first element of the chunk (128 bytes: a multiple of 16), y = first row of the group (rows past
            // the tensor read as zeros)
            tma_load_rows(ring0 + stage * kStageBytes, &tm_w, bar, static_cast<int>(chunk * kChunkElems),
                          static_cast<int>(part * p.d + rg * kRows), policy);
        }
    };
    // The weights do not depend on the activations (no kernel writes them): start streaming them at once, let the next
    // kernel of the stream be scheduled, and only then wait for the previous kernel, whose output x (and out) are.
    for (uint32_t i = 0; i < p.stages && i < total; ++i) issue(i);
    grid_dep_launch_dependents();
    grid_dep_wait();

    const bool has_col = g < p.batch;  // lanes of the other columns feed zeros
    const uint32_t* my_x = s_x + (has_col ? g : 0) * p.x_col_pitch + t * 4;
    // ldmatrix row address of this lane inside a swizzled tile: matrix m = lane / 8 holds rows 8 (m & 1) .. +8 and the
    // 16-byte chunk 2 kk + (m >> 1) of k-step kk; the TMA stored chunk j of row r at r * 128 + ((j ^ (r & 7)) << 4)
    const uint32_t lm_row = (lane & 7) + ((lane >> 3) & 1) * 8;
    const uint32_t lm_hi = lane >> 4;
    bool timed_out = false;
    uint32_t item = 0, round = 0;
    for (uint32_t slice = slice_begin; slice < slice_end; ++slice) {
        // Activations of this slice as B fragments: for sequence c, k-step ks (16 elements), quarter t: four 32-bit
        // words {hi(x0,x1), hi(x8,x9), lo(x0,x1), lo(x8,x9)} with x0 = x[16 ks + 2 t]. Every warp has passed the
        // previous slice's last block-wide barrier, so nobody still reads the old fragments.
        const float* xs = p.x + static_cast<size_t>(slice) * p.slice_chunks * kChunkElems;
        const uint32_t per_seq = p.slice_chunks * (kChunkElems / 16) * 4;  // (k-step, quarter) pairs per sequence
        for (uint32_t i = tid; i < p.batch * per_seq; i += kQ8Threads) {
            const uint32_t c = i / per_seq, r = i - c * per_seq;
            const uint32_t ks = r >> 2, tt = r & 3;
            const float* src = xs + c * p.x_batch_stride + 16 * ks + 2 * tt;
            float2 a = *reinterpret_cast<const float2*>(src), b = *reinterpret_cast<const float2*>(src + 8);
            a.x = fminf(fmaxf(a.x, -65504.f), 65504.f);
            a.y = fminf(fmaxf(a.y, -65504.f), 65504.f);
            b.x = fminf(fmaxf(b.x, -65504.f), 65504.f);
            b.y = fminf(fmaxf(b.y, -65504.f), 65504.f);
            const __half2 ha = __floats2half2_rn(a.x, a.y), hb = __floats2half2_rn(b.x, b.y);
            const float2 fa = __half22float2(ha), fb = __half22float2(hb);
            const __half2 la = __floats2half2_rn(a.x - fa.x, a.y - fa.y), lb = __floats2half2_rn(b.x - fb.x, b.y - fb.y);
            uint4 o;
            o.x = *reinterpret_cast<const uint32_t*>(&ha);
            o.y = *reinterpret_cast<const uint32_t*>(&hb);
            o.z = *reinterpret_cast<const uint32_t*>(&la);
            o.w = *reinterpret_cast<const uint32_t*>(&lb);
            *reinterpret_cast<uint4*>(s_x + c * p.x_col_pitch + r * 4) = o;
        }
        __syncthreads();

        for (uint32_t gi = 0; gi < my_groups; ++gi, ++round) {
            const uint32_t rg = cta + gi * ctas;
            float* red = s_red + (round & 1) * 2 * kQ8Warps * 128;
            for (uint32_t part = 0; part < parts; ++part) {
                float tot[4] = {0.f, 0.f, 0.f, 0.f};
                for (uint32_t ci = 0; ci < cpw; ++ci, ++item) {
                    const uint32_t stage = item % p.stages;
                    if (!mbar_wait(bar0 + 8 * stage, (item / p.stages) & 1)) timed_out = true;
                    const uint32_t tile = ring0 + stage * kStageBytes + lm_row * 128;
                    const uint32_t* xb = my_x + (warp + ci * kQ8Warps) * (kChunkElems / 16) * 16;
#pragma unroll
                    for (uint32_t kk = 0; kk < kChunkElems / 16; ++kk) {
                        uint32_t a[4];
                        ldmatrix_a(a, tile + (((2 * kk + lm_hi) ^ (lm_row & 7)) << 4));
                        uint4 xv = make_uint4(0, 0, 0, 0);
                        if (has_col) xv = *reinterpret_cast<const uint4*>(xb + kk * 16);
                        mma_f16(tot, a[0], a[1], a[2], a[3], xv.z, xv.w);  // residual
                        mma_f16(tot, a[0], a[1], a[2], a[3], xv.x, xv.y);  // value
                    }
                    __syncwarp();
                    if (item + p.stages < total) {
                        // order this warp's reads of the stage before the asynchronous writes that refill it
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        issue(item + p.stages);
                    }
                }
                float* mine = red + (part * kQ8Warps + warp) * 128;
                mine[g * 8 + 2 * t] = tot[0];
                mine[g * 8 + 2 * t + 1] = tot[1];
                mine[(g + 8) * 8 + 2 * t] = tot[2];
                mine[(g + 8) * 8 + 2 * t + 1] = tot[3];
            }
            __syncthreads();
            if (tid < 128) {
                // fixed-order sum of the warps' partial sums; carried across slices in shared memory
                float y[2] = {0.f, 0.f};
                for (uint32_t part = 0; part < parts; ++part) {
                    const float* src = red + part * kQ8Warps * 128 + tid;
                    float v = 0.f;
#pragma unroll
                    for (int w = 0; w < kQ8Warps; ++w) v += src[w * 128];
                    if (slice_end - slice_begin > 1) {
                        float* carry = s_acc + (gi * 2 + part) * 128 + tid;
                        if (slice > slice_begin) v += *carry;
                        if (slice + 1 < slice_end) *carry = v;
                    }
                    y[part] = v;
                }
                const uint32_t row = rg * kRows + (tid >> 3), c = tid & 7;
                if (slice + 1 == slice_end && row < p.d && c < p.batch) {
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
                    const size_t o = static_cast<size_t>(c) * stride + (row - r0) +
                                     (p.k_split > 1 ? slice_begin * p.partial_stride : 0);
                    if (p.out_dtype == ATTN_DTYPE_F32) {
                        float* dst = reinterpret_cast<float*>(out) + o;
                        *dst = p.accumulate ? *dst + v : v;
                    } else {
                        reinterpret_cast<__half*>(out)[o] = __float2half_rn(v);
                    }
                }
            }
        }
    }
    if (timed_out && lane == 0 && p.status) atomicOr(p.status, ATTN_STATUS_WAIT_TIMEOUT);
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up once (a host-side computation; nothing is allocated).
EncodeTiledFn encode_tiled_fn() {
    static std::atomic<void*> cached{nullptr};
    void* fn = cached.load(std::memory_order_acquire);
    if (!fn) {
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            return nullptr;
        cached.store(fn, std::memory_order_release);
    }
    return reinterpret_cast<EncodeTiledFn>(fn);
}

}  // namespace
}  // namespace b200

// Host side of attn_gemv_f16 for batches and for the fused forms (row segments, SwiGLU, k_split); the argument
// checks that do not depend on the kernel are made by the caller in attn_gemv.cu.
int b200::launch_gemv_f16_mma(const AttnGemvArgs* a, cudaStream_t stream) {
    if (a->n % kChunkElems != 0 || a->batch > 8) return ATTN_ERR_UNSUPPORTED;
    if (a->swiglu && (a->d % kRows != 0 || a->split1 || a->split2)) return ATTN_ERR_UNSUPPORTED;
    const uint32_t k_split = a->k_split > 1 ? a->k_split : 1;
    if (k_split > 1 && (a->swiglu || a->split1 || a->accumulate || a->clip > 0.f || a->out_dtype != ATTN_DTYPE_F32))
        return ATTN_ERR_UNSUPPORTED;
    if ((a->split1 && (!a->out2 || a->split1 >= a->d)) || (a->split2 && (!a->out3 || a->split2 <= a->split1 || a->split2 >= a->d)))
        return ATTN_ERR_INVALID_ARG;
    DeviceInfo dev{};
    int rc = current_device_info(&dev);
    if (rc != ATTN_OK) return rc;
    const uint32_t n_chunks = a->n / kChunkElems;
    const uint32_t groups = (a->d + kRows - 1) / kRows;
    const uint32_t set_max = static_cast<uint32_t>(dev.sm_count) / k_split;  // CTAs per k-slice set
    if (set_max == 0) return ATTN_ERR_UNSUPPORTED;
    const uint32_t set_ctas = groups < set_max ? groups : set_max;
    const uint32_t grid = set_ctas * k_split;
    const uint32_t groups_per_cta = (groups + set_ctas - 1) / set_ctas;
    const size_t budget = static_cast<size_t>(dev.max_smem_optin);
    // staged activations: 4 bytes per element and sequence, sequences 64 bytes apart modulo 128 (bank spread)
    auto x_bytes = [&](uint32_t chunks) { return static_cast<size_t>(a->batch) * (chunks * kChunkElems * 4 + 64); };
    auto fixed_bytes = [&](uint32_t slices) {
        return 2 * 2 * kQ8Warps * 128 * sizeof(float) + ((slices > 1 && k_split == 1) ? groups_per_cta * 2 * 128 * sizeof(float) : 0) +
               kQ8Warps * kMaxStages * sizeof(uint64_t) + 1024;
    };
    const size_t ring2 = 2 * static_cast<size_t>(kQ8Warps) * kStageBytes;
    uint32_t slices = k_split;
    if (k_split > 1) {
        if (n_chunks % k_split != 0 || fixed_bytes(1) + ring2 + x_bytes(n_chunks / k_split) > budget) return ATTN_ERR_UNSUPPORTED;
    } else {
        while (slices <= n_chunks && (n_chunks % slices != 0 || fixed_bytes(slices) + ring2 + x_bytes(n_chunks / slices) > budget))
            ++slices;
        if (slices > n_chunks) return ATTN_ERR_UNSUPPORTED;
    }
    const uint32_t slice_chunks = n_chunks / slices;
    uint32_t stages = kMaxStages;
    while (stages > 2 && fixed_bytes(slices) + stages * kQ8Warps * kStageBytes + x_bytes(slice_chunks) > budget) --stages;
    const size_t smem = fixed_bytes(slices) + static_cast<size_t>(stages) * kQ8Warps * kStageBytes + x_bytes(slice_chunks);

    // W as a 2-D tensor of 16-bit elements [rows][n]; one box = 16 rows x 64 elements, 128-byte swizzle.
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return ATTN_ERR_CUDA;
    CUtensorMap tm_w;
    {
        const cuuint64_t dims[2] = {a->n, static_cast<cuuint64_t>(a->d) * (a->swiglu ? 2 : 1)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a->n) * 2};
        const cuuint32_t box[2] = {kChunkElems, kRows};
        const cuuint32_t estr[2] = {1, 1};
        CUresult r = enc(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(a->w), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            g_last_cuda_error = static_cast<int>(r);
            return ATTN_ERR_CUDA;
        }
    }
    MmaParams p{};
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
    p.slice_chunks = slice_chunks;
    p.n_slices = slices;
    p.d = a->d;
    p.batch = a->batch;
    p.stages = stages;
    p.x_col_pitch = slice_chunks * kChunkElems + 16;
    p.acc_groups = (slices > 1 && k_split == 1) ? groups_per_cta : 0;
    p.k_split = k_split;
    p.partial_stride = static_cast<uint64_t>(a->batch) * stride0;
    p.swiglu = a->swiglu ? 1u : 0u;
    p.clip = a->clip;
    p.out_dtype = a->out_dtype;
    p.accumulate = a->accumulate;
    B200_CUDA_TRY(cudaFuncSetAttribute(gemv_f16_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    B200_CUDA_TRY(launch_dependent(gemv_f16_mma_kernel, dim3(grid), dim3(kQ8Threads), smem, stream, tm_w, p));
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return ATTN_OK;
}
