// Weight GEMV over fp16 weights on the tensor cores, for batches: out[b][j] = clamp(sum_i x[b][i] * W[j][i]) with W
// [d][n] fp16 (n fastest) and fp32 activations of 1..8 sequences. It is the formulation of the Q8_0 kernel next to it
// applied to the engine's own weight type (matmul() of include/kernels_cpu.hpp:69-80, clamp of
// src/model/block.cpp:130-138): the streaming kernel of attn_gemv.cu multiplies every weight by every sequence's
// activation on the CUDA cores and reads those activations from shared memory once per weight (batch 8: 1.5 TB/s),
// whereas here a batch of up to 8 sequences is the N dimension of one m16n8k16 MMA and costs nothing extra.
//
// One persistent CTA per SM, 16 warps. A CTA owns groups of 16 consecutive rows; its warps split the inner dimension
// in chunks of 64 elements. The weights go from global memory straight into the MMA's A registers: lane (g, t) of a
// warp reads 32 contiguous bytes of row g (and of row g + 8) - the four lanes of a row cover one 128-byte line - with
// streaming 256-bit loads, eight in flight per lane (128 KB per SM), and those sixteen values are the lane's A
// operands of four k-steps as they are: the order of the inner dimension inside a chunk is free as long as the
// activations follow it, so k-step j of lane t multiplies elements 16 t + 4 j .. + 3 of the chunk. (A first version
// staged swizzled TMA tiles in shared memory and read them with ldmatrix; it stopped at ~ 3.8 TB/s because the TMA
// engine delivers the 128-byte rows of a tile at ~ 0.1 row per clock and SM.) B = the activations as fp16 value +
// fp16 residual (two MMAs per k-step, ~ 22 significant bits; |x| clamped to the fp16 range), staged once per CTA in
// shared memory in that order; fp32 accumulation in the MMA over the whole inner dimension. The warps' partial sums of
// a row group are added in a fixed order. Row segments, the SwiGLU epilogue over stacked gate / up rows, in-kernel
// slices of the inner dimension and k_split work as in the Q8_0 kernel.
//
// Algorithmic bytes per call = rows * n * 2 + batch * (n*4 + d*sizeof(out)).
#include "gemv_mma_common.cuh"

namespace b200 {
namespace {

using namespace gemv_mma;

constexpr uint32_t kChunkElems = 64;  // elements of one row per chunk: 32 bytes per lane, one 128-byte line per row
constexpr int kF16Warps = 16;
constexpr int kF16Threads = kF16Warps * 32;
constexpr int kUnroll = 4;            // chunks in flight per warp: 2 x 4 loads of 32 bytes per lane

struct alignas(32) W8 {
    uint32_t v[8];
};

// 256-bit streaming load (sm_100): read-only path, no L1 allocation, evict-first in L2.
__device__ __forceinline__ W8 ld_stream32(const void* p) {
    W8 r;
    asm volatile("ld.global.nc.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]), "=r"(r.v[5]), "=r"(r.v[6]), "=r"(r.v[7])
                 : "l"(p));
    return r;
}

__global__ void __launch_bounds__(kF16Threads, 1) gemv_f16_mma_kernel(const uint16_t* __restrict__ w, uint64_t w_rows,
                                                                      uint64_t n, const __grid_constant__ Params p) {
    extern __shared__ __align__(16) uint8_t smem[];
    // layout: [red: 2 x 2 x warps x 128 floats][acc: acc_groups x 2 x 128 floats][x fragments]
    float* s_red = reinterpret_cast<float*>(smem);
    float* s_acc = s_red + 2 * 2 * kF16Warps * 128;
    uint32_t* s_x = reinterpret_cast<uint32_t*>(s_acc + p.acc_groups * 2 * 128);

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t groups = (p.d + kRows - 1) / kRows;
    const uint32_t parts = p.swiglu ? 2u : 1u;  // row groups of W per output row group (gate, up)
    // split-k: the grid is k_split sets of CTAs; set s handles slice s of every row group it owns
    const uint32_t ctas = gridDim.x / p.k_split, cta = blockIdx.x % ctas;
    const uint32_t slice_begin = p.k_split > 1 ? blockIdx.x / ctas : 0;
    const uint32_t slice_end = p.k_split > 1 ? slice_begin + 1 : p.n_slices;
    const uint32_t my_groups = (groups > cta) ? (groups - cta + ctas - 1) / ctas : 0;

    grid_dep_launch_dependents();
    grid_dep_wait();  // x (and out, when accumulating) come from the previous kernel

    const bool has_col = g < p.batch;  // lanes of the other columns feed zeros
    const uint32_t* my_x = s_x + (has_col ? g : 0) * p.x_col_pitch + t * 4;
    uint32_t round = 0;
    for (uint32_t slice = slice_begin; slice < slice_end; ++slice) {
        // Activations of this slice as B fragments, in the order the A registers hold the weights: for sequence c,
        // chunk ch, k-step j, lane quarter tt: four 32-bit words {hi(x0,x1), hi(x2,x3), lo(x0,x1), lo(x2,x3)} of the
        // elements x[64 ch + 16 tt + 4 j .. + 4). Every warp has passed the previous slice's last block-wide barrier,
        // so nobody still reads the old fragments.
        const float* xs = p.x + static_cast<size_t>(slice) * p.slice_units * kChunkElems;
        const uint32_t per_seq = p.slice_units * 16;  // groups of four elements per sequence
        for (uint32_t i = tid; i < p.batch * per_seq; i += kF16Threads) {
            const uint32_t c = i / per_seq, r = i - c * per_seq;
            const uint32_t ch = r >> 4, j = (r >> 2) & 3, tt = r & 3;
            const float4 v = *reinterpret_cast<const float4*>(xs + c * p.x_batch_stride + 64 * ch + 16 * tt + 4 * j);
            *reinterpret_cast<uint4*>(s_x + c * p.x_col_pitch + r * 4) = split_activations(v.x, v.y, v.z, v.w);
        }
        __syncthreads();

        const size_t slice_elem0 = static_cast<size_t>(slice) * p.slice_units * kChunkElems;
        for (uint32_t gi = 0; gi < my_groups; ++gi, ++round) {
            const uint32_t rg = cta + gi * ctas;
            float* red = s_red + (round & 1) * 2 * kF16Warps * 128;
            for (uint32_t part = 0; part < parts; ++part) {
                // rows g and g + 8 of the group; a ragged last group re-reads the last row (its results are dropped)
                uint64_t row_lo = static_cast<uint64_t>(part) * p.d + rg * kRows + g, row_hi = row_lo + 8;
                row_lo = row_lo < w_rows ? row_lo : w_rows - 1;
                row_hi = row_hi < w_rows ? row_hi : w_rows - 1;
                const uint16_t* w_lo = w + row_lo * n + slice_elem0 + 16 * t;
                const uint16_t* w_hi = w + row_hi * n + slice_elem0 + 16 * t;
                float tot[4] = {0.f, 0.f, 0.f, 0.f};
                for (uint32_t c0 = warp; c0 < p.slice_units; c0 += kF16Warps * kUnroll) {
                    W8 alo[kUnroll], ahi[kUnroll];
#pragma unroll
                    for (int u = 0; u < kUnroll; ++u) {
                        const uint32_t ch = c0 + u * kF16Warps;
                        if (ch < p.slice_units) {
                            alo[u] = ld_stream32(w_lo + static_cast<size_t>(ch) * kChunkElems);
                            ahi[u] = ld_stream32(w_hi + static_cast<size_t>(ch) * kChunkElems);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < kUnroll; ++u) {
                        const uint32_t ch = c0 + u * kF16Warps;
                        if (ch < p.slice_units) {
                            const uint32_t* xb = my_x + ch * 64;
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                uint4 xv = make_uint4(0, 0, 0, 0);
                                if (has_col) xv = *reinterpret_cast<const uint4*>(xb + j * 16);
                                // a0 = row g, a1 = row g + 8 (first element pair); a2, a3 = the second pair
                                mma_f16(tot, alo[u].v[2 * j], ahi[u].v[2 * j], alo[u].v[2 * j + 1], ahi[u].v[2 * j + 1], xv.z, xv.w);
                                mma_f16(tot, alo[u].v[2 * j], ahi[u].v[2 * j], alo[u].v[2 * j + 1], ahi[u].v[2 * j + 1], xv.x, xv.y);
                            }
                        }
                    }
                }
                store_partial<kF16Warps>(red, part, warp, g, t, tot);
            }
            __syncthreads();
            reduce_and_store<kF16Warps>(p, red, s_acc, tid, parts, gi, rg, slice, slice_begin, slice_end);
        }
    }
}

}  // namespace
}  // namespace b200

// Host side of attn_gemv_f16 for batches and for the fused forms (row segments, SwiGLU, k_split); the argument
// checks that do not depend on the kernel are made by the caller in attn_gemv.cu.
int b200::launch_gemv_f16_mma(const AttnGemvArgs* a, cudaStream_t stream) {
    if (a->n % kChunkElems != 0 || a->batch > 8) return ATTN_ERR_UNSUPPORTED;
    uint32_t k_split = 1;
    if (int rc0 = check_fused_args(a, &k_split); rc0 != ATTN_OK) return rc0;
    if (a->out_dtype == ATTN_DTYPE_SPLIT16) return ATTN_ERR_UNSUPPORTED;
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
        return 2 * 2 * kF16Warps * 128 * sizeof(float) + ((slices > 1 && k_split == 1) ? groups_per_cta * 2 * 128 * sizeof(float) : 0);
    };
    // The activations are staged in equal slices of the inner dimension, as few as fit in shared memory; the partial
    // sums of the CTA's row groups are carried from slice to slice (or, with k_split, go to separate sets of CTAs).
    uint32_t slices = k_split;
    if (k_split > 1) {
        if (n_chunks % k_split != 0 || fixed_bytes(1) + x_bytes(n_chunks / k_split) > budget) return ATTN_ERR_UNSUPPORTED;
    } else {
        while (slices <= n_chunks && (n_chunks % slices != 0 || fixed_bytes(slices) + x_bytes(n_chunks / slices) > budget)) ++slices;
        if (slices > n_chunks) return ATTN_ERR_UNSUPPORTED;
    }
    const uint32_t slice_chunks = n_chunks / slices;
    const size_t smem = fixed_bytes(slices) + x_bytes(slice_chunks);

    Params p{};
    fill_common(p, a, k_split);
    p.slice_units = slice_chunks;
    p.n_slices = slices;
    p.stages = 0;
    p.x_col_pitch = slice_chunks * kChunkElems + 16;
    p.acc_groups = (slices > 1 && k_split == 1) ? groups_per_cta : 0;
    const uint64_t w_rows = static_cast<uint64_t>(a->d) * (a->swiglu ? 2 : 1);
    B200_CUDA_TRY(cudaFuncSetAttribute(gemv_f16_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    B200_CUDA_TRY(launch_dependent(gemv_f16_mma_kernel, dim3(grid), dim3(kF16Threads), smem, stream,
                                   static_cast<const uint16_t*>(a->w), w_rows, static_cast<uint64_t>(a->n), p));
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return ATTN_OK;
}
