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
#include "gemv_mma_common.cuh"

namespace b200 {
namespace {

using namespace gemv_mma;

constexpr uint32_t kChunkElems = 64;                        // elements of one row per stage: one 128-byte swizzle row
constexpr uint32_t kStageBytes = kRows * kChunkElems * 2;   // 2048: one swizzle-128B tile of 16 rows
constexpr uint32_t kMaxStages = 6;                          // barrier slots per warp

// Four 8x8 fp16 matrices from shared memory, one row address per lane: the A fragment of one k-step.
__device__ __forceinline__ void ldmatrix_a(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__global__ void __launch_bounds__(kThreads, 1) gemv_f16_mma_kernel(const __grid_constant__ CUtensorMap tm_w,
                                                                     const __grid_constant__ Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);  // swizzled tiles want 1024-byte alignment
    // layout: [ring: warps x stages x kStageBytes][red: 2 x 2 x warps x 128 floats][acc: acc_groups x 2 x 128 floats]
    //         [bars: warps x kMaxStages][x fragments]
    const uint32_t ring_bytes = kWarps * p.stages * kStageBytes;
    float* s_red = reinterpret_cast<float*>(smem + ring_bytes);
    float* s_acc = s_red + 2 * 2 * kWarps * 128;
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_acc + p.acc_groups * 2 * 128);
    uint32_t* s_x = reinterpret_cast<uint32_t*>(s_bar + kWarps * kMaxStages);

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t groups = (p.d + kRows - 1) / kRows;
    const uint32_t parts = p.swiglu ? 2u : 1u;  // row groups of W per output row group (gate, up)
    // chunks of one slice of one row group that this warp owns: warp, warp + 8, ...
    const uint32_t cpw = (p.slice_units > warp) ? (p.slice_units - warp + kWarps - 1) / kWarps : 0;
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
        const uint32_t chunk = slice * p.slice_units + warp + ci * kWarps;
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
        const float* xs = p.x + static_cast<size_t>(slice) * p.slice_units * kChunkElems;
        const uint32_t per_seq = p.slice_units * (kChunkElems / 16) * 4;  // (k-step, quarter) pairs per sequence
        for (uint32_t i = tid; i < p.batch * per_seq; i += kThreads) {
            const uint32_t c = i / per_seq, r = i - c * per_seq;
            const uint32_t ks = r >> 2, tt = r & 3;
            const float* src = xs + c * p.x_batch_stride + 16 * ks + 2 * tt;
            const float2 a = *reinterpret_cast<const float2*>(src), b = *reinterpret_cast<const float2*>(src + 8);
            const uint4 o = split_activations(a.x, a.y, b.x, b.y);
            *reinterpret_cast<uint4*>(s_x + c * p.x_col_pitch + r * 4) = o;
        }
        __syncthreads();

        for (uint32_t gi = 0; gi < my_groups; ++gi, ++round) {
            const uint32_t rg = cta + gi * ctas;
            float* red = s_red + (round & 1) * 2 * kWarps * 128;
            for (uint32_t part = 0; part < parts; ++part) {
                float tot[4] = {0.f, 0.f, 0.f, 0.f};
                for (uint32_t ci = 0; ci < cpw; ++ci, ++item) {
                    const uint32_t stage = item % p.stages;
                    if (!mbar_wait(bar0 + 8 * stage, (item / p.stages) & 1)) timed_out = true;
                    const uint32_t tile = ring0 + stage * kStageBytes + lm_row * 128;
                    const uint32_t* xb = my_x + (warp + ci * kWarps) * (kChunkElems / 16) * 16;
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
                store_partial(red, part, warp, g, t, tot);
            }
            __syncthreads();
            reduce_and_store(p, red, s_acc, tid, parts, gi, rg, slice, slice_begin, slice_end);
        }
    }
    if (timed_out && lane == 0 && p.status) atomicOr(p.status, ATTN_STATUS_WAIT_TIMEOUT);
}

}  // namespace
}  // namespace b200

// Host side of attn_gemv_f16 for batches and for the fused forms (row segments, SwiGLU, k_split); the argument
// checks that do not depend on the kernel are made by the caller in attn_gemv.cu.
int b200::launch_gemv_f16_mma(const AttnGemvArgs* a, cudaStream_t stream) {
    if (a->n % kChunkElems != 0 || a->batch > 8) return ATTN_ERR_UNSUPPORTED;
    uint32_t k_split = 1;
    if (int rc0 = check_fused_args(a, &k_split); rc0 != ATTN_OK) return rc0;
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
        return 2 * 2 * kWarps * 128 * sizeof(float) + ((slices > 1 && k_split == 1) ? groups_per_cta * 2 * 128 * sizeof(float) : 0) +
               kWarps * kMaxStages * sizeof(uint64_t) + 1024;
    };
    const size_t ring2 = 2 * static_cast<size_t>(kWarps) * kStageBytes;
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
    while (stages > 2 && fixed_bytes(slices) + stages * kWarps * kStageBytes + x_bytes(slice_chunks) > budget) --stages;
    const size_t smem = fixed_bytes(slices) + static_cast<size_t>(stages) * kWarps * kStageBytes + x_bytes(slice_chunks);

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
    Params p{};
    fill_common(p, a, k_split);
    p.slice_units = slice_chunks;
    p.n_slices = slices;
    p.stages = stages;
    p.x_col_pitch = slice_chunks * kChunkElems + 16;
    p.acc_groups = (slices > 1 && k_split == 1) ? groups_per_cta : 0;
    B200_CUDA_TRY(cudaFuncSetAttribute(gemv_f16_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    B200_CUDA_TRY(launch_dependent(gemv_f16_mma_kernel, dim3(grid), dim3(kThreads), smem, stream, tm_w, p));
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return ATTN_OK;
}
