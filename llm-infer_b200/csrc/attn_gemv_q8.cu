// Weight GEMV over Q8_0 weights: out[b][j] = clamp(sum_i x[b][i] * W[j][i]) with W stored in the public GGML Q8_0
// block format - blocks of 32 consecutive elements of a row, each block a little-endian fp16 scale followed by 32
// signed bytes (34 bytes), value = scale * q - rows [d][n/32] blocks, n fastest. The engine lists the type
// (include/gguf.hpp:28) but has no kernel or CPU path for it (its loader accepts F32 / F16 only,
// src/model/config.cpp:11-17,26-34); this kernel is what the projections of a Q8_0 model need, with the same
// interface as the fp16 GEMV next to it (clamp of src/model/block.cpp:130-138, residual accumulate).
//
// 34 bytes per 32 weights, every byte read once. One persistent CTA per SM, 8 warps. A CTA owns groups of
// 16 consecutive rows; its warps split the inner dimension in chunks of 8 blocks (256 elements). Each warp runs its
// own ring of shared-memory stages, each filled by one TMA tile load (16 rows x 272 bytes; one request per stage - 16
// separate row copies per stage were limited by the copy engine's request rate, 2.5 TB/s), completion counted on an
// mbarrier; the warp refills a stage as soon as it has consumed it, so up to 139 KB per SM are in flight with no
// register cost. The arithmetic runs on the tensor cores as m16n8k16 fp16 MMAs: A = the 16 rows' int8
// values, exactly representable in fp16 (built with one byte-permute and one half2 subtract per pair), B = the
// activations of up to 8 sequences split into an fp16 value plus an fp16 residual (two MMAs, ~ 22 significant bits;
// |x| is clamped to the fp16 range, 65504), fp32 accumulation per block, then one fp32 multiply-add by the block's
// scale per row. The eight warps' partial sums of a row group are added in a fixed order.
//
// Three extras serve the transformer block: the output rows may be split into up to three segments with their own
// buffers (one launch for the Q, K and V projections over a stacked matrix); with `swiglu` the matrix holds gate rows
// followed by up rows and the kernel writes silu(gate x) * (up x) (one launch for the FFN's first half); and when the
// activations of all sequences do not fit in shared memory next to the ring (batch 8 x 14336), the inner dimension is
// staged in equal slices inside the one launch, partial sums carried in shared memory - or, with `k_split`, the slices
// go to separate sets of CTAs that store their partial sums for the consumer (the next RMSNorm) to add.
//
// Algorithmic bytes per call = rows * n/32 * 34 + batch * (n*4 + d*sizeof(out)).
#include "gemv_mma_common.cuh"

namespace b200 {
namespace {

using namespace gemv_mma;

constexpr uint32_t kBlockBytes = 34;                        // fp16 scale + 32 int8
// Blocks of one row per stage (CB): 8 (272-byte row segments, up to four stages per warp) or 16 (544-byte segments,
// two stages: ~10 % faster streaming, used when the activations leave room). A row segment is 68 or 136 words long
// (4 or 8 mod 32), so the 8 rows x 4 lanes of one shared-memory load never share a bank.
constexpr uint32_t kMaxStages = 4;                          // barrier slots per warp
constexpr uint32_t seg_bytes(uint32_t cb) { return cb * kBlockBytes; }          // one row's share of a stage
constexpr uint32_t stage_bytes(uint32_t cb) { return kRows * seg_bytes(cb); }   // 4352 or 8704, multiples of 128

// Two bytes of w (already XORed with 0x80, i.e. q + 128) -> half2 (q_lo, q_hi): 0x6400 | u is the fp16 number
// 1024 + u, and 1024 + u - 1152 = q exactly.
template <int FIRST>
__device__ __forceinline__ uint32_t bytes_to_half2(uint32_t w) {
    constexpr uint32_t sel = 0x4040u | FIRST | ((FIRST + 1) << 8);
    const uint32_t biased = __byte_perm(w, 0x64646464u, sel);
    const __half2 h = __hsub2(*reinterpret_cast<const __half2*>(&biased), __half2half2(__ushort_as_half(0x6480)));
    return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ float lds_scale(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return __half2float(__ushort_as_half(v));
}

// The eight int8 values of block `bi` of one staged row segment that lane quarter t owns, as the lane's A-fragment
// halves: q[4t .. 4t+4) feed the first k-step (r[0], r[1]), q[16+4t .. 16+4t+4) the second (r[2], r[3]). The four
// lanes of a row read consecutive words and the rows are 68 words apart, so a load touches every bank once. A block
// starts at 34*bi, its values at +2: four-byte aligned for odd bi, two bytes off for even bi (two words, one permute).
template <bool EVEN>
__device__ __forceinline__ void load_a(uint32_t (&r)[4], uint32_t seg_addr, uint32_t bi, uint32_t t) {
    const uint32_t base = seg_addr + kBlockBytes * bi + 4 * t;
    uint32_t v0, v1;
    if constexpr (EVEN) {
        v0 = __byte_perm(lds32(base), lds32(base + 4), 0x5432);
        v1 = __byte_perm(lds32(base + 16), lds32(base + 20), 0x5432);
    } else {
        v0 = lds32(base + 2);
        v1 = lds32(base + 18);
    }
    v0 ^= 0x80808080u;
    v1 ^= 0x80808080u;
    r[0] = bytes_to_half2<0>(v0);
    r[1] = bytes_to_half2<2>(v0);
    r[2] = bytes_to_half2<0>(v1);
    r[3] = bytes_to_half2<2>(v1);
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// Tiled layout (attn_repack_q8_0_tiled): one word = the four values of one row that a lane feeds to one k-step, stored
// as bytes q + 128 in the order (e0, e2, e1, e3). The even bytes are then the half2 (e0, e1) after one AND/OR
// (0x6400 | u = 1024 + u) and the odd bytes the half2 (e2, e3) after one byte-permute; 1024 + u - 1152 = q exactly.
__device__ __forceinline__ void word_to_fragments(uint32_t w, uint32_t& first, uint32_t& second) {
    const uint32_t even = (w & 0x00ff00ffu) | 0x64006400u;
    const uint32_t odd = __byte_perm(w, 0x64646464u, 0x4341);
    const __half2 bias = __half2half2(__ushort_as_half(0x6480));
    const __half2 a = __hsub2(*reinterpret_cast<const __half2*>(&even), bias);
    const __half2 b = __hsub2(*reinterpret_cast<const __half2*>(&odd), bias);
    first = *reinterpret_cast<const uint32_t*>(&a);
    second = *reinterpret_cast<const uint32_t*>(&b);
}

// NW warps per CTA. REGX: the inner dimension (or, with split-k, the CTA's slice of it) is exactly NW chunks, so a warp always multiplies by the same CB blocks
// of the activations and keeps them in registers as MMA B fragments (64 registers for CB = 8) for the whole launch:
// no shared memory for the activations (which at batch 8 x 4096 would take 128 KB and leave room for 8 warps only), no
// shared-memory loads for them in the inner loop, and twice the warps per SM to hide the latency of the
// byte -> fp16 operand construction.
// TILED: the weights are in the tiled layout (one contiguous 4352-byte tile per 16 rows x 8 blocks, values already in
// MMA fragment order, see attn_repack_q8_0_tiled): a stage is filled by one plain bulk copy, and a lane gets its
// sixteen values of a block with one 16-byte shared-memory load and the two scales with one 4-byte load, in place of
// four to eight 4-byte loads, two alignment permutes, two XORs and two 2-byte loads.
template <uint32_t CB, int NW, bool REGX, bool TILED>
__global__ void __launch_bounds__(NW * 32, 1) gemv_q8_0_kernel(const __grid_constant__ CUtensorMap tm_w,
                                                                 const __grid_constant__ Params p) {
    constexpr uint32_t kWarps = NW, kThreads = NW * 32;
    constexpr uint32_t kChunkBlocks = CB, kSegBytes = seg_bytes(CB), kSegPitch = kSegBytes, kStageBytes = stage_bytes(CB);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);  // tile loads want 128-byte alignment
    // layout: [ring: warps x stages x kStageBytes][red: 2 x 2 x warps x 128 floats][acc: acc_groups x 2 x 128 floats]
    //         [bars: warps x kMaxStages][x fragments]
    const uint32_t ring_bytes = kWarps * p.stages * kStageBytes;
    float* s_red = reinterpret_cast<float*>(smem + ring_bytes);
    float* s_acc = s_red + 2 * 2 * kWarps * 128;
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_acc + p.acc_groups * 2 * 128);
    uint32_t* s_x = reinterpret_cast<uint32_t*>(s_bar + kWarps * kMaxStages + 2);  // + the activations' barrier (padded to 16 bytes)
    const uint32_t bar_x = smem_u32(s_bar + kWarps * kMaxStages);

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t groups = (p.d + kRows - 1) / kRows;
    const uint32_t parts = p.swiglu ? 2u : 1u;  // row groups of W per output row group (gate, up)
    const uint32_t slice_chunks = p.slice_units / kChunkBlocks;
    // chunks of one slice of one row group that this warp owns: warp, warp + 8, ...
    const uint32_t cpw = (slice_chunks > warp) ? (slice_chunks - warp + kWarps - 1) / kWarps : 0;
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
        if (warp == 0) mbar_init(bar_x, 1);
        mbar_init_fence();
    }
    __syncwarp();

    auto issue = [&](uint32_t item) {
        const uint32_t ci = item % cpw, q = item / cpw;
        const uint32_t part = q % parts, q2 = q / parts;
        const uint32_t gi = q2 % my_groups, slice = slice_begin + q2 / my_groups;
        const uint32_t rg = cta + gi * ctas;
        const uint32_t chunk = slice * slice_chunks + warp + ci * kWarps;
        const uint32_t stage = item % p.stages;
        const uint32_t bar = bar0 + 8 * stage;
        if (lane == 0) {
            mbar_arrive_expect_tx(bar, kStageBytes);
            if constexpr (TILED) {
                const uint8_t* src =
                    p.w_tiles + (static_cast<size_t>(part * groups + rg) * p.row_chunks + chunk) * kStageBytes;
                bulk_g2s(ring0 + stage * kStageBytes, src, kStageBytes, bar, policy);
                return;
            }
            // x in 32-bit elements (a multiple of 4: 16-byte rule), y = first row of the group (rows past the
            // tensor read as zeros)
            tma_load_rows(ring0 + stage * kStageBytes, &tm_w, bar, static_cast<int>(chunk * (kSegBytes / 4)),
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
    bool timed_out = false;
    uint32_t item = 0, round = 0;
    uint4 xr[REGX ? CB : 1][2];
    if constexpr (REGX) {
        // B fragments of this warp's chunk (blocks [warp*CB, +CB) of sequence g), straight from global memory: the
        // prepared form is already laid out as fragments, fp32 activations are split here
#pragma unroll
        for (uint32_t bi = 0; bi < CB; ++bi) {
#pragma unroll
            for (uint32_t s2 = 0; s2 < 2; ++s2) {
                xr[bi][s2] = make_uint4(0, 0, 0, 0);
                if (has_col) {
                    // (with split-k this CTA's slice starts slice_begin * NW chunks into the row)
                    const size_t e = static_cast<size_t>(g) * p.x_batch_stride + 32 * ((slice_begin * NW + warp) * CB + bi) +
                                     16 * s2 + 4 * t;
                    if (p.x_split) {
                        xr[bi][s2] = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint32_t*>(p.x) + e);
                    } else {
                        const float4 v = *reinterpret_cast<const float4*>(p.x + e);
                        xr[bi][s2] = split_activations(v.x, v.y, v.z, v.w);
                    }
                }
            }
        }
    }
    for (uint32_t slice = slice_begin; slice < slice_end; ++slice) {
        // Activations of this slice as B fragments: for sequence c, block blk, k-step s, quarter t: four 32-bit words
        // {hi(x0,x1), hi(x2,x3), lo(x0,x1), lo(x2,x3)} of the elements x[32 blk + 16 s + 4 t .. +4). Every warp has
        // passed the previous slice's last block-wide barrier, so nobody still reads the old fragments.
        if constexpr (REGX) {
            // activations are in registers
        } else if (p.x_split) {
            // prepared activations: one bulk copy per sequence, as they are; the barrier's phase counts the slices
            __syncthreads();  // (barrier initialised; with more than one slice: the old fragments are no longer read)
            if (tid == 0) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                const uint32_t bytes = p.slice_units * 32 * 4;
                mbar_arrive_expect_tx(bar_x, bytes * p.batch);
                const uint32_t* xw = reinterpret_cast<const uint32_t*>(p.x) + static_cast<size_t>(slice) * p.slice_units * 32;
                for (uint32_t c = 0; c < p.batch; ++c) {
                    bulk_g2s(smem_u32(s_x + c * p.x_col_pitch), xw + c * p.x_batch_stride, bytes, bar_x, l2_policy_evict_last());
                }
            }
            if (!mbar_wait(bar_x, (slice - slice_begin) & 1)) timed_out = true;
        } else {
            const float* xs = p.x + static_cast<size_t>(slice) * p.slice_units * 32;
            for (uint32_t i = tid; i < p.batch * p.slice_units * 8; i += kThreads) {
                const uint32_t c = i / (p.slice_units * 8), r = i - c * (p.slice_units * 8);
                const uint32_t blk = r >> 3, s = (r >> 2) & 1, tt = r & 3;
                const float4 v = *reinterpret_cast<const float4*>(xs + c * p.x_batch_stride + 32 * blk + 16 * s + 4 * tt);
                const uint4 o = split_activations(v.x, v.y, v.z, v.w);
                *reinterpret_cast<uint4*>(s_x + c * p.x_col_pitch + (blk * 2 + s) * 16 + tt * 4) = o;
            }
            __syncthreads();
        }

        for (uint32_t gi = 0; gi < my_groups; ++gi, ++round) {
            const uint32_t rg = cta + gi * ctas;
            float* red = s_red + (round & 1) * 2 * kWarps * 128;
            for (uint32_t part = 0; part < parts; ++part) {
                float tot[4] = {0.f, 0.f, 0.f, 0.f};
                for (uint32_t ci = 0; ci < cpw; ++ci, ++item) {
                    const uint32_t stage = item % p.stages;
                    if (!mbar_wait(bar0 + 8 * stage, (item / p.stages) & 1)) timed_out = true;
                    const uint32_t seg_lo = ring0 + stage * kStageBytes + g * kSegPitch;
                    const uint32_t seg_hi = seg_lo + 8 * kSegPitch;
                    const uint32_t* xb = my_x + (warp + ci * kWarps) * kChunkBlocks * 32;
#pragma unroll
                    for (uint32_t bi = 0; bi < kChunkBlocks; ++bi) {
                        uint32_t alo[4], ahi[4];
                        float s_lo, s_hi;
                        if constexpr (TILED) {
                            const uint32_t blk = ring0 + stage * kStageBytes + bi * (kRows * kBlockBytes);
                            const uint4 w = lds128(blk + lane * 16);
                            word_to_fragments(w.x, alo[0], alo[1]);  // row g, k-step 0
                            word_to_fragments(w.y, ahi[0], ahi[1]);  // row g + 8, k-step 0
                            word_to_fragments(w.z, alo[2], alo[3]);  // row g, k-step 1
                            word_to_fragments(w.w, ahi[2], ahi[3]);  // row g + 8, k-step 1
                            const uint32_t sc = lds32(blk + kRows * 32 + g * 4);
                            const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&sc));
                            s_lo = sf.x;
                            s_hi = sf.y;
                        } else if (bi & 1) {
                            load_a<false>(alo, seg_lo, bi, t);
                            load_a<false>(ahi, seg_hi, bi, t);
                        } else {
                            load_a<true>(alo, seg_lo, bi, t);
                            load_a<true>(ahi, seg_hi, bi, t);
                        }
                        uint4 x0 = make_uint4(0, 0, 0, 0), x1 = make_uint4(0, 0, 0, 0);
                        if constexpr (REGX) {
                            x0 = xr[bi][0];
                            x1 = xr[bi][1];
                        } else if (has_col) {
                            x0 = *reinterpret_cast<const uint4*>(xb + bi * 32);
                            x1 = *reinterpret_cast<const uint4*>(xb + bi * 32 + 16);
                        }
                        float acc[4];
                        mma_f16_first(acc, alo[0], ahi[0], alo[1], ahi[1], x0.z, x0.w);  // k-step 0, residual
                        mma_f16(acc, alo[2], ahi[2], alo[3], ahi[3], x1.z, x1.w);        // k-step 1, residual
                        mma_f16(acc, alo[0], ahi[0], alo[1], ahi[1], x0.x, x0.y);        // k-step 0, value
                        mma_f16(acc, alo[2], ahi[2], alo[3], ahi[3], x1.x, x1.y);        // k-step 1, value
                        if constexpr (!TILED) {
                            s_lo = lds_scale(seg_lo + kBlockBytes * bi);
                            s_hi = lds_scale(seg_hi + kBlockBytes * bi);
                        }
                        tot[0] = fmaf(s_lo, acc[0], tot[0]);
                        tot[1] = fmaf(s_lo, acc[1], tot[1]);
                        tot[2] = fmaf(s_hi, acc[2], tot[2]);
                        tot[3] = fmaf(s_hi, acc[3], tot[3]);
                    }
                    __syncwarp();
                    if (item + p.stages < total) {
                        // order this warp's reads of the stage before the asynchronous writes that refill it
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        issue(item + p.stages);
                    }
                }
                store_partial<NW>(red, part, warp, g, t, tot);
            }
            __syncthreads();
            reduce_and_store<NW>(p, red, s_acc, tid, parts, gi, rg, slice, slice_begin, slice_end);
        }
    }
    if (timed_out && lane == 0 && p.status) atomicOr(p.status, ATTN_STATUS_WAIT_TIMEOUT);
}

}  // namespace
}  // namespace b200

namespace b200 {
namespace {


// One 16-byte unit of the tiled layout per thread: tile (row group rg, chunk c of 8 blocks), block bi, lane (g, t) ->
// the words {row g k-step 0, row g+8 k-step 0, row g k-step 1, row g+8 k-step 1}, each the row's elements
// 32 blk + 16 s + 4 t + (0, 2, 1, 3) as bytes q + 128; lanes 0-7 also write the block's scale pair (rows g, g + 8).
__global__ void repack_q8_0_tiled_kernel(uint8_t* dst, const uint8_t* src, uint32_t d, uint32_t n_blocks, uint64_t units) {
    const uint64_t u = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (u >= units) return;
    const uint32_t lane = static_cast<uint32_t>(u & 31), g = lane >> 2, t = lane & 3;
    const uint64_t blk_id = u >> 5;                       // (rg * n_blocks + blk): tiles of a row group are consecutive
    const uint32_t blk = static_cast<uint32_t>(blk_id % n_blocks);
    const uint32_t rg = static_cast<uint32_t>(blk_id / n_blocks);
    uint8_t* out_blk = dst + blk_id * (kRows * kBlockBytes);
    uint32_t words[4];
    uint16_t scales[2];
#pragma unroll
    for (uint32_t half = 0; half < 2; ++half) {
        const uint32_t row = rg * kRows + g + 8 * half;
        const uint8_t* b = src + (static_cast<uint64_t>(row) * n_blocks + blk) * kBlockBytes;
        const bool live = row < d;
        scales[half] = live ? static_cast<uint16_t>(b[0] | (b[1] << 8)) : 0;
#pragma unroll
        for (uint32_t s = 0; s < 2; ++s) {
            const uint8_t* q = b + 2 + 16 * s + 4 * t;
            const uint32_t e0 = live ? q[0] : 0u, e1 = live ? q[1] : 0u, e2 = live ? q[2] : 0u, e3 = live ? q[3] : 0u;
            words[2 * s + half] = (e0 | (e2 << 8) | (e1 << 16) | (e3 << 24)) ^ 0x80808080u;
        }
    }
    *reinterpret_cast<uint4*>(out_blk + lane * 16) = make_uint4(words[0], words[1], words[2], words[3]);
    // the scale pair of rows (g, g + 8) is the same for the four lanes of a row: the t == 0 lane writes it
    if (t == 0) *reinterpret_cast<uint32_t*>(out_blk + kRows * 32 + g * 4) = scales[0] | (static_cast<uint32_t>(scales[1]) << 16);
}

int gemv_q8_0_launch(const AttnGemvArgs* a, void* stream_v, bool tiled) {
    if (!a || !a->out || !a->x || !a->w || a->n == 0 || a->d == 0 || a->batch == 0) return ATTN_ERR_INVALID_ARG;
    if (a->out_dtype != ATTN_DTYPE_F32 && a->out_dtype != ATTN_DTYPE_F16 && a->out_dtype != ATTN_DTYPE_SPLIT16)
        return ATTN_ERR_INVALID_ARG;
    if (a->n % 256 != 0 || a->batch > 8) return ATTN_ERR_UNSUPPORTED;
    uint32_t k_split = 1;
    if (int rc0 = check_fused_args(a, &k_split); rc0 != ATTN_OK) return rc0;
    if ((reinterpret_cast<uintptr_t>(a->x) & 15u) || (reinterpret_cast<uintptr_t>(a->w) & 15u)) return ATTN_ERR_ALIGNMENT;
    DeviceInfo dev{};
    int rc = current_device_info(&dev);
    if (rc != ATTN_OK) return rc;
    const uint32_t n_blocks = a->n / 32;
    const uint32_t groups = (a->d + kRows - 1) / kRows;
    const uint32_t set_max = static_cast<uint32_t>(dev.sm_count) / k_split;  // CTAs per k-slice set
    if (set_max == 0) return ATTN_ERR_UNSUPPORTED;
    const uint32_t set_ctas = groups < set_max ? groups : set_max;
    const uint32_t grid = set_ctas * k_split;
    const uint32_t groups_per_cta = (groups + set_ctas - 1) / set_ctas;
    const size_t budget = static_cast<size_t>(dev.max_smem_optin);
    // staged activations: 128 bytes per block and sequence, sequences 64 bytes apart modulo 128 (bank spread)
    auto x_bytes = [&](uint32_t blocks) { return static_cast<size_t>(a->batch) * (blocks * 128 + 64); };
    auto fixed_bytes = [&](uint32_t slices) {
        return 2 * 2 * kWarps * 128 * sizeof(float) + ((slices > 1 && k_split == 1) ? groups_per_cta * 2 * 128 * sizeof(float) : 0) +
               (kWarps * kMaxStages + 2) * sizeof(uint64_t) + 128;
    };
    // The activations are staged in equal slices of the inner dimension, as few as leave room for a two-stage ring; the
    // partial sums of the CTA's row groups are carried from slice to slice in shared memory (or, with k_split, the
    // slices go to separate sets of CTAs). 16-block chunks are used when everything fits in one slice with them.
    struct Plan {
        uint32_t cb, slices, stages;
        size_t smem;
    };
    auto make_plan = [&](uint32_t cb, Plan* out) {
        if (n_blocks % cb != 0) return false;
        const uint32_t n_chunks = n_blocks / cb;
        const size_t ring2 = 2 * static_cast<size_t>(kWarps) * stage_bytes(cb);
        uint32_t slices = k_split;
        if (k_split > 1) {
            if (n_chunks % k_split != 0 || fixed_bytes(1) + ring2 + x_bytes(n_blocks / k_split) > budget) return false;
        } else {
            while (slices <= n_chunks && (n_chunks % slices != 0 || fixed_bytes(slices) + ring2 + x_bytes(n_blocks / slices) > budget))
                ++slices;
            if (slices > n_chunks) return false;
        }
        uint32_t stages = cb == 8 ? 4 : 2;
        while (stages > 2 && fixed_bytes(slices) + stages * kWarps * stage_bytes(cb) + x_bytes(n_blocks / slices) > budget) --stages;
        *out = Plan{cb, slices, stages,
                    fixed_bytes(slices) + static_cast<size_t>(stages) * kWarps * stage_bytes(cb) + x_bytes(n_blocks / slices)};
        return true;
    };
    Plan plan{};
    Plan wide{};
    if (!make_plan(8, &plan)) return ATTN_ERR_UNSUPPORTED;  // (the slices must be equal and one must fit next to the ring)
    if (!tiled && k_split == 1 && make_plan(16, &wide) && wide.slices == 1) plan = wide;
    // Inner dimension of exactly 16 chunks of 8 blocks (n = 4096, the model width of the 8B shape): 16 warps, each
    // with its chunk of the activations in registers, two stages per warp, nothing else staged.
    constexpr uint32_t kRegxWarps = 16;
    // (a single sequence of fp32 activations is faster on the 8-warp form: measured 16.1 vs 18.5 us at 14336 x 4096)
    const bool regx_x = a->batch >= 2 || a->x_format == ATTN_DTYPE_SPLIT16;
    const bool regx = k_split == 1 && n_blocks == kRegxWarps * 8 && regx_x;
    // The same with 14 warps for split-k slices of 14 chunks (the 14336-wide down projection cut in four), tiled copy
    // only.
    constexpr uint32_t kRegxSliceWarps = 14;
    const bool regx_slice = tiled && k_split > 1 && n_blocks == k_split * kRegxSliceWarps * 8 && regx_x;
    if (regx || regx_slice) {
        const uint32_t w = regx ? kRegxWarps : kRegxSliceWarps;
        plan = Plan{8, k_split, 2,
                    2 * 2 * w * 128 * sizeof(float) + (w * kMaxStages + 2) * sizeof(uint64_t) + 128 +
                        static_cast<size_t>(2) * w * stage_bytes(8)};
    }
    const uint32_t slices = plan.slices, stages = plan.stages, slice_blocks = n_blocks / slices;
    const size_t smem = plan.smem;

    // W as a 2-D tensor of 32-bit elements [rows][row_bytes / 4]; one box = 16 rows x 272 bytes, no swizzle.
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return ATTN_ERR_CUDA;
    CUtensorMap tm_w{};
    if (!tiled) {
        const cuuint64_t row_bytes = static_cast<cuuint64_t>(n_blocks) * kBlockBytes;
        const cuuint64_t dims[2] = {row_bytes / 4, static_cast<cuuint64_t>(a->d) * (a->swiglu ? 2 : 1)};
        const cuuint64_t strides[1] = {row_bytes};
        const cuuint32_t box[2] = {seg_bytes(plan.cb) / 4, kRows};
        const cuuint32_t estr[2] = {1, 1};
        CUresult r = enc(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(a->w), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            g_last_cuda_error = static_cast<int>(r);
            return ATTN_ERR_CUDA;
        }
    }
    Params p{};
    fill_common(p, a, k_split);
    p.slice_units = slice_blocks;
    p.n_slices = slices;
    p.stages = stages;
    p.x_col_pitch = slice_blocks * 32 + 16;
    p.acc_groups = (slices > 1 && k_split == 1) ? groups_per_cta : 0;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    p.w_tiles = static_cast<const uint8_t*>(a->w);
    p.row_chunks = n_blocks / 8;
    auto kernel = regx_slice ? gemv_q8_0_kernel<8, kRegxSliceWarps, true, true>
                  : tiled    ? (regx ? gemv_q8_0_kernel<8, kRegxWarps, true, true> : gemv_q8_0_kernel<8, kWarps, false, true>)
                  : regx     ? gemv_q8_0_kernel<8, kRegxWarps, true, false>
                  : plan.cb == 16 ? gemv_q8_0_kernel<16, kWarps, false, false> : gemv_q8_0_kernel<8, kWarps, false, false>;
    const uint32_t threads = regx_slice ? kRegxSliceWarps * 32 : regx ? kRegxWarps * 32 : kThreads;
    B200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    B200_CUDA_TRY(launch_dependent(kernel, dim3(grid), dim3(threads), smem, stream, tm_w, p));
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return ATTN_OK;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int attn_gemv_q8_0(const AttnGemvArgs* a, void* stream_v) { return gemv_q8_0_launch(a, stream_v, false); }

extern "C" int attn_gemv_q8_0_tiled(const AttnGemvArgs* a, void* stream_v) { return gemv_q8_0_launch(a, stream_v, true); }

extern "C" size_t attn_q8_0_tiled_bytes(uint32_t d, uint32_t n) {
    return static_cast<size_t>((d + kRows - 1) / kRows) * (n / 32) * (kRows * kBlockBytes);
}

extern "C" int attn_repack_q8_0_tiled(void* dst, const void* src, uint32_t d, uint32_t n, void* stream_v) {
    if (!dst || !src || d == 0 || n == 0) return ATTN_ERR_INVALID_ARG;
    if (n % 256 != 0) return ATTN_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(dst) & 15u) return ATTN_ERR_ALIGNMENT;
    const uint32_t n_blocks = n / 32;
    const uint64_t units = static_cast<uint64_t>((d + kRows - 1) / kRows) * n_blocks * 32;
    const uint64_t grid = (units + 255) / 256;
    if (grid > 0x7fffffffull) return ATTN_ERR_UNSUPPORTED;
    repack_q8_0_tiled_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream_v)>>>(
        static_cast<uint8_t*>(dst), static_cast<const uint8_t*>(src), d, n_blocks, units);
    B200_CUDA_TRY(cudaGetLastError());
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return ATTN_OK;
}
