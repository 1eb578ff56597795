// Split-KV single-token (decode) attention for sm_100a.
//
// What it replaces: the per-head attn() loop of the engine's CPU block
// (include/kernels_cpu.hpp:140-167 called from src/model/block.cpp:157-164) and
// the unfinished device kernel of src/attention.cu:284-370, whose idea of letting
// all G query heads of one kv head share each K/V tile is kept. The KV cache
// layout is the engine's: 16-bit elements, [row][kv_head][head_dim].
//
// Shape of the kernel (one persistent CTA per SM, 9 warps):
//   * warp 8 is the producer. For every tile it issues one bulk asynchronous
//     copy (TMA engine, untiled form) per cache row: HPC*D*2 contiguous bytes
//     that hold HPC kv heads, landing in shared memory at a row pitch of
//     HPC*D*2 + 16 bytes so that ldmatrix reads are bank-conflict free. K and V
//     of a stage complete on separate mbarriers.
//   * warps 0..7 are consumers. Warp w owns kv head w / TS of the CTA's head
//     group and rows [16*(w % TS), +16) of every tile. The G query heads of that
//     kv head are the (zero-padded) 16 rows of an m16n8k16 tensor-core MMA:
//     S = Q K^T, online softmax in fp32 with quad shuffles, O += P V.
//     Q given in fp32 and the probabilities P are each split into a 16-bit high
//     part and a 16-bit residual (two MMAs) so that scores and outputs keep
//     near-fp32 accuracy; K and V enter the tensor cores exactly.
//   * when the CTA's tile range leaves a segment, every warp normalises its
//     state and writes one partial (O, LSE); the merge pass (attn_merge.cu)
//     combines the partials of each head with the online-softmax state merge of
//     src/attention.cu:41-65.
//
// HBM traffic per launch: every K/V byte once (+ the clamped tail rows of the
// last tile of a segment), Q once per (CTA, segment), partials once.
#pragma once

#include "attn_internal.cuh"
#include "merge_device.cuh"
#include "ptx_sm100.cuh"

namespace b200 {

namespace decode_detail {

constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;

struct SegInfo {
    uint32_t seg;       // segment index = b * head_groups + hg
    uint32_t b;
    uint32_t hg;
    uint32_t len;       // valid rows of sequence b
    uint32_t tile0;     // flat index of the segment's first tile
    uint32_t tile_end;  // flat index one past its last tile
};

template <int TT>
struct SegTable {
    const DecodeParams& p;
    const uint32_t* prefix;  // shared memory, [nseg+1]; unused when lengths are uniform
    uint32_t tiles_uniform;

    __device__ __forceinline__ SegInfo load(uint32_t seg) const {
        SegInfo s;
        s.seg = seg;
        s.b = seg / p.head_groups;
        s.hg = seg - s.b * p.head_groups;
        if (p.kv_len) {
            s.len = clamped_len(p.kv_len[s.b], p.kv_capacity);
            s.tile0 = prefix[seg];
            s.tile_end = prefix[seg + 1];
        } else {
            s.len = clamped_len(p.kv_len_uniform, p.kv_capacity);
            s.tile0 = seg * tiles_uniform;
            s.tile_end = s.tile0 + tiles_uniform;
        }
        return s;
    }
    // Segment that contains flat tile t (t < total tiles).
    __device__ __forceinline__ uint32_t find(uint32_t t, uint32_t nseg) const {
        if (!p.kv_len) return t / tiles_uniform;
        uint32_t lo = 0, hi = nseg;  // largest s with prefix[s] <= t  (prefix[nseg] > t)
        while (hi - lo > 1) {
            uint32_t mid = (lo + hi) >> 1;
            if (prefix[mid] <= t) lo = mid; else hi = mid;
        }
        return lo;
    }
};

// Two consecutive elements of q as floats (one 4- or 8-byte load).
template <typename T>
__device__ __forceinline__ float2 load_q_pair(const T* p);
template <>
__device__ __forceinline__ float2 load_q_pair<float>(const float* p) {
    return *reinterpret_cast<const float2*>(p);
}
template <>
__device__ __forceinline__ float2 load_q_pair<__half>(const __half* p) {
    return __half22float2(*reinterpret_cast<const __half2*>(p));
}
template <>
__device__ __forceinline__ float2 load_q_pair<__nv_bfloat16>(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

// The A fragments (m16n8k16, row-major 16 x D) of one kv head's query heads for one lane: rows gq and gq + 8, columns
// kc*16 + cq*2 + {0, 1, 8, 9}. The element type is fixed per instantiation and no data-dependent branch sits between
// the pair loads, so the compiler issues them together and the fetch costs about one memory round trip (a
// per-element load behind a run-time type switch serialised them: several microseconds per call). Rows past the G
// real heads read row G-1 and are zeroed.
template <typename T, int KC, bool QSPLIT, bool BF16>
__device__ __forceinline__ void load_q_fragments(const T* q_head0, int D, int G, int gq, int cq, bool ghi,
                                                 uint32_t (&qhi)[KC][4], uint32_t (&qlo)[QSPLIT ? KC : 1][4]) {
    const int r0 = gq < G ? gq : G - 1;
    const int r1 = gq + 8 < G ? gq + 8 : G - 1;
    const T* p0 = q_head0 + static_cast<size_t>(r0) * D + cq * 2;
    const T* p1 = q_head0 + static_cast<size_t>(r1) * D + cq * 2;
    const float keep0 = gq < G ? 1.f : 0.f;
    const float keep1 = gq + 8 < G ? 1.f : 0.f;
#pragma unroll
    for (int kc = 0; kc < KC; ++kc) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            // a0:(gq, k) a1:(gq+8, k) a2:(gq, k+8) a3:(gq+8, k+8), k = kc*16 + cq*2 + {0,1}
            const bool hi_row = r & 1;
            float x0 = 0.f, x1 = 0.f;
            if (!hi_row || ghi) {  // ghi is uniform over the grid: no divergence, no load for rows that hold no head
                const float2 v = load_q_pair<T>((hi_row ? p1 : p0) + kc * 16 + ((r >> 1) << 3));
                const float keep = hi_row ? keep1 : keep0;
                x0 = v.x * keep;
                x1 = v.y * keep;
            }
            qhi[kc][r] = pack2<BF16>(x0, x1);
            if constexpr (QSPLIT) {
                qlo[kc][r] = pack2<BF16>(x0 - round16<BF16>(x0), x1 - round16<BF16>(x1));
            }
        }
    }
}

// LOW8: the caller guarantees at most eight query heads per kv head. Rows 8-15 of every MMA are then empty, and the
// query fragments, score and output accumulators of those rows (half of each: 64 registers with value + residual
// queries and head_dim 128) are not kept at all.
template <int D, int HPC, bool QSPLIT, bool BF16, bool FUSED, bool LOW8 = false>
__device__ __forceinline__ void decode_split_body(const DecodeParams& p, unsigned char* smem) {
    constexpr int TS = kConsumerWarps / HPC;     // row sub-tiles per kv head
    constexpr int TT = 16 * TS;                  // rows per tile
    constexpr int ROWB = HPC * D * 2;            // bytes of one cache row slice (HPC kv heads)
    constexpr int PITCH = ROWB + 16;             // shared-memory row pitch
    constexpr int TILEB = TT * PITCH;            // one K (or V) tile
    constexpr int KC = D / 16;                   // k-chunks of the QK^T contraction
    constexpr int DN = D / 8;                    // n-tiles of the PV product

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const uint32_t nst = p.nstages;
    const uint32_t nseg = p.batch * p.head_groups;

    unsigned char* tiles = smem;
    // layout behind the tile ring: the query rows of the running segment (HPC*G rows of D elements, room for 4 bytes
    // each; 16-byte aligned like the tiles, as a bulk copy needs), barriers [3*nst + 2], the tile prefix [nseg + 1]
    // and two words of the single-launch mode (the arrival ticket carried from thread 0 to the other warps, and the
    // "a wait ran out somewhere in this CTA" mark)
    unsigned char* q_smem = smem + static_cast<size_t>(nst) * 2 * TILEB;
    uint64_t* bars = reinterpret_cast<uint64_t*>(q_smem + static_cast<size_t>(HPC) * p.group * D * 4);
    uint32_t* prefix = reinterpret_cast<uint32_t*>(bars + 3 * nst + 2);
    volatile uint32_t* s_ticket = prefix + nseg + 1;
    volatile uint32_t* s_abort = prefix + nseg + 2;
    const uint32_t bar_full_k = smem_u32(bars);
    const uint32_t bar_full_v = bar_full_k + 8 * nst;
    const uint32_t bar_empty = bar_full_v + 8 * nst;
    const uint32_t bar_q_full = bar_empty + 8 * nst;
    const uint32_t bar_q_empty = bar_q_full + 8;
    const uint32_t tiles_u32 = smem_u32(tiles);
    const uint32_t q_esize = p.q_dtype == ATTN_DTYPE_F32 ? 4u : 2u;
    const uint32_t q_seg_bytes = HPC * p.group * D * q_esize;  // the query rows of one segment are contiguous in q

#ifdef ATTN_TRACE
#define DTRACE(k) ATTN_TRACE_AT(p.trace ? p.trace + static_cast<size_t>(blockIdx.x) * 8 : nullptr, k)
#else
#define DTRACE(k) \
    do {          \
    } while (0)
#endif
    if (tid == 0) DTRACE(0);
    // The merge pass may be scheduled as soon as every CTA got here; it waits for
    // this grid to finish before reading the partials.
    grid_dep_launch_dependents();

    // Set-up that reads nothing another kernel writes runs while the previous kernel of the stream may still be
    // finishing.
    if (tid == 0) {
        for (uint32_t s = 0; s < nst; ++s) {
            mbar_init(bar_full_k + 8 * s, 1);
            mbar_init(bar_full_v + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, kConsumerWarps);
        }
        mbar_init(bar_q_full, 1);
        mbar_init(bar_q_empty, kConsumerWarps);
        mbar_init_fence();
        if constexpr (FUSED) *s_abort = 0u;
    }
    // This grid waits for the kernel before it (which wrote q, the newest cache row and possibly the lengths) before
    // it reads any of them. With kv_early the caller vouches that the lengths were in place before that kernel was
    // launched and that the only cache row it writes is each sequence's last valid one: the wait then moves behind the
    // tile prefix, and the producer warp starts the tiles that cannot hold that row before it waits (below), so the
    // first K/V bytes are already on their way while the previous kernel finishes.
    // With uniform lengths (no length array to wait for) the wait moves behind the tile arithmetic in the same way.
    // (Tried there and dropped: asking L2 for the CTA's first tiles with bulk prefetches before the wait. In a chain of
    // decode steps it made the step 3 us slower, 48.0 -> 51.0 us at batch 16 x 4096 rows: the hints compete for HBM
    // with the previous step's slowest CTAs instead of filling a gap.)
    const bool early = p.kv_early != 0;
    const bool deferred = early || p.kv_len == nullptr;
    if (!deferred) grid_dep_wait();
    if (tid == 0) DTRACE(1);

    // ---- tile prefix over segments (ragged lengths only) --------------------
    uint64_t nt;
    uint32_t tiles_uniform = 0;
    if (p.kv_len) {
        for (uint32_t s = tid; s < nseg; s += kThreads) {
            const uint32_t stated = p.kv_len[s / p.head_groups];
            const uint32_t len = clamped_len(stated, p.kv_capacity);
            if (len != stated && blockIdx.x == 0 && p.status) atomicOr(p.status, ATTN_STATUS_BAD_SHAPE);
            prefix[s + 1] = (len + TT - 1) / TT;
        }
        if (tid == 0) prefix[0] = 0;
        __syncthreads();
        if (warp == 0) {
            uint32_t carry = 0;
            for (uint32_t base = 0; base < nseg; base += 32) {
                uint32_t i = base + lane;
                uint32_t x = (i < nseg) ? prefix[i + 1] : 0;
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    uint32_t y = __shfl_up_sync(0xffffffffu, x, off);
                    if (lane >= off) x += y;
                }
                x += carry;
                if (i < nseg) prefix[i + 1] = x;
                carry = __shfl_sync(0xffffffffu, x, 31);
            }
        }
        __syncthreads();
        nt = prefix[nseg];
        if (blockIdx.x == 0 && p.seg_prefix) {
            if (early) grid_dep_wait();  // the previous kernel may still be reading the old table
            for (uint32_t s = tid; s <= nseg; s += kThreads) p.seg_prefix[s] = prefix[s];
        }
    } else {
        tiles_uniform = (clamped_len(p.kv_len_uniform, p.kv_capacity) + TT - 1) / TT;
        nt = static_cast<uint64_t>(tiles_uniform) * nseg;
        __syncthreads();
    }
    if (nt == 0) return;
    if (tid == 0) DTRACE(2);

    const uint32_t active = active_ctas(gridDim.x, p.max_ctas, p.min_tiles_per_cta, nt);
    const uint32_t cta = blockIdx.x;
    if (cta >= active) return;
    const uint32_t t_begin = static_cast<uint32_t>(static_cast<uint64_t>(cta) * nt / active);
    const uint32_t t_end = static_cast<uint32_t>(static_cast<uint64_t>(cta + 1) * nt / active);
    const uint32_t n_my = t_end - t_begin;
    if (n_my == 0) return;

    SegTable<TT> table{p, prefix, tiles_uniform};
    SegInfo seg = table.load(table.find(t_begin, nseg));

    if (warp == kConsumerWarps) {
        // ===================== producer warp =====================
        const uint64_t policy = l2_policy_evict_first();
        const uint64_t q_policy = l2_policy_evict_last();  // a segment's query rows are read by every CTA that shares it
        uint32_t q_seg = 0xffffffffu, n_seg = 0;           // segment whose query rows were requested last; segments so far

        // One K tile and one V tile of `seg` into ring stage i % nst: a bulk copy per cache row.
        auto issue_tile = [&](uint32_t i, uint32_t gt) {
            const uint32_t st = i % nst;
            const uint32_t tok0 = (gt - seg.tile0) * TT;
            const size_t seq_off = static_cast<size_t>(seg.b) * p.kv_batch_stride + static_cast<size_t>(seg.hg) * (HPC * D);
            const uint32_t kdst = tiles_u32 + st * 2 * TILEB;
            const uint32_t vdst = kdst + TILEB;
            if (lane == 0) {
                mbar_arrive_expect_tx(bar_full_k + 8 * st, TT * ROWB);
                mbar_arrive_expect_tx(bar_full_v + 8 * st, TT * ROWB);
            }
            __syncwarp();
            // Rows past the end of the sequence re-read its last valid row: the
            // tile is always full (constant byte count) and always finite; those
            // rows are masked to probability zero by the consumers.
#pragma unroll
            for (int j = lane; j < TT; j += 32) {
                uint32_t row = tok0 + j;
                row = row < seg.len ? row : seg.len - 1;
                const uint16_t* src = p.k + seq_off + static_cast<size_t>(row) * p.kv_row_stride;
                bulk_g2s(kdst + j * PITCH, src, ROWB, bar_full_k + 8 * st, policy);
            }
#pragma unroll
            for (int j = lane; j < TT; j += 32) {
                uint32_t row = tok0 + j;
                row = row < seg.len ? row : seg.len - 1;
                const uint16_t* src = p.v + seq_off + static_cast<size_t>(row) * p.kv_row_stride;
                bulk_g2s(vdst + j * PITCH, src, ROWB, bar_full_v + 8 * st, policy);
            }
        };
        // The query rows of `seg` into their buffer (the previous segment's must have been taken).
        auto issue_q = [&]() -> bool {
            if (n_seg > 0 && !mbar_wait(bar_q_empty, (n_seg - 1) & 1)) {
                if (lane == 0 && p.status) atomicOr(p.status, ATTN_STATUS_WAIT_TIMEOUT);
                return false;
            }
            if (lane == 0) {
                const unsigned char* src = reinterpret_cast<const unsigned char*>(p.q) +
                    (static_cast<size_t>(seg.b) * p.n_heads + static_cast<size_t>(seg.hg) * HPC * p.group) * D * q_esize;
                mbar_arrive_expect_tx(bar_q_full, q_seg_bytes);
                bulk_g2s(smem_u32(q_smem), src, q_seg_bytes, bar_q_full, q_policy);
            }
            q_seg = seg.seg;
            ++n_seg;
            return true;
        };

        uint32_t i = 0;
        if (early) {
            // Fill the ring before waiting for the previous kernel, stopping in front of a segment's last tile (the
            // one that holds the row that kernel may be writing); a segment boundary is therefore never crossed here.
            for (; i < n_my && i < nst; ++i) {
                const uint32_t gt = t_begin + i;
                if (gt + 1 >= seg.tile_end) break;
                issue_tile(i, gt);
            }
            grid_dep_wait();
            if (i > 0 && !issue_q()) return;  // the running segment's query rows, which that kernel produced
        } else if (deferred) {
            grid_dep_wait();
        }
        for (; i < n_my; ++i) {
            const uint32_t gt = t_begin + i;
            while (gt >= seg.tile_end) seg = table.load(seg.seg + 1);
            // The query rows travel in front of the segment's first tile, on the same copy engine: they land before the
            // tile does, instead of queueing (as loads issued by the consumer warps did, for several microseconds)
            // behind three stages of K/V traffic. One buffer: the consumers copy it into registers at the start of
            // the segment and release it at once.
            if (seg.seg != q_seg && !issue_q()) return;
            if (i >= nst) {
                if (!mbar_wait(bar_empty + 8 * (i % nst), ((i / nst) - 1) & 1)) {
                    if (lane == 0 && p.status) atomicOr(p.status, ATTN_STATUS_WAIT_TIMEOUT);
                    return;
                }
            }
            issue_tile(i, gt);
        }
        if (lane == 0) DTRACE(7);
        return;
    }

    // ===================== consumer warps =====================
    // (No setmaxnreg here: with nine warps, warps 0, 4 and 8 share one of the SM's four register files of 512
    // registers per lane, 3 x 168 of which are taken at launch; an increase for the consumer warpgroups can never be
    // granted and the instruction would wait for ever.)
    if (deferred) grid_dep_wait();   // before the first partial is written and the query rows are used
    const int hh = warp / TS;        // kv head within the head group
    const int ts = warp - hh * TS;   // row sub-tile
    const int gq = lane >> 2;        // MMA row owned by this lane (and gq + 8)
    const int cq = lane & 3;
    const uint32_t G = p.group;
    const bool ghi = !LOW8 && G > 8;  // rows 8..15 of the MMA hold real heads

    // per-lane ldmatrix row addresses inside a tile (stage base added per tile)
    const uint32_t k_lane_off = (ts * 16 + ((lane >> 4) << 3) + (lane & 7)) * PITCH + hh * (D * 2) + (((lane >> 3) & 1) << 4);
    const uint32_t v_lane_off = (ts * 16 + (((lane >> 3) & 1) << 3) + (lane & 7)) * PITCH + hh * (D * 2) + ((lane >> 4) << 4);

    uint32_t qhi[KC][4];
    uint32_t qlo[QSPLIT ? KC : 1][4];
    float o[DN][4];
    float m0, m1, l0, l1;  // running max (scaled, log2 domain) and sum for rows gq, gq + 8

    uint32_t n_seg = 0;  // segments this CTA has started (parity of the query-row barriers)
    bool failed = false;
    // What a warp does when one of its bounded waits runs out: two-pass mode has no barrier after this point, so the
    // warp simply leaves (its partials are missing and the status bit says so); in single-launch mode it stays, see
    // fused_merge below.
    auto wait_failed = [&]() {
        if (lane == 0 && p.status) atomicOr(p.status, ATTN_STATUS_WAIT_TIMEOUT);
        if constexpr (FUSED) {
            *s_abort = 1u;
            failed = true;
        }
    };

    // Returns false when the wait for the query rows ran out.
    auto begin_segment = [&]() -> bool {
        if (!mbar_wait(bar_q_full, n_seg & 1)) {
            wait_failed();
            return false;
        }
        ++n_seg;
        const size_t off = static_cast<size_t>(hh) * G * D;  // this warp's kv head inside the staged rows
        if (p.q_dtype == ATTN_DTYPE_F16) {
            load_q_fragments<__half, KC, QSPLIT, BF16>(reinterpret_cast<const __half*>(q_smem) + off, D, G, gq, cq, ghi, qhi, qlo);
        } else if (p.q_dtype == ATTN_DTYPE_F32) {
            load_q_fragments<float, KC, QSPLIT, BF16>(reinterpret_cast<const float*>(q_smem) + off, D, G, gq, cq, ghi, qhi, qlo);
        } else {
            load_q_fragments<__nv_bfloat16, KC, QSPLIT, BF16>(reinterpret_cast<const __nv_bfloat16*>(q_smem) + off, D, G, gq,
                                                              cq, ghi, qhi, qlo);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_q_empty);
#pragma unroll
        for (int dn = 0; dn < DN; ++dn) {
            o[dn][0] = o[dn][1] = o[dn][2] = o[dn][3] = 0.f;
        }
        m0 = m1 = -INFINITY;
        l0 = l1 = 0.f;
        return true;
    };

    auto end_segment = [&]() {
        // quad-reduce the row sums, normalise, write this warp's partial
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
        const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f;
        const float inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
        const size_t slot = (static_cast<size_t>(cta) + seg.seg) * TS + ts;
        const size_t row0 = (slot * HPC + hh) * G;
#ifdef ATTN_BOUNDS_CHECK
        if (row0 + G > p.part_rows) {  // the slot arithmetic left the workspace: record it, write nothing
            if (lane == 0 && p.status) atomicOr(p.status, ATTN_STATUS_BAD_INDEX);
            return;
        }
#endif
        constexpr float kLn2 = 0.6931471805599453f;
        if (gq < static_cast<int>(G)) {
            float* dst = p.part_o + (row0 + gq) * D + cq * 2;
#pragma unroll
            for (int dn = 0; dn < DN; ++dn) {
                *reinterpret_cast<float2*>(dst + dn * 8) = make_float2(o[dn][0] * inv0, o[dn][1] * inv0);
            }
            if (cq == 0) p.part_lse[row0 + gq] = l0 > 0.f ? (m0 + log2f(l0)) * kLn2 : -INFINITY;
        }
        if (ghi && gq + 8 < static_cast<int>(G)) {
            float* dst = p.part_o + (row0 + gq + 8) * D + cq * 2;
#pragma unroll
            for (int dn = 0; dn < DN; ++dn) {
                *reinterpret_cast<float2*>(dst + dn * 8) = make_float2(o[dn][2] * inv1, o[dn][3] * inv1);
            }
            if (cq == 0) p.part_lse[row0 + gq + 8] = l1 > 0.f ? (m1 + log2f(l1)) * kLn2 : -INFINITY;
        }
    };

    // Single-launch mode: the CTAs that deliver the last partials merge. No CTA ever waits for another: each one adds
    // 1 to a counter after its partials are visible, and whoever sees the final count does the merging and puts the
    // counter back to zero. A segment shared by few CTAs has one counter and one merge. A segment shared by many (one
    // long sequence: a single CTA would take tens of microseconds to read every partial) is merged in two levels:
    // consecutive CTAs form groups of gs ~ sqrt(CTAs / TS), the last CTA of a group to arrive merges the group's
    // gs * TS partials into one group record, then counts itself on the segment's counter, and the last group merges
    // the records - two short rounds of loads on different SMs in place of one long one.
    // A consumer warp whose bounded wait ran out does not leave: it marks the CTA as aborted, stops computing and keeps
    // walking the tile list so that it still meets the other warps at the named barriers below. An aborted CTA
    // raises the status bit BEFORE it takes its ticket, and a CTA that takes a last ticket reads the status word
    // AFTER: every merge is skipped (output untouched, counters back to zero) whenever a partial is missing.
    auto fused_merge = [&]() {
        if constexpr (FUSED) {
            constexpr uint32_t kOneLevelMax = 32;  // partials that one merge reads in four rounds of loads
            __threadfence();
            asm volatile("bar.sync 1, 256;" ::: "memory");
            const uint32_t c_first = cta_of_tile(seg.tile0, nt, active);
            const uint32_t c_last = cta_of_tile(seg.tile_end - 1, nt, active);
            const uint32_t nc = c_last - c_first + 1;  // CTAs that share the segment
            const uint32_t R = HPC * G;                // output rows of the segment = rows of one partial record
            const bool two_level = p.group_counters != nullptr && nc * TS > kOneLevelMax;
            uint32_t gs = nc, gi = 0, ng = 1;
            if (two_level) {
                gs = static_cast<uint32_t>(sqrtf(static_cast<float>(nc) / TS) + 0.5f);
                gs = gs < 2 ? 2 : gs;
                gi = (cta - c_first) / gs;
                ng = (nc + gs - 1) / gs;
            }
            const uint32_t gsz = nc - gi * gs < gs ? nc - gi * gs : gs;  // CTAs in this CTA's group
            // groups are disjoint CTA ranges and a CTA is shared by at most two consecutive segments, so (first CTA of
            // the group + segment) numbers the groups of the whole launch without collisions, below grid + nseg
            const size_t group_slot = static_cast<size_t>(c_first) + gi * gs + seg.seg;
#ifdef ATTN_BOUNDS_CHECK
            if (two_level && group_slot >= p.group_slots) {  // the group arithmetic left the workspace: record, do nothing
                if (tid == 0 && p.status) atomicOr(p.status, ATTN_STATUS_BAD_INDEX);
                return;
            }
#endif
            uint32_t* counter = two_level ? p.group_counters + group_slot : p.counters + seg.seg;
            auto take_ticket = [&](uint32_t* c) {
                if (tid == 0) {
                    if (*s_abort) {
                        if (p.status) atomicOr(p.status, ATTN_STATUS_WAIT_TIMEOUT);
                        __threadfence();
                    }
                    *s_ticket = atomicAdd(c, 1u);
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");
                return *s_ticket;
            };
            auto poisoned = [&]() {
                __threadfence();
                return *s_abort ||
                       (p.status && (*reinterpret_cast<volatile uint32_t*>(p.status) & ATTN_STATUS_WAIT_TIMEOUT));
            };
            const size_t out_row0 = static_cast<size_t>(seg.b) * p.n_heads + static_cast<size_t>(seg.hg) * R;
            auto store_final = [&](uint32_t r, uint32_t f, float4 v, float lse) {
                const size_t idx = (out_row0 + r) * D + f * 4;
                if (p.o_dtype == ATTN_DTYPE_F32) {
                    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.o) + idx) = v;
                } else {
                    store_out(p.o, p.o_dtype, idx, v.x);
                    store_out(p.o, p.o_dtype, idx + 1, v.y);
                    store_out(p.o, p.o_dtype, idx + 2, v.z);
                    store_out(p.o, p.o_dtype, idx + 3, v.w);
                }
                if (p.lse && f == 0) p.lse[out_row0 + r] = lse;
            };
            if (take_ticket(counter) != gsz - 1) return;
            // this CTA delivered the last partial of its group (one level: of the segment)
            const size_t first_slot = (static_cast<size_t>(c_first) + gi * gs + seg.seg) * TS;
            const float* src_o = p.part_o + first_slot * R * D;
            const float* src_l = p.part_lse + first_slot * R;
            if (!two_level) {
                if (!poisoned()) cta_merge_rows<D>(src_o, src_l, static_cast<uint64_t>(R) * D, R, nc * TS, R, tid, store_final);
                if (tid == 0) *counter = 0u;
                return;
            }
            if (!poisoned()) {
                float* rec_o = p.group_o + group_slot * R * D;
                float* rec_l = p.group_lse + group_slot * R;
                cta_merge_rows<D>(src_o, src_l, static_cast<uint64_t>(R) * D, R, gsz * TS, R, tid,
                                  [&](uint32_t r, uint32_t f, float4 v, float lse) {
                                      *reinterpret_cast<float4*>(rec_o + static_cast<size_t>(r) * D + f * 4) = v;
                                      if (f == 0) rec_l[r] = lse;
                                  });
            }
            if (tid == 0) *counter = 0u;
            __threadfence();
            asm volatile("bar.sync 1, 256;" ::: "memory");  // every thread's record stores before the ticket
            if (take_ticket(p.counters + seg.seg) != ng - 1) return;
            // this group's record was the segment's last: records of group k at slot (c_first + seg) + k * gs
            if (!poisoned()) {
                const size_t rec0 = static_cast<size_t>(c_first) + seg.seg;
                cta_merge_rows<D>(p.group_o + rec0 * R * D, p.group_lse + rec0 * R, static_cast<uint64_t>(gs) * R * D,
                                  static_cast<uint64_t>(gs) * R, ng, R, tid, store_final);
            }
            if (tid == 0) p.counters[seg.seg] = 0u;
        }
    };

    if (!begin_segment()) {
        if constexpr (!FUSED) return;
    }
    if (warp == 0 && lane == 0) DTRACE(3);

    for (uint32_t i = 0; i < n_my; ++i) {
        const uint32_t gt = t_begin + i;
        if (gt >= seg.tile_end) {
            if (!failed) end_segment();
            fused_merge();
            do { seg = table.load(seg.seg + 1); } while (gt >= seg.tile_end);
            if (!failed && !begin_segment()) {
                if constexpr (!FUSED) return;
            }
        }
        if constexpr (FUSED) {
            if (failed) continue;
        }
        const uint32_t st = i % nst;
        const uint32_t par = (i / nst) & 1;
        const uint32_t kbase = tiles_u32 + st * 2 * TILEB;
        const uint32_t vbase = kbase + TILEB;

        if (!mbar_wait(bar_full_k + 8 * st, par)) {
            wait_failed();
            if constexpr (FUSED) continue; else return;
        }
        if (i == 0 && warp == 0 && lane == 0) DTRACE(4);

        // ---- S = Q K^T : 16 (heads) x 16 (rows of this sub-tile) ----
        float s[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
        for (int kc = 0; kc < KC; ++kc) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(b0, b1, b2, b3, kbase + k_lane_off + kc * 32);
            if constexpr (LOW8) {
                mma_16816_low8<BF16>(s[0][0], s[0][1], qhi[kc][0], qhi[kc][2], b0, b1);
                mma_16816_low8<BF16>(s[1][0], s[1][1], qhi[kc][0], qhi[kc][2], b2, b3);
                if constexpr (QSPLIT) {
                    mma_16816_low8<BF16>(s[0][0], s[0][1], qlo[kc][0], qlo[kc][2], b0, b1);
                    mma_16816_low8<BF16>(s[1][0], s[1][1], qlo[kc][0], qlo[kc][2], b2, b3);
                }
            } else {
                mma_16816<BF16>(s[0], qhi[kc], b0, b1);
                mma_16816<BF16>(s[1], qhi[kc], b2, b3);
                if constexpr (QSPLIT) {
                    mma_16816<BF16>(s[0], qlo[kc], b0, b1);
                    mma_16816<BF16>(s[1], qlo[kc], b2, b3);
                }
            }
        }

        // ---- scale, mask rows past the sequence end ----
        const uint32_t tok = (gt - seg.tile0) * TT + ts * 16 + cq * 2;  // row of s[0][0]; s[1][*] is +8
#pragma unroll
        for (int n = 0; n < 2; ++n) {
#pragma unroll
            for (int e = 0; e < (LOW8 ? 2 : 4); ++e) {
                const uint32_t r = tok + n * 8 + (e & 1);
                s[n][e] = r < seg.len ? s[n][e] * p.scale_log2 : -INFINITY;
            }
        }

        // ---- online softmax (rows gq and gq + 8) ----
        float mx0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        const float mn0 = fmaxf(m0, mx0);
        const float ref0 = mn0 == -INFINITY ? 0.f : mn0;
        const float sc0 = exp2f(m0 - ref0);
        m0 = mn0;
        const float p00 = exp2f(s[0][0] - ref0), p01 = exp2f(s[0][1] - ref0);
        const float p10 = exp2f(s[1][0] - ref0), p11 = exp2f(s[1][1] - ref0);
        l0 = l0 * sc0 + (p00 + p01 + p10 + p11);

        float sc1 = 1.f;
        uint32_t pa[4];
        // P goes to the tensor cores as a 16-bit value plus a 16-bit residual (two MMAs per tile), so the
        // PV product keeps ~2^-22 (fp16) / 2^-17 (bf16) relative accuracy instead of the 2^-11 / 2^-8 of one
        // rounded operand.
        uint32_t pb[4];
        pa[0] = pack2<BF16>(p00, p01);
        pa[2] = pack2<BF16>(p10, p11);
        pb[0] = pack2<BF16>(p00 - round16<BF16>(p00), p01 - round16<BF16>(p01));
        pb[2] = pack2<BF16>(p10 - round16<BF16>(p10), p11 - round16<BF16>(p11));
        if (ghi) {
            float mx1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn1 = fmaxf(m1, mx1);
            const float ref1 = mn1 == -INFINITY ? 0.f : mn1;
            sc1 = exp2f(m1 - ref1);
            m1 = mn1;
            const float q00 = exp2f(s[0][2] - ref1), q01 = exp2f(s[0][3] - ref1);
            const float q10 = exp2f(s[1][2] - ref1), q11 = exp2f(s[1][3] - ref1);
            l1 = l1 * sc1 + (q00 + q01 + q10 + q11);
            pa[1] = pack2<BF16>(q00, q01);
            pa[3] = pack2<BF16>(q10, q11);
            pb[1] = pack2<BF16>(q00 - round16<BF16>(q00), q01 - round16<BF16>(q01));
            pb[3] = pack2<BF16>(q10 - round16<BF16>(q10), q11 - round16<BF16>(q11));
        } else {
            pa[1] = pa[3] = 0u;
            pb[1] = pb[3] = 0u;
        }

        // rescale the accumulator only when some row's maximum moved
        if (__any_sync(0xffffffffu, sc0 != 1.f || sc1 != 1.f)) {
#pragma unroll
            for (int dn = 0; dn < DN; ++dn) {
                o[dn][0] *= sc0;
                o[dn][1] *= sc0;
                if constexpr (!LOW8) {
                    o[dn][2] *= sc1;
                    o[dn][3] *= sc1;
                }
            }
        }

        if (!mbar_wait(bar_full_v + 8 * st, par)) {
            wait_failed();
            if constexpr (FUSED) continue; else return;
        }

        // ---- O += P V : 16 (heads) x D, contraction over this sub-tile's 16 rows ----
#pragma unroll
        for (int d2 = 0; d2 < DN / 2; ++d2) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(b0, b1, b2, b3, vbase + v_lane_off + d2 * 32);
            if constexpr (LOW8) {
                mma_16816_low8<BF16>(o[2 * d2][0], o[2 * d2][1], pa[0], pa[2], b0, b1);
                mma_16816_low8<BF16>(o[2 * d2 + 1][0], o[2 * d2 + 1][1], pa[0], pa[2], b2, b3);
                mma_16816_low8<BF16>(o[2 * d2][0], o[2 * d2][1], pb[0], pb[2], b0, b1);
                mma_16816_low8<BF16>(o[2 * d2 + 1][0], o[2 * d2 + 1][1], pb[0], pb[2], b2, b3);
            } else {
                mma_16816<BF16>(o[2 * d2], pa, b0, b1);
                mma_16816<BF16>(o[2 * d2 + 1], pa, b2, b3);
                mma_16816<BF16>(o[2 * d2], pb, b0, b1);
                mma_16816<BF16>(o[2 * d2 + 1], pb, b2, b3);
            }
        }

        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty + 8 * st);
    }
    if (warp == 0 && lane == 0) DTRACE(5);
    if (!failed) end_segment();
    if (warp == 0 && lane == 0) DTRACE(6);
    fused_merge();
#undef DTRACE
}

}  // namespace decode_detail
}  // namespace b200
