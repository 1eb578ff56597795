// Causal prefill attention for sm_100a on the 5th-generation tensor cores (tcgen05 + tensor memory).
//
// What it computes: for every sequence b, query head h and row t,
//     O[b][t][h] = softmax_{u <= t}( Q[b][t][h] . K[b][u][h / G] * scale ) V[b][u][h / G]
// which is what the engine produces when it runs its single-token forward once per prompt token with
// kv_len = t + 1 (tools/infer.cpp:271-274, src/model/model.cpp:68, attn() of include/kernels_cpu.hpp:140-167).
// The engine has no S x S kernel of its own; the results are pinned by that row-by-row definition.
//
// Layouts (dense, head_dim = 128 or 64, 16-bit elements): Q, O [B][S][H][D]; K, V [B][S][Hkv][D] — the engine's
// cache layout [row][kv_head][head_dim] per sequence.
//
// One CTA = two 128-row query tiles that share one K/V stream (two query heads of the same kv head at the
// same rows when the GQA group is even, else two consecutive row tiles of one head), 12 warps:
//   warps 0-3   softmax of tile 0: thread r owns query row r (tensor-memory lane r), no shuffles needed
//   warps 4-7   softmax of tile 1
//   warp  8     TMA producer: Q tiles once, then K and V tiles (128 keys x 128 dims, 128-byte swizzle)
//               through a 2-stage ring with separate barriers for K and V
//   warp  9     one thread issues every tcgen05.mma: S_t = Q_t K^T (both operands in shared memory,
//               accumulator in tensor memory) and O_t += P_t V (P read from tensor memory, V from shared
//               memory as an MN-major operand), in the order PV_0(j), QK_0(j+1), PV_1(j), QK_1(j+1) so the
//               softmax of one tile overlaps the tensor work of the other
//   warps 10-11 idle (they only take part in the register re-allocation of their warpgroup)
// Tensor memory (512 columns): S_0 | S_1 | O_0 | O_1, 128 fp32 columns each. P overwrites S in place as
// packed 16-bit pairs in columns [0,64). Two ways to hand P to the tensor cores (template PMODE):
//   kPResidual  P in the input type plus its rounding residual in columns [64,128) and a second PV MMA: ~2^-17,
//               the mode that meets the parity tolerance on every row (the default).
//   kPInput     P rounded once to the input type (fp16: 2^-11, bf16: 2^-9 per element), one PV MMA.
// A and B of one MMA must have the same 16-bit format: an fp16 P against a bf16 V (the instruction descriptor has
// separate format fields) raises an illegal-instruction error on this part, so there is no such mode.
// Online softmax follows the engine's state merge (src/attention.cu:41-65): running maximum m, sum l,
// accumulator rescaled by exp(m_old - m_new); the rescale is skipped until the maximum has grown by more
// than 2^8, and the true l normalises at the end, so the result is unchanged.
//
// Every wait is bounded; on expiry the role records ATTN_STATUS_WAIT_TIMEOUT, stops, and the CTA still
// runs its common exit (final barrier, tensor-memory release).
#include <cuda.h>

#include "attn_internal.cuh"
#include "ptx_sm100.cuh"
#include "tma_tile.cuh"

namespace b200 {
namespace {

constexpr int BM = 128;   // query rows per tile
constexpr int BN = 128;   // keys per block
constexpr int kMaxHD = 128;  // head_dim is 128 or 64 (template HDIM); shared memory is laid out for 128
constexpr int kThreads = 384;
constexpr uint32_t kSubTileBytes = 128 * 64 * 2;       // [128 rows][64 elements], 128-byte rows, swizzled
constexpr uint32_t kTileBytes = 2 * kSubTileBytes;     // 128 x 128 16-bit elements (head_dim 64 fills the first half)
constexpr int kStages = 2;
constexpr uint32_t kTmemCols = 512;
#ifdef ATTN_TRACE
float* g_prefill_debug = nullptr;
#endif

struct PrefillParams {
    void* o;
    int32_t o_dtype;
    int32_t in_dtype;  // ATTN_DTYPE_F16 | ATTN_DTYPE_BF16
    uint32_t batch, seq, n_heads, n_kv_heads, group;
    uint32_t m_tiles;     // ceil(seq / 128)
    uint32_t pair_heads;  // 1: tiles are heads (2*hp, 2*hp+1) at the same rows; 0: rows (2*mp, 2*mp+1) of one head
    float scale_log2;
    uint32_t* status;
#ifdef ATTN_TRACE
    float* debug;  // optional [128][128] dump of the first S tile of CTA (0,0,0)
#endif
};

enum : int { kPResidual = 0, kPInput = 1 };

// ---- barriers (8 bytes each) inside shared memory ----
enum {
    BAR_Q_FULL = 0,
    BAR_K_FULL = 1,                   // [kStages]
    BAR_V_FULL = BAR_K_FULL + kStages,
    BAR_K_EMPTY = BAR_V_FULL + kStages,
    BAR_V_EMPTY = BAR_K_EMPTY + kStages,
    BAR_S_FULL = BAR_V_EMPTY + kStages,  // [2] per tile
    BAR_P_FULL = BAR_S_FULL + 2,
    BAR_O_FULL = BAR_P_FULL + 2,
    BAR_COUNT = BAR_O_FULL + 2
};

constexpr uint32_t kSmemQ = 0;
constexpr uint32_t kSmemK = kSmemQ + 2 * kTileBytes;
constexpr uint32_t kSmemV = kSmemK + kStages * kTileBytes;
constexpr uint32_t kSmemStage = kSmemV + kStages * kTileBytes;   // per tile: [128 rows][128 B] output staging
constexpr uint32_t kStageTileBytes = 128 * 128;
constexpr uint32_t kSmemBars = kSmemStage + 2 * kStageTileBytes;
constexpr uint32_t kSmemTmemPtr = kSmemBars + BAR_COUNT * 8;
constexpr uint32_t kSmemTotal = kSmemTmemPtr + 16;
constexpr uint32_t kSmemAlloc = kSmemTotal + 1024;  // slack to align the base to 1024 bytes

// ---- tcgen05 / TMA wrappers ----
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
// Tile store shared -> global through the TMA engine (asynchronous; rows outside the tensor are clipped).
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the shared-memory source of every committed store has been read
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// every committed store is complete
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D(tmem) (+)= A(smem) * B(smem)
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
        : "memory");
}
// D(tmem) (+)= A(tmem) * B(smem)
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&r)[32]) {
    uint32_t* u = reinterpret_cast<uint32_t*>(r);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
        "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
          "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]), "=r"(u[16]),
          "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]), "=r"(u[24]),
          "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&u)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
        "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]), "r"(u[8]),
          "r"(u[9]), "r"(u[10]), "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15]), "r"(u[16]), "r"(u[17]),
          "r"(u[18]), "r"(u[19]), "r"(u[20]), "r"(u[21]), "r"(u[22]), "r"(u[23]), "r"(u[24]), "r"(u[25]), "r"(u[26]),
          "r"(u[27]), "r"(u[28]), "r"(u[29]), "r"(u[30]), "r"(u[31])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Packed 16-bit pair -> two floats (exact).
template <bool BF16>
__device__ __forceinline__ void unpack2(uint32_t u, float& a, float& b) {
    if constexpr (BF16) {
        a = __uint_as_float(u << 16);
        b = __uint_as_float(u & 0xffff0000u);
    } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u));
        a = f.x;
        b = f.y;
    }
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(lbo_bytes >> 4) << 16) |
           (static_cast<uint64_t>(sbo_bytes >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor of kind::f16: fp32 accumulate, A format a_fmt and B format b_fmt (0 = f16, 1 = bf16; always
// given the same value here), A K-major, B K-major (b_mn = 0) or MN-major (b_mn = 1), M = 128, N = n.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t a_fmt, uint32_t b_fmt, uint32_t b_mn, uint32_t n) {
    return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | (b_mn << 16) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

__device__ __forceinline__ void report_timeout(uint32_t* status) {
    if (status) atomicOr(status, ATTN_STATUS_WAIT_TIMEOUT);
}

template <bool BF16, int PMODE, int HDIM>
__global__ void __launch_bounds__(kThreads, 1)
prefill_causal_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                      const __grid_constant__ PrefillParams p) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* smem = smem_raw + (base - raw);
    const uint32_t bars = base + kSmemBars;
    auto bar = [&](int i) { return bars + 8u * i; };
    volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + kSmemTmemPtr);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    constexpr int HD = HDIM;
    constexpr uint32_t kLoadBytes = (HD / 64) * kSubTileBytes;  // bytes of one Q / K / V tile actually loaded

    // ---- which two tiles does this CTA own ----
    // The row-tile index is the slowest-varying grid dimension and counts down, so every CTA with the longest
    // causal span is dispatched before any shorter one and the kernel's tail is made of one-block CTAs.
    const uint32_t b = blockIdx.y;
    uint32_t head[2], m0[2];
    if (p.pair_heads) {
        const uint32_t mt = p.m_tiles - 1 - blockIdx.z;
        head[0] = 2 * blockIdx.x;
        head[1] = 2 * blockIdx.x + 1;
        m0[0] = m0[1] = mt * BM;
    } else {
        const uint32_t pairs = (p.m_tiles + 1) / 2;
        const uint32_t mp = pairs - 1 - blockIdx.z;
        head[0] = head[1] = blockIdx.x;
        m0[0] = (2 * mp) * BM;
        m0[1] = (2 * mp + 1) * BM;
    }
    const uint32_t kvh = head[0] / p.group;
    const uint32_t nblk_total = (p.seq + BN - 1) / BN;
    uint32_t nblk[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        nblk[t] = m0[t] < p.seq ? min(nblk_total, m0[t] / BN + 1) : 0u;
    }
    const uint32_t n_iter = max(nblk[0], nblk[1]);

    // ---- set-up: barriers, tensor memory ----
    if (tid == 0) {
        mbar_init(bar(BAR_Q_FULL), 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar(BAR_K_FULL + s), 1);
            mbar_init(bar(BAR_V_FULL + s), 1);
            mbar_init(bar(BAR_K_EMPTY + s), 1);
            mbar_init(bar(BAR_V_EMPTY + s), 1);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(bar(BAR_S_FULL + t), 1);
            mbar_init(bar(BAR_P_FULL + t), 128);
            mbar_init(bar(BAR_O_FULL + t), 1);
        }
        mbar_init_fence();
    }
    if (warp == 8) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_smem;
    auto tmem_s = [&](int t) { return tmem_base + static_cast<uint32_t>(t) * 128u; };
    auto tmem_o = [&](int t) { return tmem_base + 256u + static_cast<uint32_t>(t) * 128u; };

    if (warp < 8) {
        // =============================== softmax warpgroups ===============================
        asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
        const int t = warp >> 2;                       // tile
        const int r = ((warp & 3) << 5) | lane;        // row inside the tile = tensor-memory lane
        const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) << 5) << 16;
        const uint32_t q_row = m0[t] + r;              // row index inside the sequence
        float m_used = -INFINITY;                      // maximum the stored probabilities are relative to (log2 units)
        float l = 0.f;
        bool ok = true;
        for (uint32_t j = 0; j < nblk[t] && ok; ++j) {
            if (!mbar_wait(bar(BAR_S_FULL + t), j & 1)) { report_timeout(p.status); ok = false; break; }
            tc_fence_after();
            float s[128];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                tmem_ld32(tmem_s(t) + lane_addr + c * 32, *reinterpret_cast<float(*)[32]>(&s[c * 32]));
            }
            tmem_wait_ld();
#ifdef ATTN_TRACE
            if (p.debug && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == gridDim.z - 1 && t == 0 && j == 0) {
#pragma unroll
                for (int c = 0; c < 128; ++c) p.debug[r * 128 + c] = s[c];
            }
#endif
            // causal mask: only the diagonal block needs it (keys of later blocks are never visited)
            if (j * BN + BN - 1 > q_row) {
#pragma unroll
                for (int c = 0; c < 128; ++c) {
                    if (j * BN + c > q_row) s[c] = -INFINITY;
                }
            }
            // eight independent chains, then a tree: a single chain of 127 dependent max operations would
            // leave this warp's scheduler idle most of the time (only two softmax warps share a scheduler)
            float mx8[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) mx8[i] = s[i];
#pragma unroll
            for (int c = 8; c < 128; ++c) mx8[c & 7] = fmaxf(mx8[c & 7], s[c]);
            float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])),
                             fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
            mx *= p.scale_log2;
            // Rescale only when the maximum grew by more than 8 (probabilities stay below 2^8).
            float factor = 1.f;
            if (mx > m_used + 8.f) {
                factor = fast_exp2(m_used - mx);  // 0 on the first block (m_used = -inf)
                m_used = mx;
            }
            if (j > 0 && __any_sync(0xffffffffu, factor != 1.f)) {
                // O_t is stable here: the MMA that produced this S tile was issued after PV_t(j-1)
                // and the tensor pipe completes in order.
#pragma unroll
                for (int c = 0; c < HD / 32; ++c) {
                    float o[32];
                    tmem_ld32(tmem_o(t) + lane_addr + c * 32, o);
                    tmem_wait_ld();
                    uint32_t u[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) u[i] = __float_as_uint(o[i] * factor);
                    tmem_st32(tmem_o(t) + lane_addr + c * 32, u);
                }
            }
            l *= factor;
            // probabilities; P overwrites S in place (every S value of this row is already in registers)
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t hi[16], lo[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float p0 = fast_exp2(fmaf(s[c * 32 + 2 * i], p.scale_log2, -m_used));
                    const float p1 = fast_exp2(fmaf(s[c * 32 + 2 * i + 1], p.scale_log2, -m_used));
                    sum4[i & 3] += p0 + p1;
                    // Rounded pair by one packed convert; its fp32 value is recovered with integer / half-add
                    // operations so that no scalar convert (special-function pipe, already busy with exp2) is used.
                    hi[i] = pack2<BF16>(p0, p1);
                    if constexpr (PMODE == kPResidual) {
                        float h0, h1;
                        unpack2<BF16>(hi[i], h0, h1);
                        lo[i] = pack2<BF16>(p0 - h0, p1 - h1);
                    }
                }
                // 32 keys -> 16 packed columns: rounded part at column 16c, residual at 64 + 16c
                asm volatile(
                    "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                    ::"r"(tmem_s(t) + lane_addr + c * 16), "r"(hi[0]), "r"(hi[1]), "r"(hi[2]), "r"(hi[3]), "r"(hi[4]),
                      "r"(hi[5]), "r"(hi[6]), "r"(hi[7]), "r"(hi[8]), "r"(hi[9]), "r"(hi[10]), "r"(hi[11]), "r"(hi[12]),
                      "r"(hi[13]), "r"(hi[14]), "r"(hi[15])
                    : "memory");
                if constexpr (PMODE == kPResidual) {
                    asm volatile(
                        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                        ::"r"(tmem_s(t) + lane_addr + 64 + c * 16), "r"(lo[0]), "r"(lo[1]), "r"(lo[2]), "r"(lo[3]),
                          "r"(lo[4]), "r"(lo[5]), "r"(lo[6]), "r"(lo[7]), "r"(lo[8]), "r"(lo[9]), "r"(lo[10]), "r"(lo[11]),
                          "r"(lo[12]), "r"(lo[13]), "r"(lo[14]), "r"(lo[15])
                        : "memory");
                }
            }
            l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar(BAR_P_FULL + t));
        }
        // ---- epilogue: O / l -> global ----
        if (ok && nblk[t] > 0) {
            if (!mbar_wait(bar(BAR_O_FULL + t), 0)) {
                report_timeout(p.status);
            } else {
                tc_fence_after();
                const float inv = l > 0.f ? 1.f / l : 0.f;
                // The tile leaves through shared memory and the TMA engine, 128 bytes of every row per pass: each
                // thread writes its row's 16-byte chunks XOR-swizzled by the row (the 128-byte swizzle the tensor
                // map expects; no bank conflicts), the four warps of the tile meet, and one thread issues the bulk
                // store, which also clips rows past the end of the sequence. Plain per-thread global stores (rows
                // are 8 KB apart) would sit in the load/store queue that this SM's MMA and TMA instructions also
                // pass through and stall them while they drain.
                const uint32_t stage = base + kSmemStage + t * kStageTileBytes;
                const bool f32_out = p.o_dtype == ATTN_DTYPE_F32;
                const int passes = f32_out ? HD / 32 : HD / 64;
#pragma unroll
                for (int pass = 0; pass < 4; ++pass) {
                    if (pass < passes) {
                        // 32 accumulator columns at a time (fp32 out: one pass; 16-bit out: half a pass)
                        const int n_ld = f32_out ? 1 : 2;
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            if (h < n_ld) {
                                float o[32];
                                tmem_ld32(tmem_o(t) + lane_addr + (f32_out ? pass * 32 : pass * 64 + h * 32), o);
                                tmem_wait_ld();
#pragma unroll
                                for (int c = 0; c < (8 >> 1) * 2; ++c) {
                                    if (f32_out) {
                                        const uint4 v = make_uint4(__float_as_uint(o[c * 4] * inv), __float_as_uint(o[c * 4 + 1] * inv),
                                                                   __float_as_uint(o[c * 4 + 2] * inv), __float_as_uint(o[c * 4 + 3] * inv));
                                        const uint32_t addr = stage + r * 128 + ((c ^ (r & 7)) << 4);
                                        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
                                    } else if (c < 4) {
                                        uint4 v;
                                        if (p.o_dtype == ATTN_DTYPE_BF16) {
                                            v = make_uint4(pack2<true>(o[c * 8] * inv, o[c * 8 + 1] * inv), pack2<true>(o[c * 8 + 2] * inv, o[c * 8 + 3] * inv),
                                                           pack2<true>(o[c * 8 + 4] * inv, o[c * 8 + 5] * inv), pack2<true>(o[c * 8 + 6] * inv, o[c * 8 + 7] * inv));
                                        } else {
                                            v = make_uint4(pack2<false>(o[c * 8] * inv, o[c * 8 + 1] * inv), pack2<false>(o[c * 8 + 2] * inv, o[c * 8 + 3] * inv),
                                                           pack2<false>(o[c * 8 + 4] * inv, o[c * 8 + 5] * inv), pack2<false>(o[c * 8 + 6] * inv, o[c * 8 + 7] * inv));
                                        }
                                        const int chunk = h * 4 + c;
                                        const uint32_t addr = stage + r * 128 + ((chunk ^ (r & 7)) << 4);
                                        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
                                    }
                                }
                            }
                        }
                        fence_async_smem();
                        named_bar_sync(1 + t, 128);
                        if ((warp & 3) == 0 && lane == 0) {
                            tma_store_4d(&tm_o, stage, pass * (f32_out ? 32 : 64), m0[t], head[t], b);
                            tma_store_commit();
                            tma_store_wait_read();  // the staging tile may be overwritten after this
                        }
                        named_bar_sync(1 + t, 128);
                    }
                }
                if ((warp & 3) == 0 && lane == 0) tma_store_wait_all();
            }
        }
    } else {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
        if (warp == 8 && lane == 0) {
            // =============================== TMA producer ===============================
            uint32_t n_q = 0;
            for (int t = 0; t < 2; ++t) n_q += nblk[t] > 0;
            mbar_arrive_expect_tx(bar(BAR_Q_FULL), n_q * kLoadBytes);
            for (int t = 0; t < 2; ++t) {
                if (nblk[t] == 0) continue;
                const uint32_t dst = base + kSmemQ + t * kTileBytes;
                tma_load_4d(dst, &tm_q, bar(BAR_Q_FULL), 0, m0[t], head[t], b);
                if (HD > 64) tma_load_4d(dst + kSubTileBytes, &tm_q, bar(BAR_Q_FULL), 64, m0[t], head[t], b);
            }
            for (uint32_t j = 0; j < n_iter; ++j) {
                const uint32_t st = j % kStages;
                if (j >= kStages && !mbar_wait(bar(BAR_K_EMPTY + st), ((j / kStages) - 1) & 1)) {
                    report_timeout(p.status);
                    break;
                }
                const uint32_t kdst = base + kSmemK + st * kTileBytes;
                mbar_arrive_expect_tx(bar(BAR_K_FULL + st), kLoadBytes);
                tma_load_4d(kdst, &tm_k, bar(BAR_K_FULL + st), 0, j * BN, kvh, b);
                if (HD > 64) tma_load_4d(kdst + kSubTileBytes, &tm_k, bar(BAR_K_FULL + st), 64, j * BN, kvh, b);
                if (j >= kStages && !mbar_wait(bar(BAR_V_EMPTY + st), ((j / kStages) - 1) & 1)) {
                    report_timeout(p.status);
                    break;
                }
                const uint32_t vdst = base + kSmemV + st * kTileBytes;
                mbar_arrive_expect_tx(bar(BAR_V_FULL + st), kLoadBytes);
                tma_load_4d(vdst, &tm_v, bar(BAR_V_FULL + st), 0, j * BN, kvh, b);
                if (HD > 64) tma_load_4d(vdst + kSubTileBytes, &tm_v, bar(BAR_V_FULL + st), 64, j * BN, kvh, b);
            }
        } else if (warp == 9 && lane == 0 && n_iter > 0) {
            // =============================== MMA issuer ===============================
            constexpr uint32_t fmt = BF16 ? 1u : 0u;
            constexpr uint32_t idesc_qk = instr_desc(fmt, fmt, 0, BN);  // S: 128 rows x 128 keys
            constexpr uint32_t idesc_pv = instr_desc(fmt, fmt, 1, HD);  // O: 128 rows x head_dim
            // S_t = Q_t K^T: 8 MMAs of K = 16 over head_dim; operands K-major, 128-byte swizzle, 8-row groups 1024 B apart
            auto issue_qk = [&](int t, uint32_t st) {
                const uint32_t qa = base + kSmemQ + t * kTileBytes;
                const uint32_t ka = base + kSmemK + st * kTileBytes;
#pragma unroll
                for (int kc = 0; kc < HD / 16; ++kc) {
                    const uint32_t off = (kc >> 2) * kSubTileBytes + (kc & 3) * 32;
                    mma_ss(tmem_s(t), smem_desc(qa + off, 16, 1024), smem_desc(ka + off, 16, 1024), idesc_qk, kc > 0);
                }
                tc_commit(bar(BAR_S_FULL + t));
            };
            // O_t += P_t V: 8 MMAs of K = 16 keys; A = P in tensor memory (8 packed columns per MMA), B = V as an
            // MN-major operand: 64-dim halves 16 KB apart (leading offset), 8-key groups 1024 B apart (stride offset)
            auto issue_pv = [&](int t, uint32_t st, bool accumulate) {
                const uint32_t va = base + kSmemV + st * kTileBytes;
#pragma unroll
                for (int kc = 0; kc < BN / 16; ++kc) {
                    mma_ts(tmem_o(t), tmem_s(t) + kc * 8, smem_desc(va + kc * 2048, kSubTileBytes, 1024), idesc_pv,
                           accumulate || kc > 0);
                }
                if constexpr (PMODE == kPResidual) {
#pragma unroll
                    for (int kc = 0; kc < BN / 16; ++kc) {
                        mma_ts(tmem_o(t), tmem_s(t) + 64 + kc * 8, smem_desc(va + kc * 2048, kSubTileBytes, 1024),
                               idesc_pv, 1);
                    }
                }
            };
            bool ok = mbar_wait(bar(BAR_Q_FULL), 0) && mbar_wait(bar(BAR_K_FULL + 0), 0);
            if (!ok) report_timeout(p.status);
            if (ok) {
                tc_fence_after();
                for (int t = 0; t < 2; ++t)
                    if (nblk[t] > 0) issue_qk(t, 0);
                tc_commit(bar(BAR_K_EMPTY + 0));
            }
            for (uint32_t j = 0; j < n_iter && ok; ++j) {
                const uint32_t st = j % kStages;
                if (!mbar_wait(bar(BAR_V_FULL + st), (j / kStages) & 1)) { report_timeout(p.status); ok = false; break; }
                bool k_next_ready = false;
                for (int t = 0; t < 2 && ok; ++t) {
                    if (j >= nblk[t]) continue;
                    if (!mbar_wait(bar(BAR_P_FULL + t), j & 1)) { report_timeout(p.status); ok = false; break; }
                    tc_fence_after();
                    issue_pv(t, st, j > 0);
                    if (j + 1 < nblk[t]) {
                        const uint32_t st1 = (j + 1) % kStages;
                        if (!k_next_ready) {
                            if (!mbar_wait(bar(BAR_K_FULL + st1), ((j + 1) / kStages) & 1)) {
                                report_timeout(p.status);
                                ok = false;
                                break;
                            }
                            tc_fence_after();
                            k_next_ready = true;
                        }
                        issue_qk(t, st1);
                    } else {
                        tc_commit(bar(BAR_O_FULL + t));
                    }
                }
                if (!ok) break;
                tc_commit(bar(BAR_V_EMPTY + st));
                if (j + 1 < n_iter) tc_commit(bar(BAR_K_EMPTY + (j + 1) % kStages));
            }
        }
    }

    // ---- common exit: everybody meets, then the allocating warp releases tensor memory ----
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------------------------------------------ host
// [B][S][heads][head_dim] tensor viewed as (dim, row, head, batch); box = 128 bytes of 128 rows, 128-byte swizzle.
int make_map(CUtensorMap* map, const void* ptr, int32_t dtype, uint32_t batch, uint32_t seq, uint32_t heads,
             uint32_t HD) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return ATTN_ERR_CUDA;
    const cuuint64_t esz = dtype == ATTN_DTYPE_F32 ? 4 : 2;
    const cuuint64_t dims[4] = {HD, seq, heads, batch};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(heads) * HD * esz, static_cast<cuuint64_t>(HD) * esz,
                                   static_cast<cuuint64_t>(seq) * heads * HD * esz};
    const cuuint32_t box[4] = {static_cast<cuuint32_t>(128 / esz), BM, 1, 1};  // 128-byte rows
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUtensorMapDataType dt = dtype == ATTN_DTYPE_F32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : dtype == ATTN_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                              : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUresult r = enc(map, dt,
                     4, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        g_last_cuda_error = static_cast<int>(r);
        return ATTN_ERR_CUDA;
    }
    return ATTN_OK;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int attn_prefill_causal(const AttnPrefillArgs* a, void* stream_v) {
    if (!a || !a->o || !a->q || !a->k || !a->v) return ATTN_ERR_INVALID_ARG;
    if (a->batch == 0 || a->seq_len == 0 || a->n_heads == 0 || a->n_kv_heads == 0) return ATTN_ERR_INVALID_ARG;
    if (a->n_heads % a->n_kv_heads != 0) return ATTN_ERR_INVALID_ARG;
    if (a->dtype != ATTN_DTYPE_F16 && a->dtype != ATTN_DTYPE_BF16) return ATTN_ERR_UNSUPPORTED;
    if (a->o_dtype != ATTN_DTYPE_F32 && a->o_dtype != a->dtype) return ATTN_ERR_UNSUPPORTED;
    if (a->head_dim != 128 && a->head_dim != 64) return ATTN_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(a->q) | reinterpret_cast<uintptr_t>(a->k) | reinterpret_cast<uintptr_t>(a->v) |
         reinterpret_cast<uintptr_t>(a->o)) & 15u)
        return ATTN_ERR_ALIGNMENT;
    DeviceInfo dev{};
    int rc = current_device_info(&dev);
    if (rc != ATTN_OK) return rc;
    if (dev.cc_major != 10) return ATTN_ERR_DEVICE;

    CUtensorMap tm_q, tm_k, tm_v, tm_o;
    if ((rc = make_map(&tm_o, a->o, a->o_dtype, a->batch, a->seq_len, a->n_heads, a->head_dim)) != ATTN_OK) return rc;
    if ((rc = make_map(&tm_q, a->q, a->dtype, a->batch, a->seq_len, a->n_heads, a->head_dim)) != ATTN_OK) return rc;
    if ((rc = make_map(&tm_k, a->k, a->dtype, a->batch, a->seq_len, a->n_kv_heads, a->head_dim)) != ATTN_OK) return rc;
    if ((rc = make_map(&tm_v, a->v, a->dtype, a->batch, a->seq_len, a->n_kv_heads, a->head_dim)) != ATTN_OK) return rc;

    PrefillParams p{};
    p.o = a->o;
    p.o_dtype = a->o_dtype;
    p.in_dtype = a->dtype;
    p.batch = a->batch;
    p.seq = a->seq_len;
    p.n_heads = a->n_heads;
    p.n_kv_heads = a->n_kv_heads;
    p.group = a->n_heads / a->n_kv_heads;
    p.m_tiles = (a->seq_len + BM - 1) / BM;
    p.pair_heads = (p.group % 2 == 0) ? 1u : 0u;
    const float scale = a->scale != 0.f ? a->scale : 1.0f / sqrtf(static_cast<float>(a->head_dim));
    p.scale_log2 = scale * 1.4426950408889634f;
    p.status = a->status;
#ifdef ATTN_TRACE
    p.debug = g_prefill_debug;
#endif
    if (a->p_mode > 1) return ATTN_ERR_INVALID_ARG;

    dim3 grid;
    if (p.pair_heads) grid = dim3(a->n_heads / 2, a->batch, p.m_tiles);
    else grid = dim3(a->n_heads, a->batch, (p.m_tiles + 1) / 2);
    if (grid.y > 65535u || grid.z > 65535u) return ATTN_ERR_UNSUPPORTED;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    auto launch = [&](auto kernel) -> int {
        B200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemAlloc)));
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = kSmemAlloc;
        cfg.stream = stream;
        B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, tm_q, tm_k, tm_v, tm_o, p));
        g_launch_count.fetch_add(1, std::memory_order_relaxed);
        return ATTN_OK;
    };
    const bool single = a->p_mode == ATTN_PREFILL_P_INPUT_TYPE;
    if (a->head_dim == 128) {
        if (a->dtype == ATTN_DTYPE_BF16) {
            return single ? launch(prefill_causal_kernel<true, kPInput, 128>) : launch(prefill_causal_kernel<true, kPResidual, 128>);
        }
        return single ? launch(prefill_causal_kernel<false, kPInput, 128>) : launch(prefill_causal_kernel<false, kPResidual, 128>);
    }
    if (a->dtype == ATTN_DTYPE_BF16) {
        return single ? launch(prefill_causal_kernel<true, kPInput, 64>) : launch(prefill_causal_kernel<true, kPResidual, 64>);
    }
    return single ? launch(prefill_causal_kernel<false, kPInput, 64>) : launch(prefill_causal_kernel<false, kPResidual, 64>);
}

#ifdef ATTN_TRACE
// Profiling build only: [128][128] floats that receive the raw Q.K^T of the first key block of the last row tile of
// head 0 / sequence 0 of every following attn_prefill_causal call (null = off).
extern "C" void attn_trace_set_prefill_debug(float* s_tile) { g_prefill_debug = s_tile; }
#endif
