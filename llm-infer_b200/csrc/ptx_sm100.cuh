// Thin inline-PTX wrappers used by the sm_100a attention kernels: shared-memory
// barriers (mbarrier) with BOUNDED waits, bulk asynchronous copies (the TMA
// engine, untiled and tensor-map forms, never with cluster multicast), ldmatrix
// and the warp-level m16n8k16 tensor-core MMA used by the decode kernel.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace b200 {

// A wait that has not succeeded after this many polls gives up; the caller then
// records ATTN_STATUS_WAIT_TIMEOUT and leaves the kernel. Each poll may itself
// block for a hardware-defined interval, so this is on the order of seconds.
constexpr uint32_t kWaitPollLimit = 1u << 20;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

// Makes barrier initialisation visible to the asynchronous proxy (bulk copies).
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: true when the phase completed, false when the poll limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t it = 0; it < kWaitPollLimit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
#ifdef ATTN_WAIT_BACKOFF_NS
        __nanosleep(ATTN_WAIT_BACKOFF_NS);
#endif
    }
    return false;
}

__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

// Untiled bulk copy global -> this CTA's shared memory, completion counted in
// bytes on an mbarrier. Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar,
                                         uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3,
                                                  uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

// D(16x8, f32) += A(16x16, row) * B(16x8, col); A/B fp16 or bf16.
template <bool BF16>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if constexpr (BF16) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    } else {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
}

// The same product when rows 8-15 of A are known to be zero (at most eight query heads per kv head): only rows 0-7
// are fed (a0: columns k, a2: columns k+8) and kept (c0, c1); the zero half of A, the zero accumulator half and the
// discarded outputs are temporaries of the instruction, so they occupy no register of the caller between MMAs.
template <bool BF16>
__device__ __forceinline__ void mma_16816_low8(float& c0, float& c1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    if constexpr (BF16) {
        asm volatile(
            "{\n\t.reg .b32 z;\n\t.reg .f32 zf, j0, j1;\n\tmov.b32 z, 0;\n\tmov.f32 zf, 0f00000000;\n\t"
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,j0,j1}, {%2,z,%3,z}, {%4,%5}, {%0,%1,zf,zf};\n\t}"
            : "+f"(c0), "+f"(c1)
            : "r"(a0), "r"(a2), "r"(b0), "r"(b1));
    } else {
        asm volatile(
            "{\n\t.reg .b32 z;\n\t.reg .f32 zf, j0, j1;\n\tmov.b32 z, 0;\n\tmov.f32 zf, 0f00000000;\n\t"
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,j0,j1}, {%2,z,%3,z}, {%4,%5}, {%0,%1,zf,zf};\n\t}"
            : "+f"(c0), "+f"(c1)
            : "r"(a0), "r"(a2), "r"(b0), "r"(b1));
    }
}

// Two floats -> packed 16-bit pair (low half = first argument), round to nearest even.
template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    if constexpr (BF16) {
        __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&t);
    } else {
        __half2 t = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&t);
    }
}

template <bool BF16>
__device__ __forceinline__ float round16(float x) {
    if constexpr (BF16) {
        return __bfloat162float(__float2bfloat16_rn(x));
    } else {
        return __half2float(__float2half_rn(x));
    }
}

// Programmatic dependent launch: the dependent grid may start once every CTA of
// this grid has called this (or exited); it still has to call grid_dep_wait()
// before it touches what this grid writes.
__device__ __forceinline__ void grid_dep_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// 64-bit system-scope accesses for records that another GPU writes into this GPU's memory (or the reverse) over
// NVLink. A naturally aligned 64-bit scalar access is single-copy atomic, so a word that carries 32 bits of data and
// a 32-bit step tag is never seen half-written: the reader needs no separate flag and the writer no fence.
__device__ __forceinline__ void st_sys_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ uint32_t dynamic_smem_bytes() {
    uint32_t v;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(v));
    return v;
}

// Time stamps of the profiling build (-DATTN_TRACE): a kernel stores the nanosecond timer at a few points per CTA
// into a buffer registered with attn_trace_set_buffer(); the product build compiles none of it.
#ifdef ATTN_TRACE
__device__ __forceinline__ unsigned long long trace_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define ATTN_TRACE_AT(buf, slot)                         \
    do {                                                 \
        if (buf) (buf)[slot] = ::b200::trace_now();      \
    } while (0)
#else
#define ATTN_TRACE_AT(buf, slot) \
    do {                         \
    } while (0)
#endif

}  // namespace b200
