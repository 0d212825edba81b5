// Device helpers shared by the tcgen05 prompt kernels (spyb_prefill.cu: Q4_0 / Q8_0, spyb_prefill_kq.cu: Q4_K / Q6_K):
// shared-memory and mbarrier accessors, operand descriptors, the MMA / commit / tensor-memory instructions, bounded waits.
#pragma once

#include "spyb_common.cuh"
#include "spyb_kernels.h"

namespace spyb {
namespace {

constexpr int PF_M           = PF_ROWS;            // weight rows per CTA = M of the MMA
constexpr int PF_NCOL        = 128;                // columns of D per block step = N of the MMA
constexpr int PF_TILE        = PF_M * 32;          // bytes of one s8 operand tile
constexpr int PF_EPI_WARPS   = 8;                  // epilogue warps: (row quadrant 0..3) x (half of the columns); 12 warps in all leave them 168 registers
constexpr int PF_BATCH       = 4;                  // blocks per batch: the unit of the copies, of the expansion and of stage reuse
constexpr int PF_RING        = 4;                  // batches in the shared-memory rings
constexpr int PF_STAGES      = PF_RING * PF_BATCH; // blocks in the rings
constexpr int PF_MMA_WARPS   = 2;                  // warps whose first thread issues the MMAs of every PF_MMA_WARPS-th block
constexpr int PF_THREADS     = (PF_EPI_WARPS + 2 + PF_MMA_WARPS) * 32;   // + the copy warp and the expander warp
constexpr int PF_EPI_WARPS_F8 = 16;                // the e4m3 form: (row quadrant) x (quarter of the columns); its epilogue needs under 96 registers
constexpr int PF_MMA_WARPS_F8 = 2;                 // two MMAs and a commit per block hold the issuing thread ~240 cycles
constexpr int PF_THREADS_F8  = (PF_EPI_WARPS_F8 + 2 + PF_MMA_WARPS_F8) * 32;
constexpr int PF_DBUF        = 4;                  // accumulator buffers in tensor memory, PF_NCOL columns each (512 columns = all of it)

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// shared-memory operand descriptor: K-major, no swizzle; element (row r, byte k) of the tile lies at
// (r / 8) * 256 + (k / 16) * 128 + (r % 8) * 16 + k % 16: leading (K-chunk) offset 128, stride (8-row group) offset 256
__device__ __forceinline__ uint64_t operand_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(128u >> 4) << 16) | ((uint64_t)(256u >> 4) << 32) | (1ull << 46);
}
// instruction descriptor: D s32, A and B s8 K-major, N = 128, M = 128
constexpr uint32_t PF_IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(PF_NCOL >> 3) << 17) | ((uint32_t)(PF_M >> 4) << 24);

__device__ __forceinline__ void mma_s8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc) {
    const uint32_t zero = 0, accumulate = 1;   // D += A B^T: D holds the offset pattern
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(PF_IDESC), "r"(accumulate), "r"(zero) : "memory");
}
// e4m3 operands (kind::f8f6f4), f32 accumulators: D (+)= A B^T. Small integers are exact in e4m3 (|v| <= 16, and multiples of 16
// up to 128), their products and the sums of a block's few products are exact in f32, so D holds (float)(integer sum) itself.
constexpr uint32_t PF_IDESC_F8 = (1u << 4) | ((uint32_t)(PF_NCOL >> 3) << 17) | ((uint32_t)(PF_M >> 4) << 24);
__device__ __forceinline__ void mma_f8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    const uint32_t zero = 0;
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(PF_IDESC_F8), "r"(accumulate), "r"(zero) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// the same 32-bit word into 32 consecutive columns of this thread's lane
__device__ __forceinline__ void tmem_st32_same(uint32_t taddr, uint32_t v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1};" ::"r"(taddr), "r"(v) : "memory");
}
// 16 consecutive columns of this thread's lane from 16 registers (callers keep a register set that holds the offset
// pattern alive across the loop, so that no copies are made per store)
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t *v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
                   "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// e4m3 code of the integer v, 0 <= v <= 15 (exact: three mantissa bits cover 8..15), and of a signed value in [-15, 15]
__host__ __device__ __forceinline__ uint32_t e4m3_of_small(uint32_t v) {
    if (v == 0) { return 0u; }
    const int e = v >= 8 ? 3 : v >= 4 ? 2 : v >= 2 ? 1 : 0;
    return ((uint32_t)(e + 7) << 3) | ((v << (3 - e)) & 7u);
}
__host__ __device__ __forceinline__ uint32_t e4m3_of_signed(int v) { return v < 0 ? (0x80u | e4m3_of_small((uint32_t)-v)) : e4m3_of_small((uint32_t)v); }
// a Q8_0 activation byte y in [-127, 127] as two e4m3 values: y = hi + lo with lo = y mod 16 in [0, 15] and hi = y - lo a
// multiple of 16 in [-128, 112] (the code of |hi| / 16 with the exponent raised by four)
__device__ __forceinline__ void e4m3_split4(uint32_t q, uint32_t &hi, uint32_t &lo) {
    hi = 0u; lo = 0u;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int y = (int)(int8_t)((q >> (8 * i)) & 0xffu);
        const int yl = y & 15, yh = (y - yl) >> 4;   // yh in [-8, 7]
        const uint32_t ch = yh == 0 ? 0u : (e4m3_of_signed(yh) + 0x20u);
        hi |= ch << (8 * i);
        lo |= e4m3_of_small((uint32_t)yl) << (8 * i);
    }
}

// feeder roles (copy, expansion, MMA issue) run ahead of the epilogue: their waits back off instead of competing with the
// epilogue warps for issue slots
__device__ __forceinline__ bool mbar_wait_relaxed(uint32_t bar, uint32_t parity, uint64_t limit_ns) {
    if (mbar_try_wait(bar, parity)) { return true; }
    const uint64_t t0 = global_timer_ns();
    for (;;) {
        __nanosleep(100);
        if (mbar_try_wait(bar, parity)) { return true; }
        if (global_timer_ns() - t0 > limit_ns) { return false; }
    }
}
// profiling aid: clock stamps of CTA (0, 0) into g.stamps [8 roles][512 blocks][4] (nullptr: off)
#define PF_STAMP(role, b, i) do { if (g.stamps != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && (b) < 512) { g.stamps[((role) * 512 + (b)) * 4 + (i)] = clock64(); } } while (0)
__device__ __forceinline__ void pf_report(int *error_flag, int code) {
    if (error_flag != nullptr) { atomicExch(error_flag, code); }
}

}  // namespace
}  // namespace spyb
