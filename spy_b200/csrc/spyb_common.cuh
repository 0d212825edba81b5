// Shared device helpers: number formats, the Q8_0 activation quantizer arithmetic and the
// integer block dot products. Everything the reference pins bit-exactly lives here so that the
// stand-alone parity kernels and the fused kernels execute the very same instructions.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace spyb {

constexpr int WARP = 32;
constexpr int QK = 32;  // elements per Q4_0 / Q8_0 block (orchestration/include/number/number_impl/quant.h:10-33,124-147)
constexpr uint64_t WAIT_LIMIT_NS = 1000000000ull;   // a bulk copy or a peer's flag that has not arrived after a second: give up and report

// ---------------------------------------------------------------------------------------------
// fp16 <-> fp32. The reference converts fp16 -> fp32 through an exact table
// (orchestration/include/number/lookup_table.h:52) and fp32 -> fp16 with round-to-nearest-even
// (lookup_table.h:54); the hardware conversions below are the same functions.
__device__ __forceinline__ float h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }
__device__ __forceinline__ uint16_t f2h(float f) { return __half_as_ushort(__float2half_rn(f)); }

// ---------------------------------------------------------------------------------------------
// programmatic dependent launch: let the next kernel of the step start its weight prefetch while
// this one is still running, and wait for the previous kernel's results before touching them.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// bulk asynchronous copies global -> shared memory, completion counted on an mbarrier (no tensor map: plain
// contiguous runs; both addresses and the size are multiples of 16 bytes)
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
// loads through 32-bit shared-space addresses (no generic-pointer arithmetic in the inner loops)
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float4 lds128f(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {   // `bar`: shared-space address of the 8-byte barrier
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait: false when the phase did not complete within `limit_ns` of wall-clock time
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void stamp(unsigned long long *stamps, int slot, bool all_ctas) {
    if (stamps == nullptr || threadIdx.x != 0) { return; }
    if (all_ctas) { atomicMax(stamps + slot, (unsigned long long)global_timer_ns()); }
    else if (blockIdx.x == 0 && blockIdx.y == 0) { stamps[slot] = global_timer_ns(); }
}
// the same with a suspend-time hint: the thread may sleep up to `hint_ns` inside the instruction instead of
// spinning through the issue slots other warps need
__device__ __forceinline__ bool mbar_try_wait_sleep(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(hint_ns) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint64_t limit_ns) {
    if (mbar_try_wait(bar, parity)) { return true; }
    const uint64_t t0 = global_timer_ns();
    for (;;) {
        if (mbar_try_wait_sleep(bar, parity, 2000u)) { return true; }
        if (global_timer_ns() - t0 > limit_ns) { return false; }
    }
}
// the same for waits that normally end within a microsecond (pipeline hand-offs inside a CTA): the plain form of
// try_wait wakes as soon as the phase completes, the suspend-hint form is only the fallback of a wait that drags on
__device__ __forceinline__ bool mbar_wait_prompt(uint32_t bar, uint32_t parity, uint64_t limit_ns) {
#pragma unroll 1
    for (int i = 0; i < 2048; ++i) {
        if (mbar_try_wait(bar, parity)) { return true; }
    }
    return mbar_wait_bounded(bar, parity, limit_ns);
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst_smem, const void *src_gmem, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(__cvta_generic_to_global(src_gmem)), "r"(bytes), "r"(bar) : "memory");
}

// system-scope flag words of the tensor-parallel exchange (written by peer GPUs over NVLink)
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { v += __shfl_xor_sync(0xffffffffu, v, o); }
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o)); }
    return v;
}

// ---------------------------------------------------------------------------------------------
// Q8_0 activation quantization, Quantizator<FP32,Q8_0>::transform
// (backend/host/include/simd/vec_convert.h:178-261). A block of 32 floats is held by 8 consecutive
// lanes, 4 floats each. Returns the 4 quantized values packed little-endian into one word;
// `d_half` receives the fp16 scale bits, `sum` the integer sum of the lane's 4 values.
//   amax = max |x|; d = amax / 127 (stored as fp16, RNE); id = amax ? 127 / amax : 0;
//   q = round-half-even(x * id)   (one f32 multiply, never fused)
__device__ __forceinline__ uint32_t quantize_q8_lane4(float4 v, uint16_t &d_half, int &sum) {
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    const float d  = __fdiv_rn(amax, 127.0f);
    const float id = (amax != 0.0f) ? __fdiv_rn(127.0f, amax) : 0.0f;
    d_half = f2h(d);
    const int q0 = __float2int_rn(__fmul_rn(v.x, id));
    const int q1 = __float2int_rn(__fmul_rn(v.y, id));
    const int q2 = __float2int_rn(__fmul_rn(v.z, id));
    const int q3 = __float2int_rn(__fmul_rn(v.w, id));
    sum = q0 + q1 + q2 + q3;
    return (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
}

// ---------------------------------------------------------------------------------------------
// Integer lane sums are produced directly as floats: the accumulator operand of the byte dot product
// carries MAGIC_I, so that the result's bit
// pattern is the float MAGIC_F + lane_sum and one exact subtraction yields (float)lane_sum.
constexpr float    MAGIC_F = 12582912.0f;     // 1.5 * 2^23: int_as_float(MAGIC_I + p) == MAGIC_F + p exactly for |p| < 2^22
constexpr uint32_t MAGIC_I = 0x4B400000u;

// One of the eight integer "lane sums" of a block pair, in the order of the reference's 8-wide accumulator
// (Dot<Q4_0,Q8_0>::exec, backend/host/include/simd/vec_dot.h:58-75 with mul_sum_i8_pairs, vec_util.h:100-110:
// lanes 0..3 = sum over k = 4j..4j+3 of (high nibble_k - 8) * y[16+k], lanes 4..7 = the same with low nibbles
// and y[k]; Dot<Q8_0,Q8_0>::exec, vec_dot.h:103-113: lane l = sum of products 4l..4l+3), returned as a float.
//   Q4_0: `w_x88` = the weight word XOR 0x88888888 (every nibble then is value - 8 in two's complement);
//   `mult` = 1 for the high nibbles, 16 for the low ones: the selected nibble of every byte lands in the high
//   half of its byte (a multiply, so that it runs on the FMA pipe beside the integer dot products), which as a signed byte is 16 * (value - 8). The result is 16 * lane_sum; the caller
//   multiplies by scale / 16, which is exact.
__device__ __forceinline__ float lane_sum16_q4_0(uint32_t w_x88, uint32_t mult, uint32_t y) {
    return __int_as_float(__dp4a((int)((w_x88 * mult) & 0xf0f0f0f0u), (int)y, (int)MAGIC_I)) - MAGIC_F;
}
__device__ __forceinline__ float lane_sum_q8_0(uint32_t w, uint32_t y) {
    return __int_as_float(__dp4a((int)w, (int)y, (int)MAGIC_I)) - MAGIC_F;
}

// the same sums as bit patterns (of the float MAGIC_F + lane_sum), for callers that subtract MAGIC_F two at a time
__device__ __forceinline__ uint32_t lane_bits16_q4_0(uint32_t w_x88, uint32_t mult, uint32_t y) {
    return (uint32_t)__dp4a((int)((w_x88 * mult) & 0xf0f0f0f0u), (int)y, (int)MAGIC_I);
}
__device__ __forceinline__ uint32_t lane_bits_q8_0(uint32_t w, uint32_t y) { return (uint32_t)__dp4a((int)w, (int)y, (int)MAGIC_I); }

// Two f32 operations per instruction (sm_100 packed f32x2): each half is the IEEE round-to-nearest operation of the
// scalar instruction, so results are the bits of two fmaf / __fadd_rn calls at half the issue slots.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ uint64_t f2_pack_bits(uint32_t lo, uint32_t hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// hsum_float_8 (vec_util.h:74-81) over the 8 consecutive lanes that hold a0..a7:
// ((a0+a4) + (a2+a6)) + ((a1+a5) + (a3+a7)). Every lane of the group ends with the same bits.
__device__ __forceinline__ float hsum8_lanes(float v) {
    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 4));
    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 2));
    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return v;
}

// FP16::block_reduce (vec_util.h:61-71) for the 4 x 8 accumulators of Dot<FP16,FP16> held one per lane
// (lane = 8 * accumulator + element): (s0+s2) + (s1+s3), then lanes l and l+4, then the two hadd steps.
__device__ __forceinline__ float reduce_f16dot_lanes(float v) {
    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 16));
    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 8));
    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 4));
    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 1));
    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 2));
    return v;
}

}  // namespace spyb
