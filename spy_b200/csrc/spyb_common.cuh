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

// 128-bit streaming load of weights: read-only path, no L1 allocation (each weight byte is used once).
__device__ __forceinline__ uint4 ldg_stream(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint16_t ldg_stream_u16(const uint16_t *p) {
    uint16_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
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
// Activation columns as the mat-vec kernels keep them in shared memory (structure of arrays, so
// that every lane's 128-bit read is conflict-free): for column t and block b
//   lo[t][b] = int8 values 0..15 of the block, hi[t][b] = values 16..31,
//   d[t][b]  = f32 of the fp16-rounded scale, s[t][b] = integer sum of the 32 values.
// The values are exactly those of the reference's block_q8_0_t (quant.h:124-147), regrouped.
struct ActView {
    uint4 *lo;
    uint4 *hi;
    float *d;
    int   *s;
    int    nb;  // blocks per column
};

__host__ __device__ inline size_t act_bytes(int nb, int t) { return (size_t)t * nb * (16 + 16 + 4 + 4); }

__device__ __forceinline__ ActView act_view(void *base, int nb, int t) {
    ActView v;
    v.lo = reinterpret_cast<uint4 *>(base);
    v.hi = v.lo + (size_t)t * nb;
    v.d  = reinterpret_cast<float *>(v.hi + (size_t)t * nb);
    v.s  = reinterpret_cast<int *>(v.d + (size_t)t * nb);
    v.nb = nb;
    return v;
}

// Integer dot of one Q4_0 block (16 bytes of nibbles) with one Q8_0 activation block:
// sum_k (nibble_k - 8) * y_k, Dot<Q4_0,Q8_0>::exec (backend/host/include/simd/vec_dot.h:58-75).
// Low nibbles pair with y[0..15], high nibbles with y[16..31]. Computed as
// sum nibble*y - 8*sum(y) with four-way byte dot products; exact in int32.
__device__ __forceinline__ int dot_q4_0_block(const uint4 w, const uint4 ylo, const uint4 yhi, const int ysum) {
    int acc = 0;
    acc = __dp4a((int)(w.x & 0x0f0f0f0fu), (int)ylo.x, acc);
    acc = __dp4a((int)((w.x >> 4) & 0x0f0f0f0fu), (int)yhi.x, acc);
    acc = __dp4a((int)(w.y & 0x0f0f0f0fu), (int)ylo.y, acc);
    acc = __dp4a((int)((w.y >> 4) & 0x0f0f0f0fu), (int)yhi.y, acc);
    acc = __dp4a((int)(w.z & 0x0f0f0f0fu), (int)ylo.z, acc);
    acc = __dp4a((int)((w.z >> 4) & 0x0f0f0f0fu), (int)yhi.z, acc);
    acc = __dp4a((int)(w.w & 0x0f0f0f0fu), (int)ylo.w, acc);
    acc = __dp4a((int)((w.w >> 4) & 0x0f0f0f0fu), (int)yhi.w, acc);
    return acc - 8 * ysum;
}

// Integer dot of one Q8_0 block (two 16-byte halves) with one Q8_0 activation block,
// Dot<Q8_0,Q8_0>::exec (vec_dot.h:103-113).
__device__ __forceinline__ int dot_q8_0_block(const uint4 wa, const uint4 wb, const uint4 ylo, const uint4 yhi) {
    int acc = 0;
    acc = __dp4a((int)wa.x, (int)ylo.x, acc);
    acc = __dp4a((int)wa.y, (int)ylo.y, acc);
    acc = __dp4a((int)wa.z, (int)ylo.z, acc);
    acc = __dp4a((int)wa.w, (int)ylo.w, acc);
    acc = __dp4a((int)wb.x, (int)yhi.x, acc);
    acc = __dp4a((int)wb.y, (int)yhi.y, acc);
    acc = __dp4a((int)wb.z, (int)yhi.z, acc);
    acc = __dp4a((int)wb.w, (int)yhi.w, acc);
    return acc;
}

}  // namespace spyb
