// The tensor-core inner loop shared by the per-matrix mat-vec kernel and the persistent step kernel: one record
// (8 consecutive blocks of the TR rows of a tile, fragment-ordered, in shared memory) against the Q8_0 activations.
//
// Integer part: one mma.sync.m16n8k32 (s8 x s8 -> s32) per block. A = the block's 32 weights of 16 rows (Q4_0: nibbles
// brought to the high half of a byte, 16 * (value - 8)); B = the block's 32 activations laid out block-diagonally:
// column n holds activations 4n .. 4n+3 and zeros elsewhere, so D[row][n] is exactly the n-th group-of-four sum the CPU
// keeps in its n-th accumulator lane (Dot<Q4_0,Q8_0>: columns 0..3 = low nibbles = accumulators 4..7, columns 4..7 =
// high nibbles = accumulators 0..3; Dot<Q8_0,Q8_0>: column n = accumulator n; backend/host/include/simd/vec_dot.h:58-113).
// C carries the int->float magic constant. Lane (g = lane / 4, q = lane % 4) owns D[g][2q], D[g][2q+1], D[g+8][2q],
// D[g+8][2q+1]: four f32 accumulators, each advanced block after block by acc = fma(d_w * d_x, (float)sum, acc) exactly
// as on the CPU. With TR = 8 the upper eight rows of A are zero.
//
// Record layout: [2 groups of four blocks][halves of a block: 1 (Q4_0) or 2 (Q8_0)][row][word q] x 16 B (the four
// blocks of the group side by side), then [row][8 fp16 scales]: a quarter-warp's 128-bit reads are 128 contiguous bytes.
#pragma once

#include "spyb_common.cuh"

namespace spyb {

// how the integer sums become floats: 2 = I2F (measured fastest: 129 warp instructions per 8-row Q4_0 record against
// 135 / 147 for the magic-constant forms 0 / 1)
#ifndef SPYB_MMA_CONV
#define SPYB_MMA_CONV 2
#endif
__device__ __forceinline__ void mma_s8_lane_sums(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(SPYB_MMA_CONV == 0 ? (int)MAGIC_I : 0));
}
// exact int -> float for |p| < 2^22
__device__ __forceinline__ float lane_sum_to_float(int p) {
#if SPYB_MMA_CONV == 0
    return __int_as_float(p) - MAGIC_F;                       // the accumulator operand carried the magic constant
#elif SPYB_MMA_CONV == 1
    return __int_as_float(p + (int)MAGIC_I) - MAGIC_F;        // an integer add (ALU pipe) and a float subtraction
#else
    return __int2float_rn(p);
#endif
}

template <int WT, int TR>
struct MmaTile {
    static constexpr int H    = (WT == 8) ? 2 : 1;     // 16-value halves of a block that are stored separately
    static constexpr int GRPB = H * TR * 64;           // quants of one group of four blocks, all rows of the tile
    static constexpr int RECB = 2 * GRPB + TR * 16;    // bytes of a record
    static constexpr int NA   = (TR == 16) ? 4 : 2;    // accumulators per lane
};

// Per-lane addressing. The B fragment of lane (g, q) is activation word q when g == q (b0, columns 0..3) or word 4 + q
// when g == 4 + q (b1, columns 4..7); the other 24 lanes contribute zeros and issue no load at all (shared-memory
// bandwidth, counted in 128-byte wavefronts, is what bounds this loop: the weights need 8 per record of an 8-row tile,
// and every broadcast-style load of activations or scales costs as much as a dense one).
struct MmaLane {
    uint32_t w_off;     // row g, word q inside a (group, half) plane of a record
    uint32_t sc_off;    // row g's scales inside a record
    uint32_t y_off;     // this lane's activation word inside a group of the Y plane (meaningful on the 8 diagonal lanes)
    uint32_t lo, hi;    // 1 when the lane holds a non-zero b0 / b1
};
template <int WT, int TR>
__device__ __forceinline__ MmaLane mma_lane(int lane) {
    const int g = lane >> 2, q = lane & 3;
    MmaLane l;
    l.w_off = (uint32_t)(g * 4 + q) * 16;
    l.sc_off = 2 * MmaTile<WT, TR>::GRPB + g * 16;
    const bool diag = (g & 3) == q;
    l.lo = (diag && g < 4) ? 1u : 0u; l.hi = (diag && g >= 4) ? 1u : 0u;
    l.y_off = (uint32_t)(g >= 4 ? 4 + q : q) * 16;
    return l;
}

// 128-bit shared-memory load executed only where `pred` is non-zero; elsewhere `v` keeps its value (the zeros it was
// initialised with) and the lane generates no shared-memory traffic.
__device__ __forceinline__ void lds128_if(uint4 &v, uint32_t addr, uint32_t pred) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %5, 0;\n\t@p ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n\t}"
                 : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w) : "r"(addr), "r"(pred));
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

// Operands of one group of four consecutive blocks, as they come out of shared memory. The loop over a stage keeps two
// of these: the loads of group i + 1 are in flight while group i is computed.
template <int WT, int TR, int TM>
struct MmaOps {
    uint4  w[MmaTile<WT, TR>::H][TR / 8];   // [low / high 16 values][rows g, g + 8]: word q of the four blocks
    uint2  sc[TR / 8];                      // four fp16 scales of rows g, g + 8
    uint4  y0[TM], y1[TM];                  // B fragments of the four blocks (zero off the diagonal)
    float4 ds[TM];                          // the four blocks' activation scales (for Q4_0 weights: / 16)
};
template <int WT, int TR, int TM>
__device__ __forceinline__ void mma_ops_init(MmaOps<WT, TR, TM> &o) {
#pragma unroll
    for (int t = 0; t < TM; ++t) { o.y0[t] = make_uint4(0u, 0u, 0u, 0u); o.y1[t] = make_uint4(0u, 0u, 0u, 0u); }
}
// ra: shared-space address of the record; gg: group inside the record (0, 1); ya / da: addresses of the group in column 0's
// Y / DS planes; col_y / col_ds: distance between two columns' planes
template <int WT, int TR, int TM>
__device__ __forceinline__ void mma_load_group(MmaOps<WT, TR, TM> &o, uint32_t ra, int gg, uint32_t ya, uint32_t da, uint32_t col_y, uint32_t col_ds, const MmaLane &L) {
    using T = MmaTile<WT, TR>;
#pragma unroll
    for (int h = 0; h < T::H; ++h) {
#pragma unroll
        for (int r = 0; r < TR / 8; ++r) { o.w[h][r] = lds128(ra + gg * T::GRPB + (h * TR + 8 * r) * 64 + L.w_off); }
    }
#pragma unroll
    for (int r = 0; r < TR / 8; ++r) { o.sc[r] = lds64(ra + L.sc_off + r * 128 + gg * 8); }
#pragma unroll
    for (int t = 0; t < TM; ++t) {
        lds128_if(o.y0[t], ya + t * col_y + L.y_off, L.lo);
        lds128_if(o.y1[t], ya + t * col_y + L.y_off, L.hi);
        o.ds[t] = lds128f(da + t * col_ds);
    }
}
// the four blocks' integer group sums: D fragments of four mma instructions
template <int WT, int TR, int TM>
__device__ __forceinline__ void mma_issue_group(const MmaOps<WT, TR, TM> &o, int (&d)[TM][4][4]) {
    using T = MmaTile<WT, TR>;
    uint32_t a0[4], a1[4], a2[4], a3[4];
    const uint32_t wl[4] = {o.w[0][0].x, o.w[0][0].y, o.w[0][0].z, o.w[0][0].w};
    const uint32_t wh[4] = {o.w[T::H - 1][0].x, o.w[T::H - 1][0].y, o.w[T::H - 1][0].z, o.w[T::H - 1][0].w};
    const uint32_t vl[4] = {o.w[0][TR / 8 - 1].x, o.w[0][TR / 8 - 1].y, o.w[0][TR / 8 - 1].z, o.w[0][TR / 8 - 1].w};
    const uint32_t vh[4] = {o.w[T::H - 1][TR / 8 - 1].x, o.w[T::H - 1][TR / 8 - 1].y, o.w[T::H - 1][TR / 8 - 1].z, o.w[T::H - 1][TR / 8 - 1].w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (WT == 2) {   // stored nibbles are (value - 8) in two's complement: in the high half of a byte, 16 * (value - 8)
            a0[i] = (wl[i] << 4) & 0xf0f0f0f0u; a2[i] = wl[i] & 0xf0f0f0f0u;
            a1[i] = (TR == 16) ? (vl[i] << 4) & 0xf0f0f0f0u : 0u; a3[i] = (TR == 16) ? vl[i] & 0xf0f0f0f0u : 0u;
        } else {
            a0[i] = wl[i]; a2[i] = wh[i];
            a1[i] = (TR == 16) ? vl[i] : 0u; a3[i] = (TR == 16) ? vh[i] : 0u;
        }
    }
#pragma unroll
    for (int t = 0; t < TM; ++t) {
        const uint32_t b0[4] = {o.y0[t].x, o.y0[t].y, o.y0[t].z, o.y0[t].w}, b1[4] = {o.y1[t].x, o.y1[t].y, o.y1[t].z, o.y1[t].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { mma_s8_lane_sums(d[t][i], a0[i], a1[i], a2[i], a3[i], b0[i], b1[i]); }
    }
}
// acc = fma(d_w * d_x, (float)sum, acc), block after block
template <int WT, int TR, int TM>
__device__ __forceinline__ void mma_fold_group(const int (&d)[TM][4][4], const uint2 (&sc)[TR / 8], const float4 (&ds)[TM], float (&acc)[TM][MmaTile<WT, TR>::NA]) {
    constexpr int NA = MmaTile<WT, TR>::NA;
    const float2 f01 = __half22float2(*reinterpret_cast<const __half2 *>(&sc[0].x)), f23 = __half22float2(*reinterpret_cast<const __half2 *>(&sc[0].y));
    const float  dw0[4] = {f01.x, f01.y, f23.x, f23.y};
    const float2 h01 = __half22float2(*reinterpret_cast<const __half2 *>(&sc[TR / 8 - 1].x)), h23 = __half22float2(*reinterpret_cast<const __half2 *>(&sc[TR / 8 - 1].y));
    const float  dw1[4] = {h01.x, h01.y, h23.x, h23.y};
#pragma unroll
    for (int t = 0; t < TM; ++t) {
        const float dx[4] = {ds[t].x, ds[t].y, ds[t].z, ds[t].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float s0 = __fmul_rn(dw0[i], dx[i]);
            acc[t][0] = fmaf(s0, lane_sum_to_float(d[t][i][0]), acc[t][0]);
            acc[t][1] = fmaf(s0, lane_sum_to_float(d[t][i][1]), acc[t][1]);
            if (TR == 16) {
                const float s1 = __fmul_rn(dw1[i], dx[i]);
                acc[t][NA - 2] = fmaf(s1, lane_sum_to_float(d[t][i][2]), acc[t][NA - 2]);
                acc[t][NA - 1] = fmaf(s1, lane_sum_to_float(d[t][i][3]), acc[t][NA - 1]);
            }
        }
    }
}

// `cnt` consecutive records starting at shared-space address ra; ya / da: addresses, in column 0's Y / DS planes, of the
// first record's first group (advanced past the records on return).
template <int WT, int TR, int TM>
__device__ __forceinline__ void mma_records(uint32_t ra, int cnt, uint32_t &ya, uint32_t &da, uint32_t col_y, uint32_t col_ds, const MmaLane &L,
                                            float (&acc)[TM][MmaTile<WT, TR>::NA]) {
    using T = MmaTile<WT, TR>;
    MmaOps<WT, TR, TM> A, B;
    mma_ops_init(A); mma_ops_init(B);
#pragma unroll 1
    for (int rc = 0; rc < cnt; ++rc, ra += T::RECB, ya += 256, da += 32) {
        int d[TM][4][4];
        mma_load_group(A, ra, 0, ya, da, col_y, col_ds, L);
        mma_load_group(B, ra, 1, ya + 128, da + 16, col_y, col_ds, L);
        mma_issue_group(A, d);
        mma_fold_group<WT, TR, TM>(d, A.sc, A.ds, acc);
        mma_issue_group(B, d);
        mma_fold_group<WT, TR, TM>(d, B.sc, B.ds, acc);
    }
}

// hsum_float_8 (vec_util.h:74-81), ((a0+a4)+(a2+a6))+((a1+a5)+(a3+a7)), over the four lanes of a row: `e` / `o` are the
// lane's accumulators of columns 2q / 2q+1; every lane of the row ends with the same bits.
__device__ __forceinline__ float mma_row_sum(float e, float o) {
    e = __fadd_rn(e, __shfl_xor_sync(0xffffffffu, e, 2)); o = __fadd_rn(o, __shfl_xor_sync(0xffffffffu, o, 2));   // a_j + a_(j+4)
    e = __fadd_rn(e, __shfl_xor_sync(0xffffffffu, e, 1)); o = __fadd_rn(o, __shfl_xor_sync(0xffffffffu, o, 1));   // (a0+a4)+(a2+a6), (a1+a5)+(a3+a7)
    return __fadd_rn(e, o);
}

}  // namespace spyb
