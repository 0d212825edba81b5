// Attention over the fp16 KV cache in the reference's exact arithmetic, the upload re-tiling kernels,
// and the small per-operator kernels that let the reference's graph run op by op on the device.
// All of these are HBM- or latency-bound byte/float work; none is a dense contraction.
//
// Exactness: the reference network quantizes activations at every layer, which amplifies any
// difference in f32 summation order to percent-level logit differences. Every reduction here therefore
// follows the CPU's order: the 4 x 8 accumulators and the scalar tail of Dot<FP16,FP16>, the four-wide
// grouping of std::reduce / std::transform_reduce, and the fixed horizontal-add trees.

#include <algorithm>

#include <cstdlib>

#include "spyb_common.cuh"
#include "spyb_kernels.h"
#include "spyb_tp.cuh"

#include <math_constants.h>

namespace spyb {

static inline cudaError_t launch_check() { return cudaGetLastError(); }

// std::reduce over floats as libstdc++ evaluates it for random-access ranges: groups of four combined as
// (e0 + e1) + (e2 + e3) and added to the running sum one after the other, the remainder one by one.
// One thread's chain; `v` is in shared memory.
__device__ __forceinline__ float reduce4_chain(const float *v, int n) {
    float sum = 0.f;
    int i = 0;
    for (; i + 4 <= n; i += 4) { sum = __fadd_rn(sum, __fadd_rn(__fadd_rn(v[i], v[i + 1]), __fadd_rn(v[i + 2], v[i + 3]))); }
    for (; i < n; ++i) { sum = __fadd_rn(sum, v[i]); }
    return sum;
}

// =============================================================================================
// Attention for one (head, query token): a CTA of 8 warps, head_dim 128.
//   scores = K(f16) . fp16(Q)            MatMul with F16 weights: backend/host/operator/mat.cpp:32-42,
//                                        Dot<FP16,FP16> backend/host/include/simd/vec_dot.h:117-146
//   probs  = masked softmax, exp through the table of expf(fp16(s - max)), std::reduce sum
//                                        backend/host/operator/non-linear.cpp:129-180
//   out    = V(f16) . fp16(probs)        same MatMul rule; V is kept transposed [d][n_ctx] as the reference
//                                        graph lays it out (model/src/llm/plugin/attention.cpp:228-262)
// Dot<FP16,FP16> runs four 8-wide accumulators over 32-element steps while i + 32 < n, reduces them as
// (s0 + s2) + (s1 + s3), element l with l + 4, two horizontal adds, and leaves the rest (1..32 elements) to
// a scalar FMA chain added as tail + vector part. All 32 accumulators of a dot product live in the
// registers of ONE thread here (scores: one thread per position, the K row read with 128-bit loads) or of a
// thread pair (PV: elements 0..3 / 4..7 of the four accumulators, the V^T row read with 64-bit loads), so the
// reduction tree is register arithmetic and the dot products of a head run side by side.
// Roofline: HBM-bound, 2 * n_kv * head_dim * 2 bytes per head read once; latency-bound at short contexts.
constexpr int ATT_THREADS = 256;
constexpr int ATT_WARPS   = ATT_THREADS / WARP;
constexpr int ATT_HD      = 128;

__device__ __forceinline__ void unpack8(const uint4 v, float f[8]) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&v.x)), b = __half22float2(*reinterpret_cast<const __half2 *>(&v.y));
    const float2 c = __half22float2(*reinterpret_cast<const __half2 *>(&v.z)), d = __half22float2(*reinterpret_cast<const __half2 *>(&v.w));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

__global__ void __launch_bounds__(ATT_THREADS) attention_kernel(const AttnParams p) {
    extern __shared__ __align__(16) float att_smem[];
    __shared__ float red[ATT_WARPS];
    __shared__ float bcast;

    const int h = blockIdx.x, t = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    pdl_launch_dependents();
    stamp(p.stamps, 0, false); stamp(p.stamps, 4, true);
    pdl_wait();
    stamp(p.stamps, 1, false); stamp(p.stamps, 5, true);

    const bool batch = p.seq_stride != 0;        // token t = sequence t of a batch in lockstep: own cache, same position, nothing else visible
    const __half *k_cache = p.k_cache + (batch ? (int64_t)t * p.seq_stride : 0), *v_cache = p.v_cache + (batch ? (int64_t)t * p.seq_stride : 0);
    const int pos   = p.pos_base[0] + (batch ? 0 : t);
    const int n_vis = pos + 1;                   // causal mask: positions 0..pos are visible
    // Row length of the score matrix = all positions known to the step (past + every token of the step), as the
    // reference graph shapes it (K view [hd, n_past + n_token, H], model/src/llm/plugin/attention.cpp:207-223). Entries
    // beyond the causal limit carry mask -inf: they become exact zeros, but they still decide how std::reduce groups
    // the sum and where Dot<FP16,FP16> switches from its vector loop to the scalar tail.
    const int n_tot = batch ? n_vis : (p.pos_base[1] > 0) ? p.pos_base[1] : p.pos_base[0] + p.T;
    const int n_pad = (p.n_ctx + 3) & ~3;
    float *qf = att_smem;                        // [hd] Q as f32 (exact widening of the fp16 values)
    float *sc = qf + ATT_HD;                     // [n_pad] scores, then probabilities
    float *gs = sc + n_pad;                      // [n_pad / 4] four-wide partial sums of std::reduce

    // Everything this thread will need from global memory is requested up front, so that Q, the first K row and
    // the V^T values of the PV product share one memory round trip instead of three: the PV thread pair of element
    // e = tid / 2 fetches the first 32-position step and the (at most 32-position) scalar tail of its row now.
    const int n_main = ((n_tot - 1) / 32) * 32;
    const int pv_e = tid >> 1, pv_half = tid & 1;
    const __half *vrow = v_cache + ((int64_t)h * ATT_HD + pv_e) * p.n_ctx;
    uint2 v_first[4], v_tail[8];
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int j = 8 * a + 4 * pv_half;
        v_first[a] = (0 < n_main && j < n_vis) ? *reinterpret_cast<const uint2 *>(vrow + j) : make_uint2(0u, 0u);
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const int j = n_main + 4 * c;
        v_tail[c] = (j < n_vis) ? *reinterpret_cast<const uint2 *>(vrow + j) : make_uint2(0u, 0u);
    }
    const __half q_mine = (tid < ATT_HD) ? p.q[(int64_t)t * p.dl + (int64_t)h * ATT_HD + tid] : __float2half(0.f);
    uint4 kv[16];                                    // a whole K row in flight at once
    {
        const uint4 *krow = reinterpret_cast<const uint4 *>(k_cache + (int64_t)min(tid, n_vis - 1) * p.dl + (int64_t)h * ATT_HD);
#pragma unroll
        for (int a = 0; a < 16; ++a) { kv[a] = krow[a]; }
    }
    if (tid < ATT_HD) { qf[tid] = __half2float(q_mine); }
    __syncthreads();

    // ---- scores of the visible positions: one thread per position
    for (int j = tid; j < n_vis; j += ATT_THREADS) {
        const uint4  *krow = reinterpret_cast<const uint4 *>(k_cache + (int64_t)j * p.dl + (int64_t)h * ATT_HD);
        const float4 *q4   = reinterpret_cast<const float4 *>(qf);
        float acc[4][8];
        if (j != tid) {
#pragma unroll
            for (int a = 0; a < 16; ++a) { kv[a] = krow[a]; }
        }
#pragma unroll
        for (int a = 0; a < 4; ++a) {
#pragma unroll
            for (int e = 0; e < 8; ++e) { acc[a][e] = 0.f; }
        }
#pragma unroll
        for (int step = 0; step < 3; ++step) {       // elements 0..95: accumulator a takes elements 32 * step + 8a .. + 7
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                float kf[8]; unpack8(kv[4 * step + a], kf);
                const float4 qa = q4[(4 * step + a) * 2], qb = q4[(4 * step + a) * 2 + 1];
                const float  qv[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
                for (int e = 0; e < 8; ++e) { acc[a][e] = fmaf(kf[e], qv[e], acc[a][e]); }
            }
        }
        float u[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float lo = __fadd_rn(__fadd_rn(acc[0][e], acc[2][e]), __fadd_rn(acc[1][e], acc[3][e]));
            const float hi = __fadd_rn(__fadd_rn(acc[0][e + 4], acc[2][e + 4]), __fadd_rn(acc[1][e + 4], acc[3][e + 4]));
            u[e] = __fadd_rn(lo, hi);
        }
        const float simd = __fadd_rn(__fadd_rn(u[0], u[1]), __fadd_rn(u[2], u[3]));
        float tail = 0.f;                             // elements 96..127: scalar chain
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            float kf[8]; unpack8(kv[12 + a], kf);
            const float4 qa = q4[(12 + a) * 2], qb = q4[(12 + a) * 2 + 1];
            const float  qv[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) { tail = fmaf(kf[e], qv[e], tail); }
        }
        sc[j] = __fadd_rn(tail, simd);
    }
    // The V^T values of the next PV steps are requested now (the K row's registers are free), so that they arrive
    // during the softmax instead of costing one memory round trip per 32 positions afterwards.
    constexpr int PV_AHEAD = 6;
    constexpr int n_ahead = PV_AHEAD;
    uint2 v_ahead[PV_AHEAD][4];
#pragma unroll
    for (int s = 0; s < PV_AHEAD; ++s) {
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const int j0 = 32 * (s + 1), j = j0 + 8 * a + 4 * pv_half;
            v_ahead[s][a] = (s < n_ahead && j0 < n_main && j < n_vis) ? *reinterpret_cast<const uint2 *>(vrow + j) : make_uint2(0u, 0u);
        }
    }
    __syncthreads();

    // ---- masked softmax: (score + mask) * scale, subtract the maximum, table exp, std::reduce, multiply by 1/sum
    float m = -CUDART_INF_F;
    for (int j = tid; j < n_vis; j += ATT_THREADS) {
        const float v = __fmul_rn(__fadd_rn(sc[j], 0.0f), p.scale);
        sc[j] = v;
        m = fmaxf(m, v);
    }
    m = warp_max(m);
    if (lane == 0) { red[warp] = m; }
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < ATT_WARPS; ++w) { m = fmaxf(m, red[w]); }
    const int n_tot4 = (n_tot + 3) & ~3;
    for (int j = tid; j < n_tot4; j += ATT_THREADS) { sc[j] = (j < n_vis) ? p.exp_table[f2h(__fsub_rn(sc[j], m))] : 0.f; }
    __syncthreads();
    // std::reduce: groups of four as (e0 + e1) + (e2 + e3), formed in parallel, then one thread's running sum; the
    // remainder (n_tot % 4 elements) is added one by one
    for (int g = tid; g < (n_tot >> 2); g += ATT_THREADS) {
        const float4 v = reinterpret_cast<const float4 *>(sc)[g];
        gs[g] = __fadd_rn(__fadd_rn(v.x, v.y), __fadd_rn(v.z, v.w));
    }
    __syncthreads();
    if (tid == 0) {
        float sum = 0.f;
        const int ng = n_tot >> 2;
        int g = 0;
        for (; g + 4 <= ng; g += 4) {
            const float4 v = *reinterpret_cast<const float4 *>(gs + g);
            sum = __fadd_rn(sum, v.x); sum = __fadd_rn(sum, v.y); sum = __fadd_rn(sum, v.z); sum = __fadd_rn(sum, v.w);
        }
        for (; g < ng; ++g) { sum = __fadd_rn(sum, gs[g]); }
        for (int j = ng << 2; j < n_tot; ++j) { sum = __fadd_rn(sum, sc[j]); }
        bcast = __fdiv_rn(1.0f, sum);
    }
    __syncthreads();
    const float inv = bcast;
    // probabilities, rounded to fp16 as the PV MatMul does with its f32 operand
    for (int j = tid; j < n_vis; j += ATT_THREADS) { sc[j] = __half2float(__float2half_rn(__fmul_rn(sc[j], inv))); }
    __syncthreads();

    // ---- out[e] = Dot<FP16,FP16>(V_t[e][0..n_tot), probs): a thread pair per element, thread `half` holding
    // elements 4 * half .. + 3 of the four accumulators. Masked positions have probability +0 and leave every
    // accumulator unchanged, so they are skipped (their cache entries may not be written yet).
    {
        const int e = pv_e, half = pv_half;
        float acc[4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a) {
#pragma unroll
            for (int k = 0; k < 4; ++k) { acc[a][k] = 0.f; }
        }
        auto pv_step = [&](const uint2 (&vv)[4], int j0) {
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const int    j  = j0 + 8 * a + 4 * half;
                const float4 pr = *reinterpret_cast<const float4 *>(sc + j);
                const float2 v01 = __half22float2(*reinterpret_cast<const __half2 *>(&vv[a].x)), v23 = __half22float2(*reinterpret_cast<const __half2 *>(&vv[a].y));
                if (j + 0 < n_vis) { acc[a][0] = fmaf(v01.x, pr.x, acc[a][0]); }
                if (j + 1 < n_vis) { acc[a][1] = fmaf(v01.y, pr.y, acc[a][1]); }
                if (j + 2 < n_vis) { acc[a][2] = fmaf(v23.x, pr.z, acc[a][2]); }
                if (j + 3 < n_vis) { acc[a][3] = fmaf(v23.y, pr.w, acc[a][3]); }
            }
        };
        if (0 < n_main) { pv_step(v_first, 0); }
#pragma unroll
        for (int s = 0; s < PV_AHEAD; ++s) {
            const int j0 = 32 * (s + 1);
            if (s < n_ahead && j0 < n_main && j0 < n_vis) { pv_step(v_ahead[s], j0); }
        }
        {   // later steps: loads one step ahead of the arithmetic
            int j0 = 32 * (n_ahead + 1);
            uint2 vv[4], vn[4];
            auto fetch = [&](uint2 (&dst)[4], int jj0) {
#pragma unroll
                for (int a = 0; a < 4; ++a) {
                    const int j = jj0 + 8 * a + 4 * half;
                    dst[a] = (jj0 < n_main && j < n_vis) ? *reinterpret_cast<const uint2 *>(vrow + j) : make_uint2(0u, 0u);
                }
            };
            fetch(vv, j0);
            for (; j0 < n_main && j0 < n_vis; j0 += 32) {
                fetch(vn, j0 + 32);
                pv_step(vv, j0);
#pragma unroll
                for (int a = 0; a < 4; ++a) { vv[a] = vn[a]; }
            }
        }
        float u[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float mine = __fadd_rn(__fadd_rn(acc[0][k], acc[2][k]), __fadd_rn(acc[1][k], acc[3][k]));
            u[k] = __fadd_rn(mine, __shfl_xor_sync(0xffffffffu, mine, 1));   // element k of one half with element k + 4 of the other
        }
        const float simd = __fadd_rn(__fadd_rn(u[0], u[1]), __fadd_rn(u[2], u[3]));
        // scalar tail: positions n_main .. n_tot-1 (at most 32)
        float tail = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const int j = n_main + 4 * c;
            if (j < n_vis) {
                const float4 pr = *reinterpret_cast<const float4 *>(sc + j);
                const float2 v01 = __half22float2(*reinterpret_cast<const __half2 *>(&v_tail[c].x)), v23 = __half22float2(*reinterpret_cast<const __half2 *>(&v_tail[c].y));
                tail = fmaf(v01.x, pr.x, tail);
                if (j + 1 < n_vis) { tail = fmaf(v01.y, pr.y, tail); }
                if (j + 2 < n_vis) { tail = fmaf(v23.x, pr.z, tail); }
                if (j + 3 < n_vis) { tail = fmaf(v23.y, pr.w, tail); }
            }
        }
        if (half == 0) { p.out[(int64_t)t * (p.out_stride ? p.out_stride : p.dl) + (int64_t)h * ATT_HD + e] = __fadd_rn(tail, simd); }
    }
    tp_publish(p.tp, p.T);
    if (p.stamps != nullptr) { __syncthreads(); stamp(p.stamps, 3, true); }
}

// ---------------------------------------------------------------------------------------------
// Long contexts (n_ctx > ATT_LONG_MIN): the same arithmetic as attention_kernel, spread over the chip in three kernels
// that meet in a scratch buffer [T][n_head][n_ctx] of floats (scores, then probabilities):
//   attn_scores_kernel   one thread per (position, head, token): Dot<FP16,FP16>(K row, Q), all 32 accumulators in registers
//   attn_softmax_kernel  one CTA per (head, token): scale, maximum, table exp, std::reduce's grouped running sum, 1/sum,
//                        probabilities rounded to fp16
//   attn_pv_kernel       one warp per output element, lane = 8 * accumulator + element of the CPU's 4 x 8 accumulators
//                        (position j of a 32-step goes to lane j % 32), sixteen elements per CTA
// HBM-bound: the K rows and the V^T rows of the visible positions are read once (2 * n_kv * 128 * 2 bytes per head).
constexpr int ATT_LONG_MIN = 1024;

// Dot<FP16,FP16>(K row, Q) with the K row in registers (16 x 8 fp16) and Q as 128 floats in shared memory: 4 x 8
// accumulators over elements 0..95, the reduction tree, the scalar chain over elements 96..127, tail + simd
__device__ __forceinline__ float score_dot(const uint4 (&kv)[16], const float4 *q4) {
    // the 4 x 8 accumulators as 4 x 4 packed f32x2 pairs (elements 2 p, 2 p + 1 of an accumulator step): one fma.rn.f32x2 is two
    // of the scalar FMAs, bit for bit
    uint64_t acc2[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a) {
#pragma unroll
        for (int e = 0; e < 4; ++e) { acc2[a][e] = 0ull; }
    }
#pragma unroll
    for (int step = 0; step < 3; ++step) {       // elements 0..95: accumulator a takes elements 32 * step + 8a .. + 7
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const uint4 kw = kv[4 * step + a];
            const float2 k0 = __half22float2(*reinterpret_cast<const __half2 *>(&kw.x)), k1 = __half22float2(*reinterpret_cast<const __half2 *>(&kw.y));
            const float2 k2 = __half22float2(*reinterpret_cast<const __half2 *>(&kw.z)), k3 = __half22float2(*reinterpret_cast<const __half2 *>(&kw.w));
            const float4 qa = q4[(4 * step + a) * 2], qb = q4[(4 * step + a) * 2 + 1];
            acc2[a][0] = f2_fma(f2_pack(k0.x, k0.y), f2_pack(qa.x, qa.y), acc2[a][0]);
            acc2[a][1] = f2_fma(f2_pack(k1.x, k1.y), f2_pack(qa.z, qa.w), acc2[a][1]);
            acc2[a][2] = f2_fma(f2_pack(k2.x, k2.y), f2_pack(qb.x, qb.y), acc2[a][2]);
            acc2[a][3] = f2_fma(f2_pack(k3.x, k3.y), f2_pack(qb.z, qb.w), acc2[a][3]);
        }
    }
    float acc[4][8];
#pragma unroll
    for (int a = 0; a < 4; ++a) {
#pragma unroll
        for (int e = 0; e < 4; ++e) { f2_unpack(acc2[a][e], acc[a][2 * e], acc[a][2 * e + 1]); }
    }
    float u[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float lo = __fadd_rn(__fadd_rn(acc[0][e], acc[2][e]), __fadd_rn(acc[1][e], acc[3][e]));
        const float hi = __fadd_rn(__fadd_rn(acc[0][e + 4], acc[2][e + 4]), __fadd_rn(acc[1][e + 4], acc[3][e + 4]));
        u[e] = __fadd_rn(lo, hi);
    }
    const float simd = __fadd_rn(__fadd_rn(u[0], u[1]), __fadd_rn(u[2], u[3]));
    float tail = 0.f;                             // elements 96..127: scalar chain
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        float kf[8]; unpack8(kv[12 + a], kf);
        const float4 qa = q4[(12 + a) * 2], qb = q4[(12 + a) * 2 + 1];
        const float  qv[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) { tail = fmaf(kf[e], qv[e], tail); }
    }
    return __fadd_rn(tail, simd);
}

__global__ void __launch_bounds__(256) attn_scores_kernel(const AttnParams p) {
    __shared__ __align__(16) float qf[ATT_HD];
    const int h = blockIdx.y, t = blockIdx.z, tid = threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const bool batch = p.seq_stride != 0;
    const int n_vis = p.pos_base[0] + (batch ? 0 : t) + 1;
    if ((int)blockIdx.x * 256 >= n_vis) { return; }
    const int n_pad = (p.n_ctx + 3) & ~3;
    if (tid < ATT_HD) { qf[tid] = __half2float(p.q[(int64_t)t * p.dl + (int64_t)h * ATT_HD + tid]); }
    __syncthreads();
    const int j = blockIdx.x * 256 + tid;
    if (j >= n_vis) { return; }
    uint4 kv[16];
    {
        const uint4 *krow = reinterpret_cast<const uint4 *>(p.k_cache + (batch ? (int64_t)t * p.seq_stride : 0) + (int64_t)j * p.dl + (int64_t)h * ATT_HD);
#pragma unroll
        for (int a = 0; a < 16; ++a) { kv[a] = krow[a]; }
    }
    p.scratch[((int64_t)t * p.n_head + h) * n_pad + j] = score_dot(kv, reinterpret_cast<const float4 *>(qf));
}

// The same for a prompt: ATT_TT consecutive tokens per CTA share the K rows, which stay in the threads' registers while
// the tokens are walked (the K cache is then read once per ATT_TT tokens instead of once per token)
constexpr int ATT_TT = 8;
__global__ void __launch_bounds__(256) attn_scores_tiled_kernel(const AttnParams p) {
    __shared__ __align__(16) float qf[ATT_TT][ATT_HD];
    const int h = blockIdx.y, t0 = blockIdx.z * ATT_TT, tid = threadIdx.x;
    const int nt = min(ATT_TT, p.T - t0);
    const int n_vis_last = p.pos_base[0] + t0 + nt;          // positions the last token of the tile sees
    if ((int)blockIdx.x * 256 >= n_vis_last) { return; }
    const int n_pad = (p.n_ctx + 3) & ~3;
    for (int i = tid; i < nt * ATT_HD; i += 256) { qf[i / ATT_HD][i % ATT_HD] = __half2float(p.q[(int64_t)(t0 + i / ATT_HD) * p.dl + (int64_t)h * ATT_HD + i % ATT_HD]); }
    __syncthreads();
    const int j = blockIdx.x * 256 + tid;
    if (j >= n_vis_last) { return; }
    uint4 kv[16];
    {
        const uint4 *krow = reinterpret_cast<const uint4 *>(p.k_cache + (int64_t)j * p.dl + (int64_t)h * ATT_HD);
#pragma unroll
        for (int a = 0; a < 16; ++a) { kv[a] = krow[a]; }
    }
#pragma unroll 1
    for (int tt = 0; tt < nt; ++tt) {
        if (j > p.pos_base[0] + t0 + tt) { continue; }       // masked for this token
        p.scratch[((int64_t)(t0 + tt) * p.n_head + h) * n_pad + j] = score_dot(kv, reinterpret_cast<const float4 *>(qf[tt]));
    }
}

constexpr int ATT_SM_THREADS = 1024;
__global__ void __launch_bounds__(ATT_SM_THREADS) attn_softmax_kernel(const AttnParams p) {
    extern __shared__ __align__(16) float att_smem[];
    __shared__ float red[ATT_SM_THREADS / WARP];
    __shared__ float bcast;
    const int h = blockIdx.x, t = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nthr = blockDim.x;   // 1024 for single steps (one CTA per head: latency), 256 for prompts (many CTAs: more of them per SM, so that
                                   // one CTA's serial sum overlaps the parallel phases of the others)
    pdl_launch_dependents();
    pdl_wait();
    const bool batch = p.seq_stride != 0;
    const int n_vis = p.pos_base[0] + (batch ? 0 : t) + 1;
    const int n_tot = batch ? n_vis : (p.pos_base[1] > 0) ? p.pos_base[1] : p.pos_base[0] + p.T;
    const int n_pad = (p.n_ctx + 3) & ~3;
    float *sc = att_smem, *gs = sc + n_pad;
    float *row = p.scratch + ((int64_t)t * p.n_head + h) * n_pad;
    // masked softmax: (score + mask) * scale, subtract the maximum, table exp, std::reduce, multiply by 1/sum
    float m = -CUDART_INF_F;
    for (int j = tid; j < n_vis; j += nthr) {
        const float v = __fmul_rn(__fadd_rn(row[j], 0.0f), p.scale);
        sc[j] = v;
        m = fmaxf(m, v);
    }
    m = warp_max(m);
    if (lane == 0) { red[warp] = m; }
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < ATT_SM_THREADS / WARP; ++w) { if (w < (nthr >> 5)) { m = fmaxf(m, red[w]); } }
    const int n_tot4 = (n_tot + 3) & ~3;
    for (int j = tid; j < n_tot4; j += nthr) { sc[j] = (j < n_vis) ? p.exp_table[f2h(__fsub_rn(sc[j], m))] : 0.f; }
    __syncthreads();
    for (int g = tid; g < (n_tot >> 2); g += nthr) {
        const float4 v = reinterpret_cast<const float4 *>(sc)[g];
        gs[g] = __fadd_rn(__fadd_rn(v.x, v.y), __fadd_rn(v.z, v.w));
    }
    __syncthreads();
    if (tid == 0) {
        float sum = 0.f;
        const int ng = n_tot >> 2;
        int g = 0;
        for (; g + 4 <= ng; g += 4) {
            const float4 v = *reinterpret_cast<const float4 *>(gs + g);
            sum = __fadd_rn(sum, v.x); sum = __fadd_rn(sum, v.y); sum = __fadd_rn(sum, v.z); sum = __fadd_rn(sum, v.w);
        }
        for (; g < ng; ++g) { sum = __fadd_rn(sum, gs[g]); }
        for (int j = ng << 2; j < n_tot; ++j) { sum = __fadd_rn(sum, sc[j]); }
        bcast = __fdiv_rn(1.0f, sum);
    }
    __syncthreads();
    const float inv = bcast;
    // probabilities, rounded to fp16 as the PV MatMul does with its f32 operand
    for (int j = tid; j < n_vis; j += nthr) { row[j] = __half2float(__float2half_rn(__fmul_rn(sc[j], inv))); }
}

constexpr int ATT_PV_WARPS = 16;
__global__ void __launch_bounds__(ATT_PV_WARPS * WARP) attn_pv_kernel(const AttnParams p) {
    extern __shared__ __align__(16) float att_smem[];
    const int per_head = ATT_HD / ATT_PV_WARPS;
    const int h = blockIdx.x / per_head, e = (blockIdx.x % per_head) * ATT_PV_WARPS + (threadIdx.x >> 5), t = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31;
    pdl_launch_dependents();
    pdl_wait();
    const bool batch = p.seq_stride != 0;
    const int n_vis = p.pos_base[0] + (batch ? 0 : t) + 1;
    const int n_tot = batch ? n_vis : (p.pos_base[1] > 0) ? p.pos_base[1] : p.pos_base[0] + p.T;
    const int n_pad = (p.n_ctx + 3) & ~3;
    const int n_main = ((n_tot - 1) / 32) * 32;
    float *pr = att_smem;
    const float *row = p.scratch + ((int64_t)t * p.n_head + h) * n_pad;
    for (int j = tid; j < n_vis; j += ATT_PV_WARPS * WARP) { pr[j] = row[j]; }
    __syncthreads();
    // out[e] = Dot<FP16,FP16>(V_t[e][0..n_tot), probs); masked positions have probability +0 and leave every accumulator
    // unchanged, so they are skipped (their cache entries may not be written yet)
    const __half *vrow = p.v_cache + (batch ? (int64_t)t * p.seq_stride : 0) + ((int64_t)h * ATT_HD + e) * p.n_ctx;
    float acc = 0.f;
    int j0 = 0;
    for (; j0 + 8 * 32 <= n_main && j0 + 8 * 32 <= n_vis; j0 += 8 * 32) {   // eight steps' loads in flight
        float v[8];
#pragma unroll
        for (int s = 0; s < 8; ++s) { v[s] = __half2float(vrow[j0 + 32 * s + lane]); }
#pragma unroll
        for (int s = 0; s < 8; ++s) { acc = fmaf(v[s], pr[j0 + 32 * s + lane], acc); }
    }
    for (; j0 < n_main; j0 += 32) {
        const int j = j0 + lane;
        if (j < n_vis) { acc = fmaf(__half2float(vrow[j]), pr[j], acc); }
    }
    acc = reduce_f16dot_lanes(acc);
    const float vt = (n_main + lane < n_vis) ? __half2float(vrow[n_main + lane]) : 0.f;
    float tail = 0.f;                         // positions n_main .. n_tot-1 (at most 32): scalar chain
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
        const float v = __shfl_sync(0xffffffffu, vt, i);
        if (n_main + i < n_vis) { tail = fmaf(v, pr[n_main + i], tail); }
    }
    if (lane == 0) { p.out[(int64_t)t * (p.out_stride ? p.out_stride : p.dl) + (int64_t)h * ATT_HD + e] = __fadd_rn(tail, acc); }
    tp_publish(p.tp, p.T);
}

// PV for a prompt: ATT_TT consecutive tokens per CTA share the V^T rows, and a warp takes ATT_EE output elements, so that a
// probability read from shared memory serves ATT_EE products. Every token's product is the untiled kernel's (same lanes,
// same steps, same tail); only the loads are shared.
constexpr int ATT_EE = 4;
__global__ void __launch_bounds__(ATT_PV_WARPS * WARP) attn_pv_tiled_kernel(const AttnParams p) {
    extern __shared__ __align__(16) float att_smem[];
    constexpr int PER_CTA = ATT_PV_WARPS * ATT_EE;            // output elements per CTA
    const int per_head = ATT_HD / PER_CTA;
    const int h = blockIdx.x / per_head, e0 = (blockIdx.x % per_head) * PER_CTA + (threadIdx.x >> 5) * ATT_EE, t0 = blockIdx.y * ATT_TT;
    const int tid = threadIdx.x, lane = tid & 31;
    const int nt = min(ATT_TT, p.T - t0);
    const int n_tot = (p.pos_base[1] > 0) ? p.pos_base[1] : p.pos_base[0] + p.T;
    const int n_pad = (p.n_ctx + 3) & ~3;
    const int n_main = ((n_tot - 1) / 32) * 32;
    const int vis0 = p.pos_base[0] + t0 + 1;                  // positions token t0 + tt sees: vis0 + tt
    const int vis_last = vis0 + nt - 1;
    // probabilities of the tile's tokens; positions a token does not see read as +0 (they leave its accumulators unchanged)
    for (int tt = 0; tt < nt; ++tt) {
        const float *row = p.scratch + ((int64_t)(t0 + tt) * p.n_head + h) * n_pad;
        float *pr = att_smem + (size_t)tt * n_pad;
        for (int j = tid; j < vis_last; j += ATT_PV_WARPS * WARP) { pr[j] = (j < vis0 + tt) ? row[j] : 0.f; }
    }
    __syncthreads();
    const __half *vrow = p.v_cache + ((int64_t)h * ATT_HD + e0) * p.n_ctx;   // row e0 + ee starts ee * n_ctx further
    float acc[ATT_TT][ATT_EE];
#pragma unroll
    for (int tt = 0; tt < ATT_TT; ++tt) {
#pragma unroll
        for (int ee = 0; ee < ATT_EE; ++ee) { acc[tt][ee] = 0.f; }
    }
    int j0 = 0;
    if (nt == ATT_TT) {
        // positions every token of the tile sees, in chunks of four 32-position steps: no masks to test, and the V^T values of
        // the next chunk are requested before the products of this one, so that their latency hides behind 128 FMAs per thread
        constexpr int CH = 4;
        const int full_end = (min(n_main, vis0) / (32 * CH)) * (32 * CH);
        __half vh[CH][ATT_EE];
        if (full_end > 0) {
#pragma unroll
            for (int s = 0; s < CH; ++s) {
#pragma unroll
                for (int ee = 0; ee < ATT_EE; ++ee) { vh[s][ee] = vrow[(int64_t)ee * p.n_ctx + 32 * s + lane]; }
            }
        }
        for (; j0 < full_end; j0 += 32 * CH) {
            float v[CH][ATT_EE];
#pragma unroll
            for (int s = 0; s < CH; ++s) {
#pragma unroll
                for (int ee = 0; ee < ATT_EE; ++ee) { v[s][ee] = __half2float(vh[s][ee]); }
            }
            if (j0 + 32 * CH < full_end) {
#pragma unroll
                for (int s = 0; s < CH; ++s) {
#pragma unroll
                    for (int ee = 0; ee < ATT_EE; ++ee) { vh[s][ee] = vrow[(int64_t)ee * p.n_ctx + j0 + 32 * (CH + s) + lane]; }
                }
            }
#pragma unroll
            for (int tt = 0; tt < ATT_TT; ++tt) {
                const float *pr = att_smem + (size_t)tt * n_pad + j0 + lane;
#pragma unroll
                for (int s = 0; s < CH; ++s) {
                    const float pv = pr[32 * s];
#pragma unroll
                    for (int ee = 0; ee < ATT_EE; ++ee) { acc[tt][ee] = fmaf(v[s][ee], pv, acc[tt][ee]); }
                }
            }
        }
    }
    for (; j0 + 2 * 32 <= n_main && j0 + 2 * 32 <= vis_last; j0 += 2 * 32) {   // two steps' loads in flight per element
        float v[2][ATT_EE];
#pragma unroll
        for (int s = 0; s < 2; ++s) {
#pragma unroll
            for (int ee = 0; ee < ATT_EE; ++ee) { v[s][ee] = __half2float(vrow[(int64_t)ee * p.n_ctx + j0 + 32 * s + lane]); }
        }
#pragma unroll
        for (int tt = 0; tt < ATT_TT; ++tt) {
            if (tt < nt) {
                const float *pr = att_smem + (size_t)tt * n_pad;
#pragma unroll
                for (int s = 0; s < 2; ++s) {
                    if (j0 + 32 * s < vis0 + tt) {   // (a step wholly behind the token's last position adds nothing: skipped as in the untiled kernel)
                        const float pv = pr[j0 + 32 * s + lane];
#pragma unroll
                        for (int ee = 0; ee < ATT_EE; ++ee) { acc[tt][ee] = fmaf(v[s][ee], pv, acc[tt][ee]); }
                    }
                }
            }
        }
    }
    for (; j0 < n_main && j0 < vis_last; j0 += 32) {   // (steps behind the tile's last visible position add nothing)
        const int j = j0 + lane;
        float v[ATT_EE];
#pragma unroll
        for (int ee = 0; ee < ATT_EE; ++ee) { v[ee] = (j < vis_last) ? __half2float(vrow[(int64_t)ee * p.n_ctx + j]) : 0.f; }
#pragma unroll
        for (int tt = 0; tt < ATT_TT; ++tt) {
            if (tt < nt && j < vis0 + tt) {
                const float pv = att_smem[(size_t)tt * n_pad + j];
#pragma unroll
                for (int ee = 0; ee < ATT_EE; ++ee) { acc[tt][ee] = fmaf(v[ee], pv, acc[tt][ee]); }
            }
        }
    }
    // The vector parts: reduce_f16dot_lanes leaves every lane with the sum; lane 4 tt + ee keeps that of (token tt, element ee).
    static_assert(ATT_TT * ATT_EE == WARP, "one lane per (token, element) of the warp's outputs");
    const int my_tt = lane >> 2, my_ee = lane & 3;
    float vec = 0.f;
#pragma unroll
    for (int tt = 0; tt < ATT_TT; ++tt) {
#pragma unroll
        for (int ee = 0; ee < ATT_EE; ++ee) {
            const float a = reduce_f16dot_lanes(acc[tt][ee]);
            if (lane == tt * ATT_EE + ee) { vec = a; }
        }
    }
    // The scalar tails (positions n_main .. n_tot - 1, at most 32, one FMA chain per output): each lane runs the chain of its own
    // (token, element) instead of all lanes running all 32 chains; the V^T value of position n_main + i sits in lane i
    float vt[ATT_EE];
#pragma unroll
    for (int ee = 0; ee < ATT_EE; ++ee) { vt[ee] = (n_main + lane < vis_last) ? __half2float(vrow[(int64_t)ee * p.n_ctx + n_main + lane]) : 0.f; }
    float tail = 0.f;
    const float *pr_mine = att_smem + (size_t)my_tt * n_pad + n_main;
    const int n_tail = min(32, vis0 + my_tt - n_main);        // positions of the tail this lane's token sees (<= 0: none)
#pragma unroll 4
    for (int i = 0; i < 32; ++i) {
        float v = 0.f;
#pragma unroll
        for (int ee = 0; ee < ATT_EE; ++ee) {
            const float w = __shfl_sync(0xffffffffu, vt[ee], i);
            if (my_ee == ee) { v = w; }
        }
        if (i < n_tail) { tail = fmaf(v, pr_mine[i], tail); }
    }
    if (my_tt < nt) { p.out[(int64_t)(t0 + my_tt) * (p.out_stride ? p.out_stride : p.dl) + (int64_t)h * ATT_HD + e0 + my_ee] = __fadd_rn(tail, vec); }
}

static cudaError_t launch_with_pdl(const void *kernel, dim3 grid, dim3 block, size_t smem, const AttnParams &p, const LaunchCfg &cfg) {
    cudaLaunchConfig_t lc = {};
    lc.gridDim = grid; lc.blockDim = block; lc.dynamicSmemBytes = smem; lc.stream = cfg.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr; lc.numAttrs = cfg.pdl ? 1 : 0;
    void *args[] = {const_cast<AttnParams *>(&p)};
    return cudaLaunchKernelExC(&lc, kernel, args);
}

size_t attention_scratch_floats(int n_ctx, int n_head, int T) {   // 0: the single-kernel path serves this context length
    if (n_ctx <= ATT_LONG_MIN) { return 0; }
    return (size_t)T * n_head * (((size_t)n_ctx + 3) & ~(size_t)3);
}

cudaError_t launch_attention(const AttnParams &p, const LaunchCfg &cfg) {
    if (p.hd != ATT_HD || p.T < 1 || p.n_ctx < 1 || (p.n_ctx & 3) || (p.dl & 7)) { return cudaErrorInvalidValue; }
    const size_t n_pad = ((size_t)p.n_ctx + 3) & ~(size_t)3;
    if ((p.n_ctx > ATT_LONG_MIN || p.force_long) && p.scratch != nullptr) {
        const bool tiled = p.T >= ATT_TT && p.tp.counter == nullptr && !cfg.pdl && p.seq_stride == 0;   // a prompt: tokens share the K rows and the V^T rows
        cudaError_t err = tiled
            ? launch_with_pdl(reinterpret_cast<const void *>(attn_scores_tiled_kernel), dim3((unsigned)((p.n_ctx + 255) / 256), p.n_head, (unsigned)((p.T + ATT_TT - 1) / ATT_TT)), dim3(256), 0, p, cfg)
            : launch_with_pdl(reinterpret_cast<const void *>(attn_scores_kernel), dim3((unsigned)((p.n_ctx + 255) / 256), p.n_head, p.T), dim3(256), 0, p, cfg);
        if (err != cudaSuccess) { return err; }
        const size_t sm_smem = (n_pad + n_pad / 4) * sizeof(float) + 16;
        if (sm_smem > 200 * 1024) { return cudaErrorInvalidValue; }
        err = allow_dynamic_smem(reinterpret_cast<const void *>(attn_softmax_kernel), sm_smem);
        if (err != cudaSuccess) { return err; }
        err = launch_with_pdl(reinterpret_cast<const void *>(attn_softmax_kernel), dim3(p.n_head, p.T), dim3(tiled ? 256 : ATT_SM_THREADS), sm_smem, p, cfg);
        if (err != cudaSuccess) { return err; }
        if (tiled && (size_t)ATT_TT * n_pad * sizeof(float) + 16 <= 200 * 1024) {
            const size_t tsm = (size_t)ATT_TT * n_pad * sizeof(float) + 16;
            err = allow_dynamic_smem(reinterpret_cast<const void *>(attn_pv_tiled_kernel), tsm);
            if (err != cudaSuccess) { return err; }
            return launch_with_pdl(reinterpret_cast<const void *>(attn_pv_tiled_kernel), dim3(p.n_head * (ATT_HD / (ATT_PV_WARPS * ATT_EE)), (unsigned)((p.T + ATT_TT - 1) / ATT_TT)),
                                   dim3(ATT_PV_WARPS * WARP), tsm, p, cfg);
        }
        const size_t pv_smem = n_pad * sizeof(float) + 16;
        err = allow_dynamic_smem(reinterpret_cast<const void *>(attn_pv_kernel), pv_smem);
        if (err != cudaSuccess) { return err; }
        return launch_with_pdl(reinterpret_cast<const void *>(attn_pv_kernel), dim3(p.n_head * (ATT_HD / ATT_PV_WARPS), p.T), dim3(ATT_PV_WARPS * WARP), pv_smem, p, cfg);
    }
    const size_t smem = (n_pad + n_pad / 4 + ATT_HD) * sizeof(float) + 16;
    if (smem > 200 * 1024) { return cudaErrorInvalidValue; }
    cudaError_t err = allow_dynamic_smem(reinterpret_cast<const void *>(attention_kernel), smem);
    if (err != cudaSuccess) { return err; }
    return launch_with_pdl(reinterpret_cast<const void *>(attention_kernel), dim3(p.n_head, p.T, 1), dim3(ATT_THREADS), smem, p, cfg);
}

// =============================================================================================
// upload-time re-tiling: raw 18-byte / 34-byte blocks -> the record stream described at DevMatrix
// (one thread per padded block; blocks beyond nb are written as zeros with a zero scale)
template <int WORDS, bool MMA>   // WORDS 4: Q4_0 (16 nibble bytes), 8: Q8_0 (32 int8 values); MMA: the fragment-ordered record of DevMatrix::mma
__global__ void retile_kernel(const uint8_t *raw, int64_t row_stride, int64_t n_rows, int nb, int nbp, uint8_t *base, int tile_rows,
                              int64_t dst_row0, int64_t src_row0, int sub_rows, int sub_off) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows * nbp) { return; }
    const int64_t  lrow = i / nbp;
    const int      b = (int)(i - lrow * nbp);
    const uint8_t *src = raw + lrow * row_stride + (int64_t)b * (2 + 4 * WORDS);
    const bool     real = b < nb;
    constexpr int  ROWB = WORDS * 32 + 16;
    const int64_t  srow = src_row0 + lrow;
    const int64_t  row  = dst_row0 + (sub_rows > 0 ? (srow / sub_rows) * tile_rows + sub_off + srow % sub_rows : srow);
    const int      r    = (int)(row % tile_rows);
    uint8_t  *rec = base + ((row / tile_rows) * (nbp >> 3) + (b >> 3)) * ((int64_t)tile_rows * ROWB);
    const uint16_t d = real ? (uint16_t)(src[0] | (src[1] << 8)) : (uint16_t)0;
    const int      grp_bytes = tile_rows * WORDS * 16;   // MMA: quants of one group of four blocks, all rows of the tile
    if (MMA) { reinterpret_cast<uint16_t *>(rec + 2 * grp_bytes + r * 16)[b & 7] = d; }
    else     { reinterpret_cast<uint16_t *>(rec + r * ROWB + WORDS * 32)[b & 7] = d; }
#pragma unroll
    for (int k = 0; k < WORDS; ++k) {
        uint32_t v = real ? (uint32_t)(src[2 + 4 * k] | (src[3 + 4 * k] << 8) | (src[4 + 4 * k] << 16) | ((uint32_t)src[5 + 4 * k] << 24)) : 0u;
        if (WORDS == 4) { v ^= 0x88888888u; }
        if (MMA) {   // [group][half of the block][row][word of the half] x 16 B, the four blocks of the group side by side
            reinterpret_cast<uint32_t *>(rec + ((b >> 2) & 1) * grp_bytes + (((k >> 2) * tile_rows + r) * 4 + (k & 3)) * 16)[b & 3] = v;
        } else {
            reinterpret_cast<uint32_t *>(rec + r * ROWB + ((b >> 2) & 1) * (WORDS * 16))[(b & 3) + 4 * k] = v;
        }
    }
}

cudaError_t launch_retile(int type, const uint8_t *raw, int64_t row_stride, int64_t n_rows, int nb, uint8_t *matrix_base, int tile_rows, bool mma,
                          int64_t dst_row0, int64_t src_row0, int sub_rows, int sub_off, cudaStream_t s) {
    const int     nbp = padded_blocks(nb);
    const int64_t n = n_rows * nbp;
    if (n == 0) { return cudaSuccess; }
    if (tile_rows != 4 && tile_rows != 8 && tile_rows != 16 && tile_rows != 32) { return cudaErrorInvalidValue; }
    if (mma && tile_rows != 8 && tile_rows != 16) { return cudaErrorInvalidValue; }
    const unsigned grid = (unsigned)((n + 255) / 256);
    if (type == 2) {
        if (mma) { retile_kernel<4, true><<<grid, 256, 0, s>>>(raw, row_stride, n_rows, nb, nbp, matrix_base, tile_rows, dst_row0, src_row0, sub_rows, sub_off); }
        else     { retile_kernel<4, false><<<grid, 256, 0, s>>>(raw, row_stride, n_rows, nb, nbp, matrix_base, tile_rows, dst_row0, src_row0, sub_rows, sub_off); }
    } else if (type == 8) {
        if (mma) { retile_kernel<8, true><<<grid, 256, 0, s>>>(raw, row_stride, n_rows, nb, nbp, matrix_base, tile_rows, dst_row0, src_row0, sub_rows, sub_off); }
        else     { retile_kernel<8, false><<<grid, 256, 0, s>>>(raw, row_stride, n_rows, nb, nbp, matrix_base, tile_rows, dst_row0, src_row0, sub_rows, sub_off); }
    } else { return cudaErrorNotSupported; }
    return launch_check();
}

// =============================================================================================
// Q8_0 quantizer writing the reference's 34-byte blocks (backend/host/include/simd/vec_convert.h:178-261)
__global__ void quantize_q8_0_ref_kernel(const float *x, int64_t n4, uint8_t *blocks) {
    const int64_t base = (int64_t)blockIdx.x * blockDim.x;
    const int64_t g    = base + threadIdx.x;
    const bool    valid = g < n4;
    const float4  v = valid ? reinterpret_cast<const float4 *>(x)[g] : make_float4(0.f, 0.f, 0.f, 0.f);
    uint16_t dh; int s;
    const uint32_t q = quantize_q8_lane4(v, dh, s);
    if (!valid) { return; }
    uint8_t *o = blocks + (g >> 3) * 34;
    const int li = (int)(g & 7);
    if (li == 0) { o[0] = (uint8_t)(dh & 0xff); o[1] = (uint8_t)(dh >> 8); }
    o[2 + 4 * li] = (uint8_t)(q & 0xff); o[3 + 4 * li] = (uint8_t)((q >> 8) & 0xff);
    o[4 + 4 * li] = (uint8_t)((q >> 16) & 0xff); o[5 + 4 * li] = (uint8_t)(q >> 24);
}

cudaError_t launch_quantize_q8_0_ref_layout(const float *x, int64_t n, uint8_t *blocks, cudaStream_t s) {
    if (n % QK != 0) { return cudaErrorInvalidValue; }
    if (n == 0) { return cudaSuccess; }
    const int64_t n4 = n / 4;
    quantize_q8_0_ref_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, s>>>(x, n4, blocks);
    return launch_check();
}

// per-block int32 dots through the same device functions the mat-vec uses (one thread per block)
__global__ void block_dots_kernel(int wtype, const uint8_t *w, const uint8_t *xb, int64_t nblk, int32_t *out) {
    const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblk) { return; }
    const uint8_t *y = xb + b * 34 + 2;
    uint32_t yw[8];
    for (int k = 0; k < 8; ++k) {
        yw[k] = y[4 * k] | (y[4 * k + 1] << 8) | (y[4 * k + 2] << 16) | ((uint32_t)y[4 * k + 3] << 24);
    }
    int total = 0;
    if (wtype == 2) {
        const uint8_t *q = w + b * 18 + 2;
        for (int k = 0; k < 4; ++k) {
            const uint32_t ww = q[4 * k] | (q[4 * k + 1] << 8) | (q[4 * k + 2] << 16) | ((uint32_t)q[4 * k + 3] << 24);
            const float hi = lane_sum16_q4_0(ww ^ 0x88888888u, 1u, yw[4 + k]);   // both come scaled by 16
            const float lo = lane_sum16_q4_0(ww ^ 0x88888888u, 16u, yw[k]);
            total += (int)hi / 16 + (int)lo / 16;
        }
    } else {
        const uint8_t *q = w + b * 34 + 2;
        for (int k = 0; k < 8; ++k) {
            const uint32_t ww = q[4 * k] | (q[4 * k + 1] << 8) | (q[4 * k + 2] << 16) | ((uint32_t)q[4 * k + 3] << 24);
            total += (int)lane_sum_q8_0(ww, yw[k]);
        }
    }
    out[b] = total;
}

cudaError_t launch_block_dots(int wtype, const uint8_t *w_row, const uint8_t *x_blocks, int64_t n, int32_t *out, cudaStream_t s) {
    if ((wtype != 2 && wtype != 8) || n % QK != 0) { return cudaErrorInvalidValue; }
    const int64_t nblk = n / QK;
    if (nblk == 0) { return cudaSuccess; }
    block_dots_kernel<<<(unsigned)((nblk + 127) / 128), 128, 0, s>>>(wtype, w_row, x_blocks, nblk, out);
    return launch_check();
}

// =============================================================================================
// K-quant weights (Q4_K: 144 B / 256 elements, Q6_K: 210 B / 256 elements; layouts
// orchestration/include/number/number_impl/k-quant.h:79-117, 162-188). The reference defines only the block layouts
// and has no compute for them, so there is nothing to be bit-identical to: the kernel multiplies the decoded weights
// with the f32 activations (the reference's MatMul semantics without an activation quantizer) and is checked against
// a numpy decode within the stated tolerance. One warp per output row and column; a lane decodes 8 consecutive
// elements of every 256-element super-block, so a warp reads each 144 / 210-byte block once, contiguously.
// HBM-bound: rows * K/256 * 144 (210) bytes per launch; activations stay in L2.
__device__ __forceinline__ void kq_scale_min_k4(const uint8_t *sc12, int j, float &sc, float &mn) {
    if (j < 4) { sc = (float)(sc12[j] & 63); mn = (float)(sc12[4 + j] & 63); }
    else { sc = (float)((sc12[4 + j] & 0xF) | ((sc12[j - 4] >> 6) << 4)); mn = (float)((sc12[4 + j] >> 4) | ((sc12[j] >> 6) << 4)); }
}

template <int TYPE>   // 12: Q4_K, 14: Q6_K
__global__ void __launch_bounds__(256) matmul_kquant_kernel(const uint8_t *w, int64_t row_bytes, const float *x, float *out, int64_t n_rows,
                                                            int64_t k, int64_t n_cols) {
    const int     lane = threadIdx.x & 31;
    const int64_t gw = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nw = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t nsb = k >> 8;
    for (int64_t item = gw; item < n_rows * n_cols; item += nw) {
        const int64_t  row = item % n_rows, col = item / n_rows;
        const uint8_t *wr = w + row * row_bytes;
        const float   *xc = x + col * k;
        float acc = 0.f;
        for (int64_t b = 0; b < nsb; ++b) {
            const float4 x0 = *reinterpret_cast<const float4 *>(xc + b * 256 + lane * 8), x1 = *reinterpret_cast<const float4 *>(xc + b * 256 + lane * 8 + 4);
            const float  xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
            if (TYPE == 12) {
                const uint8_t *blk = wr + b * 144;
                const float d = h2f((uint16_t)(blk[0] | (blk[1] << 8))), dmin = h2f((uint16_t)(blk[2] | (blk[3] << 8)));
                // elements 8*lane .. 8*lane+7 lie in sub-block j = lane / 4; 64-element group g = j / 2 keeps its first 32
                // elements in the low nibbles and the next 32 in the high nibbles of bytes 32g .. 32g+31
                const int j = lane >> 2, g = j >> 1, hi = j & 1, off = (lane & 3) * 8;
                float sc, mn; kq_scale_min_k4(blk + 4, j, sc, mn);
                const uint2 q = *reinterpret_cast<const uint2 *>(blk + 16 + 32 * g + off);
                const float dl = __fmul_rn(d, sc), ml = __fmul_rn(dmin, mn);
                float part = 0.f, xs = 0.f;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const uint32_t byte = ((e < 4 ? q.x : q.y) >> (8 * (e & 3))) & 0xff;
                    part = fmaf((float)(hi ? (byte >> 4) : (byte & 0xF)), xv[e], part);
                    xs += xv[e];
                }
                acc += dl * part - ml * xs;
            } else {
                const uint8_t *blk = wr + b * 210;
                const float d = h2f((uint16_t)(blk[208] | (blk[209] << 8)));
                // element i = 8*lane + e: half h = i / 128, quarter qq = (i % 128) / 32, l = i % 32; six bits =
                // nibble of ql[64h + 32(qq & 1) + l] (low for qq < 2, high else) | two bits (2*qq) of qh[32h + l]
                const int i0 = lane * 8, h = i0 >> 7, qq = (i0 & 127) >> 5, l0 = i0 & 31;
                const uint8_t *ql = blk + 64 * h + 32 * (qq & 1) + l0;   // 210-byte blocks: only 2-byte alignment holds, byte loads
                const uint8_t *qh = blk + 128 + 32 * h + l0;
                const float sc = (float)(int8_t)blk[192 + (i0 >> 4)];
                float part = 0.f;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const uint32_t byte = ql[e];
                    const int      six  = (int)((qq < 2 ? (byte & 0xF) : (byte >> 4)) | (((qh[e] >> (2 * qq)) & 3) << 4)) - 32;
                    part = fmaf((float)six, xv[e], part);
                }
                acc += __fmul_rn(d, sc) * part;
            }
        }
        acc = warp_sum(acc);
        if (lane == 0) { out[col * n_rows + row] = acc; }
    }
}

cudaError_t launch_matmul_kquant(int type, const uint8_t *w, int64_t n_rows, int64_t k, const float *x, int64_t n_cols, float *out, cudaStream_t s) {
    if ((type != 12 && type != 14) || k % 256 != 0) { return cudaErrorInvalidValue; }
    if (n_rows == 0 || n_cols == 0) { return cudaSuccess; }
    const int64_t warps = n_rows * n_cols;
    const unsigned grid = (unsigned)std::min<int64_t>((warps + 7) / 8, 148 * 8);
    if (type == 12) { matmul_kquant_kernel<12><<<grid, 256, 0, s>>>(w, k / 256 * 144, x, out, n_rows, k, n_cols); }
    else            { matmul_kquant_kernel<14><<<grid, 256, 0, s>>>(w, k / 256 * 210, x, out, n_rows, k, n_cols); }
    return launch_check();
}

// =============================================================================================
// per-operator kernels (each mirrors one OperatorImpl of backend/host/operator/*.cpp)

// OperatorNormRMSImpl::execute, non-linear.cpp:194-223; one CTA per row. Sum of squares in the order of
// std::transform_reduce: (x0^2 + x1^2) + (x2^2 + x3^2) per group of four (second product of each pair fused into the first),
// groups added to the running sum in order.
__global__ void rmsnorm_kernel(const float *x, float *out, int64_t n, float eps) {
    extern __shared__ __align__(16) float v3[];
    __shared__ float scale_s;
    const float *xr = x + (int64_t)blockIdx.x * n;
    float       *o  = out + (int64_t)blockIdx.x * n;
    const int n4 = (int)(n >> 2);
    for (int g = threadIdx.x; g < n4; g += blockDim.x) {
        const float4 v = reinterpret_cast<const float4 *>(xr)[g];
        v3[g] = __fadd_rn(fmaf(v.y, v.y, __fmul_rn(v.x, v.x)), fmaf(v.w, v.w, __fmul_rn(v.z, v.z)));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float sum = 0.f;
        for (int g = 0; g < n4; ++g) { sum = __fadd_rn(sum, v3[g]); }
        for (int64_t i = (int64_t)n4 * 4; i < n; ++i) { sum = fmaf(xr[i], xr[i], sum); }
        scale_s = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum, (float)n), eps)));
    }
    __syncthreads();
    const float scale = scale_s;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) { o[i] = __fmul_rn(xr[i], scale); }
}
cudaError_t launch_rmsnorm(const float *x, float *out, int64_t n, int64_t rows, float eps, cudaStream_t s) {
    if (rows == 0 || n == 0) { return cudaSuccess; }
    if ((n & 3) != 0 || n > 180 * 1024) { return cudaErrorNotSupported; }   // rows are read as float4 groups
    const size_t smem = (size_t)n;   // n/4 floats
    static size_t smem_allowed = 48 * 1024;
    if (smem > smem_allowed) {
        cudaError_t err = cudaFuncSetAttribute(rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) { return err; }
        smem_allowed = smem;
    }
    rmsnorm_kernel<<<(unsigned)rows, 256, smem, s>>>(x, out, n, eps);
    return launch_check();
}

// binary_execution<plus / multiplies>, basic.cpp:15-50: row r of `a` with row (r % b_rows) of `b`
__global__ void binary_rows_kernel(int op, const float *a, const float *b, float *out, int64_t n, int64_t rows, int64_t b_rows) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n * rows) { return; }
    const int64_t r = i / n, c = i - r * n;
    const float   y = b[(r % b_rows) * n + c];
    out[i] = op == 0 ? __fadd_rn(a[i], y) : __fmul_rn(a[i], y);
}
cudaError_t launch_binary_rows(int op, const float *a, const float *b, float *out, int64_t n, int64_t rows, int64_t b_rows, cudaStream_t s) {
    const int64_t tot = n * rows;
    if (tot == 0) { return cudaSuccess; }
    binary_rows_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, s>>>(op, a, b, out, n, rows, b_rows);
    return launch_check();
}

// OperatorSiluImpl::execute, non-linear.cpp:57-77
__global__ void silu_kernel(const float *x, float *out, int64_t n, const float *table) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) { out[i] = table[f2h(x[i])]; }
}
cudaError_t launch_silu(const float *x, float *out, int64_t n, const float *silu_table, cudaStream_t s) {
    if (n == 0) { return cudaSuccess; }
    silu_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(x, out, n, silu_table);
    return launch_check();
}

// operator_masked_softmax_execute, non-linear.cpp:129-180; one CTA per row (i1, i2), row length ne0,
// the row kept in shared memory; the sum follows std::reduce's order (reduce4_chain).
__global__ void softmax_masked_kernel(const float *scores, const float *mask, float *out, int64_t ne0, int64_t ne1,
                                      int64_t mask_stride, float scale, const float *exp_table) {
    extern __shared__ __align__(16) float row_s[];
    __shared__ float red[8];
    __shared__ float bcast;
    const int64_t row = blockIdx.x;
    const int64_t i1  = row % ne1;
    const float  *src = scores + row * ne0;
    const float  *mk  = mask + i1 * mask_stride;
    float        *dst = out + row * ne0;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float m = -CUDART_INF_F;
    for (int64_t i = threadIdx.x; i < ne0; i += blockDim.x) {
        const float v = __fmul_rn(__fadd_rn(src[i], mk[i]), scale);
        row_s[i] = v;
        m = fmaxf(m, v);
    }
    m = warp_max(m);
    if (lane == 0) { red[warp] = m; }
    __syncthreads();
    m = red[0];
    for (int w = 1; w < nw; ++w) { m = fmaxf(m, red[w]); }
    for (int64_t i = threadIdx.x; i < ne0; i += blockDim.x) {
        row_s[i] = (mk[i] == -CUDART_INF_F) ? 0.f : exp_table[f2h(__fsub_rn(row_s[i], m))];
    }
    __syncthreads();
    if (threadIdx.x == 0) { bcast = __fdiv_rn(1.0f, reduce4_chain(row_s, (int)ne0)); }
    __syncthreads();
    const float inv = bcast;
    for (int64_t i = threadIdx.x; i < ne0; i += blockDim.x) { dst[i] = __fmul_rn(row_s[i], inv); }
}
cudaError_t launch_softmax_masked(const float *scores, const float *mask, float *out, int64_t ne0, int64_t ne1, int64_t ne2,
                                  int64_t mask_stride, float scale, const float *exp_table, cudaStream_t s) {
    if (ne0 == 0 || ne1 * ne2 == 0) { return cudaSuccess; }
    const size_t smem = (size_t)ne0 * sizeof(float);
    if (smem > 200 * 1024) { return cudaErrorNotSupported; }
    static size_t smem_allowed = 48 * 1024;
    if (smem > smem_allowed) {
        cudaError_t err = cudaFuncSetAttribute(softmax_masked_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) { return err; }
        smem_allowed = smem;
    }
    softmax_masked_kernel<<<(unsigned)(ne1 * ne2), 256, smem, s>>>(scores, mask, out, ne0, ne1, mask_stride, scale, exp_table);
    return launch_check();
}

__device__ __forceinline__ int64_t soff(const Strided &t, int64_t i0, int64_t i1, int64_t i2, int64_t i3) {
    return i0 * t.nb[0] + i1 * t.nb[1] + i2 * t.nb[2] + i3 * t.nb[3];
}

// OperatorRopeImpl::execute in mode Norm with default YaRN settings, non-linear.cpp:270-371.
// One thread per (pair, head, token); the (cos, sin) of every (token, pair) comes from a table the host
// fills with the same libm calls and the same repeated f32 multiplication of theta as the CPU operator.
__global__ void rope_kernel(const Strided x, const float2 *cos_sin, const Strided out) {
    const int64_t npair = x.ne[0] >> 1;
    const int64_t i     = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t tot   = npair * x.ne[1] * x.ne[2];
    if (i >= tot) { return; }
    const int64_t k = i % npair, i1 = (i / npair) % x.ne[1], i2 = i / (npair * x.ne[1]);
    const float2 cs = cos_sin[i2 * npair + k];
    const float *src = reinterpret_cast<const float *>(reinterpret_cast<const uint8_t *>(x.data) + soff(x, 2 * k, i1, i2, 0));
    float       *dst = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(out.data) + soff(out, 2 * k, i1, i2, 0));
    const float x0 = src[0], x1 = src[1];
    dst[0] = __fsub_rn(__fmul_rn(x0, cs.x), __fmul_rn(x1, cs.y));
    dst[1] = __fadd_rn(__fmul_rn(x0, cs.y), __fmul_rn(x1, cs.x));
}
cudaError_t launch_rope(const Strided &x, const float2 *cos_sin, const Strided &out, cudaStream_t s) {
    const int64_t tot = (x.ne[0] >> 1) * x.ne[1] * x.ne[2];
    if (tot == 0) { return cudaSuccess; }
    rope_kernel<<<(unsigned)((tot + 127) / 128), 128, 0, s>>>(x, cos_sin, out);
    return launch_check();
}

// dup_execute (Copy / Contiguous), view.cpp:83-227, 285-321: element (i0..i3) of src in source order goes to
// the element with the same flat index of dst (dst indexed through its own shape and strides).
__global__ void copy_strided_kernel(const Strided src, int src_type, const Strided dst, int dst_type) {
    const int64_t tot = src.ne[0] * src.ne[1] * src.ne[2] * src.ne[3];
    const int64_t i   = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= tot) { return; }
    const int64_t s0 = i % src.ne[0], s1 = (i / src.ne[0]) % src.ne[1], s2 = (i / (src.ne[0] * src.ne[1])) % src.ne[2],
                  s3 = i / (src.ne[0] * src.ne[1] * src.ne[2]);
    const int64_t d0 = i % dst.ne[0], d1 = (i / dst.ne[0]) % dst.ne[1], d2 = (i / (dst.ne[0] * dst.ne[1])) % dst.ne[2],
                  d3 = i / (dst.ne[0] * dst.ne[1] * dst.ne[2]);
    const uint8_t *sp = reinterpret_cast<const uint8_t *>(src.data) + soff(src, s0, s1, s2, s3);
    uint8_t       *dp = reinterpret_cast<uint8_t *>(dst.data) + soff(dst, d0, d1, d2, d3);
    const float v = (src_type == 0) ? *reinterpret_cast<const float *>(sp) : h2f(*reinterpret_cast<const uint16_t *>(sp));
    if (dst_type == 0) { *reinterpret_cast<float *>(dp) = v; } else { *reinterpret_cast<uint16_t *>(dp) = f2h(v); }
}
cudaError_t launch_copy_strided(const Strided &src, int src_type, const Strided &dst, int dst_type, cudaStream_t s) {
    if ((src_type != 0 && src_type != 1) || (dst_type != 0 && dst_type != 1)) { return cudaErrorNotSupported; }
    const int64_t tot = src.ne[0] * src.ne[1] * src.ne[2] * src.ne[3];
    if (tot == 0) { return cudaSuccess; }
    copy_strided_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, s>>>(src, src_type, dst, dst_type);
    return launch_check();
}

// bytes of one table row of ne0 elements
__host__ __device__ __forceinline__ int64_t table_row_bytes(int type, int64_t ne0) {
    return type == 0 ? ne0 * 4 : type == 1 ? ne0 * 2 : type == 8 ? ne0 / 32 * 34 : type == 12 ? ne0 / 256 * 144 : type == 14 ? ne0 / 256 * 210 : ne0 / 32 * 18;
}
// embedding row -> f32: memcpy for F32, Q8_0 -> F32 as OperatorGetRowImpl::execute (view.cpp:33-81);
// Q4_0 rows (which the CPU backend cannot gather) decode as (nibble - 8) * d; K-quant rows (no reference arithmetic; the block
// layouts of number_impl/k-quant.h) as (d * sc) * q - dmin * m (Q4_K) and q * (d * sc) (Q6_K), every operation a separate f32 one.
__device__ __forceinline__ float embd_value(const uint8_t *row, int type, int64_t i) {
    if (type == 0) { return reinterpret_cast<const float *>(row)[i]; }
    if (type == 1) { return h2f(reinterpret_cast<const uint16_t *>(row)[i]); }
    if (type == 12) {
        const uint8_t *s = row + (i >> 8) * 144;
        const int e = (int)(i & 255), j = e >> 5, l = e & 31;
        const float d = h2f((uint16_t)(s[0] | (s[1] << 8))), dmin = h2f((uint16_t)(s[2] | (s[3] << 8)));
        const uint8_t *sc12 = s + 4;
        uint32_t sc, mn;
        if (j < 4) { sc = sc12[j] & 63u; mn = sc12[j + 4] & 63u; }
        else { sc = (sc12[j + 4] & 0xFu) | ((uint32_t)(sc12[j - 4] >> 6) << 4); mn = (uint32_t)(sc12[j + 4] >> 4) | ((uint32_t)(sc12[j] >> 6) << 4); }
        const uint8_t qb = s[16 + 32 * (j >> 1) + l];
        const int q = (j & 1) ? (qb >> 4) : (qb & 0xF);
        return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)mn));
    }
    if (type == 14) {
        const uint8_t *s = row + (i >> 8) * 210;
        const int e = (int)(i & 255), hf = e >> 7, seg = (e >> 5) & 3, l = e & 31;
        const uint8_t lo = s[64 * hf + 32 * (seg & 1) + l], h = s[128 + 32 * hf + l];
        const int q = (((seg & 2) ? (lo >> 4) : (lo & 0xF)) | (((h >> (2 * seg)) & 3) << 4)) - 32;
        const float d = h2f((uint16_t)(s[208] | (s[209] << 8)));
        const int sc = (int)(int8_t)s[192 + (e >> 4)];
        return __fmul_rn((float)q, __fmul_rn(d, (float)sc));
    }
    const int64_t b = i >> 5; const int k = (int)(i & 31);
    if (type == 8) {
        const uint8_t *blk = row + b * 34;
        return __fmul_rn((float)(int8_t)blk[2 + k], h2f((uint16_t)(blk[0] | (blk[1] << 8))));
    }
    const uint8_t *blk = row + b * 18;   // Q4_0
    const int nib = (k < 16) ? (blk[2 + k] & 0xF) : (blk[2 + k - 16] >> 4);
    return __fmul_rn((float)(nib - 8), h2f((uint16_t)(blk[0] | (blk[1] << 8))));
}

__global__ void getrow_kernel(const uint8_t *table, int type, int64_t row_bytes, int64_t ne0, const int32_t *ids, float *out) {
    const int64_t r   = blockIdx.x;
    const uint8_t *row = table + (int64_t)ids[r] * row_bytes;
    for (int64_t i = threadIdx.x; i < ne0; i += blockDim.x) { out[r * ne0 + i] = embd_value(row, type, i); }
}
cudaError_t launch_getrow(const uint8_t *table, int table_type, int64_t row_bytes, int64_t ne0, const int32_t *ids, int64_t n_ids, float *out, cudaStream_t s) {
    if (table_type != 0 && table_type != 1 && table_type != 2 && table_type != 8 && table_type != 12 && table_type != 14) { return cudaErrorNotSupported; }
    if (n_ids == 0) { return cudaSuccess; }
    getrow_kernel<<<(unsigned)n_ids, 256, 0, s>>>(table, table_type, row_bytes, ne0, ids, out);
    return launch_check();
}
cudaError_t launch_embed(const int32_t *ids, int n_ids, const uint8_t *embd, int embd_type, int64_t d_model, float *x_out, cudaStream_t s) {
    return launch_getrow(embd, embd_type, table_row_bytes(embd_type, d_model), d_model, ids, n_ids, x_out, s);
}

// MatMul with an F16 weight and f32 activations (the attention products when run op by op): activations
// are rounded to fp16 first (mat.cpp:32-42), then Dot<FP16,FP16> (vec_dot.h:117-146) in its exact order.
// One warp per output element; arbitrary byte strides.
__global__ void matmul_f16_kernel(const Strided w, const Strided x, const Strided out) {
    const int64_t n_out = out.ne[0] * out.ne[1] * out.ne[2];
    const int64_t o     = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int     lane  = threadIdx.x & 31;
    if (o >= n_out) { return; }
    const int64_t i01 = o % out.ne[0], i11 = (o / out.ne[0]) % out.ne[1], i02 = o / (out.ne[0] * out.ne[1]);
    const uint8_t *wp = reinterpret_cast<const uint8_t *>(w.data) + soff(w, 0, i01, i02, 0);
    const uint8_t *xp = reinterpret_cast<const uint8_t *>(x.data) + soff(x, 0, i11, i02, 0);
    const int64_t n = w.ne[0];
    const int64_t n_main = n > 0 ? ((n - 1) / 32) * 32 : 0;
    float acc = 0.f;
    for (int64_t k = 0; k < n_main; k += 32) {
        const float a = h2f(*reinterpret_cast<const uint16_t *>(wp + (k + lane) * w.nb[0]));
        const float b = h2f(f2h(*reinterpret_cast<const float *>(xp + (k + lane) * x.nb[0])));
        acc = fmaf(a, b, acc);
    }
    acc = reduce_f16dot_lanes(acc);
    if (lane == 0) {
        float tail = 0.f;
        for (int64_t k = n_main; k < n; ++k) {
            const float a = h2f(*reinterpret_cast<const uint16_t *>(wp + k * w.nb[0]));
            const float b = h2f(f2h(*reinterpret_cast<const float *>(xp + k * x.nb[0])));
            tail = fmaf(a, b, tail);
        }
        *reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(out.data) + soff(out, i01, i11, i02, 0)) = __fadd_rn(tail, acc);
    }
}
cudaError_t launch_matmul_f16(const Strided &w, const Strided &x, const Strided &out, cudaStream_t s) {
    const int64_t n_out = out.ne[0] * out.ne[1] * out.ne[2];
    if (n_out == 0) { return cudaSuccess; }
    matmul_f16_kernel<<<(unsigned)((n_out * 32 + 255) / 256), 256, 0, s>>>(w, x, out);
    return launch_check();
}

// Greedy sampling on the device (first maximum wins, model/include/llm/sampler/greedy.h:20-25), followed by
// the next step's embedding gather and the position increment, so a decode step needs no host round trip.
__global__ void __launch_bounds__(1024) argmax_embed_kernel(const float *logits, int64_t n_vocab, int32_t *token_out, int32_t *history,
                                                           int *pos_counter, const uint8_t *embd, int embd_type, int64_t d_model, float *x_out) {
    __shared__ float bv[32];
    __shared__ int   bi[32];
    __shared__ int   winner;
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float best = -CUDART_INF_F; int idx = 0x7fffffff;
    for (int64_t i = tid; i < n_vocab; i += blockDim.x) {
        const float v = logits[i];
        if (v > best || (v == best && (int)i < idx)) { best = v; idx = (int)i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int   oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        best = (lane < (int)(blockDim.x >> 5)) ? bv[lane] : -CUDART_INF_F;
        idx  = (lane < (int)(blockDim.x >> 5)) ? bi[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int   oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
        }
        if (lane == 0) {
            if (idx == 0x7fffffff) { idx = 0; }   // all-NaN row: the CPU's max_element returns the first element
            winner = idx;
            *token_out = idx;
            const int step_pos = *pos_counter;
            if (history != nullptr) { history[step_pos] = idx; }
            *pos_counter = step_pos + 1;
            pos_counter[2] += 1;   // exchange epoch of the next step (tensor parallel)
        }
    }
    __syncthreads();
    if (embd != nullptr) {
        const uint8_t *row = embd + (int64_t)winner * table_row_bytes(embd_type, d_model);
        for (int64_t i = tid; i < d_model; i += blockDim.x) { x_out[i] = embd_value(row, embd_type, i); }
    }
}
cudaError_t launch_argmax_embed(const float *logits, int64_t n_vocab, int32_t *token_out, int32_t *history, int *pos_counter,
                                const uint8_t *embd, int embd_type, int64_t d_model, float *x_out, const LaunchCfg &cfg) {
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(1); lc.blockDim = dim3(1024); lc.dynamicSmemBytes = 0; lc.stream = cfg.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr; lc.numAttrs = cfg.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&lc, argmax_embed_kernel, logits, n_vocab, token_out, history, pos_counter, embd, embd_type, d_model, x_out);
}

// Greedy sampling for a batch of sequences in lockstep: block c takes the logits of sequence c, writes its token (for the next
// step's embedding gather and into ids_out[step][c]) and gathers the embedding into column c of x. The position is advanced
// by advance_pos_kernel afterwards (one word for the whole batch).
__global__ void __launch_bounds__(1024) argmax_embed_batch_kernel(const float *logits, int64_t n_vocab, int32_t *tokens, int32_t *ids_out,
                                                                 const uint8_t *embd, int embd_type, int64_t d_model, float *x_out, int64_t x_stride) {
    __shared__ float bv[32];
    __shared__ int   bi[32];
    __shared__ int   winner;
    const int c = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float *row_logits = logits + (int64_t)c * n_vocab;
    float best = -CUDART_INF_F; int idx = 0x7fffffff;
    for (int64_t i = tid; i < n_vocab; i += blockDim.x) {
        const float v = row_logits[i];
        if (v > best || (v == best && (int)i < idx)) { best = v; idx = (int)i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int   oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        best = (lane < (int)(blockDim.x >> 5)) ? bv[lane] : -CUDART_INF_F;
        idx  = (lane < (int)(blockDim.x >> 5)) ? bi[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int   oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
        }
        if (lane == 0) {
            if (idx == 0x7fffffff) { idx = 0; }   // all-NaN row: the CPU's max_element returns the first element
            winner = idx;
            tokens[c] = idx;
            ids_out[c] = idx;
        }
    }
    __syncthreads();
    if (embd != nullptr && x_out != nullptr) {
        const uint8_t *row = embd + (int64_t)winner * table_row_bytes(embd_type, d_model);
        for (int64_t i = tid; i < d_model; i += blockDim.x) { x_out[(int64_t)c * x_stride + i] = embd_value(row, embd_type, i); }
    }
}
__global__ void advance_pos_kernel(int *pos_counter) { pos_counter[0] += 1; pos_counter[2] += 1; }

cudaError_t launch_argmax_embed_batch(const float *logits, int64_t n_vocab, int n_seq, int32_t *tokens, int32_t *ids_out, const uint8_t *embd, int embd_type,
                                      int64_t d_model, float *x_out, int64_t x_stride, int *pos_counter, cudaStream_t s) {
    argmax_embed_batch_kernel<<<n_seq, 1024, 0, s>>>(logits, n_vocab, tokens, ids_out, embd, embd_type, d_model, x_out, x_stride);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) { return err; }
    advance_pos_kernel<<<1, 1, 0, s>>>(pos_counter);
    return cudaGetLastError();
}

}  // namespace spyb
