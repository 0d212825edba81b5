// Dequant-fused mat-vec for sm_100a, bit-exact with the reference's CPU arithmetic.
//
// Reference semantics: OperatorMatMulImpl::execute (backend/host/operator/mat.cpp:71-146) quantizes every
// f32 activation column to Q8_0 and takes Dot<Q4_0,Q8_0> / Dot<Q8_0,Q8_0>
// (backend/host/include/simd/vec_dot.h:42-115) per output: eight f32 accumulators, one per group of four
// products, each updated block after block with acc = fma(d_w * d_x, (float)lane_sum, acc), and a fixed
// reduction tree at the end. Because the network re-quantizes its activations at every layer, any
// difference in f32 summation order is amplified to percent-level logit differences within a few layers,
// so this kernel reproduces that order exactly:
//   phase 1 (parallel over the row: lane = block)  weights streamed from HBM with 128-bit loads held in a
//            register pipeline; per block the eight integer lane sums by byte dot products, converted to
//            f32 without rounding, and the f32 block scale; both parked in shared memory
//   phase 2 (sequential along the row: lane = (row, accumulator) for 4 rows x 8 accumulators) the 32
//            blocks of the chunk are folded into the accumulators in block order with one FMA each
// The small neighbouring operators of the LLaMa layer are folded into the prologue (RMSNorm + weight +
// Q8_0 quantization, in the CPU's summation order) and the epilogue (residual add, SiLU-gate-mul,
// RoPE + KV append).
//
// Roofline: HBM-bound. Algorithmic bytes per launch = rows * K/32 * 18 (Q4_0) or 34 (Q8_0); activations
// and outputs are a few KB and stay in L2.

#include "spyb_common.cuh"
#include "spyb_kernels.h"

namespace spyb {

constexpr int MV_THREADS = 256;
constexpr int MV_WARPS   = MV_THREADS / WARP;
constexpr int P_STRIDE   = 36;                       // floats per (row, accumulator) line: 32 blocks + pad, keeps 128-bit reads conflict-free
constexpr int P_FLOATS   = 32 * P_STRIDE;            // lane sums: 4 rows x 8 accumulators
constexpr int S_FLOATS   = 4 * P_STRIDE;             // block scales: 4 rows
constexpr int WARP_SCRATCH_FLOATS = P_FLOATS + 2 * S_FLOATS;

__host__ __device__ static inline size_t matvec_smem_layout(int nb, int TM, size_t *off_v3, size_t *off_warp) {
    size_t o = act_bytes(nb, TM);
    o = (o + 15) / 16 * 16;
    *off_v3 = o;
    o += (size_t)TM * (nb * 8) * sizeof(float);      // sum-of-squares partials: K/4 floats per column
    o = (o + 15) / 16 * 16;
    *off_warp = o;
    o += (size_t)MV_WARPS * WARP_SCRATCH_FLOATS * sizeof(float);
    return o + 16;
}

size_t matvec_smem_bytes(int nb, int T) { size_t a, b; return matvec_smem_layout(nb, T, &a, &b); }

// ---------------------------------------------------------------------------------------------
// prologue: f32 activations -> Q8_0 columns in shared memory (optionally through RMSNorm * weight)
//   NormRMS (backend/host/operator/non-linear.cpp:194-223): sum of squares by std::transform_reduce, whose
//   order for random-access ranges is: groups of four combined as (x0^2 + x1^2) + (x2^2 + x3^2) (the first
//   product of each pair plain, the second fused into an FMA, as the CPU build evaluates it) and added to the running sum one group after
//   the other; y = x * (1 / sqrt(sum/n + eps)). The groups are formed in parallel, the running sum is
//   one thread's chain. Mul (basic.cpp:15-50): y * norm_weight.
template <int TM>
__device__ __forceinline__ void matvec_prologue(const MatvecParams &p, ActView act, float *v3, float *scales) {
    const int     tid = threadIdx.x;
    const int64_t K   = p.A.k;
    const int     nb  = p.A.nb;
    const int     n4  = (int)(K >> 2);
    if (p.pro == PRO_NORM_QUANT) {
        for (int t = 0; t < p.T; ++t) {
            const float4 *x4 = reinterpret_cast<const float4 *>(p.x + (int64_t)t * p.x_stride);
            for (int g = tid; g < n4; g += MV_THREADS) {
                const float4 v = x4[g];
                const float v1 = fmaf(v.y, v.y, __fmul_rn(v.x, v.x));
                const float v2 = fmaf(v.w, v.w, __fmul_rn(v.z, v.z));
                v3[t * n4 + g] = __fadd_rn(v1, v2);
            }
        }
        __syncthreads();
        if (tid < p.T) {
            const float4 *g4 = reinterpret_cast<const float4 *>(v3 + tid * n4);
            float sum = 0.f;
            int g = 0;
            for (; g + 4 <= n4; g += 4) {
                const float4 q = g4[g >> 2];
                sum = __fadd_rn(sum, q.x); sum = __fadd_rn(sum, q.y); sum = __fadd_rn(sum, q.z); sum = __fadd_rn(sum, q.w);
            }
            for (; g < n4; ++g) { sum = __fadd_rn(sum, v3[tid * n4 + g]); }
            const float mean = __fdiv_rn(sum, (float)K);
            scales[tid] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, p.eps)));
        }
        __syncthreads();
    }
#pragma unroll 1
    for (int t = 0; t < TM; ++t) {
        if (t >= p.T) {
            // unused columns: zero scales make every contribution vanish
            for (int b = tid; b < nb; b += MV_THREADS) {
                act.d[t * nb + b] = 0.f;
                act.lo[t * nb + b] = make_uint4(0, 0, 0, 0); act.hi[t * nb + b] = make_uint4(0, 0, 0, 0);
                act.blo[t * nb + b] = make_int4(MAGIC_I, MAGIC_I, MAGIC_I, MAGIC_I); act.bhi[t * nb + b] = make_int4(MAGIC_I, MAGIC_I, MAGIC_I, MAGIC_I);
            }
            continue;
        }
        const float4 *x4 = reinterpret_cast<const float4 *>(p.x + (int64_t)t * p.x_stride);
        const float4 *w4 = reinterpret_cast<const float4 *>(p.norm_w);
        const float scale = (p.pro == PRO_NORM_QUANT) ? scales[t] : 1.f;
        for (int base = 0; base < n4; base += MV_THREADS) {
            const int  g     = base + tid;
            const bool valid = g < n4;
            float4 v = valid ? x4[g] : make_float4(0.f, 0.f, 0.f, 0.f);
            if (p.pro == PRO_NORM_QUANT && valid) {
                const float4 w = w4[g];
                v.x = __fmul_rn(__fmul_rn(v.x, scale), w.x);
                v.y = __fmul_rn(__fmul_rn(v.y, scale), w.y);
                v.z = __fmul_rn(__fmul_rn(v.z, scale), w.z);
                v.w = __fmul_rn(__fmul_rn(v.w, scale), w.w);
            }
            uint16_t dh; int s;
            const uint32_t q = quantize_q8_lane4(v, dh, s);
            if (valid) {
                const int b  = g >> 3;
                const int li = g & 7;
                if (li < 4) {
                    reinterpret_cast<uint32_t *>(act.lo + t * nb + b)[li] = q;
                    reinterpret_cast<int *>(act.blo + t * nb + b)[li] = (int)MAGIC_I - 8 * s;
                } else {
                    reinterpret_cast<uint32_t *>(act.hi + t * nb + b)[li - 4] = q;
                    reinterpret_cast<int *>(act.bhi + t * nb + b)[li - 4] = (int)MAGIC_I - 128 * s;
                }
                if (li == 0) { act.d[t * nb + b] = h2f(dh); }
            }
        }
    }
}

// reference-layout copy of column 0 (34-byte blocks) for parity taps
__device__ __forceinline__ void matvec_tap(const MatvecParams &p, ActView act) {
    if (p.tap_xq == nullptr || blockIdx.x != 0) { return; }
    for (int b = threadIdx.x; b < act.nb; b += MV_THREADS) {
        volatile uint8_t *o = p.tap_xq + (size_t)b * 34;   // 34-byte records: only byte alignment holds
        const uint32_t dh = f2h(act.d[b]);
        const uint8_t *lo = reinterpret_cast<const uint8_t *>(act.lo + b);
        const uint8_t *hi = reinterpret_cast<const uint8_t *>(act.hi + b);
        for (int i = 0; i < 16; ++i) { o[2 + i] = lo[i]; o[18 + i] = hi[i]; }
        *reinterpret_cast<volatile uint16_t *>(p.tap_xq + (size_t)b * 34) = (uint16_t)dh;   // records start on even addresses
    }
}

// ---------------------------------------------------------------------------------------------
// epilogue for the four finished dot products r[0..3] of unit u, column t
__device__ __forceinline__ void matvec_epilogue(const MatvecParams &p, int64_t u, int t, const float r[4]) {
    switch (p.epi) {
    case EPI_STORE: {
        float4 *o = reinterpret_cast<float4 *>(p.out + (int64_t)t * p.out_stride + 4 * u);
        *o = make_float4(r[0], r[1], r[2], r[3]);
    } break;
    case EPI_RESID: {   // Add(attn_out, x) / Add(ffn_inp, ffn_out): model/src/llm/model/llama.cpp:194-211
        const int64_t i = (int64_t)t * p.out_stride + 4 * u;
        const float4 q = *reinterpret_cast<const float4 *>(p.resid + i);
        *reinterpret_cast<float4 *>(p.out + i) = make_float4(__fadd_rn(r[0], q.x), __fadd_rn(r[1], q.y), __fadd_rn(r[2], q.z), __fadd_rn(r[3], q.w));
    } break;
    case EPI_SILU_MUL: {  // up * silu(gate): model/src/llm/plugin/ffn.cpp:28-35; silu = table on the fp16-rounded argument
        float2 *o = reinterpret_cast<float2 *>(p.out + (int64_t)t * p.out_stride + 2 * u);
        *o = make_float2(__fmul_rn(r[0], p.silu_table[f2h(r[1])]), __fmul_rn(r[2], p.silu_table[f2h(r[3])]));
    } break;
    case EPI_QKV_ROPE: {
        const int64_t row = 4 * u;
        const int     sec = (int)(row / p.dl);
        const int     e   = (int)(row - (int64_t)sec * p.dl);
        const int     pos = *p.pos_base + t;
        if (sec == 2) {   // V: f32 -> f16 RNE into the transposed cache [dl][n_ctx] (dup_execute, backend/host/operator/view.cpp:163-191)
#pragma unroll
            for (int k = 0; k < 4; ++k) { p.v_cache[(int64_t)(e + k) * p.n_ctx + pos] = __float2half_rn(r[k]); }
        } else {          // RoPE, mode Norm: backend/host/operator/non-linear.cpp:270-371
            const int    i0 = (e % p.hd) >> 1;
            const float2 c0 = p.rope_table[(int64_t)pos * (p.hd >> 1) + i0];
            const float2 c1 = p.rope_table[(int64_t)pos * (p.hd >> 1) + i0 + 1];
            const float a0 = __fsub_rn(__fmul_rn(r[0], c0.x), __fmul_rn(r[1], c0.y));
            const float a1 = __fadd_rn(__fmul_rn(r[0], c0.y), __fmul_rn(r[1], c0.x));
            const float a2 = __fsub_rn(__fmul_rn(r[2], c1.x), __fmul_rn(r[3], c1.y));
            const float a3 = __fadd_rn(__fmul_rn(r[2], c1.y), __fmul_rn(r[3], c1.x));
            __half *base = (sec == 0) ? p.q_out + (int64_t)t * p.dl + e : p.k_cache + (int64_t)pos * p.dl + e;
            reinterpret_cast<__half2 *>(base)[0] = __halves2half2(__float2half_rn(a0), __float2half_rn(a1));
            reinterpret_cast<__half2 *>(base)[1] = __halves2half2(__float2half_rn(a2), __float2half_rn(a3));
        }
    } break;
    default: break;
    }
}

// ---------------------------------------------------------------------------------------------
// Register pipeline: D work items in flight per lane. One item = one 32-block chunk of a 4-row unit,
// i.e. per lane one block of each of the four rows: D * 4 * 16 B (Q4_0) of loads per lane outstanding,
// 256 threads * 256 B = 64 KB per SM, enough to cover HBM latency.
template <int WT> struct Pipe;
template <> struct Pipe<2> { static constexpr int D = 4; };   // Q4_0
template <> struct Pipe<8> { static constexpr int D = 2; };   // Q8_0

template <int WT, int TM>
__global__ void __launch_bounds__(MV_THREADS, (TM == 1) ? 2 : 1) matvec_kernel(const MatvecParams p) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __shared__ float norm_scales[8];
    constexpr int D  = Pipe<WT>::D;
    constexpr int DB = (WT == 8) ? D : 1;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nb     = p.A.nb;
    const int nchunk = (nb + 31) >> 5;

    // unit = 4 rows: rows 4u..4u+3 of A, or (pair mode) rows 2u, 2u+1 of A interleaved with the same rows of B
    const int64_t n_units     = p.pair_mode ? (p.A.n_rows >> 1) : (p.A.n_rows >> 2);
    const int64_t total_warps = (int64_t)gridDim.x * MV_WARPS;
    const int64_t gw          = (int64_t)blockIdx.x * MV_WARPS + warp;
    const int64_t u0          = n_units * gw / total_warps;
    const int64_t u1          = n_units * (gw + 1) / total_warps;
    const int64_t n_items     = (u1 - u0) * nchunk;

    const int64_t ustride = p.pair_mode ? 2 * (int64_t)nb : 4 * (int64_t)nb;
    const uint4 *qa_r[4]; const uint4 *qb_r[4]; const uint16_t *d_r[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const DevMatrix &M = (p.pair_mode && (r & 1)) ? p.B : p.A;
        const int64_t ro = p.pair_mode ? (int64_t)(r >> 1) * nb : (int64_t)r * nb;
        qa_r[r] = M.qa + ro; qb_r[r] = (WT == 8) ? M.qb + ro : nullptr; d_r[r] = M.d + ro;
    }

    uint4    wa[D][4];
    uint4    wb[DB][4];
    uint16_t wd[D][4];

    auto load_item = [&](int j, int64_t u, int c) {
        const int b = (c << 5) + lane;
        if (b < nb) {
            const int64_t off = u * ustride + b;
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                wa[j][r] = ldg_stream(qa_r[r] + off);
                if (WT == 8) { wb[(WT == 8) ? j : 0][r] = ldg_stream(qb_r[r] + off); }
                wd[j][r] = ldg_stream_u16(d_r[r] + off);
            }
        } else {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                wa[j][r] = make_uint4(0, 0, 0, 0);
                if (WT == 8) { wb[(WT == 8) ? j : 0][r] = make_uint4(0, 0, 0, 0); }
                wd[j][r] = 0;
            }
        }
    };

    // Let the next kernel of the step begin (its own weight prefetch), then prefetch ours: weights
    // never change during a step, so these loads may run ahead of the previous kernel's results.
    pdl_launch_dependents();
    int64_t lu = u0; int lc = 0; int64_t issued = 0;
#pragma unroll
    for (int j = 0; j < D; ++j) {
        if (issued < n_items) {
            load_item(j, lu, lc);
            ++issued; if (++lc == nchunk) { lc = 0; ++lu; }
        }
    }
    pdl_wait();

    size_t off_v3, off_warp;
    matvec_smem_layout(nb, TM, &off_v3, &off_warp);
    ActView act = act_view(smem_raw, nb, TM);
    float *v3  = reinterpret_cast<float *>(smem_raw + off_v3);
    float *P   = reinterpret_cast<float *>(smem_raw + off_warp) + warp * WARP_SCRATCH_FLOATS;
    float *S   = P + P_FLOATS;            // block scales d_w * d_x per (row, block)
    float *S16 = S + S_FLOATS;            // the same divided by 16 (Q4_0 high-nibble accumulators)
    matvec_prologue<TM>(p, act, v3, norm_scales);
    __syncthreads();
    matvec_tap(p, act);

    float acc[TM];
#pragma unroll
    for (int t = 0; t < TM; ++t) { acc[t] = 0.f; }
    const int    my_row = lane >> 3, my_acc = lane & 7;
    const float *Pmine  = P + lane * P_STRIDE;
    const float *Smine  = ((WT == 2 && my_acc < 4) ? S16 : S) + my_row * P_STRIDE;

    int64_t cu = u0; int cc = 0;
    for (int64_t base = 0; base < n_items; base += D) {
#pragma unroll
        for (int j = 0; j < D; ++j) {
            if (base + j < n_items) {
                const int  b     = (cc << 5) + lane;
                const bool valid = b < nb;
                const int  bq    = valid ? b : nb - 1;
                const int  nval  = min(32, nb - (cc << 5));
                const int  ngrp  = (nval + 3) >> 2;
                float sw[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) { sw[r] = h2f(wd[j][r]); }
#pragma unroll
                for (int t = 0; t < TM; ++t) {
                    // ---- phase 1: this lane's block of each of the four rows
                    const uint4 ylo = act.lo[t * nb + bq];
                    const uint4 yhi = act.hi[t * nb + bq];
                    const float yd  = valid ? act.d[t * nb + bq] : 0.f;
                    int4 blo = make_int4(0, 0, 0, 0), bhi = make_int4(0, 0, 0, 0);
                    if (WT == 2) { blo = act.blo[t * nb + bq]; bhi = act.bhi[t * nb + bq]; }
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        float f[8];
                        if (WT == 2) { lanes_q4_0(wa[j][r], ylo, yhi, blo, bhi, f); }
                        else         { lanes_q8_0(wa[j][r], wb[(WT == 8) ? j : 0][r], ylo, yhi, f); }
#pragma unroll
                        for (int l = 0; l < 8; ++l) { P[(r * 8 + l) * P_STRIDE + lane] = f[l]; }
                        const float d = __fmul_rn(sw[r], yd);
                        S[r * P_STRIDE + lane] = d;
                        if (WT == 2) { S16[r * P_STRIDE + lane] = __fmul_rn(d, 0.0625f); }
                    }
                    __syncwarp();
                    // ---- phase 2: lane (row, accumulator) folds the chunk's blocks in order
                    float a = acc[t];
#pragma unroll 2
                    for (int g = 0; g < ngrp; ++g) {
                        const float4 pv = *reinterpret_cast<const float4 *>(Pmine + 4 * g);
                        const float4 sv = *reinterpret_cast<const float4 *>(Smine + 4 * g);
                        a = fmaf(sv.x, pv.x, a); a = fmaf(sv.y, pv.y, a); a = fmaf(sv.z, pv.z, a); a = fmaf(sv.w, pv.w, a);
                    }
                    acc[t] = a;
                    __syncwarp();
                }
                if (issued < n_items) {
                    load_item(j, lu, lc);
                    ++issued; if (++lc == nchunk) { lc = 0; ++lu; }
                }
                if (++cc == nchunk) {   // unit finished: fixed reduction tree over the 8 accumulators of each row, then the epilogue
                    float r4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int t = 0; t < TM; ++t) {
                        const float h = hsum8_lanes(acc[t]);
                        const float r0 = __shfl_sync(0xffffffffu, h, 0), r1 = __shfl_sync(0xffffffffu, h, 8);
                        const float r2 = __shfl_sync(0xffffffffu, h, 16), r3 = __shfl_sync(0xffffffffu, h, 24);
                        if (lane == t) { r4[0] = r0; r4[1] = r1; r4[2] = r2; r4[3] = r3; }
                        acc[t] = 0.f;
                    }
                    if (lane < p.T) { matvec_epilogue(p, cu, lane, r4); }
                    cc = 0; ++cu;
                }
            }
        }
    }
}

template <int WT, int TM>
static cudaError_t launch_matvec_t(const MatvecParams &p, const LaunchCfg &cfg) {
    const size_t smem = matvec_smem_bytes(p.A.nb, TM);
    static size_t smem_allowed = 48 * 1024;   // one process drives one device, so one high-water mark per kernel suffices
    if (smem > smem_allowed) {
        cudaError_t err = cudaFuncSetAttribute(matvec_kernel<WT, TM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) { return err; }
        smem_allowed = smem;
    }
    const int64_t n_units = p.pair_mode ? (p.A.n_rows >> 1) : (p.A.n_rows >> 2);
    int grid = cfg.num_sms * ((TM == 1) ? cfg.mv_ctas_per_sm : 1);
    if ((int64_t)grid * MV_WARPS > n_units) { grid = (int)((n_units + MV_WARPS - 1) / MV_WARPS); }
    if (grid < 1) { grid = 1; }

    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(grid); lc.blockDim = dim3(MV_THREADS); lc.dynamicSmemBytes = smem; lc.stream = cfg.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr; lc.numAttrs = cfg.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&lc, matvec_kernel<WT, TM>, p);
}

int matvec_max_columns(int nb) {
    for (int t = 8; t > 1; t >>= 1) { if (matvec_smem_bytes(nb, t) <= 200 * 1024) { return t; } }
    return 1;
}

template <int WT>
static cudaError_t launch_matvec_w(const MatvecParams &p, const LaunchCfg &cfg) {
    if (p.T <= 1) { return launch_matvec_t<WT, 1>(p, cfg); }
    if (p.T <= 2) { return launch_matvec_t<WT, 2>(p, cfg); }
    if (p.T <= 4) { return launch_matvec_t<WT, 4>(p, cfg); }
    return launch_matvec_t<WT, 8>(p, cfg);
}

cudaError_t launch_matvec(const MatvecParams &p, const LaunchCfg &cfg) {
    if (p.T < 1 || p.T > matvec_max_columns(p.A.nb)) { return cudaErrorInvalidValue; }
    if (p.A.k % QK != 0 || p.A.nb < 1) { return cudaErrorInvalidValue; }
    if (!p.pair_mode && (p.A.n_rows & 3)) { return cudaErrorInvalidValue; }
    if (p.pair_mode && ((p.A.n_rows & 1) || p.B.type != p.A.type || p.B.n_rows != p.A.n_rows || p.B.k != p.A.k)) { return cudaErrorInvalidValue; }
    switch (p.A.type) {
    case 2: return launch_matvec_w<2>(p, cfg);
    case 8: return launch_matvec_w<8>(p, cfg);
    default: return cudaErrorNotSupported;
    }
}

}  // namespace spyb
