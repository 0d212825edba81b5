// Dequant-fused mat-vec for sm_100a: quantized weight rows streamed once from HBM with 128-bit
// loads held in a register pipeline, multiplied against Q8_0-quantized activation columns kept in
// shared memory, with the neighbouring small operators of the LLaMa layer folded into the prologue
// (RMSNorm + weight + Q8_0 quantization) and the epilogue (residual add, SiLU-gate-mul, RoPE + KV
// append).
//
// Reference semantics: OperatorMatMulImpl::execute (backend/host/operator/mat.cpp:71-146) quantizes
// every f32 activation column to Q8_0 and takes Dot<Q4_0,Q8_0> / Dot<Q8_0,Q8_0>
// (backend/host/include/simd/vec_dot.h:42-115) per output. The integer block dots here are exact;
// the f32 accumulation order over blocks differs from the CPU's 8-lane order (tolerance only).
//
// Roofline: HBM-bound. Algorithmic bytes per launch = rows * K/32 * 18 (Q4_0) or 34 (Q8_0);
// activations and outputs are a few KB and stay in L2.

#include "spyb_common.cuh"
#include "spyb_kernels.h"

namespace spyb {

constexpr int MV_THREADS = 256;
constexpr int MV_WARPS   = MV_THREADS / WARP;

size_t matvec_smem_bytes(int nb, int T) { return act_bytes(nb, T) + 64; }

// ---------------------------------------------------------------------------------------------
// prologue: f32 activations -> Q8_0 columns in shared memory (optionally through RMSNorm * weight)
//   NormRMS: y = x * (1 / sqrt(sum(x^2)/n + eps))   (backend/host/operator/non-linear.cpp:194-223)
//   Mul    : y * norm_weight                         (backend/host/operator/basic.cpp:15-50)
template <int TM>
__device__ __forceinline__ void matvec_prologue(const MatvecParams &p, ActView act, float *red) {
    const int     tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t K   = p.A.k;
    const int     nb  = p.A.nb;
    const int64_t n4  = K >> 2;
#pragma unroll 1
    for (int t = 0; t < TM; ++t) {
        if (t >= p.T) {
            // unused columns: zero scale and zero sums make every contribution vanish
            for (int b = tid; b < nb; b += MV_THREADS) { act.d[t * nb + b] = 0.f; act.s[t * nb + b] = 0; }
            for (int i = tid; i < nb; i += MV_THREADS) { act.lo[t * nb + i] = make_uint4(0, 0, 0, 0); act.hi[t * nb + i] = make_uint4(0, 0, 0, 0); }
            continue;
        }
        const float4 *x4 = reinterpret_cast<const float4 *>(p.x + (int64_t)t * p.x_stride);
        float scale = 1.f;
        if (p.pro == PRO_NORM_QUANT) {
            float ss = 0.f;
            for (int64_t g = tid; g < n4; g += MV_THREADS) {
                const float4 v = x4[g];
                ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
            }
            ss = warp_sum(ss);
            __syncthreads();                       // red[] free from the previous column
            if (lane == 0) { red[warp] = ss; }
            __syncthreads();
            float tot = 0.f;
#pragma unroll
            for (int w = 0; w < MV_WARPS; ++w) { tot += red[w]; }
            const float mean = __fdiv_rn(tot, (float)K);
            scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, p.eps)));
        }
        const float4 *w4 = reinterpret_cast<const float4 *>(p.norm_w);
        for (int64_t base = 0; base < n4; base += MV_THREADS) {
            const int64_t g     = base + tid;
            const bool    valid = g < n4;
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
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            if (valid) {
                const int b  = (int)(g >> 3);
                const int li = (int)(g & 7);
                uint32_t *dst = (li < 4) ? reinterpret_cast<uint32_t *>(act.lo + t * nb + b) + li
                                         : reinterpret_cast<uint32_t *>(act.hi + t * nb + b) + (li - 4);
                *dst = q;
                if (li == 0) { act.d[t * nb + b] = h2f(dh); act.s[t * nb + b] = s; }
            }
        }
    }
}

// reference-layout copy of column 0 (34-byte blocks) for parity taps
__device__ __forceinline__ void matvec_tap(const MatvecParams &p, ActView act) {
    if (p.tap_xq == nullptr || blockIdx.x != 0) { return; }
    for (int b = threadIdx.x; b < act.nb; b += MV_THREADS) {
        uint8_t *o = p.tap_xq + (size_t)b * 34;
        const uint16_t dh = f2h(act.d[b]);
        o[0] = (uint8_t)(dh & 0xff); o[1] = (uint8_t)(dh >> 8);
        const uint8_t *lo = reinterpret_cast<const uint8_t *>(act.lo + b);
        const uint8_t *hi = reinterpret_cast<const uint8_t *>(act.hi + b);
        for (int i = 0; i < 16; ++i) { o[2 + i] = lo[i]; o[18 + i] = hi[i]; }
    }
}

// ---------------------------------------------------------------------------------------------
// epilogue for one finished pair of dot products per column (a0 = first row, a1 = second row)
__device__ __forceinline__ void matvec_epilogue(const MatvecParams &p, int64_t u, int t, float a0, float a1) {
    switch (p.epi) {
    case EPI_STORE: {
        float *o = p.out + (int64_t)t * p.out_stride + 2 * u;
        o[0] = a0; o[1] = a1;
    } break;
    case EPI_RESID: {   // Add(attn_out, x) / Add(ffn_inp, ffn_out): model/src/llm/model/llama.cpp:194-211
        const int64_t i = (int64_t)t * p.out_stride + 2 * u;
        const float r0 = p.resid[i], r1 = p.resid[i + 1];
        p.out[i] = __fadd_rn(a0, r0); p.out[i + 1] = __fadd_rn(a1, r1);
    } break;
    case EPI_SILU_MUL: {  // up * silu(gate): model/src/llm/plugin/ffn.cpp:28-35; silu = table on the fp16-rounded argument
        const float g = p.silu_table[f2h(a1)];
        p.out[(int64_t)t * p.out_stride + u] = __fmul_rn(a0, g);
    } break;
    case EPI_QKV_ROPE: {
        const int64_t row = 2 * u;
        const int     sec = (int)(row / p.dl);
        const int     e   = (int)(row - (int64_t)sec * p.dl);
        const int     pos = *p.pos_base + t;
        if (sec == 2) {   // V: f32 -> f16 RNE into the cache (dup_execute, backend/host/operator/view.cpp:83-227)
            __half2 *dst = reinterpret_cast<__half2 *>(p.v_cache + (int64_t)pos * p.dl + e);
            *dst = __halves2half2(__float2half_rn(a0), __float2half_rn(a1));
        } else {          // RoPE, mode Norm: backend/host/operator/non-linear.cpp:270-371
            const float2 cs = p.rope_table[(int64_t)pos * (p.hd >> 1) + ((e % p.hd) >> 1)];
            const float r0 = __fsub_rn(__fmul_rn(a0, cs.x), __fmul_rn(a1, cs.y));
            const float r1 = __fadd_rn(__fmul_rn(a0, cs.y), __fmul_rn(a1, cs.x));
            __half *base = (sec == 0) ? p.q_out + (int64_t)t * p.dl + e : p.k_cache + (int64_t)pos * p.dl + e;
            *reinterpret_cast<__half2 *>(base) = __halves2half2(__float2half_rn(r0), __float2half_rn(r1));
        }
    } break;
    default: break;
    }
}

// ---------------------------------------------------------------------------------------------
// Register pipeline: D work items in flight per lane. One item = one 32-block chunk of a row pair,
// i.e. per lane one block of each of the two rows. D * 2 * 16 B (Q4_0) of loads per lane are
// outstanding at any time: 256 threads * 256 B = 64 KB per SM, enough to cover HBM latency.
template <int WT> struct Pipe;
template <> struct Pipe<2> { static constexpr int D = 8; };   // Q4_0
template <> struct Pipe<8> { static constexpr int D = 4; };   // Q8_0

template <int WT, int TM>
__global__ void __launch_bounds__(MV_THREADS, (TM == 1) ? 2 : 1) matvec_kernel(const MatvecParams p) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    constexpr int D = Pipe<WT>::D;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nb     = p.A.nb;
    const int nchunk = (nb + 31) >> 5;

    const int64_t n_units     = p.pair_mode ? p.A.n_rows : (p.A.n_rows >> 1);
    const int64_t total_warps = (int64_t)gridDim.x * MV_WARPS;
    const int64_t gw          = (int64_t)blockIdx.x * MV_WARPS + warp;
    const int64_t u0          = n_units * gw / total_warps;
    const int64_t u1          = n_units * (gw + 1) / total_warps;
    const int64_t n_items     = (u1 - u0) * nchunk;

    // row pair addressing: plane0 + u * ustride, plane1 + u * ustride
    const int64_t   ustride = p.pair_mode ? nb : 2 * (int64_t)nb;
    const uint4    *qa0 = p.A.qa;
    const uint4    *qa1 = p.pair_mode ? p.B.qa : p.A.qa + nb;
    const uint4    *qb0 = p.A.qb;
    const uint4    *qb1 = p.pair_mode ? p.B.qb : (p.A.qb ? p.A.qb + nb : nullptr);
    const uint16_t *d0  = p.A.d;
    const uint16_t *d1  = p.pair_mode ? p.B.d : p.A.d + nb;

    uint4    wa[D][2];
    uint4    wb[(WT == 8) ? D : 1][2];
    uint16_t wd[D][2];

    auto load_item = [&](int j, int64_t u, int c) {
        const int b = (c << 5) + lane;
        if (b < nb) {
            const int64_t off = u * ustride + b;
            wa[j][0] = ldg_stream(qa0 + off);
            wa[j][1] = ldg_stream(qa1 + off);
            if (WT == 8) { wb[(WT == 8) ? j : 0][0] = ldg_stream(qb0 + off); wb[(WT == 8) ? j : 0][1] = ldg_stream(qb1 + off); }
            wd[j][0] = ldg_stream_u16(d0 + off);
            wd[j][1] = ldg_stream_u16(d1 + off);
        } else {
            wa[j][0] = make_uint4(0, 0, 0, 0); wa[j][1] = make_uint4(0, 0, 0, 0);
            if (WT == 8) { wb[(WT == 8) ? j : 0][0] = make_uint4(0, 0, 0, 0); wb[(WT == 8) ? j : 0][1] = make_uint4(0, 0, 0, 0); }
            wd[j][0] = 0; wd[j][1] = 0;
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

    ActView act = act_view(smem_raw, nb, TM);
    float  *red = reinterpret_cast<float *>(smem_raw + act_bytes(nb, TM));
    matvec_prologue<TM>(p, act, red);
    __syncthreads();
    matvec_tap(p, act);

    float acc0[TM], acc1[TM];
#pragma unroll
    for (int t = 0; t < TM; ++t) { acc0[t] = 0.f; acc1[t] = 0.f; }

    int64_t cu = u0; int cc = 0;
    for (int64_t base = 0; base < n_items; base += D) {
#pragma unroll
        for (int j = 0; j < D; ++j) {
            if (base + j < n_items) {
                const int   b  = min((cc << 5) + lane, nb - 1);   // out-of-range lanes carry zero weights
                const float s0 = h2f(wd[j][0]), s1 = h2f(wd[j][1]);
#pragma unroll
                for (int t = 0; t < TM; ++t) {
                    const uint4 ylo = act.lo[t * nb + b];
                    const uint4 yhi = act.hi[t * nb + b];
                    const float yd  = act.d[t * nb + b];
                    int i0, i1;
                    if (WT == 2) {
                        const int ys = act.s[t * nb + b];
                        i0 = dot_q4_0_block(wa[j][0], ylo, yhi, ys);
                        i1 = dot_q4_0_block(wa[j][1], ylo, yhi, ys);
                    } else {
                        i0 = dot_q8_0_block(wa[j][0], wb[(WT == 8) ? j : 0][0], ylo, yhi);
                        i1 = dot_q8_0_block(wa[j][1], wb[(WT == 8) ? j : 0][1], ylo, yhi);
                    }
                    acc0[t] = fmaf(__fmul_rn(s0, yd), (float)i0, acc0[t]);
                    acc1[t] = fmaf(__fmul_rn(s1, yd), (float)i1, acc1[t]);
                }
                if (issued < n_items) {
                    load_item(j, lu, lc);
                    ++issued; if (++lc == nchunk) { lc = 0; ++lu; }
                }
                if (++cc == nchunk) {   // row pair finished: reduce over the warp, run the epilogue
                    float v0 = 0.f, v1 = 0.f;
#pragma unroll
                    for (int t = 0; t < TM; ++t) {
                        const float r0 = warp_sum(acc0[t]);
                        const float r1 = warp_sum(acc1[t]);
                        if (lane == t) { v0 = r0; v1 = r1; }
                        acc0[t] = 0.f; acc1[t] = 0.f;
                    }
                    if (lane < p.T) { matvec_epilogue(p, cu, lane, v0, v1); }
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
    const int64_t n_units = p.pair_mode ? p.A.n_rows : (p.A.n_rows >> 1);
    int grid = cfg.num_sms;
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

template <int WT>
static cudaError_t launch_matvec_w(const MatvecParams &p, const LaunchCfg &cfg) {
    if (p.T <= 1) { return launch_matvec_t<WT, 1>(p, cfg); }
    if (p.T <= 2) { return launch_matvec_t<WT, 2>(p, cfg); }
    if (p.T <= 4) { return launch_matvec_t<WT, 4>(p, cfg); }
    return launch_matvec_t<WT, 8>(p, cfg);
}

cudaError_t launch_matvec(const MatvecParams &p, const LaunchCfg &cfg) {
    if (p.T < 1 || p.T > 8) { return cudaErrorInvalidValue; }
    if (p.A.k % QK != 0 || (p.A.k & 3) != 0) { return cudaErrorInvalidValue; }
    if (!p.pair_mode && (p.A.n_rows & 1)) { return cudaErrorInvalidValue; }
    if (p.pair_mode && (p.B.type != p.A.type || p.B.n_rows != p.A.n_rows || p.B.k != p.A.k)) { return cudaErrorInvalidValue; }
    if (matvec_smem_bytes(p.A.nb, p.T <= 1 ? 1 : p.T <= 2 ? 2 : p.T <= 4 ? 4 : 8) > 220 * 1024) { return cudaErrorInvalidValue; }
    switch (p.A.type) {
    case 2: return launch_matvec_w<2>(p, cfg);
    case 8: return launch_matvec_w<8>(p, cfg);
    default: return cudaErrorNotSupported;
    }
}

}  // namespace spyb
