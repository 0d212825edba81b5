// Dequant-fused mat-vec for K-quant weights (Q4_K: 144 B / 256 values, Q6_K: 210 B / 256 values; block layouts
// orchestration/include/number/number_impl/k-quant.h:79-117, 162-188) inside the fused step plan.
//
// Parity is unpinned by the reference: it defines these layouts but no arithmetic for them (a K-quant weight makes its
// MatMul pick a quantizer that throws, backend/host/include/simd/vec_convert.h:30-36). What is reproduced here, bit for
// bit, is the CPU restatement used as the checker: the reference's MatMul rule for quantized weights - activations
// quantized to Q8_0 first (backend/host/operator/mat.cpp:32-42, 95-128) - with, per 256-value super-block,
//   Q4_K:  acc = 0; for the 8 sub-blocks j of 32 values: acc = fma((d * sc_j) * dx_j, (float)sum(q * y), acc);
//                                                         acc = fma(-((dmin * m_j) * dx_j), (float)sum(y), acc)
//   Q6_K:  acc = 0; for the 16 groups g of 16 values:    acc = fma((d * sc_g) * dx_(g/2), (float)sum(q * y), acc)
// and the row's result = the super-blocks' values added in order. The integer sums are exact, so only this order matters.
//
// Mapping: a super-block's value depends on nothing before it, so the lanes of a (half-)warp take the super-blocks of
// one row side by side - each lane streams its 144 (208 + 2) bytes with 128-bit read-only loads, consecutive lanes
// consecutive super-blocks, i.e. the warp reads the row as one contiguous run - and the per-row sum is a short ordered
// walk over the lanes' values. A warp owns a pair of rows (rows 2u, 2u+1 rotate together in RoPE; FFN up row i and gate
// row i meet in the SiLU epilogue). HBM-bound: rows * K/256 * 144 (210) bytes per launch, read once, no re-tiling for
// Q4_K; Q6_K rows are re-laid at upload so that every piece is 16-byte aligned (208-byte bodies, the fp16 scales of a
// row together at its end). Activations: Q8_0 in shared memory, one 68-word stride per super-block so that a block's words
// are aligned 128-bit reads and the lanes of a quarter-warp, working on different super-blocks, hit different banks.

#include <algorithm>

#include "spyb_common.cuh"
#include "spyb_kernels.h"
#include "spyb_tp.cuh"
#include "spyb_mv_common.cuh"

namespace spyb {

constexpr int KQ_THREADS = 512;
constexpr int KQ_WARPS   = KQ_THREADS / WARP;
constexpr int KQ_SB_WORDS = 68;   // words per super-block of activations in shared memory: 64 + 4, so that a block's eight words are two aligned
                                  // 128-bit reads and the eight lanes of a quarter-warp (one super-block each) hit distinct banks

// the planes of one activation column; column t of a pass lies t * col 32-bit words further (all three planes)
struct KqPlanes { uint32_t *y; float *dx; int *ysum; int col; };

// NormRMS + Mul(weight) (optional) + Quantizator<FP32,Q8_0> of one activation column into the K-quant planes; the
// arithmetic is that of the Q4_0 / Q8_0 kernels' prologue (same device functions)
template <bool NORM>
__device__ __forceinline__ void kq_prologue(const MatvecParams &p, const float *x, KqPlanes a, float *v3, float *scale_s) {
    const int tid = threadIdx.x;
    const int n4  = (int)(p.A.k >> 2);
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    float scale = 1.f;
    if (NORM) {
        for (int g = tid; g < n4; g += KQ_THREADS) {
            const float4 v = __ldcg(x4 + g);
            const float v1 = fmaf(v.y, v.y, __fmul_rn(v.x, v.x));
            const float v2 = fmaf(v.w, v.w, __fmul_rn(v.z, v.z));
            v3[g] = __fadd_rn(v1, v2);
        }
        __syncthreads();
        if (tid == 0) {
            const float sum  = running_sum_serial(v3, n4);
            const float mean = __fdiv_rn(sum, (float)p.A.k);
            *scale_s = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, p.eps)));
        }
        __syncthreads();   // also: the partials (aliasing the planes) are dead from here on
        scale = *scale_s;
    }
    const float4 *w4 = reinterpret_cast<const float4 *>(p.norm_w);
    for (int base = 0; base < n4; base += KQ_THREADS) {   // n4 is a multiple of 64: whole warps, whole blocks
        const int g = base + tid;
        const bool valid = g < n4;
        float4 v = valid ? __ldcg(x4 + g) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (NORM && valid) {
            const float4 w = w4[g];
            v.x = __fmul_rn(__fmul_rn(v.x, scale), w.x); v.y = __fmul_rn(__fmul_rn(v.y, scale), w.y);
            v.z = __fmul_rn(__fmul_rn(v.z, scale), w.z); v.w = __fmul_rn(__fmul_rn(v.w, scale), w.w);
        }
        uint16_t dh; int s;
        const uint32_t q = quantize_q8_lane4(v, dh, s);
        s += __shfl_xor_sync(0xffffffffu, s, 1); s += __shfl_xor_sync(0xffffffffu, s, 2); s += __shfl_xor_sync(0xffffffffu, s, 4);
        if (valid) {
            const int b = g >> 3, w = g & 7;
            a.y[(b >> 3) * KQ_SB_WORDS + (b & 7) * 8 + w] = q;
            if (w == 0) { a.dx[b] = h2f(dh); a.ysum[b] = s; }
        }
    }
}

__device__ __forceinline__ uint4 ldg_nc(const uint8_t *p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// 6-bit scale / min j of a Q4_K super-block from its 12 packed bytes (three words)
__device__ __forceinline__ void kq_scale_min(const uint32_t (&sw)[3], int j, float &sc, float &mn) {
    auto byte = [&](int i) { return (sw[i >> 2] >> (8 * (i & 3))) & 0xffu; };
    if (j < 4) { sc = (float)(byte(j) & 63u); mn = (float)(byte(j + 4) & 63u); }
    else { sc = (float)((byte(j + 4) & 0xFu) | ((byte(j - 4) >> 6) << 4)); mn = (float)((byte(j + 4) >> 4) | ((byte(j) >> 6) << 4)); }
}

// values of one Q4_K super-block for the nT <= TM activation columns of a pass: wb = its 144 bytes in global memory, sb = its
// index (the activations of column t: 8 blocks x 8 words at a.y + t * a.col + sb * KQ_SB_WORDS, their scales and integer
// sums at a.dx / a.ysum + t * a.col + 8 * sb). The weights are read and unpacked once for all columns.
template <int TM>
__device__ __forceinline__ void kq_values_q4k(const uint8_t *wb, const KqPlanes &a, int sb, int nT, float (&acc)[TM]) {
    const uint4 hd = ldg_nc(wb);
    uint4 q[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { q[i] = ldg_nc(wb + 16 + 16 * i); }
    const float2 dm = __half22float2(*reinterpret_cast<const __half2 *>(&hd.x));   // d, dmin
    const uint32_t sw[3] = {hd.y, hd.z, hd.w};
#pragma unroll
    for (int t = 0; t < TM; ++t) { acc[t] = 0.f; }
#pragma unroll
    for (int j = 0; j < 8; ++j) {          // sub-block j: bytes 32 * (j / 2) .. + 31 of qs, low nibbles when j is even
        const uint4 qa = q[2 * (j >> 1)], qb = q[2 * (j >> 1) + 1];
        const uint32_t w8[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
        uint32_t nib[8];
#pragma unroll
        for (int w = 0; w < 8; ++w) { nib[w] = (j & 1) ? (w8[w] >> 4) & 0x0f0f0f0fu : w8[w] & 0x0f0f0f0fu; }
        float sc, mn; kq_scale_min(sw, j, sc, mn);
        const float dsc = __fmul_rn(dm.x, sc), dmn = __fmul_rn(dm.y, mn);
#pragma unroll
        for (int t = 0; t < TM; ++t) {
            if (TM == 1 || t < nT) {
                const uint32_t *ysb = a.y + t * a.col + sb * KQ_SB_WORDS;
                const uint4 ya = *reinterpret_cast<const uint4 *>(ysb + j * 8), yb = *reinterpret_cast<const uint4 *>(ysb + j * 8 + 4);
                const uint32_t y8[8] = {ya.x, ya.y, ya.z, ya.w, yb.x, yb.y, yb.z, yb.w};
                int isum = 0;
#pragma unroll
                for (int w = 0; w < 8; ++w) { isum = __dp4a((int)nib[w], (int)y8[w], isum); }
                const float dxj = a.dx[t * a.col + 8 * sb + j];
                acc[t] = fmaf(__fmul_rn(dsc, dxj), (float)isum, acc[t]);
                acc[t] = fmaf(-__fmul_rn(dmn, dxj), (float)a.ysum[t * a.col + 8 * sb + j], acc[t]);
            }
        }
    }
}

// values of one Q6_K super-block in the upload layout: wb = 208 bytes (ql 128, qh 64, 16 int8 scales), d = its fp16 scale
template <int TM>
__device__ __forceinline__ void kq_values_q6k(const uint8_t *wb, uint16_t d_half, const KqPlanes &a, int sb, int nT, float (&acc)[TM]) {
    uint4 ql[8], qh[4];
#pragma unroll
    for (int i = 0; i < 8; ++i) { ql[i] = ldg_nc(wb + 16 * i); }
#pragma unroll
    for (int i = 0; i < 4; ++i) { qh[i] = ldg_nc(wb + 128 + 16 * i); }
    const uint4 scw = ldg_nc(wb + 192);
    const float d = h2f(d_half);
    const uint32_t scs[4] = {scw.x, scw.y, scw.z, scw.w};
#pragma unroll
    for (int t = 0; t < TM; ++t) { acc[t] = 0.f; }
#pragma unroll
    for (int g = 0; g < 16; ++g) {
        // group g = values 16g .. 16g+15: half h of the super-block, segment s of 32 values, l = 16 * (g & 1) .. + 15
        //   s 0: ql[64h + l] low | qh[32h + l] bits 0-1     s 1: ql[64h + 32 + l] low  | bits 2-3
        //   s 2: ql[64h + l] high | bits 4-5                s 3: ql[64h + 32 + l] high | bits 6-7
        const int h = g >> 3, sg = (g >> 1) & 3, l0 = 16 * (g & 1);
        const uint4 lv = ql[(64 * h + 32 * (sg & 1) + l0) >> 4], hv = qh[(32 * h + l0) >> 4];
        const uint32_t lw[4] = {lv.x, lv.y, lv.z, lv.w}, hw[4] = {hv.x, hv.y, hv.z, hv.w};
        uint32_t v6[4];                                          // the group's values 0..63, four per word
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const uint32_t lo = (sg & 2) ? (lw[w] >> 4) & 0x0f0f0f0fu : lw[w] & 0x0f0f0f0fu;
            v6[w] = lo | (((hw[w] >> (2 * sg)) & 0x03030303u) << 4);
        }
        const int sc = (int)(int8_t)((scs[g >> 2] >> (8 * (g & 3))) & 0xffu);
        const float dsc = __fmul_rn(d, (float)sc);
#pragma unroll
        for (int t = 0; t < TM; ++t) {
            if (TM == 1 || t < nT) {
                const uint4 yv = *reinterpret_cast<const uint4 *>(a.y + t * a.col + sb * KQ_SB_WORDS + (g >> 1) * 8 + 4 * (g & 1));
                const uint32_t y4[4] = {yv.x, yv.y, yv.z, yv.w};
                int isum = 0, ys = 0;
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    isum = __dp4a((int)v6[w], (int)y4[w], isum);
                    ys   = __dp4a(0x01010101, (int)y4[w], ys);
                }
                isum -= 32 * ys;                                 // value = stored - 32
                acc[t] = fmaf(__fmul_rn(dsc, a.dx[t * a.col + 8 * sb + (g >> 1)]), (float)isum, acc[t]);
            }
        }
    }
}

struct KqRow { const uint8_t *w; int type; };
__device__ __forceinline__ KqRow kq_row(const MatvecParams &p, int64_t row, int pair_second) {
    KqRow r;
    if (p.pair_mode) { const KqSeg &s = p.kq[pair_second]; r.w = s.w + row * s.row_bytes; r.type = s.type; return r; }
    int i = 0;
    while (i + 1 < p.kq_n && row >= p.kq[i].n_rows) { row -= p.kq[i].n_rows; ++i; }
    r.w = p.kq[i].w + row * p.kq[i].row_bytes; r.type = p.kq[i].type;
    return r;
}

// dot products of one row with the nT <= TM activation columns of the pass, for the lanes [lane0, lane0 + G) of the warp;
// every lane of the group ends with the same values
template <int G, int TM>
__device__ __forceinline__ void kq_row_dot(const KqRow &r, int nsb, const KqPlanes &a, int nT, int l /* lane inside the group */, int lane0, float (&total)[TM]) {
    constexpr int ROUNDS = 4;      // super-blocks per lane (K <= 256 * G * ROUNDS)
    float part[ROUNDS][TM];
#pragma unroll
    for (int k = 0; k < ROUNDS; ++k) {
        const int sb = l + k * G;
#pragma unroll
        for (int t = 0; t < TM; ++t) { part[k][t] = 0.f; }
        if (k * G < nsb && sb < nsb) {
            if (r.type == 12) { kq_values_q4k<TM>(r.w + (size_t)sb * 144, a, sb, nT, part[k]); }
            else {
                const uint16_t dh = *reinterpret_cast<const uint16_t *>(r.w + (size_t)nsb * 208 + 2 * sb);
                kq_values_q6k<TM>(r.w + (size_t)sb * 208, dh, a, sb, nT, part[k]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < TM; ++t) {
        float sum = 0.f;             // the super-blocks' values in order
        if (TM == 1 || t < nT) {
#pragma unroll
            for (int k = 0; k < ROUNDS; ++k) {
                if (k * G >= nsb) { break; }
                for (int i = 0; i < G; ++i) {
                    const float v = __shfl_sync(0xffffffffu, part[k][t], lane0 + i);
                    if (i + k * G < nsb) { sum = __fadd_rn(sum, v); }
                }
            }
        }
        total[t] = sum;
    }
}

template <int TM>
__global__ void __launch_bounds__(KQ_THREADS, 1) matvec_kq_kernel(const MatvecParams p) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ float scale_s;
    const int nb = p.A.nb, nsb = nb >> 3;
    const int nT = (TM == 1) ? 1 : p.T;
    KqPlanes a;
    a.col  = nsb * KQ_SB_WORDS + 2 * nb;
    a.y    = reinterpret_cast<uint32_t *>(smem_raw);
    a.dx   = reinterpret_cast<float *>(a.y + (size_t)nsb * KQ_SB_WORDS);
    a.ysum = reinterpret_cast<int *>(a.dx + nb);
    pdl_launch_dependents();
    pdl_wait();
    tp_wait(p.tp, p.error_flag);
#pragma unroll 1
    for (int t = 0; t < nT; ++t) {
        KqPlanes c = a;
        c.y += t * a.col; c.dx += t * a.col; c.ysum += t * a.col;
        float *v3 = reinterpret_cast<float *>(c.y);   // nb * 8 floats = the size of the y plane (nb * 32 bytes): aliases it
        const float *x = p.x + (int64_t)t * p.x_stride;
        if (p.pro == PRO_NORM_QUANT) { kq_prologue<true>(p, x, c, v3, &scale_s); } else { kq_prologue<false>(p, x, c, v3, &scale_s); }
        __syncthreads();
    }

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t n_units = p.pair_mode ? p.kq[0].n_rows : (p.A.n_rows >> 1);
    for (int64_t u = (int64_t)blockIdx.x * KQ_WARPS + warp; u < n_units; u += (int64_t)gridDim.x * KQ_WARPS) {
        const int64_t row_a = p.pair_mode ? u : 2 * u, row_b = p.pair_mode ? u : 2 * u + 1;
        float va[TM], vb[TM];
        if (nsb <= 16) {            // both rows at once, a half-warp each
            const int half = lane >> 4;
            const KqRow r = kq_row(p, half ? row_b : row_a, half);
            float v[TM];
            kq_row_dot<16, TM>(r, nsb, a, nT, lane & 15, lane & 16, v);
#pragma unroll
            for (int t = 0; t < TM; ++t) { va[t] = __shfl_sync(0xffffffffu, v[t], 0); vb[t] = __shfl_sync(0xffffffffu, v[t], 16); }
        } else {
            kq_row_dot<32, TM>(kq_row(p, row_a, 0), nsb, a, nT, lane, 0, va);
            kq_row_dot<32, TM>(kq_row(p, row_b, 1), nsb, a, nT, lane, 0, vb);
        }
#pragma unroll
        for (int t = 0; t < TM; ++t) {
            const bool store = lane == 0 && t < nT;
            if (p.epi == EPI_SILU_MUL) { matvec_epilogue_silu(p, u, t, va[t], vb[t], store); }
            else {
                matvec_epilogue(p, row_a, t, va[t], vb[t], store);
                matvec_epilogue(p, row_b, t, vb[t], va[t], store);
            }
        }
    }
    tp_publish(p.tp, p.T);
}

cudaError_t launch_matvec_kq(const MatvecParams &p, const LaunchCfg &cfg) {
    if (p.T < 1 || p.T > KQ_MAX_COLUMNS || p.kq_n < 1 || p.kq_n > 3 || p.A.k % 256 != 0 || p.A.k > 256 * 32 * 4 || p.A.nb != (int)(p.A.k / QK)) { return cudaErrorInvalidValue; }
    if (p.pair_mode ? (p.kq_n != 2 || p.kq[0].n_rows != p.kq[1].n_rows || p.epi != EPI_SILU_MUL) : (p.epi == EPI_SILU_MUL || (p.A.n_rows & 1))) { return cudaErrorInvalidValue; }
    for (int i = 0; i < p.kq_n; ++i) {
        if ((p.kq[i].type != 12 && p.kq[i].type != 14) || p.kq[i].w == nullptr || (p.kq[i].n_rows & 1) || (reinterpret_cast<uintptr_t>(p.kq[i].w) & 15) || (p.kq[i].row_bytes & 15)) { return cudaErrorInvalidValue; }
    }
    const int nsb = (int)(p.A.k / 256);
    const int    TM   = p.T == 1 ? 1 : KQ_MAX_COLUMNS;
    const size_t smem = (size_t)TM * ((size_t)nsb * KQ_SB_WORDS * 4 + (size_t)p.A.nb * 8) + 16;
    void (*kernel)(const MatvecParams) = p.T == 1 ? matvec_kq_kernel<1> : matvec_kq_kernel<KQ_MAX_COLUMNS>;
    cudaError_t err = allow_dynamic_smem(reinterpret_cast<const void *>(kernel), smem);
    if (err != cudaSuccess) { return err; }
    MatvecParams q = p;
    if (q.error_flag == nullptr) { q.error_flag = cfg.error_flag; }
    const int64_t n_units = p.pair_mode ? p.kq[0].n_rows : (p.A.n_rows >> 1);
    const int64_t grid = std::max<int64_t>(1, std::min<int64_t>(cfg.num_sms, (n_units + KQ_WARPS - 1) / KQ_WARPS));
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)grid); lc.blockDim = dim3(KQ_THREADS); lc.dynamicSmemBytes = smem; lc.stream = cfg.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr; lc.numAttrs = cfg.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&lc, kernel, q);
}

// upload-time re-layout of Q6_K rows: [sb][ql 128 | qh 64 | scales 16 | d 2] (210 bytes each) ->
// [sb][ql 128 | qh 64 | scales 16] (208 bytes each), then the row's fp16 d values, the row padded to a multiple of 16 bytes
__global__ void kq_relayout_q6k_kernel(const uint8_t *raw, int64_t n_rows, int nsb, uint8_t *dst, int64_t dst_row_bytes) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows * nsb) { return; }
    const int64_t row = i / nsb; const int sb = (int)(i - row * nsb);
    const uint8_t *s = raw + (row * nsb + sb) * 210;
    uint8_t *d = dst + row * dst_row_bytes + (size_t)sb * 208;
    for (int k = 0; k < 208; ++k) { d[k] = s[k]; }
    uint8_t *dd = dst + row * dst_row_bytes + (size_t)nsb * 208 + 2 * sb;
    dd[0] = s[208]; dd[1] = s[209];
}
int64_t kq_row_bytes(int type, int64_t k) {
    const int64_t nsb = k / 256;
    return type == 12 ? nsb * 144 : ((nsb * 210 + 15) / 16) * 16;
}
cudaError_t launch_kq_relayout_q6k(const uint8_t *raw, int64_t n_rows, int64_t k, uint8_t *dst, cudaStream_t s) {
    const int nsb = (int)(k / 256);
    const int64_t n = n_rows * nsb;
    if (n == 0) { return cudaSuccess; }
    kq_relayout_q6k_kernel<<<(unsigned)((n + 127) / 128), 128, 0, s>>>(raw, n_rows, nsb, dst, kq_row_bytes(14, k));
    return cudaGetLastError();
}

}  // namespace spyb
