// Attention over the fp16 KV cache (single pass with the reference's exact softmax, or split-K with
// an online-softmax combine for long contexts), the upload re-tiling kernels, and the small
// per-operator kernels that let the reference's graph run op by op on the device.
// All of these are HBM- or latency-bound byte/float work; none is a dense contraction.

#include "spyb_common.cuh"
#include "spyb_kernels.h"

#include <math_constants.h>

namespace spyb {

static inline cudaError_t launch_check() { return cudaGetLastError(); }

// =============================================================================================
// Attention for one (head, query token, KV split).
//   scores = K(f16) . fp16(Q)            MatMul with F16 weights: backend/host/operator/mat.cpp:32-42,
//                                        Dot<FP16,FP16> backend/host/include/simd/vec_dot.h:117-146
//   probs  = masked softmax, exp through the table of expf(fp16(s - max))
//                                        backend/host/operator/non-linear.cpp:129-180
//   out    = V(f16) . fp16(probs)        same MatMul rule
// With n_split == 1 the order of operations and every rounding point (fp16 Q, fp16 exp argument,
// fp16 probabilities) are the reference's; only the f32 summation order differs. With n_split > 1
// each split keeps its own running maximum and the last split to finish merges the partial sums
// (online softmax), which also moves the fp16 rounding of the probabilities: tolerance only.
// Roofline: HBM-bound, 2 * n_kv * head_dim * 2 bytes per head read once.
constexpr int ATT_THREADS = 128;

__global__ void __launch_bounds__(ATT_THREADS) attention_kernel(const AttnParams p) {
    extern __shared__ __align__(16) float att_smem[];
    __shared__ float red[ATT_THREADS / WARP];
    __shared__ int   is_last;

    const int h = blockIdx.x, t = blockIdx.y, sp = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int NW = ATT_THREADS / WARP;

    pdl_launch_dependents();
    pdl_wait();

    const int pos  = *p.pos_base + t;
    const int n_kv = pos + 1;                               // causal mask: positions 0..pos are visible
    const int chunk = (n_kv + p.n_split - 1) / p.n_split;
    const int j0 = min(n_kv, sp * chunk), j1 = min(n_kv, j0 + chunk);
    const int n  = j1 - j0;
    float *sc = att_smem;                                   // n floats

    // head_dim == 128: each lane owns 4 consecutive dims
    const __half2 *q2 = reinterpret_cast<const __half2 *>(p.q + (int64_t)t * p.dl + (int64_t)h * p.hd) + lane * 2;
    const float2 qa = __half22float2(q2[0]), qb = __half22float2(q2[1]);

    for (int j = j0 + warp; j < j1; j += NW) {
        const uint2 kv = *reinterpret_cast<const uint2 *>(p.k_cache + (int64_t)j * p.dl + (int64_t)h * p.hd + lane * 4);
        const float2 ka = __half22float2(*reinterpret_cast<const __half2 *>(&kv.x));
        const float2 kb = __half22float2(*reinterpret_cast<const __half2 *>(&kv.y));
        float s = ka.x * qa.x;
        s = fmaf(ka.y, qa.y, s); s = fmaf(kb.x, qb.x, s); s = fmaf(kb.y, qb.y, s);
        s = warp_sum(s);
        if (lane == 0) { sc[j - j0] = __fmul_rn(s, p.scale); }   // (score + 0) * scale
    }
    __syncthreads();

    float m = -CUDART_INF_F;
    for (int j = tid; j < n; j += ATT_THREADS) { m = fmaxf(m, sc[j]); }
    m = warp_max(m);
    if (lane == 0) { red[warp] = m; }
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < NW; ++w) { m = fmaxf(m, red[w]); }
    __syncthreads();

    float l = 0.f;
    for (int j = tid; j < n; j += ATT_THREADS) {
        const float e = p.exp_table[f2h(__fsub_rn(sc[j], m))];
        sc[j] = e;
        l += e;
    }
    l = warp_sum(l);
    if (lane == 0) { red[warp] = l; }
    __syncthreads();
    l = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) { l += red[w]; }

    if (p.n_split == 1) {
        const float inv = __fdiv_rn(1.0f, l);
        for (int j = tid; j < n; j += ATT_THREADS) { sc[j] = h2f(f2h(__fmul_rn(sc[j], inv))); }
    }
    __syncthreads();

    // out[e] = sum_j prob_j * V[j][e]; thread e walks the positions with 4 loads in flight
    const __half *vcol = p.v_cache + (int64_t)h * p.hd + tid;
    float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
    int j = 0;
    for (; j + 4 <= n; j += 4) {
        const float v0 = __half2float(vcol[(int64_t)(j0 + j) * p.dl]);
        const float v1 = __half2float(vcol[(int64_t)(j0 + j + 1) * p.dl]);
        const float v2 = __half2float(vcol[(int64_t)(j0 + j + 2) * p.dl]);
        const float v3 = __half2float(vcol[(int64_t)(j0 + j + 3) * p.dl]);
        o0 = fmaf(sc[j], v0, o0); o1 = fmaf(sc[j + 1], v1, o1); o2 = fmaf(sc[j + 2], v2, o2); o3 = fmaf(sc[j + 3], v3, o3);
    }
    for (; j < n; ++j) { o0 = fmaf(sc[j], __half2float(vcol[(int64_t)(j0 + j) * p.dl]), o0); }
    const float o = (o0 + o1) + (o2 + o3);

    if (p.n_split == 1) {
        p.out[(int64_t)t * p.dl + (int64_t)h * p.hd + tid] = o;
        return;
    }

    // split-K: publish (max, sum, partial out) and let the last split of this (token, head) merge
    const int    slot_w = p.hd + 2;
    const int    th     = t * p.n_head + h;
    float       *mine   = p.scratch + ((int64_t)th * p.n_split + sp) * slot_w;
    mine[2 + tid] = o;
    if (tid == 0) { mine[0] = m; mine[1] = l; }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int prev = atomicAdd(p.counters + th, 1);
        is_last = (prev == p.n_split - 1);
        if (is_last) { p.counters[th] = 0; }   // ready for the next launch
    }
    __syncthreads();
    if (!is_last) { return; }
    __threadfence();
    const float *all = p.scratch + (int64_t)th * p.n_split * slot_w;
    float gm = -CUDART_INF_F;
    for (int s = 0; s < p.n_split; ++s) { gm = fmaxf(gm, __ldcg(all + s * slot_w)); }
    float gl = 0.f, go = 0.f;
    for (int s = 0; s < p.n_split; ++s) {
        const float ms = __ldcg(all + s * slot_w), ls = __ldcg(all + s * slot_w + 1);
        if (ls > 0.f) {
            const float w = expf(ms - gm);
            gl = fmaf(ls, w, gl);
            go = fmaf(__ldcg(all + s * slot_w + 2 + tid), w, go);
        }
    }
    p.out[(int64_t)t * p.dl + (int64_t)h * p.hd + tid] = __fdiv_rn(go, gl);
}

size_t attention_scratch_floats(int T, int n_head, int n_split, int hd) { return (size_t)T * n_head * n_split * (hd + 2); }

cudaError_t launch_attention(const AttnParams &p, const LaunchCfg &cfg) {
    if (p.hd != 128 || p.n_split < 1 || p.T < 1) { return cudaErrorInvalidValue; }
    if (p.n_split > 1 && (p.scratch == nullptr || p.counters == nullptr)) { return cudaErrorInvalidValue; }
    const int    chunk_max = (p.n_ctx + p.n_split - 1) / p.n_split;
    const size_t smem      = (size_t)chunk_max * sizeof(float) + 16;
    if (smem > 200 * 1024) { return cudaErrorInvalidValue; }
    static size_t smem_allowed = 40 * 1024;
    if (smem > smem_allowed) {
        cudaError_t err = cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) { return err; }
        smem_allowed = smem;
    }
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(p.n_head, p.T, p.n_split); lc.blockDim = dim3(ATT_THREADS); lc.dynamicSmemBytes = smem; lc.stream = cfg.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr; lc.numAttrs = cfg.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&lc, attention_kernel, p);
}

// =============================================================================================
// upload-time re-tiling: raw 18-byte / 34-byte blocks -> aligned planes (one thread per block)
__global__ void retile_q4_0_kernel(const uint8_t *raw, int64_t row_stride, int64_t n_rows, int nb, uint4 *qa, uint16_t *d) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows * nb) { return; }
    const int64_t  r = i / nb, b = i - r * nb;
    const uint8_t *src = raw + r * row_stride + b * 18;
    d[i] = (uint16_t)(src[0] | (src[1] << 8));
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) { w[k] = src[2 + 4 * k] | (src[3 + 4 * k] << 8) | (src[4 + 4 * k] << 16) | ((uint32_t)src[5 + 4 * k] << 24); }
    qa[i] = make_uint4(w[0], w[1], w[2], w[3]);
}

__global__ void retile_q8_0_kernel(const uint8_t *raw, int64_t row_stride, int64_t n_rows, int nb, uint4 *qa, uint4 *qb, uint16_t *d) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows * nb) { return; }
    const int64_t  r = i / nb, b = i - r * nb;
    const uint8_t *src = raw + r * row_stride + b * 34;
    d[i] = (uint16_t)(src[0] | (src[1] << 8));
    uint32_t w[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) { w[k] = src[2 + 4 * k] | (src[3 + 4 * k] << 8) | (src[4 + 4 * k] << 16) | ((uint32_t)src[5 + 4 * k] << 24); }
    qa[i] = make_uint4(w[0], w[1], w[2], w[3]);
    qb[i] = make_uint4(w[4], w[5], w[6], w[7]);
}

cudaError_t launch_retile_q4_0(const uint8_t *raw, int64_t row_stride, int64_t n_rows, int nb, uint4 *qa, uint16_t *d, cudaStream_t s) {
    const int64_t n = n_rows * nb;
    if (n == 0) { return cudaSuccess; }
    retile_q4_0_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(raw, row_stride, n_rows, nb, qa, d);
    return launch_check();
}
cudaError_t launch_retile_q8_0(const uint8_t *raw, int64_t row_stride, int64_t n_rows, int nb, uint4 *qa, uint4 *qb, uint16_t *d, cudaStream_t s) {
    const int64_t n = n_rows * nb;
    if (n == 0) { return cudaSuccess; }
    retile_q8_0_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(raw, row_stride, n_rows, nb, qa, qb, d);
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
    uint32_t yw[8]; int ys = 0;
    for (int k = 0; k < 8; ++k) { yw[k] = y[4 * k] | (y[4 * k + 1] << 8) | (y[4 * k + 2] << 16) | ((uint32_t)y[4 * k + 3] << 24); }
    for (int k = 0; k < 32; ++k) { ys += (int)(int8_t)y[k]; }
    const uint4 ylo = make_uint4(yw[0], yw[1], yw[2], yw[3]), yhi = make_uint4(yw[4], yw[5], yw[6], yw[7]);
    if (wtype == 2) {
        const uint8_t *q = w + b * 18 + 2;
        uint32_t ww[4];
        for (int k = 0; k < 4; ++k) { ww[k] = q[4 * k] | (q[4 * k + 1] << 8) | (q[4 * k + 2] << 16) | ((uint32_t)q[4 * k + 3] << 24); }
        out[b] = dot_q4_0_block(make_uint4(ww[0], ww[1], ww[2], ww[3]), ylo, yhi, ys);
    } else {
        const uint8_t *q = w + b * 34 + 2;
        uint32_t ww[8];
        for (int k = 0; k < 8; ++k) { ww[k] = q[4 * k] | (q[4 * k + 1] << 8) | (q[4 * k + 2] << 16) | ((uint32_t)q[4 * k + 3] << 24); }
        out[b] = dot_q8_0_block(make_uint4(ww[0], ww[1], ww[2], ww[3]), make_uint4(ww[4], ww[5], ww[6], ww[7]), ylo, yhi);
    }
}

cudaError_t launch_block_dots(int wtype, const uint8_t *w_row, const uint8_t *x_blocks, int64_t n, int32_t *out, cudaStream_t s) {
    if ((wtype != 2 && wtype != 8) || n % QK != 0) { return cudaErrorInvalidValue; }
    const int64_t nblk = n / QK;
    if (nblk == 0) { return cudaSuccess; }
    block_dots_kernel<<<(unsigned)((nblk + 127) / 128), 128, 0, s>>>(wtype, w_row, x_blocks, nblk, out);
    return launch_check();
}

// =============================================================================================
// per-operator kernels (each mirrors one OperatorImpl of backend/host/operator/*.cpp)

// OperatorNormRMSImpl::execute, non-linear.cpp:194-223; one CTA per row
__global__ void rmsnorm_kernel(const float *x, float *out, int64_t n, float eps) {
    __shared__ float red[8];
    const float *xr = x + (int64_t)blockIdx.x * n;
    float       *o  = out + (int64_t)blockIdx.x * n;
    float ss = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) { ss = fmaf(xr[i], xr[i], ss); }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) { red[threadIdx.x >> 5] = ss; }
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) { tot += red[w]; }
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)n), eps)));
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) { o[i] = __fmul_rn(xr[i], scale); }
}
cudaError_t launch_rmsnorm(const float *x, float *out, int64_t n, int64_t rows, float eps, cudaStream_t s) {
    if (rows == 0 || n == 0) { return cudaSuccess; }
    rmsnorm_kernel<<<(unsigned)rows, 256, 0, s>>>(x, out, n, eps);
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

// operator_masked_softmax_execute, non-linear.cpp:129-180; one CTA per row (i1, i2), row length ne0
__global__ void softmax_masked_kernel(const float *scores, const float *mask, float *out, int64_t ne0, int64_t ne1,
                                      int64_t mask_stride, float scale, const float *exp_table) {
    __shared__ float red[8];
    const int64_t row = blockIdx.x;
    const int64_t i1  = row % ne1;
    const float  *src = scores + row * ne0;
    const float  *mk  = mask + i1 * mask_stride;
    float        *dst = out + row * ne0;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float m = -CUDART_INF_F;
    for (int64_t i = threadIdx.x; i < ne0; i += blockDim.x) {
        const float v = __fmul_rn(__fadd_rn(src[i], mk[i]), scale);
        dst[i] = v;
        m = fmaxf(m, v);
    }
    m = warp_max(m);
    if (lane == 0) { red[warp] = m; }
    __syncthreads();
    m = red[0];
    for (int w = 1; w < nw; ++w) { m = fmaxf(m, red[w]); }
    __syncthreads();
    float l = 0.f;
    for (int64_t i = threadIdx.x; i < ne0; i += blockDim.x) {
        const float e = (mk[i] == -CUDART_INF_F) ? 0.f : exp_table[f2h(__fsub_rn(dst[i], m))];
        dst[i] = e;
        l += e;
    }
    l = warp_sum(l);
    if (lane == 0) { red[warp] = l; }
    __syncthreads();
    l = 0.f;
    for (int w = 0; w < nw; ++w) { l += red[w]; }
    const float inv = __fdiv_rn(1.0f, l);
    for (int64_t i = threadIdx.x; i < ne0; i += blockDim.x) { dst[i] = __fmul_rn(dst[i], inv); }
}
cudaError_t launch_softmax_masked(const float *scores, const float *mask, float *out, int64_t ne0, int64_t ne1, int64_t ne2,
                                  int64_t mask_stride, float scale, const float *exp_table, cudaStream_t s) {
    if (ne0 == 0 || ne1 * ne2 == 0) { return cudaSuccess; }
    softmax_masked_kernel<<<(unsigned)(ne1 * ne2), 256, 0, s>>>(scores, mask, out, ne0, ne1, mask_stride, scale, exp_table);
    return launch_check();
}

__device__ __forceinline__ int64_t soff(const Strided &t, int64_t i0, int64_t i1, int64_t i2, int64_t i3) {
    return i0 * t.nb[0] + i1 * t.nb[1] + i2 * t.nb[2] + i3 * t.nb[3];
}

// OperatorRopeImpl::execute in mode Norm with default YaRN settings, non-linear.cpp:270-371.
// One thread per (pair, head, token); theta is advanced by repeated f32 multiplication as the CPU does.
__global__ void rope_kernel(const Strided x, const int32_t *pos, const Strided out, float theta_scale, int n_dim) {
    const int64_t npair = x.ne[0] >> 1;
    const int64_t i     = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t tot   = npair * x.ne[1] * x.ne[2];
    if (i >= tot) { return; }
    const int64_t k = i % npair, i1 = (i / npair) % x.ne[1], i2 = i / (npair * x.ne[1]);
    float theta = (float)pos[i2];
    for (int64_t j = 0; j < k; ++j) { theta = __fmul_rn(theta, theta_scale); }
    const float c = cosf(theta), s = sinf(theta);
    const float *src = reinterpret_cast<const float *>(reinterpret_cast<const uint8_t *>(x.data) + soff(x, 2 * k, i1, i2, 0));
    float       *dst = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(out.data) + soff(out, 2 * k, i1, i2, 0));
    const float x0 = src[0], x1 = src[1];
    dst[0] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
    dst[1] = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
    (void)n_dim;
}
cudaError_t launch_rope(const Strided &x, const int32_t *pos, const Strided &out, float freq_base, int n_dim, cudaStream_t s) {
    const int64_t tot = (x.ne[0] >> 1) * x.ne[1] * x.ne[2];
    if (tot == 0) { return cudaSuccess; }
    const float theta_scale = powf(freq_base, -2.0f / (float)n_dim);
    rope_kernel<<<(unsigned)((tot + 127) / 128), 128, 0, s>>>(x, pos, out, theta_scale, n_dim);
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

// embedding row -> f32: memcpy for F32, Q8_0 -> F32 as OperatorGetRowImpl::execute (view.cpp:33-81);
// Q4_0 rows (which the CPU backend cannot gather) decode as (nibble - 8) * d.
__device__ __forceinline__ float embd_value(const uint8_t *row, int type, int64_t i) {
    if (type == 0) { return reinterpret_cast<const float *>(row)[i]; }
    if (type == 1) { return h2f(reinterpret_cast<const uint16_t *>(row)[i]); }
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
    if (table_type != 0 && table_type != 1 && table_type != 2 && table_type != 8) { return cudaErrorNotSupported; }
    if (n_ids == 0) { return cudaSuccess; }
    getrow_kernel<<<(unsigned)n_ids, 256, 0, s>>>(table, table_type, row_bytes, ne0, ids, out);
    return launch_check();
}
cudaError_t launch_embed(const int32_t *ids, int n_ids, const uint8_t *embd, int embd_type, int64_t d_model, float *x_out, cudaStream_t s) {
    const int64_t rb = embd_type == 0 ? d_model * 4 : embd_type == 1 ? d_model * 2 : embd_type == 8 ? d_model / 32 * 34 : d_model / 32 * 18;
    return launch_getrow(embd, embd_type, rb, d_model, ids, n_ids, x_out, s);
}

// MatMul with an F16 weight and f32 activations (the attention products when run op by op):
// activations are rounded to fp16 first (mat.cpp:32-42), f32 accumulate. One warp per output.
__global__ void matmul_f16_kernel(const Strided w, const Strided x, const Strided out) {
    const int64_t n_out = out.ne[0] * out.ne[1] * out.ne[2];
    const int64_t o     = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int     lane  = threadIdx.x & 31;
    if (o >= n_out) { return; }
    const int64_t i01 = o % out.ne[0], i11 = (o / out.ne[0]) % out.ne[1], i02 = o / (out.ne[0] * out.ne[1]);
    const uint8_t *wp = reinterpret_cast<const uint8_t *>(w.data) + soff(w, 0, i01, i02, 0);
    const uint8_t *xp = reinterpret_cast<const uint8_t *>(x.data) + soff(x, 0, i11, i02, 0);
    float acc = 0.f;
    for (int64_t k = lane; k < w.ne[0]; k += 32) {
        const float a = h2f(*reinterpret_cast<const uint16_t *>(wp + k * w.nb[0]));
        const float b = h2f(f2h(*reinterpret_cast<const float *>(xp + k * x.nb[0])));
        acc = fmaf(a, b, acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) { *reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(out.data) + soff(out, i01, i11, i02, 0)) = acc; }
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
        }
    }
    __syncthreads();
    if (embd != nullptr) {
        const int64_t rb = embd_type == 0 ? d_model * 4 : embd_type == 1 ? d_model * 2 : embd_type == 8 ? d_model / 32 * 34 : d_model / 32 * 18;
        const uint8_t *row = embd + (int64_t)winner * rb;
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

}  // namespace spyb
