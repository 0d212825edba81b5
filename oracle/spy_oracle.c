/*
 * Test infrastructure, not product code: a plain-C restatement of the reference
 * (BL-GS/Spy) CPU algorithm for the LLaMa token loop. Only tests/, smoke() and the
 * CPU-baseline leg of bench.py may load this library; the GPU library never does.
 *
 * Parity pin: every function below is checked bit-for-bit (integers, bytes, and the
 * f32 results of the block dots, norm, softmax, rope and whole-model logits) against
 * the reference's own sources compiled unmodified into oracle/_ref/libspy_ref.so
 * (tests/test_oracle_vs_reference.py), and against the golden vectors generated from
 * that build under tests/golden/. The reference itself ships no golden vectors
 * (test/src/temp.cpp:3-5 is a placeholder).
 *
 * Q4_K / Q6_K: the reference declares only the block layouts
 * (orchestration/include/number/number_impl/k-quant.h:79-117, 162-188) and has no dot
 * product for them, so those paths here are "parity unpinned": they extend the
 * reference's MatMul rule (quantize f32 activations to Q8_0, integer block dots) to the
 * K-quant layouts.
 *
 * File:line citations are paths inside the reference project.
 * Build: gcc -std=c11 -O2 -ffp-contract=off (every fused multiply-add is an explicit fmaf).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

enum { T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q8_0 = 8, T_Q4_K = 12, T_Q6_K = 14 };

/* ---------------------------------------------------------------- fp16 <-> fp32 */
/* spy_fp16_to_fp32 is an exact table lookup (orchestration/include/number/lookup_table.h:52);
 * spy_fp32_to_fp16 rounds to nearest even (lookup_table.h:54). */
static inline float h2f(uint16_t h) { _Float16 v; memcpy(&v, &h, 2); return (float)v; }
static inline uint16_t f2h(float f) { _Float16 v = (_Float16)f; uint16_t h; memcpy(&h, &v, 2); return h; }

float    oracle_fp16_to_fp32(uint16_t h) { return h2f(h); }
uint16_t oracle_fp32_to_fp16(float f)    { return f2h(f); }

/* The silu and exp tables hold f(xh) for the fp16 value xh
 * (orchestration/include/number/lookup_table_impl/non-linear.h:42-47, 134-139);
 * key 0xFFFF is never written there and reads back 0. */
static inline float silu_h(uint16_t k) { if (k == 0xFFFF) { return 0.0f; } const float x = h2f(k); return x / (1.0f + expf(-x)); }
static inline float exp_h(uint16_t k)  { if (k == 0xFFFF) { return 0.0f; } return expf(h2f(k)); }

void oracle_tables(float *silu_table, float *exp_table) {
    for (uint32_t k = 0; k < 65536; ++k) {
        if (silu_table) { silu_table[k] = silu_h((uint16_t)k); }
        if (exp_table)  { exp_table[k]  = exp_h((uint16_t)k); }
    }
}

/* ---------------------------------------------------------------- Q8_0 activation quantizer */
/* Quantizator<FP32,Q8_0>::transform, backend/host/include/simd/vec_convert.h:178-261:
 * amax over 32 floats, d = amax/127 stored as fp16, id = 127/amax (0 if amax == 0),
 * q = round-half-even(x * id). */
void oracle_quantize_q8_0(const float *x, int64_t n, uint8_t *out) {
    const int64_t nb = n / 32;
    for (int64_t b = 0; b < nb; ++b) {
        const float *xb = x + b * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) { const float a = fabsf(xb[i]); if (a > amax) { amax = a; } }
        const float d  = amax / 127.0f;
        const float id = (amax != 0.0f) ? 127.0f / amax : 0.0f;
        uint8_t *ob = out + b * 34;
        const uint16_t dh = f2h(d);
        memcpy(ob, &dh, 2);
        for (int i = 0; i < 32; ++i) { ob[2 + i] = (uint8_t)(int8_t)(int32_t)nearbyintf(xb[i] * id); }
    }
}

/* Quantizator<FP32,FP16>::transform, vec_convert.h:39-65 (round to nearest even). */
void oracle_quantize_f16(const float *x, int64_t n, uint16_t *out) { for (int64_t i = 0; i < n; ++i) { out[i] = f2h(x[i]); } }

/* ---------------------------------------------------------------- block dot products */
/* hsum_float_8, backend/host/include/simd/vec_util.h:74-81:
 * ((a0+a4) + (a2+a6)) + ((a1+a5) + (a3+a7)). */
static inline float hsum8(const float a[8]) {
    const float r0 = a[4] + a[0], r1 = a[5] + a[1], r2 = a[6] + a[2], r3 = a[7] + a[3];
    const float s0 = r0 + r2, s1 = r1 + r3;
    return s0 + s1;
}

/* Integer lane sums of one Q4_0 x Q8_0 block: Dot<Q4_0,Q8_0>::exec, vec_dot.h:58-75 with
 * mul_sum_i8_pairs (vec_util.h:100-110). lanes[0..3] = high-nibble sums against y[16..31],
 * lanes[4..7] = low-nibble sums against y[0..15] (set_m128i(i32_0, i32_1) puts i32_1 low). */
static inline void lanes_q4_0(const uint8_t *wb, const uint8_t *xb, int32_t lanes[8]) {
    const uint8_t *qs = wb + 2;
    const int8_t  *y  = (const int8_t *)(xb + 2);
    for (int j = 0; j < 4; ++j) {
        int32_t lo = 0, hi = 0;
        for (int k = 4 * j; k < 4 * j + 4; ++k) {
            lo += ((int32_t)(qs[k] & 0xF) - 8) * (int32_t)y[k];
            hi += ((int32_t)(qs[k] >> 4) - 8) * (int32_t)y[16 + k];
        }
        lanes[j]     = hi;
        lanes[4 + j] = lo;
    }
}

int32_t oracle_blockdot_q4_0_q8_0(const uint8_t *wb, const uint8_t *xb) {
    int32_t l[8]; lanes_q4_0(wb, xb, l);
    int32_t s = 0; for (int i = 0; i < 8; ++i) { s += l[i]; }
    return s;
}

/* Dot<Q4_0,Q8_0>::exec, vec_dot.h:42-86: acc[lane] = fma(dw*dx, (float)lane_sum, acc[lane]). */
float oracle_dot_q4_0_q8_0(const uint8_t *w, const uint8_t *x, int64_t n) {
    float acc[8] = { 0 };
    const int64_t nb = n / 32;
    for (int64_t b = 0; b < nb; ++b) {
        const uint8_t *wb = w + b * 18, *xb = x + b * 34;
        uint16_t dw, dx; memcpy(&dw, wb, 2); memcpy(&dx, xb, 2);
        const float d = h2f(dw) * h2f(dx);
        int32_t l[8]; lanes_q4_0(wb, xb, l);
        for (int i = 0; i < 8; ++i) { acc[i] = fmaf(d, (float)l[i], acc[i]); }
    }
    return hsum8(acc);
}

/* Lane sums for Q8_0 x Q8_0: mul_sum_i8_pairs_float, vec_util.h:112-132 (lane i = products 4i..4i+3). */
static inline void lanes_q8_0(const uint8_t *wb, const uint8_t *xb, int32_t lanes[8]) {
    const int8_t *q = (const int8_t *)(wb + 2), *y = (const int8_t *)(xb + 2);
    for (int j = 0; j < 8; ++j) {
        int32_t s = 0;
        for (int k = 4 * j; k < 4 * j + 4; ++k) { s += (int32_t)q[k] * (int32_t)y[k]; }
        lanes[j] = s;
    }
}

int32_t oracle_blockdot_q8_0_q8_0(const uint8_t *wb, const uint8_t *xb) {
    int32_t l[8]; lanes_q8_0(wb, xb, l);
    int32_t s = 0; for (int i = 0; i < 8; ++i) { s += l[i]; }
    return s;
}

/* Dot<Q8_0,Q8_0>::exec, vec_dot.h:88-115. */
float oracle_dot_q8_0_q8_0(const uint8_t *w, const uint8_t *x, int64_t n) {
    float acc[8] = { 0 };
    const int64_t nb = n / 32;
    for (int64_t b = 0; b < nb; ++b) {
        const uint8_t *wb = w + b * 34, *xb = x + b * 34;
        uint16_t dw, dx; memcpy(&dw, wb, 2); memcpy(&dx, xb, 2);
        const float d = h2f(dw) * h2f(dx);
        int32_t l[8]; lanes_q8_0(wb, xb, l);
        for (int i = 0; i < 8; ++i) { acc[i] = fmaf(d, (float)l[i], acc[i]); }
    }
    return hsum8(acc);
}

/* Dot<FP16,FP16>::exec, vec_dot.h:117-146 with FP16::block_reduce (vec_util.h:61-71):
 * four 8-lane accumulators over 32-element steps while i + 32 < n; the rest (at least the
 * last 32 elements) goes through a scalar tail; result = tail + vector part. */
float oracle_dot_f16_f16(const uint16_t *a, const uint16_t *b, int64_t n) {
    float sum[4][8];
    memset(sum, 0, sizeof(sum));
    int64_t i = 0;
    for (; i + 32 < n; i += 32) {
        for (int j = 0; j < 4; ++j) {
            for (int l = 0; l < 8; ++l) { sum[j][l] = fmaf(h2f(a[i + 8 * j + l]), h2f(b[i + 8 * j + l]), sum[j][l]); }
        }
    }
    float x0[8];
    for (int l = 0; l < 8; ++l) { x0[l] = (sum[0][l] + sum[2][l]) + (sum[1][l] + sum[3][l]); }
    float t0[4];
    for (int l = 0; l < 4; ++l) { t0[l] = x0[l] + x0[4 + l]; }
    const float simd_res = (t0[0] + t0[1]) + (t0[2] + t0[3]);
    float tail = 0.0f;
    for (; i < n; ++i) { tail = fmaf(h2f(a[i]), h2f(b[i]), tail); }
    return tail + simd_res;
}

/* ---------------------------------------------------------------- K-quant decoding (layout only in the reference) */
static inline void scale_min_k4(int j, const uint8_t *s, uint8_t *sc, uint8_t *mn) {
    if (j < 4) { *sc = s[j] & 63; *mn = s[j + 4] & 63; }
    else { *sc = (uint8_t)((s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4)); *mn = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4)); }
}

/* One Q4_K super-block (144 B, 256 values) against 8 Q8_0 activation blocks.
 * value = d*sc*q - dmin*m per 32-element sub-block; parity unpinned. */
static float dot_q4_k_block(const uint8_t *wb, const uint8_t *xb, int32_t *isum_out) {
    uint16_t dh, mh; memcpy(&dh, wb, 2); memcpy(&mh, wb + 2, 2);
    const float d = h2f(dh), dmin = h2f(mh);
    const uint8_t *scales = wb + 4, *qs = wb + 16;
    float acc = 0.0f;
    for (int j = 0; j < 8; ++j) {
        uint8_t sc, mn; scale_min_k4(j, scales, &sc, &mn);
        const uint8_t *xj = xb + j * 34;
        uint16_t dxh; memcpy(&dxh, xj, 2);
        const float dx = h2f(dxh);
        const int8_t *y = (const int8_t *)(xj + 2);
        const uint8_t *q = qs + 32 * (j / 2);
        int32_t isum = 0, ysum = 0;
        for (int l = 0; l < 32; ++l) {
            const int32_t v = (j & 1) ? (q[l] >> 4) : (q[l] & 0xF);
            isum += v * (int32_t)y[l];
            ysum += (int32_t)y[l];
        }
        if (isum_out) { isum_out[j] = isum; }
        acc = fmaf(d * (float)sc * dx, (float)isum, acc);
        acc = fmaf(-(dmin * (float)mn * dx), (float)ysum, acc);
    }
    return acc;
}

float oracle_dot_q4_k_q8_0(const uint8_t *w, const uint8_t *x, int64_t n) {
    float acc = 0.0f;
    for (int64_t b = 0; b < n / 256; ++b) { acc += dot_q4_k_block(w + b * 144, x + b * 8 * 34, NULL); }
    return acc;
}

/* One Q6_K super-block (210 B) against 8 Q8_0 activation blocks; value = d*sc*q, q in -32..31,
 * one int8 scale per 16 values; parity unpinned. */
static float dot_q6_k_block(const uint8_t *wb, const uint8_t *xb) {
    const uint8_t *ql = wb, *qh = wb + 128;
    const int8_t *sc = (const int8_t *)(wb + 192);
    uint16_t dh; memcpy(&dh, wb + 208, 2);
    const float d = h2f(dh);
    int8_t q[256];
    for (int half = 0; half < 2; ++half) {
        for (int l = 0; l < 32; ++l) {
            const uint8_t h = qh[32 * half + l];
            q[128 * half + l]      = (int8_t)(((ql[64 * half + l] & 0xF)      | (((h >> 0) & 3) << 4)) - 32);
            q[128 * half + l + 32] = (int8_t)(((ql[64 * half + l + 32] & 0xF) | (((h >> 2) & 3) << 4)) - 32);
            q[128 * half + l + 64] = (int8_t)(((ql[64 * half + l] >> 4)       | (((h >> 4) & 3) << 4)) - 32);
            q[128 * half + l + 96] = (int8_t)(((ql[64 * half + l + 32] >> 4)  | (((h >> 6) & 3) << 4)) - 32);
        }
    }
    float acc = 0.0f;
    for (int g = 0; g < 16; ++g) {
        const uint8_t *xj = xb + (g / 2) * 34;
        uint16_t dxh; memcpy(&dxh, xj, 2);
        const int8_t *y = (const int8_t *)(xj + 2) + 16 * (g & 1);
        int32_t isum = 0;
        for (int l = 0; l < 16; ++l) { isum += (int32_t)q[16 * g + l] * (int32_t)y[l]; }
        acc = fmaf(d * (float)sc[g] * h2f(dxh), (float)isum, acc);
    }
    return acc;
}

float oracle_dot_q6_k_q8_0(const uint8_t *w, const uint8_t *x, int64_t n) {
    float acc = 0.0f;
    for (int64_t b = 0; b < n / 256; ++b) { acc += dot_q6_k_block(w + b * 210, x + b * 8 * 34); }
    return acc;
}

static int64_t row_bytes(int type, int64_t k) {
    switch (type) {
    case T_F32:  return k * 4;
    case T_F16:  return k * 2;
    case T_Q4_0: return k / 32 * 18;
    case T_Q8_0: return k / 32 * 34;
    case T_Q4_K: return k / 256 * 144;
    case T_Q6_K: return k / 256 * 210;
    default:     return -1;
    }
}

/* ---------------------------------------------------------------- MatMul */
/* OperatorMatMulImpl::execute, backend/host/operator/mat.cpp:71-146: for a quantized weight and
 * f32 activations every activation column is first quantized to Q8_0 (target_buffer_type,
 * mat.cpp:32-42), then dst[n, t] = Dot(W row n, Xq column t).
 * w: [n_out rows of k], x: [t columns of k] f32, out: [t][n_out] f32. xq (optional) receives the
 * Q8_0 activation blocks, t * k/32*34 bytes. */
int oracle_matmul(int wtype, const uint8_t *w, int64_t k, int64_t n_out, const float *x, int64_t t, float *out, uint8_t *xq_out) {
    const int64_t wrb = row_bytes(wtype, k);
    const int64_t xrb = k / 32 * 34;
    if (wrb < 0 || k % 32 != 0) { return 1; }
    if ((wtype == T_Q4_K || wtype == T_Q6_K) && k % 256 != 0) { return 1; }
    uint8_t *xq = xq_out ? xq_out : (uint8_t *)malloc((size_t)(t * xrb));
    if (!xq) { return 2; }
    for (int64_t c = 0; c < t; ++c) { oracle_quantize_q8_0(x + c * k, k, xq + c * xrb); }
    int rc = 0;
    for (int64_t c = 0; c < t; ++c) {
        for (int64_t r = 0; r < n_out; ++r) {
            const uint8_t *wr = w + r * wrb, *xc = xq + c * xrb;
            float v = 0.0f;
            switch (wtype) {
            case T_Q4_0: v = oracle_dot_q4_0_q8_0(wr, xc, k); break;
            case T_Q8_0: v = oracle_dot_q8_0_q8_0(wr, xc, k); break;
            case T_Q4_K: v = oracle_dot_q4_k_q8_0(wr, xc, k); break;
            case T_Q6_K: v = oracle_dot_q6_k_q8_0(wr, xc, k); break;
            default: rc = 1; break;
            }
            out[c * n_out + r] = v;
        }
    }
    if (!xq_out) { free(xq); }
    return rc;
}

/* ---------------------------------------------------------------- element-wise and norm ops */
/* std::reduce / std::transform_reduce on random-access iterators (libstdc++ <numeric>):
 * groups of four are combined as ((v0 + v1) + (v2 + v3)) and added to the running sum, the
 * remainder one by one. With the reference's build flags the compiler contracts
 * x0*x0 + x1*x1 into fma(x1, x1, x0*x0) (checked on wide-range inputs against that build). */
static float sum_of_squares(const float *x, int64_t n) {
    float init = 0.0f;
    int64_t i = 0;
    for (; n - i >= 4; i += 4) {
        const float v1 = fmaf(x[i + 1], x[i + 1], x[i] * x[i]);
        const float v2 = fmaf(x[i + 3], x[i + 3], x[i + 2] * x[i + 2]);
        init = init + (v1 + v2);
    }
    for (; i < n; ++i) { init = fmaf(x[i], x[i], init); }
    return init;
}

static float reduce_sum(const float *x, int64_t n) {
    float init = 0.0f;
    int64_t i = 0;
    for (; n - i >= 4; i += 4) { init = init + ((x[i] + x[i + 1]) + (x[i + 2] + x[i + 3])); }
    for (; i < n; ++i) { init = init + x[i]; }
    return init;
}

/* OperatorNormRMSImpl::execute, backend/host/operator/non-linear.cpp:194-223. */
void oracle_rmsnorm(const float *x, int64_t n, int64_t rows, float eps, float *out) {
    for (int64_t r = 0; r < rows; ++r) {
        const float *xr = x + r * n;
        const float sum   = sum_of_squares(xr, n);
        const float mean  = sum / (float)n;
        const float scale = 1.0f / sqrtf(mean + eps);
        for (int64_t i = 0; i < n; ++i) { out[r * n + i] = xr[i] * scale; }
    }
}

/* binary_execution<multiplies / plus>, backend/host/operator/basic.cpp:15-50, for a [n, rows] x [n] broadcast. */
void oracle_mul_rows(const float *x, const float *w, int64_t n, int64_t rows, float *out) {
    for (int64_t r = 0; r < rows; ++r) { for (int64_t i = 0; i < n; ++i) { out[r * n + i] = x[r * n + i] * w[i]; } }
}
void oracle_add(const float *a, const float *b, int64_t n, float *out) { for (int64_t i = 0; i < n; ++i) { out[i] = a[i] + b[i]; } }
void oracle_mul(const float *a, const float *b, int64_t n, float *out) { for (int64_t i = 0; i < n; ++i) { out[i] = a[i] * b[i]; } }

/* OperatorSiluImpl::execute, non-linear.cpp:57-77: table lookup on the fp16-rounded argument. */
void oracle_silu(const float *x, int64_t n, float *out) { for (int64_t i = 0; i < n; ++i) { out[i] = silu_h(f2h(x[i])); } }

/* operator_masked_softmax_execute, non-linear.cpp:129-180; mask row = n_ctx floats (0 or -inf). */
void oracle_softmax_masked(const float *scores, const float *mask, int64_t n, float scale, float *out) {
    for (int64_t i = 0; i < n; ++i) { out[i] = scores[i] + mask[i]; }
    for (int64_t i = 0; i < n; ++i) { out[i] *= scale; }
    float mx = out[0];
    for (int64_t i = 1; i < n; ++i) { if (mx < out[i]) { mx = out[i]; } }
    for (int64_t i = 0; i < n; ++i) { out[i] -= mx; }
    for (int64_t i = 0; i < n; ++i) { out[i] = (mask[i] == -INFINITY) ? 0.0f : exp_h(f2h(out[i])); }
    const float inv = 1.0f / reduce_sum(out, n);
    for (int64_t i = 0; i < n; ++i) { out[i] *= inv; }
}

/* OperatorRopeImpl::execute in mode Norm with the CLI defaults (ext_factor 0, freq_scale 1,
 * attn_factor 1), non-linear.cpp:247-260, 270-371: theta_0 = pos, theta_{k+1} = theta_k * theta_scale,
 * pair (x[2k], x[2k+1]) rotated by (cos, sin). x: [tokens][heads][hd] (hd innermost). */
void oracle_rope(const float *x, const int32_t *pos, int64_t hd, int64_t heads, int64_t tokens, float freq_base, float *out) {
    const float theta_scale = powf(freq_base, -2.0f / (float)hd);
    float *cache = (float *)malloc((size_t)hd * sizeof(float));
    for (int64_t t = 0; t < tokens; ++t) {
        float theta = (float)pos[t];
        for (int64_t i = 0; i < hd; i += 2) {
            cache[i]     = cosf(theta) * 1.0f;
            cache[i + 1] = sinf(theta) * 1.0f;
            theta *= theta_scale;
        }
        for (int64_t h = 0; h < heads; ++h) {
            const float *s = x + (t * heads + h) * hd;
            float *d = out + (t * heads + h) * hd;
            for (int64_t i = 0; i < hd; i += 2) {
                const float x0 = s[i], x1 = s[i + 1];
                d[i]     = x0 * cache[i] - x1 * cache[i + 1];
                d[i + 1] = x0 * cache[i + 1] + x1 * cache[i];
            }
        }
    }
    free(cache);
}

/* SamplerImpl<Greedy>::sample, model/include/llm/sampler/greedy.h:20-25: first maximum wins. */
int32_t oracle_argmax(const float *x, int64_t n) {
    int64_t best = 0;
    for (int64_t i = 1; i < n; ++i) { if (x[best] < x[i]) { best = i; } }
    return (int32_t)best;
}

/* ---------------------------------------------------------------- whole model */
typedef struct {
    int32_t n_layer, d_model, n_head, n_ff, n_vocab, n_ctx;
    float   rms_eps, rope_base;
    int32_t embd_type, output_type;
    const uint8_t *token_embd;      /* [n_vocab rows of d_model], F32 or Q8_0 */
    const float   *output_norm;
    const uint8_t *output;
    /* per-layer arrays of length n_layer */
    const float   **attn_norm, **ffn_norm;
    const uint8_t **wq, **wk, **wv, **wo, **w_up, **w_gate, **w_down;
    const int32_t *t_wq, *t_wk, *t_wv, *t_wo, *t_up, *t_gate, *t_down;
} oracle_model;

typedef struct {
    uint16_t *k_cache;   /* per layer: [n_ctx][d_model] f16            (attention.cpp:188-205) */
    uint16_t *v_cache;   /* per layer: [d_model][n_ctx] f16, transposed (attention.cpp:228-246) */
} oracle_state;

oracle_state *oracle_state_new(const oracle_model *m) {
    oracle_state *s = (oracle_state *)calloc(1, sizeof(*s));
    const size_t n = (size_t)m->n_layer * (size_t)m->n_ctx * (size_t)m->d_model;
    s->k_cache = (uint16_t *)calloc(n, 2);
    s->v_cache = (uint16_t *)calloc(n, 2);
    return s;
}
void oracle_state_free(oracle_state *s) { if (s) { free(s->k_cache); free(s->v_cache); free(s); } }

/* Optional debugging tap: when set, oracle_eval stores, for layer 0 and the last token of the call,
 * for the layer chosen with oracle_set_debug_layer: [q after rope (d) | attention output (d) | x after the attention residual (d) | up*silu(gate) (F) | x after the FFN residual (d)]. */
static float *g_debug_tap = NULL;
static int g_debug_layer = 0;
void oracle_set_debug_tap(float *buf) { g_debug_tap = buf; }
void oracle_set_debug_layer(int layer) { g_debug_layer = layer; }
/* second tap: residual stream after the chosen layer, then that layer's attention output, then Q after RoPE, for every token of the call ([t][d] each) */
static float *g_debug_x = NULL;
void oracle_set_debug_x(float *buf) { g_debug_x = buf; }

/* One execution of the graph LLAMAModel::build_graph emits (model/src/llm/model/llama.cpp:123-222,
 * plugin/attention.cpp:267-302, plugin/ffn.cpp:5-42, plugin/inout.cpp:5-78) for `t` tokens at
 * positions n_past .. n_past+t-1. logits: [t][n_vocab]. Optional taps (may be NULL):
 *   tap_xq   Q8_0 blocks of the first layer's attention-norm output, token 0 (d_model/32*34 bytes)
 */
int oracle_eval(const oracle_model *m, oracle_state *st, const int32_t *tokens, int32_t t, int32_t n_past, float *logits, uint8_t *tap_xq) {
    const int64_t d = m->d_model, H = m->n_head, hd = d / H, F = m->n_ff, V = m->n_vocab, C = m->n_ctx;
    const int64_t n_kv = n_past + t;
    if (n_kv > C) { return 1; }
    float *x    = (float *)malloc((size_t)(t * d) * 4);
    float *xn   = (float *)malloc((size_t)(t * d) * 4);
    float *q    = (float *)malloc((size_t)(t * d) * 4);
    float *k    = (float *)malloc((size_t)(t * d) * 4);
    float *v    = (float *)malloc((size_t)(t * d) * 4);
    float *att  = (float *)malloc((size_t)(t * d) * 4);
    float *tmp  = (float *)malloc((size_t)(t * d) * 4);
    float *up   = (float *)malloc((size_t)(t * F) * 4);
    float *gate = (float *)malloc((size_t)(t * F) * 4);
    float *sc   = (float *)malloc((size_t)n_kv * 4);
    float *pr   = (float *)malloc((size_t)n_kv * 4);
    float *mask = (float *)malloc((size_t)C * 4);
    uint16_t *qh = (uint16_t *)malloc((size_t)hd * 2);
    uint16_t *ph = (uint16_t *)malloc((size_t)n_kv * 2);
    int32_t *pos = (int32_t *)malloc((size_t)t * 4);
    for (int32_t i = 0; i < t; ++i) { pos[i] = n_past + i; }
    const float scale = 1.0f / sqrtf((float)hd);
    int rc = 0;

    /* GetRow: OperatorGetRowImpl::execute, backend/host/operator/view.cpp:33-81 (memcpy, or Q8_0 -> F32) */
    for (int32_t i = 0; i < t; ++i) {
        if (m->embd_type == T_F32) { memcpy(x + i * d, m->token_embd + (size_t)tokens[i] * d * 4, (size_t)d * 4); }
        else if (m->embd_type == T_Q8_0) {
            const uint8_t *row = m->token_embd + (size_t)tokens[i] * (d / 32 * 34);
            for (int64_t b = 0; b < d / 32; ++b) {
                uint16_t dh; memcpy(&dh, row + b * 34, 2);
                const float dd = h2f(dh);
                for (int l = 0; l < 32; ++l) { x[i * d + b * 32 + l] = (float)(int8_t)row[b * 34 + 2 + l] * dd; }
            }
        } else if (m->embd_type == T_Q4_K) {   /* no reference arithmetic: (d * sc) * q - dmin * m, every operation a separate f32 one */
            const uint8_t *row = m->token_embd + (size_t)tokens[i] * (d / 256 * 144);
            for (int64_t b = 0; b < d / 256; ++b) {
                const uint8_t *s = row + b * 144;
                uint16_t dh, mh; memcpy(&dh, s, 2); memcpy(&mh, s + 2, 2);
                const float dd = h2f(dh), dmin = h2f(mh);
                for (int j = 0; j < 8; ++j) {
                    uint8_t sc, mn; scale_min_k4(j, s + 4, &sc, &mn);
                    const float d1 = dd * (float)sc, m1 = dmin * (float)mn;
                    for (int l = 0; l < 32; ++l) {
                        const uint8_t qb = s[16 + 32 * (j / 2) + l];
                        const float q = (float)((j & 1) ? (qb >> 4) : (qb & 0xF));
                        const float prod = d1 * q;
                        x[i * d + b * 256 + j * 32 + l] = prod - m1;
                    }
                }
            }
        } else if (m->embd_type == T_Q6_K) {   /* q * (d * sc) */
            const uint8_t *row = m->token_embd + (size_t)tokens[i] * (d / 256 * 210);
            for (int64_t b = 0; b < d / 256; ++b) {
                const uint8_t *s = row + b * 210;
                uint16_t dh; memcpy(&dh, s + 208, 2);
                const float dd = h2f(dh);
                for (int e = 0; e < 256; ++e) {
                    const int hf = e >> 7, seg = (e >> 5) & 3, l = e & 31;
                    const uint8_t lo = s[64 * hf + 32 * (seg & 1) + l], h = s[128 + 32 * hf + l];
                    const int q = (((seg & 2) ? (lo >> 4) : (lo & 0xF)) | (((h >> (2 * seg)) & 3) << 4)) - 32;
                    const float ds = dd * (float)(int8_t)s[192 + (e >> 4)];
                    x[i * d + b * 256 + e] = (float)q * ds;
                }
            }
        } else { rc = 3; goto done; }
    }

    for (int32_t L = 0; L < m->n_layer; ++L) {
        uint16_t *kc = st->k_cache + (size_t)L * C * d;
        uint16_t *vc = st->v_cache + (size_t)L * C * d;
        oracle_rmsnorm(x, d, t, m->rms_eps, tmp);
        oracle_mul_rows(tmp, m->attn_norm[L], d, t, xn);
        if (L == 0 && tap_xq) { oracle_quantize_q8_0(xn, d, tap_xq); }   /* token 0 only */
        rc |= oracle_matmul(m->t_wq[L], m->wq[L], d, d, xn, t, q, NULL);
        rc |= oracle_matmul(m->t_wk[L], m->wk[L], d, d, xn, t, k, NULL);
        rc |= oracle_matmul(m->t_wv[L], m->wv[L], d, d, xn, t, v, NULL);
        if (rc) { goto done; }
        oracle_rope(q, pos, hd, H, t, m->rope_base, q);
        oracle_rope(k, pos, hd, H, t, m->rope_base, k);
        /* KV append, f32 -> f16 RNE: dup_execute, view.cpp:83-227 */
        for (int32_t i = 0; i < t; ++i) {
            for (int64_t e = 0; e < d; ++e) {
                kc[(size_t)(n_past + i) * d + e] = f2h(k[i * d + e]);
                vc[(size_t)e * C + (n_past + i)] = f2h(v[i * d + e]);
            }
        }
        for (int32_t i = 0; i < t; ++i) {
            /* KQ mask row: llama.cpp:248-257 */
            for (int64_t j = 0; j < C; ++j) { mask[j] = (j <= n_past + i) ? 0.0f : -INFINITY; }
            for (int64_t h = 0; h < H; ++h) {
                /* scores = K (f16) . Q rounded to f16: mat.cpp target_buffer_type F16 path */
                oracle_quantize_f16(q + i * d + h * hd, hd, qh);
                for (int64_t j = 0; j < n_kv; ++j) { sc[j] = oracle_dot_f16_f16(kc + (size_t)j * d + h * hd, qh, hd); }
                oracle_softmax_masked(sc, mask, n_kv, scale, pr);
                oracle_quantize_f16(pr, n_kv, ph);
                for (int64_t e = 0; e < hd; ++e) { att[i * d + h * hd + e] = oracle_dot_f16_f16(vc + (size_t)(h * hd + e) * C, ph, n_kv); }
            }
        }
        rc |= oracle_matmul(m->t_wo[L], m->wo[L], d, d, att, t, tmp, NULL);
        oracle_add(tmp, x, t * d, x);                       /* ffn_input = attn_out + x, llama.cpp:194-197 */
        if (g_debug_tap && L == g_debug_layer) {
            memcpy(g_debug_tap, q + (t - 1) * d, (size_t)d * 4);
            memcpy(g_debug_tap + d, att + (t - 1) * d, (size_t)d * 4);
            memcpy(g_debug_tap + 2 * d, x + (t - 1) * d, (size_t)d * 4);
        }
        oracle_rmsnorm(x, d, t, m->rms_eps, tmp);
        oracle_mul_rows(tmp, m->ffn_norm[L], d, t, xn);
        rc |= oracle_matmul(m->t_up[L], m->w_up[L], d, F, xn, t, up, NULL);
        rc |= oracle_matmul(m->t_gate[L], m->w_gate[L], d, F, xn, t, gate, NULL);
        oracle_silu(gate, t * F, gate);
        oracle_mul(up, gate, t * F, up);                    /* ffn_par = up * silu(gate), ffn.cpp:32-35 */
        rc |= oracle_matmul(m->t_down[L], m->w_down[L], F, d, up, t, tmp, NULL);
        if (g_debug_tap && L == g_debug_layer) { memcpy(g_debug_tap + 3 * d, up + (t - 1) * F, (size_t)F * 4); }
        oracle_add(x, tmp, t * d, x);                       /* llama.cpp:206-211 */
        if (g_debug_tap && L == g_debug_layer) { memcpy(g_debug_tap + 3 * d + F, x + (t - 1) * d, (size_t)d * 4); }
        if (g_debug_x && L == g_debug_layer) { memcpy(g_debug_x, x, (size_t)t * d * 4); memcpy(g_debug_x + (size_t)t * d, att, (size_t)t * d * 4); memcpy(g_debug_x + (size_t)2 * t * d, q, (size_t)t * d * 4); }
        if (rc) { goto done; }
    }
    oracle_rmsnorm(x, d, t, m->rms_eps, tmp);
    oracle_mul_rows(tmp, m->output_norm, d, t, xn);
    rc |= oracle_matmul(m->output_type, m->output, d, V, xn, t, logits, NULL);
done:
    free(x); free(xn); free(q); free(k); free(v); free(att); free(tmp); free(up); free(gate);
    free(sc); free(pr); free(mask); free(qh); free(ph); free(pos);
    return rc;
}
