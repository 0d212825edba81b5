// Pieces shared by the mat-vec kernels of every weight format: the RMSNorm running sum and the fused epilogues.
#pragma once

#include "spyb_common.cuh"
#include "spyb_kernels.h"

namespace spyb {

// the RMSNorm running sum: one thread's chain of dependent f32 additions, in the CPU's order
__device__ __forceinline__ float running_sum_serial(const float *v3, int n4) {
    const float4 *g4 = reinterpret_cast<const float4 *>(v3);
    float sum = 0.f;
    int g = 0;
    if (n4 >= 16) {   // the 128-bit reads run one step (16 values) ahead of the dependent adds
        float4 q0 = g4[0], q1 = g4[1], q2 = g4[2], q3 = g4[3];
        for (g = 16; g + 16 <= n4; g += 16) {
            const float4 n0 = g4[(g >> 2)], n1 = g4[(g >> 2) + 1], n2 = g4[(g >> 2) + 2], n3 = g4[(g >> 2) + 3];
            sum = __fadd_rn(sum, q0.x); sum = __fadd_rn(sum, q0.y); sum = __fadd_rn(sum, q0.z); sum = __fadd_rn(sum, q0.w);
            sum = __fadd_rn(sum, q1.x); sum = __fadd_rn(sum, q1.y); sum = __fadd_rn(sum, q1.z); sum = __fadd_rn(sum, q1.w);
            sum = __fadd_rn(sum, q2.x); sum = __fadd_rn(sum, q2.y); sum = __fadd_rn(sum, q2.z); sum = __fadd_rn(sum, q2.w);
            sum = __fadd_rn(sum, q3.x); sum = __fadd_rn(sum, q3.y); sum = __fadd_rn(sum, q3.z); sum = __fadd_rn(sum, q3.w);
            q0 = n0; q1 = n1; q2 = n2; q3 = n3;
        }
        sum = __fadd_rn(sum, q0.x); sum = __fadd_rn(sum, q0.y); sum = __fadd_rn(sum, q0.z); sum = __fadd_rn(sum, q0.w);
        sum = __fadd_rn(sum, q1.x); sum = __fadd_rn(sum, q1.y); sum = __fadd_rn(sum, q1.z); sum = __fadd_rn(sum, q1.w);
        sum = __fadd_rn(sum, q2.x); sum = __fadd_rn(sum, q2.y); sum = __fadd_rn(sum, q2.z); sum = __fadd_rn(sum, q2.w);
        sum = __fadd_rn(sum, q3.x); sum = __fadd_rn(sum, q3.y); sum = __fadd_rn(sum, q3.z); sum = __fadd_rn(sum, q3.w);
    }
    for (; g < n4; ++g) { sum = __fadd_rn(sum, v3[g]); }
    return sum;
}
// ---------------------------------------------------------------------------------------------
// epilogue for one finished dot product `v` (identical on the 8 lanes of its row) of row `row`, column t.
// `partner` is the value of the neighbouring row (row ^ 1), needed by RoPE. Called by all lanes; lane l == 0 writes.
__device__ __forceinline__ void matvec_epilogue(const MatvecParams &p, int64_t row, int t, float v, float partner, bool writer) {
    switch (p.epi) {
    case EPI_STORE:
        if (writer) { p.out[(int64_t)t * p.out_stride + row] = v; }
        break;
    case EPI_RESID:   // Add(attn_out, x) / Add(ffn_inp, ffn_out): model/src/llm/model/llama.cpp:194-211
        if (writer) { const int64_t i = (int64_t)t * p.out_stride + row; p.out[i] = __fadd_rn(v, p.resid[i]); }
        break;
    case EPI_QKV_ROPE: {
        if (!writer) { break; }
        const int sec = (int)(row / p.dl);
        const int e   = (int)(row - (int64_t)sec * p.dl);
        const int pos = *p.pos_base + (p.seq_stride ? 0 : t);          // a batch in lockstep: every column at the same position,
        const int64_t seq_off = p.seq_stride ? (int64_t)t * p.seq_stride : 0;   // each in its own cache
        if (sec == 2) {   // V: f32 -> f16 RNE into the transposed cache [dl][n_ctx] (dup_execute, backend/host/operator/view.cpp:163-191)
            p.v_cache[seq_off + (int64_t)e * p.n_ctx + pos] = __float2half_rn(v);
        } else {          // RoPE, mode Norm: backend/host/operator/non-linear.cpp:270-371 (rows 2i, 2i+1 rotate together)
            const float2 cs = p.rope_table[(int64_t)pos * (p.hd >> 1) + ((e % p.hd) >> 1)];
            const float x0 = (e & 1) ? partner : v, x1 = (e & 1) ? v : partner;
            const float a = (e & 1) ? __fadd_rn(__fmul_rn(x0, cs.y), __fmul_rn(x1, cs.x))
                                    : __fsub_rn(__fmul_rn(x0, cs.x), __fmul_rn(x1, cs.y));
            __half *dst = (sec == 0) ? p.q_out + (int64_t)t * p.dl + e : p.k_cache + seq_off + (int64_t)pos * p.dl + e;
            *dst = __float2half_rn(a);
        }
    } break;
    default: break;
    }
}

// up * silu(gate): model/src/llm/plugin/ffn.cpp:28-35; silu = table on the fp16-rounded argument
__device__ __forceinline__ void matvec_epilogue_silu(const MatvecParams &p, int64_t row, int t, float up, float gate, bool writer) {
    if (writer) { p.out[(int64_t)t * p.out_stride + row] = __fmul_rn(up, p.silu_table[f2h(gate)]); }
}

}  // namespace spyb
