// One single-token step of the LLaMa graph (every layer and the output head) as ONE persistent kernel.
//
// The graph is the one LLAMAModel::build_graph emits (model/src/llm/model/llama.cpp:123-222, plugin/attention.cpp:267-302,
// plugin/ffn.cpp:5-42, plugin/inout.cpp:61-75); per layer it runs as five phases with a grid-wide barrier in front of
// each (every phase needs all outputs of the one before):
//   1  NormRMS + Mul(attn_norm) + Q8_0 quantize -> Wq|Wk|Wv mat-vec -> RoPE(Q, K) + f16 KV append
//   2  attention of one head on up to four CTAs (scores and softmax redundantly, PV split by output elements);
//      the CTA quantizes its 32 outputs to a Q8_0 block straight away
//   3  (pre-quantized input) Wo mat-vec -> + residual
//   4  NormRMS + Mul(ffn_norm) + quantize -> Wup|Wgate mat-vec -> up * silu(gate)
//   5  quantize -> Wdown mat-vec -> + residual
// and finally NormRMS + Mul(output_norm) + quantize -> output mat-vec -> logits.
//
// Why one kernel: a decode step streams every weight byte once (HBM-bound), but between two mat-vecs there are a few
// microseconds in which nothing can be computed (barrier, RMSNorm's serial sum, quantization, attention). With one
// launch per mat-vec the copy engines idle through those gaps, because the next kernel's CTAs only get their shared
// memory when the previous kernel's CTAs have left. Here ONE ring of bulk-copy stages per SM is fed by a dedicated
// warp that walks the CTA's whole weight schedule of the step (all phases, all layers) and is held back only by ring
// space - weights are constants, so the copies run ahead of the phase that will use them. The fifteen consumer warps
// take the stages of their tiles in schedule order (a tile walks along K on one warp, as the CPU's accumulation
// order demands), signal each stage empty, and meet at the phase barriers.
//
// Arithmetic: identical to the per-matrix kernels (spyb_matvec.cu: fragment-ordered records, one mma.sync per block
// for the integer group sums, block-order f32 FMA chains, hsum_float_8 tree), so the results are the CPU backend's bits.
// Every wait is bounded (barriers, stage barriers); on expiry the CTA raises the abort word, the copies in flight are
// awaited with a bound, and the kernel returns.

#include <algorithm>

#include "spyb_common.cuh"
#include "spyb_kernels.h"
#include "spyb_mma.cuh"

#include <math_constants.h>

namespace spyb {

constexpr int ST_WARPS     = 15;                  // consumer warps (with the copy-issuing warp: 512 threads, 128 registers each)
constexpr int ST_CONSUMERS = ST_WARPS * WARP;     // 480
constexpr int ST_THREADS   = ST_CONSUMERS + WARP; // + the warp that issues the bulk copies
constexpr int ST_HD        = 128;

__device__ __forceinline__ void bar_consumers() { asm volatile("bar.sync 1, %0;" ::"n"(ST_CONSUMERS) : "memory"); }
__device__ __forceinline__ void mbar_arrive_plain(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }

struct StepShared {           // static shared memory of the kernel
    int      abort;           // a bounded wait ran out somewhere: stop
    float    scale;           // RMSNorm scale of the phase
    float    red[ST_WARPS];
    float    bcast;
};

__device__ __forceinline__ void step_raise_abort(const StepParams &p, StepShared *sh, int code) {
    *reinterpret_cast<volatile int *>(&sh->abort) = 1;
    atomicExch(p.sync + 2, 1ull);
    if (p.error_flag != nullptr) { atomicExch(p.error_flag, code); }
}

// Grid-wide barrier of the consumer warps: a monotonic arrival counter in global memory (cleared by the host before
// the launch); `target` = arrivals expected so far. Returns false when the step was aborted.
__device__ __noinline__ bool step_grid_sync(const StepParams &p, StepShared *sh, unsigned long long target) {
    bar_consumers();
    if (threadIdx.x == 0 && *reinterpret_cast<volatile int *>(&sh->abort) == 0) {
        __threadfence();
        atomicAdd(p.sync, 1ull);
        const uint64_t t0 = global_timer_ns();
        unsigned spins = 0;
        for (;;) {
            unsigned long long v;
            asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p.sync) : "memory");
            if (v >= target) { break; }
            if ((++spins & 63u) == 0u) {
                unsigned long long a;
                asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(a) : "l"(p.sync + 2) : "memory");
                if (a != 0ull || global_timer_ns() - t0 > p.wait_limit_ns) { step_raise_abort(p, sh, 2); break; }
            }
        }
    }
    bar_consumers();
    return *reinterpret_cast<volatile int *>(&sh->abort) == 0;
}

__device__ __forceinline__ const StepMat &step_mat(const StepParams &p, int ph) {
    if (ph >= 4 * p.n_layer) { return p.head; }
    const StepLayer &ly = p.layers[ph >> 2];
    switch (ph & 3) { case 0: return ly.qkv; case 1: return ly.wo; case 2: return ly.upgate; default: return ly.down; }
}

// ------------------------------------------------------------------------------------------ the copy-issuing warp
// Walks the CTA's weight schedule: for every phase, the CTA's tiles in rounds of fifteen (one per consumer warp),
// chunk by chunk; item i goes to ring stage i % NS once the consumer of item i - NS has released it.
// Before a stage is armed for item i, seq[stage] = i is published: a consumer only waits on a stage's barrier once it
// sees its own item number there, so it can never mistake an earlier phase of the barrier for its own.
__device__ __noinline__ void step_producer(const StepParams &p, StepShared *sh, uint32_t ring_s, uint32_t full_s, uint32_t empty_s, volatile uint32_t *seq, int NS) {
    const int G = gridDim.x, c = blockIdx.x;
    int slot = 0; uint32_t wrap = 0, it = 0;
    bool stop = false;
    const int n_ph = 4 * p.n_layer + 1;
    for (int ph = 0; ph < n_ph && !stop; ++ph) {
        const StepMat M = step_mat(p, ph);
        const int lo = (int)((int64_t)M.n_tiles * c / G), hi = (int)((int64_t)M.n_tiles * (c + 1) / G);
        const size_t tile_bytes = (size_t)M.nrec * M.recb;
        for (int r0 = lo; r0 < hi && !stop; r0 += ST_WARPS) {
            const int ntr = min(ST_WARPS, hi - r0);
            for (int ch = 0; ch < M.nch && !stop; ++ch) {
                const uint32_t bytes = (uint32_t)min(M.crecs, M.nrec - ch * M.crecs) * M.recb;
                const uint8_t *src = M.w + (size_t)r0 * tile_bytes + (size_t)ch * M.crecs * M.recb;
                for (int j = 0; j < ntr; ++j, src += tile_bytes) {
                    if (wrap > 0 && !mbar_wait_bounded(empty_s + slot * 8, (wrap - 1) & 1u, p.wait_limit_ns)) { step_raise_abort(p, sh, 1); stop = true; break; }
                    if (*reinterpret_cast<volatile int *>(&sh->abort) != 0) { stop = true; break; }
                    const uint32_t bar = full_s + slot * 8;
                    mbar_expect_tx(bar, bytes);
                    seq[slot] = it++;
                    bulk_copy_g2s(ring_s + (uint32_t)slot * ST_STAGE_BYTES, src, bytes, bar);
                    if (++slot == NS) { slot = 0; ++wrap; }
                }
            }
        }
    }
    if (stop) {   // give the copies in flight a bounded chance to land (they target this CTA's shared memory)
        for (int s = 0; s < NS; ++s) {
            const bool issued_this_wrap = s < slot;
            if (!issued_this_wrap && wrap == 0) { continue; }
            const uint32_t idx = issued_this_wrap ? wrap : wrap - 1;
            mbar_wait_bounded(full_s + s * 8, idx & 1u, 10000000ull);
        }
    }
}

// ------------------------------------------------------------------------------------------ prologues
struct StepPlanes { uint32_t *Yw; float *DS; };

// Y[g][w][i]: word w (values 4w..4w+3) of block 4g+i; DS[b]: the block's fp16-rounded scale as f32 (/16 for Q4_0 weights)
__device__ __forceinline__ void step_store_q(const StepPlanes &a, int g4, uint32_t q, uint16_t dh, int wtype) {
    const int b = g4 >> 3, w = g4 & 7;
    a.Yw[(((b >> 2)) * 8 + w) * 4 + (b & 3)] = q;
    if (w == 0) { const float d = h2f(dh); a.DS[b] = (wtype == 2) ? __fmul_rn(d, 0.0625f) : d; }
}

__device__ __forceinline__ float step_running_sum(const float *v3, int n4) {
    // std::transform_reduce's running sum (backend/host/operator/non-linear.cpp:216): one chain of dependent f32 adds
    const float4 *g4 = reinterpret_cast<const float4 *>(v3);
    float sum = 0.f;
    int g = 0;
    if (n4 >= 16) {
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

// NormRMS (non-linear.cpp:194-223) + Mul(norm weight) (basic.cpp:15-50) + Quantizator<FP32,Q8_0> (vec_convert.h:178-261)
// of the residual stream x[k]; k <= 4 * ST_NORM_GROUPS * 512. The sum-of-squares partials alias the Y plane.
constexpr int ST_NORM_GROUPS = 4;
__device__ __noinline__ void step_prologue_norm(const StepParams &p, StepShared *sh, const StepPlanes &a, const float *x, const float *norm_w, int k, int nbp, int wtype) {
    const int tid = threadIdx.x;
    const int n4 = k >> 2, n4p = nbp * 8;
    float *v3 = reinterpret_cast<float *>(a.Yw);
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    const float4 *w4 = reinterpret_cast<const float4 *>(norm_w);
    float4 xv[ST_NORM_GROUPS], wv[ST_NORM_GROUPS];
#pragma unroll
    for (int i = 0; i < ST_NORM_GROUPS; ++i) {
        const int g = tid + i * ST_CONSUMERS;
        xv[i] = (g < n4) ? __ldcg(x4 + g) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < ST_NORM_GROUPS; ++i) {
        const int g = tid + i * ST_CONSUMERS;
        wv[i] = (g < n4) ? w4[g] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < ST_NORM_GROUPS; ++i) {
        const int g = tid + i * ST_CONSUMERS;
        if (g < n4) {
            const float4 v = xv[i];
            const float v1 = fmaf(v.y, v.y, __fmul_rn(v.x, v.x));
            const float v2 = fmaf(v.w, v.w, __fmul_rn(v.z, v.z));
            v3[g] = __fadd_rn(v1, v2);
        }
    }
    bar_consumers();
    if (tid == 0) {
        const float sum  = step_running_sum(v3, n4);
        const float mean = __fdiv_rn(sum, (float)k);
        sh->scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, p.eps)));
    }
    bar_consumers();   // also: the partials (aliasing Y) are dead from here on
    const float scale = sh->scale;
#pragma unroll
    for (int i = 0; i < ST_NORM_GROUPS; ++i) {
        if (i * ST_CONSUMERS < n4p) {   // uniform over the CTA: the quantizer's shuffles see full warps
            const int g = tid + i * ST_CONSUMERS;
            float4 v = xv[i];
            v.x = __fmul_rn(__fmul_rn(v.x, scale), wv[i].x); v.y = __fmul_rn(__fmul_rn(v.y, scale), wv[i].y);
            v.z = __fmul_rn(__fmul_rn(v.z, scale), wv[i].z); v.w = __fmul_rn(__fmul_rn(v.w, scale), wv[i].w);
            uint16_t dh; int s;
            const uint32_t q = quantize_q8_lane4(v, dh, s);
            if (g < n4p) { step_store_q(a, g, q, dh, wtype); }
        }
    }
}

// Quantizator<FP32,Q8_0> of a plain activation vector (FFN down's input)
__device__ __noinline__ void step_prologue_quant(const StepPlanes &a, const float *x, int k, int nbp, int wtype) {
    const int tid = threadIdx.x;
    const int n4 = k >> 2, n4p = nbp * 8;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    for (int base = 0; base < n4p; base += 4 * ST_CONSUMERS) {
        float4 xv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int g = base + tid + i * ST_CONSUMERS;
            xv[i] = (g < n4) ? __ldcg(x4 + g) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (base + i * ST_CONSUMERS < n4p) {
                const int g = base + tid + i * ST_CONSUMERS;
                uint16_t dh; int s;
                const uint32_t q = quantize_q8_lane4(xv[i], dh, s);
                if (g < n4p) { step_store_q(a, g, q, dh, wtype); }
            }
        }
    }
}

// Input that its producer already quantized (attention output): int8 values [k] and one f32 scale per block
__device__ __noinline__ void step_prologue_preq(const StepPlanes &a, const int8_t *xq, const float *xd, int k, int nbp, int wtype) {
    const int tid = threadIdx.x;
    const int nw = k >> 2, nwp = nbp * 8;
    const uint32_t *x32 = reinterpret_cast<const uint32_t *>(xq);
    for (int g = tid; g < nwp; g += ST_CONSUMERS) {
        const uint32_t q = (g < nw) ? __ldcg(x32 + g) : 0u;
        const int b = g >> 3, w = g & 7;
        a.Yw[(((b >> 2)) * 8 + w) * 4 + (b & 3)] = q;
        if (w == 0) { const float d = (g < nw) ? __ldcg(xd + b) : 0.f; a.DS[b] = (wtype == 2) ? __fmul_rn(d, 0.0625f) : d; }
    }
}

// ------------------------------------------------------------------------------------------ mat-vec phase
enum StepEpi { SE_QKV = 0, SE_RESID = 1, SE_SILU = 2, SE_LOGITS = 3 };

struct StepRing { uint32_t ring_s, full_s, empty_s; volatile uint32_t *seq; int NS; uint32_t items; };   // items: stages this CTA has consumed so far

__device__ __forceinline__ void step_epilogue(const StepParams &p, const StepLayer *ly, int epi, int row, float v, float partner, bool writer) {
    switch (epi) {
    case SE_RESID:    // Add(attn_out, x) / Add(ffn_inp, ffn_out): model/src/llm/model/llama.cpp:194-211
        if (writer) { p.x[row] = __fadd_rn(v, __ldcg(p.x + row)); }
        break;
    case SE_LOGITS:
        if (writer) { p.logits[row] = v; }
        break;
    case SE_QKV: {
        if (!writer) { break; }
        const int sec = row / p.d, e = row - sec * p.d;
        const int pos = p.pos[0];
        if (sec == 2) {   // V: f32 -> f16 RNE into the transposed cache (dup_execute, backend/host/operator/view.cpp:163-191)
            ly->v_cache[(int64_t)e * p.n_ctx + pos] = __float2half_rn(v);
        } else {          // RoPE, mode Norm: backend/host/operator/non-linear.cpp:270-371 (rows 2i, 2i+1 rotate together)
            const float2 cs = p.rope[(int64_t)pos * (ST_HD >> 1) + ((e % ST_HD) >> 1)];
            const float x0 = (e & 1) ? partner : v, x1 = (e & 1) ? v : partner;
            const float r = (e & 1) ? __fadd_rn(__fmul_rn(x0, cs.y), __fmul_rn(x1, cs.x)) : __fsub_rn(__fmul_rn(x0, cs.x), __fmul_rn(x1, cs.y));
            __half *dst = (sec == 0) ? p.q + e : ly->k_cache + (int64_t)pos * p.d + e;
            *dst = __float2half_rn(r);
        }
    } break;
    default: break;
    }
}

// A warp that gives up on a wait raises the abort word and skips its remaining tiles; every warp still reaches the
// next barrier of the consumer warps, where the step ends for the whole CTA.
template <int WT, int TR>
__device__ __noinline__ void step_matvec(const StepParams &p, StepShared *sh, const StepMat &M, const StepLayer *ly, int epi, const StepPlanes &planes, StepRing &R) {
    constexpr int NA = MmaTile<WT, TR>::NA;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, q = lane & 3;
    const int G = gridDim.x, c = blockIdx.x;
    const int lo = (int)((int64_t)M.n_tiles * c / G), hi = (int)((int64_t)M.n_tiles * (c + 1) / G);
    const MmaLane  ML = mma_lane<WT, TR>(lane);
    const uint32_t y_s = smem_u32(planes.Yw), ds_s = smem_u32(planes.DS);
    bool ok = true;

    for (int r0 = lo; r0 < hi; r0 += ST_WARPS) {
        const int ntr = min(ST_WARPS, hi - r0);
        if (warp < ntr && ok) {
            float acc[1][NA];
#pragma unroll
            for (int a = 0; a < NA; ++a) { acc[0][a] = 0.f; }
            uint32_t ya = y_s, da = ds_s;
            for (int ch = 0; ch < M.nch; ++ch) {
                const uint32_t it = R.items + (uint32_t)(ch * ntr + warp);
                const uint32_t slot = it % (uint32_t)R.NS, par = (it / (uint32_t)R.NS) & 1u;
                bool got = true;
                if (R.seq[slot] != it) {   // the stage still belongs to an earlier item: wait until it is armed for this one
                    const uint64_t t0 = global_timer_ns();
                    while (R.seq[slot] != it) {
                        __nanosleep(64);
                        if (global_timer_ns() - t0 > p.wait_limit_ns) { got = false; break; }
                    }
                }
                got = got && mbar_wait_bounded(R.full_s + slot * 8, par, p.wait_limit_ns);
                if (__any_sync(0xffffffffu, !got)) { ok = false; break; }
                mma_records<WT, TR, 1>(R.ring_s + slot * ST_STAGE_BYTES, min(M.crecs, M.nrec - ch * M.crecs), ya, da, 0u, 0u, ML, acc);
                __syncwarp();                                         // every lane is done reading the stage
                if (lane == 0) { mbar_arrive_plain(R.empty_s + slot * 8); }   // hand it back to the copy-issuing warp
            }
            if (ok) {   // tile finished: hsum_float_8 tree ((a0+a4)+(a2+a6))+((a1+a5)+(a3+a7)), then the epilogue
                float h[2] = {0.f, 0.f};
#pragma unroll
                for (int r = 0; r < NA / 2; ++r) { h[r] = mma_row_sum(acc[0][2 * r], acc[0][2 * r + 1]); }
                const int  tile = r0 + warp;
                const bool wr = (q == 0);
                if (epi == SE_SILU) {   // up * silu(gate): model/src/llm/plugin/ffn.cpp:28-35; rows 0..TR/2-1 of a tile are up rows, the rest the matching gate rows
                    if (TR == 16) { if (wr) { p.act[8 * tile + g] = __fmul_rn(h[0], p.silu_table[f2h(h[1])]); } }
                    else { const float gate = __shfl_down_sync(0xffffffffu, h[0], 16); if (wr && g < 4) { p.act[4 * tile + g] = __fmul_rn(h[0], p.silu_table[f2h(gate)]); } }
                } else {
#pragma unroll
                    for (int r = 0; r < NA / 2; ++r) {
                        const float partner = __shfl_xor_sync(0xffffffffu, h[r], 4);
                        step_epilogue(p, ly, epi, TR * tile + 8 * r + g, h[r], partner, wr);
                    }
                }
            }
        }
        R.items += (uint32_t)(M.nch * ntr);
    }
    if (!ok && lane == 0) { step_raise_abort(p, sh, 1); }
}

__device__ __noinline__ void step_matvec_any(const StepParams &p, StepShared *sh, const StepMat &Mg, const StepLayer *ly, int epi, const StepPlanes &planes, StepRing &R) {
    const StepMat M = Mg;
    if (M.type == 2) { if (M.tr == 16) { step_matvec<2, 16>(p, sh, M, ly, epi, planes, R); } else { step_matvec<2, 8>(p, sh, M, ly, epi, planes, R); } }
    else             { if (M.tr == 16) { step_matvec<8, 16>(p, sh, M, ly, epi, planes, R); } else { step_matvec<8, 8>(p, sh, M, ly, epi, planes, R); } }
}

// ------------------------------------------------------------------------------------------ attention phase
__device__ __forceinline__ void step_unpack8(const uint4 v, float f[8]) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&v.x)), b = __half22float2(*reinterpret_cast<const __half2 *>(&v.y));
    const float2 c = __half22float2(*reinterpret_cast<const __half2 *>(&v.z)), d = __half22float2(*reinterpret_cast<const __half2 *>(&v.w));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 ldcg_u4(const uint4 *p) { return __ldcg(p); }
__device__ __forceinline__ float ldcg_h(const __half *p) { return __half2float(__ushort_as_half(__ldcg(reinterpret_cast<const unsigned short *>(p)))); }

// MatMul(K, Q) -> masked Softmax -> MatMul(V, probs) of one head for the step's token
// (MultiHeadAttentionBlock::attention_projection, model/src/llm/plugin/attention.cpp:102-132) in the CPU's arithmetic:
// Dot<FP16,FP16> (backend/host/include/simd/vec_dot.h:117-146) with its 4 x 8 accumulators, scalar tail and reduction
// tree; softmax through the fp16-argument exp table with std::reduce's grouping (non-linear.cpp:129-180).
// Work item = (head, part): the part's CTA computes all scores and the softmax of the head (cheap, KBs) and the PV
// products of output elements [part * ne, (part + 1) * ne), ne = 128 / parts, then quantizes them to Q8_0 blocks
// (Quantizator<FP32,Q8_0>, vec_convert.h:178-261: what Wo's MatMul does to its input first).
__device__ __noinline__ void step_attention(const StepParams &p, StepShared *sh, const StepLayer *ly, float *scratch) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int parts = p.att_parts, ne = ST_HD / parts;
    const int pos = p.pos[0];
    const int n_vis = pos + 1;
    const int n_tot = (p.pos[1] > n_vis) ? p.pos[1] : n_vis;
    const int n_pad = (p.n_ctx + 3) & ~3;
    float *qf = scratch;              // [128]
    float *outv = qf + ST_HD;         // [128]
    float *sc = outv + ST_HD;         // [n_pad]
    float *gs = sc + n_pad;           // [n_pad / 4]
    const int n_main = ((n_tot - 1) / 32) * 32;
    constexpr int NE_MAX = (ST_HD + ST_WARPS - 1) / ST_WARPS;   // elements per warp when one CTA takes the whole head
    constexpr int NE_PRE = 3;                  // elements per warp (all of them with four parts per head) ...
    constexpr int PV_PRE = 4;                  // ... whose first PV steps and tail are requested before the scores

#pragma unroll 1
    for (int item = blockIdx.x; item < p.n_head * parts; item += gridDim.x) {
        const int h = item / parts, part = item - h * parts;
        const int e0 = part * ne;
        // the part's output elements go round the warps: warp w takes e0 + w, e0 + w + 15, ...
        // ---- requests first: Q, this thread's K row, and the first PV steps of this warp's elements
        const float q_mine = (tid < ST_HD) ? ldcg_h(p.q + h * ST_HD + tid) : 0.f;
        uint4 kv[16];
        {
            const uint4 *krow = reinterpret_cast<const uint4 *>(ly->k_cache + (int64_t)min(tid, n_vis - 1) * p.d + h * ST_HD);
#pragma unroll
            for (int a = 0; a < 16; ++a) { kv[a] = ldcg_u4(krow + a); }
        }
        float v_pre[NE_PRE][PV_PRE], v_tail[NE_PRE];
#pragma unroll
        for (int k = 0; k < NE_PRE; ++k) {
            const int  el = warp + k * ST_WARPS;
            const bool mine = el < ne;
            const __half *vrow = ly->v_cache + ((int64_t)h * ST_HD + e0 + (mine ? el : 0)) * p.n_ctx;
#pragma unroll
            for (int s = 0; s < PV_PRE; ++s) {
                const int j = 32 * s + lane;
                v_pre[k][s] = (mine && 32 * s < n_main && j < n_vis) ? ldcg_h(vrow + j) : 0.f;
            }
            v_tail[k] = (mine && n_main + lane < n_vis) ? ldcg_h(vrow + n_main + lane) : 0.f;
        }
        if (tid < ST_HD) { qf[tid] = q_mine; }
        bar_consumers();

        // ---- scores of the visible positions: one thread per position, all 32 accumulators in its registers
#pragma unroll 1
        for (int j = tid; j < n_vis; j += ST_CONSUMERS) {
            const float4 *q4 = reinterpret_cast<const float4 *>(qf);
            if (j != tid) {
                const uint4 *krow = reinterpret_cast<const uint4 *>(ly->k_cache + (int64_t)j * p.d + h * ST_HD);
#pragma unroll
                for (int a = 0; a < 16; ++a) { kv[a] = ldcg_u4(krow + a); }
            }
            float acc[4][8];
#pragma unroll
            for (int a = 0; a < 4; ++a) {
#pragma unroll
                for (int e = 0; e < 8; ++e) { acc[a][e] = 0.f; }
            }
#pragma unroll
            for (int step = 0; step < 3; ++step) {       // elements 0..95: accumulator a takes elements 32 * step + 8a .. + 7
#pragma unroll
                for (int a = 0; a < 4; ++a) {
                    float kf[8]; step_unpack8(kv[4 * step + a], kf);
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
                float kf[8]; step_unpack8(kv[12 + a], kf);
                const float4 qa = q4[(12 + a) * 2], qb = q4[(12 + a) * 2 + 1];
                const float  qv[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
                for (int e = 0; e < 8; ++e) { tail = fmaf(kf[e], qv[e], tail); }
            }
            sc[j] = __fadd_rn(tail, simd);
        }
        bar_consumers();

        // ---- masked softmax: (score + mask) * scale, subtract the maximum, table exp, std::reduce, multiply by 1/sum
        float m = -CUDART_INF_F;
#pragma unroll 1
        for (int j = tid; j < n_vis; j += ST_CONSUMERS) {
            const float v = __fmul_rn(__fadd_rn(sc[j], 0.0f), p.att_scale);
            sc[j] = v;
            m = fmaxf(m, v);
        }
        m = warp_max(m);
        if (lane == 0) { sh->red[warp] = m; }
        bar_consumers();
        m = sh->red[0];
#pragma unroll
        for (int w = 1; w < ST_WARPS; ++w) { m = fmaxf(m, sh->red[w]); }
        const int n_tot4 = (n_tot + 3) & ~3;
#pragma unroll 1
        for (int j = tid; j < n_tot4; j += ST_CONSUMERS) { sc[j] = (j < n_vis) ? p.exp_table[f2h(__fsub_rn(sc[j], m))] : 0.f; }
        bar_consumers();
#pragma unroll 1
        for (int g = tid; g < (n_tot >> 2); g += ST_CONSUMERS) {
            const float4 v = reinterpret_cast<const float4 *>(sc)[g];
            gs[g] = __fadd_rn(__fadd_rn(v.x, v.y), __fadd_rn(v.z, v.w));
        }
        bar_consumers();
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
            sh->bcast = __fdiv_rn(1.0f, sum);
        }
        bar_consumers();
        const float inv = sh->bcast;
        // probabilities, rounded to fp16 as the PV MatMul does with its f32 operand
#pragma unroll 1
        for (int j = tid; j < n_vis; j += ST_CONSUMERS) { sc[j] = __half2float(__float2half_rn(__fmul_rn(sc[j], inv))); }
        bar_consumers();

        // ---- out[e] = Dot<FP16,FP16>(V_t[e][0..n_tot), probs): a warp per element, lane = 8 * accumulator + element of
        // the CPU's 4 x 8 accumulators (position j of a 32-step goes to lane j % 32); masked positions have probability +0
        // and leave every accumulator unchanged, so they are skipped
#pragma unroll
        for (int k = 0; k < NE_PRE; ++k) {
            const int el = warp + k * ST_WARPS;
            if (el < ne) {
                const __half *vrow = ly->v_cache + ((int64_t)h * ST_HD + e0 + el) * p.n_ctx;
                float acc = 0.f;
#pragma unroll
                for (int s = 0; s < PV_PRE; ++s) {
                    const int j = 32 * s + lane;
                    if (32 * s < n_main && j < n_vis) { acc = fmaf(v_pre[k][s], sc[j], acc); }
                }
#pragma unroll 1
                for (int j0 = 32 * PV_PRE; j0 < n_main; j0 += 32) {
                    const int j = j0 + lane;
                    if (j < n_vis) { acc = fmaf(ldcg_h(vrow + j), sc[j], acc); }
                }
                acc = reduce_f16dot_lanes(acc);
                float tail = 0.f;                         // positions n_main .. n_tot-1 (at most 32): scalar chain
#pragma unroll 1
                for (int i = 0; i < 32; ++i) {
                    const float v = __shfl_sync(0xffffffffu, v_tail[k], i);
                    if (n_main + i < n_vis) { tail = fmaf(v, sc[n_main + i], tail); }
                }
                if (lane == 0) { outv[el] = __fadd_rn(tail, acc); }
            }
        }
#pragma unroll 1
        for (int k = NE_PRE; k < NE_MAX; ++k) {           // fewer than four parts per head: the remaining elements, loads in the loop
            const int el = warp + k * ST_WARPS;
            if (el < ne) {
                const __half *vrow = ly->v_cache + ((int64_t)h * ST_HD + e0 + el) * p.n_ctx;
                float acc = 0.f;
#pragma unroll 2
                for (int j0 = 0; j0 < n_main; j0 += 32) {
                    const int j = j0 + lane;
                    if (j < n_vis) { acc = fmaf(ldcg_h(vrow + j), sc[j], acc); }
                }
                acc = reduce_f16dot_lanes(acc);
                const float vt = (n_main + lane < n_vis) ? ldcg_h(vrow + n_main + lane) : 0.f;
                float tail = 0.f;
#pragma unroll 1
                for (int i = 0; i < 32; ++i) {
                    const float v = __shfl_sync(0xffffffffu, vt, i);
                    if (n_main + i < n_vis) { tail = fmaf(v, sc[n_main + i], tail); }
                }
                if (lane == 0) { outv[el] = __fadd_rn(tail, acc); }
            }
        }
        bar_consumers();
        // ---- Q8_0 blocks of this part's outputs
        if (warp < ne / 32) {
            const float x = outv[warp * 32 + lane];
            const float amax = warp_max(fabsf(x));
            const float d  = __fdiv_rn(amax, 127.0f);
            const float id = (amax != 0.0f) ? __fdiv_rn(127.0f, amax) : 0.0f;
            const int   qv = __float2int_rn(__fmul_rn(x, id));
            const int   o  = h * ST_HD + e0 + warp * 32;
            p.att_q[o + lane] = (int8_t)qv;
            if (lane == 0) { p.att_d[o >> 5] = h2f(f2h(d)); }
        }
        bar_consumers();   // the scratch is reused by the next item / phase
    }
}

// reference-layout copy of the quantized activations (34-byte blocks) for parity taps
__device__ __noinline__ void step_tap(const StepParams &p, const StepPlanes &a, int nb, int wtype) {
#pragma unroll 1
    for (int b = threadIdx.x; b < nb; b += ST_CONSUMERS) {
        volatile uint8_t *o = p.tap_xq + (size_t)b * 34;
#pragma unroll 1
        for (int w = 0; w < 8; ++w) {
            const uint32_t v = a.Yw[((b >> 2) * 8 + w) * 4 + (b & 3)];
            o[2 + 4 * w] = (uint8_t)v; o[3 + 4 * w] = (uint8_t)(v >> 8); o[4 + 4 * w] = (uint8_t)(v >> 16); o[5 + 4 * w] = (uint8_t)(v >> 24);
        }
        *reinterpret_cast<volatile uint16_t *>(p.tap_xq + (size_t)b * 34) = f2h((wtype == 2) ? __fmul_rn(a.DS[b], 16.0f) : a.DS[b]);
    }
}

__device__ __forceinline__ void step_stamp(const StepParams &p, int idx) {
    if (p.stamps != nullptr && threadIdx.x == 0) {
        const unsigned long long t = global_timer_ns();
        if (blockIdx.x == 0) { p.stamps[2 * idx] = t; }
        atomicMax(p.stamps + 2 * idx + 1, t);
    }
}

// ------------------------------------------------------------------------------------------ the kernel
__global__ void __launch_bounds__(ST_THREADS, 1) step_kernel(const StepParams p, const int NS, const int act_bytes) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ StepShared sh;
    // dynamic shared memory: [activation planes / attention scratch: act_bytes][full barriers][empty barriers][item numbers][ring: NS stages]
    const uint32_t full_s  = smem_u32(smem_raw + act_bytes);
    const uint32_t empty_s = full_s + NS * 8;
    volatile uint32_t *seq = reinterpret_cast<volatile uint32_t *>(smem_raw + act_bytes + NS * 16);
    const uint32_t ring_off = ((uint32_t)act_bytes + (uint32_t)NS * 20 + 127u) & ~127u;
    const uint32_t ring_s  = smem_u32(smem_raw + ring_off);
    const int tid = threadIdx.x;

    if (tid == 0) {
        sh.abort = 0;
        for (int s = 0; s < NS; ++s) { mbar_init(full_s + s * 8, 1); mbar_init(empty_s + s * 8, 1); seq[s] = 0xffffffffu; }
        mbar_init_fence();
    }
    __syncthreads();

    if (tid >= ST_CONSUMERS) {   // the copy-issuing warp: one thread walks the schedule, the others have nothing to do
        if (tid == ST_CONSUMERS) { step_producer(p, &sh, ring_s, full_s, empty_s, seq, NS); }
        return;
    }

    StepRing R; R.ring_s = ring_s; R.full_s = full_s; R.empty_s = empty_s; R.seq = seq; R.NS = NS; R.items = 0;
    StepPlanes planes;
    planes.Yw = reinterpret_cast<uint32_t *>(smem_raw);
    planes.DS = reinterpret_cast<float *>(smem_raw + (size_t)p.nbp_max * 32);
    float *scratch = reinterpret_cast<float *>(smem_raw);
    const unsigned long long G = gridDim.x + (unsigned)p.barrier_extra;
    unsigned long long arrivals = 0;
    int st = 0;
    step_stamp(p, st++);

    // One loop over the step's mat-vec phases (4 per layer: Wq|Wk|Wv, Wo, up|gate, down; then the head) keeps a single
    // copy of every routine in the instruction cache. The residual stream of layer 0 was written before the launch.
    const int n_ph = 4 * p.n_layer + 1;
    for (int ph = 0; ph < n_ph; ++ph) {
        const int kind = (ph == n_ph - 1) ? 4 : (ph & 3);
        const StepLayer *ly = (kind == 4) ? nullptr : p.layers + (ph >> 2);
        if (ph > 0) { arrivals += G; if (!step_grid_sync(p, &sh, arrivals)) { return; } }
        step_stamp(p, st++);
        if (kind == 1) {   // attention sits between the Wq|Wk|Wv phase and the Wo phase
            step_attention(p, &sh, ly, scratch);
            step_stamp(p, st++);
            arrivals += G; if (!step_grid_sync(p, &sh, arrivals)) { return; }
            step_stamp(p, st++);
        }
        const StepMat &M = (kind == 4) ? p.head : (kind == 0) ? ly->qkv : (kind == 1) ? ly->wo : (kind == 2) ? ly->upgate : ly->down;
        const int nbp = M.nbp, wtype = M.type;
        switch (kind) {
        case 1:  step_prologue_preq(planes, p.att_q, p.att_d, p.d, nbp, wtype); break;
        case 3:  step_prologue_quant(planes, p.act, p.fl, nbp, wtype); break;
        default: step_prologue_norm(p, &sh, planes, p.x, (kind == 4) ? p.output_norm : (kind == 0) ? ly->attn_norm : ly->ffn_norm, p.d, nbp, wtype); break;
        }
        bar_consumers();
        if (ph == 0 && p.tap_xq != nullptr && blockIdx.x == 0) { step_tap(p, planes, p.d / 32, wtype); }
        step_stamp(p, st++);
        step_matvec_any(p, &sh, M, ly, (kind == 4) ? SE_LOGITS : (kind == 0) ? SE_QKV : (kind == 2) ? SE_SILU : SE_RESID, planes, R);
        step_stamp(p, st++);
    }
}

// ------------------------------------------------------------------------------------------ host side
size_t step_act_bytes(const StepParams &p) {
    const size_t planes = (size_t)p.nbp_max * 36;
    const size_t n_pad = ((size_t)p.n_ctx + 3) & ~(size_t)3;
    const size_t att = (2 * ST_HD + n_pad + n_pad / 4 + 16) * sizeof(float);
    return (std::max(planes, att) + 127) / 128 * 128;
}

int step_ring_stages(const StepParams &p, size_t smem_limit) {
    const size_t act = step_act_bytes(p);
    const size_t fixed = act + 128 + 1024;   // alignment slack and the kernel's static shared memory
    if (smem_limit <= fixed) { return 0; }
    int ns = (int)((smem_limit - fixed) / (ST_STAGE_BYTES + 20));
    return std::min(ns, 64);
}

// can `grid` CTAs of the step kernel with a ring of `ns` stages be resident at once on the current device?
cudaError_t step_resident_ctas(const StepParams &p, int ns, int *ctas_per_sm) {
    const size_t act = step_act_bytes(p);
    const size_t smem = ((act + (size_t)ns * 20 + 127) & ~(size_t)127) + (size_t)ns * ST_STAGE_BYTES;
    cudaError_t err = allow_dynamic_smem(reinterpret_cast<const void *>(step_kernel), smem);
    if (err != cudaSuccess) { return err; }
    return cudaOccupancyMaxActiveBlocksPerMultiprocessor(ctas_per_sm, step_kernel, ST_THREADS, smem);
}

cudaError_t launch_step(const StepParams &p, int grid, int ns, bool cooperative, cudaStream_t stream) {
    if (ns <= ST_WARPS || grid < 1 || p.d > 4 * ST_NORM_GROUPS * ST_CONSUMERS || (p.d & 127) || (p.fl & 31)) { return cudaErrorInvalidValue; }
    const size_t act = step_act_bytes(p);
    const size_t smem = ((act + (size_t)ns * 20 + 127) & ~(size_t)127) + (size_t)ns * ST_STAGE_BYTES;
    cudaError_t err = allow_dynamic_smem(reinterpret_cast<const void *>(step_kernel), smem);
    if (err != cudaSuccess) { return err; }
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)grid); lc.blockDim = dim3(ST_THREADS); lc.dynamicSmemBytes = smem; lc.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    lc.attrs = attr; lc.numAttrs = cooperative ? 1 : 0;
    return cudaLaunchKernelEx(&lc, step_kernel, p, ns, (int)act);
}

}  // namespace spyb
