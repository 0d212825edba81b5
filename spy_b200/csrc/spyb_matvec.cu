// Dequant-fused mat-vec for sm_100a, bit-exact with the reference's CPU arithmetic.
//
// Reference semantics: OperatorMatMulImpl::execute (backend/host/operator/mat.cpp:71-146) quantizes every
// f32 activation column to Q8_0 and takes Dot<Q4_0,Q8_0> / Dot<Q8_0,Q8_0>
// (backend/host/include/simd/vec_dot.h:42-115) per output: eight f32 accumulators, one per group of four
// products, each updated block after block with acc = fma(d_w * d_x, (float)lane_sum, acc), and a fixed
// reduction tree at the end. Because the network re-quantizes its activations at every layer, any
// difference in f32 summation order is amplified to percent-level logit differences within a few layers,
// so this kernel reproduces that order exactly, by giving every one of the CPU's accumulators to one lane:
//   lane = (row r of 4, accumulator l of 8); a warp owns R tiles of 4 rows and walks them along K. Per group
//   of four blocks a lane reads ONE 128-bit word per row (its own 4 bytes of each of the 4 blocks - the
//   weights are stored word-transposed for this), selects its nibbles, takes four byte dot products against
//   the Q8_0 activations in shared memory and folds them into its accumulator with four FMAs in block order.
//   No intra-warp synchronisation in the arithmetic; the eight lanes of a row meet once per row in the
//   reduction tree.
// The small neighbouring operators of the LLaMa layer are folded into the prologue (RMSNorm + weight +
// Q8_0 quantization, in the CPU's summation order) and the epilogue (residual add, SiLU-gate-mul,
// RoPE + KV append).
//
// Roofline: HBM-bound. Algorithmic bytes per launch = rows * K/32 * 18 (Q4_0) or 34 (Q8_0); activations
// and outputs are a few KB and stay in L2. The weights of a tile are one contiguous run in HBM; every warp
// streams its tiles through a private ring in shared memory with bulk asynchronous copies
// (cp.async.bulk, completion on mbarriers), issued before the kernel waits for its predecessor: tens of KB
// per SM are in flight without holding registers, the copies are long sequential runs (DRAM-page friendly),
// and they keep HBM busy through the serial prologue and across kernel boundaries.

#include <algorithm>
#include <map>
#include <mutex>

#include "spyb_common.cuh"
#include "spyb_kernels.h"
#include "spyb_mma.cuh"
#include "spyb_tp.cuh"
#include "spyb_mv_common.cuh"

namespace spyb {

constexpr int MV_THREADS = 512;
constexpr int MV_WARPS   = MV_THREADS / WARP;

constexpr int MAX_STAGES = 16;              // ring stages per warp (mbarriers per warp)

// shared memory: per column t, per group g of four blocks
//   Y [t][g][w][i]  (w = 0..7, i = 0..3)  word w of the 32 int8 values of block 4g+i (w 0..3 = values 0..15)
//   DS[t][b]        f32 of the fp16-rounded scale; divided by 16 (exact) for Q4_0 weights, whose lane sums come
//                   scaled by 16
// The sum-of-squares partials of the RMSNorm prologue alias Y (they are dead before Y is written).
struct ActPlanes {
    uint4  *Y;
    float4 *DS;
};
__host__ __device__ static inline size_t act_plane_bytes(int nbp, int TM) { return (size_t)TM * nbp * (32 + 4); }
__device__ __forceinline__ ActPlanes act_planes(void *base, int nbp, int TM) {
    ActPlanes a;
    a.Y  = reinterpret_cast<uint4 *>(base);
    a.DS = reinterpret_cast<float4 *>(a.Y + (size_t)TM * nbp * 2);
    return a;
}

struct MatvecSmem { size_t act, bars, ring, total; };
__host__ __device__ static inline MatvecSmem matvec_smem_layout(int nbp, int TM, size_t ring_bytes) {
    MatvecSmem m;
    m.act  = 0;
    m.bars = (act_plane_bytes(nbp, TM) + 15) / 16 * 16;
    m.ring = (m.bars + (size_t)MV_WARPS * MAX_STAGES * 8 + 127) / 128 * 128;
    m.total = m.ring + ring_bytes;
    return m;
}

size_t matvec_smem_bytes(int nb, int T) { return matvec_smem_layout(padded_blocks(nb), T, 0).total; }

// cudaFuncAttributeMaxDynamicSharedMemorySize is a property of (device, kernel): the largest size allowed so far is kept
// per pair, so that a process driving several devices raises the limit on each of them.
SmemLedger::Decision SmemLedger::decide(int device, const void *kernel, size_t bytes) {
    std::lock_guard<std::mutex> g(mutex_);
    size_t &have = allowed_[std::make_pair(device, kernel)];
    if (have == 0) { have = 48 * 1024; }
    if (bytes <= have) { return KEEP; }
    have = bytes;
    return RAISE;
}
void SmemLedger::forget(int device, const void *kernel) {
    std::lock_guard<std::mutex> g(mutex_);
    allowed_.erase(std::make_pair(device, kernel));
}
// host-only check of the ledger's rules (no device needed): 0 when they hold
int smem_ledger_selftest() {
    SmemLedger l;
    const int k1 = 1, k2 = 2;
    if (l.decide(0, &k1, 40 * 1024) != SmemLedger::KEEP) { return 1; }       // below the default limit: nothing to do
    if (l.decide(0, &k1, 100 * 1024) != SmemLedger::RAISE) { return 2; }     // first large launch on device 0
    if (l.decide(0, &k1, 90 * 1024) != SmemLedger::KEEP) { return 3; }       // already allowed
    if (l.decide(1, &k1, 100 * 1024) != SmemLedger::RAISE) { return 4; }     // the same kernel on another device: its own mark
    if (l.decide(0, &k2, 100 * 1024) != SmemLedger::RAISE) { return 5; }     // another kernel on device 0: its own mark
    if (l.decide(0, &k1, 160 * 1024) != SmemLedger::RAISE) { return 6; }
    l.forget(0, &k1);                                                        // a failed cudaFuncSetAttribute: back to the default
    if (l.decide(0, &k1, 100 * 1024) != SmemLedger::RAISE) { return 7; }
    return 0;
}

cudaError_t allow_dynamic_smem(const void *kernel, size_t bytes) {
    static SmemLedger ledger;
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) { return err; }
    if (ledger.decide(device, kernel, bytes) == SmemLedger::KEEP) { return cudaSuccess; }
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (err != cudaSuccess) { ledger.forget(device, kernel); }
    return err;
}

// ---------------------------------------------------------------------------------------------
// prologue: f32 activations -> Q8_0 columns in shared memory (optionally through RMSNorm * weight)
//   NormRMS (backend/host/operator/non-linear.cpp:194-223): sum of squares by std::transform_reduce, whose
//   order for random-access ranges is: groups of four combined as (x0^2 + x1^2) + (x2^2 + x3^2) (the first
//   product of each pair plain, the second fused into an FMA, as the CPU build evaluates it) and added to
//   the running sum one group after the other; y = x * (1 / sqrt(sum/n + eps)). The groups are formed in
//   parallel, the running sum is one thread's chain. Mul (basic.cpp:15-50): y * norm_weight.
// Single column, K <= 12288: every thread keeps its (at most PG) float4 groups of x in registers from the one
// global read through the sum of squares to the quantizer; same arithmetic as the general prologue below.
constexpr int PRO_GROUPS = 6;
template <int PG, bool NORM>
__device__ __forceinline__ void matvec_prologue_1col(const MatvecParams &p, ActPlanes act, float *v3, float *scales) {
    const int tid = threadIdx.x;
    const int nbp = p.A.nbp;
    const int n4  = (int)(p.A.k >> 2);
    const int n4p = nbp * 8;                                   // float4 groups including the zero padding up to nbp blocks
    const int npass = (n4p + MV_THREADS - 1) / MV_THREADS;     // <= PG
    const float4 *x4 = reinterpret_cast<const float4 *>(p.x);
    float4 xv[PG];
    // (activations are read past L1: under tensor parallelism other GPUs wrote part of them)
#pragma unroll
    for (int k = 0; k < PG; ++k) {
        const int g = tid + k * MV_THREADS;
        xv[k] = (k < npass && g < n4) ? __ldcg(x4 + g) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (NORM) {
        const float4 *w4 = reinterpret_cast<const float4 *>(p.norm_w);
#pragma unroll
        for (int k = 0; k < PG; ++k) {
            const int g = tid + k * MV_THREADS;
            if (k < npass && g < n4) {
                const float4 v = xv[k];
                const float v1 = fmaf(v.y, v.y, __fmul_rn(v.x, v.x));
                const float v2 = fmaf(v.w, v.w, __fmul_rn(v.z, v.z));
                v3[g] = __fadd_rn(v1, v2);
            }
        }
        // the norm weights arrive while the sum of squares is formed
        float4 wv[PG];
#pragma unroll
        for (int k = 0; k < PG; ++k) {
            const int g = tid + k * MV_THREADS;
            wv[k] = (k < npass && g < n4) ? w4[g] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        __syncthreads();
        const float sum = (tid == 0) ? running_sum_serial(v3, n4) : 0.f;
        if (tid == 0) {
            const float mean = __fdiv_rn(sum, (float)p.A.k);
            scales[0] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, p.eps)));
        }
        __syncthreads();   // also: the partials (aliasing Y) are dead from here on
        const float scale = scales[0];
#pragma unroll
        for (int k = 0; k < PG; ++k) {
            xv[k].x = __fmul_rn(__fmul_rn(xv[k].x, scale), wv[k].x);
            xv[k].y = __fmul_rn(__fmul_rn(xv[k].y, scale), wv[k].y);
            xv[k].z = __fmul_rn(__fmul_rn(xv[k].z, scale), wv[k].z);
            xv[k].w = __fmul_rn(__fmul_rn(xv[k].w, scale), wv[k].w);
        }
    }
    uint32_t *Yw = reinterpret_cast<uint32_t *>(act.Y);
    float    *DS = reinterpret_cast<float *>(act.DS);
#pragma unroll
    for (int k = 0; k < PG; ++k) {
        if (k < npass) {   // uniform over the CTA: the quantizer's shuffles see full warps
            const int g = tid + k * MV_THREADS;
            uint16_t dh; int sum;
            const uint32_t q = quantize_q8_lane4(xv[k], dh, sum);
            if (g < n4p) {
                const int b = g >> 3, w = g & 7;
                Yw[(((b >> 2)) * 8 + w) * 4 + (b & 3)] = q;
                if (w == 0) { const float d = h2f(dh); DS[b] = (p.A.type == 2) ? __fmul_rn(d, 0.0625f) : d; }
            }
        }
    }
}

template <int TM>
__device__ __forceinline__ void matvec_prologue(const MatvecParams &p, ActPlanes act, float *v3, float *scales) {
    const int     tid = threadIdx.x;
    const int64_t K   = p.A.k;
    const int     nb = p.A.nb, nbp = p.A.nbp;
    const int     n4  = (int)(K >> 2);
    if (p.pro == PRO_NORM_QUANT) {
        for (int t = 0; t < p.T; ++t) {
            const float4 *x4 = reinterpret_cast<const float4 *>(p.x + (int64_t)t * p.x_stride);
            for (int g = tid; g < n4; g += MV_THREADS) {
                const float4 v = __ldcg(x4 + g);
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
            for (; g + 16 <= n4; g += 16) {   // four 128-bit reads ahead of their 16 dependent adds
                const float4 q0 = g4[(g >> 2)], q1 = g4[(g >> 2) + 1], q2 = g4[(g >> 2) + 2], q3 = g4[(g >> 2) + 3];
                sum = __fadd_rn(sum, q0.x); sum = __fadd_rn(sum, q0.y); sum = __fadd_rn(sum, q0.z); sum = __fadd_rn(sum, q0.w);
                sum = __fadd_rn(sum, q1.x); sum = __fadd_rn(sum, q1.y); sum = __fadd_rn(sum, q1.z); sum = __fadd_rn(sum, q1.w);
                sum = __fadd_rn(sum, q2.x); sum = __fadd_rn(sum, q2.y); sum = __fadd_rn(sum, q2.z); sum = __fadd_rn(sum, q2.w);
                sum = __fadd_rn(sum, q3.x); sum = __fadd_rn(sum, q3.y); sum = __fadd_rn(sum, q3.z); sum = __fadd_rn(sum, q3.w);
            }
            for (; g < n4; ++g) { sum = __fadd_rn(sum, v3[tid * n4 + g]); }
            const float mean = __fdiv_rn(sum, (float)K);
            scales[tid] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, p.eps)));
        }
        __syncthreads();   // also: the partials (aliasing Y) are dead from here on
    }
    uint32_t *Yw = reinterpret_cast<uint32_t *>(act.Y);
    float    *DS = reinterpret_cast<float *>(act.DS);
    const int n4p = nbp * 8;   // float4 groups including the zero padding up to nbp blocks
#pragma unroll 1
    for (int t = 0; t < TM; ++t) {
        const bool    col  = t < p.T;    // unused columns are zeros with zero scales: every contribution vanishes
        const float4 *x4 = reinterpret_cast<const float4 *>(p.x + (int64_t)(col ? t : 0) * p.x_stride);
        const float4 *w4 = reinterpret_cast<const float4 *>(p.norm_w);
        const float scale = (col && p.pro == PRO_NORM_QUANT) ? scales[t] : 1.f;
        for (int base = 0; base < n4p; base += MV_THREADS) {
            const int  g     = base + tid;
            const bool valid = col && g < n4;
            float4 v = valid ? __ldcg(x4 + g) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (p.pro == PRO_NORM_QUANT && valid) {
                const float4 w = w4[g];
                v.x = __fmul_rn(__fmul_rn(v.x, scale), w.x);
                v.y = __fmul_rn(__fmul_rn(v.y, scale), w.y);
                v.z = __fmul_rn(__fmul_rn(v.z, scale), w.z);
                v.w = __fmul_rn(__fmul_rn(v.w, scale), w.w);
            }
            uint16_t dh; int s;
            const uint32_t q = quantize_q8_lane4(v, dh, s);
            if (g < n4p) {
                const int b = g >> 3, w = g & 7;
                const int idx = ((t * (nbp >> 2) + (b >> 2)) * 8 + w) * 4 + (b & 3);
                Yw[idx] = q;
                if (w == 0) { const float d = h2f(dh); DS[t * nbp + b] = (p.A.type == 2) ? __fmul_rn(d, 0.0625f) : d; }
            }
        }
    }
    (void)nb;
}

// reference-layout copy of column 0 (34-byte blocks) for parity taps
__device__ __forceinline__ void matvec_tap(const MatvecParams &p, ActPlanes act) {
    if (p.tap_xq == nullptr || blockIdx.x != 0) { return; }
    const uint32_t *Yw = reinterpret_cast<const uint32_t *>(act.Y);
    const float    *DS = reinterpret_cast<const float *>(act.DS);
    for (int b = threadIdx.x; b < p.A.nb; b += MV_THREADS) {
        volatile uint8_t *o = p.tap_xq + (size_t)b * 34;   // 34-byte records: only 2-byte alignment holds
        for (int w = 0; w < 8; ++w) {
            const uint32_t v = Yw[((b >> 2) * 8 + w) * 4 + (b & 3)];
            o[2 + 4 * w] = (uint8_t)v; o[3 + 4 * w] = (uint8_t)(v >> 8); o[4 + 4 * w] = (uint8_t)(v >> 16); o[5 + 4 * w] = (uint8_t)(v >> 24);
        }
        *reinterpret_cast<volatile uint16_t *>(p.tap_xq + (size_t)b * 34) = f2h((p.A.type == 2) ? __fmul_rn(DS[b], 16.0f) : DS[b]);
    }
}

// ---------------------------------------------------------------------------------------------
template <int WT, int TM, int R>
__global__ void __launch_bounds__(MV_THREADS, (TM == 1) ? 2 : 1) matvec_kernel(const MatvecParams p, const int ring_bytes, const int S, const int wact) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ float norm_scales[8];
    constexpr int ROWB = ((WT == 8) ? 256 : 128) + 16;   // one row's share of a record: quants of 8 blocks + 8 scales
    constexpr int RECB = 4 * ROWB;
    constexpr int GRPB = (WT == 8) ? 128 : 64;           // quants of one group of four blocks

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = lane >> 3, l = lane & 7;
    const int nbp  = p.A.nbp;
    const int ng   = nbp >> 2;
    const int nrec = nbp >> 3;

    // units of this CTA (a contiguous range) and of this warp (every wact-th of them; warps >= wact only help with
    // the prologue: fewer, longer streams per CTA leave each one a deeper ring and larger copies); a unit is R tiles:
    // tiles R*u .. R*u + R-1 of A, or (pair mode, R == 2) tile u of A and tile u of B
    const int64_t n_units  = p.pair_mode ? (p.A.n_rows >> 2) : (p.A.n_rows / (4 * R));
    const int64_t unit_lo  = n_units * blockIdx.x / gridDim.x;
    const int64_t unit_hi  = n_units * (blockIdx.x + 1) / gridDim.x;
    const int64_t my_first = unit_lo + warp;
    const int     my_units = (warp < wact && my_first < unit_hi) ? (int)((unit_hi - my_first + wact - 1) / wact) : 0;
    const int     n_act    = (int)min((int64_t)wact, unit_hi - unit_lo);   // warps of this CTA that have work
    const int     nch      = (nrec + S - 1) / S;                               // stages per unit
    const int     n_items  = my_units * nch;
    const int     stage_bytes = R * S * RECB;
    const int     NS = max(1, min(MAX_STAGES, ring_bytes / (max(n_act, 1) * stage_bytes)));

    const MatvecSmem L = matvec_smem_layout(nbp, TM, (size_t)ring_bytes);
    uint8_t       *ring   = smem_raw + L.ring + (size_t)warp * NS * stage_bytes;
    const uint32_t ring_s = smem_u32(ring);
    const uint32_t bar_s  = smem_u32(smem_raw + L.bars) + warp * MAX_STAGES * 8;
    const size_t   tile_bytes = (size_t)nrec * RECB;

    // producer side (lane 0 of the warp): stage `lslot` <- the next <= S records of the unit's R tiles
    const uint8_t *src[R];
    int64_t lu = my_first; int lrec = 0, lslot = 0, issued = 0;
    auto unit_sources = [&](int64_t u) {
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const DevMatrix &M = (p.pair_mode && i == 1) ? p.B : p.A;
            src[i] = M.w + (size_t)(p.pair_mode ? u : R * u + i) * tile_bytes;
        }
    };
    auto issue_next = [&]() {
        const uint32_t bytes = (uint32_t)min(S, nrec - lrec) * RECB;
        const uint32_t bar = bar_s + lslot * 8, dst = ring_s + lslot * stage_bytes;
        mbar_expect_tx(bar, bytes * R);
#pragma unroll
        for (int i = 0; i < R; ++i) { bulk_copy_g2s(dst + i * S * RECB, src[i], bytes, bar); src[i] += bytes; }
        ++issued;
        if (++lslot == NS) { lslot = 0; }
        lrec += S;
        if (lrec >= nrec) { lrec = 0; lu += wact; unit_sources(lu); }
    };

    // Let the next kernel of the step begin, and start streaming: weights never change during a step, so the
    // copies may run ahead of the previous kernel's results.
    pdl_launch_dependents();
    stamp(p.stamps, 0, false); stamp(p.stamps, 4, true);
    if (lane == 0 && n_items > 0) {
        for (int s = 0; s < NS; ++s) { mbar_init(bar_s + s * 8, 1); }
        mbar_init_fence();
        unit_sources(lu);
        for (int s = 0; s < NS && issued < n_items; ++s) { issue_next(); }
    }
    __syncwarp();
    pdl_wait();
    stamp(p.stamps, 1, false); stamp(p.stamps, 5, true);
    tp_wait(p.tp, p.error_flag);

    ActPlanes act = act_planes(smem_raw, nbp, TM);
    {
        float *v3 = reinterpret_cast<float *>(smem_raw);
        const int  n4p  = nbp * 8;
        const bool norm = p.pro == PRO_NORM_QUANT;
        if (TM == 1 && n4p <= 2 * MV_THREADS) {
            if (norm) { matvec_prologue_1col<2, true>(p, act, v3, norm_scales); } else { matvec_prologue_1col<2, false>(p, act, v3, norm_scales); }
        } else if (TM == 1 && n4p <= PRO_GROUPS * MV_THREADS) {
            if (norm) { matvec_prologue_1col<PRO_GROUPS, true>(p, act, v3, norm_scales); } else { matvec_prologue_1col<PRO_GROUPS, false>(p, act, v3, norm_scales); }
        } else {
            matvec_prologue<TM>(p, act, v3, norm_scales);
        }
    }
    __syncthreads();
    stamp(p.stamps, 2, false); stamp(p.stamps, 6, true);
    matvec_tap(p, act);

    // this lane's operands, as 32-bit shared-space addresses: activation word (Q8_0 weights: word l; Q4_0: lanes 0..3
    // hold the high nibbles, which meet values 16..31 = words 4..7), the scales, its row and word in a record; and, for
    // Q4_0, the factor that brings its nibbles into the high half of every byte
    const uint32_t y_s   = smem_u32(act.Y) + ((WT == 8) ? l : (l ^ 4)) * 16;
    const uint32_t ds_s  = smem_u32(act.DS);
    const uint32_t row_s = ring_s + r * ROWB + ((WT == 8) ? l : (l & 3)) * 16;
    const uint32_t mult  = (l < 4) ? 1u : 16u;
    const uint32_t tile_off = (uint32_t)S * RECB;        // second tile of the unit inside a stage
    const uint32_t col_y = (uint32_t)ng * 128, col_ds = (uint32_t)ng * 16;   // next activation column

    float acc[TM][R];
#pragma unroll
    for (int t = 0; t < TM; ++t) {
#pragma unroll
        for (int i = 0; i < R; ++i) { acc[t][i] = 0.f; }
    }

    int64_t  cu = my_first; int crec = 0, slot = 0; uint32_t parity = 0;
    uint32_t ya = y_s, da = ds_s;                        // activations of the unit's current group of four blocks
    int      n = 0;
    bool     ok = true;
    for (; n < n_items; ++n) {
        ok = mbar_wait_bounded(bar_s + slot * 8, parity, WAIT_LIMIT_NS);
        if (__any_sync(0xffffffffu, !ok)) { ok = false; break; }
        uint32_t  ra  = row_s + slot * stage_bytes;
        const int cnt = min(S, nrec - crec);
#pragma unroll 1
        for (int rc = 0; rc < cnt; ++rc, ra += RECB) {
            uint4 wq[R][2]; uint4 sc[R];
#pragma unroll
            for (int i = 0; i < R; ++i) {
                const uint32_t rowa = ra + i * tile_off;
                wq[i][0] = lds128(rowa);
                wq[i][1] = lds128(rowa + GRPB);
                sc[i]    = lds128(rowa - ((WT == 8) ? l : (l & 3)) * 16 + (ROWB - 16));
            }
#pragma unroll
            for (int gg = 0; gg < 2; ++gg, ya += 128, da += 16) {
                float s[R][4];
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    const uint32_t s01 = gg ? sc[i].z : sc[i].x, s23 = gg ? sc[i].w : sc[i].y;
                    const float2   f01 = __half22float2(*reinterpret_cast<const __half2 *>(&s01)), f23 = __half22float2(*reinterpret_cast<const __half2 *>(&s23));
                    s[i][0] = f01.x; s[i][1] = f01.y; s[i][2] = f23.x; s[i][3] = f23.y;
                }
#pragma unroll
                for (int t = 0; t < TM; ++t) {
                    const uint4  y  = lds128(ya + t * col_y);
                    const float4 ds = lds128f(da + t * col_ds);
#pragma unroll
                    for (int i = 0; i < R; ++i) {
                        const uint4 w = wq[i][gg];
                        float a = acc[t][i];
                        if (WT == 2) {
                            a = fmaf(__fmul_rn(s[i][0], ds.x), lane_sum16_q4_0(w.x, mult, y.x), a);
                            a = fmaf(__fmul_rn(s[i][1], ds.y), lane_sum16_q4_0(w.y, mult, y.y), a);
                            a = fmaf(__fmul_rn(s[i][2], ds.z), lane_sum16_q4_0(w.z, mult, y.z), a);
                            a = fmaf(__fmul_rn(s[i][3], ds.w), lane_sum16_q4_0(w.w, mult, y.w), a);
                        } else {
                            a = fmaf(__fmul_rn(s[i][0], ds.x), lane_sum_q8_0(w.x, y.x), a);
                            a = fmaf(__fmul_rn(s[i][1], ds.y), lane_sum_q8_0(w.y, y.y), a);
                            a = fmaf(__fmul_rn(s[i][2], ds.z), lane_sum_q8_0(w.z, y.z), a);
                            a = fmaf(__fmul_rn(s[i][3], ds.w), lane_sum_q8_0(w.w, y.w), a);
                        }
                        acc[t][i] = a;
                    }
                }
            }
        }
        __syncwarp();   // every lane is done reading the stage: hand it back to the copy engine
        if (lane == 0 && issued < n_items) { issue_next(); }
        if (++slot == NS) { slot = 0; parity ^= 1u; }
        crec += S;
        if (crec >= nrec) {   // unit finished: fixed reduction tree over the 8 accumulators of each row, then the epilogue
#pragma unroll
            for (int t = 0; t < TM; ++t) {
                float h[R];
#pragma unroll
                for (int i = 0; i < R; ++i) { h[i] = hsum8_lanes(acc[t][i]); acc[t][i] = 0.f; }
                const bool    writer = (l == 0) && (t < p.T);
                const int64_t row0 = p.pair_mode ? 4 * cu + r : 4 * R * cu + r;
                if (p.epi == EPI_SILU_MUL) {
                    if (R == 2) { matvec_epilogue_silu(p, row0, t, h[0], h[R - 1], writer); }
                } else {
#pragma unroll
                    for (int i = 0; i < R; ++i) {
                        const float partner = __shfl_xor_sync(0xffffffffu, h[i], 8);
                        matvec_epilogue(p, row0 + 4 * i, t, h[i], partner, writer);
                    }
                }
            }
            crec = 0; cu += wact; ya = y_s; da = ds_s;
        }
    }
    if (!ok) {
        // a copy did not arrive: report, give the copies still in flight a last bounded chance to land (they
        // target this CTA's shared memory) and stop; the host sees the flag at its next synchronisation
        if (lane == 0 && p.error_flag != nullptr) { atomicExch(p.error_flag, 1); }
        for (int k = n; k < __shfl_sync(0xffffffffu, issued, 0); ++k) {
            mbar_wait_bounded(bar_s + slot * 8, parity, 10000000ull);
            if (++slot == NS) { slot = 0; parity ^= 1u; }
        }
    }

    tp_publish(p.tp, p.T);
    if (p.stamps != nullptr) { __syncthreads(); stamp(p.stamps, 3, true); }
}

// ---------------------------------------------------------------------------------------------
// Variant for matrices stored in tiles of TR = 32, 16 or 8 rows (DevMatrix::tile_rows): a row belongs to LPR = 32 / TR
// lanes of one warp, lane = (part, row), and a lane keeps 8 / LPR whole accumulators of its row in registers:
//   LPR == 1: all eight accumulators
//   LPR == 2: part h takes the accumulator pairs (2h, 2h + 4) and (2h + 1, 2h + 5)
//   LPR == 4: part q takes the pair (q, q + 4) (Q4_0: both nibbles of quant word q; Q8_0: words q and q + 4)
// - exactly the pairs hsum_float_8 adds first, ((a0+a4)+(a2+a6))+((a1+a5)+(a3+a7)); the pair sums of a row meet by
// shuffle. The scale product d_w * d_x and the activation words are fetched once per lane and block instead of once per
// accumulator, so the kernel issues about half the instructions per weight byte of the lane-per-accumulator kernel.
// A tile walks along K sequentially on one warp; the tile height is chosen per matrix so that a CTA has about as many
// tiles as warps (tall matrices: 32 or 16 rows, d_model-sized ones: 8).
// Every warp streams its tiles through a private ring: lane 0 issues the bulk copies (one per stage), all lanes wait on
// the stage's mbarrier, and the warp's own __syncwarp hands a stage back for the refill.
// A record is [TR rows][2 groups x 64 B (Q4_0) or 128 B (Q8_0) | 8 fp16 scales]; the 144-byte (272-byte) row pitch
// makes the 128-bit reads of eight consecutive rows conflict-free.
// With fused_pair, rows 0..TR/2-1 of tile u are FFN-up rows (TR/2)u.. and rows TR/2..TR-1 the matching FFN-gate rows.
template <int WT, int TM, int LPR>
__global__ void __launch_bounds__(MV_THREADS, 1) matvec_rows_kernel(const MatvecParams p, const int ring_bytes, const int S, const int wact) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ float norm_scales[8];
    constexpr int TR   = 32 / LPR;                       // rows per tile
    constexpr int ROWB = ((WT == 8) ? 256 : 128) + 16;
    constexpr int RECB = TR * ROWB;
    constexpr int GRPB = (WT == 8) ? 128 : 64;
    constexpr int NP   = 4 / LPR;                        // accumulator pairs (j, j + 4) per lane

    const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
    const int part = lane / TR, lrow = lane % TR;
    const int nbp  = p.A.nbp;
    const int ng   = nbp >> 2;
    const int nrec = nbp >> 3;

    const int64_t n_units  = p.A.n_rows / TR;
    const int64_t unit_lo  = n_units * blockIdx.x / gridDim.x;
    const int64_t unit_hi  = n_units * (blockIdx.x + 1) / gridDim.x;
    const int64_t my_first = unit_lo + grp;
    const int     my_units = (grp < wact && my_first < unit_hi) ? (int)((unit_hi - my_first + wact - 1) / wact) : 0;
    const int     n_act    = (int)min((int64_t)wact, unit_hi - unit_lo);   // warps of this CTA that have work
    const int     nch      = (nrec + S - 1) / S;
    const int     n_items  = my_units * nch;
    const int     stage_bytes = S * RECB;
    const int     NS = max(1, min(MAX_STAGES, ring_bytes / (max(n_act, 1) * stage_bytes)));

    const MatvecSmem L = matvec_smem_layout(nbp, TM, (size_t)ring_bytes);
    const uint32_t ring_s  = smem_u32(smem_raw + L.ring) + (uint32_t)grp * NS * stage_bytes;
    const uint32_t full_s  = smem_u32(smem_raw + L.bars) + grp * MAX_STAGES * 8;
    const size_t   tile_bytes = (size_t)nrec * RECB;

    const uint8_t *src = nullptr;
    int64_t lu = my_first; int lrec = 0, lslot = 0, issued = 0;
    bool    ok = true;
    // lane 0: stage lslot <- the next <= S records (the stage was handed back by this warp's own __syncwarp)
    auto issue_next = [&]() {
        const uint32_t bytes = (uint32_t)min(S, nrec - lrec) * RECB;
        const uint32_t bar = full_s + lslot * 8;
        mbar_expect_tx(bar, bytes);
        bulk_copy_g2s(ring_s + lslot * stage_bytes, src, bytes, bar);
        src += bytes;
        ++issued;
        if (++lslot == NS) { lslot = 0; }
        lrec += S;
        if (lrec >= nrec) { lrec = 0; lu += wact; src = p.A.w + (size_t)lu * tile_bytes; }
    };

    pdl_launch_dependents();
    stamp(p.stamps, 0, false); stamp(p.stamps, 4, true);
    if (lane == 0 && n_items > 0) {
        for (int s = 0; s < NS; ++s) { mbar_init(full_s + s * 8, 1); }
        mbar_init_fence();
        src = p.A.w + (size_t)lu * tile_bytes;
        for (int s = 0; s < NS && issued < n_items; ++s) { issue_next(); }
    }
    __syncwarp();
    pdl_wait();
    stamp(p.stamps, 1, false); stamp(p.stamps, 5, true);
    tp_wait(p.tp, p.error_flag);

    ActPlanes act = act_planes(smem_raw, nbp, TM);
    {
        float *v3 = reinterpret_cast<float *>(smem_raw);
        const int  n4p  = nbp * 8;
        const bool norm = p.pro == PRO_NORM_QUANT;
        if (TM == 1 && n4p <= 2 * MV_THREADS) {
            if (norm) { matvec_prologue_1col<2, true>(p, act, v3, norm_scales); } else { matvec_prologue_1col<2, false>(p, act, v3, norm_scales); }
        } else if (TM == 1 && n4p <= PRO_GROUPS * MV_THREADS) {
            if (norm) { matvec_prologue_1col<PRO_GROUPS, true>(p, act, v3, norm_scales); } else { matvec_prologue_1col<PRO_GROUPS, false>(p, act, v3, norm_scales); }
        } else {
            matvec_prologue<TM>(p, act, v3, norm_scales);
        }
    }
    __syncthreads();
    stamp(p.stamps, 2, false); stamp(p.stamps, 6, true);
    matvec_tap(p, act);

    const uint32_t y_s   = smem_u32(act.Y);
    const uint32_t ds_s  = smem_u32(act.DS);
    const uint32_t row_s = ring_s + lrow * ROWB;
    const uint32_t col_y = (uint32_t)ng * 128, col_ds = (uint32_t)ng * 16;

    // pair k of column t as one packed f32x2 value: low half = accumulator j, high half = accumulator j + 4, j = part * NP + k
    // (both take the same scale in every step, so one packed subtraction and one packed FMA serve the two)
    uint64_t acc2[TM][NP];
#pragma unroll
    for (int t = 0; t < TM; ++t) {
#pragma unroll
        for (int k = 0; k < NP; ++k) { acc2[t][k] = 0ull; }
    }
    const uint64_t minus_magic = f2_pack(-MAGIC_F, -MAGIC_F);

    int64_t  cu = my_first; int crec = 0, slot = 0; uint32_t parity = 0;
    uint32_t ya = y_s, da = ds_s;
    int      n = 0;
    for (; n < n_items; ++n) {
        bool got = mbar_wait_bounded(full_s + slot * 8, parity, WAIT_LIMIT_NS);
        if (__any_sync(0xffffffffu, !got || !ok)) { ok = false; break; }
        uint32_t  ra  = row_s + slot * stage_bytes;
        const int cnt = min(S, nrec - crec);
#pragma unroll 1
        for (int rc = 0; rc < cnt; ++rc, ra += RECB) {
            const uint4 sc = lds128(ra + 2 * GRPB);
#pragma unroll
            for (int gg = 0; gg < 2; ++gg, ya += 128, da += 16) {
                const uint32_t s01 = gg ? sc.z : sc.x, s23 = gg ? sc.w : sc.y;
                const float2   f01 = __half22float2(*reinterpret_cast<const __half2 *>(&s01)), f23 = __half22float2(*reinterpret_cast<const __half2 *>(&s23));
                uint4 w[(WT == 8) ? 2 * NP : NP];
#pragma unroll
                for (int k = 0; k < NP; ++k) {
                    const int j = part * NP + k;
                    if (WT == 8) { w[2 * k] = lds128(ra + gg * GRPB + j * 16); w[2 * k + 1] = lds128(ra + gg * GRPB + (4 + j) * 16); }
                    else         { w[k] = lds128(ra + gg * GRPB + j * 16); }
                }
#pragma unroll
                for (int t = 0; t < TM; ++t) {
                    const float4 ds = lds128f(da + t * col_ds);
                    const float  s0 = __fmul_rn(f01.x, ds.x), s1 = __fmul_rn(f01.y, ds.y), s2 = __fmul_rn(f23.x, ds.z), s3 = __fmul_rn(f23.y, ds.w);
                    const uint64_t S0 = f2_pack(s0, s0), S1 = f2_pack(s1, s1), S2 = f2_pack(s2, s2), S3 = f2_pack(s3, s3);
#pragma unroll
                    for (int k = 0; k < NP; ++k) {
                        const int j = part * NP + k;
                        // accumulator j: Q4_0 high nibbles of word j (values 16 + 4j.. meet activation word 4 + j), Q8_0 word j;
                        // accumulator 4 + j: Q4_0 low nibbles of word j (activation word j), Q8_0 word 4 + j
                        const uint4 y0 = lds128(ya + t * col_y + ((WT == 8) ? j : 4 + j) * 16), y1 = lds128(ya + t * col_y + ((WT == 8) ? 4 + j : j) * 16);
                        uint64_t a = acc2[t][k];
                        if (WT == 2) {
                            a = f2_fma(S0, f2_add(f2_pack_bits(lane_bits16_q4_0(w[k].x, 1u, y0.x), lane_bits16_q4_0(w[k].x, 16u, y1.x)), minus_magic), a);
                            a = f2_fma(S1, f2_add(f2_pack_bits(lane_bits16_q4_0(w[k].y, 1u, y0.y), lane_bits16_q4_0(w[k].y, 16u, y1.y)), minus_magic), a);
                            a = f2_fma(S2, f2_add(f2_pack_bits(lane_bits16_q4_0(w[k].z, 1u, y0.z), lane_bits16_q4_0(w[k].z, 16u, y1.z)), minus_magic), a);
                            a = f2_fma(S3, f2_add(f2_pack_bits(lane_bits16_q4_0(w[k].w, 1u, y0.w), lane_bits16_q4_0(w[k].w, 16u, y1.w)), minus_magic), a);
                        } else {
                            a = f2_fma(S0, f2_add(f2_pack_bits(lane_bits_q8_0(w[2 * k].x, y0.x), lane_bits_q8_0(w[2 * k + 1].x, y1.x)), minus_magic), a);
                            a = f2_fma(S1, f2_add(f2_pack_bits(lane_bits_q8_0(w[2 * k].y, y0.y), lane_bits_q8_0(w[2 * k + 1].y, y1.y)), minus_magic), a);
                            a = f2_fma(S2, f2_add(f2_pack_bits(lane_bits_q8_0(w[2 * k].z, y0.z), lane_bits_q8_0(w[2 * k + 1].z, y1.z)), minus_magic), a);
                            a = f2_fma(S3, f2_add(f2_pack_bits(lane_bits_q8_0(w[2 * k].w, y0.w), lane_bits_q8_0(w[2 * k + 1].w, y1.w)), minus_magic), a);
                        }
                        acc2[t][k] = a;
                    }
                }
            }
        }
        __syncwarp();   // every lane is done reading the stage
        if (lane == 0 && issued < n_items) { issue_next(); }
        if (++slot == NS) { slot = 0; parity ^= 1u; }
        crec += S;
        if (crec >= nrec) {   // tile finished: hsum_float_8 tree ((a0+a4)+(a2+a6))+((a1+a5)+(a3+a7)), then the epilogue
            // pair sums p_j = a_j + a_(j+4); h = (p0 + p2) + (p1 + p3); a row's LPR lanes exchange theirs by shuffle
            float h[TM];
#pragma unroll
            for (int t = 0; t < TM; ++t) {
                float acc[1][2 * NP];   // (indexed [0][..] below: this column's accumulators unpacked)
#pragma unroll
                for (int k = 0; k < NP; ++k) { f2_unpack(acc2[t][k], acc[0][2 * k], acc[0][2 * k + 1]); acc2[t][k] = 0ull; }
                if (LPR == 1) {
                    h[t] = __fadd_rn(__fadd_rn(__fadd_rn(acc[0][0], acc[0][1]), __fadd_rn(acc[0][4], acc[0][5])),
                                     __fadd_rn(__fadd_rn(acc[0][2], acc[0][3]), __fadd_rn(acc[0][6], acc[0][7])));
                } else if (LPR == 2) {   // part 0 holds p0, p1; part 1 holds p2, p3
                    const float pa = __fadd_rn(acc[0][0], acc[0][1]), pb = __fadd_rn(acc[0][2], acc[0][3]);
                    const float qa = __fadd_rn(pa, __shfl_xor_sync(0xffffffffu, pa, 16)), qb = __fadd_rn(pb, __shfl_xor_sync(0xffffffffu, pb, 16));
                    h[t] = __fadd_rn(qa, qb);
                } else {                 // part q holds p_q
                    const float pa = __fadd_rn(acc[0][0], acc[0][1]);
                    const float qa = __fadd_rn(pa, __shfl_xor_sync(0xffffffffu, pa, 16));
                    h[t] = __fadd_rn(qa, __shfl_xor_sync(0xffffffffu, qa, 8));
                }
            }
#pragma unroll
            for (int t = 0; t < TM; ++t) {
                if (p.epi == EPI_SILU_MUL) {
                    const float gate = __shfl_down_sync(0xffffffffu, h[t], TR / 2);
                    matvec_epilogue_silu(p, (TR / 2) * cu + lane, t, h[t], gate, lane < TR / 2 && t < p.T);
                } else {
                    const float partner = __shfl_xor_sync(0xffffffffu, h[t], 1);
                    matvec_epilogue(p, TR * cu + lane, t, h[t], partner, lane < TR && t < p.T);
                }
            }
            crec = 0; cu += wact; ya = y_s; da = ds_s;
        }
    }
    if (!ok) {
        // a copy (or a partner warp) did not arrive: report, give the copies still in flight a last bounded chance to
        // land (they target this CTA's shared memory) and stop; the host sees the flag at its next synchronisation
        if (lane == 0 && p.error_flag != nullptr) { atomicExch(p.error_flag, 1); }
        for (int k = n; k < __shfl_sync(0xffffffffu, issued, 0); ++k) {
            mbar_wait_bounded(full_s + slot * 8, parity, 10000000ull);
            if (++slot == NS) { slot = 0; parity ^= 1u; }
        }
    }
    tp_publish(p.tp, p.T);
    if (p.stamps != nullptr) { __syncthreads(); stamp(p.stamps, 3, true); }
}

// ---------------------------------------------------------------------------------------------
// Tensor-core variant for matrices stored in fragment order (DevMatrix::mma, tiles of TR = 16 or 8 rows): the integer
// group sums of a block come out of one mma.sync per block and 16 rows instead of eight byte dot products per row; the
// inner loop and its exactness argument are in spyb_mma.cuh. Streaming, prologue and epilogues as in matvec_rows_kernel.
template <int WT, int TM, int TR>
__global__ void __launch_bounds__(MV_THREADS, 1) matvec_mma_kernel(const MatvecParams p, const int ring_bytes, const int S, const int wact) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ float norm_scales[8];
    constexpr int RECB = MmaTile<WT, TR>::RECB;
    constexpr int NA   = MmaTile<WT, TR>::NA;            // accumulators per lane

    const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
    const int g = lane >> 2, q = lane & 3;
    const int nbp  = p.A.nbp;
    const int ng   = nbp >> 2;
    const int nrec = nbp >> 3;

    const int64_t n_units  = p.A.n_rows / TR;
    const int64_t unit_lo  = n_units * blockIdx.x / gridDim.x;
    const int64_t unit_hi  = n_units * (blockIdx.x + 1) / gridDim.x;
    const int64_t my_first = unit_lo + grp;
    const int     my_units = (grp < wact && my_first < unit_hi) ? (int)((unit_hi - my_first + wact - 1) / wact) : 0;
    const int     n_act    = (int)min((int64_t)wact, unit_hi - unit_lo);
    const int     nch      = (nrec + S - 1) / S;
    const int     n_items  = my_units * nch;
    const int     stage_bytes = S * RECB;
    const int     NS = max(1, min(MAX_STAGES, ring_bytes / (max(n_act, 1) * stage_bytes)));

    const MatvecSmem L = matvec_smem_layout(nbp, TM, (size_t)ring_bytes);
    const uint32_t ring_s  = smem_u32(smem_raw + L.ring) + (uint32_t)grp * NS * stage_bytes;
    const uint32_t full_s  = smem_u32(smem_raw + L.bars) + grp * MAX_STAGES * 8;
    const size_t   tile_bytes = (size_t)nrec * RECB;

    const uint8_t *src = nullptr;
    int64_t lu = my_first; int lrec = 0, lslot = 0, issued = 0;
    bool    ok = true;
    auto issue_next = [&]() {
        const uint32_t bytes = (uint32_t)min(S, nrec - lrec) * RECB;
        const uint32_t bar = full_s + lslot * 8;
        mbar_expect_tx(bar, bytes);
        bulk_copy_g2s(ring_s + lslot * stage_bytes, src, bytes, bar);
        src += bytes;
        ++issued;
        if (++lslot == NS) { lslot = 0; }
        lrec += S;
        if (lrec >= nrec) { lrec = 0; lu += wact; src = p.A.w + (size_t)lu * tile_bytes; }
    };

    pdl_launch_dependents();
    stamp(p.stamps, 0, false); stamp(p.stamps, 4, true);
    if (lane == 0 && n_items > 0) {
        for (int s = 0; s < NS; ++s) { mbar_init(full_s + s * 8, 1); }
        mbar_init_fence();
        src = p.A.w + (size_t)lu * tile_bytes;
        for (int s = 0; s < NS && issued < n_items; ++s) { issue_next(); }
    }
    __syncwarp();
    pdl_wait();
    stamp(p.stamps, 1, false); stamp(p.stamps, 5, true);
    tp_wait(p.tp, p.error_flag);

    ActPlanes act = act_planes(smem_raw, nbp, TM);
    {
        float *v3 = reinterpret_cast<float *>(smem_raw);
        const int  n4p  = nbp * 8;
        const bool norm = p.pro == PRO_NORM_QUANT;
        if (TM == 1 && n4p <= 2 * MV_THREADS) {
            if (norm) { matvec_prologue_1col<2, true>(p, act, v3, norm_scales); } else { matvec_prologue_1col<2, false>(p, act, v3, norm_scales); }
        } else if (TM == 1 && n4p <= PRO_GROUPS * MV_THREADS) {
            if (norm) { matvec_prologue_1col<PRO_GROUPS, true>(p, act, v3, norm_scales); } else { matvec_prologue_1col<PRO_GROUPS, false>(p, act, v3, norm_scales); }
        } else {
            matvec_prologue<TM>(p, act, v3, norm_scales);
        }
    }
    __syncthreads();
    stamp(p.stamps, 2, false); stamp(p.stamps, 6, true);
    matvec_tap(p, act);

    const MmaLane  ML = mma_lane<WT, TR>(lane);
    const uint32_t y_s = smem_u32(act.Y), ds_s = smem_u32(act.DS);
    const uint32_t col_y = (uint32_t)ng * 128, col_ds = (uint32_t)ng * 16;

    float acc[TM][NA];
#pragma unroll
    for (int t = 0; t < TM; ++t) {
#pragma unroll
        for (int a = 0; a < NA; ++a) { acc[t][a] = 0.f; }
    }

    int64_t  cu = my_first; int crec = 0, slot = 0; uint32_t parity = 0;
    uint32_t ya = y_s, da = ds_s;
    int      n = 0;
    for (; n < n_items; ++n) {
        bool got = mbar_wait_bounded(full_s + slot * 8, parity, WAIT_LIMIT_NS);
        if (__any_sync(0xffffffffu, !got || !ok)) { ok = false; break; }
        mma_records<WT, TR, TM>(ring_s + slot * stage_bytes, min(S, nrec - crec), ya, da, col_y, col_ds, ML, acc);
        __syncwarp();   // every lane is done reading the stage
        if (lane == 0 && issued < n_items) { issue_next(); }
        if (++slot == NS) { slot = 0; parity ^= 1u; }
        crec += S;
        if (crec >= nrec) {   // tile finished: hsum_float_8 tree, then the epilogue
#pragma unroll
            for (int t = 0; t < TM; ++t) {
                float h[2] = {0.f, 0.f};
#pragma unroll
                for (int r = 0; r < NA / 2; ++r) { h[r] = mma_row_sum(acc[t][2 * r], acc[t][2 * r + 1]); acc[t][2 * r] = 0.f; acc[t][2 * r + 1] = 0.f; }
                const bool wr = (q == 0) && (t < p.T);
                if (p.epi == EPI_SILU_MUL) {
                    if (TR == 16) { matvec_epilogue_silu(p, 8 * cu + g, t, h[0], h[1], wr); }
                    else { const float gate = __shfl_down_sync(0xffffffffu, h[0], 16); matvec_epilogue_silu(p, 4 * cu + g, t, h[0], gate, wr && g < 4); }
                } else {
#pragma unroll
                    for (int r = 0; r < NA / 2; ++r) {
                        const float partner = __shfl_xor_sync(0xffffffffu, h[r], 4);   // the neighbouring row (RoPE pairs)
                        matvec_epilogue(p, TR * cu + 8 * r + g, t, h[r], partner, wr);
                    }
                }
            }
            crec = 0; cu += wact; ya = y_s; da = ds_s;
        }
    }
    if (!ok) {
        if (lane == 0 && p.error_flag != nullptr) { atomicExch(p.error_flag, 1); }
        for (int k = n; k < __shfl_sync(0xffffffffu, issued, 0); ++k) {
            mbar_wait_bounded(full_s + slot * 8, parity, 10000000ull);
            if (++slot == NS) { slot = 0; parity ^= 1u; }
        }
    }
    tp_publish(p.tp, p.T);
    if (p.stamps != nullptr) { __syncthreads(); stamp(p.stamps, 3, true); }
}

template <int WT, int TM, int TR>
static cudaError_t launch_matvec_mma_t(const MatvecParams &p, const LaunchCfg &cfg) {
    constexpr int RECB = TR * (((WT == 8) ? 256 : 128) + 16);
    const int64_t n_units = p.A.n_rows / TR;
    int64_t grid = std::min<int64_t>(cfg.num_sms, n_units);
    if (grid < 1) { grid = 1; }
    const int64_t units_per_cta = (n_units + grid - 1) / grid;
    const MatvecSmem fixed = matvec_smem_layout(p.A.nbp, TM, 0);
    const size_t budget = 216 * 1024;
    if (fixed.total + (size_t)RECB > budget) { return cudaErrorInvalidValue; }
    const size_t ring = std::min<size_t>((size_t)cfg.mv_ring_kb * 2 * 1024, budget - fixed.total) / 128 * 128;
    const int nrec = p.A.nbp >> 3;
    int wact = (int)std::min<int64_t>(MV_WARPS, units_per_cta);
    int S = 64 / TR;                      // stages of about 9 KB (Q4_0); at least three per warp, else smaller ones
    while (S > nrec) { S >>= 1; }
    if (S < 1) { S = 1; }
    while (ring / ((size_t)wact * S * RECB) < 3) {
        if (S > 1) { S >>= 1; }
        else if (wact > 1) { wact = (wact + 1) / 2; }
        else { break; }
    }
    if (cfg.mv_force_s > 0) { S = std::min(cfg.mv_force_s, std::max(nrec, 1)); }
    if (cfg.mv_force_wact > 0) { wact = std::min(cfg.mv_force_wact, MV_WARPS); }
    if (ring / ((size_t)wact * S * RECB) < 1) { return cudaErrorInvalidValue; }
    const size_t smem = fixed.total + ring;
    cudaError_t err = allow_dynamic_smem(reinterpret_cast<const void *>(matvec_mma_kernel<WT, TM, TR>), smem);
    if (err != cudaSuccess) { return err; }
    MatvecParams q = p;
    if (q.error_flag == nullptr) { q.error_flag = cfg.error_flag; }
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)grid); lc.blockDim = dim3(MV_THREADS); lc.dynamicSmemBytes = smem; lc.stream = cfg.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr; lc.numAttrs = cfg.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&lc, matvec_mma_kernel<WT, TM, TR>, q, (int)ring, S, wact);
}

template <int WT, int TR>
static cudaError_t launch_matvec_mma_w(const MatvecParams &p, const LaunchCfg &cfg) {
    if (p.T <= 1) { return launch_matvec_mma_t<WT, 1, TR>(p, cfg); }
    if (p.T <= 2) { return launch_matvec_mma_t<WT, 2, TR>(p, cfg); }
    return launch_matvec_mma_t<WT, 4, TR>(p, cfg);
}

template <int WT, int TM, int LPR>
static cudaError_t launch_matvec_rows_t(const MatvecParams &p, const LaunchCfg &cfg) {
    constexpr int TR = 32 / LPR;
    constexpr int RECB = TR * (((WT == 8) ? 256 : 128) + 16);
    const int64_t n_units = p.A.n_rows / TR;
    int64_t grid = std::min<int64_t>(cfg.num_sms, n_units);
    if (grid < 1) { grid = 1; }
    const int64_t units_per_cta = (n_units + grid - 1) / grid;
    const MatvecSmem fixed = matvec_smem_layout(p.A.nbp, TM, 0);
    const size_t budget = 216 * 1024;   // (the kernels also hold a few KB of static shared memory)
    if (fixed.total + (size_t)RECB > budget) { return cudaErrorInvalidValue; }
    const size_t ring = std::min<size_t>((size_t)cfg.mv_ring_kb * 2 * 1024, budget - fixed.total) / 128 * 128;
    const int nrec = p.A.nbp >> 3;
    int wact = (int)std::min<int64_t>(MV_WARPS, units_per_cta);
    int S = 2 * LPR;                      // stages of about 9 KB (Q4_0); at least three per warp, else smaller ones
    while (S > nrec) { S >>= 1; }
    if (S < 1) { S = 1; }
    while (ring / ((size_t)wact * S * RECB) < 3) {
        if (S > 1) { S >>= 1; }
        else if (wact > 1) { wact = (wact + 1) / 2; }
        else { break; }
    }
    if (cfg.mv_force_s > 0) { S = std::min(cfg.mv_force_s, std::max(nrec, 1)); }
    if (cfg.mv_force_wact > 0) { wact = std::min(cfg.mv_force_wact, MV_WARPS); }
    if (ring / ((size_t)wact * S * RECB) < 1) { return cudaErrorInvalidValue; }
    const size_t smem = fixed.total + ring;
    cudaError_t err = allow_dynamic_smem(reinterpret_cast<const void *>(matvec_rows_kernel<WT, TM, LPR>), smem);
    if (err != cudaSuccess) { return err; }
    MatvecParams q = p;
    if (q.error_flag == nullptr) { q.error_flag = cfg.error_flag; }
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)grid); lc.blockDim = dim3(MV_THREADS); lc.dynamicSmemBytes = smem; lc.stream = cfg.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr; lc.numAttrs = cfg.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&lc, matvec_rows_kernel<WT, TM, LPR>, q, (int)ring, S, wact);
}

template <int WT, int LPR>
static cudaError_t launch_matvec_rows_w(const MatvecParams &p, const LaunchCfg &cfg) {
    if (p.T <= 1) { return launch_matvec_rows_t<WT, 1, LPR>(p, cfg); }
    if (p.T <= 2) { return launch_matvec_rows_t<WT, 2, LPR>(p, cfg); }
    return launch_matvec_rows_t<WT, 4, LPR>(p, cfg);
}

int matvec_max_columns(int nb) {   // (the lane-per-row kernel keeps 8 accumulators per column in registers: at most 4 columns)
    for (int t = 4; t > 1; t >>= 1) { if (act_plane_bytes(padded_blocks(nb), t) <= 120 * 1024) { return t; } }
    return 1;
}

template <int WT, int TM, int R>
static cudaError_t launch_matvec_t(const MatvecParams &p, const LaunchCfg &cfg) {
    constexpr int RECB = 4 * (((WT == 8) ? 256 : 128) + 16);
    // every SM gets CTAs even when there are fewer units than warps: a unit is a sequential walk along K, so
    // spreading units over all SMs (with some warps idle) beats filling a few CTAs
    const int64_t n_units = p.pair_mode ? (p.A.n_rows >> 2) : (p.A.n_rows / (4 * R));
    const int     per_sm  = (TM == 1) ? cfg.mv_ctas_per_sm : 1;
    int64_t grid = (int64_t)cfg.num_sms * per_sm;
    if (grid > n_units) { grid = n_units; }
    if (grid < 1) { grid = 1; }
    const int64_t units_per_cta = (n_units + grid - 1) / grid;

    // ring: what the SM's shared memory leaves after the activation planes (two CTAs per SM for single columns)
    const MatvecSmem fixed = matvec_smem_layout(p.A.nbp, TM, 0);
    const size_t budget = (per_sm == 2) ? 108 * 1024 : 216 * 1024;   // (the kernels also hold a few KB of static shared memory)
    if (fixed.total + (size_t)2 * R * RECB > budget) { return cudaErrorInvalidValue; }   // rows too long for this kernel
    size_t ring = std::min<size_t>((size_t)cfg.mv_ring_kb * 1024 * ((TM == 1) ? 1 : 2), budget - fixed.total) / 128 * 128;
    // S records per stage (one bulk copy per tile and stage) and the number of warps that stream: copies of a few KB
    // and at least three stages per stream; when the ring is too small for that with every warp streaming, fewer
    // warps take more units each
    const int nrec = p.A.nbp >> 3;
    int wact = (int)std::min<int64_t>(MV_WARPS, units_per_cta);
    int S = 8;
    while (S > nrec) { S >>= 1; }
    if (S < 1) { S = 1; }
    const int s_small = std::max(1, std::min(S, 4096 / RECB));   // do not go below ~4 KB copies while warps can still be merged
    while (ring / ((size_t)wact * R * S * RECB) < 3) {
        if (S > s_small) { S >>= 1; }
        else if (wact > 4) { wact = (wact + 1) / 2; }
        else if (S > 1) { S >>= 1; }
        else if (wact > 1) { wact = (wact + 1) / 2; }
        else { break; }
    }
    if (cfg.mv_force_s > 0) { S = std::min(cfg.mv_force_s, std::max(nrec, 1)); }
    if (cfg.mv_force_wact > 0) { wact = std::min(cfg.mv_force_wact, MV_WARPS); }
    if (ring / ((size_t)wact * R * S * RECB) < 1) { return cudaErrorInvalidValue; }
    const size_t smem = fixed.total + ring;

    cudaError_t err = allow_dynamic_smem(reinterpret_cast<const void *>(matvec_kernel<WT, TM, R>), smem);
    if (err != cudaSuccess) { return err; }
    MatvecParams q = p;
    if (q.error_flag == nullptr) { q.error_flag = cfg.error_flag; }

    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)grid); lc.blockDim = dim3(MV_THREADS); lc.dynamicSmemBytes = smem; lc.stream = cfg.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr; lc.numAttrs = cfg.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&lc, matvec_kernel<WT, TM, R>, q, (int)ring, S, wact);
}

template <int WT, int R>
static cudaError_t launch_matvec_w(const MatvecParams &p, const LaunchCfg &cfg) {
    if (p.T <= 1) { return launch_matvec_t<WT, 1, R>(p, cfg); }
    if (p.T <= 2) { return launch_matvec_t<WT, 2, R>(p, cfg); }
    if (p.T <= 4) { return launch_matvec_t<WT, 4, R>(p, cfg); }
    return launch_matvec_t<WT, 8, R>(p, cfg);
}

cudaError_t launch_matvec(const MatvecParams &p, const LaunchCfg &cfg) {
    if (p.kq_n > 0) { return launch_matvec_kq(p, cfg); }
    if (p.T < 1 || p.T > matvec_max_columns(p.A.nb)) { return cudaErrorInvalidValue; }
    if ((p.tp.counter != nullptr || p.tp.flag_in != nullptr) && (p.tp.n < 2 || p.tp.n > TP_MAX || p.tp.epoch == nullptr)) { return cudaErrorInvalidValue; }
    if (p.tp.counter != nullptr && ((p.tp.len & 3) || (p.tp.off & 3) || (p.tp.stride & 3))) { return cudaErrorInvalidValue; }
    if (p.A.k % QK != 0 || p.A.nb < 1 || p.A.nbp != padded_blocks(p.A.nb) || p.A.w == nullptr) { return cudaErrorInvalidValue; }
    if (p.A.mma) {
        if ((p.A.tile_rows != 16 && p.A.tile_rows != 8) || (p.A.n_rows % p.A.tile_rows) || p.pair_mode || (p.epi == EPI_SILU_MUL) != (p.A.fused_pair != 0)) { return cudaErrorInvalidValue; }
        switch (p.A.type) {
        case 2: return p.A.tile_rows == 16 ? launch_matvec_mma_w<2, 16>(p, cfg) : launch_matvec_mma_w<2, 8>(p, cfg);
        case 8: return p.A.tile_rows == 16 ? launch_matvec_mma_w<8, 16>(p, cfg) : launch_matvec_mma_w<8, 8>(p, cfg);
        default: return cudaErrorNotSupported;
        }
    }
    if (p.A.tile_rows == 32 || p.A.tile_rows == 16 || p.A.tile_rows == 8) {
        if ((p.A.n_rows % p.A.tile_rows) || p.pair_mode || (p.epi == EPI_SILU_MUL) != (p.A.fused_pair != 0)) { return cudaErrorInvalidValue; }
        const int lpr = 32 / p.A.tile_rows;
        switch (p.A.type) {
        case 2: return lpr == 1 ? launch_matvec_rows_w<2, 1>(p, cfg) : lpr == 2 ? launch_matvec_rows_w<2, 2>(p, cfg) : launch_matvec_rows_w<2, 4>(p, cfg);
        case 8: return lpr == 1 ? launch_matvec_rows_w<8, 1>(p, cfg) : lpr == 2 ? launch_matvec_rows_w<8, 2>(p, cfg) : launch_matvec_rows_w<8, 4>(p, cfg);
        default: return cudaErrorNotSupported;
        }
    }
    if (p.A.tile_rows != 4 || (p.A.n_rows & 3)) { return cudaErrorInvalidValue; }
    if (p.pair_mode && (p.B.type != p.A.type || p.B.n_rows != p.A.n_rows || p.B.k != p.A.k || p.B.nbp != p.A.nbp || p.B.w == nullptr)) { return cudaErrorInvalidValue; }
    if ((p.epi == EPI_SILU_MUL) != (p.pair_mode != 0)) { return cudaErrorInvalidValue; }
    // tiles per warp: two when one would leave units waiting for a free warp (single column), or in pair mode
    bool two = p.pair_mode != 0;
    if (!two && p.T == 1 && (p.A.n_rows & 7) == 0) {
        const int64_t slots = (int64_t)cfg.num_sms * cfg.mv_ctas_per_sm * MV_WARPS;
        two = (p.A.n_rows >> 2) > slots;
    }
    switch (p.A.type) {
    case 2: return two ? launch_matvec_w<2, 2>(p, cfg) : launch_matvec_w<2, 1>(p, cfg);
    case 8: return two ? launch_matvec_w<8, 2>(p, cfg) : launch_matvec_w<8, 1>(p, cfg);
    default: return cudaErrorNotSupported;
    }
}

}  // namespace spyb
