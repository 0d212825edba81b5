// Prompt evaluation as a dequant-fused GEMM on the 5th-generation tensor cores (tcgen05, accumulators in tensor memory).
//
// The reference evaluates MatMul(W[Q4_0 | Q8_0], x) for a prompt of T tokens as T independent dot products per row
// (backend/host/operator/mat.cpp:95-128 with Dot<Q4_0,Q8_0> / Dot<Q8_0,Q8_0>, backend/host/include/simd/vec_dot.h:42-115):
// per 32-element block the eight integer "lane sums" (4 products each) are converted to f32 and folded into eight f32
// accumulators with acc = fma(d_w * d_x, lane_sum, acc), block after block, and the eight accumulators meet in the
// hsum_float_8 tree at the end of the row. Only the integer lane sums are a contraction; everything after them is
// order-bound f32 work. So one MMA computes the lane sums of one block for a tile of 128 rows x 16 tokens:
//
//   A (128 x 32, s8)  = the block's weights of 128 rows (Q4_0: 16 * (nibble - 8), the factor 16 goes into the scale)
//   B (128 x 32, s8)  = for token t and accumulator n the row 8 t + n holds the four activation bytes of accumulator n
//                       at their place in the block and zeros elsewhere (block-diagonal per token)
//   D (128 x 128, s32, tensor memory) = A B^T: D[r][8 t + n] = lane sum n of (row r, token t) of this block
//
// with accumulate = 0 for every block, four D buffers in flight. The eight epilogue warps read D back with tcgen05.ld
// (lane = row, 64 columns = 8 tokens per thread), convert, and run the CPU's FMA chains in block order on 64 f32
// accumulators per thread. Operands reach shared memory by cp.async.bulk (weights in a 128-row x 1-block tile layout
// made at upload, activations as compact Q8_0 blocks); the epilogue warps also expand them into the canonical K-major
// no-swizzle operand layout (core matrices of 8 rows x 16 bytes) ahead of the MMA. Every wait is bounded.
#include "spyb_common.cuh"
#include "spyb_kernels.h"

#include <algorithm>

namespace spyb {

namespace {

constexpr int PF_M           = PF_ROWS;            // weight rows per CTA = M of the MMA
constexpr int PF_N           = 8 * PF_TOK;         // 8 accumulator columns per token
constexpr int PF_EPI_THREADS = 256;                // 8 epilogue warps: (row quadrant 0..3) x (token half 0..1)
constexpr int PF_THREADS     = PF_EPI_THREADS + 64;   // + one copy warp + one MMA warp
constexpr int PF_TILE        = PF_M * 32;          // bytes of one s8 operand tile
constexpr int PF_DBUF        = 4;                  // accumulator buffers in tensor memory, PF_N columns each (512 columns = all of it)
constexpr int PF_AHEAD       = 3;                  // blocks whose operands are expanded before their lane sums are read back
constexpr int PF_QUANT_THREADS = 512;
constexpr int PF_QUANT_GROUPS  = PF_MAX_K / (4 * PF_QUANT_THREADS);   // float4 groups per thread

// shared-memory stage of one block step
template <int WT> struct PfStage {
    static constexpr int RAW    = WT == 2 ? 2304 : 4352;           // the weight tile as it lies in HBM (Q8_0: already the A operand)
    static constexpr int SC_OFF = WT == 2 ? 2048 : 4096;           // its 128 fp16 scales
    static constexpr int YQ_OFF = RAW;                             // 16 tokens x 32 s8, then 16 f32 scales
    static constexpr int A_OFF  = WT == 2 ? RAW + PF_YQ_BYTES : 0;
    static constexpr int B_OFF  = WT == 2 ? A_OFF + PF_TILE : RAW + PF_YQ_BYTES;
    static constexpr int BYTES  = B_OFF + PF_TILE;
};

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// shared-memory operand descriptor: K-major, no swizzle; element (row r, byte k) of the tile lies at
// (r / 8) * 256 + (k / 16) * 128 + (r % 8) * 16 + k % 16: leading (K-chunk) offset 128, stride (8-row group) offset 256
__device__ __forceinline__ uint64_t operand_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(128u >> 4) << 16) | ((uint64_t)(256u >> 4) << 32) | (1ull << 46);
}
// instruction descriptor: D s32, A and B s8 K-major, N = 128, M = 128
constexpr uint32_t PF_IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(PF_N >> 3) << 17) | ((uint32_t)(PF_M >> 4) << 24);

__device__ __forceinline__ void mma_s8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc) {
    const uint32_t zero = 0;
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(PF_IDESC), "r"(zero), "r"(zero) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
                   "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
                   "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void pf_report(int *error_flag, int code) {
    if (error_flag != nullptr) { atomicExch(error_flag, code); }
}

// ---------------------------------------------------------------------------------------------
// the GEMM. grid = (row tiles, token tiles); one CTA per SM (it takes all 512 tensor-memory columns).
template <int WT>
__global__ void __launch_bounds__(PF_THREADS, 1) prefill_gemm_kernel(PrefillGemm g, int NS) {
    using S = PfStage<WT>;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bars  = sbase + (uint32_t)NS * S::BYTES;
    auto stage    = [&](int s) { return sbase + (uint32_t)s * S::BYTES; };
    auto raw_full = [&](int s) { return bars + 8u * s; };                        // weights and activations of the stage have landed
    auto ops_full = [&](int s) { return bars + 8u * (NS + s); };                 // both operand tiles are written (256 arrivals)
    auto st_free  = [&](int s) { return bars + 8u * (2 * NS + s); };             // the stage may be refilled (256 arrivals)
    auto d_full   = [&](int i) { return bars + 8u * (3 * NS + i); };             // the MMA into buffer i has completed
    auto d_free   = [&](int i) { return bars + 8u * (3 * NS + PF_DBUF + i); };   // buffer i has been read back (256 arrivals)
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + (size_t)NS * S::BYTES + 8 * (3 * NS + 2 * PF_DBUF));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nb = g.nb;
    const uint64_t limit = g.wait_limit_ns;
    const uint8_t *wsrc = g.w + ((int64_t)blockIdx.x * nb) * S::RAW;
    const uint8_t *ysrc = g.yq + ((int64_t)blockIdx.y * nb) * PF_YQ_BYTES;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) { mbar_init(raw_full(s), 1); mbar_init(ops_full(s), PF_EPI_THREADS); mbar_init(st_free(s), PF_EPI_THREADS); }
        for (int i = 0; i < PF_DBUF; ++i) { mbar_init(d_full(i), 1); mbar_init(d_free(i), PF_EPI_THREADS); }
        mbar_init_fence();
    }
    // the B tiles are zero except where the expansion writes, and it writes the same places for every block
    for (int i = tid; i < NS * (PF_TILE / 16); i += PF_THREADS) {
        sts128(stage(i / (PF_TILE / 16)) + S::B_OFF + (uint32_t)(i % (PF_TILE / 16)) * 16u, make_uint4(0u, 0u, 0u, 0u));
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(PF_DBUF * PF_N) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == PF_EPI_THREADS / 32) {
        // ---- copy warp: one thread streams the stages
        if (lane == 0) {
            int issued = 0;
            for (int b = 0; b < nb; ++b) {
                const int s = b % NS;
                if (b >= NS && !mbar_wait_bounded(st_free(s), (uint32_t)((b / NS) - 1) & 1u, limit)) { pf_report(g.error_flag, 4); break; }
                mbar_expect_tx(raw_full(s), (uint32_t)(S::RAW + PF_YQ_BYTES));
                bulk_copy_g2s(stage(s), wsrc + (int64_t)b * S::RAW, (uint32_t)S::RAW, raw_full(s));
                bulk_copy_g2s(stage(s) + S::YQ_OFF, ysrc + (int64_t)b * PF_YQ_BYTES, (uint32_t)PF_YQ_BYTES, raw_full(s));
                issued = b + 1;
            }
            // no copy of this CTA is in flight when it leaves
            for (int b = max(0, issued - NS); b < issued; ++b) {
                if (!mbar_wait_bounded(raw_full(b % NS), (uint32_t)(b / NS) & 1u, limit)) { pf_report(g.error_flag, 4); break; }
            }
        }
    } else if (warp == PF_EPI_THREADS / 32 + 1) {
        // ---- MMA warp: one thread issues one 128 x 128 x 32 MMA per block
        if (lane == 0) {
            int issued = 0;
            for (int b = 0; b < nb; ++b) {
                const int s = b % NS, buf = b % PF_DBUF;
                if (!mbar_wait_bounded(ops_full(s), (uint32_t)(b / NS) & 1u, limit)) { pf_report(g.error_flag, 5); break; }
                if (b >= PF_DBUF && !mbar_wait_bounded(d_free(buf), (uint32_t)((b / PF_DBUF) - 1) & 1u, limit)) { pf_report(g.error_flag, 5); break; }
                tc_fence_after();
                mma_s8_ss(tmem + (uint32_t)(buf * PF_N), operand_desc(stage(s) + S::A_OFF), operand_desc(stage(s) + S::B_OFF));
                mma_commit(d_full(buf));
                issued = b + 1;
            }
            // every MMA has completed (it reads shared memory and writes tensor memory) before the CTA leaves
            if (issued > 0) {
                const int b = issued - 1;
                if (!mbar_wait_bounded(d_full(b % PF_DBUF), (uint32_t)(b / PF_DBUF) & 1u, limit)) { pf_report(g.error_flag, 5); }
            }
        }
    } else {
        // ---- epilogue warps: expand operands ahead, read the lane sums back, run the f32 chains
        const int quad = warp & 3, half = warp >> 2;
        const int row = 32 * quad + lane;
        float acc[8][8];
#pragma unroll
        for (int t = 0; t < 8; ++t) {
#pragma unroll
            for (int n = 0; n < 8; ++n) { acc[t][n] = 0.f; }
        }
        auto expand = [&](int b) -> bool {
            const int s = b % NS;
            bool ok = mbar_wait_bounded(raw_full(s), (uint32_t)(b / NS) & 1u, limit);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { return false; }
            const uint32_t st = stage(s);
            if (WT == 2) {   // nibbles (stored XOR 8) -> 16 * (value - 8) as s8: low nibbles are elements 0..15, high nibbles 16..31
                const uint4 w = lds128(st + (uint32_t)row * 16u);
                uint4 o;
                if (half == 0) { o.x = (w.x << 4) & 0xf0f0f0f0u; o.y = (w.y << 4) & 0xf0f0f0f0u; o.z = (w.z << 4) & 0xf0f0f0f0u; o.w = (w.w << 4) & 0xf0f0f0f0u; }
                else           { o.x = w.x & 0xf0f0f0f0u; o.y = w.y & 0xf0f0f0f0u; o.z = w.z & 0xf0f0f0f0u; o.w = w.w & 0xf0f0f0f0u; }
                sts128(st + S::A_OFF + (uint32_t)(row >> 3) * 256u + (uint32_t)half * 128u + (uint32_t)(row & 7) * 16u, o);
            }
            if (tid < PF_TOK * 8) {   // word w of token tt -> row 8 tt + w of B, at its own place in the block
                const int tt = tid >> 3, w = tid & 7;
                const uint32_t v = lds32(st + S::YQ_OFF + (uint32_t)tt * 32u + (uint32_t)w * 4u);
                sts32(st + S::B_OFF + (uint32_t)tt * 256u + (uint32_t)(w >> 2) * 128u + (uint32_t)w * 16u + (uint32_t)(w & 3) * 4u, v);
            }
            fence_async_smem();
            mbar_arrive(ops_full(s));
            return true;
        };
        bool ok = true;
        for (int b = 0; b < PF_AHEAD && b < nb && ok; ++b) { ok = expand(b); }
        for (int b = 0; b < nb && ok; ++b) {
            if (b + PF_AHEAD < nb) { ok = expand(b + PF_AHEAD); if (!ok) { break; } }
            const int s = b % NS, buf = b % PF_DBUF;
            ok = mbar_wait_bounded(d_full(buf), (uint32_t)(b / PF_DBUF) & 1u, limit);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { break; }
            tc_fence_after();
            uint32_t r[64];
            const uint32_t taddr = tmem + ((uint32_t)(32 * quad) << 16) + (uint32_t)(buf * PF_N + 64 * half);
            tmem_ld32(taddr, r);
            tmem_ld32(taddr + 32u, r + 32);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(d_free(buf));
            const uint32_t st = stage(s);
            float dw = h2f((uint16_t)lds16(st + S::SC_OFF + 2u * (uint32_t)row));
            if (WT == 2) { dw = __fmul_rn(dw, 0.0625f); }   // exact: undoes the factor 16 of the nibble trick
            const float4 dxa = lds128f(st + S::YQ_OFF + PF_TOK * 32 + 32u * (uint32_t)half);
            const float4 dxb = lds128f(st + S::YQ_OFF + PF_TOK * 32 + 32u * (uint32_t)half + 16u);
            const float dx[8] = {dxa.x, dxa.y, dxa.z, dxa.w, dxb.x, dxb.y, dxb.z, dxb.w};
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                const float sc = __fmul_rn(dw, dx[t]);
#pragma unroll
                for (int n = 0; n < 8; ++n) { acc[t][n] = fmaf(sc, __int2float_rn((int)r[8 * t + n]), acc[t][n]); }
            }
            mbar_arrive(st_free(s));
        }
        if (!ok) { pf_report(g.error_flag, 6); }
        else {
            // hsum_float_8 (vec_util.h:74-81): column n < 4 is accumulator 4 + n for Q4_0 (low nibbles) and accumulator n for Q8_0;
            // either way the tree is (c0 + c4) + (c2 + c6) and (c1 + c5) + (c3 + c7)
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                const int token = blockIdx.y * PF_TOK + 8 * half + t;
                if (token < g.T) {
                    const float r0 = __fadd_rn(acc[t][0], acc[t][4]), r1 = __fadd_rn(acc[t][1], acc[t][5]);
                    const float r2 = __fadd_rn(acc[t][2], acc[t][6]), r3 = __fadd_rn(acc[t][3], acc[t][7]);
                    const float v = __fadd_rn(__fadd_rn(r0, r2), __fadd_rn(r1, r3));
                    const int64_t i = (int64_t)token * g.out_stride + (int64_t)blockIdx.x * PF_M + row;
                    g.out[i] = g.resid != nullptr ? __fadd_rn(v, g.resid[i]) : v;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(PF_DBUF * PF_N) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// activations of T tokens -> compact Q8_0 blocks grouped by (token tile, block): [T/16][nb][16 x 32 s8 | 16 f32 scales].
// One CTA per token; RMSNorm and the quantizer as in the mat-vec prologue (NormRMS, backend/host/operator/non-linear.cpp:194-223:
// groups of four squares formed in parallel, the running sum on one thread; Quantizator<FP32,Q8_0>, simd/vec_convert.h:178-261).
template <bool NORM>
__global__ void __launch_bounds__(PF_QUANT_THREADS) prefill_quant_kernel(const float *x, int64_t x_stride, int K, const float *norm_w, float eps, uint8_t *yq) {
    extern __shared__ __align__(16) float v3[];
    __shared__ float scale_s;
    const int tid = threadIdx.x, token = blockIdx.x;
    const int n4 = K >> 2, nb = K >> 5;
    const int npass = (n4 + PF_QUANT_THREADS - 1) / PF_QUANT_THREADS;
    const float4 *x4 = reinterpret_cast<const float4 *>(x + (int64_t)token * x_stride);
    float4 xv[PF_QUANT_GROUPS];
#pragma unroll
    for (int k = 0; k < PF_QUANT_GROUPS; ++k) {
        const int gi = tid + k * PF_QUANT_THREADS;
        xv[k] = (k < npass && gi < n4) ? x4[gi] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (NORM) {
        const float4 *w4 = reinterpret_cast<const float4 *>(norm_w);
        float4 wv[PF_QUANT_GROUPS];
#pragma unroll
        for (int k = 0; k < PF_QUANT_GROUPS; ++k) {
            const int gi = tid + k * PF_QUANT_THREADS;
            if (k < npass && gi < n4) {
                const float4 v = xv[k];
                v3[gi] = __fadd_rn(fmaf(v.y, v.y, __fmul_rn(v.x, v.x)), fmaf(v.w, v.w, __fmul_rn(v.z, v.z)));
                wv[k] = w4[gi];
            } else { wv[k] = make_float4(0.f, 0.f, 0.f, 0.f); }
        }
        __syncthreads();
        if (tid == 0) {
            float sum = 0.f;
            const float4 *g4 = reinterpret_cast<const float4 *>(v3);
            int gi = 0;
            for (; gi + 4 <= n4; gi += 4) {
                const float4 q = g4[gi >> 2];
                sum = __fadd_rn(sum, q.x); sum = __fadd_rn(sum, q.y); sum = __fadd_rn(sum, q.z); sum = __fadd_rn(sum, q.w);
            }
            for (; gi < n4; ++gi) { sum = __fadd_rn(sum, v3[gi]); }
            scale_s = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum, (float)K), eps)));
        }
        __syncthreads();
        const float scale = scale_s;
#pragma unroll
        for (int k = 0; k < PF_QUANT_GROUPS; ++k) {
            xv[k].x = __fmul_rn(__fmul_rn(xv[k].x, scale), wv[k].x);
            xv[k].y = __fmul_rn(__fmul_rn(xv[k].y, scale), wv[k].y);
            xv[k].z = __fmul_rn(__fmul_rn(xv[k].z, scale), wv[k].z);
            xv[k].w = __fmul_rn(__fmul_rn(xv[k].w, scale), wv[k].w);
        }
    }
    uint8_t *tile = yq + ((int64_t)(token / PF_TOK) * nb) * PF_YQ_BYTES;
    const int tt = token % PF_TOK;
#pragma unroll
    for (int k = 0; k < PF_QUANT_GROUPS; ++k) {
        if (k < npass) {   // uniform over the CTA: the quantizer's shuffles see full warps
            const int gi = tid + k * PF_QUANT_THREADS;
            uint16_t dh; int sum;
            const uint32_t q = quantize_q8_lane4(xv[k], dh, sum);
            if (gi < n4) {
                const int b = gi >> 3, w = gi & 7;
                uint8_t *blk = tile + (int64_t)b * PF_YQ_BYTES;
                reinterpret_cast<uint32_t *>(blk + tt * 32)[w] = q;
                if (w == 0) { reinterpret_cast<float *>(blk + PF_TOK * 32)[tt] = h2f(dh); }
            }
        }
    }
}

// upload-time re-layout: raw 18-byte / 34-byte blocks of rows [0, n_rows) -> tiles of 128 rows x 1 block
//   Q4_0: [128 rows][16 nibble bytes XOR 0x88] then [128] fp16 scales              (2304 bytes)
//   Q8_0: the s8 operand tile itself (core matrices of 8 rows x 16 bytes) then the scales   (4352 bytes)
template <int WT>
__global__ void prefill_retile_kernel(const uint8_t *raw, int64_t row_stride, int64_t n_rows, int nb, uint8_t *base, int64_t dst_row0) {
    using S = PfStage<WT>;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows * nb) { return; }
    const int64_t lrow = i / nb;
    const int     b = (int)(i - lrow * nb);
    const uint8_t *src = raw + lrow * row_stride + (int64_t)b * (WT == 2 ? 18 : 34);
    const int64_t row = dst_row0 + lrow;
    const int     r = (int)(row % PF_M);
    uint8_t *tile = base + ((row / PF_M) * nb + b) * (int64_t)S::RAW;
    reinterpret_cast<uint16_t *>(tile + S::SC_OFF)[r] = (uint16_t)(src[0] | (src[1] << 8));
    constexpr int WORDS = WT == 2 ? 4 : 8;
#pragma unroll
    for (int k = 0; k < WORDS; ++k) {
        uint32_t v = (uint32_t)(src[2 + 4 * k] | (src[3 + 4 * k] << 8) | (src[4 + 4 * k] << 16) | ((uint32_t)src[5 + 4 * k] << 24));
        if (WT == 2) { reinterpret_cast<uint32_t *>(tile + r * 16)[k] = v ^ 0x88888888u; }
        else         { reinterpret_cast<uint32_t *>(tile + (r >> 3) * 256 + (k >> 2) * 128 + (r & 7) * 16)[k & 3] = v; }
    }
}

// RoPE(Q, K) + fp16 stores of Q / K / V after the QKV GEMM (the arithmetic of the mat-vec epilogue EPI_QKV_ROPE:
// backend/host/operator/non-linear.cpp:270-371, view.cpp:163-191). One thread per pair of neighbouring elements.
__global__ void prefill_qkv_post_kernel(const float *qkv, int T, int dl, int hd, const int *pos_base, const float2 *rope, __half *q_out, __half *k_cache,
                                        __half *v_cache, int n_ctx) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t per_token = 3 * (int64_t)dl / 2;
    if (i >= per_token * T) { return; }
    const int t = (int)(i / per_token);
    const int64_t col = 2 * (i - (int64_t)t * per_token);
    const int sec = (int)(col / dl), e = (int)(col - (int64_t)sec * dl);
    const int pos = *pos_base + t;
    const float2 x = *reinterpret_cast<const float2 *>(qkv + (int64_t)t * 3 * dl + col);
    if (sec == 2) {
        v_cache[(int64_t)e * n_ctx + pos] = __float2half_rn(x.x);
        v_cache[(int64_t)(e + 1) * n_ctx + pos] = __float2half_rn(x.y);
        return;
    }
    const float2 cs = rope[(int64_t)pos * (hd >> 1) + ((e % hd) >> 1)];
    const float a0 = __fsub_rn(__fmul_rn(x.x, cs.x), __fmul_rn(x.y, cs.y));
    const float a1 = __fadd_rn(__fmul_rn(x.x, cs.y), __fmul_rn(x.y, cs.x));
    __half *dst = (sec == 0) ? q_out + (int64_t)t * dl + e : k_cache + (int64_t)pos * dl + e;
    *reinterpret_cast<__half2 *>(dst) = __halves2half2(__float2half_rn(a0), __float2half_rn(a1));
}

// up * silu(gate) (model/src/llm/plugin/ffn.cpp:28-35) on the output [T][2 F] of the stacked up|gate GEMM
__global__ void prefill_silu_mul_kernel(const float *upgate, int T, int F, const float *silu_table, float *act) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)T * F) { return; }
    const int t = (int)(i / F);
    const int64_t f = i - (int64_t)t * F;
    const float up = upgate[(int64_t)t * 2 * F + f], gate = upgate[(int64_t)t * 2 * F + F + f];
    act[i] = __fmul_rn(up, silu_table[f2h(gate)]);
}

template <int WT> size_t pf_smem_bytes(int NS) { return (size_t)NS * PfStage<WT>::BYTES + 8 * (3 * NS + 2 * PF_DBUF) + 16; }

template <int WT>
cudaError_t launch_gemm_t(const PrefillGemm &g, cudaStream_t stream) {
    int NS = 12;
    if (g.stages > PF_AHEAD + 1 && g.stages <= 16) { NS = g.stages; }
    const size_t smem = pf_smem_bytes<WT>(NS);
    cudaError_t err = allow_dynamic_smem(reinterpret_cast<const void *>(prefill_gemm_kernel<WT>), smem);
    if (err != cudaSuccess) { return err; }
    const dim3 grid((unsigned)(g.n_rows / PF_M), (unsigned)((g.T + PF_TOK - 1) / PF_TOK));
    prefill_gemm_kernel<WT><<<grid, PF_THREADS, smem, stream>>>(g, NS);
    return cudaGetLastError();
}

}  // namespace

size_t prefill_weight_bytes(int type, int64_t n_rows, int nb) { return (size_t)(n_rows / PF_ROWS) * nb * (type == 2 ? PfStage<2>::RAW : PfStage<8>::RAW); }
size_t prefill_act_bytes(int T, int nb) { return (size_t)((T + PF_TOK - 1) / PF_TOK) * nb * PF_YQ_BYTES; }

cudaError_t launch_prefill_retile(int type, const uint8_t *raw, int64_t row_stride, int64_t n_rows, int nb, uint8_t *base, int64_t dst_row0, cudaStream_t stream) {
    if ((type != 2 && type != 8) || n_rows < 1 || nb < 1) { return cudaErrorInvalidValue; }
    const int64_t n = n_rows * nb;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (type == 2) { prefill_retile_kernel<2><<<blocks, 256, 0, stream>>>(raw, row_stride, n_rows, nb, base, dst_row0); }
    else           { prefill_retile_kernel<8><<<blocks, 256, 0, stream>>>(raw, row_stride, n_rows, nb, base, dst_row0); }
    return cudaGetLastError();
}

cudaError_t launch_prefill_quant(const float *x, int64_t x_stride, int T, int K, const float *norm_w, float eps, uint8_t *yq, cudaStream_t stream) {
    if (T < 1 || K < 32 || (K & 31) || K > PF_MAX_K || (x_stride & 3) || ((uintptr_t)x & 15)) { return cudaErrorInvalidValue; }
    const size_t smem = norm_w != nullptr ? (size_t)K : 0;   // K / 4 floats
    if (norm_w != nullptr) { prefill_quant_kernel<true><<<T, PF_QUANT_THREADS, smem, stream>>>(x, x_stride, K, norm_w, eps, yq); }
    else                   { prefill_quant_kernel<false><<<T, PF_QUANT_THREADS, 0, stream>>>(x, x_stride, K, nullptr, 0.f, yq); }
    return cudaGetLastError();
}

cudaError_t launch_prefill_gemm(const PrefillGemm &g, cudaStream_t stream) {
    if (g.w == nullptr || g.yq == nullptr || g.out == nullptr || g.T < 1 || g.nb < 1 || g.n_rows < PF_ROWS || g.n_rows % PF_ROWS != 0) { return cudaErrorInvalidValue; }
    if (g.type == 2) { return launch_gemm_t<2>(g, stream); }
    if (g.type == 8) { return launch_gemm_t<8>(g, stream); }
    return cudaErrorInvalidValue;
}

cudaError_t launch_prefill_qkv_post(const float *qkv, int T, int dl, int hd, const int *pos_base, const float2 *rope, __half *q_out, __half *k_cache,
                                    __half *v_cache, int n_ctx, cudaStream_t stream) {
    const int64_t n = 3 * (int64_t)dl / 2 * T;
    prefill_qkv_post_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(qkv, T, dl, hd, pos_base, rope, q_out, k_cache, v_cache, n_ctx);
    return cudaGetLastError();
}

cudaError_t launch_prefill_silu_mul(const float *upgate, int T, int F, const float *silu_table, float *act, cudaStream_t stream) {
    const int64_t n = (int64_t)T * F;
    prefill_silu_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(upgate, T, F, silu_table, act);
    return cudaGetLastError();
}

}  // namespace spyb
