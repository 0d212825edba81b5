// Prompt evaluation as a dequant-fused GEMM on the 5th-generation tensor cores (tcgen05, accumulators in tensor memory).
//
// The reference evaluates MatMul(W[Q4_0 | Q8_0], x) for a prompt of T tokens as T independent dot products per row
// (backend/host/operator/mat.cpp:95-128 with Dot<Q4_0,Q8_0> / Dot<Q8_0,Q8_0>, backend/host/include/simd/vec_dot.h:42-115):
// per 32-element block the eight integer "lane sums" (4 products each) are converted to f32 and folded into eight f32
// accumulators with acc = fma(d_w * d_x, lane_sum, acc), block after block, and the eight accumulators meet in the
// hsum_float_8 tree at the end of the row. Only the integer lane sums are a contraction; everything after them is
// order-bound f32 work. So the tensor core computes the lane sums of one block for a tile of 128 rows x 16 tokens:
//
//   A (128 x 32)  = the block's weights of 128 rows
//   B (128 x 32)  = for token t and accumulator n the row 8 t + n holds the four activation bytes of accumulator n
//                   at their place in the block and zeros elsewhere (block-diagonal per token)
//   D (128 x 128, tensor memory) = A B^T: D[r][8 t + n] = lane sum n of (row r, token t) of this block
//
// with e4m3 operands and f32 accumulators (tcgen05.mma kind::f8f6f4), four D buffers in flight. Small integers are exact in
// e4m3: a Q4_0 weight nibble - 8 directly; an 8-bit value y (an activation byte, a Q8_0 weight) as the sum of two e4m3 values,
// y - (y mod 16) and y mod 16. So a block takes two MMAs (Q4_0) or four (Q8_0: weights split as well) onto the same buffer,
// the first with accumulate = 0. Every product and every sum of a lane's four products are integers below 2^17, exact in
// f32, so D holds (float)lane_sum itself: no conversion, no preset, and a buffer is free for the next MMA as soon as it has
// been read. (The K-quant kernel of spyb_prefill_kq.cu keeps an s8 / s32 form for Q6_K, whose values do not fit.)
// The epilogue warps read D back with tcgen05.ld (lane = row) and run the CPU's FMA chains in block order on f32 accumulators
// held as packed f32x2 pairs. Operands reach shared memory by cp.async.bulk (weights in a 128-row x 1-block tile layout
// made at upload, activations as compact blocks); an expander warp writes the activations into the canonical K-major
// no-swizzle operand layout (core matrices of 8 rows x 16 bytes) ahead of the MMA. Every wait is bounded.
#include "spyb_tc.cuh"

#include <algorithm>

namespace spyb {

namespace {

constexpr int PF_N           = 8 * PF_TOK;         // 8 accumulator columns per token
static_assert(PF_N == PF_NCOL, "16 tokens x 8 accumulators fill the MMA's columns");
constexpr int PF_QUANT_THREADS = 512;
constexpr int PF_QUANT_GROUPS  = PF_MAX_K / (4 * PF_QUANT_THREADS);   // float4 groups per thread

// ---------------------------------------------------------------------------------------------
// the GEMM. grid = (token tiles, row tiles); one CTA per SM (it takes all 512 tensor-memory columns).
//
// 20 warps (96 registers):
// warps 0-15  epilogue - row = 32 (warp % 4) + lane, tokens 4 (warp / 4) .. + 3 of the tile; four warps per scheduler hide the
//             latency of tensor memory behind one another's f32 chains
// warp 16     its first thread streams batches of PF_BATCH blocks with cp.async.bulk: two copies per batch (the weight tiles,
//             which arrive as A operands, and the compact activations) - issuing a bulk copy costs its thread hundreds of cycles
// warp 17     expands the compact activations of a batch into the B operands
// warps 18-19 their first threads issue the MMAs of alternate blocks (MMAs and commit hold the issuing thread for hundreds
//             of cycles; threads of different warps issue in parallel)
//
// Shared memory: rings of NS blocks (NQ batches), one ring per kind so that a batch is one contiguous run:
//   A ring  [NS][4352 | 8448]   weight tiles (one or two A operands + 128 fp16 scales), written by cp.async.bulk
//   Y ring  [NS][1088]          compact activations (two e4m3 planes of 16 tokens x 32 codes; 16 f32 scales)
//   B ring  [NS][8192]          expanded activations (two B operands), written by the expander warp
template <int WT> struct PfGeom {
    static constexpr int  NA      = WT == 8 ? 2 : 1;                       // A operands per block: Q8_0 weights are split like the activations
    static constexpr int  WTILE   = NA * PF_TILE + 256;                    // a weight tile in HBM: the A operand(s) of 128 rows x 32 e4m3 codes, then 128 fp16 block scales
    static constexpr int  YQ      = PF_YQ_BYTES_F8;                        // a block's compact activations
    static constexpr int  BT      = 2 * PF_TILE;                           // a block's two B operands
    static constexpr int  NQ      = WT == 8 ? 3 : PF_RING;                 // batches in the rings (what fits the shared memory)
    static constexpr int  NS      = NQ * PF_BATCH;                         // blocks in the rings
    static constexpr int  EPI_W   = PF_EPI_WARPS_F8;
    static constexpr int  MMA_W   = PF_MMA_WARPS_F8;
    static constexpr int  THREADS = PF_THREADS_F8;
    static constexpr size_t SMEM  = (size_t)NS * (WTILE + YQ + BT) + 8 * (3 * NQ + 2 * PF_DBUF) + 16;
};

template <int WT>
__global__ void __launch_bounds__(PfGeom<WT>::THREADS, 1) prefill_gemm_kernel(PrefillGemm g) {
    constexpr int NS = PfGeom<WT>::NS, NQ = PfGeom<WT>::NQ, NA = PfGeom<WT>::NA, PF_WTILE = PfGeom<WT>::WTILE;
    constexpr int YQ = PfGeom<WT>::YQ, BT = PfGeom<WT>::BT, EPI_W = PfGeom<WT>::EPI_W, MMA_W = PfGeom<WT>::MMA_W, THREADS = PfGeom<WT>::THREADS;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    const uint32_t a_ring = sbase, y_ring = a_ring + NS * PF_WTILE, b_ring = y_ring + NS * YQ;
    const uint32_t bars  = b_ring + NS * BT;
    auto raw_full = [&](int q) { return bars + 8u * q; };                        // the batch's weights and activations have landed
    auto ops_full = [&](int q) { return bars + 8u * (NQ + q); };                 // the batch's B operands are written and fenced
    auto st_free  = [&](int q) { return bars + 8u * (2 * NQ + q); };             // the batch's stages may be refilled (one arrival per epilogue warp)
    auto d_full   = [&](int i) { return bars + 8u * (3 * NQ + i); };             // the MMA into buffer i has completed
    auto d_free   = [&](int i) { return bars + 8u * (3 * NQ + PF_DBUF + i); };   // buffer i has been read (one arrival per epilogue warp)
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + (size_t)NS * (PF_WTILE + YQ + BT) + 8 * (3 * NQ + 2 * PF_DBUF));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nb = g.nb, n_batch = (nb + PF_BATCH - 1) / PF_BATCH;
    const uint64_t limit = g.wait_limit_ns;
    const int row_tile = blockIdx.y, tok_tile = blockIdx.x;   // CTAs that run together share a weight tile: it crosses HBM once
    const uint8_t *wsrc = g.w + ((int64_t)row_tile * nb) * PF_WTILE;
    const uint8_t *ysrc = g.yq + ((int64_t)tok_tile * nb) * YQ;

    if (tid == 0) {
        for (int q = 0; q < NQ; ++q) { mbar_init(raw_full(q), 1); mbar_init(ops_full(q), 1); mbar_init(st_free(q), EPI_W); }
        for (int i = 0; i < PF_DBUF; ++i) { mbar_init(d_full(i), 1); mbar_init(d_free(i), EPI_W); }
        mbar_init_fence();
    }
    // the B tiles are zero except where the expansion writes, and it writes the same places for every block
    for (int i = tid; i < NS * (BT / 16); i += THREADS) { sts128(b_ring + (uint32_t)i * 16u, make_uint4(0u, 0u, 0u, 0u)); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(PF_DBUF * PF_N) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp >= EPI_W + 2) {
        // ---- MMA warps: the first thread of warp m issues the 128 x 128 x 32 MMAs of blocks m, m + MMA_W, ... onto a buffer
        // the epilogue has read; MMAs into different buffers do not depend on one another
        if (lane == 0) {
            int last = -1;
            for (int b = warp - (EPI_W + 2); b < nb; b += MMA_W) {
                const int s = b % NS, q = b / PF_BATCH, buf = b % PF_DBUF;
                PF_STAMP(2, b, 0);
                if (!mbar_wait_relaxed(ops_full(q % NQ), (uint32_t)(q / NQ) & 1u, limit)) { pf_report(g.error_flag, 5); break; }
                PF_STAMP(2, b, 1);
                if (!mbar_wait_relaxed(d_free(buf), (uint32_t)(b / PF_DBUF) & 1u, limit)) { pf_report(g.error_flag, 5); break; }
                PF_STAMP(2, b, 2);
                tc_fence_after();
                // the e4m3 parts of the activation bytes (and of Q8_0 weights), one product after the other onto the same accumulators
                const uint32_t d_tmem = tmem + (uint32_t)(buf * PF_N);
                const uint64_t b_hi = operand_desc(b_ring + (uint32_t)s * BT), b_lo = operand_desc(b_ring + (uint32_t)s * BT + PF_TILE);
#pragma unroll
                for (int a = 0; a < NA; ++a) {
                    const uint64_t a_desc = operand_desc(a_ring + (uint32_t)s * PF_WTILE + (uint32_t)a * PF_TILE);
                    mma_f8_ss(d_tmem, a_desc, b_hi, a == 0 ? 0u : 1u);
                    mma_f8_ss(d_tmem, a_desc, b_lo, 1u);
                }
                mma_commit(d_full(buf));
                PF_STAMP(2, b, 3);
                last = b;
            }
            // every MMA has completed (it reads shared memory and writes tensor memory) before the CTA leaves
            if (last >= 0 && !mbar_wait_relaxed(d_full(last % PF_DBUF), (uint32_t)(last / PF_DBUF) & 1u, limit)) { pf_report(g.error_flag, 5); }
        }
    } else if (warp == EPI_W) {
        // ---- copy warp: one thread requests batch after batch
        if (lane == 0) {
            int issued = 0;
            for (int q = 0; q < n_batch; ++q) {
                if (q == g.selftest_skip_batch) { issued = q + 1; continue; }   // (failure-path check: this batch never arrives)
                if (q >= NQ && !mbar_wait_relaxed(st_free(q % NQ), (uint32_t)((q / NQ) - 1) & 1u, limit)) { pf_report(g.error_flag, 4); break; }
                const int b0 = q * PF_BATCH, n = min(PF_BATCH, nb - b0), s0 = b0 % NS;
                PF_STAMP(0, b0, 0);
                mbar_expect_tx(raw_full(q % NQ), (uint32_t)(n * (PF_WTILE + YQ)));
                bulk_copy_g2s(a_ring + (uint32_t)s0 * PF_WTILE, wsrc + (int64_t)b0 * PF_WTILE, (uint32_t)(n * PF_WTILE), raw_full(q % NQ));
                bulk_copy_g2s(y_ring + (uint32_t)s0 * YQ, ysrc + (int64_t)b0 * YQ, (uint32_t)(n * YQ), raw_full(q % NQ));
                issued = q + 1;
            }
            // no copy of this CTA is in flight when it leaves
            for (int q = max(0, issued - NQ); q < issued; ++q) {
                if (!mbar_wait_relaxed(raw_full(q % NQ), (uint32_t)(q / NQ) & 1u, limit)) { pf_report(g.error_flag, 4); break; }
            }
        }
    } else if (warp == EPI_W + 1) {
        // ---- expander warp: word w of token tt of the compact activations -> row 8 tt + w of B, at its own place in the
        // block (the rest of B stays zero); one proxy fence per batch makes the writes visible to the tensor core
        for (int q = 0; q < n_batch; ++q) {
            bool ok = mbar_wait_relaxed(raw_full(q % NQ), (uint32_t)(q / NQ) & 1u, limit);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { if (lane == 0) { pf_report(g.error_flag, 4); } break; }
            const int b0 = q * PF_BATCH, n = min(PF_BATCH, nb - b0), s0 = b0 % NS;
            if (lane == 0) { PF_STAMP(1, b0, 0); }
            for (int j = 0; j < n; ++j) {
                const uint32_t ysrc_s = y_ring + (uint32_t)(s0 + j) * YQ, bdst = b_ring + (uint32_t)(s0 + j) * BT;
                constexpr int NW = 2 * PF_TOK * 8 / 32;   // words per lane (the second plane of words goes to the second B operand)
                uint32_t v[NW];
#pragma unroll
                for (int k = 0; k < NW; ++k) { v[k] = lds32(ysrc_s + (uint32_t)(lane + 32 * k) * 4u); }   // all loads in flight before the first store
#pragma unroll
                for (int k = 0; k < NW; ++k) {
                    const int i = lane + 32 * k, plane = i >> 7, tt = (i >> 3) & (PF_TOK - 1), w = i & 7;
                    sts32(bdst + (uint32_t)plane * PF_TILE + (uint32_t)tt * 256u + (uint32_t)(w >> 2) * 128u + (uint32_t)w * 16u + (uint32_t)(w & 3) * 4u, v[k]);
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) { mbar_arrive(ops_full(q % NQ)); PF_STAMP(1, b0, 1); }
        }
    } else {
        // ---- epilogue warps: row = 32 (warp % 4) + lane, tokens 8 (warp / 4) .. + 7 of the tile = 64 columns of D, read back 16
        // columns (two tokens) at a time into two alternating register sets: a set is requested again as soon as its values
        // have been folded, so that the tensor-memory loads overlap the f32 chains of the other set
        const int quad = warp & 3;
        const int row = 32 * quad + lane;
        const uint32_t dw_addr = a_ring + NA * PF_TILE + 2u * (uint32_t)row;
        bool ok = true;
        {
            // ---- e4m3 operands: D is f32 and holds (float)lane_sum itself, so a lane sum costs half a packed FMA. Sixteen warps:
            // warp = (row quadrant, quarter of the columns = tokens 4 part .. + 3), both halves of its 32 columns requested
            // together, so the buffer is free for the next MMA as soon as they have arrived.
            const int part = warp >> 2;
            const uint32_t tbase = tmem + ((uint32_t)(32 * quad) << 16) + (uint32_t)(32 * part);
            const uint32_t dx_addr = y_ring + 2 * PF_TOK * 32 + 16u * (uint32_t)part;
            uint64_t acc[4][4];   // [token][pair]: accumulators 2 pair and 2 pair + 1 of the token, as one packed f32x2 value
#pragma unroll
            for (int t = 0; t < 4; ++t) {
#pragma unroll
                for (int n = 0; n < 4; ++n) { acc[t][n] = 0ull; }
            }
            if (lane == 0) { for (int i = 0; i < PF_DBUF; ++i) { mbar_arrive(d_free(i)); } }
            uint32_t ra[16], rb[16];
            auto fold2 = [&](const uint32_t *r, int t0, float sa, float sb) {   // two tokens: columns 8 t0 .. 8 t0 + 15 of the warp's 32
                const uint64_t sc[2] = {f2_pack(sa, sa), f2_pack(sb, sb)};
#pragma unroll
                for (int t = 0; t < 2; ++t) {
#pragma unroll
                    for (int n = 0; n < 4; ++n) { acc[t0 + t][n] = f2_fma(sc[t], f2_pack_bits(r[8 * t + 2 * n], r[8 * t + 2 * n + 1]), acc[t0 + t][n]); }
                }
            };
            ok = mbar_wait_bounded(d_full(0), 0u, limit);
            ok = __all_sync(0xffffffffu, ok);
            if (ok) { tc_fence_after(); tmem_ld16(tbase, ra); tmem_ld16(tbase + 16u, rb); }
            static_assert(PF_BATCH == PF_DBUF, "the unrolled epilogue pairs block j of a batch with accumulator buffer j");
            for (int q = 0; q < n_batch && ok; ++q) {
                const uint32_t ring_q = (uint32_t)(q % NQ) * PF_BATCH;
                const uint32_t dw_q = dw_addr + ring_q * PF_WTILE, dx_q = dx_addr + ring_q * YQ;
#pragma unroll
                for (int j = 0; j < PF_BATCH; ++j) {
                    const int b = q * PF_BATCH + j;
                    if (b >= nb || !ok) { break; }
                    const float dw = h2f((uint16_t)lds16(dw_q + (uint32_t)j * PF_WTILE));
                    const float4 dx = lds128f(dx_q + (uint32_t)j * YQ);
                    tmem_ld_wait();                       // the warp's 32 columns of block b are in registers: the buffer has been read
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) { mbar_arrive(d_free(j)); }
                    fold2(ra, 0, __fmul_rn(dw, dx.x), __fmul_rn(dw, dx.y));
                    const bool more = b + 1 < nb;
                    const uint32_t tnext = tbase + (uint32_t)(((j + 1) % PF_DBUF) * PF_N);
                    if (more) {                           // the next block's columns arrive while the last two tokens are folded
                        ok = mbar_wait_bounded(d_full((j + 1) % PF_DBUF), (uint32_t)(q + (j + 1) / PF_DBUF) & 1u, limit);
                        ok = __all_sync(0xffffffffu, ok);
                        if (ok) { tc_fence_after(); tmem_ld16(tnext, ra); }
                    }
                    fold2(rb, 2, __fmul_rn(dw, dx.z), __fmul_rn(dw, dx.w));
                    if (more && ok) { tmem_ld16(tnext + 16u, rb); }
                    if (lane == 0 && (j == PF_BATCH - 1 || b == nb - 1)) { mbar_arrive(st_free(q % NQ)); }   // the batch's scales have been read
                }
            }
            tmem_ld_wait();
            if (!ok) { if (lane == 0) { pf_report(g.error_flag, 6); } }
            else {
#pragma unroll
                for (int t = 0; t < 4; ++t) {   // hsum_float_8 (vec_util.h:74-81): column n < 4 is accumulator 4 + n for Q4_0 (low nibbles) and accumulator n for Q8_0; either way the tree is (c0 + c4) + (c2 + c6) and (c1 + c5) + (c3 + c7)
                    const int token = tok_tile * PF_TOK + 4 * part + t;
                    if (token < g.T && (int64_t)row_tile * PF_M + row < g.n_rows) {   // (the last row tile may be partly padding)
                        float c[8];
#pragma unroll
                        for (int n = 0; n < 4; ++n) { f2_unpack(acc[t][n], c[2 * n], c[2 * n + 1]); }
                        const float r0 = __fadd_rn(c[0], c[4]), r1 = __fadd_rn(c[1], c[5]);
                        const float r2 = __fadd_rn(c[2], c[6]), r3 = __fadd_rn(c[3], c[7]);
                        const float v = __fadd_rn(__fadd_rn(r0, r2), __fadd_rn(r1, r3));
                        const int64_t i = (int64_t)token * g.out_stride + (int64_t)row_tile * PF_M + row;
                        g.out[i] = g.resid != nullptr ? __fadd_rn(v, g.resid[i]) : v;
                    }
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
// TOKT tokens per tile; YSUM: the blocks' integer sums follow the scales as floats (the K-quant kernels need them); F8: every
// activation byte as two e4m3 values (a plane of TOKT x 32 codes each: the multiple of 16 and the rest) for the Q4_0 kernel
template <bool NORM, int TOKT, bool YSUM, bool F8>
__global__ void __launch_bounds__(PF_QUANT_THREADS) prefill_quant_kernel(const float *x, int64_t x_stride, int K, const float *norm_w, float eps, uint8_t *yq,
                                                                         int part_len, int64_t part_stride) {
    constexpr int YQB = (F8 ? 2 : 1) * TOKT * 32 + TOKT * 4 * (YSUM ? 2 : 1);
    constexpr int SCALES = (F8 ? 2 : 1) * TOKT * 32;   // offset of the scales inside a block's record
    extern __shared__ __align__(16) float v3[];
    __shared__ float scale_s;
    const int tid = threadIdx.x, token = blockIdx.x;
    const int n4 = K >> 2, nb = K >> 5;
    const int npass = (n4 + PF_QUANT_THREADS - 1) / PF_QUANT_THREADS;
    // a row may lie in parts (the slices the ranks of a tensor-parallel group gathered): elements [i part_len, (i + 1) part_len)
    // of token t at x + i part_stride + t x_stride; one part = the plain row
    const float *xrow = x + (int64_t)token * x_stride;
    float4 xv[PF_QUANT_GROUPS];
#pragma unroll
    for (int k = 0; k < PF_QUANT_GROUPS; ++k) {
        const int gi = tid + k * PF_QUANT_THREADS;
        if (k < npass && gi < n4) {
            const int e = 4 * gi, part = e / part_len;
            xv[k] = *reinterpret_cast<const float4 *>(xrow + (int64_t)part * part_stride + (e - part * part_len));
        } else { xv[k] = make_float4(0.f, 0.f, 0.f, 0.f); }
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
    uint8_t *tile = yq + ((int64_t)(token / TOKT) * nb) * YQB;
    const int tt = token % TOKT;
#pragma unroll
    for (int k = 0; k < PF_QUANT_GROUPS; ++k) {
        if (k < npass) {   // uniform over the CTA: the quantizer's shuffles see full warps
            const int gi = tid + k * PF_QUANT_THREADS;
            uint16_t dh; int sum;
            const uint32_t q = quantize_q8_lane4(xv[k], dh, sum);
            if (YSUM) {   // the block's sum over its eight lanes
                sum += __shfl_xor_sync(0xffffffffu, sum, 1); sum += __shfl_xor_sync(0xffffffffu, sum, 2); sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            }
            if (gi < n4) {
                const int b = gi >> 3, w = gi & 7;
                uint8_t *blk = tile + (int64_t)b * YQB;
                if (F8) {
                    uint32_t hi, lo;
                    e4m3_split4(q, hi, lo);
                    reinterpret_cast<uint32_t *>(blk + tt * 32)[w] = hi;
                    reinterpret_cast<uint32_t *>(blk + TOKT * 32 + tt * 32)[w] = lo;
                } else {
                    reinterpret_cast<uint32_t *>(blk + tt * 32)[w] = q;
                }
                if (w == 0) {
                    reinterpret_cast<float *>(blk + SCALES)[tt] = h2f(dh);
                    if (YSUM) { reinterpret_cast<float *>(blk + SCALES + TOKT * 4)[tt] = (float)sum; }
                }
            }
        }
    }
}

// upload-time re-layout: raw 18-byte / 34-byte blocks of rows [0, n_rows) -> tiles of 128 rows x 1 block: the A operand
// (core matrices of 8 rows x 16 bytes; Q8_0: the s8 values; Q4_0: element k < 16 is the e4m3 code of (low nibble of byte k - 8),
// element 16 + k the same of the high nibble) followed by the 128 fp16 block scales
template <int WT>
__global__ void prefill_retile_kernel(const uint8_t *raw, int64_t row_stride, int64_t n_rows, int nb, uint8_t *base, int64_t dst_row0) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows * nb) { return; }
    const int64_t lrow = i / nb;
    const int     b = (int)(i - lrow * nb);
    const uint8_t *src = raw + lrow * row_stride + (int64_t)b * (WT == 2 ? 18 : 34);
    const int64_t row = dst_row0 + lrow;
    const int     r = (int)(row % PF_M);
    uint8_t *tile = base + ((row / PF_M) * nb + b) * (int64_t)PfGeom<WT>::WTILE;
    reinterpret_cast<uint16_t *>(tile + PfGeom<WT>::NA * PF_TILE)[r] = (uint16_t)(src[0] | (src[1] << 8));
    uint32_t *lo = reinterpret_cast<uint32_t *>(tile + (r >> 3) * 256 + (r & 7) * 16), *hi = lo + 32;   // elements 0..15 and 16..31
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (WT == 2) {
            uint32_t l = 0u, h = 0u;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int byte = src[2 + 4 * k + i];
                l |= e4m3_of_signed((byte & 15) - 8) << (8 * i);
                h |= e4m3_of_signed((byte >> 4) - 8) << (8 * i);
            }
            lo[k] = l;
            hi[k] = h;
        } else {   // Q8_0: every s8 weight as two e4m3 values, the multiple of 16 in the first operand tile and the rest in the second
            const uint32_t w_lo = (uint32_t)(src[2 + 4 * k] | (src[3 + 4 * k] << 8) | (src[4 + 4 * k] << 16) | ((uint32_t)src[5 + 4 * k] << 24));
            const uint32_t w_hi = (uint32_t)(src[18 + 4 * k] | (src[19 + 4 * k] << 8) | (src[20 + 4 * k] << 16) | ((uint32_t)src[21 + 4 * k] << 24));
            e4m3_split4(w_lo, lo[k], lo[k + PF_TILE / 4]);
            e4m3_split4(w_hi, hi[k], hi[k + PF_TILE / 4]);
        }
    }
}

// RoPE(Q, K) + fp16 stores of Q / K / V after the QKV GEMM (the arithmetic of the mat-vec epilogue EPI_QKV_ROPE:
// backend/host/operator/non-linear.cpp:270-371, view.cpp:163-191). One thread per pair of neighbouring elements.
__global__ void prefill_qkv_post_kernel(const float *qkv, int T, int dl, int hd, const int *pos_base, const float2 *rope, __half *q_out, __half *k_cache,
                                        __half *v_cache, int n_ctx, int64_t seq_stride) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t per_token = 3 * (int64_t)dl / 2;
    if (i >= per_token * T) { return; }
    const int t = (int)(i / per_token);
    const int64_t col = 2 * (i - (int64_t)t * per_token);
    const int sec = (int)(col / dl), e = (int)(col - (int64_t)sec * dl);
    const int pos = *pos_base + (seq_stride ? 0 : t);   // (seq_stride > 0: token t is sequence t of a batch in lockstep, with its own cache)
    k_cache += seq_stride ? (int64_t)t * seq_stride : 0; v_cache += seq_stride ? (int64_t)t * seq_stride : 0;
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

template <int WT>
cudaError_t launch_gemm_t(const PrefillGemm &g, cudaStream_t stream) {
    const size_t smem = PfGeom<WT>::SMEM;
    cudaError_t err = allow_dynamic_smem(reinterpret_cast<const void *>(prefill_gemm_kernel<WT>), smem);
    if (err != cudaSuccess) { return err; }
    const dim3 grid((unsigned)((g.T + PF_TOK - 1) / PF_TOK), (unsigned)((g.n_rows + PF_M - 1) / PF_M));
    prefill_gemm_kernel<WT><<<grid, PfGeom<WT>::THREADS, smem, stream>>>(g);
    return cudaGetLastError();
}

}  // namespace

// host-only check of the e4m3 codes the exactness of the prompt GEMM rests on (no device needed): 0 when every code decodes
// to the integer it stands for and every 8-bit value is the sum of its two parts
int prefill_e4m3_selftest() {
    auto decode = [](uint32_t c) {   // e4m3: sign, 4 exponent bits (bias 7), 3 mantissa bits; exponent 0 = subnormal
        const int e = (int)((c >> 3) & 15u), m = (int)(c & 7u);
        const double v = e == 0 ? m / 8.0 / 64.0 : (1.0 + m / 8.0) * (double)(1 << e) / 128.0;
        return (c & 0x80u) ? -v : v;
    };
    for (int v = 0; v <= 15; ++v) { if (decode(e4m3_of_small((uint32_t)v)) != (double)v) { return 100 + v; } }
    for (int v = -15; v <= 15; ++v) { if (decode(e4m3_of_signed(v)) != (double)v) { return 200 + v + 15; } }
    for (int y = -128; y <= 127; ++y) {   // the split of e4m3_split4, one byte at a time
        const int yl = y & 15, yh = (y - yl) >> 4;
        const uint32_t ch = yh == 0 ? 0u : (e4m3_of_signed(yh) + 0x20u), cl = e4m3_of_small((uint32_t)yl);
        if (decode(ch) != 16.0 * yh || decode(cl) != (double)yl || 16 * yh + yl != y || (ch & 0x7fu) > 0x7eu) { return 1000 + y + 128; }
    }
    return 0;
}

size_t prefill_weight_bytes(int type, int64_t n_rows, int nb) {
    const size_t tile = (type == 12 || type == 14) ? (size_t)PF_KQ_WTILE : type == 8 ? (size_t)PfGeom<8>::WTILE : (size_t)PfGeom<2>::WTILE;
    return (size_t)((n_rows + PF_ROWS - 1) / PF_ROWS) * nb * tile;
}
size_t prefill_act_bytes(int T, int nb) {   // (the largest of the layouts)
    return std::max((size_t)((T + PF_TOK - 1) / PF_TOK) * nb * std::max(PF_YQ_BYTES, PF_YQ_BYTES_F8),
                    (size_t)((T + PF_KQ_TOK - 1) / PF_KQ_TOK) * nb * std::max(PF_KQ_YQ_BYTES, PF_KQ_YQ_BYTES_F8));
}

cudaError_t launch_prefill_retile(int type, const uint8_t *raw, int64_t row_stride, int64_t n_rows, int nb, uint8_t *base, int64_t dst_row0, cudaStream_t stream) {
    if (type == 12 || type == 14) { return launch_prefill_retile_kq(type, raw, row_stride, n_rows, nb, base, dst_row0, stream); }
    if ((type != 2 && type != 8) || n_rows < 1 || nb < 1) { return cudaErrorInvalidValue; }
    const int64_t n = n_rows * nb;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (type == 2) { prefill_retile_kernel<2><<<blocks, 256, 0, stream>>>(raw, row_stride, n_rows, nb, base, dst_row0); }
    else           { prefill_retile_kernel<8><<<blocks, 256, 0, stream>>>(raw, row_stride, n_rows, nb, base, dst_row0); }
    return cudaGetLastError();
}

cudaError_t launch_prefill_quant(const float *x, int64_t x_stride, int T, int K, const float *norm_w, float eps, uint8_t *yq, cudaStream_t stream, int weight_type,
                                 int part_len, int64_t part_stride) {
    if (weight_type != 2 && weight_type != 8 && weight_type != 12 && weight_type != 14) { return cudaErrorInvalidValue; }
    const bool kq_layout = weight_type == 12 || weight_type == 14;
    if (part_len <= 0) { part_len = K; part_stride = 0; }
    if ((part_len & 3) || (part_stride & 3) || K % part_len != 0) { return cudaErrorInvalidValue; }
    if (T < 1 || K < 32 || (K & 31) || K > PF_MAX_K || (x_stride & 3) || ((uintptr_t)x & 15)) { return cudaErrorInvalidValue; }
    const size_t smem = norm_w != nullptr ? (size_t)K : 0;   // K / 4 floats
    if (weight_type == 12) {
        if (norm_w != nullptr) { prefill_quant_kernel<true, PF_KQ_TOK, true, true><<<T, PF_QUANT_THREADS, smem, stream>>>(x, x_stride, K, norm_w, eps, yq, part_len, part_stride); }
        else                   { prefill_quant_kernel<false, PF_KQ_TOK, true, true><<<T, PF_QUANT_THREADS, 0, stream>>>(x, x_stride, K, nullptr, 0.f, yq, part_len, part_stride); }
    } else if (kq_layout) {
        if (norm_w != nullptr) { prefill_quant_kernel<true, PF_KQ_TOK, true, false><<<T, PF_QUANT_THREADS, smem, stream>>>(x, x_stride, K, norm_w, eps, yq, part_len, part_stride); }
        else                   { prefill_quant_kernel<false, PF_KQ_TOK, true, false><<<T, PF_QUANT_THREADS, 0, stream>>>(x, x_stride, K, nullptr, 0.f, yq, part_len, part_stride); }
    } else {   // Q4_0 and Q8_0 weights: tiles of 16 tokens, the two e4m3 planes
        if (norm_w != nullptr) { prefill_quant_kernel<true, PF_TOK, false, true><<<T, PF_QUANT_THREADS, smem, stream>>>(x, x_stride, K, norm_w, eps, yq, part_len, part_stride); }
        else                   { prefill_quant_kernel<false, PF_TOK, false, true><<<T, PF_QUANT_THREADS, 0, stream>>>(x, x_stride, K, nullptr, 0.f, yq, part_len, part_stride); }
    }
    return cudaGetLastError();
}

cudaError_t launch_prefill_gemm(const PrefillGemm &g, cudaStream_t stream) {
    if (g.type == 12 || g.type == 14) { return launch_prefill_gemm_kq(g, stream); }
    if (g.w == nullptr || g.yq == nullptr || g.out == nullptr || g.T < 1 || g.nb < 1 || g.n_rows < 1) { return cudaErrorInvalidValue; }
    if (g.type == 2) { return launch_gemm_t<2>(g, stream); }
    if (g.type == 8) { return launch_gemm_t<8>(g, stream); }
    return cudaErrorInvalidValue;
}

cudaError_t launch_prefill_qkv_post(const float *qkv, int T, int dl, int hd, const int *pos_base, const float2 *rope, __half *q_out, __half *k_cache,
                                    __half *v_cache, int n_ctx, int64_t seq_stride, cudaStream_t stream) {
    const int64_t n = 3 * (int64_t)dl / 2 * T;
    prefill_qkv_post_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(qkv, T, dl, hd, pos_base, rope, q_out, k_cache, v_cache, n_ctx, seq_stride);
    return cudaGetLastError();
}

cudaError_t launch_prefill_silu_mul(const float *upgate, int T, int F, const float *silu_table, float *act, cudaStream_t stream) {
    const int64_t n = (int64_t)T * F;
    prefill_silu_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(upgate, T, F, silu_table, act);
    return cudaGetLastError();
}

}  // namespace spyb
