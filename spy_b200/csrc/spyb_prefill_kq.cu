// Prompt evaluation for K-quant weights (Q4_K, Q6_K) as a GEMM on the tcgen05 tensor cores: the K-quant counterpart of
// spyb_prefill.cu, same roles and rings, a different tile and epilogue.
//
// Parity is unpinned by the reference (it defines the K-quant block layouts, orchestration/include/number/number_impl/
// k-quant.h:79-117, 162-188, but no arithmetic for them); what is reproduced bit for bit is the restatement the single-token
// kernel of spyb_kquant.cu follows: activations quantized to Q8_0 first, and per 256-value super-block
//   Q4_K:  acc = 0; for the 8 sub-blocks j of 32 values: acc = fma((d * sc_j) * dx_j, (float)sum(q * y), acc);
//                                                         acc = fma(-((dmin * m_j) * dx_j), (float)sum(y), acc)
//   Q6_K:  acc = 0; for the 16 groups g of 16 values:    acc = fma((d * sc_g) * dx_(g/2), (float)sum(q * y), acc)
// the row's result being the super-blocks' values added in order.
//
// One MMA (Q6_K, s8 operands) or two (Q4_K, e4m3 operands: see KqGeom) per 32-element block for a tile of 128 rows x 64 tokens:
// A = the block's integer weights (Q4_K: 0..15, Q6_K: -32..31), B = 128 x 32 s8 whose rows 2 t and 2 t + 1 hold the first and the second 16 activation bytes of token t
// at their place and zeros elsewhere (the kernel orders the columns 4 (t / 2) + 2 h + t % 2), D[r][column of (t, h)] = the integer sum of half h of the block. Q6_K folds the two halves one
// after the other with their own scales (they are two of its groups); Q4_K adds them first (exact: both are small integers).
// The weight tile carries, per row, the two f32 products the restatement forms first (Q4_K: d * sc_j and dmin * m_j;
// Q6_K: d * sc of the two groups), made at upload with the same f32 multiplication.
#include "spyb_tc.cuh"

#include <algorithm>

namespace spyb {

namespace {

constexpr int KQ_TOK = PF_KQ_TOK, KQ_WT = PF_KQ_WTILE;
static_assert(2 * KQ_TOK == PF_NCOL, "64 tokens x 2 halves fill the MMA's columns");
// Q4_K takes the e4m3 form of spyb_prefill.cu (its values 0..15 are exact in e4m3; the activation bytes as two e4m3 planes, two
// MMAs per block, f32 accumulators that hold (float)sum itself: no offset pattern, no subtraction); its larger activation
// records and B operands leave room for rings of three batches. Q6_K (-32..31 does not fit e4m3) keeps the s8 form.
template <int WT> struct KqGeom {
    static constexpr bool F8 = WT == 12;
    static constexpr int  YQ = F8 ? PF_KQ_YQ_BYTES_F8 : PF_KQ_YQ_BYTES;
    static constexpr int  BT = F8 ? 2 * PF_TILE : PF_TILE;
    static constexpr int  NQ = F8 ? 3 : PF_RING;            // batches in the rings
    static constexpr int  NS = NQ * PF_BATCH;               // blocks in the rings
    static constexpr size_t SMEM = (size_t)NS * (KQ_WT + YQ + BT) + 8 * (3 * NQ + 2 * PF_DBUF) + 16;
};

__device__ __forceinline__ float2 lds64f(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint64_t lds64u(uint32_t addr) {
    uint64_t v;
    asm volatile("ld.shared.u64 %0, [%1];" : "=l"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void lds128_2x64(uint32_t addr, uint64_t &a, uint64_t &b) {
    asm volatile("ld.shared.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "r"(addr));
}

// eight tokens (T0 .. T0 + 7 of a warp's 32) from one register set of 16 columns, two tokens per packed f32x2 operation:
// columns 4 u, 4 u + 1 hold the first-half sums of tokens T0 + 2 u and T0 + 2 u + 1, columns 4 u + 2, 4 u + 3 their second-half
// sums. `scx`, `scy` = the row's two scale products of the block, each in both halves of a pair (Q4_K: scy negated);
// dx_s = the warp's 32 activation scales of the block in shared memory (the 32 block sums lie KQ_TOK * 4 bytes further)
template <int WT, int T0>
__device__ __forceinline__ void kq_fold8(uint64_t (&acc)[16], const uint32_t (&r)[16], uint64_t scx, uint64_t scy, uint32_t dx_s, uint64_t minus_magic) {
    constexpr bool F8 = KqGeom<WT>::F8;   // the columns already hold floats
    uint64_t dx[4];
    if (WT == 14) {
        lds128_2x64(dx_s + 4u * T0, dx[0], dx[1]);
        lds128_2x64(dx_s + 4u * T0 + 16u, dx[2], dx[3]);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const uint64_t b0 = f2_pack_bits(r[4 * u], r[4 * u + 1]), b1 = f2_pack_bits(r[4 * u + 2], r[4 * u + 3]);
        const uint64_t p0 = F8 ? b0 : f2_add(b0, minus_magic), p1 = F8 ? b1 : f2_add(b1, minus_magic);
        uint64_t a = acc[T0 / 2 + u];
        if (WT == 12) { dx[u] = lds64u(dx_s + 4u * T0 + 8u * u); }   // (Q4_K also reads the block sums: fewer values live at a time)
        if (WT == 14) {
            a = f2_fma(f2_mul(scx, dx[u]), p0, a);
            a = f2_fma(f2_mul(scy, dx[u]), p1, a);
        } else {
            a = f2_fma(f2_mul(scx, dx[u]), f2_add(p0, p1), a);
            a = f2_fma(f2_mul(scy, dx[u]), lds64u(dx_s + KQ_TOK * 4 + 4u * T0 + 8u * u), a);   // scy = -(dmin * m_j): the negation commutes with the rounding of the product
        }
        acc[T0 / 2 + u] = a;
    }
}

// grid = (token tiles, row tiles); one CTA per SM. Warps 0-7 epilogue (row = 32 (warp % 4) + lane, tokens 32 (warp / 4) .. + 31
// of the tile), warp 8 copies, warp 9 expands the activations, warps 10-11 issue the MMAs - as in prefill_gemm_kernel.
template <int WT>   // 12 = Q4_K, 14 = Q6_K
__global__ void __launch_bounds__(PF_THREADS, 1) prefill_kq_gemm_kernel(PrefillGemm g) {
    constexpr bool F8 = KqGeom<WT>::F8;
    constexpr int NS = KqGeom<WT>::NS, NQ = KqGeom<WT>::NQ, KQ_YQ = KqGeom<WT>::YQ, BT = KqGeom<WT>::BT;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    const uint32_t a_ring = sbase, y_ring = a_ring + NS * KQ_WT, b_ring = y_ring + NS * KQ_YQ;
    const uint32_t bars  = b_ring + NS * BT;
    auto raw_full = [&](int q) { return bars + 8u * q; };
    auto ops_full = [&](int q) { return bars + 8u * (NQ + q); };
    auto st_free  = [&](int q) { return bars + 8u * (2 * NQ + q); };
    auto d_full   = [&](int i) { return bars + 8u * (3 * NQ + i); };
    auto d_free   = [&](int i) { return bars + 8u * (3 * NQ + PF_DBUF + i); };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + (size_t)NS * (KQ_WT + KQ_YQ + BT) + 8 * (3 * NQ + 2 * PF_DBUF));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nb = g.nb, n_batch = (nb + PF_BATCH - 1) / PF_BATCH;
    const uint64_t limit = g.wait_limit_ns;
    const int row_tile = blockIdx.y, tok_tile = blockIdx.x;
    const uint8_t *wsrc = g.w + ((int64_t)row_tile * nb) * KQ_WT;
    const uint8_t *ysrc = g.yq + ((int64_t)tok_tile * nb) * KQ_YQ;

    if (tid == 0) {
        for (int q = 0; q < NQ; ++q) { mbar_init(raw_full(q), 1); mbar_init(ops_full(q), 1); mbar_init(st_free(q), PF_EPI_WARPS); }
        for (int i = 0; i < PF_DBUF; ++i) { mbar_init(d_full(i), 1); mbar_init(d_free(i), PF_EPI_WARPS); }
        mbar_init_fence();
    }
    for (int i = tid; i < NS * (BT / 16); i += PF_THREADS) { sts128(b_ring + (uint32_t)i * 16u, make_uint4(0u, 0u, 0u, 0u)); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(PF_DBUF * PF_NCOL) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp >= PF_EPI_WARPS + 2) {
        // ---- MMA warps
        if (lane == 0) {
            int last = -1;
            for (int b = warp - (PF_EPI_WARPS + 2); b < nb; b += PF_MMA_WARPS) {
                const int s = b % NS, q = b / PF_BATCH, buf = b % PF_DBUF;
                if (!mbar_wait_relaxed(ops_full(q % NQ), (uint32_t)(q / NQ) & 1u, limit)) { pf_report(g.error_flag, 5); break; }
                if (!mbar_wait_relaxed(d_free(buf), (uint32_t)(b / PF_DBUF) & 1u, limit)) { pf_report(g.error_flag, 5); break; }
                tc_fence_after();
                if (F8) {
                    const uint64_t a_desc = operand_desc(a_ring + (uint32_t)s * KQ_WT);
                    mma_f8_ss(tmem + (uint32_t)(buf * PF_NCOL), a_desc, operand_desc(b_ring + (uint32_t)s * BT), 0u);
                    mma_f8_ss(tmem + (uint32_t)(buf * PF_NCOL), a_desc, operand_desc(b_ring + (uint32_t)s * BT + PF_TILE), 1u);
                } else {
                    mma_s8_ss(tmem + (uint32_t)(buf * PF_NCOL), operand_desc(a_ring + (uint32_t)s * KQ_WT), operand_desc(b_ring + (uint32_t)s * BT));
                }
                mma_commit(d_full(buf));
                last = b;
            }
            if (last >= 0 && !mbar_wait_relaxed(d_full(last % PF_DBUF), (uint32_t)(last / PF_DBUF) & 1u, limit)) { pf_report(g.error_flag, 5); }
        }
    } else if (warp == PF_EPI_WARPS) {
        // ---- copy warp
        if (lane == 0) {
            int issued = 0;
            for (int q = 0; q < n_batch; ++q) {
                if (q >= NQ && !mbar_wait_relaxed(st_free(q % NQ), (uint32_t)((q / NQ) - 1) & 1u, limit)) { pf_report(g.error_flag, 4); break; }
                const int b0 = q * PF_BATCH, n = min(PF_BATCH, nb - b0), s0 = b0 % NS;
                mbar_expect_tx(raw_full(q % NQ), (uint32_t)(n * (KQ_WT + KQ_YQ)));
                bulk_copy_g2s(a_ring + (uint32_t)s0 * KQ_WT, wsrc + (int64_t)b0 * KQ_WT, (uint32_t)(n * KQ_WT), raw_full(q % NQ));
                bulk_copy_g2s(y_ring + (uint32_t)s0 * KQ_YQ, ysrc + (int64_t)b0 * KQ_YQ, (uint32_t)(n * KQ_YQ), raw_full(q % NQ));
                issued = q + 1;
            }
            for (int q = max(0, issued - NQ); q < issued; ++q) {
                if (!mbar_wait_relaxed(raw_full(q % NQ), (uint32_t)(q / NQ) & 1u, limit)) { pf_report(g.error_flag, 4); break; }
            }
        }
    } else if (warp == PF_EPI_WARPS + 1) {
        // ---- expander warp: word w of token tt -> row 4 (tt / 2) + 2 (w / 4) + tt % 2 of B (the same half of two neighbouring
        // tokens in neighbouring columns of D, for the packed arithmetic of the epilogue), at its own place in the block
        for (int q = 0; q < n_batch; ++q) {
            bool ok = mbar_wait_relaxed(raw_full(q % NQ), (uint32_t)(q / NQ) & 1u, limit);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { if (lane == 0) { pf_report(g.error_flag, 4); } break; }
            const int b0 = q * PF_BATCH, n = min(PF_BATCH, nb - b0), s0 = b0 % NS;
            for (int j = 0; j < n; ++j) {
                const uint32_t ysrc_s = y_ring + (uint32_t)(s0 + j) * KQ_YQ, bdst = b_ring + (uint32_t)(s0 + j) * BT;
#pragma unroll
                for (int plane = 0; plane < (F8 ? 2 : 1); ++plane) {   // (e4m3 form: the second plane of words goes to the second B operand)
                    uint32_t v[KQ_TOK * 8 / 32];
#pragma unroll
                    for (int k = 0; k < KQ_TOK * 8 / 32; ++k) { v[k] = lds32(ysrc_s + (uint32_t)(plane * KQ_TOK * 8 + lane + 32 * k) * 4u); }   // all loads in flight before the first store
#pragma unroll
                    for (int k = 0; k < KQ_TOK * 8 / 32; ++k) {
                        const int i = lane + 32 * k, tt = i >> 3, w = i & 7, row = 4 * (tt >> 1) + 2 * (w >> 2) + (tt & 1);
                        sts32(bdst + (uint32_t)plane * PF_TILE + (uint32_t)(row >> 3) * 256u + (uint32_t)(w >> 2) * 128u + (uint32_t)(row & 7) * 16u + (uint32_t)(w & 3) * 4u, v[k]);
                    }
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) { mbar_arrive(ops_full(q % NQ)); }
        }
    } else {
        // ---- epilogue warps: 64 columns = 32 tokens, read back 16 columns (8 tokens) at a time into two alternating register sets
        const int quad = warp & 3, half = warp >> 2;
        const int row = 32 * quad + lane;
        const uint32_t tbase = tmem + ((uint32_t)(32 * quad) << 16) + (uint32_t)(64 * half);
        const uint32_t sc_addr = a_ring + PF_TILE + 8u * (uint32_t)row;
        const uint32_t dx_addr = y_ring + (F8 ? 2 : 1) * KQ_TOK * 32 + 128u * (uint32_t)half;   // this warp's 32 scales; the block sums lie KQ_TOK * 4 further
        uint64_t acc[16], tot[16];   // packed pairs: tokens 2 u and 2 u + 1 of the warp's 32
#pragma unroll
        for (int t = 0; t < 16; ++t) { acc[t] = 0ull; tot[t] = 0ull; }
        const uint64_t minus_magic = f2_pack(-MAGIC_F, -MAGIC_F);
        if (!F8) {   // the offset pattern into this thread's part of every buffer
            for (int i = 0; i < PF_DBUF; ++i) {
                tmem_st32_same(tbase + (uint32_t)(i * PF_NCOL), MAGIC_I);
                tmem_st32_same(tbase + (uint32_t)(i * PF_NCOL) + 32u, MAGIC_I);
            }
            tmem_st_wait();
            tc_fence_before();
        }
        __syncwarp();
        if (lane == 0) { for (int i = 0; i < PF_DBUF; ++i) { mbar_arrive(d_free(i)); } }

        uint32_t ra[16], rb[16];
        bool ok = mbar_wait_bounded(d_full(0), 0u, limit);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) { tc_fence_after(); tmem_ld16(tbase, ra); tmem_ld16(tbase + 16u, rb); }
        static_assert(PF_BATCH == PF_DBUF, "the unrolled epilogue pairs block j of a batch with accumulator buffer j");
        for (int q = 0; q < n_batch && ok; ++q) {
            const uint32_t ring_q = (uint32_t)(q % NQ) * PF_BATCH;
            const uint32_t sc_q = sc_addr + ring_q * KQ_WT, dx_q = dx_addr + ring_q * KQ_YQ;
#pragma unroll
            for (int j = 0; j < PF_BATCH; ++j) {
                const int b = q * PF_BATCH + j;
                if (b >= nb || !ok) { break; }
                const uint32_t taddr = tbase + (uint32_t)(j * PF_NCOL);
                const float2 sc = lds64f(sc_q + (uint32_t)j * KQ_WT);
                const uint64_t scx = f2_pack(sc.x, sc.x), scy = (WT == 12) ? f2_pack(-sc.y, -sc.y) : f2_pack(sc.y, sc.y);
                const uint32_t dx_s = dx_q + (uint32_t)j * KQ_YQ;
                tmem_ld_wait();                       // columns 0..31 of block b are in registers
                kq_fold8<WT, 0>(acc, ra, scx, scy, dx_s, minus_magic);
                tmem_ld16(taddr + 32u, ra);
                kq_fold8<WT, 8>(acc, rb, scx, scy, dx_s, minus_magic);
                tmem_ld16(taddr + 48u, rb);
                tmem_ld_wait();                       // columns 32..63 too: the buffer has been read
                if (F8) {                             // free for the next MMA at once
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) { mbar_arrive(d_free(j)); }
                } else {                              // put the offset pattern back
                    tmem_st32_same(taddr, MAGIC_I);
                    tmem_st32_same(taddr + 32u, MAGIC_I);
                }
                kq_fold8<WT, 16>(acc, ra, scx, scy, dx_s, minus_magic);
                const bool more = b + 1 < nb;
                const uint32_t tnext = tbase + (uint32_t)(((j + 1) % PF_DBUF) * PF_NCOL);
                if (more) {
                    ok = mbar_wait_bounded(d_full((j + 1) % PF_DBUF), (uint32_t)(q + (j + 1) / PF_DBUF) & 1u, limit);
                    ok = __all_sync(0xffffffffu, ok);
                    if (ok) { tc_fence_after(); tmem_ld16(tnext, ra); }
                }
                kq_fold8<WT, 24>(acc, rb, scx, scy, dx_s, minus_magic);
                if (more && ok) { tmem_ld16(tnext + 16u, rb); }
                if ((b & 7) == 7) {                   // a super-block ends: its value joins the row's sum
#pragma unroll
                    for (int t = 0; t < 16; ++t) { tot[t] = f2_add(tot[t], acc[t]); acc[t] = 0ull; }
                }
                if (!F8) {
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                }
                if (lane == 0) {
                    if (!F8) { mbar_arrive(d_free(j)); }
                    if (j == PF_BATCH - 1 || b == nb - 1) { mbar_arrive(st_free(q % NQ)); }
                }
            }
        }
        tmem_ld_wait();
        if (!ok) { if (lane == 0) { pf_report(g.error_flag, 6); } }
        else {
#pragma unroll
            for (int t = 0; t < 32; ++t) {
                const int token = tok_tile * KQ_TOK + 32 * half + t;
                float lo, hi;
                f2_unpack(tot[t >> 1], lo, hi);
                const float v = (t & 1) ? hi : lo;
                if (token < g.T && (int64_t)row_tile * PF_M + row < g.n_rows) {
                    const int64_t i = (int64_t)token * g.out_stride + (int64_t)row_tile * PF_M + row;
                    g.out[i] = g.resid != nullptr ? __fadd_rn(v, g.resid[i]) : v;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(PF_DBUF * PF_NCOL) : "memory");
    }
}

// element k of a block's row at its place in the s8 operand tile (core matrices of 8 rows x 16 bytes)
__device__ __forceinline__ int8_t *tile_elem(uint8_t *tile, int r, int k) { return reinterpret_cast<int8_t *>(tile + (r >> 3) * 256 + (k >> 4) * 128 + (r & 7) * 16 + (k & 15)); }

// upload-time re-layout: GGUF super-blocks (Q4_K 144 B, Q6_K 210 B per 256 values) of rows [0, n_rows) -> tiles of 128 rows x one
// 32-element block: the integer weights as s8, then per row the two f32 scale products of the block. One thread per (row, block).
template <int WT>
__global__ void prefill_kq_retile_kernel(const uint8_t *raw, int64_t row_stride, int64_t n_rows, int nb, uint8_t *base, int64_t dst_row0) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows * nb) { return; }
    const int64_t lrow = i / nb;
    const int     b = (int)(i - lrow * nb), sb = b >> 3, j = b & 7;
    const int64_t row = dst_row0 + lrow;
    const int     r = (int)(row % PF_M);
    uint8_t *tile = base + ((row / PF_M) * nb + b) * (int64_t)KQ_WT;
    float *scales = reinterpret_cast<float *>(tile + PF_TILE + 8 * r);
    if (WT == 12) {
        const uint8_t *s = raw + lrow * row_stride + (int64_t)sb * 144;
        const float d = h2f((uint16_t)(s[0] | (s[1] << 8))), dmin = h2f((uint16_t)(s[2] | (s[3] << 8)));
        const uint8_t *sc12 = s + 4, *qs = s + 16 + 32 * (j >> 1);
        uint32_t sc, mn;
        if (j < 4) { sc = sc12[j] & 63u; mn = sc12[j + 4] & 63u; }
        else { sc = (sc12[j + 4] & 0xFu) | ((sc12[j - 4] >> 6) << 4); mn = (uint32_t)(sc12[j + 4] >> 4) | ((uint32_t)(sc12[j] >> 6) << 4); }
        scales[0] = __fmul_rn(d, (float)sc);
        scales[1] = __fmul_rn(dmin, (float)mn);
        for (int l = 0; l < 32; ++l) { *tile_elem(tile, r, l) = (int8_t)e4m3_of_small((uint32_t)((j & 1) ? (qs[l] >> 4) : (qs[l] & 0xF))); }   // (the e4m3 code of 0..15)
    } else {
        const uint8_t *s = raw + lrow * row_stride + (int64_t)sb * 210;
        const uint8_t *ql = s, *qh = s + 128;
        const int8_t *sc = reinterpret_cast<const int8_t *>(s + 192);
        const float d = h2f((uint16_t)(s[208] | (s[209] << 8)));
        const int hf = j >> 2, seg = j & 3;                  // half of the super-block, segment of 32 values
        scales[0] = __fmul_rn(d, (float)sc[2 * j]);
        scales[1] = __fmul_rn(d, (float)sc[2 * j + 1]);
        for (int l = 0; l < 32; ++l) {
            const uint8_t lo = ql[64 * hf + 32 * (seg & 1) + l], h = qh[32 * hf + l];
            const int v = ((seg & 2) ? (lo >> 4) : (lo & 0xF)) | (((h >> (2 * seg)) & 3) << 4);
            *tile_elem(tile, r, l) = (int8_t)(v - 32);
        }
    }
}

template <int WT>
cudaError_t launch_kq_t(const PrefillGemm &g, cudaStream_t stream) {
    constexpr size_t KQ_SMEM_BYTES = KqGeom<WT>::SMEM;
    cudaError_t err = allow_dynamic_smem(reinterpret_cast<const void *>(prefill_kq_gemm_kernel<WT>), KQ_SMEM_BYTES);
    if (err != cudaSuccess) { return err; }
    const dim3 grid((unsigned)((g.T + KQ_TOK - 1) / KQ_TOK), (unsigned)((g.n_rows + PF_M - 1) / PF_M));
    prefill_kq_gemm_kernel<WT><<<grid, PF_THREADS, KQ_SMEM_BYTES, stream>>>(g);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_prefill_gemm_kq(const PrefillGemm &g, cudaStream_t stream) {
    if (g.w == nullptr || g.yq == nullptr || g.out == nullptr || g.T < 1 || g.nb < 8 || (g.nb & 7) || g.n_rows < 1) { return cudaErrorInvalidValue; }
    if (g.type == 12) { return launch_kq_t<12>(g, stream); }
    if (g.type == 14) { return launch_kq_t<14>(g, stream); }
    return cudaErrorInvalidValue;
}

cudaError_t launch_prefill_retile_kq(int type, const uint8_t *raw, int64_t row_stride, int64_t n_rows, int nb, uint8_t *base, int64_t dst_row0, cudaStream_t stream) {
    if ((type != 12 && type != 14) || n_rows < 1 || nb < 8 || (nb & 7)) { return cudaErrorInvalidValue; }
    const int64_t n = n_rows * nb;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (type == 12) { prefill_kq_retile_kernel<12><<<blocks, 256, 0, stream>>>(raw, row_stride, n_rows, nb, base, dst_row0); }
    else            { prefill_kq_retile_kernel<14><<<blocks, 256, 0, stream>>>(raw, row_stride, n_rows, nb, base, dst_row0); }
    return cudaGetLastError();
}

}  // namespace spyb
