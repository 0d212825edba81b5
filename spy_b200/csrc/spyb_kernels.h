// Host-side launch interface of the sm_100a kernels (internal to the library).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace spyb {

// A quantized weight matrix resident in HBM, re-tiled at upload. Rows are padded to a multiple of four
// blocks (nbp; the padding blocks are zeros with a zero scale) and every group of four consecutive
// blocks of a row is stored word-transposed, so that the lane that owns accumulator l of the CPU's
// 8-wide dot product loads, with one aligned 128-bit word, exactly its own four bytes of four blocks:
//   Q4_0: q[row][group][j]  (j = 0..3)  = 32-bit word j of the 16 nibble bytes of blocks 4g..4g+3
//   Q8_0: q[row][group][l]  (l = 0..7)  = 32-bit word l of the 32 int8 values of blocks 4g..4g+3
//   d[row][block]                       = fp16 scale
// The bytes are those of the reference's block_q4_0_t / block_q8_0_t
// (orchestration/include/number/number_impl/quant.h:10-33, 124-147), only regrouped.
struct DevMatrix {
    int             type = -1;
    int64_t         n_rows = 0;
    int64_t         k = 0;
    int             nb = 0;    // blocks per row
    int             nbp = 0;   // blocks per row in memory (nb rounded up to a multiple of 4)
    const uint4    *q = nullptr;
    const uint16_t *d = nullptr;
    size_t bytes() const { return (size_t)n_rows * nb * ((type == 8 ? 32 : 16) + 2); }   // algorithmic bytes (without padding)
};
inline int    padded_blocks(int nb) { return (nb + 3) & ~3; }
inline size_t q_row_words(int type, int nb) { return (size_t)padded_blocks(nb) * (type == 8 ? 2 : 1); }   // uint4 per row of the q plane
inline size_t q_plane_bytes(int type, int64_t n_rows, int nb) { return (size_t)n_rows * q_row_words(type, nb) * 16; }
inline size_t d_plane_bytes(int64_t n_rows, int nb) { return (size_t)n_rows * padded_blocks(nb) * 2; }

enum Prologue { PRO_QUANT = 0, PRO_NORM_QUANT = 1 };
enum Epilogue { EPI_STORE = 0, EPI_RESID = 1, EPI_SILU_MUL = 2, EPI_QKV_ROPE = 3 };

struct MatvecParams {
    DevMatrix A;
    DevMatrix B;               // second matrix when pair_mode == 1 (same shape as A)
    int       pair_mode = 0;   // 1: a warp's tile is rows 4u..4u+3 of A together with the same rows of B (FFN up and gate)
    int       T = 1;           // activation columns (tokens) in this launch, <= matvec_max_columns(nb)
    // prologue
    int          pro = PRO_QUANT;
    const float *x = nullptr;  // [T][x_stride] f32
    int64_t      x_stride = 0;
    const float *norm_w = nullptr;
    float        eps = 0.f;
    // epilogue
    int          epi = EPI_STORE;
    float       *out = nullptr;   // [T][out_stride]
    int64_t      out_stride = 0;
    const float *resid = nullptr; // [T][out_stride]
    const float *silu_table = nullptr;
    // EPI_QKV_ROPE: rows [0,dl) = Q, [dl,2dl) = K, [2dl,3dl) = V
    const int    *pos_base = nullptr;   // device scalar: position of column 0
    const float2 *rope_table = nullptr; // [n_ctx][hd/2] (cos, sin)
    int           hd = 128;
    int           dl = 0;
    __half       *q_out = nullptr;      // [T][dl]
    __half       *k_cache = nullptr;    // [n_ctx][dl]
    __half       *v_cache = nullptr;    // [dl][n_ctx] (transposed, as the reference keeps it)
    int           n_ctx = 0;
    // optional tap: reference-layout Q8_0 blocks of column 0 (nb * 34 bytes)
    uint8_t      *tap_xq = nullptr;
    // weights a later kernel of the step will stream: pulled into L2 once this CTA's own loads are issued
    const void   *pf_ptr[4] = {nullptr, nullptr, nullptr, nullptr};
    size_t        pf_bytes[4] = {0, 0, 0, 0};
};

struct AttnParams {
    const __half *q = nullptr;        // [T][dl], already rounded to fp16
    const __half *k_cache = nullptr;  // [n_ctx][dl]
    const __half *v_cache = nullptr;  // [dl][n_ctx]
    float        *out = nullptr;      // [T][dl]
    const int    *pos_base = nullptr;
    const float  *exp_table = nullptr;
    int   n_head = 0, hd = 128, dl = 0, T = 1, n_ctx = 0;
    float scale = 0.f;
    const void *pf_ptr[4] = {nullptr, nullptr, nullptr, nullptr};   // as in MatvecParams
    size_t      pf_bytes[4] = {0, 0, 0, 0};
};

struct LaunchCfg {
    cudaStream_t stream = nullptr;
    bool         pdl = false;   // launch with the programmatic-stream-serialization attribute
    int          num_sms = 148;
    int          mv_ctas_per_sm = 2;   // mat-vec CTAs per SM for single-column launches (their register budget allows 2)
};

size_t      matvec_smem_bytes(int nb, int T);
int         matvec_max_columns(int nb);   // most activation columns one launch can hold in shared memory for rows of nb blocks
cudaError_t launch_matvec(const MatvecParams &p, const LaunchCfg &cfg);
cudaError_t launch_attention(const AttnParams &p, const LaunchCfg &cfg);

// upload-time re-tiling of raw reference-layout blocks into DevMatrix planes
// (q_row0, d_row0 point at the first destination row; nb blocks are read per row, the padding is zero-filled)
cudaError_t launch_retile(int type, const uint8_t *raw, int64_t row_stride_bytes, int64_t n_rows, int nb, uint4 *q_row0, uint16_t *d_row0, cudaStream_t s);

// stand-alone arithmetic kernels (parity checks and the per-operator path)
cudaError_t launch_quantize_q8_0_ref_layout(const float *x, int64_t n, uint8_t *blocks, cudaStream_t s);
cudaError_t launch_block_dots(int wtype, const uint8_t *w_row, const uint8_t *x_blocks, int64_t n, int32_t *out, cudaStream_t s);

struct Strided {   // a tensor as the reference's Shape describes it: elements + byte strides
    void   *data;
    int64_t ne[4];
    int64_t nb[4];
};
cudaError_t launch_rmsnorm(const float *x, float *out, int64_t n, int64_t rows, float eps, cudaStream_t s);
cudaError_t launch_binary_rows(int op /*0 add, 1 mul*/, const float *a, const float *b, float *out, int64_t n, int64_t rows, int64_t b_rows, cudaStream_t s);
cudaError_t launch_silu(const float *x, float *out, int64_t n, const float *silu_table, cudaStream_t s);
cudaError_t launch_softmax_masked(const float *scores, const float *mask, float *out, int64_t ne0, int64_t ne1, int64_t ne2,
                                  int64_t mask_stride, float scale, const float *exp_table, cudaStream_t s);
// cos_sin: device table [ne2 tokens][ne0/2] of (cos, sin) built on the host with the host libm
cudaError_t launch_rope(const Strided &x, const float2 *cos_sin, const Strided &out, cudaStream_t s);
cudaError_t launch_copy_strided(const Strided &src, int src_type, const Strided &dst, int dst_type, cudaStream_t s);
cudaError_t launch_getrow(const uint8_t *table, int table_type, int64_t row_bytes, int64_t ne0, const int32_t *ids, int64_t n_ids, float *out, cudaStream_t s);
cudaError_t launch_matmul_f16(const Strided &w /*f16*/, const Strided &x /*f32*/, const Strided &out /*f32*/, cudaStream_t s);
cudaError_t launch_argmax_embed(const float *logits, int64_t n_vocab, int32_t *token_out, int32_t *history, int *pos_counter,
                                const uint8_t *embd, int embd_type, int64_t d_model, float *x_out, const LaunchCfg &cfg);
cudaError_t launch_embed(const int32_t *ids, int n_ids, const uint8_t *embd, int embd_type, int64_t d_model, float *x_out, cudaStream_t s);

}  // namespace spyb
