// Host-side launch interface of the sm_100a kernels (internal to the library).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <mutex>
#include <utility>

namespace spyb {

// A quantized weight matrix resident in HBM, re-tiled at upload into the stream a warp consumes:
//   tile   = 4 (or 32) consecutive rows; a tile's data is one contiguous run, so a warp walks sequential addresses
//   record = 8 consecutive blocks of the rows of a tile:
//              [row 0..tile_rows-1][ q: 2 groups x WORDS x 16 B | d: 8 fp16 scales ]      (WORDS = 4 for Q4_0, 8 for Q8_0)
//            inside a group of four blocks the quants are word-transposed: 128-bit word j holds 32-bit word j of
//            each of the four blocks, so the lane that owns accumulator l of the CPU's 8-wide dot product finds
//            its own four bytes of four blocks in one aligned 128-bit word
//   Q4_0 quants are stored XOR 0x88: a nibble then reads as (value - 8) in two's complement, and a byte masked
//   to its high nibble is 16 * (value - 8) as a signed byte - no "- 8" correction term is needed at run time.
//   Rows are padded to a multiple of 8 blocks (nbp) with zero scales.
// The information is that of the reference's block_q4_0_t / block_q8_0_t
// (orchestration/include/number/number_impl/quant.h:10-33, 124-147), only regrouped.
struct DevMatrix {
    int            type = -1;
    int64_t        n_rows = 0;   // multiple of 4
    int64_t        k = 0;
    int            nb = 0;       // blocks per row
    int            nbp = 0;      // blocks per row in memory (nb rounded up to a multiple of 8)
    int            tile_rows = 4;   // rows per tile: 4 (lane-per-accumulator kernel) or 8 / 16 / 32 (lane-per-row kernels)
    int            mma = 0;         // tile_rows 8 / 16 only: records in the fragment order of the tensor-core kernel (see below)
    int            fused_pair = 0;  // tile_rows >= 8 only: the first half of a tile's rows are FFN-up rows, the second half the matching FFN-gate rows
    const uint8_t *w = nullptr;  // [n_rows / tile_rows][nbp / 8] records of tile_rows rows
    size_t bytes() const { return (size_t)n_rows * nb * ((type == 8 ? 32 : 16) + 2); }   // algorithmic bytes (without padding)
};
inline int    padded_blocks(int nb) { return (nb + 7) & ~7; }
inline int    record_row_bytes(int type) { return (type == 8 ? 256 : 128) + 16; }
inline size_t matrix_bytes(int type, int64_t n_rows, int nb) { return (size_t)n_rows * (padded_blocks(nb) / 8) * record_row_bytes(type); }

enum Prologue { PRO_QUANT = 0, PRO_NORM_QUANT = 1 };
enum Epilogue { EPI_STORE = 0, EPI_RESID = 1, EPI_SILU_MUL = 2, EPI_QKV_ROPE = 3 };
constexpr int TP_MAX = 8;

// One exchange site of the tensor-parallel all-gather over peer memory (memory of the other ranks mapped into this
// process). A producing kernel writes its share of the gathered vector [T][stride] - elements [off, off + len) of every
// column - into its own copy; its last CTA copies the share into every other rank's copy and then writes *epoch into
// every rank's flag word `rank` of the site. A consuming kernel waits (bounded) until all n flag words of the site in its
// own memory show *epoch.
struct TpLink {
    int             n = 0, rank = 0;
    float          *gather[TP_MAX] = {};      // producer: the gathered vector in each rank's memory (gather[rank] = the local copy)
    int64_t         stride = 0, off = 0, len = 0;
    unsigned       *flag_out[TP_MAX] = {};    // producer: flag word `rank` of the site in each rank's memory
    unsigned       *counter = nullptr;        // producer: local CTA counter of the site (self-resetting); nullptr = not a producer
    const unsigned *flag_in = nullptr;        // consumer: the site's n flag words in local memory; nullptr = not a consumer
    const int      *epoch = nullptr;          // device word: the step's exchange epoch
};

// K-quant weights stay in their GGUF row layout (Q4_K) or a 16-byte-aligned re-layout of it (Q6_K, see spyb_kquant.cu):
// up to three row ranges form one virtual matrix (Wq | Wk | Wv), or, in pair mode, two matrices whose rows i meet (up, gate)
struct KqSeg {
    const uint8_t *w = nullptr;
    int     type = 0;          // 12 = Q4_K, 14 = Q6_K
    int64_t n_rows = 0;
    int64_t row_bytes = 0;
};

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
    // batch of independent sequences in lockstep (seq_stride > 0): column t is sequence t - its position is *pos_base for every
    // column, and its K / V cache lies t * seq_stride elements behind k_cache / v_cache
    int64_t       seq_stride = 0;
    // optional tap: reference-layout Q8_0 blocks of column 0 (nb * 34 bytes)
    uint8_t      *tap_xq = nullptr;
    int          *error_flag = nullptr; // set non-zero when a bounded wait on a bulk copy ran out
    // optional profiling aid: eight %globaltimer stamps (CTA 0: entry, predecessor finished, prologue done; last CTA done;
    // latest CTA: entry, predecessor finished, prologue done; unused)
    unsigned long long *stamps = nullptr;
    TpLink tp;                          // tensor-parallel all-gather fused into the kernel (producer and / or consumer side)
    KqSeg  kq[3];                       // K-quant weights: kq_n > 0 selects the K-quant kernel (A then only carries k, nb and n_rows)
    int    kq_n = 0;
};

// Prompt evaluation as a GEMM on the tcgen05 tensor cores (spyb_prefill.cu). Weights in tiles of PF_ROWS rows x 1 block,
// activations as compact Q8_0 blocks grouped by (tile of PF_TOK tokens, block).
constexpr int PF_ROWS = 128, PF_TOK = 16;
constexpr int PF_YQ_BYTES = PF_TOK * 32 + PF_TOK * 4;           // the s8 form (16 x 32 s8, 16 f32 scales; no Q4_0 / Q8_0 kernel uses it any more)
constexpr int PF_YQ_BYTES_F8 = 2 * PF_TOK * 32 + PF_TOK * 4;    // Q4_0 / Q8_0 weights: the activation bytes split into two e4m3 planes (16 x 32 each), 16 f32 scales
constexpr int PF_KQ_TOK = 64;                                   // K-quant kernels: 64 tokens per tile, two columns of D per token
constexpr int PF_KQ_YQ_BYTES = PF_KQ_TOK * 32 + PF_KQ_TOK * 8;   // Q6_K weights: 64 x 32 s8, 64 f32 scales, 64 f32 block sums
constexpr int PF_KQ_YQ_BYTES_F8 = 2 * PF_KQ_TOK * 32 + PF_KQ_TOK * 8;   // Q4_K weights: two e4m3 planes of 64 x 32, scales, block sums
constexpr int PF_KQ_WTILE = 128 * 32 + 128 * 8;                 // the s8 A operand of a 32-element block, then two f32 scale products per row
constexpr int PF_MAX_K = 14336;   // widest activation row the quantizer kernel holds in registers
struct PrefillGemm {
    const uint8_t *w = nullptr;       // [n_rows / PF_ROWS][nb] weight tiles (launch_prefill_retile)
    int            type = 0;          // 2 = Q4_0, 8 = Q8_0, 12 = Q4_K, 14 = Q6_K
    int64_t        n_rows = 0;        // (the last tile of PF_ROWS rows may be partly padding: zero weights, rows not stored)
    int            nb = 0;            // blocks per row
    const uint8_t *yq = nullptr;      // [ceil(T / PF_TOK)][nb][PF_YQ_BYTES or PF_YQ_BYTES_F8] (launch_prefill_quant for this weight type)
    int            T = 0;
    float         *out = nullptr;     // [T][out_stride]
    int64_t        out_stride = 0;
    const float   *resid = nullptr;   // optional [T][out_stride]: out = W x + resid (may alias out)
    int           *error_flag = nullptr;
    uint64_t       wait_limit_ns = 1000000000ull;
    long long     *stamps = nullptr;  // profiling aid: clock stamps of CTA (0, 0), [8 roles][512 blocks][4]
    int            selftest_skip_batch = -1;   // failure-path check: the copy thread leaves this batch out, so the waits for it run out
};
int         prefill_e4m3_selftest();   // host-only: 0 when the e4m3 codes of the prompt GEMM decode to the integers they stand for
size_t      prefill_weight_bytes(int type, int64_t n_rows, int nb);
size_t      prefill_act_bytes(int T, int nb);
cudaError_t launch_prefill_retile(int type, const uint8_t *raw, int64_t row_stride, int64_t n_rows, int nb, uint8_t *base, int64_t dst_row0, cudaStream_t stream);
// weight_type: the type of the matrix the activations will meet (2, 8, 12 or 14): it decides their layout;
// part_len > 0: a row lies in K / part_len parts, part_stride floats apart
cudaError_t launch_prefill_quant(const float *x, int64_t x_stride, int T, int K, const float *norm_w, float eps, uint8_t *yq, cudaStream_t stream, int weight_type,
                                 int part_len = 0, int64_t part_stride = 0);
cudaError_t launch_prefill_gemm_kq(const PrefillGemm &g, cudaStream_t stream);   // type 12 = Q4_K, 14 = Q6_K (spyb_prefill_kq.cu)
cudaError_t launch_prefill_retile_kq(int type, const uint8_t *raw, int64_t row_stride, int64_t n_rows, int nb, uint8_t *base, int64_t dst_row0, cudaStream_t stream);
cudaError_t launch_prefill_gemm(const PrefillGemm &g, cudaStream_t stream);
cudaError_t launch_prefill_qkv_post(const float *qkv, int T, int dl, int hd, const int *pos_base, const float2 *rope, __half *q_out, __half *k_cache,
                                    __half *v_cache, int n_ctx, int64_t seq_stride, cudaStream_t stream);
cudaError_t launch_prefill_silu_mul(const float *upgate, int T, int F, const float *silu_table, float *act, cudaStream_t stream);

struct AttnParams {
    int           force_long = 0;     // take the three-kernel path (scratch needed) also at short contexts
    const __half *q = nullptr;        // [T][dl], already rounded to fp16
    const __half *k_cache = nullptr;  // [n_ctx][dl]
    const __half *v_cache = nullptr;  // [dl][n_ctx]
    float        *out = nullptr;      // [T][out_stride]
    int64_t       out_stride = 0;     // 0 = dl
    const int    *pos_base = nullptr;
    const float  *exp_table = nullptr;
    float        *scratch = nullptr;  // [T][n_head][n_ctx] floats; needed when attention_scratch_floats() > 0 (long contexts)
    int   n_head = 0, hd = 128, dl = 0, T = 1, n_ctx = 0;
    float scale = 0.f;
    int64_t seq_stride = 0;           // > 0: token t is sequence t of a batch in lockstep (position pos_base[0], cache t * seq_stride elements further, no other token visible)
    unsigned long long *stamps = nullptr;                           // as in MatvecParams
    TpLink tp;                                                      // producer side of the all-gather of the attention output
    int   *error_flag = nullptr;
};

struct LaunchCfg {
    cudaStream_t stream = nullptr;
    bool         pdl = false;   // launch with the programmatic-stream-serialization attribute
    int          num_sms = 148;
    int          mv_ctas_per_sm = 2;   // mat-vec CTAs per SM for single-column launches (their register budget allows 2)
    int          mv_ring_kb = 80;      // shared-memory ring per CTA that bulk copies stream the weights through
    int          mv_force_s = 0, mv_force_wact = 0;   // tuning overrides (0 = choose)
    int         *error_flag = nullptr;
};

// Book-keeping for cudaFuncAttributeMaxDynamicSharedMemorySize, which is set per (device, kernel): decide() says
// whether a launch that needs `bytes` must raise the attribute first (and records the new mark).
class SmemLedger {
public:
    enum Decision { KEEP = 0, RAISE = 1 };
    Decision decide(int device, const void *kernel, size_t bytes);
    void     forget(int device, const void *kernel);
private:
    std::map<std::pair<int, const void *>, size_t> allowed_;
    std::mutex mutex_;
};
// raises the current device's dynamic shared-memory limit of `kernel` to `bytes` when it is below (thread-safe)
cudaError_t allow_dynamic_smem(const void *kernel, size_t bytes);
int         smem_ledger_selftest();   // host-only check of SmemLedger, 0 = passed

size_t      matvec_smem_bytes(int nb, int T);
int         matvec_max_columns(int nb);   // most activation columns one launch can hold in shared memory for rows of nb blocks
cudaError_t launch_matvec(const MatvecParams &p, const LaunchCfg &cfg);
constexpr int KQ_MAX_COLUMNS = 4;                                             // activation columns of one pass of the K-quant mat-vec kernel
cudaError_t launch_matvec_kq(const MatvecParams &p, const LaunchCfg &cfg);   // (launch_matvec forwards to it when p.kq_n > 0)
int64_t     kq_row_bytes(int type, int64_t k);                             // bytes of one K-quant row in device memory
cudaError_t launch_kq_relayout_q6k(const uint8_t *raw, int64_t n_rows, int64_t k, uint8_t *dst, cudaStream_t s);
cudaError_t launch_attention(const AttnParams &p, const LaunchCfg &cfg);
size_t      attention_scratch_floats(int n_ctx, int n_head, int T);

// upload-time re-tiling of raw reference-layout blocks into DevMatrix planes
// Source row i (i = src_row0 .. src_row0 + n_rows - 1 of the tensor being uploaded; `raw` points at row src_row0) lands
// at matrix row dst_row0 + i, or, with sub_rows > 0, at dst_row0 + (i / sub_rows) * tile_rows + sub_off + i % sub_rows
// (interleaving two tensors tile by tile). nb blocks are read per row, the padding up to a multiple of 8 is zero-filled.
cudaError_t launch_retile(int type, const uint8_t *raw, int64_t row_stride_bytes, int64_t n_rows, int nb, uint8_t *matrix_base, int tile_rows, bool mma,
                          int64_t dst_row0, int64_t src_row0, int sub_rows, int sub_off, cudaStream_t s);

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
// K-quant weights (raw GGUF rows: Q4_K = 12, Q6_K = 14) times f32 activations [n_cols][k] -> out [n_cols][n_rows]
cudaError_t launch_matmul_kquant(int type, const uint8_t *w, int64_t n_rows, int64_t k, const float *x, int64_t n_cols, float *out, cudaStream_t s);
cudaError_t launch_argmax_embed_batch(const float *logits, int64_t n_vocab, int n_seq, int32_t *tokens, int32_t *ids_out, const uint8_t *embd, int embd_type,
                                      int64_t d_model, float *x_out, int64_t x_stride, int *pos_counter, cudaStream_t s);
cudaError_t launch_argmax_embed(const float *logits, int64_t n_vocab, int32_t *token_out, int32_t *history, int *pos_counter,
                                const uint8_t *embd, int embd_type, int64_t d_model, float *x_out, const LaunchCfg &cfg);
cudaError_t launch_embed(const int32_t *ids, int n_ids, const uint8_t *embd, int embd_type, int64_t d_model, float *x_out, cudaStream_t s);

// ---- one decode step as a single persistent kernel (spyb_step.cu)
constexpr int ST_STAGE_BYTES = 9216;   // one ring stage: 8 / 4 records of an 8- / 16-row Q4_0 tile (4 / 2 of a Q8_0 tile)
struct StepMat {                // a matrix the step streams, in fragment-ordered records (DevMatrix::mma)
    const uint8_t *w = nullptr;
    int n_tiles = 0;            // tiles of `tr` rows
    int nrec = 0;               // records (8 blocks) per tile
    int recb = 0;               // bytes per record
    int tr = 8;                 // rows per tile: 8 or 16
    int type = 2;               // 2 = Q4_0, 8 = Q8_0
    int nbp = 0;                // blocks per row (padded to a multiple of 8)
    int crecs = 1;              // records per ring stage
    int nch = 1;                // stages per tile
};
struct StepLayer {
    StepMat      qkv, wo, upgate, down;
    const float *attn_norm = nullptr, *ffn_norm = nullptr;
    __half      *k_cache = nullptr, *v_cache = nullptr;   // K [n_ctx][d], V transposed [d][n_ctx]
};
struct StepParams {
    const StepLayer *layers = nullptr;   // device array
    int          n_layer = 0;
    StepMat      head;
    const float *output_norm = nullptr;
    float       *x = nullptr;            // residual stream [d] (in: the token's embedding)
    float       *act = nullptr;          // up * silu(gate) [fl]
    float       *logits = nullptr;       // [n_vocab]
    int8_t      *att_q = nullptr;        // attention output as Q8_0 values [d] ...
    float       *att_d = nullptr;        // ... and one scale per 32 (the fp16-rounded scale as f32)
    __half      *q = nullptr;            // Q after RoPE [d]
    const int   *pos = nullptr;          // [0] position of the token, [1] row length of the score matrix (0: position + 1)
    const float2 *rope = nullptr;        // [n_ctx][64] (cos, sin)
    const float *silu_table = nullptr, *exp_table = nullptr;
    int          d = 0, fl = 0, n_ctx = 0, n_head = 0, att_parts = 1, nbp_max = 0;
    float        eps = 0.f, att_scale = 0.f;
    unsigned long long *sync = nullptr;  // [0] barrier arrivals, [2] abort word; zeroed before every launch
    int         *error_flag = nullptr;
    unsigned long long wait_limit_ns = 1000000000ull;
    int          barrier_extra = 0;      // failure-path check only: arrivals a barrier expects beyond the grid size (it then runs out)
    uint8_t     *tap_xq = nullptr;       // optional: reference-layout Q8_0 blocks of layer 0's attention-norm output
    unsigned long long *stamps = nullptr; // optional profiling aid: per check point, CTA 0's time and the latest CTA's time
};
size_t      step_act_bytes(const StepParams &p);
int         step_ring_stages(const StepParams &p, size_t smem_limit);   // stages the ring gets out of `smem_limit` bytes per CTA
cudaError_t step_resident_ctas(const StepParams &p, int ns, int *ctas_per_sm);
cudaError_t launch_step(const StepParams &p, int grid, int ns, bool cooperative, cudaStream_t stream);

}  // namespace spyb
