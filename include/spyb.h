/*
 * spyb.h - C ABI of the sm_100a backend library (libspyb200.so).
 *
 * Every entry point takes plain pointers and sizes; no C++ or framework types cross the
 * boundary, so the library can be bound from the reference's C++ (a `spy::Backend`
 * subclass), from C, or from Python ctypes alike.
 *
 * Each declaration cites the reference (BL-GS/Spy) interface it stands in for, as a path
 * inside that project. There is no CPU fallback behind any of these calls: an operator or
 * number type the GPU path does not implement returns SPYB_UNSUPPORTED.
 */
#ifndef SPYB_H_
#define SPYB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* OperatorStatus, backend/interface/include/backend/backend.h:22-29 */
typedef enum { SPYB_SUCCESS = 0, SPYB_FAIL = 1, SPYB_UNSUPPORTED = 2 } spyb_status;

/* NumberType, orchestration/include/number/number_impl/type.h:12-45 (GGML numbering) */
enum {
    SPYB_FP32 = 0, SPYB_FP16 = 1, SPYB_Q4_0 = 2, SPYB_Q8_0 = 8, SPYB_Q4_K = 12, SPYB_Q6_K = 14, SPYB_INT32 = 26
};

/* OperatorType, orchestration/include/operator/type.h:38-52 (order matters) */
enum {
    SPYB_OP_INPUT = 0, SPYB_OP_NOP = 1, SPYB_OP_DUP = 2, SPYB_OP_COPY = 3, SPYB_OP_VIEW = 4, SPYB_OP_RESHAPE = 5,
    SPYB_OP_GETROW = 8, SPYB_OP_TRANSPOSE = 9, SPYB_OP_PERMUTE = 10, SPYB_OP_CONTIGUOUS = 11, SPYB_OP_SILU = 13,
    SPYB_OP_SOFTMAX = 17, SPYB_OP_ADD = 18, SPYB_OP_MUL = 20, SPYB_OP_MATMUL = 23, SPYB_OP_NORM_RMS = 26,
    SPYB_OP_ROPE = 27
};

/* DataNodeType, orchestration/include/graph/data_node.h:12-36 */
enum { SPYB_NODE_CONSTANT = 0, SPYB_NODE_IO = 1, SPYB_NODE_CACHE = 2, SPYB_NODE_DYNAMIC = 6 };

typedef struct spyb_backend spyb_backend;
typedef struct spyb_model   spyb_model;

/* Backend configuration; the string keys of the reference's ConfigTable
 * (util/include/util/wrapper/config_table.h:10-72; GPU key `device_id` at
 * backend/cuda/include/default_backend.h:38-40) become plain fields. */
typedef struct {
    int32_t device_id;     /* CUDA device ordinal */
    int32_t tp_size;       /* tensor-parallel world size, 1 = single GPU */
    int32_t tp_rank;       /* this process's rank in [0, tp_size) */
    int32_t use_pdl;       /* 1 = programmatic dependent launch between the kernels of a step */
    int32_t use_graph;     /* 1 = replay decode steps from a captured CUDA graph */
    int32_t reserved;
    uint64_t arena_bytes;  /* size of the device arena behind spyb_alloc, 0 = default (256 MiB) */
} spyb_config;

/* Tensor as an operator sees it: Shape + data pointer
 * (orchestration/include/number/tensor.h:23-263). `bytes` are byte strides; bytes[0] is the
 * size of one block of `number_type`. `node_type` tells host (IO) from device pointers. */
typedef struct {
    int32_t number_type;
    uint32_t dim;
    int64_t elements[4];
    int64_t bytes[4];
    void   *data;
    int32_t node_type;
    int32_t reserved;
} spyb_tensor;

/* RopeParam, orchestration/include/operator/non-linear.h:191-207 */
typedef struct {
    int32_t mode, num_past, num_dim, num_context, num_origin_context;
    float   freq_base, freq_scale, extend_factor, attention_factor, beta_fast, beta_slow, xpos_base;
    int32_t xpos_down;
} spyb_rope_param;

/* One operator node as Backend::submit receives it
 * (backend/interface/include/backend/backend.h:94; operand contract in
 * orchestration/include/graph/op_node.h:11-60). */
typedef struct {
    int32_t op_type;
    int32_t num_input;
    spyb_tensor input[3];
    spyb_tensor output;
    float   softmax_scale;     /* SoftmaxParam,  operator/non-linear.h:45 */
    float   norm_eps;          /* NormRMSParam,  operator/non-linear.h:117 */
    int64_t view_offset;       /* ViewParam,     operator/view.h:333-336 */
    spyb_rope_param rope;
} spyb_op_desc;

/* ---- backend object: BackendFactory::init_backend + Backend ctor/dtor (backend.h:31-40, 109-117) */
spyb_status spyb_create(const spyb_config *config, spyb_backend **out);
void        spyb_destroy(spyb_backend *backend);
/* message of the last failure on this backend ("" if none); replaces the reference's
 * spy_assert/std::terminate error path (util/include/util/log/logger.h:96-150) */
const char *spyb_last_error(const spyb_backend *backend);

/* Host-only self-check of the library's book-keeping (per-device shared-memory limits of the kernels) and of the e4m3 codes
 * the prompt GEMM feeds the tensor cores (every code decodes to its integer, every 8-bit value is the sum of its two
 * parts); needs no GPU. 0 = passed. No reference counterpart. */
int32_t spyb_selftest_host(void);

/* ---- Backend::get_max/avail_memory_capacity (backend.h:46-51) */
uint64_t spyb_max_memory(const spyb_backend *backend);
uint64_t spyb_avail_memory(const spyb_backend *backend);

/* ---- Backend::alloc_memory / dealloc_memory (backend.h:59-67): device memory, thread-safe */
void *spyb_alloc(spyb_backend *backend, uint64_t bytes);
void  spyb_free(spyb_backend *backend, void *ptr, uint64_t bytes);

/* ---- Backend::is_support (backend.h:87) */
int32_t spyb_is_support(int32_t op_type);

/* ---- ModelLoader::load for a Constant tensor (storage/include/loader/simple_loader.h:57-70):
 * copies the tensor's raw blocks to the device once and returns the device pointer that
 * stands in for the loader's host span. Repeated calls with the same name, host span and size return the same pointer. */
void *spyb_upload_constant(spyb_backend *backend, const char *name, const void *host_ptr, uint64_t bytes,
                           int32_t number_type, const int64_t elements[4]);

/* ---- Backend::submit (backend.h:94): enqueues one operator on the backend's stream.
 * View-type operators (operator/type.h:115-126) write the aliased pointer to desc->output.data.
 * `callback(user)` runs on a backend thread once the operator has finished on the device; NULL = none. */
spyb_status spyb_submit(spyb_backend *backend, spyb_op_desc *desc, void (*callback)(void *), void *user);
/* waits for everything submitted so far */
spyb_status spyb_sync(spyb_backend *backend);
/* (Entry points that exist for measurement only - timed submits, single-kernel timing, kernel time stamps - are left out of a
 * library built with -DSPYB_NO_MEASUREMENT_AIDS.) */
#ifndef SPYB_NO_MEASUREMENT_AIDS
/* measurement aid: submits descs[0], descs[1], ... round-robin `repeats` times (no callbacks; device-resident operands) between
 * two events on the backend's stream and returns the device time of the whole sequence in milliseconds. Passing several
 * descriptors whose operands together exceed the L2 cache gives cold-cache figures for a single operator. */
spyb_status spyb_submit_timed(spyb_backend *backend, spyb_op_desc *descs, int32_t n_descs, int32_t repeats, float *ms_out);
#endif

/* ---- staging of IO tensors, which the reference keeps in host vectors (model/src/llm/model/llama.cpp:259-263) */
spyb_status spyb_memcpy_h2d(spyb_backend *backend, void *dst_device, const void *src_host, uint64_t bytes);
spyb_status spyb_memcpy_d2h(spyb_backend *backend, void *dst_host, const void *src_device, uint64_t bytes);

/* ---- single kernels exposed for parity checks of the arithmetic the reference pins exactly */
/* Quantizator<FP32,Q8_0>::transform (backend/host/include/simd/vec_convert.h:178-261):
 * n floats on the device -> n/32 blocks of 34 bytes in the reference layout */
spyb_status spyb_quantize_q8_0(spyb_backend *backend, const float *x_device, int64_t n, void *blocks_device);
/* per-block int32 dots of one Q4_0 / Q8_0 weight row against one Q8_0 activation column
 * (Dot<Q4_0,Q8_0>::exec / Dot<Q8_0,Q8_0>::exec, backend/host/include/simd/vec_dot.h:42-115), all pointers
 * to raw reference-layout blocks on the device, out: n/32 int32 */
spyb_status spyb_block_dots(spyb_backend *backend, int32_t weight_type, const void *w_row_device,
                            const void *x_blocks_device, int64_t n, int32_t *out_device);

/* Copies of the two 65 536-entry fp16-argument tables the device kernels gather from, silu(xh) and expf(xh)
 * (FP16LookupTable, orchestration/include/number/lookup_table.h:12-54); either pointer may be NULL. */
spyb_status spyb_read_tables(spyb_backend *backend, float *silu_host, float *exp_host);

/* The attention sub-graph of one layer for n_tokens query tokens at positions pos0..pos0+n_tokens-1 over caller-provided
 * caches, all on the device: MatMul(K, Q) -> masked Softmax(scale = 1/sqrt(head_dim)) -> MatMul(V, probs)
 * (MultiHeadAttentionBlock::attention_projection, model/src/llm/plugin/attention.cpp:102-132, with the causal mask of
 * model/src/llm/model/llama.cpp:248-257). q: fp16 [n_tokens][n_head*head_dim]; k_cache: fp16 [n_ctx][n_head*head_dim];
 * v_cache_t: fp16 [n_head*head_dim][n_ctx] (transposed, model/src/llm/plugin/attention.cpp:228-262); out: f32 like q.
 * n_total = number of positions the step knows (n_past + all tokens of the step, the row length of the reference's score
 * tensor; 0 = pos0 + n_tokens): masked entries are exact zeros but take part in the grouping of the reference's sums. */
spyb_status spyb_attention(spyb_backend *backend, const void *q_f16, const void *k_cache_f16, const void *v_cache_t_f16, float *out,
                           int32_t pos0, int32_t n_tokens, int32_t n_total, int32_t n_head, int32_t head_dim, int32_t n_ctx);

/* MatMul of quantized weights in the reference's row layout (Q4_0 / Q8_0 blocks, [n_rows][k], device memory) with f32
 * activations x [n_cols][k], out [n_cols][n_rows] - the same arithmetic and bits as a MatMul submitted through spyb_submit -
 * for callers that may not allocate. No reference counterpart: the reference's CPU MatMul takes its scratch from the
 * scheduler's allocator.
 *
 * Who needs it: a caller that replays its own CUDA graph or runs inside a stream capture (cudaMalloc and cudaFree are
 * illegal there and would invalidate the capture), or a serving loop that has handed all device memory to its own pool
 * and must not see the allocator's latency or failure in the token loop. spyb_submit re-tiles weights that were not
 * registered with spyb_upload_constant into a temporary buffer taken from the backend's arena (which falls back to
 * cudaMalloc when the arena is full); this entry point re-tiles into a fixed scratch array that is part of the library
 * image instead and calls no allocating routine at all.
 *
 * Limits and rules:
 *  - the re-tiled matrix (n_rows * ceil8(k/32) * 18 or 34 bytes) must fit SPYB_NOALLOC_SCRATCH_BYTES (32 MiB: every
 *    matrix of a 7B layer; the 32000 x 4096 head does not fit) - larger requests are rejected with SPYB_UNSUPPORTED;
 *    n_rows must be a multiple of 4 and k a multiple of 32; x_dev must be 16-byte aligned (the kernels read it with
 *    128-bit loads), out_dev 4-byte and w_rows_dev 2-byte aligned - anything else is rejected with SPYB_UNSUPPORTED
 *    before a kernel is launched (the same rule holds for MatMul operands passed to spyb_submit);
 *  - the first call on a device looks the scratch array's address up and raises the kernels' shared-memory limit for
 *    the given shape: make one call per shape before a stream capture begins, later calls only enqueue kernels on the
 *    backend's stream (they do not synchronise; use spyb_sync);
 *  - there is ONE scratch array per device and process: calls are safe one after the other on the backend's stream
 *    (stream order keeps a call's kernels ahead of the next call's re-tiling); two backends on the same device, or any
 *    other concurrent use, would race on it. Nothing needs clearing between calls: a call writes every byte it later
 *    reads, padding included. */
#define SPYB_NOALLOC_SCRATCH_BYTES (32u << 20)
spyb_status spyb_matmul_noalloc(spyb_backend *backend, int32_t weight_type, const void *w_rows_dev, int64_t n_rows, int64_t k,
                                const float *x_dev, int64_t n_cols, float *out_dev);

/* MatMul(W[Q4_0 | Q8_0], x) for a prompt of n_cols tokens on the tensor cores - the operator the reference evaluates as
 * n_cols x n_rows independent dot products (OperatorMatMul, backend/host/operator/mat.cpp:95-128, Dot<Q4_0,Q8_0> /
 * Dot<Q8_0,Q8_0>, backend/host/include/simd/vec_dot.h:42-115), with the same f32 arithmetic and order, so the result is
 * bit-identical to spyb_submit(MatMul) and to the CPU backend. The integer lane sums of a block come from one
 * tcgen05 MMA per tile of 128 rows x 16 tokens; the f32 chains follow in block order.
 *   w_rows_host : n_rows rows of k / 32 blocks in GGUF order (18 or 34 bytes per block), host memory
 *   x_host      : [n_cols][k] f32; norm_w_host (optional, [k]): RMSNorm(x) * norm_w is applied first, as in front of
 *                 the QKV and FFN MatMuls of the graph (eps as in NormRMS)
 *   out_host    : [n_cols][n_rows] f32
 * Needs k a multiple of 32 (256 for Q4_K / Q6_K; <= 14336) and 1..4096 columns; anything else is SPYB_UNSUPPORTED.
 * Stages everything inside the call (it allocates and synchronises): the entry point of the parity tests, while
 * spyb_model_eval runs the same kernels on resident buffers for prompts of SPYB_PREFILL_MIN_TOKENS tokens and more. */
#define SPYB_PREFILL_MIN_TOKENS 16
spyb_status spyb_prefill_matmul(spyb_backend *backend, int32_t weight_type, const void *w_rows_host, int64_t n_rows, int64_t k,
                                const float *x_host, int64_t n_cols, const float *norm_w_host, float eps, float *out_host);

/* Failure-path check of the prompt kernel that faults nothing: a small launch whose second batch of blocks is never
 * copied, with `limit_ns` as the bound of every wait. Succeeds when the kernel returned by itself and recorded one of
 * its codes (4 = a shared-memory stage, 5 = operands or a free accumulator buffer, 6 = a tensor-core result; also
 * written to *error_code_out); the record is cleared again, so the backend stays usable. No reference counterpart. */
spyb_status spyb_prefill_selftest_wait_timeout(spyb_backend *backend, uint64_t limit_ns, int32_t *error_code_out);

/* ---- whole-model path: the graph LLAMAModel::build_graph emits (model/src/llm/model/llama.cpp:86-264)
 * executed as a fixed plan of fused kernels. */
typedef struct {
    int32_t n_layer, d_model, n_head, n_ff, n_vocab, n_ctx, head_dim;
    int32_t tp_size, tp_rank;
    float   rms_eps, rope_base;
    uint64_t weight_bytes;        /* quantized weight bytes resident on this GPU */
    uint64_t kv_bytes_per_token;  /* KV-cache bytes appended per token on this GPU */
} spyb_model_info;

/* GGUFAdapter::init_from_file + SimpleModeLoader::preload (storage/src/adapter/gguf_adapter.cpp:90-190,
 * storage/include/loader/simple_loader.h:36-55) followed by the upload of every tensor's quantized
 * blocks to device memory; with tp_size > 1 only this rank's shard (heads / FFN columns) is kept. */
spyb_status spyb_model_load_gguf(spyb_backend *backend, const char *path, int32_t n_ctx, spyb_model **out);
void        spyb_model_free(spyb_model *model);
spyb_status spyb_model_info_get(const spyb_model *model, spyb_model_info *info);
/* attach an NCCL communicator for tensor parallelism: `unique_id` is the 128-byte ncclUniqueId
 * every rank received from rank 0 (spyb_nccl_unique_id) */
spyb_status spyb_nccl_unique_id(void *unique_id_128);
spyb_status spyb_model_init_tp(spyb_model *model, const void *unique_id_128);

/* The tensor-parallel partition of a layer, as spyb_model_load_gguf cuts it (host arithmetic only, no GPU needed):
 * out[0], out[1] = first row and number of rows of Wq, Wk and Wv this rank holds (whole heads; also its share of the
 * gathered attention output), out[2], out[3] = the same for W_up and W_gate (its share of the gathered FFN activation).
 * Wo and W_down are replicated: they consume the gathered vectors, so no f32 sum is split across ranks and the
 * tensor-parallel results are the single-GPU bits. SPYB_FAIL when tp_size does not divide the heads or the FFN width
 * into whole 32-element blocks. No reference counterpart (backend/distributor's graph divider is empty). */
spyb_status spyb_tp_layer_shard(int32_t d_model, int32_t n_head, int32_t n_ff, int32_t tp_size, int32_t tp_rank, int64_t out[4]);

/* Tensor parallel, optional: the all-gather of the attention output and the FFN activation through peer memory inside
 * the kernels (plain peer stores and flag words, bounded waits) instead of NCCL all-gathers. No reference counterpart
 * (the reference has no multi-device path). Every rank calls spyb_model_tp_export (a 64-byte CUDA IPC handle of its
 * exchange buffer), the handles are gathered over the caller's channel in rank order, and every rank calls
 * spyb_model_tp_import with the tp_size * 64 bytes. Without these calls the NCCL path is used throughout. */
spyb_status spyb_model_tp_export(spyb_model *model, void *handle_64);
spyb_status spyb_model_tp_import(spyb_model *model, const void *handles);

/* One distributor->execute() (backend/distributor/include/distributor/simple_distributor.h:47-78)
 * for `n_tokens` host token ids at positions n_past..n_past+n_tokens-1: host ids in, the last
 * token's n_vocab logits out to host memory (as model_io.logits, app/cli/include/cli.h:103-105). */
spyb_status spyb_model_eval(spyb_model *model, const int32_t *tokens_host, int32_t n_tokens, int32_t n_past,
                            float *logits_host);
/* The decode loop of AutoModelGenerator::generate (app/cli/include/cli.h:88-128) kept on the device:
 * `n_steps` single-token steps starting from `first_token` at position n_past, greedy argmax
 * (SamplerImpl<Greedy>, model/include/llm/sampler/greedy.h:20-25) on the device feeding the next step;
 * only the token ids come back. logits_host (optional) receives n_steps * n_vocab floats. */
spyb_status spyb_model_decode(spyb_model *model, int32_t first_token, int32_t n_past, int32_t n_steps,
                              int32_t *ids_host, float *logits_host);
/* Bound, in nanoseconds, of every device-side wait of the single-token step kernel (grid barriers, shared-memory stage
 * barriers); default 1 s. When a wait runs out the kernel records a code (1 = a bulk copy did not land, 2 = a barrier or
 * another rank's result did not arrive), lets its copies in flight land and returns; the call that synchronises next
 * returns SPYB_FAIL with that text in spyb_last_error, and the backend has to be re-created. Stands in for the
 * reference's only failure path, spy_assert -> std::terminate (backend/host/include/default_backend.h:75-78). */
spyb_status spyb_set_wait_limit_ns(spyb_backend *backend, uint64_t ns);
/* Failure-path check that faults nothing: runs one step whose first grid barrier expects one arrival more than there
 * are CTAs, with `limit_ns` as the bound. Succeeds when the kernel returned by itself and recorded code 2 (also written
 * to *error_code_out); the record is cleared again, so the model stays usable. No reference counterpart. */
spyb_status spyb_model_selftest_wait_timeout(spyb_model *model, uint64_t limit_ns, int32_t *error_code_out);
/* ---- batches of independent sequences (no reference counterpart: the reference decodes one sequence; the batch > 1
 * configurations are replicas of it that share the weights, so every sequence must give the bits of a run on its own).
 * spyb_model_set_sequences gives the model n_seq KV caches (1..64; unsharded Q4_0 / Q8_0 models); spyb_model_select_sequence
 * makes spyb_model_eval / spyb_model_decode act on one of them (e.g. to evaluate each sequence's prompt);
 * spyb_model_decode_batch then decodes sequences 0 .. n_seq-1 greedily in lockstep from the common position n_past
 * (all prompts must have that length): per step the layer weights are streamed once per group of activation columns
 * instead of once per sequence. ids_host receives [n_steps][n_seq] token ids, logits_host (optional)
 * [n_steps][n_seq][n_vocab] floats. */
spyb_status spyb_model_set_sequences(spyb_model *model, int32_t n_seq);
spyb_status spyb_model_select_sequence(spyb_model *model, int32_t seq);
spyb_status spyb_model_decode_batch(spyb_model *model, const int32_t *first_tokens, int32_t n_seq, int32_t n_past, int32_t n_steps,
                                    int32_t *ids_host, float *logits_host);
/* device time in milliseconds of the most recent spyb_model_decode / spyb_model_eval call,
 * measured with CUDA events on the backend's stream; number of kernels that call launched */
float   spyb_model_last_ms(const spyb_model *model);
int64_t spyb_model_last_launches(const spyb_model *model);
#ifndef SPYB_NO_MEASUREMENT_AIDS
/* Measurement aid: launches one kind of mat-vec kernel of the plan alone, `sweeps` times over every layer's
 * weights back to back (kind 0 = Wq|Wk|Wv, 1 = attention output, 2 = FFN up+gate, 3 = FFN down, 4 = output head),
 * and returns the average device time per launch in milliseconds (CUDA events on the backend's stream);
 * *bytes_per_launch receives the quantized weight bytes one launch streams. Scratch activations only:
 * the KV cache below position n_ctx-1 and the residual stream are left untouched. No reference counterpart
 * (the reference times whole steps only, util/include/util/timer.h:51-80). */
float spyb_model_bench_kernel(spyb_model *model, int32_t kind, int32_t sweeps, uint64_t *bytes_per_launch);
#endif
/* Parity tap: copies one activation buffer of the last pass (up to 8 token columns) to the host:
 * which 0 = Q after RoPE as fp16 [T][d_local], 1 = attention output f32 [T][d_local], 2 = residual stream f32 [T][d_model],
 * 3 = up*silu(gate) f32 [T][ff_local], 4 = logits f32 [n_vocab]; the layer buffers hold the LAST layer's values.
 * Stands in for reading Dynamic tensors of the reference graph (orchestration/include/graph/data_node.h:38-73). */
spyb_status spyb_model_read_activation(spyb_model *model, int32_t which, void *host, uint64_t bytes);
/* taps for parity tests: copy the Q8_0 blocks of layer-0's attention-norm output of the last eval
 * (d_model/32 * 34 bytes, reference layout) to host */
spyb_status spyb_model_tap_xq(spyb_model *model, void *blocks_host);

#ifndef SPYB_NO_MEASUREMENT_AIDS
/* Profiling aid without a reference counterpart. When the model was loaded with SPYB_TIMELINE=1 in the
 * environment, every kernel of the step plan records eight device-clock stamps (ns): CTA 0 started,
 * its predecessor finished, its activations quantized, last CTA finished, then the latest CTA's start,
 * predecessor-finished and activations-quantized times, and one unused word. Copies up to max_kernels records of
 * eight stamps (layer-major: QKV, attention, attention-out, FFN up/gate, FFN down; then the head) and
 * returns their number (0 when the timeline is off). */
int32_t spyb_model_read_timeline(spyb_model *model, uint64_t *stamps_host, int32_t max_kernels);
/* The same for single-token steps that run as one persistent kernel: pairs (CTA 0's time, the latest CTA's time) at
 * every check point of the step - kernel entry, then per layer: barrier passed / activations quantized / mat-vec done for
 * Wq|Wk|Wv, attention begun / done, and the same triples for Wo, up|gate and down, finally the head. Returns the number of pairs. */
int32_t spyb_model_read_step_timeline(spyb_model *model, uint64_t *stamps_host, int32_t max_points);
#endif

#ifdef __cplusplus
}
#endif
#endif /* SPYB_H_ */
