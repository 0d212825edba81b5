// The backend object and the per-operator path of the C ABI: memory, constants, submit.
// This is the part that stands in for the reference's DefaultGPUBackend
// (backend/cuda/include/default_backend.h:22-99) behind Backend::{alloc_memory, dealloc_memory, submit}.

#include <cmath>
#include <cstring>

#include "spyb_common.cuh"
#include "spyb_internal.h"

namespace spyb {

// ------------------------------------------------------------------------------------------ arena
bool Arena::init(size_t bytes) {
    capacity_ = (bytes + ALIGN - 1) / ALIGN * ALIGN;
    if (cudaMalloc(reinterpret_cast<void **>(&base_), capacity_) != cudaSuccess) { base_ = nullptr; capacity_ = 0; return false; }
    free_.clear();
    free_[0] = capacity_;
    return true;
}

void Arena::destroy() {
    for (auto &kv : overflow_) { cudaFree(kv.first); }
    overflow_.clear();
    if (base_) { cudaFree(base_); base_ = nullptr; }
    capacity_ = 0;
    free_.clear();
}

void *Arena::alloc(size_t bytes) {
    if (bytes == 0) { bytes = 1; }
    const size_t need = (bytes + ALIGN - 1) / ALIGN * ALIGN;
    std::lock_guard<std::mutex> g(mutex_);
    for (auto it = free_.begin(); it != free_.end(); ++it) {
        if (it->second >= need) {
            const size_t off = it->first, rest = it->second - need;
            free_.erase(it);
            if (rest) { free_[off + need] = rest; }
            return base_ + off;
        }
    }
    void *p = nullptr;   // arena exhausted: fall back to the CUDA allocator rather than fail
    if (cudaMalloc(&p, need) != cudaSuccess) { return nullptr; }
    overflow_[p] = need;
    return p;
}

void Arena::free(void *ptr, size_t bytes) {
    if (ptr == nullptr) { return; }
    std::lock_guard<std::mutex> g(mutex_);
    auto ov = overflow_.find(ptr);
    if (ov != overflow_.end()) { cudaFree(ptr); overflow_.erase(ov); return; }
    if (bytes == 0) { bytes = 1; }
    size_t off = static_cast<uint8_t *>(ptr) - base_, size = (bytes + ALIGN - 1) / ALIGN * ALIGN;
    auto next = free_.lower_bound(off);
    if (next != free_.begin()) {
        auto prev = std::prev(next);
        if (prev->first + prev->second == off) { off = prev->first; size += prev->second; free_.erase(prev); }
    }
    if (next != free_.end() && off + size == next->first) { size += next->second; free_.erase(next); }
    free_[off] = size;
}

size_t Arena::available() {
    std::lock_guard<std::mutex> g(mutex_);
    size_t tot = 0;
    for (auto &kv : free_) { tot += kv.second; }
    return tot;
}

// ------------------------------------------------------------------------------------------ matrices
spyb_status alloc_matrix(spyb_backend *be, int type, int64_t n_rows, int nb, DevMatrix *out, int tile_rows, int mma) {
    if (type != SPYB_Q4_0 && type != SPYB_Q8_0) { be->set_error("weight type %d has no device layout", type); return SPYB_UNSUPPORTED; }
    if ((tile_rows != 4 && tile_rows != 8 && tile_rows != 16 && tile_rows != 32) || n_rows % tile_rows != 0) { be->set_error("quantized matrices need a multiple of %d rows (got %lld)", tile_rows, (long long)n_rows); return SPYB_UNSUPPORTED; }
    DevMatrix m;
    m.type = type; m.n_rows = n_rows; m.nb = nb; m.nbp = padded_blocks(nb); m.k = (int64_t)nb * QK; m.tile_rows = tile_rows;
    m.mma = (mma != 0 && (tile_rows == 8 || tile_rows == 16)) ? 1 : 0;
    void *w = nullptr;
    SPYB_CUDA(be, cudaMalloc(&w, matrix_bytes(type, n_rows, nb) + 16));
    be->owned.push_back(w);
    m.w = static_cast<const uint8_t *>(w);
    *out = m;
    return SPYB_SUCCESS;
}

spyb_status upload_matrix(spyb_backend *be, int type, const uint8_t *host_rows, int64_t n_rows, int64_t row_stride_bytes,
                          int64_t blk0, int nb, DevMatrix *out, const DevMatrix *into, int64_t dst_row, int sub_rows, int sub_off) {
    if (into == nullptr) {
        spyb_status st = alloc_matrix(be, type, n_rows, nb, out, 4);
        if (st != SPYB_SUCCESS) { return st; }
        into = out; dst_row = 0; sub_rows = 0; sub_off = 0;
    } else {
        const int64_t last = sub_rows > 0 ? dst_row + (n_rows / sub_rows) * into->tile_rows : dst_row + n_rows;
        if (into->type != type || into->nb != nb || last > into->n_rows || (sub_rows > 0 && (n_rows % sub_rows != 0 || sub_off + sub_rows > into->tile_rows))) {
            be->set_error("weight upload: destination rows do not match"); return SPYB_FAIL;
        }
    }
    const int     bb = (type == SPYB_Q4_0) ? 18 : 34;
    const int64_t max_rows = std::max<int64_t>(1, (int64_t)(64u << 20) / row_stride_bytes);   // 64 MiB staging pieces
    void *stage = nullptr;
    SPYB_CUDA(be, cudaMalloc(&stage, (size_t)std::min(max_rows, n_rows) * row_stride_bytes + 64));
    for (int64_t r0 = 0; r0 < n_rows; r0 += max_rows) {
        const int64_t nr = std::min(max_rows, n_rows - r0);
        cudaError_t err = cudaMemcpyAsync(stage, host_rows + r0 * row_stride_bytes, (size_t)nr * row_stride_bytes, cudaMemcpyHostToDevice, be->stream);
        if (err == cudaSuccess) {
            const uint8_t *raw = static_cast<const uint8_t *>(stage) + blk0 * bb;
            err = launch_retile(type, raw, row_stride_bytes, nr, nb, const_cast<uint8_t *>(into->w), into->tile_rows, into->mma != 0, dst_row, r0, sub_rows, sub_off, be->stream);
        }
        if (err == cudaSuccess) { err = cudaStreamSynchronize(be->stream); }
        if (err != cudaSuccess) { cudaFree(stage); be->set_error("weight upload failed: %s", cudaGetErrorString(err)); return SPYB_FAIL; }
    }
    cudaFree(stage);
    return SPYB_SUCCESS;
}

static void callback_worker(spyb_backend *be) {
    cudaSetDevice(be->config.device_id);
    for (;;) {
        PendingCallback cb;
        {
            std::unique_lock<std::mutex> g(be->cb_mutex);
            be->cb_cv.wait(g, [be] { return be->cb_stop || !be->cb_queue.empty(); });
            if (be->cb_queue.empty()) { return; }
            cb = be->cb_queue.front();
            be->cb_queue.pop_front();
        }
        cudaEventSynchronize(cb.event);
        cudaEventDestroy(cb.event);
        cb.fn(cb.user);
    }
}

static int64_t type_block_bytes(int t) {
    switch (t) { case SPYB_FP32: return 4; case SPYB_FP16: return 2; case SPYB_INT32: return 4; case SPYB_Q4_0: return 18; case SPYB_Q8_0: return 34;
                 case SPYB_Q4_K: return 144; case SPYB_Q6_K: return 210; default: return -1; }
}
static int64_t type_block_elems(int t) {
    switch (t) { case SPYB_Q4_0: case SPYB_Q8_0: return 32; case SPYB_Q4_K: case SPYB_Q6_K: return 256; default: return 1; }
}
static int64_t tensor_elems(const spyb_tensor &t) { return t.elements[0] * t.elements[1] * t.elements[2] * t.elements[3]; }
// Shape::total_size, orchestration/include/number/tensor.h:137-143
static int64_t tensor_total_size(const spyb_tensor &t) {
    int64_t size = t.bytes[0] * t.elements[0] / type_block_elems(t.number_type);
    for (uint32_t i = 1; i < t.dim && i < 4; ++i) { size += t.bytes[i] * (t.elements[i] - 1); }
    return size;
}
static bool tensor_contiguous(const spyb_tensor &t) {
    const int64_t bs = type_block_bytes(t.number_type), be = type_block_elems(t.number_type);
    return t.bytes[0] == bs && t.bytes[1] == bs * t.elements[0] / be && t.bytes[2] == t.bytes[1] * t.elements[1] &&
           t.bytes[3] == t.bytes[2] * t.elements[2];
}
static Strided to_strided(const spyb_tensor &t, void *data) {
    Strided s; s.data = data;
    for (int i = 0; i < 4; ++i) { s.ne[i] = t.elements[i]; s.nb[i] = t.bytes[i]; }
    return s;
}

}  // namespace spyb

using namespace spyb;

extern "C" {

int32_t spyb_selftest_host(void) {
    const int a = smem_ledger_selftest();
    return a != 0 ? a : prefill_e4m3_selftest();
}

spyb_status spyb_create(const spyb_config *config, spyb_backend **out) {
    if (config == nullptr || out == nullptr) { return SPYB_FAIL; }
    *out = nullptr;
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev == 0) { return SPYB_FAIL; }   // no CPU fallback exists
    if (config->device_id < 0 || config->device_id >= n_dev) { return SPYB_FAIL; }
    if (cudaSetDevice(config->device_id) != cudaSuccess) { return SPYB_FAIL; }
    spyb_backend *be = new spyb_backend();
    be->config = *config;
    if (be->config.tp_size < 1) { be->config.tp_size = 1; }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, config->device_id) != cudaSuccess) { delete be; return SPYB_FAIL; }
    be->num_sms = prop.multiProcessorCount;
    be->num_sms_total = prop.multiProcessorCount;
    be->smem_optin = prop.sharedMemPerBlockOptin;
    // CTAs of a mat-vec grid: a few SMs fewer than the chip has. The next kernel's CTAs then never have to wait for the
    // SMs of the previous kernel's last CTAs (they are launched, and have their rings filling, before the previous
    // kernel ends); measured on B200: 140 of 148 gives 1 % more tokens/s than 148, 132 less again.
    if (be->num_sms >= 128) { be->num_sms -= 8; }
    if (const char *v = std::getenv("SPYB_MV_SMS")) { const int n = std::atoi(v); if (n > 0 && n <= prop.multiProcessorCount) { be->num_sms = n; } }
    if (const char *v = std::getenv("SPYB_MV_CTAS_PER_SM")) { be->mv_ctas_per_sm = std::max(1, std::min(2, std::atoi(v))); }   // tuning knob
    if (const char *v = std::getenv("SPYB_MV_S")) { be->mv_force_s = std::atoi(v); }         // tuning knobs
    if (const char *v = std::getenv("SPYB_MV_WACT")) { be->mv_force_wact = std::atoi(v); }
    if (const char *v = std::getenv("SPYB_MV_RING_KB")) { be->mv_ring_kb = std::max(8, std::min(96, std::atoi(v))); }   // tuning knob
    if (cudaStreamCreateWithFlags(&be->stream, cudaStreamNonBlocking) != cudaSuccess) { delete be; return SPYB_FAIL; }
    if (cudaHostAlloc(reinterpret_cast<void **>(&be->h_error_flag), sizeof(int), cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer(reinterpret_cast<void **>(&be->d_error_flag), be->h_error_flag, 0) != cudaSuccess) {
        cudaStreamDestroy(be->stream); delete be; return SPYB_FAIL;
    }
    *be->h_error_flag = 0;
    const size_t arena = config->arena_bytes ? config->arena_bytes : (size_t)256 << 20;
    if (!be->arena.init(arena)) { cudaStreamDestroy(be->stream); delete be; return SPYB_FAIL; }

    // fp16-argument tables, built with the host libm exactly as the reference builds them
    // (orchestration/include/number/lookup_table_impl/non-linear.h:42-47, 134-139); key 0xFFFF stays 0.
    std::vector<float> silu(65536, 0.f), ex(65536, 0.f);
    for (uint32_t k = 0; k < 65535; ++k) {
        _Float16 hv; const uint16_t kk = (uint16_t)k; std::memcpy(&hv, &kk, 2);
        const float x = (float)hv;
        silu[k] = x / (1.0f + std::exp(-x));
        ex[k]   = std::exp(x);
    }
    bool ok = cudaMalloc(reinterpret_cast<void **>(&be->d_silu_table), 65536 * 4) == cudaSuccess &&
              cudaMalloc(reinterpret_cast<void **>(&be->d_exp_table), 65536 * 4) == cudaSuccess &&
              cudaMemcpy(be->d_silu_table, silu.data(), 65536 * 4, cudaMemcpyHostToDevice) == cudaSuccess &&
              cudaMemcpy(be->d_exp_table, ex.data(), 65536 * 4, cudaMemcpyHostToDevice) == cudaSuccess;
    if (!ok) { spyb_destroy(be); return SPYB_FAIL; }
    be->cb_thread = std::thread(callback_worker, be);
    *out = be;
    return SPYB_SUCCESS;
}

void spyb_destroy(spyb_backend *be) {
    if (be == nullptr) { return; }
    cudaSetDevice(be->config.device_id);
    if (be->stream) { cudaStreamSynchronize(be->stream); }
    if (be->cb_thread.joinable()) {
        { std::lock_guard<std::mutex> g(be->cb_mutex); be->cb_stop = true; }
        be->cb_cv.notify_all();
        be->cb_thread.join();
    }
    for (void *p : be->owned) { cudaFree(p); }
    if (be->d_silu_table) { cudaFree(be->d_silu_table); }
    if (be->d_exp_table) { cudaFree(be->d_exp_table); }
    if (be->h_error_flag) { cudaFreeHost(be->h_error_flag); }
    be->arena.destroy();
    if (be->stream) { cudaStreamDestroy(be->stream); }
    delete be;
}

const char *spyb_last_error(const spyb_backend *be) {
    if (be == nullptr) { return "no backend (no CUDA device, or creation failed)"; }
    return be->last_error.c_str();
}

uint64_t spyb_max_memory(const spyb_backend *be) {
    size_t free_b = 0, total = 0;
    cudaSetDevice(be->config.device_id);
    cudaMemGetInfo(&free_b, &total);
    return total;
}
uint64_t spyb_avail_memory(const spyb_backend *be) {
    size_t free_b = 0, total = 0;
    cudaSetDevice(be->config.device_id);
    cudaMemGetInfo(&free_b, &total);
    return free_b + const_cast<spyb_backend *>(be)->arena.available();
}

void *spyb_alloc(spyb_backend *be, uint64_t bytes) {
    cudaSetDevice(be->config.device_id);
    void *p = be->arena.alloc(bytes);
    if (p == nullptr) { be->set_error("out of device memory allocating %llu bytes", (unsigned long long)bytes); }
    return p;
}
void spyb_free(spyb_backend *be, void *ptr, uint64_t bytes) { be->arena.free(ptr, bytes); }

int32_t spyb_is_support(int32_t op) {
    switch (op) {
    case SPYB_OP_INPUT: case SPYB_OP_NOP: case SPYB_OP_DUP: case SPYB_OP_COPY: case SPYB_OP_VIEW: case SPYB_OP_RESHAPE:
    case SPYB_OP_GETROW: case SPYB_OP_TRANSPOSE: case SPYB_OP_PERMUTE: case SPYB_OP_CONTIGUOUS: case SPYB_OP_SILU:
    case SPYB_OP_SOFTMAX: case SPYB_OP_ADD: case SPYB_OP_MUL: case SPYB_OP_MATMUL: case SPYB_OP_NORM_RMS: case SPYB_OP_ROPE:
        return 1;
    default:
        return 0;
    }
}

void *spyb_upload_constant(spyb_backend *be, const char *name, const void *host_ptr, uint64_t bytes, int32_t number_type,
                           const int64_t elements[4]) {
    cudaSetDevice(be->config.device_id);
    std::lock_guard<std::mutex> g(be->const_mutex);
    // a constant is identified by its name together with the host span it came from: another model loaded later under
    // the same tensor names (a different mapping or size) is uploaded afresh
    const std::string key = std::string(name) + "@" + std::to_string(reinterpret_cast<uintptr_t>(host_ptr)) + "+" + std::to_string(bytes);
    auto it = be->constants.find(key);
    if (it != be->constants.end()) { return it->second; }
    void *raw = nullptr;
    if (cudaMalloc(&raw, bytes + 64) != cudaSuccess) { be->set_error("cudaMalloc(%llu) failed for constant %s", (unsigned long long)bytes, name); return nullptr; }
    be->owned.push_back(raw);
    if (cudaMemcpy(raw, host_ptr, bytes, cudaMemcpyHostToDevice) != cudaSuccess) { be->set_error("upload of %s failed", name); return nullptr; }
    if ((number_type == SPYB_Q4_0 || number_type == SPYB_Q8_0) && elements != nullptr) {
        // matrices also get the plane layout the mat-vec kernels stream; the raw copy stays for GetRow and parity checks
        const int64_t k = elements[0], rows = elements[1] * elements[2] * elements[3];
        const int64_t bb = number_type == SPYB_Q4_0 ? 18 : 34;
        if (k % QK == 0 && rows > 0 && (rows & 3) == 0) {
            DevMatrix m;
            if (alloc_matrix(be, number_type, rows, (int)(k / QK), &m, 4) != SPYB_SUCCESS) { return nullptr; }
            cudaError_t err = launch_retile(number_type, static_cast<const uint8_t *>(raw), k / QK * bb, rows, m.nb, const_cast<uint8_t *>(m.w), 4, false, 0, 0, 0, 0, be->stream);
            if (err != cudaSuccess || cudaStreamSynchronize(be->stream) != cudaSuccess) { be->set_error("re-tiling of %s failed", name); return nullptr; }
            be->retiled[raw] = m;
        }
    }
    be->constants[key] = raw;
    be->const_types[raw] = number_type;
    return raw;
}

spyb_status spyb_sync(spyb_backend *be) {
    SPYB_CUDA(be, cudaStreamSynchronize(be->stream));
    if (be->device_error()) { return SPYB_FAIL; }
    return SPYB_SUCCESS;
}

spyb_status spyb_memcpy_h2d(spyb_backend *be, void *dst, const void *src, uint64_t bytes) {
    SPYB_CUDA(be, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, be->stream));
    SPYB_CUDA(be, cudaStreamSynchronize(be->stream));
    return SPYB_SUCCESS;
}
spyb_status spyb_memcpy_d2h(spyb_backend *be, void *dst, const void *src, uint64_t bytes) {
    SPYB_CUDA(be, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, be->stream));
    SPYB_CUDA(be, cudaStreamSynchronize(be->stream));
    return SPYB_SUCCESS;
}

spyb_status spyb_quantize_q8_0(spyb_backend *be, const float *x, int64_t n, void *blocks) {
    if (n % QK != 0) { be->set_error("quantize_q8_0: %lld elements is not a multiple of 32", (long long)n); return SPYB_FAIL; }
    SPYB_CUDA(be, launch_quantize_q8_0_ref_layout(x, n, static_cast<uint8_t *>(blocks), be->stream));
    return SPYB_SUCCESS;
}

spyb_status spyb_block_dots(spyb_backend *be, int32_t wtype, const void *w, const void *xb, int64_t n, int32_t *out) {
    if (wtype != SPYB_Q4_0 && wtype != SPYB_Q8_0) { be->set_error("block_dots: unsupported weight type %d", wtype); return SPYB_UNSUPPORTED; }
    SPYB_CUDA(be, launch_block_dots(wtype, static_cast<const uint8_t *>(w), static_cast<const uint8_t *>(xb), n, out, be->stream));
    return SPYB_SUCCESS;
}

spyb_status spyb_read_tables(spyb_backend *be, float *silu_host, float *exp_host) {
    SPYB_CUDA(be, cudaStreamSynchronize(be->stream));
    if (silu_host) { SPYB_CUDA(be, cudaMemcpy(silu_host, be->d_silu_table, 65536 * sizeof(float), cudaMemcpyDeviceToHost)); }
    if (exp_host)  { SPYB_CUDA(be, cudaMemcpy(exp_host, be->d_exp_table, 65536 * sizeof(float), cudaMemcpyDeviceToHost)); }
    return SPYB_SUCCESS;
}

spyb_status spyb_attention(spyb_backend *be, const void *q_f16, const void *k_cache_f16, const void *v_cache_t_f16, float *out,
                           int32_t pos0, int32_t n_tokens, int32_t n_total, int32_t n_head, int32_t head_dim, int32_t n_ctx) {
    if (n_total == 0) { n_total = pos0 + n_tokens; }
    if (n_tokens < 1 || n_head < 1 || pos0 < 0 || pos0 + n_tokens > n_total || n_total > n_ctx) { be->set_error("attention: positions %d..%d outside the context %d", pos0, pos0 + n_tokens - 1, n_ctx); return SPYB_FAIL; }
    int *d_pos = static_cast<int *>(be->arena.alloc(2 * sizeof(int)));
    const int host_pos[2] = {pos0, n_total};
    if (d_pos == nullptr) { be->set_error("attention: out of device memory"); return SPYB_FAIL; }
    AttnParams a;
    a.q = static_cast<const __half *>(q_f16); a.k_cache = static_cast<const __half *>(k_cache_f16); a.v_cache = static_cast<const __half *>(v_cache_t_f16);
    a.out = out; a.pos_base = d_pos; a.exp_table = be->d_exp_table; a.n_head = n_head; a.hd = head_dim; a.dl = n_head * head_dim; a.T = n_tokens; a.n_ctx = n_ctx;
    a.scale = 1.0f / std::sqrt((float)head_dim);
    const size_t scratch_bytes = attention_scratch_floats(n_ctx, n_head, n_tokens) * sizeof(float);
    if (scratch_bytes > 0) {
        a.scratch = static_cast<float *>(be->arena.alloc(scratch_bytes));
        if (a.scratch == nullptr) { be->arena.free(d_pos, 2 * sizeof(int)); be->set_error("attention: out of device memory"); return SPYB_FAIL; }
    }
    cudaError_t err = cudaMemcpyAsync(d_pos, host_pos, sizeof(host_pos), cudaMemcpyHostToDevice, be->stream);
    if (err == cudaSuccess) { err = launch_attention(a, be->launch_cfg(false)); }
    if (err == cudaSuccess) { err = cudaStreamSynchronize(be->stream); }
    be->arena.free(d_pos, 2 * sizeof(int));
    if (a.scratch != nullptr) { be->arena.free(a.scratch, scratch_bytes); }
    if (err != cudaSuccess) { be->set_error("attention failed: %s", cudaGetErrorString(err)); return SPYB_FAIL; }
    return SPYB_SUCCESS;
}

// ------------------------------------------------------------------------------------------ MatMul without allocation
// Scratch for the re-tiled weights of spyb_matmul_noalloc: part of the library image, one per device and process.
static __device__ __align__(256) uint8_t g_noalloc_scratch[SPYB_NOALLOC_SCRATCH_BYTES];

spyb_status spyb_matmul_noalloc(spyb_backend *be, int32_t weight_type, const void *w_rows_dev, int64_t n_rows, int64_t k,
                                const float *x_dev, int64_t n_cols, float *out_dev) {
    if (be == nullptr) { return SPYB_FAIL; }
    if (weight_type != SPYB_Q4_0 && weight_type != SPYB_Q8_0) { be->set_error("matmul_noalloc: weight type %d", weight_type); return SPYB_UNSUPPORTED; }
    if (w_rows_dev == nullptr || x_dev == nullptr || out_dev == nullptr || n_rows < 4 || (n_rows & 3) || k < QK || k % QK != 0 || n_cols < 1) {
        be->set_error("matmul_noalloc: needs n_rows a multiple of 4, k a multiple of 32, at least one column"); return SPYB_UNSUPPORTED;
    }
    // the kernels read the activations with 128-bit loads and the raw blocks with 16-bit ones: a misaligned pointer would
    // raise a device fault (and lose the context), so it is refused here
    if ((reinterpret_cast<uintptr_t>(x_dev) & 15) || (reinterpret_cast<uintptr_t>(out_dev) & 3) || (reinterpret_cast<uintptr_t>(w_rows_dev) & 1)) {
        be->set_error("matmul_noalloc: x must be 16-byte aligned, out 4-byte aligned, the weight blocks 2-byte aligned"); return SPYB_UNSUPPORTED;
    }
    const int nb = (int)(k / QK);
    if (matrix_bytes(weight_type, n_rows, nb) > SPYB_NOALLOC_SCRATCH_BYTES) {
        be->set_error("matmul_noalloc: the re-tiled matrix (%llu bytes) exceeds the %u-byte scratch array", (unsigned long long)matrix_bytes(weight_type, n_rows, nb),
                      (unsigned)SPYB_NOALLOC_SCRATCH_BYTES);
        return SPYB_UNSUPPORTED;
    }
    cudaSetDevice(be->config.device_id);
    if (be->noalloc_scratch == nullptr) {   // once per device: address of the image's scratch array
        void *ptr = nullptr;
        SPYB_CUDA(be, cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
        if (ptr == nullptr) { be->set_error("matmul_noalloc: no address for the scratch array"); return SPYB_FAIL; }
        be->noalloc_scratch = static_cast<uint8_t *>(ptr);
    }
    DevMatrix m;
    m.type = weight_type; m.n_rows = n_rows; m.nb = nb; m.nbp = padded_blocks(nb); m.k = k; m.tile_rows = 4; m.w = be->noalloc_scratch;
    const int64_t bb = weight_type == SPYB_Q4_0 ? 18 : 34;
    SPYB_CUDA(be, launch_retile(weight_type, static_cast<const uint8_t *>(w_rows_dev), nb * bb, n_rows, nb, be->noalloc_scratch, 4, false, 0, 0, 0, 0, be->stream));
    const int64_t tmax = matvec_max_columns(nb);
    for (int64_t t0 = 0; t0 < n_cols; t0 += tmax) {
        MatvecParams p;
        p.A = m; p.T = (int)std::min<int64_t>(tmax, n_cols - t0);
        p.pro = PRO_QUANT; p.x = x_dev + t0 * k; p.x_stride = k;
        p.epi = EPI_STORE; p.out = out_dev + t0 * n_rows; p.out_stride = n_rows;
        SPYB_CUDA(be, launch_matvec(p, be->launch_cfg(false)));
    }
    return SPYB_SUCCESS;
}

// ------------------------------------------------------------------------------------------ MatMul of a prompt on the tensor cores
// OperatorMatMul (backend/host/operator/mat.cpp:95-128) for n_cols activation columns through the tcgen05 prompt kernel:
// host pointers in and out, everything staged inside the call. The entry point the parity tests drive; the model path
// uses the same kernels on resident buffers.
spyb_status spyb_prefill_matmul(spyb_backend *be, int32_t weight_type, const void *w_rows_host, int64_t n_rows, int64_t k, const float *x_host,
                                int64_t n_cols, const float *norm_w_host, float eps, float *out_host) {
    if (be == nullptr) { return SPYB_FAIL; }
    const bool kq = weight_type == SPYB_Q4_K || weight_type == SPYB_Q6_K;
    if (weight_type != SPYB_Q4_0 && weight_type != SPYB_Q8_0 && !kq) { be->set_error("prefill_matmul: weight type %d", weight_type); return SPYB_UNSUPPORTED; }
    if (kq && k % 256 != 0) { be->set_error("prefill_matmul: K-quant rows need k a multiple of 256"); return SPYB_UNSUPPORTED; }
    if (w_rows_host == nullptr || x_host == nullptr || out_host == nullptr || n_rows < 1 || k < QK || k % QK != 0 || k > PF_MAX_K ||
        n_cols < 1 || n_cols > 4096) {
        be->set_error("prefill_matmul: needs k a multiple of 32 up to %d, 1..4096 columns", PF_MAX_K); return SPYB_UNSUPPORTED;
    }
    cudaSetDevice(be->config.device_id);
    const int nb = (int)(k / QK), T = (int)n_cols;
    const int64_t rb = kq ? (k / 256) * (weight_type == SPYB_Q4_K ? 144 : 210) : (int64_t)nb * (weight_type == SPYB_Q4_0 ? 18 : 34);
    const size_t wbytes = prefill_weight_bytes(weight_type, n_rows, nb), ybytes = prefill_act_bytes(T, nb);
    uint8_t *raw = nullptr, *w = nullptr, *yq = nullptr; float *x = nullptr, *nw = nullptr, *out = nullptr;
    auto release = [&]() { cudaFree(raw); cudaFree(w); cudaFree(yq); cudaFree(x); cudaFree(nw); cudaFree(out); };
    cudaError_t err = cudaMalloc(&raw, (size_t)n_rows * rb + 64);
    if (err == cudaSuccess) { err = cudaMalloc(&w, wbytes); }
    if (err == cudaSuccess) { err = cudaMemsetAsync(w, 0, wbytes, be->stream); }   // (rows that pad the last tile stay zero)
    if (err == cudaSuccess) { err = cudaMalloc(&yq, ybytes); }
    if (err == cudaSuccess) { err = cudaMalloc(&x, (size_t)T * k * 4); }
    if (err == cudaSuccess) { err = cudaMalloc(&out, (size_t)T * n_rows * 4); }
    if (err == cudaSuccess && norm_w_host != nullptr) { err = cudaMalloc(&nw, (size_t)k * 4); }
    if (err == cudaSuccess) { err = cudaMemsetAsync(yq, 0, ybytes, be->stream); }
    if (err == cudaSuccess) { err = cudaMemcpyAsync(raw, w_rows_host, (size_t)n_rows * rb, cudaMemcpyHostToDevice, be->stream); }
    if (err == cudaSuccess) { err = cudaMemcpyAsync(x, x_host, (size_t)T * k * 4, cudaMemcpyHostToDevice, be->stream); }
    if (err == cudaSuccess && nw != nullptr) { err = cudaMemcpyAsync(nw, norm_w_host, (size_t)k * 4, cudaMemcpyHostToDevice, be->stream); }
    if (err == cudaSuccess) { err = launch_prefill_retile(weight_type, raw, rb, n_rows, nb, w, 0, be->stream); }
    if (err == cudaSuccess) { err = launch_prefill_quant(x, k, T, (int)k, nw, eps, yq, be->stream, weight_type); }
    if (err == cudaSuccess) {
        PrefillGemm g;
        g.w = w; g.type = weight_type; g.n_rows = n_rows; g.nb = nb; g.yq = yq; g.T = T; g.out = out; g.out_stride = n_rows;
        g.error_flag = be->d_error_flag; g.wait_limit_ns = be->wait_limit_ns;
        // profiling aid (SPYB_PF_STAMPS=<file>): clock stamps of the roles of one CTA of a second, warm launch
        long long *stamps = nullptr;
        const char *dump = std::getenv("SPYB_PF_STAMPS");
        const size_t stamp_bytes = 8 * 512 * 4 * sizeof(long long);
        err = launch_prefill_gemm(g, be->stream);
        if (err == cudaSuccess && dump != nullptr && cudaMalloc(&stamps, stamp_bytes) == cudaSuccess) {
            cudaMemsetAsync(stamps, 0, stamp_bytes, be->stream);
            g.stamps = stamps;
            err = launch_prefill_gemm(g, be->stream);
            std::vector<long long> h(stamp_bytes / sizeof(long long));
            cudaStreamSynchronize(be->stream);
            cudaMemcpy(h.data(), stamps, stamp_bytes, cudaMemcpyDeviceToHost);
            if (FILE *f = std::fopen(dump, "wb")) { std::fwrite(h.data(), 8, h.size(), f); std::fclose(f); }
            cudaFree(stamps);
        }
    }
    if (err == cudaSuccess) { err = cudaMemcpyAsync(out_host, out, (size_t)T * n_rows * 4, cudaMemcpyDeviceToHost, be->stream); }
    if (err == cudaSuccess) { err = cudaStreamSynchronize(be->stream); }
    release();
    if (err != cudaSuccess) { be->set_error("prefill_matmul: %s", cudaGetErrorString(err)); return SPYB_FAIL; }
    if (be->device_error()) { return SPYB_FAIL; }
    return SPYB_SUCCESS;
}

// Failure-path check of the prompt GEMM that faults nothing: one small launch whose copy thread leaves the second batch of
// blocks out, with `limit_ns` as the bound of every wait. The roles that wait for that batch give up one after the other,
// the kernel frees its tensor memory and returns, and the error word holds a code of the prompt kernel (4, 5 or 6).
spyb_status spyb_prefill_selftest_wait_timeout(spyb_backend *be, uint64_t limit_ns, int32_t *error_code_out) {
    if (be == nullptr || limit_ns == 0) { return SPYB_FAIL; }
    cudaSetDevice(be->config.device_id);
    SPYB_CUDA(be, cudaStreamSynchronize(be->stream));
    if (be->device_error()) { return SPYB_FAIL; }
    const int nb = 12, T = PF_TOK;
    const size_t wbytes = prefill_weight_bytes(SPYB_Q8_0, PF_ROWS, nb), ybytes = prefill_act_bytes(T, nb);
    uint8_t *w = nullptr, *yq = nullptr; float *out = nullptr;
    auto release = [&]() { cudaFree(w); cudaFree(yq); cudaFree(out); };
    cudaError_t err = cudaMalloc(&w, wbytes);
    if (err == cudaSuccess) { err = cudaMalloc(&yq, ybytes); }
    if (err == cudaSuccess) { err = cudaMalloc(&out, (size_t)T * PF_ROWS * 4); }
    if (err == cudaSuccess) { err = cudaMemsetAsync(w, 0, wbytes, be->stream); }
    if (err == cudaSuccess) { err = cudaMemsetAsync(yq, 0, ybytes, be->stream); }
    if (err == cudaSuccess) {
        PrefillGemm g;
        g.w = w; g.type = SPYB_Q8_0; g.n_rows = PF_ROWS; g.nb = nb; g.yq = yq; g.T = T; g.out = out; g.out_stride = PF_ROWS;
        g.error_flag = be->d_error_flag; g.wait_limit_ns = limit_ns; g.selftest_skip_batch = 1;
        err = launch_prefill_gemm(g, be->stream);
    }
    if (err == cudaSuccess) { err = cudaStreamSynchronize(be->stream); }   // returns: the kernel ended by itself
    release();
    if (err != cudaSuccess) { be->set_error("prefill selftest: %s", cudaGetErrorString(err)); return SPYB_FAIL; }
    const int code = *reinterpret_cast<volatile int *>(be->h_error_flag);
    if (error_code_out != nullptr) { *error_code_out = code; }
    *reinterpret_cast<volatile int *>(be->h_error_flag) = 0;   // the check leaves the backend usable
    if (code < 4 || code > 6) { be->set_error("prefill selftest: expected a wait of the prompt kernel to give up (codes 4-6), got %d", code); return SPYB_FAIL; }
    return SPYB_SUCCESS;
}

// ------------------------------------------------------------------------------------------ submit
namespace {

struct Staged {   // a host (IO) tensor mirrored in device memory for the duration of one operator
    void   *dev = nullptr;
    size_t  bytes = 0;
    bool    temp = false;
};

spyb_status stage_in(spyb_backend *be, const spyb_tensor &t, Staged *s) {
    if (t.node_type != SPYB_NODE_IO) { s->dev = t.data; return SPYB_SUCCESS; }
    s->bytes = (size_t)tensor_total_size(t);
    s->dev = be->arena.alloc(s->bytes);
    s->temp = true;
    if (s->dev == nullptr) { be->set_error("out of device memory staging an IO tensor"); return SPYB_FAIL; }
    SPYB_CUDA(be, cudaMemcpyAsync(s->dev, t.data, s->bytes, cudaMemcpyHostToDevice, be->stream));
    return SPYB_SUCCESS;
}

spyb_status stage_out_begin(spyb_backend *be, const spyb_tensor &t, Staged *s) {
    if (t.node_type != SPYB_NODE_IO) { s->dev = t.data; return SPYB_SUCCESS; }
    s->bytes = (size_t)tensor_total_size(t);
    s->dev = be->arena.alloc(s->bytes);
    s->temp = true;
    if (s->dev == nullptr) { be->set_error("out of device memory staging an IO tensor"); return SPYB_FAIL; }
    return SPYB_SUCCESS;
}

void stage_release(spyb_backend *be, Staged *s) {
    if (s->temp && s->dev) { be->arena.free(s->dev, s->bytes); }
    s->dev = nullptr; s->temp = false;
}

// MatMul of 16 and more activation columns against an uploaded constant: the tcgen05 GEMM of the prompt path (same bits as
// the mat-vec kernels). The matrix gets a second copy in that kernel's tile layout at first use, kept with the constant.
// Returns SPYB_UNSUPPORTED without an error text when the operands do not qualify (the caller then takes the mat-vec route).
spyb_status run_matmul_gemm(spyb_backend *be, const spyb_tensor &w, const spyb_tensor &x, void *out_dev) {
    const int type = w.number_type;
    const bool kq = type == SPYB_Q4_K || type == SPYB_Q6_K;
    if (type != SPYB_Q4_0 && type != SPYB_Q8_0 && !kq) { return SPYB_UNSUPPORTED; }
    const int64_t k = w.elements[0], n_rows = w.elements[1], T = x.elements[1] * x.elements[2] * x.elements[3];
    if (T < SPYB_PREFILL_MIN_TOKENS || w.node_type != SPYB_NODE_CONSTANT || k != x.elements[0] || k < QK || k % QK != 0 || k > PF_MAX_K || (kq && k % 256 != 0) ||
        n_rows < 1 || w.elements[2] != 1 || w.elements[3] != 1 || !tensor_contiguous(w) || !tensor_contiguous(x) ||
        (reinterpret_cast<uintptr_t>(x.data) & 15) || (reinterpret_cast<uintptr_t>(out_dev) & 3)) {
        return SPYB_UNSUPPORTED;
    }
    // Q4_0 / Q8_0: a GEMM CTA walks all of K for 128 rows x 16 columns, so few tiles leave most SMs idle and passes of four
    // columns through the mat-vec kernel are faster (measured: 4096 rows x 16 columns slower, 11008 x 16 faster)
    if (!kq && ((n_rows + PF_ROWS - 1) / PF_ROWS) * ((T + PF_TOK - 1) / PF_TOK) < 74) { return SPYB_UNSUPPORTED; }
    static const bool off = [] { const char *e = std::getenv("SPYB_PREFILL"); return e != nullptr && e[0] == '0'; }();
    if (off) { return SPYB_UNSUPPORTED; }
    const int nb = (int)(k / QK);
    uint8_t *tiles = nullptr;
    {
        std::lock_guard<std::mutex> g(be->const_mutex);
        auto ct = be->const_types.find(w.data);
        if (ct == be->const_types.end() || ct->second != type) { return SPYB_UNSUPPORTED; }   // not (or no longer) the constant that was uploaded
        auto it = be->pf_tiles.find(w.data);
        if (it != be->pf_tiles.end()) { tiles = it->second; }
        else {
            const int64_t rb = kq ? (k / 256) * (type == SPYB_Q4_K ? 144 : 210) : (int64_t)nb * (type == SPYB_Q4_0 ? 18 : 34);
            const size_t wbytes = prefill_weight_bytes(type, n_rows, nb);
            void *raw = nullptr;
            SPYB_CUDA(be, cudaMalloc(&raw, wbytes));
            be->owned.push_back(raw);
            tiles = static_cast<uint8_t *>(raw);
            SPYB_CUDA(be, cudaMemsetAsync(tiles, 0, wbytes, be->stream));   // (rows that pad the last tile stay zero)
            SPYB_CUDA(be, launch_prefill_retile(type, static_cast<const uint8_t *>(w.data), rb, n_rows, nb, tiles, 0, be->stream));
            be->pf_tiles[w.data] = tiles;
        }
    }
    const int64_t chunk = 1024;
    const size_t ybytes = prefill_act_bytes((int)std::min(chunk, T), nb);
    void *yq = be->arena.alloc(ybytes);
    if (yq == nullptr) { be->set_error("MatMul: out of device memory for the quantized activations"); return SPYB_FAIL; }
    struct Release { spyb_backend *be; void *a; size_t n; ~Release() { be->arena.free(a, n); } } release{be, yq, ybytes};   // (stream-ordered reuse)
    for (int64_t t0 = 0; t0 < T; t0 += chunk) {
        const int Tc = (int)std::min(chunk, T - t0);
        SPYB_CUDA(be, cudaMemsetAsync(yq, 0, prefill_act_bytes(Tc, nb), be->stream));
        SPYB_CUDA(be, launch_prefill_quant(static_cast<const float *>(x.data) + t0 * k, k, Tc, (int)k, nullptr, 0.f, static_cast<uint8_t *>(yq), be->stream, type));
        PrefillGemm g;
        g.w = tiles; g.type = type; g.n_rows = n_rows; g.nb = nb; g.yq = static_cast<uint8_t *>(yq); g.T = Tc;
        g.out = static_cast<float *>(out_dev) + t0 * n_rows; g.out_stride = n_rows;
        g.error_flag = be->d_error_flag; g.wait_limit_ns = be->wait_limit_ns;
        SPYB_CUDA(be, launch_prefill_gemm(g, be->stream));
    }
    return SPYB_SUCCESS;
}

// MatMul of fewer than 16 columns against an uploaded Q4_K / Q6_K constant: the model path's K-quant mat-vec kernel, up to four
// columns per launch (activations quantized to Q8_0 first, the arithmetic of the restatement; the tensor-core route above gives the
// same bits for 16 columns and more). Q6_K rows get a copy in that kernel's layout at first use.
spyb_status run_matmul_kq_constant(spyb_backend *be, const spyb_tensor &w, const spyb_tensor &x, void *out_dev) {
    const int type = w.number_type;
    const int64_t k = w.elements[0], n_rows = w.elements[1], T = x.elements[1] * x.elements[2] * x.elements[3];
    if (w.node_type != SPYB_NODE_CONSTANT || k != x.elements[0] || k % 256 != 0 || k > 256 * 32 * 4 || n_rows < 2 || (n_rows & 1) || w.elements[2] != 1 || w.elements[3] != 1 ||
        !tensor_contiguous(w) || !tensor_contiguous(x) || (reinterpret_cast<uintptr_t>(x.data) & 15) || (reinterpret_cast<uintptr_t>(out_dev) & 3) ||
        (reinterpret_cast<uintptr_t>(w.data) & 15)) {
        return SPYB_UNSUPPORTED;
    }
    const uint8_t *rows = static_cast<const uint8_t *>(w.data);
    {
        std::lock_guard<std::mutex> g(be->const_mutex);
        auto ct = be->const_types.find(w.data);
        if (ct == be->const_types.end() || ct->second != type) { return SPYB_UNSUPPORTED; }
        if (type == SPYB_Q6_K) {
            auto it = be->kq_relaid.find(w.data);
            if (it != be->kq_relaid.end()) { rows = it->second; }
            else {
                void *raw = nullptr;
                SPYB_CUDA(be, cudaMalloc(&raw, (size_t)n_rows * kq_row_bytes(type, k) + 64));
                be->owned.push_back(raw);
                SPYB_CUDA(be, launch_kq_relayout_q6k(static_cast<const uint8_t *>(w.data), n_rows, k, static_cast<uint8_t *>(raw), be->stream));
                be->kq_relaid[w.data] = static_cast<uint8_t *>(raw);
                rows = static_cast<const uint8_t *>(raw);
            }
        }
    }
    for (int64_t t = 0; t < T; t += KQ_MAX_COLUMNS) {
        MatvecParams p;
        p.A.type = SPYB_Q4_K; p.A.k = k; p.A.nb = (int)(k / QK); p.A.nbp = p.A.nb; p.A.n_rows = n_rows;   // (only the shape is used)
        p.kq[0].w = rows; p.kq[0].type = type; p.kq[0].n_rows = n_rows; p.kq[0].row_bytes = kq_row_bytes(type, k); p.kq_n = 1;
        p.T = (int)std::min<int64_t>(KQ_MAX_COLUMNS, T - t); p.pro = PRO_QUANT; p.x = static_cast<const float *>(x.data) + t * k; p.x_stride = k;
        p.epi = EPI_STORE; p.out = static_cast<float *>(out_dev) + t * n_rows; p.out_stride = n_rows;
        SPYB_CUDA(be, launch_matvec_kq(p, be->launch_cfg(false)));
    }
    return SPYB_SUCCESS;
}

spyb_status run_matmul(spyb_backend *be, spyb_op_desc *d, void *out_dev) {
    const spyb_tensor &w = d->input[0], &x = d->input[1];
    if (x.number_type != SPYB_FP32) { be->set_error("MatMul: activations of type %d", x.number_type); return SPYB_UNSUPPORTED; }
    {
        const spyb_status st = run_matmul_gemm(be, w, x, out_dev);
        if (st != SPYB_UNSUPPORTED) { return st; }
    }
    if (w.number_type == SPYB_FP16) {
        SPYB_CUDA(be, launch_matmul_f16(to_strided(w, w.data), to_strided(x, x.data), to_strided(d->output, out_dev), be->stream));
        return SPYB_SUCCESS;
    }
    if (w.number_type == SPYB_Q4_K || w.number_type == SPYB_Q6_K) {
        {
            const spyb_status st = run_matmul_kq_constant(be, w, x, out_dev);
            if (st != SPYB_UNSUPPORTED) { return st; }
        }
        // operands that are not uploaded constants: decoded weights times f32 activations (tolerance-level parity)
        if (!tensor_contiguous(w) || !tensor_contiguous(x) || w.elements[2] != 1 || w.elements[3] != 1 || w.elements[0] % 256 != 0 || w.elements[0] != x.elements[0]) {
            be->set_error("MatMul: K-quant weights need contiguous 2-D operands with K a multiple of 256");
            return SPYB_UNSUPPORTED;
        }
        SPYB_CUDA(be, launch_matmul_kquant(w.number_type, static_cast<const uint8_t *>(w.data), w.elements[1], w.elements[0], static_cast<const float *>(x.data),
                                           x.elements[1] * x.elements[2] * x.elements[3], static_cast<float *>(out_dev), be->stream));
        return SPYB_SUCCESS;
    }
    if (w.number_type != SPYB_Q4_0 && w.number_type != SPYB_Q8_0) {
        be->set_error("MatMul: weight type %d is not implemented", w.number_type);
        return SPYB_UNSUPPORTED;
    }
    if ((reinterpret_cast<uintptr_t>(x.data) & 15) || (reinterpret_cast<uintptr_t>(out_dev) & 3) || (reinterpret_cast<uintptr_t>(w.data) & 1)) {
        be->set_error("MatMul: activations must be 16-byte aligned, the output 4-byte aligned, quantized blocks 2-byte aligned");
        return SPYB_UNSUPPORTED;   // (the kernels use 128-bit loads: a misaligned view would fault on the device)
    }
    if (!tensor_contiguous(w) || !tensor_contiguous(x) || w.elements[2] != 1 || w.elements[3] != 1) {
        be->set_error("MatMul: quantized weights need contiguous 2-D operands");
        return SPYB_UNSUPPORTED;
    }
    DevMatrix m;
    bool found = false;
    void *tmp_w = nullptr;
    const int    nb_w = (int)(w.elements[0] / QK);
    if (w.elements[1] & 3) { be->set_error("MatMul: %lld output rows (quantized weights need a multiple of 4)", (long long)w.elements[1]); return SPYB_UNSUPPORTED; }
    const size_t w_bytes = matrix_bytes(w.number_type, w.elements[1], nb_w) + 16;
    {
        std::lock_guard<std::mutex> g(be->const_mutex);
        auto it = be->retiled.find(w.data);
        if (it != be->retiled.end() && w.node_type == SPYB_NODE_CONSTANT) { m = it->second; found = true; }
    }
    if (!found) {
        // a quantized operand that did not come through spyb_upload_constant (its address may be reused for other
        // data later, so nothing is cached): re-tile into a buffer that lives for this operator only
        const int64_t bb = w.number_type == SPYB_Q4_0 ? 18 : 34;
        m.type = w.number_type; m.n_rows = w.elements[1]; m.nb = nb_w; m.nbp = padded_blocks(nb_w); m.k = w.elements[0];
        tmp_w = be->arena.alloc(w_bytes);
        if (!tmp_w) { be->set_error("MatMul: out of device memory for re-tiled weights"); return SPYB_FAIL; }
        m.w = static_cast<const uint8_t *>(tmp_w);
        cudaError_t err = launch_retile(w.number_type, static_cast<const uint8_t *>(w.data), w.elements[0] / QK * bb, w.elements[1], m.nb,
                                        static_cast<uint8_t *>(tmp_w), 4, false, 0, 0, 0, 0, be->stream);
        if (err != cudaSuccess) { be->set_error("MatMul: re-tiling failed: %s", cudaGetErrorString(err)); return SPYB_FAIL; }
    }
    struct TmpRelease {   // stream-ordered reuse: safe to hand back as soon as the kernels are enqueued
        spyb_backend *be; void *a; size_t na;
        ~TmpRelease() { if (a) { be->arena.free(a, na); } }
    } release{be, tmp_w, w_bytes};
    if (m.k != x.elements[0]) { be->set_error("MatMul: inner dimensions differ"); return SPYB_FAIL; }
    if (m.n_rows & 3) { be->set_error("MatMul: %lld output rows (quantized weights need a multiple of 4)", (long long)m.n_rows); return SPYB_UNSUPPORTED; }
    const int64_t T = x.elements[1] * x.elements[2] * x.elements[3];
    const int64_t tmax = matvec_max_columns(m.nb);
    for (int64_t t0 = 0; t0 < T; t0 += tmax) {
        MatvecParams p;
        p.A = m; p.T = (int)std::min<int64_t>(tmax, T - t0);
        p.pro = PRO_QUANT; p.x = static_cast<const float *>(x.data) + t0 * m.k; p.x_stride = m.k;
        p.epi = EPI_STORE; p.out = static_cast<float *>(out_dev) + t0 * m.n_rows; p.out_stride = m.n_rows;
        SPYB_CUDA(be, launch_matvec(p, be->launch_cfg(false)));
    }
    return SPYB_SUCCESS;
}

}  // namespace

spyb_status spyb_submit(spyb_backend *be, spyb_op_desc *d, void (*callback)(void *), void *user) {
    if (be == nullptr || d == nullptr) { return SPYB_FAIL; }
    cudaSetDevice(be->config.device_id);
    spyb_status st = SPYB_SUCCESS;
    Staged in[3], out;
    bool   has_out_copy = false;

    switch (d->op_type) {
    // view-type operators alias their input (backend/host/operator/view.cpp:229-276)
    case SPYB_OP_INPUT: case SPYB_OP_NOP: break;
    case SPYB_OP_RESHAPE: case SPYB_OP_TRANSPOSE: case SPYB_OP_PERMUTE: d->output.data = d->input[0].data; break;
    case SPYB_OP_VIEW: d->output.data = static_cast<uint8_t *>(d->input[0].data) + d->view_offset; break;
    default: {
        for (int i = 0; i < d->num_input && i < 3 && st == SPYB_SUCCESS; ++i) { st = stage_in(be, d->input[i], &in[i]); }
        if (st == SPYB_SUCCESS && d->op_type != SPYB_OP_COPY) { st = stage_out_begin(be, d->output, &out); has_out_copy = out.temp; }
        if (st != SPYB_SUCCESS) { break; }
        spyb_op_desc local = *d;
        for (int i = 0; i < d->num_input && i < 3; ++i) { local.input[i].data = in[i].dev; }
        const spyb_tensor &a = local.input[0];
        cudaError_t err = cudaSuccess;
        switch (d->op_type) {
        case SPYB_OP_MATMUL: st = run_matmul(be, &local, out.dev); break;
        case SPYB_OP_ADD: case SPYB_OP_MUL: {
            const spyb_tensor &b = local.input[1];
            if (!tensor_contiguous(a) || !tensor_contiguous(b) || a.number_type != SPYB_FP32 || b.number_type != SPYB_FP32 || a.elements[0] != b.elements[0]) {
                be->set_error("Add/Mul: operands must be contiguous f32 rows of equal length"); st = SPYB_UNSUPPORTED; break;
            }
            const int64_t rows = tensor_elems(a) / a.elements[0], brows = tensor_elems(b) / b.elements[0];
            err = launch_binary_rows(d->op_type == SPYB_OP_ADD ? 0 : 1, static_cast<const float *>(a.data), static_cast<const float *>(b.data),
                                     static_cast<float *>(out.dev), a.elements[0], rows, brows, be->stream);
        } break;
        case SPYB_OP_NORM_RMS:
            if (!tensor_contiguous(a) || a.number_type != SPYB_FP32) { be->set_error("NormRMS: contiguous f32 expected"); st = SPYB_UNSUPPORTED; break; }
            err = launch_rmsnorm(static_cast<const float *>(a.data), static_cast<float *>(out.dev), a.elements[0], tensor_elems(a) / a.elements[0], d->norm_eps, be->stream);
            break;
        case SPYB_OP_SILU:
            if (!tensor_contiguous(a) || a.number_type != SPYB_FP32) { be->set_error("Silu: contiguous f32 expected"); st = SPYB_UNSUPPORTED; break; }
            err = launch_silu(static_cast<const float *>(a.data), static_cast<float *>(out.dev), tensor_elems(a), be->d_silu_table, be->stream);
            break;
        case SPYB_OP_SOFTMAX: {
            if (d->num_input != 2 || !tensor_contiguous(a)) { be->set_error("Softmax: contiguous scores and a mask expected"); st = SPYB_UNSUPPORTED; break; }
            const spyb_tensor &mk = local.input[1];
            err = launch_softmax_masked(static_cast<const float *>(a.data), static_cast<const float *>(mk.data), static_cast<float *>(out.dev),
                                        a.elements[0], a.elements[1], a.elements[2] * a.elements[3], mk.bytes[1] / 4, d->softmax_scale, be->d_exp_table, be->stream);
        } break;
        case SPYB_OP_ROPE:
            if (d->rope.mode != 0 || d->rope.extend_factor != 0.f || d->rope.freq_scale != 1.f || d->rope.attention_factor != 1.f) {
                be->set_error("Rope: only mode Norm with default scaling is implemented"); st = SPYB_UNSUPPORTED; break;
            }
            {
                // (cos, sin) per (token, pair) with the host libm and the CPU operator's repeated f32 multiplication of theta
                // (backend/host/operator/non-linear.cpp:282, 300-309), so the rotation is bit-identical to the CPU's
                const int64_t n_tok = a.elements[2], npair = a.elements[0] / 2;
                std::vector<int32_t> pos((size_t)n_tok);
                if (d->input[1].node_type == SPYB_NODE_IO) { std::memcpy(pos.data(), d->input[1].data, (size_t)n_tok * 4); }
                else if (cudaMemcpyAsync(pos.data(), d->input[1].data, (size_t)n_tok * 4, cudaMemcpyDeviceToHost, be->stream) != cudaSuccess ||
                         cudaStreamSynchronize(be->stream) != cudaSuccess) { be->set_error("Rope: reading positions failed"); st = SPYB_FAIL; break; }
                std::vector<float2> tab((size_t)(n_tok * npair));
                const float theta_scale = std::pow(d->rope.freq_base, -2.0f / (float)d->rope.num_dim);
                for (int64_t i = 0; i < n_tok; ++i) {
                    float theta = (float)pos[(size_t)i];
                    for (int64_t k = 0; k < npair; ++k) { tab[(size_t)(i * npair + k)] = make_float2(std::cos(theta) * 1.0f, std::sin(theta) * 1.0f); theta *= theta_scale; }
                }
                void *dtab = be->arena.alloc(tab.size() * sizeof(float2));
                if (dtab == nullptr) { be->set_error("Rope: out of device memory"); st = SPYB_FAIL; break; }
                err = cudaMemcpyAsync(dtab, tab.data(), tab.size() * sizeof(float2), cudaMemcpyHostToDevice, be->stream);
                if (err == cudaSuccess) { err = launch_rope(to_strided(a, a.data), static_cast<const float2 *>(dtab), to_strided(local.output, out.dev), be->stream); }
                be->arena.free(dtab, tab.size() * sizeof(float2));
            }
            break;
        case SPYB_OP_COPY: {   // destination = input[1]; the output aliases it (view.cpp:216-227)
            const spyb_tensor &dst = local.input[1];
            err = launch_copy_strided(to_strided(a, a.data), a.number_type, to_strided(dst, dst.data), dst.number_type, be->stream);
            d->output.data = d->input[1].data;
        } break;
        case SPYB_OP_DUP: case SPYB_OP_CONTIGUOUS:
            err = launch_copy_strided(to_strided(a, a.data), a.number_type, to_strided(local.output, out.dev), local.output.number_type, be->stream);
            break;
        case SPYB_OP_GETROW: {
            const spyb_tensor &ids = local.input[1];
            const int64_t rb = a.bytes[1];
            err = launch_getrow(static_cast<const uint8_t *>(a.data), a.number_type, rb, a.elements[0], static_cast<const int32_t *>(ids.data),
                                tensor_elems(ids), static_cast<float *>(out.dev), be->stream);
            if (err == cudaErrorNotSupported) { be->set_error("GetRow: table type %d", a.number_type); st = SPYB_UNSUPPORTED; err = cudaSuccess; }
        } break;
        default:
            be->set_error("operator type %d is not implemented on this backend", d->op_type);
            st = SPYB_UNSUPPORTED;
        }
        if (st == SPYB_SUCCESS && err != cudaSuccess) { be->set_error("operator %d launch failed: %s", d->op_type, cudaGetErrorString(err)); st = SPYB_FAIL; }
        if (st == SPYB_SUCCESS && has_out_copy) {
            cudaError_t e2 = cudaMemcpyAsync(d->output.data, out.dev, out.bytes, cudaMemcpyDeviceToHost, be->stream);
            if (e2 != cudaSuccess) { be->set_error("copy of an IO result failed: %s", cudaGetErrorString(e2)); st = SPYB_FAIL; }
        }
    } break;
    }
    for (auto &s : in) { stage_release(be, &s); }
    stage_release(be, &out);
    if (st != SPYB_SUCCESS) { return st; }

    if (callback != nullptr) {
        PendingCallback cb; cb.fn = callback; cb.user = user;
        SPYB_CUDA(be, cudaEventCreateWithFlags(&cb.event, cudaEventDisableTiming));
        SPYB_CUDA(be, cudaEventRecord(cb.event, be->stream));
        { std::lock_guard<std::mutex> g(be->cb_mutex); be->cb_queue.push_back(cb); }
        be->cb_cv.notify_one();
    }
    return SPYB_SUCCESS;
}

#ifndef SPYB_NO_MEASUREMENT_AIDS
spyb_status spyb_submit_timed(spyb_backend *be, spyb_op_desc *descs, int32_t n_descs, int32_t repeats, float *ms_out) {
    if (be == nullptr || descs == nullptr || n_descs < 1 || repeats < 1 || ms_out == nullptr) { return SPYB_FAIL; }
    cudaSetDevice(be->config.device_id);
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    SPYB_CUDA(be, cudaEventCreate(&e0));
    SPYB_CUDA(be, cudaEventCreate(&e1));
    spyb_status st = SPYB_SUCCESS;
    cudaError_t err = cudaEventRecord(e0, be->stream);
    for (int r = 0; r < repeats && st == SPYB_SUCCESS && err == cudaSuccess; ++r) { st = spyb_submit(be, &descs[r % n_descs], nullptr, nullptr); }
    if (err == cudaSuccess) { err = cudaEventRecord(e1, be->stream); }
    if (err == cudaSuccess) { err = cudaStreamSynchronize(be->stream); }
    if (err == cudaSuccess && st == SPYB_SUCCESS) { err = cudaEventElapsedTime(ms_out, e0, e1); }
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    if (st != SPYB_SUCCESS) { return st; }
    if (err != cudaSuccess) { be->set_error("submit_timed: %s", cudaGetErrorString(err)); return SPYB_FAIL; }
    if (be->device_error()) { return SPYB_FAIL; }
    return SPYB_SUCCESS;
}
#endif

}  // extern "C"
