// Internal state of the backend object behind the C ABI.
#pragma once

#include <condition_variable>
#include <cstdarg>
#include <cstdio>
#include <deque>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include <cuda_runtime.h>

#include "../../include/spyb.h"
#include "spyb_kernels.h"

namespace spyb {

// First-fit device arena behind spyb_alloc / spyb_free. The reference's scheduler allocates every
// operator output and frees dead tensors from two threads
// (backend/distributor/include/scheduler/default_scheduler.h:167-228), so both calls are O(log n)
// host work under one mutex and never touch the CUDA allocator on the hot path.
class Arena {
public:
    bool     init(size_t bytes);
    void     destroy();
    void    *alloc(size_t bytes);
    void     free(void *ptr, size_t bytes);
    size_t   capacity() const { return capacity_; }
    size_t   available();
    bool     owns(const void *p) const { return p >= base_ && p < base_ + capacity_; }

private:
    static constexpr size_t ALIGN = 256;
    uint8_t                 *base_ = nullptr;
    size_t                   capacity_ = 0;
    std::map<size_t, size_t> free_;       // offset -> size
    std::unordered_map<void *, size_t> overflow_;   // allocations that did not fit the arena
    std::mutex               mutex_;
};

struct PendingCallback {
    cudaEvent_t event;
    void (*fn)(void *);
    void *user;
};

}  // namespace spyb

struct spyb_backend {
    spyb_config  config{};
    int          num_sms = 148;            // CTAs of a per-matrix mat-vec grid
    int          num_sms_total = 148;      // SMs of the device (grid of the persistent step kernel)
    size_t       smem_optin = 227 * 1024;  // largest dynamic shared memory a CTA may ask for
    unsigned long long wait_limit_ns = 1000000000ull;   // bound of the waits inside the step kernel
    int          mv_ctas_per_sm = 2;
    int          mv_ring_kb = 80;
    int          mv_force_s = 0, mv_force_wact = 0;
    cudaStream_t stream = nullptr;
    spyb::Arena  arena;
    int         *h_error_flag = nullptr;   // mapped pinned word the kernels set when a bounded wait runs out
    int         *d_error_flag = nullptr;   // its device address
    uint8_t     *noalloc_scratch = nullptr; // device address of the scratch array of spyb_matmul_noalloc (looked up once)
    float       *d_silu_table = nullptr;   // 65536 entries: xh / (1 + expf(-xh)) for the fp16 value xh
    float       *d_exp_table = nullptr;    // 65536 entries: expf(xh)

    std::mutex  err_mutex;
    std::string last_error;

    // constants uploaded through spyb_upload_constant: name -> raw device copy, and raw pointer -> re-tiled planes
    std::mutex                               const_mutex;
    std::unordered_map<std::string, void *>  constants;
    std::unordered_map<const void *, spyb::DevMatrix> retiled;
    std::unordered_map<const void *, int>             const_types;   // raw pointer -> number type of every uploaded constant
    std::unordered_map<const void *, uint8_t *>       kq_relaid;     // raw pointer of a Q6_K constant -> its rows in the K-quant mat-vec kernel's layout (made at first use)
    std::unordered_map<const void *, uint8_t *>       pf_tiles;      // raw pointer -> the same matrix in the prompt GEMM's tile layout (made at first use)
    std::vector<void *>                      owned;   // cudaMalloc'd blocks to release at destroy

    // completion callbacks
    std::thread                      cb_thread;
    std::mutex                       cb_mutex;
    std::condition_variable          cb_cv;
    std::deque<spyb::PendingCallback> cb_queue;
    bool                             cb_stop = false;

    void set_error(const char *fmt, ...) {
        char buf[512];
        va_list ap; va_start(ap, fmt); vsnprintf(buf, sizeof(buf), fmt, ap); va_end(ap);
        std::lock_guard<std::mutex> g(err_mutex);
        last_error = buf;
    }
    // after a stream synchronisation: did a kernel give up on a bounded wait?
    bool device_error() {
        if (h_error_flag != nullptr && *reinterpret_cast<volatile int *>(h_error_flag) != 0) {
            const int code = *reinterpret_cast<volatile int *>(h_error_flag);
            if (code == 1) { set_error("a kernel gave up waiting for a bulk copy into shared memory (device error flag 1); the backend must be re-created"); }
            else if (code >= 4 && code <= 6) { set_error("the prompt GEMM gave up waiting for %s (device error flag %d); the backend must be re-created", code == 4 ? "a shared-memory stage" : code == 5 ? "its operands or a free accumulator buffer" : "a tensor-core result", code); }
            else { set_error("a kernel gave up waiting at a barrier or for another rank's partial result (device error flag %d); the backend must be re-created", code); }
            return true;
        }
        return false;
    }
    spyb::LaunchCfg launch_cfg(bool pdl) const {
        spyb::LaunchCfg c; c.stream = stream; c.pdl = pdl; c.num_sms = num_sms; c.mv_ctas_per_sm = mv_ctas_per_sm;
        c.mv_ring_kb = mv_ring_kb; c.mv_force_s = mv_force_s; c.mv_force_wact = mv_force_wact; c.error_flag = d_error_flag; return c;
    }
};

namespace spyb {

#define SPYB_CUDA(backend, expr)                                                                     \
    do {                                                                                             \
        cudaError_t err__ = (expr);                                                                  \
        if (err__ != cudaSuccess) {                                                                  \
            (backend)->set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(err__), __FILE__, __LINE__); \
            return SPYB_FAIL;                                                                        \
        }                                                                                            \
    } while (0)

// upload raw reference-layout rows [n_rows][row_stride_bytes] (host) and re-tile the block range
// [blk0, blk0 + nb) of every row into freshly allocated planes; used for row shards (contiguous rows)
// and K shards (a block sub-range of each row) alike. With `into`, the rows land at row dst_row of an existing matrix,
// or (sub_rows > 0) interleaved tile by tile: source row i at dst_row + (i / sub_rows) * tile_rows + sub_off + i % sub_rows.
spyb_status upload_matrix(spyb_backend *be, int type, const uint8_t *host_rows, int64_t n_rows, int64_t row_stride_bytes,
                          int64_t blk0, int nb, DevMatrix *out, const DevMatrix *into = nullptr, int64_t dst_row = 0,
                          int sub_rows = 0, int sub_off = 0);
spyb_status alloc_matrix(spyb_backend *be, int type, int64_t n_rows, int nb, DevMatrix *out, int tile_rows = 4, int mma = 0);

}  // namespace spyb
