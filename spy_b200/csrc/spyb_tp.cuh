// Device side of the tensor-parallel exchange shared by the mat-vec kernels and the attention kernel.
#pragma once

#include "spyb_common.cuh"
#include "spyb_kernels.h"

namespace spyb {

// ---------------------------------------------------------------------------------------------
// Tensor parallelism, fused into the kernels as an ALL-GATHER over peer memory (no sums cross ranks, so every f32
// chain stays whole on one GPU and the results are the single-GPU bits):
//   producer (attention, FFN up|gate): writes its share of the gathered vector into its own copy; the CTA that finishes
//   last copies that share into every other rank's copy with wide peer stores, issues one system-scope fence and
//   publishes the step's epoch in every rank's flag word of the site;
//   consumer (Wo, FFN down, both replicated): waits - bounded - until all ranks' flags of the site show the epoch, then
//   reads the complete vector from its own memory.
__device__ __forceinline__ void tp_wait(const TpLink &tp, int *error_flag) {
    if (tp.flag_in == nullptr) { return; }
    if ((int)threadIdx.x < tp.n) {
        const unsigned want = (unsigned)*tp.epoch;
        const uint64_t t0 = global_timer_ns();
        while (ld_acquire_sys(tp.flag_in + threadIdx.x) != want) {
            if (global_timer_ns() - t0 > WAIT_LIMIT_NS) { if (error_flag != nullptr) { atomicExch(error_flag, 2); } break; }
        }
    }
    __syncthreads();
}
// called by every thread of every CTA at the end of a producing kernel; T columns
__device__ __forceinline__ void tp_publish(const TpLink &tp, int T) {
    if (tp.counter == nullptr) { return; }
    __shared__ int tp_last;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned n_ctas = gridDim.x * gridDim.y * gridDim.z;
        tp_last = (atomicAdd(tp.counter, 1u) == n_ctas - 1) ? 1 : 0;
        if (tp_last) { *tp.counter = 0; __threadfence(); }
    }
    __syncthreads();
    if (!tp_last) { return; }
    const int n4 = (int)(tp.len >> 2);
    for (int t = 0; t < T; ++t) {
        const float4 *src = reinterpret_cast<const float4 *>(tp.gather[tp.rank] + (int64_t)t * tp.stride + tp.off);
        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
            const float4 v = __ldcg(src + i);
            for (int rk = 0; rk < tp.n; ++rk) {
                if (rk != tp.rank) { reinterpret_cast<float4 *>(tp.gather[rk] + (int64_t)t * tp.stride + tp.off)[i] = v; }
            }
        }
    }
    __syncthreads();   // the CTA's peer stores happen-before thread 0's system-scope fence (cumulativity)
    if (threadIdx.x == 0) {
        const unsigned epoch = (unsigned)*tp.epoch;
        __threadfence_system();
        for (int rk = 0; rk < tp.n; ++rk) { *reinterpret_cast<volatile unsigned *>(tp.flag_out[rk]) = epoch; }
    }
}

}  // namespace spyb
