// Shared device/host helpers of the eptq_b200 kernels (sm_100a only).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/eptq_b200.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "eptq_b200 kernels are written for sm_100a"
#endif

namespace eptq {

constexpr unsigned kMarkerIndex = 65535u;   // codebook index that marks a critical block
constexpr int kMaxSplits = 16;              // column splits a GEMV may use (sizes the scratch)
constexpr int kRowsPerCta = 8;              // Q rows (groups of 8 outputs) per SIMT GEMV block

extern std::atomic<uint64_t> g_launches;    // kernels launched by this library
extern std::atomic<uint64_t> g_kernel_launches[EPTQ_KERNEL_COUNT];   // the same per kernel family (EPTQ_KERNEL_*)
inline void count_launch(int which) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    g_kernel_launches[which].fetch_add(1, std::memory_order_relaxed);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Scratch layout shared by every GEMV variant.  The regions that must stay zero between calls have a
// fixed position and size, so that the same scratch can serve layers of different shapes and every
// kernel variant: whoever writes there puts the zeros back before it ends.
//   [0, kCounterBytes)              unsigned arrival counters
//   [kCounterBytes, kPartialOffset) fp32 accumulators of the persistent group GEMV (atomic adds)
//   [kPartialOffset, ...)           float partial sums [split][batch][8*M], overwritten before read
constexpr size_t kCounterBytes = 4096;
constexpr size_t kPartialOffset = 1u << 20;
constexpr int kMaxCounters = static_cast<int>(kCounterBytes / sizeof(unsigned));
constexpr int kGemmMinBatch = 16;           // batches above this run on the tensor-core GEMM
constexpr int kDenseMinTokens = 1024;       // from here on the weight is reconstructed once into scratch and a dense GEMM follows
// The last counter word is the GEMM's status word (EPTQ_ERR_TIMEOUT if a bounded wait ran out), so
// GEMV plans may use at most kMaxCounters - 1 counters.

__device__ __forceinline__ uint4 ldg128(const void* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&out)[8]) {
    const __half2* h2 = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 f = __half22float2(h2[i]);
        out[2 * i] = f.x;
        out[2 * i + 1] = f.y;
    }
}

}  // namespace eptq
