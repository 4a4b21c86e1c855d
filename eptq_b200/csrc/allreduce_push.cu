// One-shot all-reduce of a small fp16 vector between the GPUs of one node, for the partial outputs of
// the row-parallel layers (o / down projections) of a tensor-parallel decode step.  The reference is
// single-GPU (kernels/patch.py:24-27); NCCL's all-reduce of 8 KB costs more than the GEMV it follows,
// so each rank instead stores its partial straight into a slot of every peer's buffer over NVLink
// (ordinary global stores through peer pointers), raises a flag, waits for the other ranks' flags and
// sums the slots locally.  No TMA, no multicast loads, no reads of remote memory: only stores go out.
//
// Buffers per rank (allocated and exchanged by the caller): data [2 parities][T sources][n_max] fp16 and
// flags [2][T][kArBlocks] u32.  Call k uses parity k & 1; a rank can enter call k+1 only after it saw
// every rank's flags of call k, i.e. after every rank has finished reading call k-1, so two parities
// suffice.  Every wait is bounded; on a timeout the kernel records EPTQ_ERR_TIMEOUT and returns.

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/eptq_b200.h"
#include "common.cuh"

namespace eptq {
namespace {

constexpr int kArBlocks = 8;
constexpr int kArThreads = 128;
constexpr int kArMaxRanks = 8;
constexpr unsigned kArSpinLimit = 400000;          // about a quarter of a second of polling

struct PushArgs {
    __half* data[kArMaxRanks];        // every rank's data buffer (this rank's own included)
    unsigned* flags[kArMaxRanks];     // every rank's flag buffer
    const __half* x;                  // this rank's partial, n elements
    __half* out;                      // the sum, n elements (may be x or residual)
    const __half* residual;           // optional: out = residual + sum (each rounded to fp16)
    unsigned* seq;                    // kArBlocks call counters of this rank
    int* status;                      // set to EPTQ_ERR_TIMEOUT if a wait ran out
    int rank, T, n, n_max;
};

__global__ void __launch_bounds__(kArThreads) allreduce_push_kernel(const PushArgs a) {
    __shared__ unsigned s_seq;
    __shared__ int s_ok;
    const int tid = threadIdx.x, b = blockIdx.x;
    // Programmatic dependent launch: the next kernel may begin its set-up while this one exchanges data;
    // this one waits for its producer before it reads x.
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tid == 0) { s_seq = a.seq[b] + 1u; s_ok = 1; }
    __syncthreads();
    const unsigned seq = s_seq;
    const unsigned parity = seq & 1u;
    const int per_block = ((a.n + kArBlocks * 8 - 1) / (kArBlocks * 8)) * 8;      // multiple of 8 elements
    const int lo = b * per_block;
    const int hi = min(a.n, lo + per_block);

    // push my chunk into my slot of every rank's buffer
    const size_t my_slot = (static_cast<size_t>(parity) * a.T + a.rank) * a.n_max;
    for (int i = lo + tid * 8; i < hi; i += kArThreads * 8) {
        const uint4 v = *reinterpret_cast<const uint4*>(a.x + i);
        for (int r = 0; r < a.T; ++r) *reinterpret_cast<uint4*>(a.data[r] + my_slot + i) = v;
    }
    __threadfence_system();
    __syncthreads();
    if (tid < a.T) {
        unsigned* f = a.flags[tid] + (parity * a.T + a.rank) * kArBlocks + b;
        asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(f), "r"(seq) : "memory");
        // wait for rank `tid`'s flag of this call in my own buffer
        const unsigned* w = a.flags[a.rank] + (parity * a.T + tid) * kArBlocks + b;
        unsigned got = 0, spins = 0;
        for (;;) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(got) : "l"(w) : "memory");
            if (got == seq) break;
            if (++spins > kArSpinLimit) { s_ok = 0; atomicExch(a.status, static_cast<int>(EPTQ_ERR_TIMEOUT)); break; }
        }
    }
    __syncthreads();
    if (s_ok) {
        const __half* mine = a.data[a.rank] + static_cast<size_t>(parity) * a.T * a.n_max;
        for (int i = lo + tid * 8; i < hi; i += kArThreads * 8) {
            float acc[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] = 0.f;
            for (int r = 0; r < a.T; ++r) {
                const uint4 v = __ldcg(reinterpret_cast<const uint4*>(mine + static_cast<size_t>(r) * a.n_max + i));
                float f[8];
                unpack8(v, f);
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[k] += f[k];
            }
            __half2 o[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) o[k] = __floats2half2_rn(acc[2 * k], acc[2 * k + 1]);
            if (a.residual != nullptr) {
                const uint4 rv = *reinterpret_cast<const uint4*>(a.residual + i);
                const __half2* rh = reinterpret_cast<const __half2*>(&rv);
#pragma unroll
                for (int k = 0; k < 4; ++k) o[k] = __hadd2(rh[k], o[k]);
            }
            *reinterpret_cast<uint4*>(a.out + i) = *reinterpret_cast<const uint4*>(o);
        }
    }
    if (tid == 0) a.seq[b] = seq;
}

}  // namespace
}  // namespace eptq

using namespace eptq;

extern "C" size_t eptq_allreduce_data_bytes(int n_ranks, int n_max) {
    if (n_ranks < 1 || n_ranks > kArMaxRanks || n_max < 8 || (n_max % 8) != 0) return 0;
    return static_cast<size_t>(2) * n_ranks * n_max * sizeof(uint16_t);
}

extern "C" size_t eptq_allreduce_flag_bytes(int n_ranks) {
    if (n_ranks < 1 || n_ranks > kArMaxRanks) return 0;
    return static_cast<size_t>(2) * n_ranks * kArBlocks * sizeof(unsigned) + kArBlocks * sizeof(unsigned) + 16;
}

extern "C" int eptq_allreduce_push(const uint16_t* x, uint16_t* out, const uint16_t* residual, int n,
                                   void* const* peer_data, void* const* peer_flags, int rank, int n_ranks,
                                   int n_max, void* stream) {
    if (x == nullptr || out == nullptr || peer_data == nullptr || peer_flags == nullptr) return EPTQ_ERR_NULL;
    if (n_ranks < 1 || n_ranks > kArMaxRanks || rank < 0 || rank >= n_ranks || n < 8 || (n % 8) != 0 ||
        n > n_max || (n_max % 8) != 0) return EPTQ_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(out) || (residual != nullptr && !aligned16(residual))) return EPTQ_ERR_ALIGN;
    PushArgs a = {};
    for (int r = 0; r < n_ranks; ++r) {
        if (peer_data[r] == nullptr || peer_flags[r] == nullptr) return EPTQ_ERR_NULL;
        if (!aligned16(peer_data[r]) || !aligned16(peer_flags[r])) return EPTQ_ERR_ALIGN;
        a.data[r] = reinterpret_cast<__half*>(peer_data[r]);
        a.flags[r] = reinterpret_cast<unsigned*>(peer_flags[r]);
    }
    // this rank's own flag buffer ends with its call counters and the status word
    unsigned* own = a.flags[rank];
    a.seq = own + 2 * n_ranks * kArBlocks;
    a.status = reinterpret_cast<int*>(a.seq + kArBlocks);
    a.x = reinterpret_cast<const __half*>(x);
    a.out = reinterpret_cast<__half*>(out);
    a.residual = reinterpret_cast<const __half*>(residual);
    a.rank = rank; a.T = n_ranks; a.n = n; a.n_max = n_max;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kArBlocks);
    cfg.blockDim = dim3(kArThreads);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, allreduce_push_kernel, a);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaGetLastError() == cudaSuccess ? EPTQ_OK : EPTQ_ERR_LAUNCH;
}
