// One-shot all-reduce of a small fp16 vector between the GPUs of one node, for the partial outputs of
// the row-parallel layers (o / down projections) of a tensor-parallel decode step.  The reference is
// single-GPU (kernels/patch.py:24-27); NCCL's all-reduce of 8 KB costs more than the GEMV it follows,
// so each rank instead stores its partial straight into a slot of every peer's buffer over NVLink
// (ordinary global stores through peer pointers, each word carrying its own arrival tag), polls its own
// slots until the peers' words are there and sums them locally.  No TMA, no multicast loads, no reads of remote memory: only stores go out.
//
// Buffers per rank (allocated and exchanged by the caller): data [2 parities][T sources][n_max/2] words of
// 8 bytes (two fp16 values + the call number), and a small block of call counters and a status word.
// Call k uses parity k & 1 and tags its words with k; a rank can enter call k+1 only after it received every
// rank's words of call k, i.e. after every rank has finished reading call k-1, so two parities suffice and a
// stale word can never carry the current tag.  Every wait is bounded (two seconds of wall time); on a timeout the kernel records
// EPTQ_ERR_TIMEOUT and returns.

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/eptq_b200.h"
#include "common.cuh"

namespace eptq {
namespace {

constexpr int kArBlocks = 8;
constexpr int kArThreads = 128;
constexpr int kArMaxRanks = 8;
constexpr unsigned long long kArWaitNs = 2000000000ull;   // default: a wait gives up after two seconds
unsigned long long g_ar_wait_ns = kArWaitNs;              // changed only by eptq_allreduce_set_wait_ns

struct PushArgs {
    __half* data[kArMaxRanks];        // every rank's data buffer (this rank's own included)
    unsigned* flags[kArMaxRanks];     // every rank's flag buffer
    const __half* x;                  // this rank's partial, n elements
    __half* out;                      // the sum, n elements (may be x or residual)
    const __half* residual;           // optional: out = residual + sum (each rounded to fp16)
    unsigned* seq;                    // kArBlocks call counters of this rank
    int* status;                      // set to EPTQ_ERR_TIMEOUT if a wait ran out
    int rank, T, n, n_max;
    unsigned long long wait_ns;       // limit of the wait for the peers' words
};

__global__ void __launch_bounds__(kArThreads) allreduce_push_kernel(const PushArgs a) {
    __shared__ unsigned s_seq;
    const int tid = threadIdx.x, b = blockIdx.x;
    // Programmatic dependent launch: the next kernel may begin its set-up while this one exchanges data;
    // this one waits for its producer before it reads x.
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tid == 0) s_seq = a.seq[b] + 1u;
    __syncthreads();
    const unsigned seq = s_seq;
    const unsigned parity = seq & 1u;
    // A word is two fp16 values plus the call number in ONE 64-bit register, written with one b64 store and read
    // with one b64 load (single-copy atomic when 8-byte aligned): the receiver polls the word itself, so no
    // fence and no separate flag are needed (the payload and its tag cannot be seen apart).
    const int words = a.n >> 1, words_max = a.n_max >> 1;
    const size_t my_slot = (static_cast<size_t>(parity) * a.T + a.rank) * words_max;
    const unsigned* x32 = reinterpret_cast<const unsigned*>(a.x);
    for (int w = b * kArThreads + tid; w < words; w += kArBlocks * kArThreads) {
        const unsigned v = x32[w];
        for (int r = 0; r < a.T; ++r) {
            unsigned long long* dst = reinterpret_cast<unsigned long long*>(a.data[r]) + my_slot + w;
            const unsigned long long word = static_cast<unsigned long long>(v) | (static_cast<unsigned long long>(seq) << 32);
            asm volatile("st.relaxed.sys.global.b64 [%0], %1;" :: "l"(dst), "l"(word) : "memory");
        }
    }
    const uint2* mine = reinterpret_cast<const uint2*>(a.data[a.rank]) + static_cast<size_t>(parity) * a.T * words_max;
    const unsigned* res32 = reinterpret_cast<const unsigned*>(a.residual);
    unsigned* out32 = reinterpret_cast<unsigned*>(a.out);
    bool ok = true;
    for (int w = b * kArThreads + tid; w < words && ok; w += kArBlocks * kArThreads) {
        // One pass issues the loads of all sources that are still missing before it looks at any of them, so
        // that the round trips overlap; the wait is bounded by wall time (the global timer), checked every
        // 256 passes.
        unsigned val[kArMaxRanks];
        unsigned missing = (1u << a.T) - 1u;
        unsigned long long t_start = 0;
        for (unsigned pass = 0; missing != 0u; ++pass) {
            unsigned lo[kArMaxRanks], flag[kArMaxRanks];
#pragma unroll
            for (int r = 0; r < kArMaxRanks; ++r)
                if ((missing >> r) & 1u) {
                    const uint2* src = mine + static_cast<size_t>(r) * words_max + w;
                    unsigned long long word;
                    asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(word) : "l"(src) : "memory");
                    lo[r] = static_cast<unsigned>(word);
                    flag[r] = static_cast<unsigned>(word >> 32);
                }
#pragma unroll
            for (int r = 0; r < kArMaxRanks; ++r)
                if (((missing >> r) & 1u) && flag[r] == seq) { val[r] = lo[r]; missing &= ~(1u << r); }
            if (missing != 0u && (pass & 255u) == 255u) {
                unsigned long long now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (t_start == 0) t_start = now;
                else if (now - t_start > a.wait_ns) { ok = false; break; }
            }
        }
        if (!ok) { atomicExch(a.status, static_cast<int>(EPTQ_ERR_TIMEOUT)); break; }
        float2 acc = make_float2(0.f, 0.f);
#pragma unroll
        for (int r = 0; r < kArMaxRanks; ++r)
            if (r < a.T) {                                   // fixed order: every rank computes the same sum
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&val[r]));
                acc.x += f.x; acc.y += f.y;
            }
        __half2 o = __floats2half2_rn(acc.x, acc.y);
        if (res32 != nullptr) {
            const unsigned rv = res32[w];
            o = __hadd2(*reinterpret_cast<const __half2*>(&rv), o);
        }
        out32[w] = *reinterpret_cast<const unsigned*>(&o);
    }
    __syncthreads();
    if (tid == 0) a.seq[b] = seq;
}

}  // namespace
}  // namespace eptq

using namespace eptq;

extern "C" size_t eptq_allreduce_data_bytes(int n_ranks, int n_max) {
    if (n_ranks < 1 || n_ranks > kArMaxRanks || n_max < 8 || (n_max % 8) != 0) return 0;
    return static_cast<size_t>(2) * n_ranks * (n_max / 2) * 8;
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
    if ((n % 2) != 0 || !aligned16(x) || !aligned16(out) || (residual != nullptr && !aligned16(residual))) return EPTQ_ERR_ALIGN;
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
    a.wait_ns = g_ar_wait_ns;
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
    count_launch(EPTQ_KERNEL_OTHER);
    return cudaGetLastError() == cudaSuccess ? EPTQ_OK : EPTQ_ERR_LAUNCH;
}

// Limit of the device-side wait of later eptq_allreduce_push calls, in nanoseconds (0 restores the default of
// two seconds).  For tests of the timeout path; process-wide.
extern "C" void eptq_allreduce_set_wait_ns(unsigned long long ns) { g_ar_wait_ns = ns == 0 ? kArWaitNs : ns; }
