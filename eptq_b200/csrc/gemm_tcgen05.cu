// Prefill dequantise + GEMM on the Blackwell tensor cores (tcgen05 / TMEM), sm_100a.
//
//   y[t, o] = sum_n x[t, n] * W16[o, n] (+ bias[o]),   W16 = the reference's reconstructed fp16 weight
//
// The weight tile is reconstructed in the kernel with exactly the arithmetic of
// `dequantize_layer` (algorithms/eptq.py:406-471): fp32 table value (or the
// critical block from O, which skips the group scale), times S_group, times g,
// times h, each a separate fp32 multiply, one round-to-nearest-even to fp16.
// So the tensor cores multiply by bit-exact W16 tiles; nothing is pre-scaled
// onto the activations (the reference's WMMA kernel rounds x*h to fp16 first,
// csrc/eptq_kernels.cu:522, and applies g after the reduction, :457).
//
// One block computes a 128-token x 128-output tile:
//   * 128 producer threads fill two shared-memory tiles per 64-wide K chunk in
//     the canonical K-major, no-swizzle core-matrix layout (8 rows x 16 bytes
//     contiguous): the activation tile (one token row per thread) and the weight
//     tile.  One thread decodes 8 consecutive indices of one Q row; the 8 output
//     rows of a Q row are exactly one core matrix per index, so every decoded
//     index is one 128-bit shared-memory store.
//   * one thread issues four tcgen05.mma (M=128, N=128, K=16, fp16 in, fp32
//     accumulate in tensor memory) per chunk and commits them to an mbarrier;
//   * after the last chunk each warp reads its 32 TMEM lanes with tcgen05.ld,
//     adds the bias, converts to fp16 and stores 256 contiguous bytes per token.
// Every wait is bounded; on expiry the block records EPTQ_ERR_TIMEOUT in the
// status word, frees its tensor memory and returns.
//
// Reference counterpart: e8d4_wmma_v2_kernel (csrc/eptq_kernels.cu:309-461),
// E8-D4 only and never tested there (kernels/linear.py:16-18).

#include "common.cuh"

namespace eptq {

struct GemmArgs {
    EptqLayer L;
    const __half* x;       // (T, N)
    __half* y;             // (T, 8M)
    int* status;           // device word, set to EPTQ_ERR_TIMEOUT if a wait ran out
    int T;
};

namespace {

constexpr int kTileTokens = 128;    // UMMA M
constexpr int kTileOuts = 128;      // UMMA N (16 Q rows)
constexpr int kChunkK = 64;         // columns per shared-memory stage
constexpr int kGemmThreads = 128;
constexpr unsigned kLBO = 128;      // bytes between core matrices adjacent in K
constexpr unsigned kSBO = (kChunkK / 8) * 128;   // bytes between 8-row groups
constexpr int kTileBytes = 128 * kChunkK * 2;    // 16 KB per operand tile
constexpr unsigned kTmemCols = 128;
constexpr unsigned long long kWaitNs = 2000000000ull;     // limit of one mbarrier wait

__device__ __forceinline__ unsigned smem_u32(const void* p) {
    return static_cast<unsigned>(__cvta_generic_to_shared(p));
}

// Shared-memory matrix descriptor, K-major, no swizzle (version 1 = sm_100 format).
__device__ __forceinline__ uint64_t smem_desc(unsigned addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(kLBO >> 4) << 16;
    d |= static_cast<uint64_t>(kSBO >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    return d;
}

// Instruction descriptor: D = f32, A = B = f16, both K-major, N = 128, M = 128.
constexpr uint32_t kInstrDesc = (1u << 4) | ((kTileOuts >> 3) << 17) | ((kTileTokens >> 4) << 24);

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count));
}
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
    // Bounded by wall time (two seconds of the global timer, looked at every 1024 polls), not by a poll count
    // whose length would depend on the clock.
    unsigned long long t0 = 0;
    for (unsigned it = 0;; ++it) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if ((it & 1023u) == 1023u) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitNs) return false;
        }
    }
}

// Rank of column n among the markers of a row (markers are sorted by column).
__device__ __forceinline__ int marker_rank(const int* __restrict__ O_col, int lo, int hi, int n) {
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(O_col + mid) < n) lo = mid + 1; else hi = mid;
    }
    return lo;
}

// Reconstruct W16[8m .. 8m+7, n] exactly as the reference does: out[k] = fp16 of row 8m+k.
template <int KIND>
__device__ __forceinline__ void reconstruct8(const EptqLayer& L, int m, int n, unsigned q16, const float (&gk)[8],
                                             float hn, __half (&out)[8]) {
    const unsigned idx = q16 ^ 0x8000u;
    float v[8];
    if (idx == kMarkerIndex) {
        const int lo = __ldg(L.O_row_ptr + m), hi = __ldg(L.O_row_ptr + m + 1);
        const int r = marker_rank(L.O_col, lo, hi, n);
        unpack8(ldg128(reinterpret_cast<const __half*>(L.O_vals) + static_cast<size_t>(r) * 8), v);
    } else {
        if (KIND == EPTQ_E8) {
            const float4* t = reinterpret_cast<const float4*>(L.table32 + static_cast<size_t>(idx) * 8);
            const float4 a = __ldg(t), b = __ldg(t + 1);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
            const unsigned ct = (idx >> 14) & 3u;
            const float4 a = __ldg(reinterpret_cast<const float4*>(L.table32) + ct * 128 + ((idx >> 7) & 127u));
            const float4 b = __ldg(reinterpret_cast<const float4*>(L.table32) + ct * 128 + (idx & 127u));
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        }
        if (L.S_group != nullptr) {
            const __half* S = reinterpret_cast<const __half*>(L.S_group);
#pragma unroll
            for (int k = 0; k < 8; ++k)
                v[k] = __fmul_rn(v[k], __half2float(__ldg(S + static_cast<size_t>((8 * m + k) / L.qb_size) * L.N + n)));
        }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) out[k] = __float2half_rn(__fmul_rn(__fmul_rn(v[k], gk[k]), hn));
}

template <int KIND>
__global__ void __launch_bounds__(kGemmThreads) gemm_tcgen05_kernel(const GemmArgs p) {
    __shared__ __align__(1024) unsigned char tile_a[kTileBytes];     // activations: 128 tokens x 64 K
    __shared__ __align__(1024) unsigned char tile_b[kTileBytes];     // weights: 128 outputs x 64 K
    __shared__ __align__(8) unsigned long long mma_done;
    __shared__ unsigned tmem_base_slot;

    const EptqLayer& L = p.L;
    const int tid = threadIdx.x, warp = tid >> 5;
    const int N = L.N, out_dim = 8 * L.M;
    const int t0 = blockIdx.y * kTileTokens;          // first token of the tile
    const int m0 = blockIdx.x * (kTileOuts / 8);      // first Q row of the tile
    const unsigned bar = smem_u32(&mma_done);

    if (tid == 0) {
        mbar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_acc = tmem_base_slot;

    // producer roles: this thread owns token row `tid` of the A tile and, in the B tile,
    // Q row m0 + tid/8 at the 8 columns (tid%8)*8 .. +7 of each chunk.
    const int token = t0 + tid;
    const int bm = m0 + (tid >> 3);
    const int boct = tid & 7;
    const bool b_valid = bm < L.M;
    float gk[8];
#pragma unroll
    for (int k = 0; k < 8; ++k)
        gk[k] = b_valid ? __half2float(__ldg(reinterpret_cast<const __half*>(L.g) + 8 * bm + k)) : 0.f;
    unsigned char* a_dst = tile_a + (tid >> 3) * kSBO + (tid & 7) * 16;           // + oct * kLBO
    unsigned char* b_dst = tile_b + (tid >> 3) * kSBO + boct * kLBO;              // one whole core matrix

    bool ok = true;
    unsigned parity = 0;
    const int n_chunks = (N + kChunkK - 1) / kChunkK;
    for (int c = 0; c < n_chunks && ok; ++c) {
        const int k0 = c * kChunkK;
        // ---- A tile: 64 activations of this thread's token
#pragma unroll
        for (int oct = 0; oct < 8; ++oct) {
            uint4 v = make_uint4(0, 0, 0, 0);
            const int n = k0 + oct * 8;
            if (token < p.T && n < N) v = ldg128(p.x + static_cast<size_t>(token) * N + n);
            *reinterpret_cast<uint4*>(a_dst + oct * kLBO) = v;
        }
        // ---- B tile: 8 indices -> 8 x 8 reconstructed weights = one core matrix
        {
            const int n0 = k0 + boct * 8;
            __half blk[8][8];                                   // [column e][output row k]
            if (b_valid && n0 < N) {
                const uint4 qv = ldg128(L.Q + static_cast<size_t>(bm) * N + n0);
                const uint4 hv = ldg128(reinterpret_cast<const __half*>(L.h) + n0);
                const unsigned qw[4] = {qv.x, qv.y, qv.z, qv.w};
                float hf[8];
                unpack8(hv, hf);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const unsigned q16 = (e & 1) ? (qw[e >> 1] >> 16) : (qw[e >> 1] & 0xffffu);
                    reconstruct8<KIND>(L, bm, n0 + e, q16, gk, hf[e], blk[e]);
                }
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e)
#pragma unroll
                    for (int k = 0; k < 8; ++k) blk[e][k] = __float2half_rn(0.f);
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {                       // row k of the core matrix: 8 consecutive columns
                __half2 h2[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) h2[e] = __halves2half2(blk[2 * e][k], blk[2 * e + 1][k]);
                uint4 row;
                row.x = *reinterpret_cast<unsigned*>(&h2[0]);
                row.y = *reinterpret_cast<unsigned*>(&h2[1]);
                row.z = *reinterpret_cast<unsigned*>(&h2[2]);
                row.w = *reinterpret_cast<unsigned*>(&h2[3]);
                *reinterpret_cast<uint4*>(b_dst + k * 16) = row;
            }
        }
        // generic-proxy writes -> visible to the tensor core (async proxy), then hand over
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t da = smem_desc(smem_u32(tile_a)), db = smem_desc(smem_u32(tile_b));
#pragma unroll
            for (int j = 0; j < kChunkK / 16; ++j) {
                const uint64_t adv = static_cast<uint64_t>((j * 2 * kLBO) >> 4);      // two core matrices per K=16 step
                const unsigned accumulate = (c > 0 || j > 0) ? 1u : 0u;
                asm volatile(
                    "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                    "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                    :: "r"(tmem_acc), "l"(da + adv), "l"(db + adv), "r"(kInstrDesc), "r"(accumulate) : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
        }
        // the tiles may be overwritten only after the MMAs that read them have completed
        ok = __syncthreads_and(mbar_wait(bar, parity) ? 1 : 0) != 0;      // one decision for the whole block
        parity ^= 1u;
    }
    if (!ok && tid == 0) atomicExch(p.status, EPTQ_ERR_TIMEOUT);

    // ---- epilogue: TMEM lane = token, column = output of the tile
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
        const unsigned lane_addr = tmem_acc + (static_cast<unsigned>(warp * 32) << 16);
#pragma unroll
        for (int part = 0; part < kTileOuts / 32; ++part) {
            unsigned r[32];
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                  "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                  "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                  "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                : "r"(lane_addr + part * 32) : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (token < p.T) {
                const int o0 = blockIdx.x * kTileOuts + part * 32;
                __half* dst = p.y + static_cast<size_t>(token) * out_dim + o0;
#pragma unroll
                for (int v8 = 0; v8 < 4; ++v8) {
                    if (o0 + v8 * 8 < out_dim) {                 // out_dim is a multiple of 8
                        __half2 h2[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            float f0 = __uint_as_float(r[v8 * 8 + 2 * e]), f1 = __uint_as_float(r[v8 * 8 + 2 * e + 1]);
                            if (L.bias != nullptr) {
                                f0 += __half2float(__ldg(reinterpret_cast<const __half*>(L.bias) + o0 + v8 * 8 + 2 * e));
                                f1 += __half2float(__ldg(reinterpret_cast<const __half*>(L.bias) + o0 + v8 * 8 + 2 * e + 1));
                            }
                            h2[e] = __floats2half2_rn(f0, f1);
                        }
                        uint4 ov;
                        ov.x = *reinterpret_cast<unsigned*>(&h2[0]);
                        ov.y = *reinterpret_cast<unsigned*>(&h2[1]);
                        ov.z = *reinterpret_cast<unsigned*>(&h2[2]);
                        ov.w = *reinterpret_cast<unsigned*>(&h2[3]);
                        *reinterpret_cast<uint4*>(dst + v8 * 8) = ov;
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_acc), "r"(kTmemCols) : "memory");
    }
}

}  // namespace

bool gemm_supported(const EptqLayer& L, int T) {
    return T >= 1 && L.table32 != nullptr && (L.N % 8) == 0 && aligned16(L.Q) && aligned16(L.h) &&
           aligned16(L.table32) && (L.n_masked == 0 || aligned16(L.O_vals)) &&
           (L.S_group == nullptr || (L.qb_size > 0 && L.qb_size % 8 == 0));
}

// `status` must point at a zero-initialised device word (the last scratch counter is used).
int launch_gemm_tcgen05(const EptqLayer& L, const uint16_t* x, uint16_t* y, int T, int* status, cudaStream_t stream) {
    GemmArgs a;
    a.L = L;
    a.x = reinterpret_cast<const __half*>(x);
    a.y = reinterpret_cast<__half*>(y);
    a.status = status;
    a.T = T;
    const dim3 grid((8 * L.M + kTileOuts - 1) / kTileOuts, (T + kTileTokens - 1) / kTileTokens);
    if (grid.y > 65535u) return EPTQ_ERR_SHAPE;
    if (L.quantizer == EPTQ_E8) gemm_tcgen05_kernel<EPTQ_E8><<<grid, kGemmThreads, 0, stream>>>(a);
    else gemm_tcgen05_kernel<EPTQ_E8D4><<<grid, kGemmThreads, 0, stream>>>(a);
    count_launch(EPTQ_KERNEL_GEMM);
    return cudaPeekAtLastError() == cudaSuccess ? EPTQ_OK : EPTQ_ERR_LAUNCH;
}

}  // namespace eptq
