// Prefill dequantise + GEMM, warp-specialised and pipelined (tcgen05 + TMEM + TMA), sm_100a.
//
// Same arithmetic as gemm_tcgen05.cu (bit-exact fp16 weight tiles, fp32
// accumulation in tensor memory), organised so that the tensor cores are not
// left waiting for the reconstruction:
//
//   tile      TM*128 tokens x 128 outputs per block (TM = 1, 2 or 4 accumulators of
//             128 TMEM columns each).  Reconstructing a weight tile costs ~35
//             instructions per index and is repeated for every token tile, so the
//             token tile is made as tall as tensor memory allows (512 tokens).
//   warp 0    TMA producer: per 64-wide K chunk, TM bulk-tensor loads of a
//             128-token x 64-column activation box (128-byte swizzle) into the
//             stage's A tiles, completion counted on the stage's `full` barrier.
//   warp 1    MMA issuer: waits for `full`, issues TM x 4 tcgen05.mma
//             (M=128, N=128, K=16) and commits them to the stage's `empty`
//             barrier; the last commit also signals `acc_ready`.
//   warps 2-9 reconstruct the stage's 128-output x 64-column weight tile into the
//             no-swizzle core-matrix layout (4 indices per thread), make it visible
//             to the async proxy and arrive on `full`; afterwards they are the
//             epilogue: tcgen05.ld, bias, fp16, 256 contiguous bytes per token.
//
// No cluster, no multicast; every wait is bounded and ends in a status word.
//
// Reference counterpart: e8d4_wmma_v2_kernel (csrc/eptq_kernels.cu:309-461).

#include <cuda.h>
#include <atomic>
#include <cudaTypedefs.h>

#include "common.cuh"

namespace eptq {

struct GemmWsArgs {
    EptqLayer L;
    __half* y;             // (T, 8M)
    int* status;
    int T;
};

namespace {

constexpr int kMaxStages = 3;
constexpr int kChunkK = 64;
constexpr int kATileBytes = 128 * kChunkK * 2;          // 16 KB: 128 tokens x 64 columns, 128-byte rows
// B tile: core matrices (8 rows x 16 B = 128 contiguous bytes) adjacent in K are placed 144 bytes apart instead of
// 128, so that the threads of a warp, which write the same row of neighbouring core matrices, hit different banks.
constexpr unsigned kB_LBO = 144;                        // bytes between core matrices adjacent in K
constexpr unsigned kB_SBO = (kChunkK / 8) * kB_LBO;     // bytes between 8-row groups (1152)
constexpr int kProducerWarps = 16;                      // reconstruction is latency-bound: many warps
constexpr int kWsThreads = (2 + kProducerWarps) * 32;   // 576
constexpr unsigned long long kWaitNs = 2000000000ull;     // limit of one mbarrier wait

// Stages that fit in 227 KB next to the 8 KB table: 2 for 512x128 tiles (80 KB each), 3 for 256x256 (64 KB each).
__host__ __device__ constexpr int ws_stage_bytes(int tm, int nt) { return tm * kATileBytes + (nt / 8) * static_cast<int>(kB_SBO); }
__host__ __device__ constexpr int ws_stages(int tm, int nt) { return ws_stage_bytes(tm, nt) > 65536 ? 2 : 3; }
__host__ __device__ constexpr int ws_smem_bytes(int tm, int nt) { return ws_stages(tm, nt) * ws_stage_bytes(tm, nt) + 1024; }

__device__ __forceinline__ unsigned smem_u32(const void* p) {
    return static_cast<unsigned>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
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

// A tile: K-major, 128-byte swizzle (what the bulk-tensor load writes): 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t desc_a_sw128(unsigned addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;                  // leading byte offset: unused with swizzled K-major
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;                  // SWIZZLE_128B
    return d;
}
// B tile: K-major, no swizzle, core matrices of 8 rows x 16 bytes.
__device__ __forceinline__ uint64_t desc_b_plain(unsigned addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(kB_LBO >> 4) << 16;
    d |= static_cast<uint64_t>(kB_SBO >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    return d;
}
__host__ __device__ constexpr uint32_t instr_desc(int nt) { return (1u << 4) | (static_cast<uint32_t>(nt >> 3) << 17) | ((128u >> 4) << 24); }

__device__ __forceinline__ int marker_rank(const int* __restrict__ O_col, int lo, int hi, int n) {
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(O_col + mid) < n) lo = mid + 1; else hi = mid;
    }
    return lo;
}

// W16[8m .. 8m+7, n], bit-for-bit the reference's reconstruction (see gemm_tcgen05.cu).
template <int KIND>
__device__ __forceinline__ void reconstruct8(const EptqLayer& L, const float4* tab_s, int m, int n, unsigned q16,
                                             const float (&gk)[8], float hn, float sg, __half (&out)[8]) {
    const unsigned idx = q16 ^ 0x8000u;
    float v[8];
    if (idx == kMarkerIndex) {
        const int lo = __ldg(L.O_row_ptr + m), hi = __ldg(L.O_row_ptr + m + 1);
        const int r = marker_rank(L.O_col, lo, hi, n);
        unpack8(ldg128(reinterpret_cast<const __half*>(L.O_vals) + static_cast<size_t>(r) * 8), v);
    } else {
        float4 a, b;
        if (KIND == EPTQ_E8) {
            const float4* t = reinterpret_cast<const float4*>(L.table32 + static_cast<size_t>(idx) * 8);
            a = __ldg(t); b = __ldg(t + 1);
        } else {
            const unsigned ct = (idx >> 14) & 3u;
            a = tab_s[ct * 128 + ((idx >> 7) & 127u)];
            b = tab_s[ct * 128 + (idx & 127u)];
        }
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        if (L.S_group != nullptr) {
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = __fmul_rn(v[k], sg);
        }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) out[k] = __float2half_rn(__fmul_rn(__fmul_rn(v[k], gk[k]), hn));
}


template <int KIND, int TM, int NT>
__global__ void __launch_bounds__(kWsThreads, 1)
gemm_tcgen05_ws_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmWsArgs p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ __align__(16) float4 tab_s[KIND == EPTQ_E8D4 ? 512 : 1];
    __shared__ __align__(8) unsigned long long bar_full[kMaxStages], bar_empty[kMaxStages], bar_acc;
    __shared__ unsigned tmem_base_slot;

    constexpr int kStages = ws_stages(TM, NT);
    constexpr int kStageBytes = ws_stage_bytes(TM, NT);
    constexpr unsigned kTmemCols = TM * NT;               // 128, 256 or 512: a power of two >= 32
    constexpr int kTileOuts = NT;
    constexpr uint32_t kInstrDesc = instr_desc(NT);
    const EptqLayer& L = p.L;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int N = L.N, out_dim = 8 * L.M;
    const int t0 = blockIdx.y * (TM * 128);
    const int m0 = blockIdx.x * (kTileOuts / 8);
    const int n_chunks = (N + kChunkK - 1) / kChunkK;
    // dynamic shared memory may start at an address that is not 1024-aligned: align by hand
    unsigned char* tiles = smem + ((1024u - (smem_u32(smem) & 1023u)) & 1023u);

    if (KIND == EPTQ_E8D4)
        for (int i = tid; i < 512; i += kWsThreads) tab_s[i] = __ldg(reinterpret_cast<const float4*>(L.table32) + i);
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1 + kProducerWarps);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        mbar_init(smem_u32(&bar_acc), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" :: "l"(reinterpret_cast<uint64_t>(&tmap_x)) : "memory");
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
    bool ok = true;

    if (warp == 0) {
        // ---------------- TMA producer
        if (lane == 0) {
            for (int c = 0; c < n_chunks && ok; ++c) {
                const int s = c % kStages;
                const unsigned phase = (c / kStages) & 1u;
                ok = mbar_wait(smem_u32(&bar_empty[s]), phase ^ 1u);
                if (!ok) break;
                const unsigned full = smem_u32(&bar_full[s]);
                mbar_arrive_expect_tx(full, TM * kATileBytes);
#pragma unroll
                for (int j = 0; j < TM; ++j) {
                    const unsigned dst = smem_u32(tiles + s * kStageBytes + j * kATileBytes);
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                        :: "r"(dst), "l"(reinterpret_cast<uint64_t>(&tmap_x)), "r"(c * kChunkK), "r"(t0 + j * 128), "r"(full)
                        : "memory");
                }
            }
            if (!ok) atomicExch(p.status, EPTQ_ERR_TIMEOUT);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer
        if (lane == 0) {
            for (int c = 0; c < n_chunks && ok; ++c) {
                const int s = c % kStages;
                const unsigned phase = (c / kStages) & 1u;
                ok = mbar_wait(smem_u32(&bar_full[s]), phase);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t db = desc_b_plain(smem_u32(tiles + s * kStageBytes + TM * kATileBytes));
#pragma unroll
                for (int j = 0; j < TM; ++j) {
                    const uint64_t da = desc_a_sw128(smem_u32(tiles + s * kStageBytes + j * kATileBytes));
#pragma unroll
                    for (int k = 0; k < kChunkK / 16; ++k) {
                        const unsigned accumulate = (c > 0 || k > 0) ? 1u : 0u;
                        asm volatile(
                            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                            :: "r"(tmem_acc + j * NT), "l"(da + static_cast<uint64_t>((k * 32) >> 4)),
                               "l"(db + static_cast<uint64_t>((k * 2 * kB_LBO) >> 4)), "r"(kInstrDesc), "r"(accumulate)
                            : "memory");
                    }
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                             :: "r"(smem_u32(&bar_empty[s])) : "memory");
            }
            if (ok)
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                             :: "r"(smem_u32(&bar_acc)) : "memory");
            else
                atomicExch(p.status, EPTQ_ERR_TIMEOUT);
        }
    } else {
        // ---------------- weight-tile producers (256 threads), then epilogue
        // NT/8 Q rows x 64 columns per chunk over 512 threads: CPT = 2 (NT=128) or 4 (NT=256) columns each
        constexpr int CPT = (NT / 8) * kChunkK / (kProducerWarps * 32);
        constexpr int kThreadsPerRow = kChunkK / CPT;
        const int pid = tid - 64;
        const int qrow = pid / kThreadsPerRow, c4 = pid % kThreadsPerRow;
        const int bm = m0 + qrow;
        const bool b_valid = bm < L.M;
        float gk[8];
#pragma unroll
        for (int k = 0; k < 8; ++k)
            gk[k] = b_valid ? __half2float(__ldg(reinterpret_cast<const __half*>(L.g) + 8 * bm + k)) : 0.f;
        const __half* srow = (L.S_group != nullptr && b_valid)
            ? reinterpret_cast<const __half*>(L.S_group) + static_cast<size_t>((8 * bm) / L.qb_size) * N : nullptr;
        const unsigned b_off = qrow * kB_SBO + ((c4 * CPT) >> 3) * kB_LBO + ((c4 * CPT) & 7) * 2;

        // this thread's indices, column scales and group scales of one chunk; loaded one chunk ahead
        struct Inputs { unsigned q[CPT / 2], h[CPT / 2], s[CPT / 2]; };
        auto fetch = [&](int c, Inputs& in) {
            const int n0 = c * kChunkK + c4 * CPT;
#pragma unroll
            for (int i = 0; i < CPT / 2; ++i) { in.q[i] = 0u; in.h[i] = 0u; in.s[i] = 0x3c003c00u; }
            if (b_valid && n0 < N && c < n_chunks) {          // N % 8 == 0: CPT columns are in or out together
                const unsigned* qp = reinterpret_cast<const unsigned*>(L.Q + static_cast<size_t>(bm) * N + n0);
                const unsigned* hp = reinterpret_cast<const unsigned*>(reinterpret_cast<const __half*>(L.h) + n0);
#pragma unroll
                for (int i = 0; i < CPT / 2; ++i) { in.q[i] = __ldg(qp + i); in.h[i] = __ldg(hp + i); }
                if (srow != nullptr) {
                    const unsigned* sp = reinterpret_cast<const unsigned*>(srow + n0);
#pragma unroll
                    for (int i = 0; i < CPT / 2; ++i) in.s[i] = __ldg(sp + i);
                }
            }
        };
        Inputs nxt;
        fetch(0, nxt);
        for (int c = 0; c < n_chunks && ok; ++c) {
            const int s = c % kStages;
            const unsigned phase = (c / kStages) & 1u;
            const int n0 = c * kChunkK + c4 * CPT;
            const Inputs cur = nxt;
            const bool live = b_valid && n0 < N;
            fetch(c + 1, nxt);
            ok = mbar_wait(smem_u32(&bar_empty[s]), phase ^ 1u);
            if (!ok) break;
            __half blk[CPT][8];
            if (live) {
#pragma unroll
                for (int e = 0; e < CPT; ++e) {
                    const unsigned q16 = (e & 1) ? (cur.q[e >> 1] >> 16) : (cur.q[e >> 1] & 0xffffu);
                    const float2 h2f = __half22float2(*reinterpret_cast<const __half2*>(&cur.h[e >> 1]));
                    const float2 s2f = __half22float2(*reinterpret_cast<const __half2*>(&cur.s[e >> 1]));
                    reconstruct8<KIND>(L, tab_s, bm, n0 + e, q16, gk, (e & 1) ? h2f.y : h2f.x, (e & 1) ? s2f.y : s2f.x, blk[e]);
                }
            } else {
#pragma unroll
                for (int e = 0; e < CPT; ++e)
#pragma unroll
                    for (int k = 0; k < 8; ++k) blk[e][k] = __float2half_rn(0.f);
            }
            unsigned char* dst = tiles + s * kStageBytes + TM * kATileBytes + b_off;
#pragma unroll
            for (int k = 0; k < 8; ++k) {                     // row k of the core matrix: CPT consecutive columns
                unsigned w[CPT / 2];
#pragma unroll
                for (int i = 0; i < CPT / 2; ++i) {
                    const __half2 pr = __halves2half2(blk[2 * i][k], blk[2 * i + 1][k]);
                    w[i] = *reinterpret_cast<const unsigned*>(&pr);
                }
                if (CPT == 8) *reinterpret_cast<uint4*>(dst + k * 16) = make_uint4(w[0], w[1], w[CPT / 2 - 2], w[CPT / 2 - 1]);
                else if (CPT == 4) *reinterpret_cast<uint2*>(dst + k * 16) = make_uint2(w[0], w[CPT / 2 - 1]);
                else *reinterpret_cast<unsigned*>(dst + k * 16) = w[0];
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_full[s]));
        }
        if (!ok && lane == 0) atomicExch(p.status, EPTQ_ERR_TIMEOUT);

        // ---------------- epilogue
        if (ok) ok = mbar_wait(smem_u32(&bar_acc), 0u);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            // The accumulators occupy TMEM columns [0, TM*NT): sub-tile j (128 tokens) at columns [j*NT, (j+1)*NT).
            // Four groups of four warps (one warp per lane quarter) each take a quarter of those columns.
            const int quarter = warp & 3;                    // TMEM lanes this warp may read
            const int group = (warp - 2) >> 2;
            constexpr int kColsPerGroup = TM * NT / 4;       // 32 .. 128, a multiple of 32
            {
                const int acc_col0 = group * kColsPerGroup;
                const int j = acc_col0 / NT;
                const int col0 = acc_col0 % NT;              // first output column (inside the tile) of this group
                const int token = t0 + j * 128 + quarter * 32 + lane;
                const unsigned lane_addr = tmem_acc + (static_cast<unsigned>(quarter * 32) << 16) + acc_col0;
#pragma unroll
                for (int part = 0; part < kColsPerGroup / 32; ++part) {
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
                        const int o0 = blockIdx.x * kTileOuts + col0 + part * 32;
                        __half* dsty = p.y + static_cast<size_t>(token) * out_dim + o0;
#pragma unroll
                        for (int v8 = 0; v8 < 4; ++v8) {
                            if (o0 + v8 * 8 < out_dim) {
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
                                *reinterpret_cast<uint4*>(dsty + v8 * 8) = ov;
                            }
                        }
                    }
                }
            }
        } else if (lane == 0) {
            atomicExch(p.status, EPTQ_ERR_TIMEOUT);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_acc), "r"(kTmemCols) : "memory");
    }
}

PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
    }
    return fn;
}

template <int KIND, int TM, int NT>
int launch_ws(const CUtensorMap& tmap, const GemmWsArgs& a, dim3 grid, cudaStream_t stream) {
    static std::atomic<bool> attr_done[64];       // setting the attribute twice is harmless; the flag itself must not race
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return EPTQ_ERR_LAUNCH;
    if (!attr_done[dev]) {
        if (cudaFuncSetAttribute(gemm_tcgen05_ws_kernel<KIND, TM, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 ws_smem_bytes(TM, NT)) != cudaSuccess)
            return EPTQ_ERR_LAUNCH;
        attr_done[dev] = true;
    }
    gemm_tcgen05_ws_kernel<KIND, TM, NT><<<grid, kWsThreads, ws_smem_bytes(TM, NT), stream>>>(tmap, a);
    count_launch(EPTQ_KERNEL_GEMM);
    return cudaPeekAtLastError() == cudaSuccess ? EPTQ_OK : EPTQ_ERR_LAUNCH;
}

template <int KIND>
int launch_ws_shape(int tm, int nt, const CUtensorMap& tmap, const GemmWsArgs& a, dim3 grid, cudaStream_t stream) {
    if (nt == 256) return tm == 1 ? launch_ws<KIND, 1, 256>(tmap, a, grid, stream) : launch_ws<KIND, 2, 256>(tmap, a, grid, stream);
    switch (tm) {
        case 1: return launch_ws<KIND, 1, 128>(tmap, a, grid, stream);
        case 2: return launch_ws<KIND, 2, 128>(tmap, a, grid, stream);
        default: return launch_ws<KIND, 4, 128>(tmap, a, grid, stream);
    }
}

}  // namespace

// The pipelined kernel needs a tensor map over x: base 16-byte aligned, row pitch a multiple of 16 bytes.
bool gemm_ws_supported(const EptqLayer& L, const void* x, int T) {
    return T >= 1 && L.table32 != nullptr && (L.N % 8) == 0 && aligned16(x) && aligned16(L.Q) && aligned16(L.h) &&
           aligned16(L.table32) && (L.n_masked == 0 || aligned16(L.O_vals)) &&
           (L.S_group == nullptr || (L.qb_size > 0 && L.qb_size % 8 == 0 && aligned16(L.S_group))) &&
           tensor_map_encoder() != nullptr;
}

int launch_gemm_tcgen05_ws(const EptqLayer& L, const uint16_t* x, uint16_t* y, int T, int* status, cudaStream_t stream) {
    const int out_dim = 8 * L.M;
    const int nt = 128;      // measured: 256-output tiles double the reconstruction per stage and run ~20 % slower
    const int tm = nt == 256 ? (T <= 128 ? 1 : 2) : (T <= 128 ? 1 : (T <= 256 ? 2 : 4));
    CUtensorMap tmap;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(L.N), static_cast<cuuint64_t>(T)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(L.N) * 2};
    const cuuint32_t box[2] = {kChunkK, 128};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult res = tensor_map_encoder()(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<uint16_t*>(x), dims, strides,
                                              box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_SUCCESS) return EPTQ_ERR_LAUNCH;
    GemmWsArgs a;
    a.L = L;
    a.y = reinterpret_cast<__half*>(y);
    a.status = status;
    a.T = T;
    const dim3 grid((out_dim + nt - 1) / nt, (T + tm * 128 - 1) / (tm * 128));
    if (grid.y > 65535u) return EPTQ_ERR_SHAPE;
    return L.quantizer == EPTQ_E8 ? launch_ws_shape<EPTQ_E8>(tm, nt, tmap, a, grid, stream)
                                  : launch_ws_shape<EPTQ_E8D4>(tm, nt, tmap, a, grid, stream);
}

}  // namespace eptq
