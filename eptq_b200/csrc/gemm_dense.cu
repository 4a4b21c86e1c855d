// Prefill GEMM on an already reconstructed fp16 weight (tcgen05 + TMEM + TMA), sm_100a.
//
// For long prefills the weight is reconstructed ONCE by dequant_kernel (bit-exact fp16, the reference's
// dequantize_layer) into scratch, and this kernel multiplies: y (T, out) = x (T, in) * W16 (out, in)^T (+ bias),
// fp32 accumulation in tensor memory.  The fused kernel (gemm_tcgen05_ws.cu) reconstructs every weight tile once
// per 512 tokens at ~35 instructions per index, which is what holds it at 40 % of the tensor peak; here both
// operands arrive by TMA and no thread touches them.
//
//   tile      256 tokens x 256 outputs per block: two accumulators of 128 lanes x 256 TMEM columns.
//   warp 0    TMA producer: per 64-wide K chunk two 128-token x 64-column boxes of x and two 128-output x 64-column
//             boxes of W16 (128-byte swizzle, 64 KB per stage, 3 stages), completion counted on the stage's
//             `full` barrier.
//   warp 1    MMA issuer: waits for `full`, issues 2 x 4 tcgen05.mma (M=128, N=256, K=16, fp16) and commits them
//             to the stage's `empty` barrier; the last commit also signals `acc_ready`.
//   warps 2-9 epilogue: tcgen05.ld (each warp its lane quarter and half of the columns), bias, fp16, 64 contiguous
//             bytes per token and pass.
//
// Same sums in the same K order as the fused kernel, so the two agree to fp32 rounding of the tensor core's
// accumulation.  No cluster, no multicast; every wait is bounded by the global timer and ends in a status word.
//
// Reference counterpart: e8d4_wmma_v2_kernel (csrc/eptq_kernels.cu:309-461) after dequantize_layer
// (algorithms/eptq.py:406-471).

#include <cuda.h>
#include <cudaTypedefs.h>

#include <mutex>

#include "common.cuh"

namespace eptq {

struct GemmDenseArgs {
    __half* y;             // (T, out)
    const __half* bias;    // (out) or null
    int* status;
    int T, out, N;
};

namespace {

constexpr int kChunkK = 64;
constexpr int kBoxBytes = 128 * kChunkK * 2;            // 16 KB: 128 rows x 64 columns, 128-byte rows
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = (2 + kEpilogueWarps) * 32;     // 320
// Tile: TM x 128 tokens by NT outputs (TM in {1, 2}, NT in {128, 256}); stages that fit in 200 KB, at most 4.
__host__ __device__ constexpr int dense_stage_bytes(int tm, int nt) { return (tm + nt / 128) * kBoxBytes; }
__host__ __device__ constexpr int dense_stages(int tm, int nt) { return 200 * 1024 / dense_stage_bytes(tm, nt) > 4 ? 4 : 200 * 1024 / dense_stage_bytes(tm, nt); }
__host__ __device__ constexpr int dense_smem_bytes(int tm, int nt) { return dense_stages(tm, nt) * dense_stage_bytes(tm, nt) + 1024; }
constexpr int kMaxStages = 4;
constexpr unsigned long long kWaitNs = 2000000000ull;   // limit of one mbarrier wait

__device__ __forceinline__ unsigned smem_u32(const void* p) {
    return static_cast<unsigned>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
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
// K-major operand tile, 128-byte swizzle (what the bulk-tensor load writes): 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t desc_sw128(unsigned addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;                  // leading byte offset: unused with swizzled K-major
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;                  // SWIZZLE_128B
    return d;
}
// fp32 accumulate, fp16 operands, both K-major, N = nt, M = 128
__host__ __device__ constexpr uint32_t instr_desc(int nt) { return (1u << 4) | (static_cast<uint32_t>(nt >> 3) << 17) | ((128u >> 4) << 24); }

template <int TM, int NT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_dense_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, const GemmDenseArgs p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ __align__(8) unsigned long long bar_full[kMaxStages], bar_empty[kMaxStages], bar_acc;
    __shared__ unsigned tmem_base_slot;
    constexpr int kStages = dense_stages(TM, NT);
    constexpr int kStageBytes = dense_stage_bytes(TM, NT);
    constexpr int kTileTokens = TM * 128, kTileOuts = NT;
    constexpr unsigned kTmemCols = TM * NT;               // 128, 256 or 512: a power of two >= 32
    constexpr uint32_t kInstrDesc = instr_desc(NT);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t0 = blockIdx.y * kTileTokens;
    const int o0 = blockIdx.x * kTileOuts;
    const int n_chunks = (p.N + kChunkK - 1) / kChunkK;
    // dynamic shared memory may start at an address that is not 1024-aligned: align by hand
    unsigned char* tiles = smem + ((1024u - (smem_u32(smem) & 1023u)) & 1023u);

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        mbar_init(smem_u32(&bar_acc), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" :: "l"(reinterpret_cast<uint64_t>(&tmap_x)) : "memory");
        asm volatile("prefetch.tensormap [%0];" :: "l"(reinterpret_cast<uint64_t>(&tmap_w)) : "memory");
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
                mbar_arrive_expect_tx(full, kStageBytes);
#pragma unroll
                for (int j = 0; j < TM; ++j)
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                        :: "r"(smem_u32(tiles + s * kStageBytes + j * kBoxBytes)), "l"(reinterpret_cast<uint64_t>(&tmap_x)),
                           "r"(c * kChunkK), "r"(t0 + j * 128), "r"(full)
                        : "memory");
#pragma unroll
                for (int j = 0; j < NT / 128; ++j)
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                        :: "r"(smem_u32(tiles + s * kStageBytes + (TM + j) * kBoxBytes)), "l"(reinterpret_cast<uint64_t>(&tmap_w)),
                           "r"(c * kChunkK), "r"(o0 + j * 128), "r"(full)
                        : "memory");
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
                // the W16 boxes are adjacent: NT rows of 128 bytes, one descriptor
                const uint64_t db = desc_sw128(smem_u32(tiles + s * kStageBytes + TM * kBoxBytes));
#pragma unroll
                for (int j = 0; j < TM; ++j) {
                    const uint64_t da = desc_sw128(smem_u32(tiles + s * kStageBytes + j * kBoxBytes));
#pragma unroll
                    for (int k = 0; k < kChunkK / 16; ++k) {
                        const unsigned accumulate = (c > 0 || k > 0) ? 1u : 0u;
                        asm volatile(
                            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                            :: "r"(tmem_acc + j * kTileOuts), "l"(da + static_cast<uint64_t>((k * 32) >> 4)),
                               "l"(db + static_cast<uint64_t>((k * 32) >> 4)), "r"(kInstrDesc), "r"(accumulate)
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
        // ---------------- epilogue: warp w reads TMEM lanes [32 (w & 3), +32) and half of each accumulator's columns
        ok = mbar_wait(smem_u32(&bar_acc), 0u);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            const int quarter = warp & 3;
            const int half = (warp - 2) >> 2;
#pragma unroll 1
            for (int j = 0; j < TM; ++j) {
                const int token = t0 + j * 128 + quarter * 32 + lane;
#pragma unroll 1
                for (int part = 0; part < NT / 64; ++part) {
                    const int col0 = half * (NT / 2) + part * 32;                  // output column inside the tile
                    const unsigned addr = tmem_acc + (static_cast<unsigned>(quarter * 32) << 16) + j * kTileOuts + col0;
                    unsigned r[32];
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                        : "r"(addr) : "memory");
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (token < p.T) {
                        const int o = o0 + col0;
                        __half* dsty = p.y + static_cast<size_t>(token) * p.out + o;
#pragma unroll
                        for (int v8 = 0; v8 < 4; ++v8) {
                            if (o + v8 * 8 < p.out) {                               // out % 8 == 0: eight outputs are in or out together
                                __half2 h2[4];
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    float f0 = __uint_as_float(r[v8 * 8 + 2 * e]), f1 = __uint_as_float(r[v8 * 8 + 2 * e + 1]);
                                    if (p.bias != nullptr) {
                                        f0 += __half2float(__ldg(p.bias + o + v8 * 8 + 2 * e));
                                        f1 += __half2float(__ldg(p.bias + o + v8 * 8 + 2 * e + 1));
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

PFN_cuTensorMapEncodeTiled_v12000 dense_map_encoder() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static std::once_flag once;
    std::call_once(once, []() {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
    });
    return fn;
}

// (rows, cols) fp16 row-major matrix as 128-row x 64-column boxes, 128-byte swizzle; rows and columns outside read zero.
bool encode_rows_map(const void* base, int rows, int cols, CUtensorMap* out) {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
    const cuuint32_t box[2] = {kChunkK, 128};
    const cuuint32_t estr[2] = {1, 1};
    return dense_map_encoder()(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int TM, int NT>
int launch_shape(const CUtensorMap& tx, const CUtensorMap& tw, const GemmDenseArgs& a, dim3 grid, int dev, cudaStream_t stream) {
    static std::once_flag attr_once[64];
    static bool attr_ok[64] = {};
    std::call_once(attr_once[dev], [dev]() {
        attr_ok[dev] = cudaFuncSetAttribute(gemm_dense_kernel<TM, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            dense_smem_bytes(TM, NT)) == cudaSuccess;
    });
    if (!attr_ok[dev]) return EPTQ_ERR_LAUNCH;
    gemm_dense_kernel<TM, NT><<<grid, kThreads, dense_smem_bytes(TM, NT), stream>>>(tx, tw, a);
    return EPTQ_OK;
}

}  // namespace

// Tokens from which "reconstruct once, then multiply" beats reconstructing every tile once per 512 tokens.
bool gemm_dense_supported(int T, int N, const void* x, const void* y, const void* bias) {
    return T >= kDenseMinTokens && (N % 8) == 0 && aligned16(x) && aligned16(y) && (bias == nullptr || aligned16(bias)) &&
           dense_map_encoder() != nullptr;
}

// y (T, out) = x (T, N) * W16 (out, N)^T (+ bias); W16 16-byte aligned.
int launch_gemm_dense(const uint16_t* W16, const uint16_t* x, uint16_t* y, const uint16_t* bias, int T, int out, int N,
                      int* status, cudaStream_t stream) {
    CUtensorMap tx, tw;
    if (!aligned16(W16) || !encode_rows_map(x, T, N, &tx) || !encode_rows_map(W16, out, N, &tw)) return EPTQ_ERR_LAUNCH;
    GemmDenseArgs a;
    a.y = reinterpret_cast<__half*>(y);
    a.bias = reinterpret_cast<const __half*>(bias);
    a.status = status;
    a.T = T; a.out = out; a.N = N;
    // Tile shape: the fewest rounds of blocks over the SMs, weighted by tile area and by what a smaller tile loses
    // in operand reuse (measured: half-size tiles run at about 0.85, quarter-size at about 0.7 of the full tile's rate).
    int n_sms = 0, dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 ||
        cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sms < 1)
        return EPTQ_ERR_LAUNCH;
    const int shapes[4][2] = {{2, 256}, {2, 128}, {1, 256}, {1, 128}};
    const double rate[4] = {1.0, 0.85, 0.85, 0.7};
    int best = 0;
    double best_cost = 0.0;
    for (int i = 0; i < 4; ++i) {
        const long long tiles = static_cast<long long>((out + shapes[i][1] - 1) / shapes[i][1]) * ((T + shapes[i][0] * 128 - 1) / (shapes[i][0] * 128));
        const double cost = static_cast<double>((tiles + n_sms - 1) / n_sms) * shapes[i][0] * shapes[i][1] / rate[i];
        if (i == 0 || cost < best_cost) { best = i; best_cost = cost; }
    }
    const int tm = shapes[best][0], nt = shapes[best][1];
    const dim3 grid((out + nt - 1) / nt, (T + tm * 128 - 1) / (tm * 128));
    if (grid.y > 65535u) return EPTQ_ERR_SHAPE;
    int st;
    if (tm == 2 && nt == 256) st = launch_shape<2, 256>(tx, tw, a, grid, dev, stream);
    else if (tm == 2) st = launch_shape<2, 128>(tx, tw, a, grid, dev, stream);
    else if (nt == 256) st = launch_shape<1, 256>(tx, tw, a, grid, dev, stream);
    else st = launch_shape<1, 128>(tx, tw, a, grid, dev, stream);
    if (st != EPTQ_OK) return st;
    count_launch(EPTQ_KERNEL_GEMM);
    return cudaPeekAtLastError() == cudaSuccess ? EPTQ_OK : EPTQ_ERR_LAUNCH;
}

}  // namespace eptq
