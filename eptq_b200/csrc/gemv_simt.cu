// General fused dequantise + GEMV on the CUDA cores.
//
// Computes, for every batch row b and Q row m (8 outputs each),
//   y[b, 8m+k] = g[8m+k] * ( sum_{n unmarked} cb[Q[m,n]][k] * s[m,n] * h[n] * x[b,n]
//                          + sum_{i marked in row m} O[i][k] * h[n_i] * x[b,n_i] ) + bias[8m+k]
// which is the formula of the reference's fused kernels
// (csrc/eptq_kernels.cu:39-150 for E8, :161-292 for E8-D4) extended by the group
// scale s[m,n] = S_group[8m/qb, n] the reference has no kernel for.
//
// This variant covers every shape, both codebooks, group scales, N that is not
// a multiple of 8 and any batch; it is the path for E8 (whose 1 MB table lives
// in L2) and for layers the tensor-core GEMV does not take.
//
// Work split: one warp streams one Q row over one column range with 128-bit
// loads and decodes each index once for up to BT batch rows.  Column ranges
// ("splits") of one row block are combined through a scratch buffer: every
// block writes its partial sums, takes a ticket, and the last block to arrive
// adds the partials in split order (so results do not depend on arrival
// order), applies g and bias and writes fp16.  The ticket counter is left at
// zero for the next call.

#include "common.cuh"

namespace eptq {

struct GemvArgs {
    const int16_t* Q;
    const __half* table16;
    const __half* g;
    const __half* h;
    const __half* x;
    const __half* O_vals;
    const int* O_col;
    const int* O_row_ptr;
    const __half* bias;
    const __half* S_group;
    __half* y;
    float* partial;
    unsigned* counters;
    int M, N, B;
    int qb_rows;          // qb_size / 8 (Q rows per scale group), 0 without group scales
    int splits;
    int cols_per_split;   // multiple of 8
};

namespace {

template <int KIND>
__device__ __forceinline__ void fetch_codeword(unsigned idx, const __half* __restrict__ table16,
                                               const float* tab_s, float (&cw)[8]) {
    if (KIND == EPTQ_E8) {
        const uint4 raw = ldg128(table16 + static_cast<size_t>(idx) * 8);
        unpack8(raw, cw);
    } else {
        const unsigned ct = (idx >> 14) & 3u;
        const float4 a = *reinterpret_cast<const float4*>(tab_s + ((ct << 7) | ((idx >> 7) & 127u)) * 4);
        const float4 b = *reinterpret_cast<const float4*>(tab_s + ((ct << 7) | (idx & 127u)) * 4);
        cw[0] = a.x; cw[1] = a.y; cw[2] = a.z; cw[3] = a.w;
        cw[4] = b.x; cw[5] = b.y; cw[6] = b.z; cw[7] = b.w;
    }
}

template <int KIND, int BT>
__global__ void __launch_bounds__(256) gemv_simt_kernel(GemvArgs p) {
    __shared__ __align__(16) float tab_s[KIND == EPTQ_E8D4 ? 2048 : 4];
    __shared__ unsigned s_last;

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    if (KIND == EPTQ_E8D4) {
        for (int i = threadIdx.x; i < 2048; i += blockDim.x) tab_s[i] = __half2float(__ldg(p.table16 + i));
        __syncthreads();
    }

    const int m = blockIdx.x * kRowsPerCta + warp;
    const int split = blockIdx.y;
    const int b0 = blockIdx.z * BT;
    const int N = p.N;
    const int c0 = split * p.cols_per_split;
    const int c1 = min(N, c0 + p.cols_per_split);

    float acc[BT][8];
#pragma unroll
    for (int bt = 0; bt < BT; ++bt)
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[bt][k] = 0.f;

    if (m < p.M) {
        const int16_t* qrow = p.Q + static_cast<size_t>(m) * N;
        const __half* srow = (p.qb_rows > 0) ? p.S_group + static_cast<size_t>(m / p.qb_rows) * N : nullptr;

        if ((N & 7) == 0) {
            for (int n = c0 + lane * 8; n < c1; n += 256) {
                const uint4 qv = ldg128(qrow + n);
                float hf[8];
                unpack8(ldg128(p.h + n), hf);
                if (srow != nullptr) {
                    float sf[8];
                    unpack8(ldg128(srow + n), sf);
#pragma unroll
                    for (int e = 0; e < 8; ++e) hf[e] *= sf[e];
                }
                float xh[BT][8];
#pragma unroll
                for (int bt = 0; bt < BT; ++bt) {
                    if (b0 + bt < p.B) {
                        unpack8(ldg128(p.x + static_cast<size_t>(b0 + bt) * N + n), xh[bt]);
#pragma unroll
                        for (int e = 0; e < 8; ++e) xh[bt][e] *= hf[e];
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; ++e) xh[bt][e] = 0.f;
                    }
                }
                const unsigned short* qs = reinterpret_cast<const unsigned short*>(&qv);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const unsigned idx = static_cast<unsigned>(qs[e]) ^ 0x8000u;
                    if (idx == kMarkerIndex) continue;
                    float cw[8];
                    fetch_codeword<KIND>(idx, p.table16, tab_s, cw);
#pragma unroll
                    for (int bt = 0; bt < BT; ++bt)
#pragma unroll
                        for (int k = 0; k < 8; ++k) acc[bt][k] = fmaf(cw[k], xh[bt][e], acc[bt][k]);
                }
            }
        } else {
            for (int n = c0 + lane; n < c1; n += 32) {
                const unsigned idx = static_cast<unsigned>(static_cast<int>(qrow[n]) + 32768);
                if (idx == kMarkerIndex) continue;
                float hs = __half2float(__ldg(p.h + n));
                if (srow != nullptr) hs *= __half2float(__ldg(srow + n));
                float cw[8];
                fetch_codeword<KIND>(idx, p.table16, tab_s, cw);
#pragma unroll
                for (int bt = 0; bt < BT; ++bt) {
                    if (b0 + bt < p.B) {
                        const float xv = hs * __half2float(__ldg(p.x + static_cast<size_t>(b0 + bt) * N + n));
#pragma unroll
                        for (int k = 0; k < 8; ++k) acc[bt][k] = fmaf(cw[k], xv, acc[bt][k]);
                    }
                }
            }
        }

        // Critical blocks of this row whose column falls into this split.  They
        // carry h but not the group scale (algorithms/eptq.py:461-466).
        const int o_lo = __ldg(p.O_row_ptr + m), o_hi = __ldg(p.O_row_ptr + m + 1);
        for (int i = o_lo + lane; i < o_hi; i += 32) {
            const int col = __ldg(p.O_col + i);
            if (col < c0 || col >= c1) continue;
            float ov[8];
            unpack8(ldg128(p.O_vals + static_cast<size_t>(i) * 8), ov);
            const float hc = __half2float(__ldg(p.h + col));
#pragma unroll
            for (int bt = 0; bt < BT; ++bt) {
                if (b0 + bt < p.B) {
                    const float xv = hc * __half2float(__ldg(p.x + static_cast<size_t>(b0 + bt) * N + col));
#pragma unroll
                    for (int k = 0; k < 8; ++k) acc[bt][k] = fmaf(ov[k], xv, acc[bt][k]);
                }
            }
        }
    }

    // Butterfly reduction over the 32 lanes; afterwards every lane holds the sums.
#pragma unroll
    for (int bt = 0; bt < BT; ++bt)
#pragma unroll
        for (int k = 0; k < 8; ++k)
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) acc[bt][k] += __shfl_xor_sync(0xffffffffu, acc[bt][k], off);

    const int out_dim = 8 * p.M;
    if (p.splits == 1) {
        if (m < p.M && lane < 8) {
            const int o = 8 * m + lane;
            const float gs = __half2float(__ldg(p.g + o));
            const float bs = p.bias ? __half2float(__ldg(p.bias + o)) : 0.f;
#pragma unroll
            for (int bt = 0; bt < BT; ++bt) {
                if (b0 + bt < p.B) {
                    float v = 0.f;
#pragma unroll
                    for (int k = 0; k < 8; ++k) v = (lane == k) ? acc[bt][k] : v;
                    p.y[static_cast<size_t>(b0 + bt) * out_dim + o] = __float2half_rn(v * gs + bs);
                }
            }
        }
        return;
    }

    // Split columns: publish partial sums, last block to arrive reduces them.
    if (m < p.M && lane < 8) {
        const int o = 8 * m + lane;
#pragma unroll
        for (int bt = 0; bt < BT; ++bt) {
            if (b0 + bt < p.B) {
                float v = 0.f;
#pragma unroll
                for (int k = 0; k < 8; ++k) v = (lane == k) ? acc[bt][k] : v;
                __stcg(p.partial + (static_cast<size_t>(split) * p.B + (b0 + bt)) * out_dim + o, v);
            }
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned* ctr = p.counters + blockIdx.z * gridDim.x + blockIdx.x;
        const unsigned ticket = atomicAdd(ctr, 1u);
        s_last = (ticket == static_cast<unsigned>(p.splits) - 1u) ? 1u : 0u;
        if (s_last) *ctr = 0u;   // nobody else touches it before the next call
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int t = threadIdx.x; t < kRowsPerCta * 8 * BT; t += blockDim.x) {
        const int bt = t / (kRowsPerCta * 8);
        const int o = blockIdx.x * kRowsPerCta * 8 + (t % (kRowsPerCta * 8));
        if (o >= out_dim || b0 + bt >= p.B) continue;
        float v = 0.f;
        for (int s = 0; s < p.splits; ++s)
            v += __ldcg(p.partial + (static_cast<size_t>(s) * p.B + (b0 + bt)) * out_dim + o);
        const float gs = __half2float(__ldg(p.g + o));
        const float bs = p.bias ? __half2float(__ldg(p.bias + o)) : 0.f;
        p.y[static_cast<size_t>(b0 + bt) * out_dim + o] = __float2half_rn(v * gs + bs);
    }
}

template <int KIND>
int launch_simt_kind(const GemvArgs& a, int bt, dim3 grid, cudaStream_t stream) {
    switch (bt) {
        case 1: gemv_simt_kernel<KIND, 1><<<grid, 256, 0, stream>>>(a); break;
        case 2: gemv_simt_kernel<KIND, 2><<<grid, 256, 0, stream>>>(a); break;
        default: gemv_simt_kernel<KIND, 4><<<grid, 256, 0, stream>>>(a); break;
    }
    count_launch(EPTQ_KERNEL_GEMV_SIMT);
    return cudaPeekAtLastError() == cudaSuccess ? EPTQ_OK : EPTQ_ERR_LAUNCH;
}

}  // namespace

int simt_batch_tile(int B) { return (B >= 4) ? 4 : (B >= 2 ? 2 : 1); }

// Column splits for a layer: enough blocks to cover the 148 SMs a few times
// over, at least two 256-column sweeps per warp, at most kMaxSplits.
int simt_plan_splits(int M, int N, int B, int* cols_per_split) {
    const int bt = simt_batch_tile(B);
    const int row_blocks = (M + kRowsPerCta - 1) / kRowsPerCta;
    const int batch_blocks = (B + bt - 1) / bt;
    const int target_blocks = 148 * 6;
    long long denom = static_cast<long long>(row_blocks) * batch_blocks;
    int splits = static_cast<int>((target_blocks + denom - 1) / denom);
    const int max_by_cols = (N + 511) / 512;
    if (splits > max_by_cols) splits = max_by_cols;
    if (splits > kMaxSplits) splits = kMaxSplits;
    if (splits < 1 || denom >= kMaxCounters) splits = 1;
    int cols = (N + splits - 1) / splits;
    cols = (cols + 7) & ~7;
    splits = (N + cols - 1) / cols;
    if (cols_per_split) *cols_per_split = cols;
    return splits;
}

// Launches the SIMT GEMV.  `workspace` may be null when the plan uses one split.
int launch_gemv_simt(const EptqLayer& L, const uint16_t* x, uint16_t* y, int B,
                     void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    GemvArgs a;
    a.Q = L.Q;
    a.table16 = reinterpret_cast<const __half*>(L.table16);
    a.g = reinterpret_cast<const __half*>(L.g);
    a.h = reinterpret_cast<const __half*>(L.h);
    a.x = reinterpret_cast<const __half*>(x);
    a.O_vals = reinterpret_cast<const __half*>(L.O_vals);
    a.O_col = L.O_col;
    a.O_row_ptr = L.O_row_ptr;
    a.bias = reinterpret_cast<const __half*>(L.bias);
    a.S_group = reinterpret_cast<const __half*>(L.S_group);
    a.y = reinterpret_cast<__half*>(y);
    a.M = L.M; a.N = L.N; a.B = B;
    a.qb_rows = (L.S_group != nullptr) ? L.qb_size / 8 : 0;

    const int bt = simt_batch_tile(B);
    const int row_blocks = (L.M + kRowsPerCta - 1) / kRowsPerCta;
    const int batch_blocks = (B + bt - 1) / bt;
    int cols = 0;
    const int splits = simt_plan_splits(L.M, L.N, B, &cols);
    a.splits = splits;
    a.cols_per_split = cols;
    a.partial = nullptr;
    a.counters = nullptr;
    if (splits > 1) {
        const size_t need = kPartialOffset + static_cast<size_t>(splits) * B * 8u * L.M * sizeof(float);
        if (workspace == nullptr || workspace_bytes < need) return EPTQ_ERR_WORKSPACE;
        a.counters = reinterpret_cast<unsigned*>(workspace);
        a.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + kPartialOffset);
    }
    dim3 grid(row_blocks, splits, batch_blocks);
    if (L.quantizer == EPTQ_E8) return launch_simt_kind<EPTQ_E8>(a, bt, grid, stream);
    return launch_simt_kind<EPTQ_E8D4>(a, bt, grid, stream);
}

}  // namespace eptq
