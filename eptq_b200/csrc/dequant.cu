// Reconstruction of the fp16 weight from the quantized layer, bit-for-bit the
// arithmetic of the reference's `dequantize_layer` (algorithms/eptq.py:406-471):
//   v = table32[index]            (fp32; E8-D4: two 4-vectors of one class)
//   v = v * S_group[row/qb, col]  (only when group scales exist, and never on a
//                                  critical block)                 eptq.py:440-449
//   v = O_vals[rank]              (critical block)                  eptq.py:461-466
//   v = (v * g[row]) * h[col]     (two fp32 multiplies, left to right) eptq.py:469
//   W = fp16(v)                   (round to nearest even)           eptq.py:471
//
// HBM-bound: 2 B of Q in, 16 B of W out per index.  One thread owns 8
// consecutive columns of one Q row, so its 8 output rows are each written as
// one 128-bit store.

#include "common.cuh"

namespace eptq {

namespace {

// Rank of column `n` among the markers of row m (markers are sorted by column).
__device__ __forceinline__ int marker_rank(const int* __restrict__ O_col, int lo, int hi, int n) {
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (__ldg(O_col + mid) < n) lo = mid + 1; else hi = mid;
    }
    return lo;
}

template <int KIND>
__global__ void __launch_bounds__(256) dequant_kernel(EptqLayer L, __half* __restrict__ W, int chunks_per_row) {
    const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int m = static_cast<int>(gid / chunks_per_row);
    if (m >= L.M) return;
    const int n0 = static_cast<int>(gid % chunks_per_row) * 8;
    const int N = L.N;
    const int16_t* qrow = L.Q + static_cast<size_t>(m) * N;
    const __half* g = reinterpret_cast<const __half*>(L.g);
    const __half* h = reinterpret_cast<const __half*>(L.h);
    const __half* O = reinterpret_cast<const __half*>(L.O_vals);
    const __half* S = reinterpret_cast<const __half*>(L.S_group);

    float gk[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) gk[k] = __half2float(__ldg(g + 8 * m + k));

    __half out[8][8];   // [k][e]
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const int n = n0 + e;
        float v[8];
        if (n < N) {
            const unsigned idx = static_cast<unsigned>(static_cast<int>(qrow[n]) + 32768);
            if (idx == kMarkerIndex) {
                const int lo = __ldg(L.O_row_ptr + m), hi = __ldg(L.O_row_ptr + m + 1);
                const int r = marker_rank(L.O_col, lo, hi, n);
#pragma unroll
                for (int k = 0; k < 8; ++k) v[k] = __half2float(__ldg(O + static_cast<size_t>(r) * 8 + k));
            } else {
                if (KIND == EPTQ_E8) {
                    const float4* t = reinterpret_cast<const float4*>(L.table32 + static_cast<size_t>(idx) * 8);
                    const float4 a = __ldg(t), b = __ldg(t + 1);
                    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
                    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
                } else {
                    const unsigned ct = (idx >> 14) & 3u, ii = (idx >> 7) & 127u, jj = idx & 127u;
                    const float4 a = __ldg(reinterpret_cast<const float4*>(L.table32) + ct * 128 + ii);
                    const float4 b = __ldg(reinterpret_cast<const float4*>(L.table32) + ct * 128 + jj);
                    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
                    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
                }
                if (S != nullptr) {
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const int grp = (8 * m + k) / L.qb_size;
                        v[k] = __fmul_rn(v[k], __half2float(__ldg(S + static_cast<size_t>(grp) * N + n)));
                    }
                }
            }
            const float hn = __half2float(__ldg(h + n));
#pragma unroll
            for (int k = 0; k < 8; ++k) out[k][e] = __float2half_rn(__fmul_rn(__fmul_rn(v[k], gk[k]), hn));
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) out[k][e] = __float2half_rn(0.f);
        }
    }

    const bool full = (n0 + 8 <= N) && ((N & 7) == 0);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        __half* dst = W + static_cast<size_t>(8 * m + k) * N + n0;
        if (full) {
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(&out[k][0]);
        } else {
            for (int e = 0; e < 8 && n0 + e < N; ++e) dst[e] = out[k][e];
        }
    }
}

}  // namespace

int launch_dequant(const EptqLayer& L, uint16_t* W, cudaStream_t stream) {
    const int chunks = (L.N + 7) / 8;
    const long long total = static_cast<long long>(L.M) * chunks;
    const int block = 256;
    const long long grid = (total + block - 1) / block;
    if (grid > 0x7fffffffLL) return EPTQ_ERR_SHAPE;
    __half* Wh = reinterpret_cast<__half*>(W);
    if (L.quantizer == EPTQ_E8) {
        dequant_kernel<EPTQ_E8><<<static_cast<unsigned>(grid), block, 0, stream>>>(L, Wh, chunks);
    } else {
        dequant_kernel<EPTQ_E8D4><<<static_cast<unsigned>(grid), block, 0, stream>>>(L, Wh, chunks);
    }
    count_launch(EPTQ_KERNEL_OTHER);
    return cudaPeekAtLastError() == cudaSuccess ? EPTQ_OK : EPTQ_ERR_LAUNCH;
}

}  // namespace eptq
