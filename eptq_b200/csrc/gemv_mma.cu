// E8-D4 decode GEMV on the tensor cores (batch 1), for sm_100a.
//
// Why tensor cores for a matrix-vector product: at HBM speed an SM has to
// consume about 11 indices per clock, and eight fp32 FMAs per index do not fit
// in that instruction budget.  Here each 8-byte half-codeword (4 fp16) read
// from shared memory is used, unmodified, as two A-fragment registers of
// mma.sync.m16n8k16 (f16 x f16 -> f32):
//
//   A[row = Q row, K = (column slot n_l, dim d)] = code[Q[row, n_l]][d]            (16 x 16)
//   B[K = (n_l, d), col = (piece p, dim d')]     = piece_p(h*x)[n_l] * [d == d']   (16 x 8)
//   D[row, (p, d')] += sum_{n_l} code[..][d'] * piece_p(h*x)[n_l]
//
// The activations keep fp32-like precision: s*h*x (s a power of two per column
// block) is split into an fp16 high part and an fp16 remainder, which are the
// two "pieces" p and are added again in fp32.  Three quarters of each MMA
// multiply the zeros of [d == d']; the tensor pipe has that much to spare.
// (FP8 mma.sync would halve the shared-memory bytes per index, but on sm_100a
// it is expanded into conversions plus two fp16 MMAs and runs slower.)
//
// Shared-memory reads are bank-conflict free because the 4 KB fp16 table is
// stored 16 times, once per lane of a half-warp (byte address = entry*128 +
// (lane%16)*8): 64 KB per block.
//
// Critical blocks: the marker index 65535 decodes to the ordinary table entry
// (3,127,127), so the main loop needs no test; dedicated warps add
// sum (O[i] - code[65535]) * h*x over the CSR of each row as one more partial.
//
// Work split: grid = (column blocks, row groups [+ correction blocks]).  A block
// of 8 warps = WR row tiles (16 Q rows each) x WC column slices (128 columns
// each); it builds table and activation pieces once and walks down its row
// blocks with a rolling 4-strip register prefetch of Q.  Partial sums of the
// column blocks meet in the caller's scratch; the last arrival per row tile adds
// them in slot order, applies g and bias and writes fp16.
//
// Programmatic dependent launch: everything that does not depend on x (table
// build, first Q loads, the static part of the corrections) runs before
// griddepcontrol.wait, so it overlaps the tail of the previous kernel in the
// stream when the launch allows it.
//
// Reference counterpart: e8d4_fused_kernel_t (csrc/eptq_kernels.cu:161-292).

#include "common.cuh"

namespace eptq {

struct MmaGemvArgs {
    const int16_t* Q;
    const uint2* table16;       // 512 entries, 4 fp16 each
    const __half* g;
    const __half* h;
    const __half* x;
    const __half* O_vals;
    const int* O_col;
    const int* O_row_ptr;
    const __half* bias;
    __half* y;
    float* partial;             // [row tile][col_blocks + 1][128]
    unsigned* counters;         // [row tile]
    int M, N;
    int row_tiles;              // ceil(M / 16)
    int row_blocks;             // ceil(row_tiles / WR)
    int col_blocks;             // grid.x
    int main_groups;            // blockIdx.y < main_groups: GEMV blocks, else correction blocks
};

namespace {

constexpr int kTableBytes = 512 * 16 * 8;         // table replicated for the 16 lanes of a half-warp
constexpr int kPiecesBytes = 1024 * 4;            // up to 8 slices x 128 columns
constexpr int kRedBytes = 2 * 8 * 128 * 4;        // double-buffered cross-warp reduction
constexpr int kSmemBytes = kTableBytes + kPiecesBytes + kRedBytes + 64;

__device__ __forceinline__ unsigned prmt(unsigned a, unsigned b, unsigned sel) {
    unsigned d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ void mma_f16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                        unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// v as fp16 high part (low 16 bits) and fp16 remainder (high 16 bits).
__device__ __forceinline__ unsigned split_pieces(float v) {
    const __half hi = __float2half_rn(v);
    const __half lo = __float2half_rn(v - __half2float(hi));
    return static_cast<unsigned>(__half_as_ushort(hi)) | (static_cast<unsigned>(__half_as_ushort(lo)) << 16);
}

// Byte offsets into the table of the two half-codewords of the index in the low
// 16 bits of `q` (raw stored bits; the table is laid out for them, so the +32768
// of the format costs nothing).  `lane8` = 8*(lane%16) occupies bits 3..6.
__device__ __forceinline__ void code_offsets(unsigned q, unsigned lane8, unsigned& oi, unsigned& oj) {
    oi = (q & 0xFF80u) | lane8;                                   // (class, i) * 128 B
    oj = ((q << 7) & 0x3F80u) | ((q & 0xC000u) | lane8);          // (class, j) * 128 B
}
__device__ __forceinline__ uint2 table_read(const unsigned char* tab, unsigned off) {
    return *reinterpret_cast<const uint2*>(tab + off);
}

// Critical-block correction of 4 consecutive Q rows by one warp (8 lanes per row,
// up to 4 entries per lane per pass).  Everything that is part of the weights
// (row pointers, columns, O, h) is loaded before `wait_dep` is called, only x after.
template <typename WaitFn>
__device__ __forceinline__ void correction_rows(const MmaGemvArgs& p, int row0, int lane, float (&acc)[8],
                                                WaitFn wait_dep) {
    const int row = row0 + (lane >> 3);
    const int sub = lane & 7;
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    const uint2 craw = __ldg(p.table16 + 511);          // what the main loop added for a marker: entry (3,127), both halves
    const float2 c01 = __half22float2(*reinterpret_cast<const __half2*>(&craw.x));
    const float2 c23 = __half22float2(*reinterpret_cast<const __half2*>(&craw.y));
    const float cstar[4] = {c01.x, c01.y, c23.x, c23.y};
    int lo = 0, hi = 0;
    if (row < p.M) {
        lo = __ldg(p.O_row_ptr + row);
        hi = __ldg(p.O_row_ptr + row + 1);
    }
    bool waited = false;
    for (int i = lo + sub; __any_sync(0xffffffffu, i < hi) || !waited; i += 32) {
        int col[4];
        float hv[4], xv[4];
        uint4 ov[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) col[j] = (i + 8 * j < hi) ? __ldg(p.O_col + i + 8 * j) : -1;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (col[j] >= 0) {
                hv[j] = __half2float(__ldg(p.h + col[j]));
                ov[j] = ldg128(p.O_vals + static_cast<size_t>(i + 8 * j) * 8);
            } else {
                hv[j] = 0.f;
                ov[j] = make_uint4(0, 0, 0, 0);
            }
        }
        if (!waited) { wait_dep(); waited = true; }
#pragma unroll
        for (int j = 0; j < 4; ++j) xv[j] = (col[j] >= 0) ? hv[j] * __half2float(__ldg(p.x + col[j])) : 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float o8[8];
            unpack8(ov[j], o8);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] = fmaf(o8[k] - cstar[k & 3], xv[j], acc[k]);
        }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], 1);
        acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], 2);
        acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], 4);
    }
}

// Publish one row tile's partial (already in global memory) and, if this warp is
// the last of `expected` arrivals, reduce all slots and write y.
__device__ __forceinline__ void arrive_and_finalize(const MmaGemvArgs& p, int rt, int lane) {
    const int slots = p.col_blocks + 1;
    __threadfence();
    __syncwarp();
    unsigned ticket = 0;
    if (lane == 0) ticket = atomicAdd(p.counters + rt, 1u);
    ticket = __shfl_sync(0xffffffffu, ticket, 0);
    if (ticket != static_cast<unsigned>(p.col_blocks) + 3u) return;     // col_blocks GEMV + 4 correction arrivals
    __threadfence();
    if (lane == 0) p.counters[rt] = 0u;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    const float* base = p.partial + static_cast<size_t>(rt) * slots * 128 + lane * 4;
    for (int k = 0; k < slots; ++k) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(base + static_cast<size_t>(k) * 128));
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    const int row = rt * 16 + (lane >> 1);
    if (row < p.M) {
        const int o = row * 8 + (lane & 1) * 4;
        const uint2 graw = __ldg(reinterpret_cast<const uint2*>(p.g + o));
        const __half2* g2 = reinterpret_cast<const __half2*>(&graw);
        float2 g01 = __half22float2(g2[0]), g23 = __half22float2(g2[1]);
        float b0 = 0.f, b1 = 0.f, b2 = 0.f, b3 = 0.f;
        if (p.bias != nullptr) {
            const uint2 braw = __ldg(reinterpret_cast<const uint2*>(p.bias + o));
            const __half2* bb = reinterpret_cast<const __half2*>(&braw);
            float2 b01 = __half22float2(bb[0]), b23 = __half22float2(bb[1]);
            b0 = b01.x; b1 = b01.y; b2 = b23.x; b3 = b23.y;
        }
        __half2 o01 = __floats2half2_rn(fmaf(s.x, g01.x, b0), fmaf(s.y, g01.y, b1));
        __half2 o23 = __floats2half2_rn(fmaf(s.z, g23.x, b2), fmaf(s.w, g23.y, b3));
        uint2 outv;
        outv.x = *reinterpret_cast<unsigned*>(&o01);
        outv.y = *reinterpret_cast<unsigned*>(&o23);
        *reinterpret_cast<uint2*>(p.y + o) = outv;
    }
}

template <int WC>
__global__ void __launch_bounds__(256, 2) gemv_mma_d4_kernel(const MmaGemvArgs p) {
    constexpr int WR = 8 / WC;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned* tab = reinterpret_cast<unsigned*>(smem_raw);
    unsigned* pieces = reinterpret_cast<unsigned*>(smem_raw + kTableBytes);
    float* red = reinterpret_cast<float*>(smem_raw + kTableBytes + kPiecesBytes);
    float* warpmax = reinterpret_cast<float*>(smem_raw + kTableBytes + kPiecesBytes + kRedBytes);

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int slots = p.col_blocks + 1;

    if (static_cast<int>(blockIdx.y) >= p.main_groups) {
        // ---- correction blocks: 4 Q rows per warp, striding over all quarter tiles
        asm volatile("griddepcontrol.launch_dependents;");
        const int nwarps = (gridDim.y - p.main_groups) * gridDim.x * 8;
        const int w0 = ((blockIdx.y - p.main_groups) * gridDim.x + blockIdx.x) * 8 + warp;
        bool waited = false;
        for (int qt = w0; qt < p.row_tiles * 4; qt += nwarps) {
            float acc[8];
            correction_rows(p, qt * 4, lane, acc, [&]() {
                if (!waited) { asm volatile("griddepcontrol.wait;" ::: "memory"); waited = true; }
            });
            const int rt = qt >> 2;
            if ((lane & 7) == 0) {
                float* dst = p.partial + (static_cast<size_t>(rt) * slots + p.col_blocks) * 128
                           + ((qt & 3) * 4 + (lane >> 3)) * 8;
                __stcg(reinterpret_cast<float4*>(dst), make_float4(acc[0], acc[1], acc[2], acc[3]));
                __stcg(reinterpret_cast<float4*>(dst + 4), make_float4(acc[4], acc[5], acc[6], acc[7]));
            }
            arrive_and_finalize(p, rt, lane);
        }
        return;
    }

    // ---- GEMV blocks
    const int g = lane >> 2, t = lane & 3;
    const int wr = warp / WC, wc = warp % WC;
    const int N = p.N;
    const int cta_col = blockIdx.x * (WC * 128);
    const int warp_col = cta_col + wc * 128;
    const int thread_col = warp_col + 8 * t;

    // Row block list of this block: by, by + groups, ...
    int rb = blockIdx.y;
    auto row_ptrs = [&](int rblock, const int16_t*& pa, const int16_t*& pb) {
        const int rtile = rblock * WR + wr;
        const int ra = min(rtile * 16 + g, p.M - 1), rbw = min(rtile * 16 + g + 8, p.M - 1);
        pa = p.Q + static_cast<size_t>(ra) * N + thread_col;
        pb = p.Q + static_cast<size_t>(rbw) * N + thread_col;
    };

    // 1. first Q strips (do not depend on the previous kernel)
    uint4 qa[4], qb[4];
    {
        const int16_t *pa, *pb;
        row_ptrs(rb, pa, pb);
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            if (warp_col + 32 * s < N) {
                qa[s] = ldg_stream(pa + 32 * s);
                qb[s] = ldg_stream(pb + 32 * s);
            } else {
                qa[s] = make_uint4(0, 0, 0, 0);
                qb[s] = make_uint4(0, 0, 0, 0);
            }
        }
    }

    // 2. lane-replicated table; entry order follows the raw stored bits (true index ^ 0x100 on 9 bits)
    for (int e = threadIdx.x; e < 512; e += 256) {
        const uint2 v = __ldg(p.table16 + (e ^ 0x100));
        const uint4 vv = make_uint4(v.x, v.y, v.x, v.y);
        uint4* dst = reinterpret_cast<uint4*>(tab + e * 32);
#pragma unroll
        for (int i = 0; i < 8; ++i) dst[i] = vv;
    }

    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // 3. activations of this column block: h*x, block maximum, power-of-two scale, four E4M3 pieces
    constexpr int CPT = (WC * 128 + 255) / 256;
    float xh[CPT];
    float mx = 0.f;
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
        const int c = threadIdx.x + 256 * i;
        const int col = cta_col + c;
        xh[i] = (c < WC * 128 && col < N) ? __half2float(__ldg(p.x + col)) * __half2float(__ldg(p.h + col)) : 0.f;
        mx = fmaxf(mx, fabsf(xh[i]));
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    if (lane == 0) warpmax[warp] = mx;
    __syncthreads();
#pragma unroll
    for (int w = 0; w < 8; ++w) mx = fmaxf(mx, warpmax[w]);
    // scale = 2^(13 - exponent(mx)): mx * scale in [2^13, 2^14), well inside the fp16 range
    int ex = static_cast<int>((__float_as_uint(mx) >> 23) & 0xffu) - 127;
    if (mx == 0.f || ex > 100) ex = 13;
    if (ex < -100) ex = -100;
    const float scale = __uint_as_float(static_cast<unsigned>(127 + 13 - ex) << 23);
    const float inv_scale = __uint_as_float(static_cast<unsigned>(127 - 13 + ex) << 23);
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
        const int c = threadIdx.x + 256 * i;
        if (c < WC * 128) pieces[c] = split_pieces(xh[i] * scale);
    }
    __syncthreads();

    // 4. main loop
    const unsigned lane8 = 8u * (lane & 15);
    const unsigned char* tab_bytes = smem_raw;
    // Column g of B is (piece g>>2, dim g&3).  K index of (n_l, d) is (d>>1)*8 + 2*n_l + (d&1), so this
    // thread's b0 holds dims 0,1 and b1 dims 2,3 of column slot n_l = t: exactly one half of one of
    // them is the piece, the rest is zero.
    unsigned sel0, sel1;
    {
        const unsigned pb = 2u * (g >> 2);                      // first byte of the piece inside the word
        const unsigned lo_half = 0x4400u | ((pb + 1) << 4) | pb;              // piece in bits 0..15
        const unsigned hi_half = (((pb + 1) << 12) | (pb << 8)) | 0x0044u;     // piece in bits 16..31
        const unsigned place = (g & 1) ? hi_half : lo_half;
        sel0 = (g & 2) ? 0x4444u : place;
        sel1 = (g & 2) ? place : 0x4444u;
    }
    const float own_scale = inv_scale;
    int buf = 0;

    for (; rb < p.row_blocks; rb += p.main_groups) {
        const int rt = rb * WR + wr;
        const int rb_next = rb + p.main_groups;
        const bool has_next = rb_next < p.row_blocks;
        const int16_t *na = nullptr, *nb = nullptr;
        if (has_next) row_ptrs(rb_next, na, nb);

        float acc[2][4];
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[a][c] = 0.f;

#pragma unroll
        for (int s = 0; s < 4; ++s) {
            if (warp_col + 32 * s < N) {                      // warp-uniform
                const uint4 ca = qa[s], cb = qb[s];
                if (has_next) {                               // rolling prefetch: refill the slot just consumed
                    qa[s] = ldg_stream(na + 32 * s);
                    qb[s] = ldg_stream(nb + 32 * s);
                }
                const uint4 w0 = *reinterpret_cast<const uint4*>(pieces + wc * 128 + 32 * s + 8 * t);
                const uint4 w1 = *reinterpret_cast<const uint4*>(pieces + wc * 128 + 32 * s + 8 * t + 4);
                const unsigned wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                const unsigned qav[4] = {ca.x, ca.y, ca.z, ca.w};
                const unsigned qbv[4] = {cb.x, cb.y, cb.z, cb.w};
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const unsigned qa16 = (e & 1) ? (qav[e >> 1] >> 16) : qav[e >> 1];
                    const unsigned qb16 = (e & 1) ? (qbv[e >> 1] >> 16) : qbv[e >> 1];
                    unsigned oi, oj;
                    code_offsets(qa16, lane8, oi, oj);
                    const uint2 ia = table_read(tab_bytes, oi), ja = table_read(tab_bytes, oj);
                    code_offsets(qb16, lane8, oi, oj);
                    const uint2 ib = table_read(tab_bytes, oi), jb = table_read(tab_bytes, oj);
                    const unsigned b0 = prmt(wv[e], 0u, sel0), b1 = prmt(wv[e], 0u, sel1);
                    mma_f16(acc[0], ia.x, ib.x, ia.y, ib.y, b0, b1);
                    mma_f16(acc[1], ja.x, jb.x, ja.y, jb.y, b0, b1);
                }
            }
        }

        // 5. add the two pieces: this thread holds piece (t>>1), partner t^2 the other
        float tot[2][4];
#pragma unroll
        for (int hf = 0; hf < 2; ++hf)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float own = acc[hf][c] * own_scale;
                tot[hf][c] = own + __shfl_xor_sync(0xffffffffu, own, 2);
            }
        // thread (g, t<2): rows g and g+8, dims hf*4 + 2*(t&1) + {0,1}
        if (WC == 1) {
            if (t < 2 && rt < p.row_tiles) {
                float* dst = p.partial + (static_cast<size_t>(rt) * slots + blockIdx.x) * 128;
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    __stcg(reinterpret_cast<float2*>(dst + g * 8 + hf * 4 + 2 * t), make_float2(tot[hf][0], tot[hf][1]));
                    __stcg(reinterpret_cast<float2*>(dst + (g + 8) * 8 + hf * 4 + 2 * t), make_float2(tot[hf][2], tot[hf][3]));
                }
            }
            if (rt < p.row_tiles) arrive_and_finalize(p, rt, lane);
        } else {
            float* rbuf = red + buf * (8 * 128) + warp * 128;
            if (t < 2) {
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    *reinterpret_cast<float2*>(rbuf + g * 8 + hf * 4 + 2 * t) = make_float2(tot[hf][0], tot[hf][1]);
                    *reinterpret_cast<float2*>(rbuf + (g + 8) * 8 + hf * 4 + 2 * t) = make_float2(tot[hf][2], tot[hf][3]);
                }
            }
            __syncthreads();
            if (wc == 0 && rt < p.row_tiles) {
                float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int k = 0; k < WC; ++k) {
                    const float4 v = *reinterpret_cast<const float4*>(red + buf * (8 * 128) + (wr * WC + k) * 128 + lane * 4);
                    s4.x += v.x; s4.y += v.y; s4.z += v.z; s4.w += v.w;
                }
                float* dst = p.partial + (static_cast<size_t>(rt) * slots + blockIdx.x) * 128 + lane * 4;
                __stcg(reinterpret_cast<float4*>(dst), s4);
                arrive_and_finalize(p, rt, lane);
            }
            buf ^= 1;
        }
    }
}

template <int WC>
int launch_wc(const MmaGemvArgs& a, dim3 grid, cudaStream_t stream) {
    static bool attr_done[16] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return EPTQ_ERR_LAUNCH;
    if (dev < 16 && !attr_done[dev]) {
        if (cudaFuncSetAttribute(gemv_mma_d4_kernel<WC>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
            return EPTQ_ERR_LAUNCH;
        attr_done[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, gemv_mma_d4_kernel<WC>, a);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return err == cudaSuccess ? EPTQ_OK : EPTQ_ERR_LAUNCH;
}

}  // namespace

// Column slices per block: aim at no more than ~16 column blocks (partials to add
// at the end) while keeping at least one block per SM.
int mma_plan(int M, int N, int* wc_out, int* col_blocks, int* groups, int* corr_groups) {
    const int row_tiles = (M + 15) / 16;
    int wc = 1;
    while (wc < 8 && (N + wc * 128 - 1) / (wc * 128) > 16) wc *= 2;
    const int cb = (N + wc * 128 - 1) / (wc * 128);
    const int wr = 8 / wc;
    const int row_blocks = (row_tiles + wr - 1) / wr;
    int gy = 148 / cb;
    if (gy < 1) gy = 1;
    if (gy > row_blocks) gy = row_blocks;
    int cg = (row_tiles * 4 + cb * 8 - 1) / (cb * 8);
    if (cg < 1) cg = 1;
    *wc_out = wc; *col_blocks = cb; *groups = gy; *corr_groups = cg;
    return row_tiles;
}

size_t mma_workspace_bytes(int M, int N) {
    int wc, cb, gy, cg;
    const int row_tiles = mma_plan(M, N, &wc, &cb, &gy, &cg);
    if (row_tiles > kMaxCounters) return 0;
    return kCounterBytes + static_cast<size_t>(row_tiles) * (cb + 1) * 128 * sizeof(float);
}

bool mma_gemv_supported(const EptqLayer& L, int B) {
    return L.quantizer == EPTQ_E8D4 && L.table16 != nullptr && L.S_group == nullptr && B == 1 &&
           (L.N % 32) == 0 && (L.M + 15) / 16 <= kMaxCounters && aligned16(L.Q) && aligned16(L.table16);
}

int launch_gemv_mma(const EptqLayer& L, const uint16_t* x, uint16_t* y,
                    void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    int wc, cb, gy, cg;
    const int row_tiles = mma_plan(L.M, L.N, &wc, &cb, &gy, &cg);
    const size_t need = mma_workspace_bytes(L.M, L.N);
    if (workspace == nullptr || workspace_bytes < need) return EPTQ_ERR_WORKSPACE;
    MmaGemvArgs a;
    a.Q = L.Q;
    a.table16 = reinterpret_cast<const uint2*>(L.table16);
    a.g = reinterpret_cast<const __half*>(L.g);
    a.h = reinterpret_cast<const __half*>(L.h);
    a.x = reinterpret_cast<const __half*>(x);
    a.O_vals = reinterpret_cast<const __half*>(L.O_vals);
    a.O_col = L.O_col;
    a.O_row_ptr = L.O_row_ptr;
    a.bias = reinterpret_cast<const __half*>(L.bias);
    a.y = reinterpret_cast<__half*>(y);
    a.counters = reinterpret_cast<unsigned*>(workspace);
    a.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + kCounterBytes);
    a.M = L.M; a.N = L.N;
    a.row_tiles = row_tiles;
    a.row_blocks = (row_tiles + (8 / wc) - 1) / (8 / wc);
    a.col_blocks = cb;
    a.main_groups = gy;
    const dim3 grid(cb, gy + cg);
    switch (wc) {
        case 1: return launch_wc<1>(a, grid, stream);
        case 2: return launch_wc<2>(a, grid, stream);
        case 4: return launch_wc<4>(a, grid, stream);
        default: return launch_wc<8>(a, grid, stream);
    }
}

}  // namespace eptq
