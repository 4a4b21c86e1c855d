// E8-D4 decode GEMV on the tensor cores (batch 1..4), for sm_100a.
//
// Why tensor cores for a matrix-vector product: at HBM speed an SM has to
// consume about 11 indices per clock, and eight fp32 FMAs per index do not fit
// in that instruction budget.  Here each 8-byte half-codeword (4 fp16) read
// from shared memory is used, unmodified, as an A-fragment register pair of
// mma.sync.m16n8k16 (f16 x f16 -> f32).  With g = lane/4, t = lane%4:
//
//   MMA row   (g, s)      Q row g of the tile, dims 2s,2s+1 of the half-codeword (s = 0,1 <-> rows g, g+8)
//   MMA K     (n_l, dd)   column slot n_l = 0..7 of the strip, dim 2s+dd;  K = 2*(n_l%4) + dd + 8*(n_l/4)
//   MMA col   (b, p, dd') batch row b = 0,1, activation piece p = 0,1, dim 2s+dd'
//
//   A[(g,s), (n_l,dd)] = code[Q[g, n_l]][2s+dd]          registers a0,a1 = one 8-byte table read (n_l = t),
//                                                         a2,a3 = another (n_l = t+4)
//   B[(n_l,dd), (b,p,dd')] = piece_p(h*x_b)[n_l] * [dd == dd']
//   D[(g,s), (b,p,dd')] += sum_{n_l} code[..][2s+dd'] * piece_p(h*x_b)[n_l]
//
// The activations keep fp32-like precision: s*h*x (s a power of two per column
// block and batch row) is split into an fp16 high part and an fp16 remainder,
// the two pieces, which are added again in fp32.  Half of each MMA multiplies
// the zeros of [dd == dd']; the tensor pipe has that much to spare, and a second
// batch row rides along for free.  (FP8 mma.sync would halve the shared-memory
// bytes per index, but on sm_100a it is expanded into conversions plus two fp16
// MMAs and runs slower.)
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
// of 16 warps = WR row tiles (16 Q rows each) x WC column slices (64 columns
// each); it builds table and activation pieces once and walks down its row
// blocks with a rolling 2-strip register prefetch of Q.  The kernel is bound by
// instruction latency, not by any pipe, so it is built for occupancy: 64
// registers per thread, two blocks (32 warps) per SM.  Partial sums of the
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
#include <atomic>

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
    float* partial;             // [row tile][col_blocks + 1][batch][128]
    unsigned* counters;         // [row tile]
    int M, N, B;
    int row_tiles;              // ceil(M / 16)
    int row_blocks;             // ceil(row_tiles / WR)
    int col_blocks;             // grid.x
    int main_groups;            // blockIdx.y < main_groups: GEMV blocks, else correction blocks
    int n_marked;               // number of critical blocks, -1 if the caller did not say
};

namespace {

constexpr int kTableBytes = 512 * 16 * 8;         // table replicated for the 16 lanes of a half-warp
constexpr int kMaxBatch = 4;
constexpr int kWarps = 16;                        // warps per block
constexpr int kThreads = kWarps * 32;
constexpr int kSliceCols = 64;                    // columns per warp slice (2 strips of 32)
constexpr int kRedBytes = 2 * kWarps * 2 * 128 * 4;   // double-buffered cross-warp reduction, 2 batch rows per pass
__host__ __device__ constexpr int pieces_bytes(int nbp) { return 2 * nbp * 1024 * 4; }       // [batch][up to 16 slices x 64 columns]
__host__ __device__ constexpr int smem_bytes(int nbp) { return kTableBytes + pieces_bytes(nbp) + kRedBytes + 256; }

__device__ __forceinline__ unsigned prmt(unsigned a, unsigned b, unsigned sel) {
    unsigned d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint2& a01, const uint2& a23, unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a01.x), "r"(a01.y), "r"(a23.x), "r"(a23.y), "r"(b0), "r"(b1));
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
// up to 4 entries per lane per pass) for batch rows [0, B).  Everything that is
// part of the weights (row pointers, columns, O, h) is loaded before `wait_dep`
// is called, only x after.  acc[b][k]: row (lane>>3), output dim k, valid in lanes with lane%8 == 0.
template <typename WaitFn>
__device__ __forceinline__ void correction_rows(const MmaGemvArgs& p, int row0, int lane,
                                                float (&acc)[kMaxBatch][8], WaitFn wait_dep) {
    const int row = row0 + (lane >> 3);
    const int sub = lane & 7;
#pragma unroll
    for (int b = 0; b < kMaxBatch; ++b)
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[b][k] = 0.f;
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
        float hv[4];
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
        for (int j = 0; j < 4; ++j) {
            float o8[8];
            unpack8(ov[j], o8);
#pragma unroll
            for (int k = 0; k < 8; ++k) o8[k] -= cstar[k & 3];
#pragma unroll
            for (int b = 0; b < kMaxBatch; ++b) {
                if (b < p.B) {
                    const float xv = (col[j] >= 0) ? hv[j] * __half2float(__ldg(p.x + static_cast<size_t>(b) * p.N + col[j])) : 0.f;
#pragma unroll
                    for (int k = 0; k < 8; ++k) acc[b][k] = fmaf(o8[k], xv, acc[b][k]);
                }
            }
        }
    }
#pragma unroll
    for (int b = 0; b < kMaxBatch; ++b) {
        if (b < p.B) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                acc[b][k] += __shfl_xor_sync(0xffffffffu, acc[b][k], 1);
                acc[b][k] += __shfl_xor_sync(0xffffffffu, acc[b][k], 2);
                acc[b][k] += __shfl_xor_sync(0xffffffffu, acc[b][k], 4);
            }
        }
    }
}

// Scale and bias of the 4 outputs this lane writes if its warp turns out to be the
// finaliser of row tile `rt` (row rt*16 + lane/2, dims 4*(lane&1)..+3).  Loaded
// early so that the final step does not wait on DRAM.
struct OutputAffine {
    float g[4];
    float b[4];
};
__device__ __forceinline__ OutputAffine load_affine(const MmaGemvArgs& p, int rt, int lane) {
    OutputAffine a;
#pragma unroll
    for (int i = 0; i < 4; ++i) { a.g[i] = 0.f; a.b[i] = 0.f; }
    const int row = rt * 16 + (lane >> 1);
    if (row < p.M) {
        const int o = row * 8 + (lane & 1) * 4;
        const uint2 graw = __ldg(reinterpret_cast<const uint2*>(p.g + o));
        const float2 g01 = __half22float2(*reinterpret_cast<const __half2*>(&graw.x));
        const float2 g23 = __half22float2(*reinterpret_cast<const __half2*>(&graw.y));
        a.g[0] = g01.x; a.g[1] = g01.y; a.g[2] = g23.x; a.g[3] = g23.y;
        if (p.bias != nullptr) {
            const uint2 braw = __ldg(reinterpret_cast<const uint2*>(p.bias + o));
            const float2 b01 = __half22float2(*reinterpret_cast<const __half2*>(&braw.x));
            const float2 b23 = __half22float2(*reinterpret_cast<const __half2*>(&braw.y));
            a.b[0] = b01.x; a.b[1] = b01.y; a.b[2] = b23.x; a.b[3] = b23.y;
        }
    }
    return a;
}

// Publish one row tile's partial (already written to global memory by this warp)
// and, if this warp is the last arrival (col_blocks GEMV partials + 4 correction
// quarters), add all slots in slot order and write y.  One acquire-release
// atomic at GPU scope orders the partial stores before it and the reads after it.
__device__ __forceinline__ void arrive_and_finalize(const MmaGemvArgs& p, int rt, int lane, const OutputAffine& aff) {
    const int slots = p.col_blocks + 1;
    __syncwarp();
    unsigned ticket = 0;
    if (lane == 0)
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(ticket) : "l"(p.counters + rt) : "memory");
    ticket = __shfl_sync(0xffffffffu, ticket, 0);
    if (ticket != static_cast<unsigned>(p.col_blocks) + 3u) return;
    if (lane == 0) p.counters[rt] = 0u;
    const int row = rt * 16 + (lane >> 1);
    if (row >= p.M) return;
    const int o = row * 8 + (lane & 1) * 4;
    for (int b = 0; b < p.B; ++b) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        const float* base = p.partial + (static_cast<size_t>(rt) * slots * p.B + b) * 128 + lane * 4;
        for (int k = 0; k < slots; ++k) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(base + static_cast<size_t>(k) * p.B * 128));
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        const __half2 o01 = __floats2half2_rn(fmaf(s.x, aff.g[0], aff.b[0]), fmaf(s.y, aff.g[1], aff.b[1]));
        const __half2 o23 = __floats2half2_rn(fmaf(s.z, aff.g[2], aff.b[2]), fmaf(s.w, aff.g[3], aff.b[3]));
        uint2 outv;
        outv.x = *reinterpret_cast<const unsigned*>(&o01);
        outv.y = *reinterpret_cast<const unsigned*>(&o23);
        *reinterpret_cast<uint2*>(p.y + static_cast<size_t>(b) * 8 * p.M + o) = outv;
    }
}

// Ask the L2 to fetch this block's share of a small array that later loads depend on.
__device__ __forceinline__ void prefetch_share(const void* base, size_t bytes, int part, int parts) {
    if (base == nullptr || bytes == 0) return;
    size_t chunk = ((bytes + parts - 1) / parts + 15) & ~static_cast<size_t>(15);
    const size_t off = chunk * part;
    if (off >= bytes) return;
    if (off + chunk > bytes) chunk = (bytes - off) & ~static_cast<size_t>(15);
    if (chunk == 0) return;
    const char* addr = reinterpret_cast<const char*>(base) + off;
    if ((reinterpret_cast<uintptr_t>(addr) & 15u) != 0) return;
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" :: "l"(addr), "r"(static_cast<unsigned>(chunk)) : "memory");
}

// WC: column slices per block (WR = 16/WC row tiles).  NBP: batch-row pairs (batch <= 2*NBP).
template <int WC, int NBP>
__global__ void __launch_bounds__(kThreads, NBP == 1 ? 2 : 1) gemv_mma_d4_kernel(const MmaGemvArgs p) {
    constexpr int WR = kWarps / WC;
    constexpr int COLS = WC * kSliceCols;
    constexpr int kPiecesBytes = pieces_bytes(NBP);
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned* pieces = reinterpret_cast<unsigned*>(smem_raw + kTableBytes);                 // [batch][1024]
    float* red = reinterpret_cast<float*>(smem_raw + kTableBytes + kPiecesBytes);           // [2][warps][2][128]
    float* warpmax = reinterpret_cast<float*>(smem_raw + kTableBytes + kPiecesBytes + kRedBytes);   // [batch][warps]

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int slots = p.col_blocks + 1;

    // Small arrays that dependent loads will walk (CSR of the critical blocks): pull them into L2 now.
    if (threadIdx.x < 3) {
        const int part = blockIdx.y * gridDim.x + blockIdx.x, parts = gridDim.x * gridDim.y;
        const int n_marked = p.n_marked > 0 ? p.n_marked : 0;
        if (threadIdx.x == 0) prefetch_share(p.O_row_ptr, static_cast<size_t>(p.M + 1) * 4, part, parts);
        if (threadIdx.x == 1) prefetch_share(p.O_col, static_cast<size_t>(n_marked) * 4, part, parts);
        if (threadIdx.x == 2) prefetch_share(p.O_vals, static_cast<size_t>(n_marked) * 16, part, parts);
    }

    if (static_cast<int>(blockIdx.y) >= p.main_groups) {
        // ---- correction blocks: 4 Q rows per warp, striding over all quarter tiles
        asm volatile("griddepcontrol.launch_dependents;");
        const int nwarps = (gridDim.y - p.main_groups) * gridDim.x * kWarps;
        const int w0 = ((blockIdx.y - p.main_groups) * gridDim.x + blockIdx.x) * kWarps + warp;
        bool waited = false;
        for (int qt = w0; qt < p.row_tiles * 4; qt += nwarps) {
            const OutputAffine aff = load_affine(p, qt >> 2, lane);
            float acc[kMaxBatch][8];
            correction_rows(p, qt * 4, lane, acc, [&]() {
                if (!waited) { asm volatile("griddepcontrol.wait;" ::: "memory"); waited = true; }
            });
            const int rt = qt >> 2;
            if ((lane & 7) == 0) {
#pragma unroll
                for (int b = 0; b < kMaxBatch; ++b) {
                    if (b < p.B) {
                        float* dst = p.partial + ((static_cast<size_t>(rt) * slots + p.col_blocks) * p.B + b) * 128
                                   + ((qt & 3) * 4 + (lane >> 3)) * 8;
                        __stcg(reinterpret_cast<float4*>(dst), make_float4(acc[b][0], acc[b][1], acc[b][2], acc[b][3]));
                        __stcg(reinterpret_cast<float4*>(dst + 4), make_float4(acc[b][4], acc[b][5], acc[b][6], acc[b][7]));
                    }
                }
            }
            arrive_and_finalize(p, rt, lane, aff);
        }
        return;
    }

    // ---- GEMV blocks
    const int g = lane >> 2, t = lane & 3;
    const int wr = warp / WC, wc = warp % WC;
    const int N = p.N;
    const int cta_col = blockIdx.x * COLS;
    const int warp_col = cta_col + wc * kSliceCols;
    const int thread_col = warp_col + 8 * t;

    int rb = blockIdx.y;                       // row blocks of this block: by, by + groups, ...
    auto row_ptrs = [&](int rblock, const int16_t*& pa, const int16_t*& pb) {
        const int rtile = rblock * WR + wr;
        const int ra = min(rtile * 16 + g, p.M - 1), rbw = min(rtile * 16 + g + 8, p.M - 1);
        pa = p.Q + static_cast<size_t>(ra) * N + thread_col;
        pb = p.Q + static_cast<size_t>(rbw) * N + thread_col;
    };

    // 1. first Q strips (do not depend on the previous kernel)
    uint4 qa[2], qb[2];
    {
        const int16_t *pa, *pb;
        row_ptrs(rb, pa, pb);
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            if (warp_col + 32 * s < N) {
                qa[s] = ldg_stream(pa + 32 * s);
                qb[s] = ldg_stream(pb + 32 * s);
            } else {
                qa[s] = make_uint4(0, 0, 0, 0);
                qb[s] = make_uint4(0, 0, 0, 0);
            }
        }
    }

    // 2. replicated table; entry order follows the raw stored bits (true index ^ 0x100 on 9 bits).
    //    Eight consecutive threads write the eight 16-byte chunks of one entry.
    {
        const int chunk = threadIdx.x & 7;
        for (int e = threadIdx.x >> 3; e < 512; e += kThreads / 8) {
            const uint2 v = __ldg(p.table16 + (e ^ 0x100));
            *reinterpret_cast<uint4*>(smem_raw + e * 128 + chunk * 16) = make_uint4(v.x, v.y, v.x, v.y);
        }
    }
    // h of this column block is part of the weights as well
    constexpr int CPT = (COLS + kThreads - 1) / kThreads;
    float hcol[CPT];
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
        const int c = threadIdx.x + kThreads * i;
        hcol[i] = (c < COLS && cta_col + c < N) ? __half2float(__ldg(p.h + cta_col + c)) : 0.f;
    }

    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // 3. activations of this column block: h*x, block maximum, power-of-two scale, fp16 hi/lo pieces
    float inv_scale[2 * NBP];
    {
        float xh[2 * NBP][CPT];
        float mx[2 * NBP];
#pragma unroll
        for (int b = 0; b < 2 * NBP; ++b) {
            mx[b] = 0.f;
#pragma unroll
            for (int i = 0; i < CPT; ++i) {
                const int c = threadIdx.x + kThreads * i;
                const int col = cta_col + c;
                xh[b][i] = (b < p.B && c < COLS && col < N)
                               ? __half2float(__ldg(p.x + static_cast<size_t>(b) * N + col)) * hcol[i] : 0.f;
                mx[b] = fmaxf(mx[b], fabsf(xh[b][i]));
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) mx[b] = fmaxf(mx[b], __shfl_xor_sync(0xffffffffu, mx[b], off));
            if (lane == 0) warpmax[b * kWarps + warp] = mx[b];
        }
        __syncthreads();
#pragma unroll
        for (int b = 0; b < 2 * NBP; ++b) {
#pragma unroll
            for (int w = 0; w < kWarps; ++w) mx[b] = fmaxf(mx[b], warpmax[b * kWarps + w]);
            // scale = 2^(13 - exponent(mx)): mx * scale in [2^13, 2^14), well inside the fp16 range
            int ex = static_cast<int>((__float_as_uint(mx[b]) >> 23) & 0xffu) - 127;
            if (mx[b] == 0.f || ex > 100) ex = 13;
            if (ex < -100) ex = -100;
            const float scale = __uint_as_float(static_cast<unsigned>(127 + 13 - ex) << 23);
            inv_scale[b] = __uint_as_float(static_cast<unsigned>(127 - 13 + ex) << 23);
#pragma unroll
            for (int i = 0; i < CPT; ++i) {
                const int c = threadIdx.x + kThreads * i;
                if (c < COLS) pieces[b * 1024 + c] = split_pieces(xh[b][i] * scale);
            }
        }
        __syncthreads();
    }

    // 4. main loop
    const unsigned lane8 = 8u * (lane & 15);
    const unsigned char* tab_bytes = smem_raw;
    // B column g = (batch g>>2, piece (g>>1)&1, dd' = g&1): the piece goes to the low or high half
    // of the B register, the other half stays zero.
    const unsigned pb = 2u * ((g >> 1) & 1);
    const unsigned sel = (g & 1) ? ((((pb + 1) << 12) | (pb << 8)) | 0x0044u) : (0x4400u | ((pb + 1) << 4) | pb);
    const unsigned* my_pieces = pieces + (g >> 2) * 1024 + wc * kSliceCols + 8 * t;     // + bp*2048 for the next batch pair
    float own_scale[NBP];
#pragma unroll
    for (int bp = 0; bp < NBP; ++bp) own_scale[bp] = (t >> 1) ? inv_scale[2 * bp + 1] : inv_scale[2 * bp];
    int buf = 0;

    for (; rb < p.row_blocks; rb += p.main_groups) {
        const int rt = rb * WR + wr;
        const OutputAffine aff = load_affine(p, rt, lane);
        const int rb_next = rb + p.main_groups;
        const bool has_next = rb_next < p.row_blocks;
        const int16_t *na = nullptr, *nb = nullptr;
        if (has_next) row_ptrs(rb_next, na, nb);

        float acc[NBP][2][2][4];              // [batch pair][row group g / g+8][half i / j][dims]
#pragma unroll
        for (int a = 0; a < NBP; ++a)
#pragma unroll
            for (int b = 0; b < 2; ++b)
#pragma unroll
                for (int c = 0; c < 2; ++c)
#pragma unroll
                    for (int d = 0; d < 4; ++d) acc[a][b][c][d] = 0.f;

#pragma unroll
        for (int s = 0; s < 2; ++s) {
            if (warp_col + 32 * s < N) {                      // warp-uniform
                const uint4 ca = qa[s], cb = qb[s];
                if (has_next) {                               // rolling prefetch: refill the slot just consumed
                    qa[s] = ldg_stream(na + 32 * s);
                    qb[s] = ldg_stream(nb + 32 * s);
                }
                unsigned wv[NBP][8];
#pragma unroll
                for (int bp = 0; bp < NBP; ++bp) {
                    const uint4 w0 = *reinterpret_cast<const uint4*>(my_pieces + bp * 2048 + 32 * s);
                    const uint4 w1 = *reinterpret_cast<const uint4*>(my_pieces + bp * 2048 + 32 * s + 4);
                    wv[bp][0] = w0.x; wv[bp][1] = w0.y; wv[bp][2] = w0.z; wv[bp][3] = w0.w;
                    wv[bp][4] = w1.x; wv[bp][5] = w1.y; wv[bp][6] = w1.z; wv[bp][7] = w1.w;
                }
                const unsigned qav[4] = {ca.x, ca.y, ca.z, ca.w};
                const unsigned qbv[4] = {cb.x, cb.y, cb.z, cb.w};
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    // this thread's columns 8t+2m (slot n_l = t) and 8t+2m+1 (slot n_l = t+4)
                    unsigned oi0, oj0, oi1, oj1;
                    code_offsets(qav[m], lane8, oi0, oj0);
                    code_offsets(qav[m] >> 16, lane8, oi1, oj1);
                    const uint2 ai0 = table_read(tab_bytes, oi0), aj0 = table_read(tab_bytes, oj0);
                    const uint2 ai1 = table_read(tab_bytes, oi1), aj1 = table_read(tab_bytes, oj1);
                    code_offsets(qbv[m], lane8, oi0, oj0);
                    code_offsets(qbv[m] >> 16, lane8, oi1, oj1);
                    const uint2 bi0 = table_read(tab_bytes, oi0), bj0 = table_read(tab_bytes, oj0);
                    const uint2 bi1 = table_read(tab_bytes, oi1), bj1 = table_read(tab_bytes, oj1);
#pragma unroll
                    for (int bp = 0; bp < NBP; ++bp) {
                        const unsigned b0 = prmt(wv[bp][2 * m], 0u, sel), b1 = prmt(wv[bp][2 * m + 1], 0u, sel);
                        mma_f16(acc[bp][0][0], ai0, ai1, b0, b1);
                        mma_f16(acc[bp][0][1], aj0, aj1, b0, b1);
                        mma_f16(acc[bp][1][0], bi0, bi1, b0, b1);
                        mma_f16(acc[bp][1][1], bj0, bj1, b0, b1);
                    }
                }
            }
        }

        // 5. add the two pieces (partner lane t^1) and hand the row tile's sums over.
        //    After the shuffle lanes with even t hold, for batch row (t>>1) of each pair and rows g, g+8,
        //    the 8 output dims: acc[..][rg][0][0..3] = dims 0..3, acc[..][rg][1][0..3] = dims 4..7.
#pragma unroll
        for (int bp = 0; bp < NBP; ++bp) {
            float tot[2][2][4];
#pragma unroll
            for (int rg = 0; rg < 2; ++rg)
#pragma unroll
                for (int hf = 0; hf < 2; ++hf)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float own = acc[bp][rg][hf][c] * own_scale[bp];
                        tot[rg][hf][c] = own + __shfl_xor_sync(0xffffffffu, own, 1);
                    }
            const int b = 2 * bp + (t >> 1);
            if (WC == 1) {
                if ((t & 1) == 0 && rt < p.row_tiles && b < p.B) {
                    float* dst = p.partial + ((static_cast<size_t>(rt) * slots + blockIdx.x) * p.B + b) * 128;
#pragma unroll
                    for (int rg = 0; rg < 2; ++rg)
#pragma unroll
                        for (int hf = 0; hf < 2; ++hf)
                            __stcg(reinterpret_cast<float4*>(dst + (g + 8 * rg) * 8 + hf * 4),
                                   make_float4(tot[rg][hf][0], tot[rg][hf][1], tot[rg][hf][2], tot[rg][hf][3]));
                }
            } else {
                float* rbuf = red + ((buf * kWarps + warp) * 2 + (t >> 1)) * 128;
                if ((t & 1) == 0) {
#pragma unroll
                    for (int rg = 0; rg < 2; ++rg)
#pragma unroll
                        for (int hf = 0; hf < 2; ++hf)
                            *reinterpret_cast<float4*>(rbuf + (g + 8 * rg) * 8 + hf * 4) =
                                make_float4(tot[rg][hf][0], tot[rg][hf][1], tot[rg][hf][2], tot[rg][hf][3]);
                }
                __syncthreads();
                if (wc == 0 && rt < p.row_tiles) {
#pragma unroll
                    for (int bb = 0; bb < 2; ++bb) {
                        if (2 * bp + bb < p.B) {
                            float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                            for (int k = 0; k < WC; ++k) {
                                const float4 v = *reinterpret_cast<const float4*>(
                                    red + ((buf * kWarps + wr * WC + k) * 2 + bb) * 128 + lane * 4);
                                s4.x += v.x; s4.y += v.y; s4.z += v.z; s4.w += v.w;
                            }
                            float* dst = p.partial + ((static_cast<size_t>(rt) * slots + blockIdx.x) * p.B + 2 * bp + bb) * 128 + lane * 4;
                            __stcg(reinterpret_cast<float4*>(dst), s4);
                        }
                    }
                }
                buf ^= 1;
            }
        }
        if ((WC == 1 || wc == 0) && rt < p.row_tiles) arrive_and_finalize(p, rt, lane, aff);
    }
}

template <int WC, int NBP>
int launch_variant(const MmaGemvArgs& a, dim3 grid, cudaStream_t stream) {
    static std::atomic<bool> attr_done[16];       // setting the attribute twice is harmless; the flag itself must not race
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return EPTQ_ERR_LAUNCH;
    if (dev < 0 || dev >= 16) return EPTQ_ERR_UNSUPPORTED;
    if (!attr_done[dev]) {
        if (cudaFuncSetAttribute(gemv_mma_d4_kernel<WC, NBP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 smem_bytes(NBP)) != cudaSuccess)
            return EPTQ_ERR_LAUNCH;
        attr_done[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes(NBP);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, gemv_mma_d4_kernel<WC, NBP>, a);
    count_launch(EPTQ_KERNEL_GEMV_MMA);
    return err == cudaSuccess ? EPTQ_OK : EPTQ_ERR_LAUNCH;
}

template <int NBP>
int launch_wc(int wc, const MmaGemvArgs& a, dim3 grid, cudaStream_t stream) {
    switch (wc) {
        case 1: return launch_variant<1, NBP>(a, grid, stream);
        case 2: return launch_variant<2, NBP>(a, grid, stream);
        case 4: return launch_variant<4, NBP>(a, grid, stream);
        case 8: return launch_variant<8, NBP>(a, grid, stream);
        default: return launch_variant<16, NBP>(a, grid, stream);
    }
}

}  // namespace

// Column slices per block: aim at no more than ~16 column blocks (partials to add
// at the end) and about two blocks per SM.
int mma_plan(int M, int N, int* wc_out, int* col_blocks, int* groups, int* corr_groups) {
    const int row_tiles = (M + 15) / 16;
    int wc = 1;
    while (wc < kWarps && (N + wc * kSliceCols - 1) / (wc * kSliceCols) > 16) wc *= 2;
    const int cb = (N + wc * kSliceCols - 1) / (wc * kSliceCols);
    const int wr = kWarps / wc;
    const int row_blocks = (row_tiles + wr - 1) / wr;
    int gy = (2 * 148) / cb;
    if (gy < 1) gy = 1;
    if (gy > row_blocks) gy = row_blocks;
    int cg = (row_tiles * 4 + cb * kWarps - 1) / (cb * kWarps);
    if (cg < 1) cg = 1;
    *wc_out = wc; *col_blocks = cb; *groups = gy; *corr_groups = cg;
    return row_tiles;
}

size_t mma_workspace_bytes(int M, int N, int B) {
    int wc, cb, gy, cg;
    const int row_tiles = mma_plan(M, N, &wc, &cb, &gy, &cg);
    if (row_tiles >= kMaxCounters) return 0;
    return kPartialOffset + static_cast<size_t>(row_tiles) * (cb + 1) * B * 128 * sizeof(float);
}

bool mma_gemv_supported(const EptqLayer& L, int B) {
    return L.quantizer == EPTQ_E8D4 && L.table16 != nullptr && L.S_group == nullptr && B >= 1 && B <= kMaxBatch &&
           (L.N % 32) == 0 && (L.M + 15) / 16 < kMaxCounters && aligned16(L.Q) && aligned16(L.table16);
}

int launch_gemv_mma(const EptqLayer& L, const uint16_t* x, uint16_t* y, int B,
                    void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    int wc, cb, gy, cg;
    const int row_tiles = mma_plan(L.M, L.N, &wc, &cb, &gy, &cg);
    const size_t need = mma_workspace_bytes(L.M, L.N, B);
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
    a.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + kPartialOffset);
    a.M = L.M; a.N = L.N; a.B = B;
    a.row_tiles = row_tiles;
    a.row_blocks = (row_tiles + (kWarps / wc) - 1) / (kWarps / wc);
    a.col_blocks = cb;
    a.main_groups = gy;
    a.n_marked = L.n_masked;
    const dim3 grid(cb, gy + cg);
    return (B <= 2) ? launch_wc<1>(wc, a, grid, stream) : launch_wc<2>(wc, a, grid, stream);
}

}  // namespace eptq
