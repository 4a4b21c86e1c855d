// Persistent decode GEMV over a group of independent layers of one codebook (E8-D4 or E8), two batch rows
// per launch (larger batches run as several launches over the same weights).
//
// One launch, one block of 16 warps per SM, covers up to kMaxGroupLayers layers
// whose inputs are all ready (q/k/v, gate/up, the experts of a mixture, or a
// single layer).  At B200 speed one 4096x4096 layer is 0.7 us of HBM traffic,
// less than a kernel launch and one DRAM round trip, so per-layer launches are
// latency-bound; here table build, launch and pipeline fill are paid once per
// group and every warp streams a long contiguous run of work.
//
// Arithmetic (same as gemv_mma.cu): every 8-byte half-codeword read from the
// shared-memory table is an A-fragment register pair of mma.sync.m16n8k16; the
// activations enter as fp16 high part + fp16 remainder in separate B columns.
//
// Work split ("stream-K"): all 16-row x 32-column strips of all layers form one
// sequence (layer, row tile, strip); main warp w takes the contiguous range
// [w*W/nw, (w+1)*W/nw).  Inside a row tile the accumulators stay in registers;
// at a row-tile boundary the warp adds its partial to the tile's fp32 accumulator
// in scratch (red.global.add, so the cost does not grow with the number of warps
// that share a tile) and takes a ticket; the last arrival reads the accumulator,
// puts the zeros back, applies g and bias, writes fp16.  Each warp
// works alone: Q arrives through a 3-deep register ring of 128-bit loads, the
// activation pieces through a 512-byte warp-private slab, no block-wide barrier
// after the table is built.
//
// Table addressing: the 64 KB replicated table sits at shared-window address
// 0x10000, so the byte address of a half-codeword is a single logic operation
// on the raw index bits: (q & 0xFF80) | (8*(lane%16) | 0x10000).
//
// Critical blocks: two warps per block walk the CSR in units of 4 Q rows and add
// sum (O[i] - code[65535]) * h*x to the same accumulators.
//
// E8 variant (KIND == EPTQ_E8): same structure; the A fragments come from a packed 4-byte entry per index
// (e8_decode), looked up in shared memory for the resident part of the table and in global memory for the
// rest (e8_lookup).
//
// Optional fused work around each layer (EptqFusion): RMSNorm of the shared input, residual add, rotary
// embedding and stores into a key/value cache, all done by the warp that finalizes a row tile.
//
// Reference counterparts: e8d4_fused_kernel_t (csrc/eptq_kernels.cu:161-292) and e8_fused_kernel
// (csrc/eptq_kernels.cu:39-150), one launch per layer and batch row there.

#include <cmath>
#include <atomic>
#include <mutex>

#include "gemv_group_common.cuh"

namespace eptq {

using namespace groupdev;


namespace {

// Phase timestamps for latency studies: compiled in only with -DEPTQ_GROUP_TRACE (never in the shipped
// library).  Slot k of block b is g_group_trace[b * 8 + k], in nanoseconds of the global timer.
#ifdef EPTQ_GROUP_TRACE
__device__ unsigned long long* g_group_trace = nullptr;
__device__ __forceinline__ void trace_mark(int slot) {
    if ((threadIdx.x & 31) == 0 && g_group_trace != nullptr) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        g_group_trace[blockIdx.x * 8 + slot] = t;
    }
}
#define EPTQ_TRACE(slot, cond) do { if (cond) trace_mark(slot); } while (0)
#else
#define EPTQ_TRACE(slot, cond) do { } while (0)
#endif

constexpr int kMainWarps = 14;
constexpr int kCorrWarps = 2;
constexpr int kGroupThreads = (kMainWarps + kCorrWarps) * 32;
constexpr unsigned kTableAddr = 0x10000u;                       // shared-window address of the table
constexpr int kGroupSmemBytes = 2 * 65536 - 1024;               // window [0x400, 0x20000)
constexpr int kRing = 3;                                        // Q strips in flight per warp (E8-D4)
// E8: the packed table (4 bytes per entry) does not fit whole; entries [0, kE8Resident) live in shared
// memory behind the slabs, the rest is read from the copy in global memory (L2).
constexpr int kRingE8 = 2;
constexpr int kE8SmemBytes = 232448;                            // the most a block may ask for
constexpr int kE8TableOffset = (kMainWarps + kCorrWarps) * 512 + 512;
constexpr unsigned kE8Resident = (kE8SmemBytes - kE8TableOffset) / 4;

__device__ __forceinline__ uint2 table_lds(unsigned addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ unsigned prmt(unsigned a, unsigned b, unsigned sel) {
    unsigned d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint2& a01, const uint2& a23, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a01.x), "r"(a01.y), "r"(a23.x), "r"(a23.y), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ unsigned split_pieces(float v) {
    const __half hi = __float2half_rn(v);
    const __half lo = __float2half_rn(v - __half2float(hi));
    return static_cast<unsigned>(__half_as_ushort(hi)) | (static_cast<unsigned>(__half_as_ushort(lo)) << 16);
}
// Shared-window addresses of the two half-codewords of the index in the low 16 bits of q.
__device__ __forceinline__ void code_addrs(unsigned q, unsigned lane_tab, unsigned& ai, unsigned& aj) {
    ai = (q & 0xFF80u) | lane_tab;
    aj = ((q << 7) & 0x3F80u) | ((q & 0xC000u) | lane_tab);
}

// Packed E8 entry -> four A-fragment registers (dims (0,1), (2,3), (4,5), (6,7) as fp16 pairs, in lattice
// units).  Each coordinate is stored as n = 2*coordinate + 6 (0..12) in a 4-bit field placed so that a mask
// drops it straight into the mantissa of the fp16 number 1024 + (n << s): fields of dims 0,1 at bits
// [5:2],[21:18], dims 2,3 at [9:6],[25:22], dims 4,5 at [13:10],[29:26], dims 6,7 at [17:14],[33:30]
// (the last one wraps around: its low two bits are bits 31:30, its high two bits 1:0), so the second
// pair of registers comes from the word rotated by 8.  One fused multiply-add per register removes the
// offset exactly: (1024 + 4n)/8 - 131 = (1024 + 64n)/128 - 11 = n/2 - 3.
__device__ __forceinline__ void e8_decode(unsigned e, unsigned (&r)[4]) {
    const unsigned rot = __funnelshift_r(e, e, 8);
    const unsigned magic = 0x64006400u;
    unsigned a0 = (e & 0x003C003Cu) | magic, a1 = (e & 0x03C003C0u) | magic;
    unsigned a2 = (rot & 0x003C003Cu) | magic, a3 = (rot & 0x03C003C0u) | magic;
    const __half2 kA = __floats2half2_rn(0.125f, 0.125f), cA = __floats2half2_rn(-131.f, -131.f);
    const __half2 kB = __floats2half2_rn(0.0078125f, 0.0078125f), cB = __floats2half2_rn(-11.f, -11.f);
    __half2 h0 = __hfma2(*reinterpret_cast<__half2*>(&a0), kA, cA), h1 = __hfma2(*reinterpret_cast<__half2*>(&a1), kB, cB);
    __half2 h2 = __hfma2(*reinterpret_cast<__half2*>(&a2), kA, cA), h3 = __hfma2(*reinterpret_cast<__half2*>(&a3), kB, cB);
    r[0] = *reinterpret_cast<unsigned*>(&h0); r[1] = *reinterpret_cast<unsigned*>(&h1);
    r[2] = *reinterpret_cast<unsigned*>(&h2); r[3] = *reinterpret_cast<unsigned*>(&h3);
}
// Entry of true index u: from shared memory when resident, else from the global copy.
__device__ __forceinline__ unsigned e8_lookup(unsigned u, unsigned tbase, const unsigned* packed) {
    unsigned v;
    asm volatile("{\n\t.reg .pred p;\n\t.reg .u64 ga;\n\t.reg .u32 sa;\n\t"
                 "setp.ge.u32 p, %1, %2;\n\t"
                 "mad.wide.u32 ga, %1, 4, %3;\n\t"
                 "mad.lo.u32 sa, %1, 4, %4;\n\t"
                 "@p ld.global.nc.u32 %0, [ga];\n\t"
                 "@!p ld.shared.u32 %0, [sa];\n\t}"
                 : "=r"(v) : "r"(u), "r"(kE8Resident), "l"(packed), "r"(tbase));
    return v;
}
__device__ __forceinline__ void mma_f16r(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}


// Number of main warps that contribute to row tile rt of layer L, and the first of them.
__device__ __forceinline__ int tile_contributors(const GroupArgs& p, const GroupLayer& L, int rt, int& first) {
    const long long s0 = L.strip0 + static_cast<long long>(rt) * L.ns;
    first = owner_warp(s0, p.W, p.nw);
    return owner_warp(s0 + L.ns - 1, p.W, p.nw) - first + 1;
}

}  // namespace
}  // namespace eptq

namespace eptq {
namespace {


// Position in the global strip sequence.
struct StripIter {
    long long s;      // global strip index
    int l, rt, strip;
    __device__ __forceinline__ void seek(const GroupArgs& p, long long pos) {
        s = pos;
        l = 0;
        while (l + 1 < p.n_layers && p.L[l + 1].strip0 <= pos) ++l;
        const unsigned local = static_cast<unsigned>(pos - p.L[l].strip0);     // < W < 2^32
        const unsigned ns = static_cast<unsigned>(p.L[l].ns);
        rt = static_cast<int>(local / ns);
        strip = static_cast<int>(local - static_cast<unsigned>(rt) * ns);
    }
};

// NB = batch rows of the launch (1 or 2): a compile-time constant, so that the batch-1 kernel carries no
// second-row loads, stores or branches in its main loop.
template <int KIND, int NB>
__global__ void __launch_bounds__(kGroupThreads, 1) gemv_group_kernel(const __grid_constant__ GroupArgs p) {
    constexpr int RING = KIND == EPTQ_E8 ? kRingE8 : kRing;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const unsigned base = smem_addr(smem_raw);                 // 0x400 on sm_100: the first KB is reserved
    // The table address is a constant of the lookup arithmetic: if dynamic shared memory does not start where
    // this layout assumes, refuse (status word of the scratch) instead of reading outside the allocation.
    if (base != 0x400u) {
        if (threadIdx.x == 0) atomicExch(reinterpret_cast<int*>(p.counters) + (kMaxCounters - 1), static_cast<int>(EPTQ_ERR_LAUNCH));
        return;
    }
    unsigned char* tab = smem_raw + (kTableAddr - base);       // generic pointer to shared address 0x10000

    asm volatile("griddepcontrol.launch_dependents;");
    EPTQ_TRACE(0, warp == 0);

    // ---- main warps: find the first strips and start their loads before anything else, so that the DRAM
    // round trip runs under the table build.  (Correction warps carry the same variables unused.)
    const bool is_main = warp < kMainWarps;
    const int g = lane >> 2, t = lane & 3;
    const int gw = is_main ? blockIdx.x * kMainWarps + warp : p.nw;
    // W * nw < 2^32 (checked on the host): unsigned 32-bit arithmetic is exact and much cheaper than 64-bit division.
    const unsigned W32 = static_cast<unsigned>(p.W), nw32 = static_cast<unsigned>(p.nw);
    const long long s_begin = gw < p.nw ? (static_cast<unsigned>(gw) * W32) / nw32 : W32;
    const long long s_end = gw < p.nw ? ((static_cast<unsigned>(gw) + 1u) * W32) / nw32 : W32;
    const int n_total = static_cast<int>(s_end - s_begin);

    unsigned* slab = reinterpret_cast<unsigned*>(smem_raw) + warp * 128;     // [parity][batch][32] words
    slab[lane] = 0u; slab[32 + lane] = 0u; slab[64 + lane] = 0u; slab[96 + lane] = 0u;

    // Cursor over the strip sequence: which row tile, how many strips are left in it, and this
    // lane's addresses (Q rows g and g+8 at its 8 columns; h and x at column `lane` of the strip).
    struct Cursor {
        int l, rt, left, N;
        const int16_t *pa, *pb;
        const __half *ph, *px;
    };
    auto place = [&](Cursor& c, int strip) {
        const GroupLayer& L = p.L[c.l];
        const int ra = min(c.rt * 16 + g, L.M - 1), rb = min(c.rt * 16 + g + 8, L.M - 1);
        c.N = L.N;
        c.left = L.ns - strip;
        c.pa = L.Q + static_cast<size_t>(ra) * L.N + strip * 32 + 8 * t;
        c.pb = L.Q + static_cast<size_t>(rb) * L.N + strip * 32 + 8 * t;
        c.ph = L.h + strip * 32 + lane;
        c.px = L.x + strip * 32 + lane;
    };
    auto step = [&](Cursor& c) {
        c.pa += 32; c.pb += 32; c.ph += 32; c.px += 32;
        if (--c.left == 0) {
            if (++c.rt == p.L[c.l].row_tiles) { c.rt = 0; ++c.l; }
            if (c.l < p.n_layers) place(c, 0);
        }
    };

    Cursor pf;                                           // prefetch position
    {
        StripIter it;
        it.seek(p, n_total > 0 ? s_begin : 0);
        pf.l = it.l; pf.rt = it.rt;
        place(pf, it.strip);
    }
    const int cur_l0 = pf.l, cur_rt0 = pf.rt, cur_left0 = pf.left;
    Cursor xfirst = pf;                                  // for the x loads that must follow the dependency wait

    uint4 qa[RING], qb[RING];
    __half hr[RING], xr0[RING], xr1[RING];
#pragma unroll
    for (int i = 0; i < RING; ++i) {
        qa[i] = make_uint4(0, 0, 0, 0); qb[i] = make_uint4(0, 0, 0, 0);
        hr[i] = __ushort_as_half(0); xr0[i] = __ushort_as_half(0); xr1[i] = __ushort_as_half(0);
    }
    int pf_todo = n_total;
#pragma unroll
    for (int i = 0; i < RING; ++i) {
        if (pf_todo > 0) {
            qa[i] = ldg_stream(pf.pa);
            qb[i] = ldg_stream(pf.pb);
            hr[i] = __ldg(pf.ph);
            step(pf);
            --pf_todo;
        }
    }
    // ---- correction warps.  They need neither the table nor, unless the input norm is fused, anything the
    // other warps compute, so in that case they start at once and the table barrier is for the main warps only.
    auto run_corrections = [&](const float* inv_rms_ptr) {
        // What the main loop adds for a marker: E8-D4 entry (3,127) in both halves; E8 entry 65535 is zero.
        float2 c01 = make_float2(0.f, 0.f), c23 = make_float2(0.f, 0.f);
        if constexpr (KIND == EPTQ_E8D4) {
            const uint2 craw = __ldg(p.table16 + 511);
            c01 = __half22float2(*reinterpret_cast<const __half2*>(&craw.x));
            c23 = __half22float2(*reinterpret_cast<const __half2*>(&craw.y));
        }
        bool waited = false;
        const int cw = blockIdx.x * kCorrWarps + (warp - kMainWarps);
        int l = 0;
        for (int u = cw; u < p.corr_units; u += p.n_corr_warps) {
            while (l + 1 < p.n_layers && p.L[l + 1].corr0 <= u) ++l;
            correction_unit(p, p.L[l], u - p.L[l].corr0, lane, c01.x, c01.y, c23.x, c23.y, inv_rms_ptr, [&]() {
                if (!waited) { asm volatile("griddepcontrol.wait;" ::: "memory"); waited = true; }
            }, [&](const GroupLayer& GL, int rt) { int first_warp; return tile_contributors(p, GL, rt, first_warp); });
        }
        EPTQ_TRACE(7, warp == kMainWarps);
    };
    const bool corr_early = p.x_norm == 0;                 // the same for every thread of the launch
    if (corr_early && warp >= kMainWarps) {
        run_corrections(nullptr);
        return;
    }
    const int builders = corr_early ? kMainWarps * 32 : kGroupThreads;
    EPTQ_TRACE(1, warp == 0);
    if constexpr (KIND == EPTQ_E8) {
        // Resident part of the packed table: asynchronous 16-byte copies, no registers in between.
        const unsigned dst0 = base + kE8TableOffset;
        const char* src0 = reinterpret_cast<const char*>(p.packed);
        for (unsigned off = threadIdx.x * 16u; off < kE8Resident * 4u; off += builders * 16u)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(dst0 + off), "l"(src0 + off) : "memory");
        asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
    } else {
        // Replicated table; entry order follows the raw stored bits (true index ^ 0x100 on 9 bits).  Both loads
        // of a thread (512 entries over 448 or 512 threads) go out before the stores: one memory round trip.
        static_assert(kMainWarps * 64 >= 512, "at most two table entries per thread");
        const int e0 = threadIdx.x, e1 = threadIdx.x + builders;
        const uint2 v0 = __ldg(p.table16 + (e0 ^ 0x100));
        const uint2 v1 = e1 < 512 ? __ldg(p.table16 + (e1 ^ 0x100)) : make_uint2(0, 0);
        const uint4 vv0 = make_uint4(v0.x, v0.y, v0.x, v0.y), vv1 = make_uint4(v1.x, v1.y, v1.x, v1.y);
#pragma unroll
        for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(tab + e0 * 128 + ((c + e0) & 7) * 16) = vv0;
        if (e1 < 512) {
#pragma unroll
            for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(tab + e1 * 128 + ((c + e1) & 7) * 16) = vv1;
        }
    }

    if (corr_early) asm volatile("bar.sync 1, %0;" :: "n"(kMainWarps * 32) : "memory");   // table complete: main warps only
    else __syncthreads();                                                                    // all 16 warps
    EPTQ_TRACE(2, warp == 0);

    // Fused RMSNorm of the input: every layer of the launch reads the same x; the column weight of the
    // norm is folded into h by the caller, the row factor rsqrt(mean(x^2) + eps) is applied by the
    // finalizing warp.  Each block computes it for itself.
    const float* inv_rms = nullptr;
    if (p.x_norm) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        float* red = reinterpret_cast<float*>(smem_raw + kGroupThreads / 32 * 512);       // behind the slabs
        const int N = p.L[0].N;
        float ss[2] = {0.f, 0.f};
        for (int b = 0; b < p.B; ++b)
            for (int c = threadIdx.x * 8; c < N; c += kGroupThreads * 8) {
                float f[8];
                unpack8(ldg128(p.L[0].x + static_cast<size_t>(b) * N + c), f);
#pragma unroll
                for (int i = 0; i < 8; ++i) ss[b] = fmaf(f[i], f[i], ss[b]);
            }
#pragma unroll
        for (int b = 0; b < 2; ++b) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss[b] += __shfl_xor_sync(0xffffffffu, ss[b], o);
            if (lane == 0) red[warp * 2 + b] = ss[b];
        }
        __syncthreads();
        if (threadIdx.x < 2) {
            float tot = 0.f;
            for (int w = 0; w < kGroupThreads / 32; ++w) tot += red[w * 2 + threadIdx.x];
            red[64 + threadIdx.x] = rsqrtf(tot / static_cast<float>(N) + p.norm_eps);
        }
        __syncthreads();
        inv_rms = red + 64;
    }

    if (warp >= kMainWarps) {
        run_corrections(inv_rms);
        return;
    }

    asm volatile("griddepcontrol.wait;" ::: "memory");
    EPTQ_TRACE(3, warp == 0);
    if (n_total <= 0) return;
#pragma unroll
    for (int i = 0; i < RING; ++i) {
        if (i < n_total) {
            xr0[i] = __ldg(xfirst.px);
            if constexpr (NB > 1) xr1[i] = __ldg(xfirst.px + xfirst.N);
            step(xfirst);
        }
    }

    const unsigned lane_tab = 8u * (lane & 15) | kTableAddr;
    // B column g = (batch g>>2, piece (g>>1)&1, dd' = g&1): the piece goes to the low or high half.
    const unsigned pbyte = 2u * ((g >> 1) & 1);
    const unsigned sel = (g & 1) ? ((((pbyte + 1) << 12) | (pbyte << 8)) | 0x0044u) : (0x4400u | ((pbyte + 1) << 4) | pbyte);
    const unsigned* my_slab = slab + (g >> 2) * 32 + 8 * t;

    EPTQ_TRACE(4, warp == 0);
    int cl = cur_l0, crt = cur_rt0, cleft = cur_left0;   // compute position: layer, row tile, strips left in it
    float cscale = p.L[cl].x_scale;
    int todo = n_total;
    int par = 0;
    float acc[2][2][4];                                // [row group g / g+8][half i / j][dims]
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 2; ++b)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[a][b][c] = 0.f;

    auto flush = [&](int l, int rt) {
        EPTQ_TRACE(5, warp == 0);
        const GroupLayer& L = p.L[l];
        const Affine aff = load_affine(L, rt, lane);   // in flight while the ticket travels
        int first_warp;
        const int n_main = tile_contributors(p, L, rt, first_warp);
        const float inv = L.x_inv_scale;
        const int b = t >> 1;
        float* dst = p.acc + L.acc_off + (static_cast<size_t>(rt) * p.B + b) * 128;
#pragma unroll
        for (int rg = 0; rg < 2; ++rg)
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                float tot[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float own = acc[rg][hf][c] * inv;
                    tot[c] = own + __shfl_xor_sync(0xffffffffu, own, 1);
                    acc[rg][hf][c] = 0.f;
                }
                if ((t & 1) == 0 && b < p.B)
                    red_add4(dst + (g + 8 * rg) * 8 + hf * 4, tot[0], tot[1], tot[2], tot[3]);
            }
        arrive_and_finalize(p, L, rt, n_main, lane, aff, inv_rms);
        EPTQ_TRACE(6, warp == 0);
    };

#define EPTQ_GROUP_STEP(I)                                                                                   \
    {                                                                                                        \
        if (todo == 0) break;                                                                                \
        const uint4 ca = qa[I], cb = qb[I];                                                                  \
        const float hx = __half2float(hr[I]) * cscale;                                                       \
        unsigned* wslab = slab + par * 64;                                                                   \
        wslab[lane] = split_pieces(__half2float(xr0[I]) * hx);                                               \
        if constexpr (NB > 1) wslab[32 + lane] = split_pieces(__half2float(xr1[I]) * hx);                             \
        if (pf_todo > 0) {                                                                                   \
            qa[I] = ldg_stream(pf.pa);                                                                       \
            qb[I] = ldg_stream(pf.pb);                                                                       \
            hr[I] = __ldg(pf.ph);                                                                            \
            xr0[I] = __ldg(pf.px);                                                                           \
            if constexpr (NB > 1) xr1[I] = __ldg(pf.px + pf.N);                                                       \
            step(pf);                                                                                        \
            --pf_todo;                                                                                       \
        }                                                                                                    \
        __syncwarp();                                                                                        \
        const uint4 w0 = *reinterpret_cast<const uint4*>(my_slab + par * 64);                                \
        const uint4 w1 = *reinterpret_cast<const uint4*>(my_slab + par * 64 + 4);                            \
        par ^= 1;                                                                                            \
        const unsigned wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};                             \
        const unsigned qav[4] = {ca.x, ca.y, ca.z, ca.w};                                                    \
        const unsigned qbv[4] = {cb.x, cb.y, cb.z, cb.w};                                                    \
        _Pragma("unroll")                                                                                    \
        for (int m = 0; m < 4; ++m) {                                                                        \
            unsigned i0, j0, i1, j1;                                                                         \
            code_addrs(qav[m], lane_tab, i0, j0);                                                            \
            code_addrs(qav[m] >> 16, lane_tab, i1, j1);                                                      \
            const uint2 ai0 = table_lds(i0), aj0 = table_lds(j0), ai1 = table_lds(i1), aj1 = table_lds(j1);  \
            code_addrs(qbv[m], lane_tab, i0, j0);                                                            \
            code_addrs(qbv[m] >> 16, lane_tab, i1, j1);                                                      \
            const uint2 bi0 = table_lds(i0), bj0 = table_lds(j0), bi1 = table_lds(i1), bj1 = table_lds(j1);  \
            const unsigned b0 = prmt(wv[2 * m], 0u, sel), b1 = prmt(wv[2 * m + 1], 0u, sel);                 \
            mma_f16(acc[0][0], ai0, ai1, b0, b1);                                                            \
            mma_f16(acc[0][1], aj0, aj1, b0, b1);                                                            \
            mma_f16(acc[1][0], bi0, bi1, b0, b1);                                                            \
            mma_f16(acc[1][1], bj0, bj1, b0, b1);                                                            \
        }                                                                                                    \
        --todo;                                                                                              \
        if (--cleft == 0 || todo == 0) {                                                                     \
            flush(cl, crt);                                                                                  \
            if (cleft == 0) {                                                                                \
                if (++crt == p.L[cl].row_tiles) { crt = 0; ++cl; }                                           \
                if (cl < p.n_layers) { cleft = p.L[cl].ns; cscale = p.L[cl].x_scale; }                       \
            }                                                                                                \
        }                                                                                                    \
    }

    // E8: all 16 lookups of a strip are issued before the first is used, so that the round trip of the
    // non-resident ones (L2) is paid once per strip and overlaps the other warps' work.
#define EPTQ_GROUP_STEP_E8(I)                                                                                \
    {                                                                                                        \
        if (todo == 0) break;                                                                                \
        const uint4 ca = qa[I], cb = qb[I];                                                                  \
        const float hx = __half2float(hr[I]) * cscale;                                                       \
        unsigned* wslab = slab + par * 64;                                                                   \
        wslab[lane] = split_pieces(__half2float(xr0[I]) * hx);                                               \
        if constexpr (NB > 1) wslab[32 + lane] = split_pieces(__half2float(xr1[I]) * hx);                             \
        if (pf_todo > 0) {                                                                                   \
            qa[I] = ldg_stream(pf.pa);                                                                       \
            qb[I] = ldg_stream(pf.pb);                                                                       \
            hr[I] = __ldg(pf.ph);                                                                            \
            xr0[I] = __ldg(pf.px);                                                                           \
            if constexpr (NB > 1) xr1[I] = __ldg(pf.px + pf.N);                                                       \
            step(pf);                                                                                        \
            --pf_todo;                                                                                       \
        }                                                                                                    \
        const unsigned qw[8] = {ca.x ^ 0x80008000u, ca.y ^ 0x80008000u, ca.z ^ 0x80008000u, ca.w ^ 0x80008000u, \
                                cb.x ^ 0x80008000u, cb.y ^ 0x80008000u, cb.z ^ 0x80008000u, cb.w ^ 0x80008000u}; \
        unsigned ent[16];                                                                                    \
        _Pragma("unroll")                                                                                    \
        for (int k = 0; k < 8; ++k) {                                                                        \
            ent[2 * k] = e8_lookup(qw[k] & 0xFFFFu, tbase_e8, p.packed);                                     \
            ent[2 * k + 1] = e8_lookup(qw[k] >> 16, tbase_e8, p.packed);                                     \
        }                                                                                                    \
        __syncwarp();                                                                                        \
        const uint4 w0 = *reinterpret_cast<const uint4*>(my_slab + par * 64);                                \
        const uint4 w1 = *reinterpret_cast<const uint4*>(my_slab + par * 64 + 4);                            \
        par ^= 1;                                                                                            \
        const unsigned wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};                             \
        _Pragma("unroll")                                                                                    \
        for (int m = 0; m < 4; ++m) {                                                                        \
            unsigned a0[4], a1[4], b0r[4], b1r[4];                                                           \
            e8_decode(ent[2 * m], a0);                                                                       \
            e8_decode(ent[2 * m + 1], a1);                                                                   \
            e8_decode(ent[8 + 2 * m], b0r);                                                                  \
            e8_decode(ent[8 + 2 * m + 1], b1r);                                                              \
            const unsigned b0 = prmt(wv[2 * m], 0u, sel), b1 = prmt(wv[2 * m + 1], 0u, sel);                 \
            mma_f16r(acc[0][0], a0[0], a0[1], a1[0], a1[1], b0, b1);                                         \
            mma_f16r(acc[0][1], a0[2], a0[3], a1[2], a1[3], b0, b1);                                         \
            mma_f16r(acc[1][0], b0r[0], b0r[1], b1r[0], b1r[1], b0, b1);                                     \
            mma_f16r(acc[1][1], b0r[2], b0r[3], b1r[2], b1r[3], b0, b1);                                     \
        }                                                                                                    \
        --todo;                                                                                              \
        if (--cleft == 0 || todo == 0) {                                                                     \
            flush(cl, crt);                                                                                  \
            if (cleft == 0) {                                                                                \
                if (++crt == p.L[cl].row_tiles) { crt = 0; ++cl; }                                           \
                if (cl < p.n_layers) { cleft = p.L[cl].ns; cscale = p.L[cl].x_scale; }                       \
            }                                                                                                \
        }                                                                                                    \
    }

    if constexpr (KIND == EPTQ_E8) {
        const unsigned tbase_e8 = base + kE8TableOffset;
        for (;;) {
            EPTQ_GROUP_STEP_E8(0)
            EPTQ_GROUP_STEP_E8(1)
        }
    } else {
        for (;;) {
            EPTQ_GROUP_STEP(0)
            EPTQ_GROUP_STEP(1)
            EPTQ_GROUP_STEP(2)
        }
    }
#undef EPTQ_GROUP_STEP_E8
#undef EPTQ_GROUP_STEP
}

}  // namespace
}  // namespace eptq

namespace eptq {

namespace {

struct GroupPlan {
    long long W = 0;
    int nw = 0;
    int n_sms = 0;
    int tiles = 0;
    int corr_units = 0;
    size_t acc_floats = 0;
};

int cached_sm_count() {
    static int sms[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (sms[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        sms[dev] = n;
    }
    return sms[dev];
}

// Shapes only: how many strips, warps and accumulator floats a group needs.
bool plan_group(const EptqLayer* layers, int n, int B, int n_sms, GroupPlan& plan) {
    if (n < 1 || n > kMaxGroupLayers || B < 1 || B > 2 || n_sms < 1) return false;
    plan = GroupPlan();
    plan.n_sms = n_sms;
    plan.nw = n_sms * kMainWarps;
    for (int i = 0; i < n; ++i) {
        const int row_tiles = (layers[i].M + 15) / 16;
        plan.W += static_cast<long long>(row_tiles) * (layers[i].N / 32);
        plan.tiles += row_tiles;
        plan.corr_units += row_tiles * 4;
    }
    if (plan.W < 1 || plan.tiles > kMaxCounters - 1) return false;
    if (plan.nw > plan.W) plan.nw = static_cast<int>(plan.W);          // every warp range non-empty
    if (plan.W * plan.nw >= (1LL << 32)) return false;                  // owner_warp works in 32 bits
    plan.acc_floats = static_cast<size_t>(plan.tiles) * B * 128;
    if (plan.acc_floats * sizeof(float) > kPartialOffset - kCounterBytes) return false;
    return true;
}

bool group_layer_supported(const EptqLayer& L) {
    const bool common = L.S_group == nullptr && L.M > 0 && L.N > 0 && (L.N % 32) == 0 && L.h_absmax > 0.f &&
                        L.Q != nullptr && L.g != nullptr && L.h != nullptr && L.O_row_ptr != nullptr &&
                        (L.n_masked == 0 || (L.O_vals != nullptr && L.O_col != nullptr)) && aligned16(L.Q) &&
                        aligned16(L.g) && (L.bias == nullptr || aligned16(L.bias)) &&
                        (L.n_masked == 0 || aligned16(L.O_vals));
    if (!common) return false;
    if (L.quantizer == EPTQ_E8D4) return L.table16 != nullptr && aligned16(L.table16);
    if (L.quantizer == EPTQ_E8)
        return L.table_packed != nullptr && aligned16(L.table_packed) && L.table_packed_scale > 0.f;
    return false;
}

}  // namespace

bool group_gemv_supported(const EptqLayer* layers, int n, int B) {
    if (layers == nullptr || n < 1 || n > kMaxGroupLayers || B < 1 || B > kGemmMinBatch) return false;   // > 2: passes of two rows
    for (int i = 0; i < n; ++i) {
        if (!group_layer_supported(layers[i])) return false;
        if (layers[i].quantizer != layers[0].quantizer || layers[i].table16 != layers[0].table16 ||
            layers[i].table_packed != layers[0].table_packed ||
            layers[i].table_packed_scale != layers[0].table_packed_scale) return false;   // one codebook per launch
    }
    return true;
}

size_t group_workspace_bytes(const EptqLayer* layers, int n, int B, int n_sms) {
    GroupPlan plan;
    if (n_sms <= 0) n_sms = 148;
    if (!plan_group(layers, n, B > 2 ? 2 : B, n_sms, plan)) return 0;
    return kPartialOffset;
}

namespace {
int launch_gemv_group_pass(const EptqLayer* layers, int n, const EptqFusion* fusions, const uint16_t* const* xs,
                           uint16_t* const* ys, int B, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    const int n_sms = cached_sm_count();
    GroupPlan plan;
    if (!plan_group(layers, n, B, n_sms, plan)) return EPTQ_ERR_UNSUPPORTED;
    const size_t need = kPartialOffset;
    if (workspace == nullptr || workspace_bytes < need) return EPTQ_ERR_WORKSPACE;

    static GroupArgs args;                     // large: keep it off the stack; filled under a lock
    static std::mutex args_mutex;
    std::lock_guard<std::mutex> lock(args_mutex);
    GroupArgs& a = args;
    const bool e8 = layers[0].quantizer == EPTQ_E8;
    a.W = plan.W;
    a.nw = plan.nw;
    a.corr_units = plan.corr_units;
    a.n_corr_warps = n_sms * kCorrWarps;
    {
        const int st = fill_group_args(a, layers, n, fusions, xs, ys, B, workspace);
        if (st != EPTQ_OK) return st;
    }

    static std::atomic<bool> attr_done[64];       // setting the attribute twice is harmless; the flag itself must not race
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return EPTQ_ERR_LAUNCH;
    if (!attr_done[dev]) {
        if (cudaFuncSetAttribute(gemv_group_kernel<EPTQ_E8D4, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGroupSmemBytes) != cudaSuccess ||
            cudaFuncSetAttribute(gemv_group_kernel<EPTQ_E8D4, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGroupSmemBytes) != cudaSuccess ||
            cudaFuncSetAttribute(gemv_group_kernel<EPTQ_E8, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kE8SmemBytes) != cudaSuccess ||
            cudaFuncSetAttribute(gemv_group_kernel<EPTQ_E8, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kE8SmemBytes) != cudaSuccess)
            return EPTQ_ERR_LAUNCH;
        attr_done[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_sms);
    cfg.blockDim = dim3(kGroupThreads);
    cfg.dynamicSmemBytes = e8 ? kE8SmemBytes : kGroupSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t err =
        e8 ? (B == 1 ? cudaLaunchKernelEx(&cfg, gemv_group_kernel<EPTQ_E8, 1>, a) : cudaLaunchKernelEx(&cfg, gemv_group_kernel<EPTQ_E8, 2>, a))
           : (B == 1 ? cudaLaunchKernelEx(&cfg, gemv_group_kernel<EPTQ_E8D4, 1>, a) : cudaLaunchKernelEx(&cfg, gemv_group_kernel<EPTQ_E8D4, 2>, a));
    count_launch(EPTQ_KERNEL_GEMV_GROUP);
    return err == cudaSuccess ? EPTQ_OK : EPTQ_ERR_LAUNCH;
}

}  // namespace

// Batches above 2 run as passes of two batch rows over the same weights (the kernel's MMA columns hold two
// rows); the scratch is reused, the passes are ordered on the stream.  Fused epilogues that index a cache
// by batch entry are limited to one pass.
int launch_gemv_group(const EptqLayer* layers, int n, const EptqFusion* fusions, const uint16_t* const* xs,
                      uint16_t* const* ys, int B, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    if (B <= 2) return launch_gemv_group_pass(layers, n, fusions, xs, ys, B, workspace, workspace_bytes, stream);
    if (fusions != nullptr || n > kMaxGroupLayers) return EPTQ_ERR_UNSUPPORTED;
    const uint16_t* xp[kMaxGroupLayers];
    uint16_t* yp[kMaxGroupLayers];
    for (int b0 = 0; b0 < B; b0 += 2) {
        for (int i = 0; i < n; ++i) {
            if (xs[i] == nullptr || ys[i] == nullptr) return EPTQ_ERR_NULL;
            xp[i] = xs[i] + static_cast<size_t>(b0) * layers[i].N;
            yp[i] = ys[i] + static_cast<size_t>(b0) * 8 * layers[i].M;
        }
        const int st = launch_gemv_group_pass(layers, n, nullptr, xp, yp, B - b0 >= 2 ? 2 : 1, workspace,
                                              workspace_bytes, stream);
        if (st != EPTQ_OK) return st;
    }
    return EPTQ_OK;
}

}  // namespace eptq

#ifdef EPTQ_GROUP_TRACE
extern "C" int eptq_debug_set_group_trace(unsigned long long* device_buffer) {
    return cudaMemcpyToSymbol(eptq::g_group_trace, &device_buffer, sizeof(device_buffer)) == cudaSuccess ? 0 : 6;
}
#endif