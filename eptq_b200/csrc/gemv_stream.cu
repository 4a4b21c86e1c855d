// Streaming decode GEMV for E8-D4 layers, batch 1: the weight indices arrive through a ring of bulk-tensor
// (TMA) loads, the codebook is an int8 table in shared memory, the products run on the integer tensor cores.
//
// One persistent block per SM; the launch covers 1..32 independent layers (as gemv_group.cu).  The work of
// all layers is one sequence of units of 64 Q rows x 128 columns (16 KB of indices), row tile after row tile;
// block b takes the contiguous range [b*U/G, (b+1)*U/G).
//
//   producer (one thread)   cp.async.bulk.tensor.3d loads, one per unit, into a ring of 6 stages; a stage is
//                           reloaded as soon as its 16 consumer warps have copied their indices to registers.
//                           The loads start at kernel entry, before the dependency on the previous kernel.
//   16 consumer warps       warp w owns columns 8w..8w+7 of the stage and all 64 rows.  ldmatrix hands lane
//                           (g,t) the index pair (row 8r+g, columns 2t, 2t+1) of row group r; each half
//                           codeword is one 32-bit read of four int8 coordinates from a table with one copy
//                           per lane (entry e of lane l at 128*e + 4*l: no bank conflicts); four such reads
//                           are the A fragment of one mma.sync.m16n8k32.s8 (rows g / g+8 = the two halves of
//                           the codeword, k = 4*t + dimension for two columns).  B holds the activation of
//                           those columns as two int8 digits in the byte of the matching dimension, so the
//                           eight result columns are (digit, dimension) and the int32 accumulators are exact.
//   activations             x*h of the layer is scaled by 32000/max|x*h| to 16 bits and split into a low and
//                           a high signed byte (planes in shared memory, built once per layer and block).
//                           Error per term <= max|x*h| / 64000, independent of the length of the sum.
//   end of a row tile       the warps add their int32 partials into a 4 KB shared-memory tile, 512 threads
//                           turn it into floats, add them to the tile's fp32 accumulators in scratch and take
//                           tickets; the last arrival (of all blocks and of the critical-block corrections)
//                           applies g, bias and the fused epilogue -- the protocol of gemv_group.cu.
//   2 correction warps      critical blocks: sum (O - code[marker]) * h*x, as in gemv_group.cu.
//
// Every wait on an mbarrier is bounded by the global timer; a wait that runs out stops further waiting in
// that warp (the control flow still reaches every barrier) and EPTQ_ERR_TIMEOUT is written to the status
// word of the scratch (the last counter).
//
// Reference counterpart: e8d4_fused_kernel_t (csrc/eptq_kernels.cu:161-292), one launch per layer there.

#include <cuda.h>
#include <cudaTypedefs.h>

#include <mutex>
#include <unordered_map>

#include "gemv_group_common.cuh"

namespace eptq {

using namespace groupdev;

namespace {

constexpr int kConsumerWarps = 16;
constexpr int kProducerWarp = kConsumerWarps;                       // warp index
constexpr int kFinalizerWarp = kConsumerWarps + 1;
constexpr int kStreamCorrWarps = 2;                                 // warps 18, 19
constexpr int kAuxWarps = 1 + kStreamCorrWarps;                     // finalizer and correction warps
constexpr int kStreamThreads = (kConsumerWarps + 1 + kAuxWarps) * 32;   // five warpgroups
constexpr int kStages = 6;
constexpr int kStageBytes = 64 * 128 * 2;
constexpr int kStreamMaxN = 25600;                                  // columns the digit planes hold
// Shared memory by absolute shared-window address (dynamic shared memory starts at 0x400 on sm_100; the
// kernel checks it).  The table sits on a 64 KB boundary so that a lookup address is (bits of q) | constant.
constexpr unsigned kBase = 0x400u;
constexpr unsigned kFullBar = 0x400u;                               // kStages x 8 bytes
constexpr unsigned kEmptyBar = 0x440u;
constexpr unsigned kRedFull = 0x480u;                               // 2 x 8: a flush buffer holds a finished tile
constexpr unsigned kRedFree = 0x490u;                               // 2 x 8: the finalizer has emptied it
constexpr unsigned kMail = 0x4A0u;                                  // 2 x {-, -, RMSNorm factor, scale}
constexpr unsigned kPrep = 0x4C0u;                                  // 8: the digit planes of a layer are ready
constexpr unsigned kMisc = 0x500u;                                  // 128 floats of reductions and results
constexpr unsigned kRed = 0x800u;                                   // 2 x [digit][64 rows][8] int32
constexpr unsigned kCorr = 0x2800u;                                 // 2 x [64 rows][8] int32, 1/16 units: critical-block corrections
constexpr float kCorrStep = 1.f / 16.f;                               // fixed-point step of the correction sums
constexpr unsigned kPlane = 0x3800u;                                // low digits, then high digits
constexpr unsigned kTable = 0x10000u;
constexpr unsigned kRing = 0x20000u;
constexpr unsigned kSmemEnd = kRing + kStages * kStageBytes;        // 0x38000
constexpr int kStreamSmemBytes = static_cast<int>(kSmemEnd - kBase);
static_assert(kPlane + 2 * kStreamMaxN <= kTable, "digit planes overlap the table");

// One-phase launches of several long layers: block b works on units [W b / G + cut[b], W (b + 1) / G + cut[b + 1]),
// the even split shifted by a few units per block, so that a block which goes on into another layer (and prepares
// that layer's input in between) gets fewer units.  Only the instantiation that uses it carries the table.
template <bool CUT> struct CutTable { signed char cut[kMaxCutBlocks + 1]; };
template <> struct CutTable<false> {};
template <int MAXL, bool CUT = false>
struct StreamArgsT {
    GroupArgsT<MAXL> g;                           // layers and scratch; W = units, nw = blocks
    alignas(64) CUtensorMap maps[MAXL];
    CutTable<CUT> shift;
    float unit;                                   // table value = integer coordinate * unit
    float inv_unit;
    unsigned zero;                                // 0: addend of the index multiplications
    unsigned mul[2];                              // 128 and 1 << 16 as run-time values: the shifts of the index words
                                                  // stay multiplications (FMA pipe) instead of ALU-pipe shifts
    int use_lists;                                // every layer brings its critical blocks as unit lists
    int* status;
    unsigned long long wait_ns;                   // limit of one mbarrier wait
};
using StreamArgs = StreamArgsT<kMaxGroupLayers, false>;
constexpr int kSmallGroup = 8;                // launches of up to this many layers pass the small parameter block

// Phase time stamps for latency studies: compiled in only with -DEPTQ_STREAM_TRACE (never in the shipped
// library).  Slot k of block b is g_stream_trace[b * 64 + k] (k = 8 * phase + event), nanoseconds of the global timer.
#ifdef EPTQ_STREAM_TRACE
__device__ unsigned long long* g_stream_trace = nullptr;
__device__ __forceinline__ void stream_trace(int slot) {
    if ((threadIdx.x & 31) == 0 && g_stream_trace != nullptr) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        g_stream_trace[blockIdx.x * 64 + slot] = t;
    }
}
#define EPTQ_STRACE(slot, cond) do { if (cond) stream_trace(slot); } while (0)
__device__ __forceinline__ void stream_trace_max(int slot) {
    if ((threadIdx.x & 31) == 0 && g_stream_trace != nullptr) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        atomicMax(g_stream_trace + blockIdx.x * 64 + slot, t);
    }
}
#define EPTQ_STRACE_MAX(slot) stream_trace_max(slot)
#else
#define EPTQ_STRACE(slot, cond) do { } while (0)
#define EPTQ_STRACE_MAX(slot) do { } while (0)
#endif

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(unsigned bar, unsigned parity) {
    unsigned done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}
// Bounded wait: false when `limit_ns` of the global timer pass without the phase completing.
__device__ __noinline__ bool mbar_wait_slow(unsigned bar, unsigned parity, unsigned long long limit_ns) {
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (;;) {
        // suspended by the hardware until the phase completes or the hint (20 us) passes: no polling in between,
        // so the issue slots stay with the warps that have work and the wake-up does not wait for a sleep to end
        unsigned done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(parity), "r"(20000u) : "memory");
        if (done != 0) return true;
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        if (t - t0 > limit_ns) return false;
    }
}
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, unsigned long long limit_ns) {
    return mbar_try(bar, parity) || mbar_wait_slow(bar, parity, limit_ns);
}
__device__ __forceinline__ unsigned lds32(unsigned addr) {
    unsigned v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(unsigned addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ unsigned lds16(unsigned addr) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts32(unsigned addr, unsigned v) {
    asm volatile("st.shared.u32 [%0], %1;" :: "r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void sts64(unsigned addr, unsigned a, unsigned b) {
    asm volatile("st.shared.v2.u32 [%0], {%1,%2};" :: "r"(addr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void sts128(unsigned addr, unsigned a, unsigned b, unsigned c, unsigned d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" :: "r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ unsigned prmt(unsigned a, unsigned b, unsigned sel) {
    unsigned d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
// (a & m) | (b & ~m)
__device__ __forceinline__ unsigned bitsel(unsigned a, unsigned b, unsigned m) {
    unsigned d;
    asm("lop3.b32 %0, %1, %2, %3, 0xE4;" : "=r"(d) : "r"(a), "r"(b), "r"(m));
    return d;
}
__device__ __forceinline__ void ldsm4(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void imma(int (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void consumer_barrier() {
    asm volatile("bar.sync 1, %0;" :: "n"(kConsumerWarps * 32) : "memory");
}
// Four fp16 table values -> four int8 lattice coordinates in one word.
__device__ __forceinline__ unsigned pack_coords(uint2 v, float inv_unit) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
    return (static_cast<unsigned>(__float2int_rn(a.x * inv_unit)) & 0xFFu) |
           ((static_cast<unsigned>(__float2int_rn(a.y * inv_unit)) & 0xFFu) << 8) |
           ((static_cast<unsigned>(__float2int_rn(b.x * inv_unit)) & 0xFFu) << 16) |
           ((static_cast<unsigned>(__float2int_rn(b.y * inv_unit)) & 0xFFu) << 24);
}

// A run of units inside one 64-row tile of one layer: what a block processes between two flushes.
struct Segment {
    int l, rt, cc, n;
    bool new_layer;          // the block has not prepared this layer's activations yet
};
// The block's work in order: for each phase its share [U*b/G, U*(b+1)/G) of the phase's units, cut at the ends
// of 64-row tiles.  Producer, consumers and finalizer each walk the same sequence.
struct SegmentWalk {
    int k = -1;
    unsigned pos = 0, end = 0;
    int l = 0, last_l = -1;
    const signed char* cut = nullptr;        // shifts of the even split (one-phase launches that carry a CutTable)
    __device__ __forceinline__ explicit SegmentWalk(const signed char* c = nullptr) : cut(c) {}
    template <class GA>
    __device__ __forceinline__ bool next(const GA& p, Segment& s) {
        while (pos == end) {
            if (++k >= p.n_phases) return false;
            const unsigned U = static_cast<unsigned>(p.phase_units[k]), G = gridDim.x;      // U * G < 2^32 (host)
            pos = static_cast<unsigned>(p.phase_unit0[k]) + (U * blockIdx.x) / G;
            end = static_cast<unsigned>(p.phase_unit0[k]) + (U * (blockIdx.x + 1u)) / G;
            if (cut != nullptr) {                            // one phase: the host's corrections to the even split
                pos += cut[blockIdx.x];
                end += cut[blockIdx.x + 1];
            }
        }
        while (l + 1 < p.n_layers && static_cast<unsigned>(p.L[l + 1].unit0) <= pos) ++l;
        const int local = static_cast<int>(pos) - p.L[l].unit0;
        s.l = l;
        s.rt = local / p.L[l].cc128;
        s.cc = local - s.rt * p.L[l].cc128;
        s.n = min(static_cast<int>(end - pos), p.L[l].cc128 - s.cc);
        s.new_layer = l != last_l;
        last_l = l;
        pos += static_cast<unsigned>(s.n);
        return true;
    }
};
template <class GA>
__device__ __forceinline__ int block_units(const GA& p, const signed char* cut) {
    int n = 0;
    for (int k = 0; k < p.n_phases; ++k) {
        const unsigned U = static_cast<unsigned>(p.phase_units[k]), G = gridDim.x;
        n += static_cast<int>((U * (blockIdx.x + 1u)) / G - (U * blockIdx.x) / G);
    }
    if (cut != nullptr) n += cut[blockIdx.x + 1] - cut[blockIdx.x];
    return n;
}

// A layer of phase k may read its input once every row tile of phase k-1 is finalized (which implies the
// phases before it).  Called by a whole warp: each lane reads one of the phase's 32 counters, the sum is the
// number of finished tiles.  Polls with a pause, bounded by the global timer; false when the limit passes.
template <class GA>
__device__ __noinline__ bool wait_phase(const GA& p, int phase, int tiles, unsigned long long limit_ns) {
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    const unsigned* line = p.done + (phase - 1) * 32 + (threadIdx.x & 31);
    for (;;) {
        unsigned v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(line) : "memory");
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (v >= static_cast<unsigned>(tiles)) return true;
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        if (t - t0 > limit_ns) return false;
        __nanosleep(100);
    }
}

// End of a warp that may finalize tiles (finalizer, correction warps) in a chained launch: the last such warp
// of the whole launch puts the zeros back into the phase counters -- every tile is finalized by then.
template <class GA>
__device__ __forceinline__ void launch_exit(const GA& p, int lane) {
    if (p.done == nullptr) return;
    __syncwarp();
    unsigned old = 0;
    unsigned* finished = p.done + kMaxGroupLayers * 32;
    if (lane == 0) asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(finished) : "memory");
    old = __shfl_sync(0xffffffffu, old, 0);
    if (old + 1u == gridDim.x * kAuxWarps) {
        for (int i = lane; i < p.n_phases * 32; i += 32) p.done[i] = 0u;
        if (lane == 0) *finished = 0u;
    }
}

// Activation of column c as the layer sees it before the RMSNorm factor: x, or silu(x) * x_aux with the
// fp16 roundings of the two separate operations.  L2 loads: another block of this launch may have written x.
__device__ __forceinline__ float activation_at(const GroupLayer& L, int c) {
    const float xv = __half2float(__ldcg(L.x + c));
    if (L.x_op != EPTQ_X_SILU_MUL) return xv;
    const float s = __half2float(__float2half_rn(xv / (1.f + __expf(-xv))));
    return __half2float(__float2half_rn(s * __half2float(__ldcg(L.x_aux + c))));
}
__device__ __forceinline__ void activations8(const GroupLayer& L, int c, float (&out)[8]) {
    unpack8(__ldcg(reinterpret_cast<const uint4*>(L.x + c)), out);
    if (L.x_op == EPTQ_X_SILU_MUL) {
        float u[8];
        unpack8(__ldcg(reinterpret_cast<const uint4*>(L.x_aux + c)), u);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float sv = __half2float(__float2half_rn(out[e] / (1.f + __expf(-out[e]))));
            out[e] = __half2float(__float2half_rn(sv * u[e]));
        }
    }
}
// rsqrt(mean(x^2) + eps) of a layer's input, by one warp (for a correction warp that finalizes a tile).
__device__ __noinline__ float warp_inv_rms(const GroupLayer& L, int lane) {
    float ss = 0.f;
    for (int c = lane * 8; c < L.N; c += 256) {
        float v[8];
        unpack8(__ldcg(reinterpret_cast<const uint4*>(L.x + c)), v);
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(v[e], v[e], ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    return rsqrtf(ss / static_cast<float>(L.N) + L.norm_eps);
}

// Critical blocks of 4 consecutive Q rows, batch 1: 8 lanes per row, two entries per lane and pass (the
// correction warps run with 64 registers).  Adds sum (O - marker code) * h*x to the tile's accumulators and
// arrives as one of the tile's four correction quarters; finalizes the tile if that completes it.
template <class GA, typename WaitFn>
__device__ __forceinline__ void stream_correction_unit(const GA& p, const GroupLayer& L, int qt, int lane,
                                                       float c0, float c1, float c2, float c3, float* inv_rms_slot,
                                                       WaitFn wait_input) {
    const int row = qt * 4 + (lane >> 3);
    const int sub = lane & 7;
    const int rt = qt >> 2;
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    int lo = 0, hi = 0;
    if (row < L.M) {
        lo = __ldg(L.O_row_ptr + row);
        hi = __ldg(L.O_row_ptr + row + 1);
    }
    bool first = true;
    for (int i = lo + sub; __any_sync(0xffffffffu, i < hi) || first; i += 16) {
        int col[2];
        float hv[2];
        uint4 ov[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) col[j] = (i + 8 * j < hi) ? __ldg(L.O_col + i + 8 * j) : -1;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            if (col[j] >= 0) {
                hv[j] = __half2float(__ldg(L.h + col[j]));
                ov[j] = ldg128(L.O_vals + static_cast<size_t>(i + 8 * j) * 8);
            } else {
                hv[j] = 0.f;
                ov[j] = make_uint4(0, 0, 0, 0);
            }
        }
        if (first) { wait_input(); first = false; }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            float o8[8];
            unpack8(ov[j], o8);
            const float xv = (col[j] >= 0) ? hv[j] * activation_at(L, col[j]) : 0.f;
            acc[0] = fmaf(o8[0] - c0, xv, acc[0]); acc[1] = fmaf(o8[1] - c1, xv, acc[1]);
            acc[2] = fmaf(o8[2] - c2, xv, acc[2]); acc[3] = fmaf(o8[3] - c3, xv, acc[3]);
            acc[4] = fmaf(o8[4] - c0, xv, acc[4]); acc[5] = fmaf(o8[5] - c1, xv, acc[5]);
            acc[6] = fmaf(o8[6] - c2, xv, acc[6]); acc[7] = fmaf(o8[7] - c3, xv, acc[7]);
        }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], 1);
        acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], 2);
        acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], 4);
    }
    if (sub == 0 && lo < hi) {
        float* dst = p.acc + L.acc_off + static_cast<size_t>(rt) * p.B * 128 + ((qt & 3) * 4 + (lane >> 3)) * 8;
        red_add4(dst, acc[0], acc[1], acc[2], acc[3]);
        red_add4(dst + 4, acc[4], acc[5], acc[6], acc[7]);
    }
    // One correction quarter arrives; a tile is complete at cc128 units + 4 quarters.
    __syncwarp();
    unsigned old = 0;
    if (lane == 0)
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(p.counters + L.tile0 + rt) : "memory");
    old = __shfl_sync(0xffffffffu, old, 0);
    if (old + 1u == static_cast<unsigned>(L.cc128) + 4u) {
        const float* inv_rms = nullptr;
        if (L.x_op == EPTQ_X_RMSNORM) {
            const float r = warp_inv_rms(L, lane);
            if (lane == 0) *inv_rms_slot = r;
            __syncwarp();
            inv_rms = inv_rms_slot;
        }
        finalize_tile(p, L, rt, lane, load_affine(L, rt, lane), inv_rms);
    }
}

// A finished 64-row tile of a launch that patches critical blocks from unit lists (batch 1): the four 16-row
// tiles at once, every load issued before the first use.  Same arithmetic as finalize_tile.
template <class GA>
__device__ __forceinline__ void finalize_tile64(const GA& p, const GroupLayer& L, int rt64, int lane,
                                                const float* inv_rms) {
    if (lane == 0) p.counters[L.tile0 + rt64 * 4] = 0u;
    __syncwarp();      // lane 0's acquire (its ticket), then the warp barrier: every lane sees the other warps' adds
    const bool rope = L.y_op == EPTQ_Y_ROPE || L.y_op == EPTQ_Y_ROPE_TO_CACHE;
    const bool to_cache = L.y_op == EPTQ_Y_ROPE_TO_CACHE || L.y_op == EPTQ_Y_TO_CACHE;
    float4 s[4];
    uint2 gq[4], bq[4], rq[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int rt16 = rt64 * 4 + j;
        const int row = rt16 * 16 + (lane >> 1);
        const int o = row * 8 + (lane & 1) * 4;
        s[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        gq[j] = make_uint2(0u, 0u); bq[j] = make_uint2(0u, 0u); rq[j] = make_uint2(0u, 0u);
        if (rt16 < L.row_tiles) {
            float* a = p.acc + L.acc_off + static_cast<size_t>(rt16) * 128 + lane * 4;
            s[j] = __ldcg(reinterpret_cast<const float4*>(a));
            __stcg(reinterpret_cast<float4*>(a), make_float4(0.f, 0.f, 0.f, 0.f));
            if (row < L.M) {
                gq[j] = __ldg(reinterpret_cast<const uint2*>(L.g + o));
                if (L.bias != nullptr) bq[j] = __ldg(reinterpret_cast<const uint2*>(L.bias + o));
                if (L.y_op == EPTQ_Y_ADD_RESIDUAL) rq[j] = __ldcg(reinterpret_cast<const uint2*>(L.residual + o));
            }
        }
    }
    long long pos = 0;
    float cs[4] = {1.f, 1.f, 1.f, 1.f}, sn[4] = {0.f, 0.f, 0.f, 0.f};
    if (rope || to_cache) pos = *L.position;
    if (rope) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float sv, cv;
            sincosf(static_cast<float>(pos) * L.inv_freq[(lane & 15) * 4 + c], &sv, &cv);
            cs[c] = __half2float(__float2half_rn(cv * L.rope_scaling));
            sn[c] = __half2float(__float2half_rn(sv * L.rope_scaling));
            if (lane < 16) sn[c] = -sn[c];
        }
    }
    const float r = inv_rms != nullptr ? inv_rms[0] : 1.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int rt16 = rt64 * 4 + j;
        if (rt16 >= L.row_tiles) continue;                 // warp-uniform
        const int row = rt16 * 16 + (lane >> 1);
        const int o = row * 8 + (lane & 1) * 4;
        const float2 g01 = __half22float2(*reinterpret_cast<const __half2*>(&gq[j].x));
        const float2 g23 = __half22float2(*reinterpret_cast<const __half2*>(&gq[j].y));
        const float2 b01 = __half22float2(*reinterpret_cast<const __half2*>(&bq[j].x));
        const float2 b23 = __half22float2(*reinterpret_cast<const __half2*>(&bq[j].y));
        __half2 o01 = __floats2half2_rn(fmaf(s[j].x * r, g01.x, b01.x), fmaf(s[j].y * r, g01.y, b01.y));
        __half2 o23 = __floats2half2_rn(fmaf(s[j].z * r, g23.x, b23.x), fmaf(s[j].w * r, g23.y, b23.y));
        if (rope) {                                        // every row of the tile exists (checked on the host)
            const float2 v01 = __half22float2(o01), v23 = __half22float2(o23);
            const float v[4] = {v01.x, v01.y, v23.x, v23.y};
            float q[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) q[c] = fmaf(v[c], cs[c], __shfl_xor_sync(0xffffffffu, v[c], 16) * sn[c]);
            o01 = __floats2half2_rn(q[0], q[1]);
            o23 = __floats2half2_rn(q[2], q[3]);
        }
        if (row >= L.M) continue;
        __half* dst = L.y + o;
        if (to_cache) {
            dst = L.y + (static_cast<size_t>(rt16) * L.max_len + pos) * 128 + lane * 4;
            if (pos < 0 || pos >= L.max_len) continue;
        }
        if (L.y_op == EPTQ_Y_ADD_RESIDUAL) {
            o01 = __hadd2(*reinterpret_cast<const __half2*>(&rq[j].x), o01);
            o23 = __hadd2(*reinterpret_cast<const __half2*>(&rq[j].y), o23);
        }
        uint2 outv;
        outv.x = *reinterpret_cast<const unsigned*>(&o01);
        outv.y = *reinterpret_cast<const unsigned*>(&o23);
        *reinterpret_cast<uint2*>(dst) = outv;
    }
    if (p.done != nullptr) {                               // one count per 64-row tile in this mode
        __syncwarp();
        if (lane == 0)
            asm volatile("red.release.gpu.global.add.u32 [%0], 1;" :: "l"(p.done + L.phase * 32 + (((L.tile0 >> 2) + rt64) & 31)) : "memory");
    }
}

template <bool CUT> struct CutPointer;
template <> struct CutPointer<true> { static __device__ __forceinline__ const signed char* of(const CutTable<true>& t) { return t.cut; } };
template <> struct CutPointer<false> { static __device__ __forceinline__ const signed char* of(const CutTable<false>&) { return nullptr; } };

template <int MAXL, bool CUT>
__global__ void __launch_bounds__(kStreamThreads, 1) gemv_stream_kernel(const __grid_constant__ StreamArgsT<MAXL, CUT> P) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const GroupArgsT<MAXL>& p = P.g;
    const signed char* const cut = CutPointer<CUT>::of(P.shift);
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const unsigned base = smem_addr(smem_raw);
    if (base != kBase) {                                   // layout assumption broken: refuse, do not touch memory
        if (threadIdx.x == 0) atomicExch(P.status, EPTQ_ERR_LAUNCH);
        return;
    }
    asm volatile("griddepcontrol.launch_dependents;");
    EPTQ_STRACE(56, warp == 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(kFullBar + 8 * s, 1);
            mbar_init(kEmptyBar + 8 * s, kConsumerWarps * 32);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(kRedFull + 8 * b, kConsumerWarps * 32 + (P.use_lists ? kStreamCorrWarps * 32 : 0));
            mbar_init(kRedFree + 8 * b, 32);
        }
        mbar_init(kPrep, kConsumerWarps * 32);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    float* misc = reinterpret_cast<float*>(smem_raw + (kMisc - kBase));

    // Registers: the block starts with 96 per thread (640 threads); the warpgroup of the producer, the
    // finalizer and the correction warps gives up 32 per thread, the four consumer warpgroups take 8 each (the
    // sums match: 128 * 32 = 512 * 8, and an increase waits for registers released inside the block).  The
    // change sits inside each role's own branch (a path that saw both would be held to the lower limit) and is
    // one instruction for the whole fifth warpgroup.
    if (warp >= kProducerWarp) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");

        // ------------------------------------------------------------ producer
        if (warp == kProducerWarp) {
            if (lane == 0) {
                SegmentWalk walk(cut);
                Segment sg;
                int s = 0, issued = 0;
                unsigned ph = 0;
                bool ok = true;
                while (ok && walk.next(p, sg)) {
                    for (int j = 0; j < sg.n; ++j) {
                        if (issued >= kStages && !mbar_wait(kEmptyBar + 8 * s, ph ^ 1u, P.wait_ns)) {
                            atomicExch(P.status, EPTQ_ERR_TIMEOUT);
                            ok = false;
                            break;
                        }
                        mbar_expect_tx(kFullBar + 8 * s, kStageBytes);
                        asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                                     :: "r"(kRing + s * kStageBytes), "l"(&P.maps[sg.l]), "r"(0), "r"(sg.rt * 64), "r"((sg.cc + j) * 2),
                                        "r"(kFullBar + 8 * s)
                                     : "memory");
                        ++issued;
                        if (++s == kStages) { s = 0; ph ^= 1u; }
                    }
                }
            }
            return;
        }

        // ------------------------------------------------------------ finalizer
        // One flush per segment, in order: the consumers leave the int32 sums of the tile in a flush buffer;
        // this warp turns them into floats, adds them to the accumulators in scratch, arrives at the four
        // 16-row tiles with the segment's units as weight and finalizes those it completes.
        if (warp == kFinalizerWarp) {
            SegmentWalk walk(cut);
            Segment sg;
            unsigned k = 0;
            bool waited = false;
            while (walk.next(p, sg)) {
                const GroupLayer& L = p.L[sg.l];
                const unsigned b = k & 1u;
                if (P.use_lists) {
                    // Whichever block completes this 64-row tile finalizes it; its epilogue operands (1 KB each of
                    // output scale, bias and residual) are asked into L2 now, while the segment is still streaming.
                    const size_t line = static_cast<size_t>(sg.rt) * 512 + (lane & 7) * 64;      // halves
                    const __half* src = lane < 8 ? L.g : lane < 16 ? L.bias : lane < 24 && L.y_op == EPTQ_Y_ADD_RESIDUAL ? L.residual : nullptr;
                    if (src != nullptr && line < static_cast<size_t>(L.M) * 8)
                        asm volatile("prefetch.global.L2 [%0];" :: "l"(src + line));
                }
                if (!mbar_wait(kRedFull + 8 * b, (k >> 1) & 1u, P.wait_ns)) {
                    if (lane == 0) atomicExch(P.status, EPTQ_ERR_TIMEOUT);
                    break;
                }
                EPTQ_STRACE(8 * L.phase + 5, true);
                const float scale = __uint_as_float(lds32(kMail + 16 * b + 12));
                if (lane == 0) misc[48] = __uint_as_float(lds32(kMail + 16 * b + 8));       // this layer's RMSNorm factor
                const unsigned buf = kRed + b * 4096;
                // This lane: row lane>>1 of each 16-row tile, dimensions 4*(lane&1)..+3.  The buffer stores
                // dimension d at d ^ 4*((row>>2)&1) ^ digit: the halves of a row swap when bit 2 of the row is
                // set, and the high-digit words are pairwise exchanged.
                // sums of the four 16-row tiles as floats (digits combined, corrections added, scaled): 16 registers
                float4 v[4];
                const unsigned my = static_cast<unsigned>((lane * 4) ^ (((lane >> 3) & 1) << 2));
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 lo = lds128(buf + (j * 128 + my) * 4);
                    const uint4 hsw = lds128(buf + 2048 + (j * 128 + my) * 4);      // words pairwise exchanged
                    float4 cr = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (P.use_lists) {
                        const uint4 c = lds128(kCorr + b * 2048 + (j * 128 + lane * 4) * 4);
                        cr = make_float4(static_cast<float>(static_cast<int>(c.x)) * kCorrStep, static_cast<float>(static_cast<int>(c.y)) * kCorrStep,
                                         static_cast<float>(static_cast<int>(c.z)) * kCorrStep, static_cast<float>(static_cast<int>(c.w)) * kCorrStep);
                    }
                    v[j].x = (fmaf(256.f, static_cast<float>(static_cast<int>(hsw.y)), static_cast<float>(static_cast<int>(lo.x))) + cr.x) * scale;
                    v[j].y = (fmaf(256.f, static_cast<float>(static_cast<int>(hsw.x)), static_cast<float>(static_cast<int>(lo.y))) + cr.y) * scale;
                    v[j].z = (fmaf(256.f, static_cast<float>(static_cast<int>(hsw.w)), static_cast<float>(static_cast<int>(lo.z))) + cr.z) * scale;
                    v[j].w = (fmaf(256.f, static_cast<float>(static_cast<int>(hsw.z)), static_cast<float>(static_cast<int>(lo.w))) + cr.w) * scale;
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    sts128(buf + (j * 128 + lane * 4) * 4, 0u, 0u, 0u, 0u);
                    sts128(buf + 2048 + (j * 128 + lane * 4) * 4, 0u, 0u, 0u, 0u);
                    if (P.use_lists) sts128(kCorr + b * 2048 + (j * 128 + lane * 4) * 4, 0u, 0u, 0u, 0u);
                }
                mbar_arrive(kRedFree + 8 * b);
                if (!waited) { asm volatile("griddepcontrol.wait;" ::: "memory"); waited = true; }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int rt16 = sg.rt * 4 + j;
                    if (rt16 < L.row_tiles)
                        red_add4(p.acc + L.acc_off + static_cast<size_t>(rt16) * p.B * 128 + lane * 4, v[j].x, v[j].y, v[j].z, v[j].w);
                }
                const unsigned weight = static_cast<unsigned>(sg.n);
                const float* inv_rms = L.x_op == EPTQ_X_RMSNORM ? misc + 48 : nullptr;
                __syncwarp();
                if (P.use_lists) {
                    // one arrival for the 64-row tile: complete when all cc128 units of it have arrived
                    unsigned old = 0;
                    if (lane == 0)
                        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;"
                                     : "=r"(old) : "l"(p.counters + L.tile0 + sg.rt * 4), "r"(weight) : "memory");
                    old = __shfl_sync(0xffffffffu, old, 0);
                    EPTQ_STRACE(8 * L.phase + 6, true);
                    if (old + weight == static_cast<unsigned>(L.cc128)) { finalize_tile64(p, L, sg.rt, lane, inv_rms); EPTQ_STRACE(8 * L.phase + 7, true); }
                } else {
                    // one round trip for the four arrivals; with the CSR corrections a 16-row tile is complete at
                    // cc128 units + 4 correction quarters
                    unsigned old = 0;
                    if (lane < 4 && sg.rt * 4 + lane < L.row_tiles)
                        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;"
                                     : "=r"(old) : "l"(p.counters + L.tile0 + sg.rt * 4 + lane), "r"(weight) : "memory");
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const unsigned oj = __shfl_sync(0xffffffffu, old, j);
                        if (sg.rt * 4 + j < L.row_tiles && oj + weight == static_cast<unsigned>(L.cc128) + 4u)
                            finalize_tile(p, L, sg.rt * 4 + j, lane, load_affine(L, sg.rt * 4 + j, lane), inv_rms);
                    }
                }
                ++k;
            }
            launch_exit(p, lane);
            EPTQ_STRACE(57, true);
            return;
        }

        // ------------------------------------------------------------ correction warps
        // What the main loop adds for a marker: entry (class 3, code 127) in both halves.
        const unsigned e511 = pack_coords(__ldg(p.table16 + 511), P.inv_unit);
        const float c0 = static_cast<float>(static_cast<signed char>(e511 & 0xFF)) * P.unit;
        const float c1 = static_cast<float>(static_cast<signed char>((e511 >> 8) & 0xFF)) * P.unit;
        const float c2 = static_cast<float>(static_cast<signed char>((e511 >> 16) & 0xFF)) * P.unit;
        const float c3 = static_cast<float>(static_cast<signed char>(e511 >> 24)) * P.unit;
        if (P.use_lists) {
            // Unit lists: the critical blocks of a segment are one contiguous run of (position, 8 values); the two
            // warps take alternate entries, read the activation digits the consumers prepared and add
            // (O - marker code) / unit * digits to the segment's correction tile, in step with the flushes.
            SegmentWalk walk(cut);
            Segment sg, nxt;
            unsigned k = 0, n_prep = 0;
            bool ok = true;
            const int me = (warp - kFinalizerWarp - 1) * 32 + lane;            // 0..63
            constexpr int kAhead = 4;                                           // entries per lane in flight
            // The entry range of a segment is read one segment ahead, and its first 256 entries before any wait:
            // a short segment's corrections are then one memory round trip behind its start, not three.
            auto range_of = [&](const Segment& g, int& a, int& b) {
                const GroupLayer& G = p.L[g.l];
                const int u0 = g.rt * G.cc128 + g.cc;
                a = __ldg(G.crit_ptr + u0);
                b = __ldg(G.crit_ptr + u0 + g.n);
            };
            bool have = walk.next(p, sg);
            int e0 = 0, e1 = 0;
            if (have) range_of(sg, e0, e1);
            while (have) {
                const GroupLayer& L = p.L[sg.l];
                unsigned pos[kAhead];
                uint4 ov[kAhead];
#pragma unroll
                for (int j = 0; j < kAhead; ++j) {
                    const int e = e0 + me + 64 * j;
                    pos[j] = 0u; ov[j] = make_uint4(0, 0, 0, 0);
                    if (e < e1) { pos[j] = __ldg(L.crit_pos + e); ov[j] = ldg128(L.crit_O + static_cast<size_t>(e) * 8); }
                }
                const bool have_next = walk.next(p, nxt);
                int n0 = 0, n1 = 0;
                if (have_next) range_of(nxt, n0, n1);
                if (sg.new_layer) {
                    if (ok) ok = mbar_wait(kPrep, n_prep & 1u, P.wait_ns);
                    ++n_prep;
                }
                const unsigned b = k & 1u;
                if (k >= 2u && ok) ok = mbar_wait(kRedFree + 8 * b, ((k >> 1) - 1u) & 1u, P.wait_ns);
                const unsigned tile = kCorr + b * 2048;
                auto apply = [&](unsigned ps, const uint4& o) {
                    const unsigned col = ps & 0xFFFFu, row = ps >> 16;
                    short dl, dh;
                    asm volatile("ld.shared.s8 %0, [%1];" : "=h"(dl) : "r"(kPlane + col));
                    asm volatile("ld.shared.s8 %0, [%1];" : "=h"(dh) : "r"(kPlane + kStreamMaxN + col));
                    const float f = static_cast<float>(static_cast<int>(dl) + 256 * static_cast<int>(dh)) * (P.inv_unit / kCorrStep);
                    float o8[8];
                    unpack8(o, o8);
                    const float cm[4] = {c0, c1, c2, c3};
                    // integer adds (shared-memory float adds are compare-and-swap loops); the sums of a row stay
                    // below 2^31 by the precondition on the lists (sum |O - code| / unit < 3900 per row)
#pragma unroll
                    for (int d = 0; d < 8; ++d)
                        asm volatile("red.shared.add.s32 [%0], %1;" :: "r"(tile + (row * 8 + d) * 4),
                                     "r"(__float2int_rn((o8[d] - cm[d & 3]) * f)) : "memory");
                };
                EPTQ_STRACE_MAX(48 + 2 * L.phase);
#pragma unroll
                for (int j = 0; j < kAhead; ++j)
                    if (e0 + me + 64 * j < e1) apply(pos[j], ov[j]);
                EPTQ_STRACE_MAX(49 + 2 * L.phase);
                for (int base = e0 + 64 * kAhead; base < e1; base += 64 * kAhead) {        // long segments: batches of 256
#pragma unroll
                    for (int j = 0; j < kAhead; ++j) {
                        const int e = base + me + 64 * j;
                        if (e < e1) { pos[j] = __ldg(L.crit_pos + e); ov[j] = ldg128(L.crit_O + static_cast<size_t>(e) * 8); }
                    }
#pragma unroll
                    for (int j = 0; j < kAhead; ++j)
                        if (base + me + 64 * j < e1) apply(pos[j], ov[j]);
                }
                mbar_arrive(kRedFull + 8 * b);
                EPTQ_STRACE_MAX(32 + 4 * L.phase + 3);
                ++k;
                sg = nxt; e0 = n0; e1 = n1; have = have_next;
            }
            if (!ok && lane == 0) atomicExch(P.status, EPTQ_ERR_TIMEOUT);
            launch_exit(p, lane);
            return;
        }
        {
            bool dep_waited = false;
            int waited_phase = 0;
            bool ok = true;
            const int cw = blockIdx.x * kStreamCorrWarps + (warp - kFinalizerWarp - 1);
            int l = 0;
            for (int u = cw; u < p.corr_units; u += p.n_corr_warps) {
                while (l + 1 < p.n_layers && p.L[l + 1].corr0 <= u) ++l;
                const GroupLayer& L = p.L[l];
                stream_correction_unit(p, L, u - L.corr0, lane, c0, c1, c2, c3, misc + 49 + (warp - kFinalizerWarp), [&]() {
                    if (!dep_waited) { asm volatile("griddepcontrol.wait;" ::: "memory"); dep_waited = true; }
                    if (L.phase > waited_phase && ok) {
                        ok = wait_phase(p, L.phase, L.wait_tiles, P.wait_ns);
                        waited_phase = L.phase;
                    }
                });
            }
            if (!ok && lane == 0) atomicExch(P.status, EPTQ_ERR_TIMEOUT);
            launch_exit(p, lane);
            return;
        }
    }

    // ---------------------------------------------------------------- consumers
    asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
    const int tid = threadIdx.x;                            // 0..511
    // Table, one copy per lane: entry e (raw index bits: true (class, code) ^ 0x100) of lane l at kTable + 128 e + 4 l.
    {
        const unsigned v = pack_coords(__ldg(p.table16 + (tid ^ 0x100)), P.inv_unit);
#pragma unroll
        for (int c = 0; c < 8; ++c) sts128(kTable + tid * 128 + ((c + tid) & 7) * 16, v, v, v, v);
    }
    for (int i = tid; i < 2048 + 1024; i += kConsumerWarps * 32) sts32(kRed + 4 * i, 0u);      // flush and correction tiles

    const int g = lane >> 2, t = lane & 3;
    const int chunk64 = warp >> 3, w8 = warp & 7;
    const unsigned lane_tab = static_cast<unsigned>(lane * 4) | kTable;
    const unsigned dsel = g & 3, psel = g >> 2;
    // B fragment: the digit of plane psel goes to byte dsel (dimension), zeros elsewhere (PRMT index 4 = 0 byte).
    const unsigned sel0 = 0x4444u ^ (0x4u << (4 * dsel));
    const unsigned sel1 = 0x4444u ^ (0x5u << (4 * dsel));
    const unsigned plane = kPlane + psel * kStreamMaxN + 8 * warp + 2 * t;
    // ldmatrix row address of this lane inside a stage: matrix lane>>3 = row group, row lane&7, 128-byte swizzle.
    const unsigned qm = kRing + static_cast<unsigned>(chunk64 * 8192 + ((lane >> 3) * 8 + (lane & 7)) * 128 + ((w8 ^ (lane & 7)) << 4));

    const unsigned zr = P.zero, m128 = P.mul[0], m64k = P.mul[1];
    bool ok = true;
    bool dep_waited = false;
    unsigned flush_no = 0, prep_no = 0;

    // Digit planes (and the fused RMSNorm factor) of layer l.  Four chunks of 8 columns per thread stay in
    // registers between the maximum and the split into digits; longer rows reload the rest.  All loads of the
    // four chunks are issued before the first use, the column scales (weights) before the wait for the phase.
    auto prepare_layer = [&](int l) {
        const GroupLayer& L = p.L[l];
        constexpr int kStride = kConsumerWarps * 32 * 8;
        uint4 hr[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int c = tid * 8 + k * kStride;
            hr[k] = make_uint4(0, 0, 0, 0);
            if (c < L.N) hr[k] = ldg128(L.h + c);
        }
        if (!dep_waited) { asm volatile("griddepcontrol.wait;" ::: "memory"); dep_waited = true; EPTQ_STRACE(58, warp == 0); }
        if (P.use_lists && flush_no > 0u && ok) {            // the correction warps still read the previous layer's planes
            const unsigned kf = flush_no - 1u;
            ok = mbar_wait(kRedFull + 8 * (kf & 1u), (kf >> 1) & 1u, P.wait_ns);
        }
        if (L.phase > 0) {                                   // input written by the previous phase of this launch
            EPTQ_STRACE(8 * L.phase + 0, warp == 0);
            if (warp == 0 && ok && !wait_phase(p, L.phase, L.wait_tiles, P.wait_ns) && lane == 0) misc[47] = 1.f;
            EPTQ_STRACE(8 * L.phase + 1, warp == 0);
            consumer_barrier();
            if (misc[47] != 0.f) ok = false;
        }
        uint4 xr[4], ur[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int c = tid * 8 + k * kStride;
            xr[k] = make_uint4(0, 0, 0, 0); ur[k] = make_uint4(0, 0, 0, 0);
            if (c < L.N) {
                xr[k] = __ldcg(reinterpret_cast<const uint4*>(L.x + c));
                if (L.x_op == EPTQ_X_SILU_MUL) ur[k] = __ldcg(reinterpret_cast<const uint4*>(L.x_aux + c));
            }
        }
        float xh[4][8];
        float mx = 0.f, ss = 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float hv[8];
            unpack8(xr[k], xh[k]);
            unpack8(hr[k], hv);
            if (L.x_op == EPTQ_X_SILU_MUL && tid * 8 + k * kStride < L.N) {
                float u[8];
                unpack8(ur[k], u);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float sv = __half2float(__float2half_rn(__fdividef(xh[k][e], 1.f + __expf(-xh[k][e]))));
                    xh[k][e] = __half2float(__float2half_rn(sv * u[e]));
                }
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                ss = fmaf(xh[k][e], xh[k][e], ss);
                xh[k][e] *= hv[e];                           // zero beyond N: both factors were zero-filled
                mx = fmaxf(mx, fabsf(xh[k][e]));
            }
        }
        for (int c = tid * 8 + 4 * kStride; c < L.N; c += kStride) {
            float xv[8], hv[8];
            activations8(L, c, xv);
            unpack8(ldg128(L.h + c), hv);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                mx = fmaxf(mx, fabsf(xv[e] * hv[e]));
                ss = fmaf(xv[e], xv[e], ss);
            }
        }
        EPTQ_STRACE(32 + 4 * L.phase + 0, warp == 0);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            ss += __shfl_xor_sync(0xffffffffu, ss, o);
        }
        // misc[0..31] alternate with the layer count, so that this layer's partial results do not meet the
        // previous layer's readers: one barrier less.
        float* part = misc + 64 + (prep_no & 1u) * 32;
        ++prep_no;
        if (lane == 0) { part[warp] = mx; part[16 + warp] = ss; }
        consumer_barrier();                                 // also: the previous layer's readers of the planes are done
        EPTQ_STRACE(32 + 4 * L.phase + 1, warp == 0);
        // lanes 0..15 hold the warps' maxima, lanes 16..31 their sums of squares
        float vmax = part[lane], vsum = vmax;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
            vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
            vsum += __shfl_xor_sync(0xffffffffu, vsum, o);
        }
        mx = __shfl_sync(0xffffffffu, vmax, 0);
        const float tot = __shfl_sync(0xffffffffu, vsum, 16);
        const float S = mx > 0.f ? __fdividef(32000.f, mx) : 1.f;
        if (tid == 0) {                                      // read back by thread 0 at each flush of this layer
            misc[56] = L.x_op == EPTQ_X_RMSNORM ? rsqrtf(tot / static_cast<float>(L.N) + L.norm_eps) : 1.f;
            misc[57] = P.unit / S;
        }
        const int n_pad = L.cc128 * 128;
        auto digits = [&](int c, const float (&v)[8]) {
            unsigned lo[2] = {0u, 0u}, hi[2] = {0u, 0u};
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int q16 = __float2int_rn(v[e] * S);
                const int h8 = (q16 + 128) >> 8, l8 = q16 - (h8 << 8);
                lo[e >> 2] |= (static_cast<unsigned>(l8) & 0xFFu) << (8 * (e & 3));
                hi[e >> 2] |= (static_cast<unsigned>(h8) & 0xFFu) << (8 * (e & 3));
            }
            sts64(kPlane + c, lo[0], lo[1]);
            sts64(kPlane + kStreamMaxN + c, hi[0], hi[1]);
        };
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int c = tid * 8 + k * kStride;
            if (c < n_pad) digits(c, xh[k]);                 // zeros beyond N
        }
        for (int c = tid * 8 + 4 * kStride; c < n_pad; c += kStride) {
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = 0.f;
            if (c < L.N) {
                float hv[8];
                activations8(L, c, v);
                unpack8(ldg128(L.h + c), hv);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] *= hv[e];
            }
            digits(c, v);
        }
        consumer_barrier();
        EPTQ_STRACE(8 * L.phase + 2, warp == 0);
        if (P.use_lists) mbar_arrive(kPrep);                 // release: the planes are visible to the correction warps
    };

    int acc[8][4];
#pragma unroll
    for (int r = 0; r < 8; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[r][c] = 0;

    // End of a segment: leave the sums in a flush buffer for the finalizer warp.
    auto flush = [&]() {
        const unsigned b = flush_no & 1u;
        if (flush_no >= 2u && ok) ok = mbar_wait(kRedFree + 8 * b, ((flush_no >> 1) - 1u) & 1u, P.wait_ns);
        // Word of (digit p, row, dimension d): p*512 + row*8 + (d ^ 4*((row>>2)&1) ^ p); the swizzle spreads the
        // 32 lanes of one instruction (8 rows g, digit t>>1, dimension pair t&1) over the 32 banks.
        const unsigned mine = kRed + b * 4096 + static_cast<unsigned>(((t >> 1) * 512 + g * 8) * 4);
        const unsigned sw = static_cast<unsigned>(((g >> 2) << 2) ^ (t >> 1));
#pragma unroll
        for (int r = 0; r < 8; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const unsigned d = static_cast<unsigned>((c >> 1) * 4 + 2 * (t & 1) + (c & 1)) ^ sw;
                asm volatile("red.shared.add.s32 [%0], %1;" :: "r"(mine + (r * 64 + d) * 4), "r"(acc[r][c]) : "memory");
                acc[r][c] = 0;
            }
        if (tid == 0) {
            sts32(kMail + 16 * b + 8, __float_as_uint(misc[56]));
            sts32(kMail + 16 * b + 12, __float_as_uint(misc[57]));
        }
        mbar_arrive(kRedFull + 8 * b);
        ++flush_no;
    };

    if (tid == 0) misc[47] = 0.f;
    const int n_units = block_units(p, cut);
    SegmentWalk walk(cut);
    Segment sg;
    unsigned q[8];
    unsigned ph = 0;
    int s = 0, i = 0;
    bool first = true;
    // One body for all stages (an unrolled ring would repeat the flush and the layer switch six times and no
    // longer fit the instruction cache).
    while (walk.next(p, sg)) {
        if (sg.new_layer) prepare_layer(sg.l);               // its barriers also publish the table and the zeroed buffers
        if (first) {
            first = false;
            ok = ok && mbar_wait(kFullBar, 0u, P.wait_ns);
            ldsm4(qm, q[0], q[1], q[2], q[3]);
            ldsm4(qm + 4096, q[4], q[5], q[6], q[7]);
        }
        unsigned plane_c = plane + sg.cc * 128;
        for (int j = 0; j < sg.n; ++j) {
            // Two halves of four row groups: the second half's lookups are in flight while the first half's
            // products issue (16 registers of table words instead of 32).
            unsigned a[4][4];
            auto lookups = [&](int half) {
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const unsigned qq = q[4 * half + r];
                    // high index of the word: the upper half of the 64-bit product q * 2^16
                    unsigned ta, tb;
                    unsigned long long wide;
                    asm("mul.wide.u32 %0, %1, %2;" : "=l"(wide) : "r"(qq), "r"(m64k));
                    const unsigned qs = static_cast<unsigned>(wide >> 32);
                    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(ta) : "r"(qq), "r"(m128), "r"(zr));
                    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(tb) : "r"(qs), "r"(m128), "r"(zr));
                    const unsigned ia = (qq & 0xFF80u) | lane_tab;
                    const unsigned ib = (qs & 0xFF80u) | lane_tab;
                    a[r][0] = lds32(ia);
                    a[r][1] = lds32(bitsel(ta, ia, 0x3F80u));
                    a[r][2] = lds32(ib);
                    a[r][3] = lds32(bitsel(tb, ib, 0x3F80u));
                }
            };
            const unsigned pv = lds16(plane_c);
            const unsigned b0 = prmt(pv, 0u, sel0), b1 = prmt(pv, 0u, sel1);
            plane_c += 128;
            lookups(0);
#pragma unroll
            for (int r = 0; r < 4; ++r) imma(acc[r], a[r][0], a[r][1], a[r][2], a[r][3], b0, b1);
            lookups(1);
            mbar_arrive(kEmptyBar + 8 * s);                 // every lane: its indices are in registers
            ++i;
            if (++s == kStages) { s = 0; ph ^= 1u; }
            if (i < n_units) {                              // the next unit of the block, whatever segment it is in
                if (ok) ok = mbar_wait(kFullBar + 8 * s, ph, P.wait_ns);
                const unsigned stage = qm + s * kStageBytes;
                ldsm4(stage, q[0], q[1], q[2], q[3]);
                ldsm4(stage + 4096, q[4], q[5], q[6], q[7]);
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) imma(acc[4 + r], a[r][0], a[r][1], a[r][2], a[r][3], b0, b1);
        }
        EPTQ_STRACE(8 * p.L[sg.l].phase + 3, warp == 0);
        flush();
        EPTQ_STRACE(8 * p.L[sg.l].phase + 4, warp == 0);
        EPTQ_STRACE_MAX(32 + 4 * p.L[sg.l].phase + 2);
    }
    if (!ok && lane == 0) atomicExch(P.status, EPTQ_ERR_TIMEOUT);
}

// ------------------------------------------------------------------------------------------------ host

PFN_cuTensorMapEncodeTiled_v12000 stream_map_encoder() {
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

// Tensor map over Q seen as (64 columns, M rows, N/64 column chunks): one load brings 64 rows x two chunks.
bool encode_q_map(const int16_t* Q, int M, int N, CUtensorMap* out) {
    const cuuint64_t dims[3] = {64, static_cast<cuuint64_t>(M), static_cast<cuuint64_t>(N / 64)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(N) * 2, 128};
    const cuuint32_t box[3] = {64, 64, 2};
    const cuuint32_t estr[3] = {1, 1, 1};
    return stream_map_encoder()(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<int16_t*>(Q), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct MapKey {
    const void* q; int m, n;
    bool operator==(const MapKey& o) const { return q == o.q && m == o.m && n == o.n; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.q) ^ (static_cast<size_t>(k.m) * 0x9E3779B97F4A7C15ull) ^ (static_cast<size_t>(k.n) << 32);
    }
};

int stream_sm_count() {
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

bool stream_layer_supported(const EptqLayer& L) {
    return L.quantizer == EPTQ_E8D4 && L.S_group == nullptr && L.M > 0 && L.N > 0 && (L.N % 64) == 0 &&
           L.N <= kStreamMaxN && L.table8 != nullptr && L.table8_scale > 0.f && L.table16 != nullptr &&
           aligned16(L.table16) && L.Q != nullptr && L.g != nullptr &&
           L.h != nullptr && L.O_row_ptr != nullptr && (L.n_masked == 0 || (L.O_vals != nullptr && L.O_col != nullptr)) &&
           aligned16(L.Q) && aligned16(L.g) && aligned16(L.h) && (L.bias == nullptr || aligned16(L.bias)) &&
           (L.n_masked == 0 || aligned16(L.O_vals));
}

}  // namespace

bool stream_gemv_supported(const EptqLayer* layers, int n, int B) {
    if (layers == nullptr || n < 1 || n > kMaxGroupLayers || B != 1 || stream_map_encoder() == nullptr) return false;
    int tiles = 0;
    long long units = 0;
    for (int i = 0; i < n; ++i) {
        if (!stream_layer_supported(layers[i])) return false;
        if (layers[i].table16 != layers[0].table16 || layers[i].table8_scale != layers[0].table8_scale) return false;
        tiles += (layers[i].M + 15) / 16;
        units += static_cast<long long>((layers[i].M + 63) / 64) * ((layers[i].N + 127) / 128);
    }
    if (tiles > kMaxCounters - 1) return false;
    if (static_cast<size_t>(tiles) * B * 128 * sizeof(float) > kPartialOffset - kCounterBytes) return false;
    return units * 1024 < (1LL << 32);                     // owner arithmetic in 32 bits (blocks <= 1024)
}

// `phases` (or null: one phase): phase of each layer, non-decreasing from 0.  Layers of phase k+1 may read
// what phase k wrote (the kernel waits for the tiles of all earlier phases before it reads their inputs); with
// more than one phase the launch is cooperative, so that every block is resident while others wait for it.
// Work split of a one-phase launch of several layers.  A block that goes on from one layer into the next prepares
// the next layer's input in between, which costs about kSwitchUnits units of streaming; its share is that much
// shorter, and a share that would end just behind a layer's first units ends at the layer's edge instead.
// starts: first unit of each layer (ascending, starts[0] == 0); cut[b] .. cut[b + 1] is block b's range.
constexpr int kSwitchUnits = 3;
void balanced_cut(const int* starts, int n_layers, int units, int blocks, int* cut) {
    int pos = 0;
    for (int b = 0; b < blocks; ++b) {
        cut[b] = pos;
        if (b == blocks - 1) { pos = units; break; }
        int inner = 0;                                        // layer edges strictly inside what is left
        for (int l = 1; l < n_layers; ++l) if (starts[l] > pos && starts[l] < units) ++inner;
        const double target = (static_cast<double>(units - pos) + kSwitchUnits * inner) / (blocks - b);
        double cost = 0.0;
        while (pos < units) {
            int edge = units;                                 // next layer edge behind pos
            for (int l = 1; l < n_layers; ++l) if (starts[l] > pos) { edge = starts[l]; break; }
            const int room = static_cast<int>(target - cost + 0.5);
            if (room <= 0) break;
            const int take = room < edge - pos ? room : edge - pos;
            pos += take;
            cost += take;
            if (pos == edge && pos < units) {                 // at an edge: go on only if the switch and a unit fit
                if (cost + kSwitchUnits + 1 > target) break;
                cost += kSwitchUnits;
            }
        }
        if (pos == cut[b] && pos < units) ++pos;              // never an empty share while work is left
    }
    for (int b = blocks; b <= kMaxCutBlocks; ++b) cut[b] = units;
    cut[blocks] = units;
}

// The first n layers (n <= kSmallGroup; phases never outnumber layers) into the small parameter block.
template <bool CUT>
void shrink_args(const StreamArgs& a, StreamArgsT<kSmallGroup, CUT>& s, int n) {
    for (int i = 0; i < kSmallGroup; ++i) {
        s.g.L[i] = a.g.L[i < n ? i : 0];
        s.g.phase_unit0[i] = a.g.phase_unit0[i];
        s.g.phase_units[i] = a.g.phase_units[i];
        s.maps[i] = a.maps[i < n ? i : 0];
    }
    s.g.table16 = a.g.table16; s.g.packed = a.g.packed; s.g.acc = a.g.acc; s.g.counters = a.g.counters;
    s.g.W = a.g.W; s.g.n_layers = a.g.n_layers; s.g.B = a.g.B; s.g.nw = a.g.nw;
    s.g.corr_units = a.g.corr_units; s.g.n_corr_warps = a.g.n_corr_warps;
    s.g.x_norm = a.g.x_norm; s.g.norm_eps = a.g.norm_eps;
    s.g.n_phases = a.g.n_phases; s.g.total_tiles = a.g.total_tiles; s.g.done = a.g.done;
    s.unit = a.unit; s.inv_unit = a.inv_unit; s.zero = a.zero; s.mul[0] = a.mul[0]; s.mul[1] = a.mul[1];
    s.use_lists = a.use_lists; s.status = a.status; s.wait_ns = a.wait_ns;
}

int launch_gemv_stream(const EptqLayer* layers, int n, const EptqFusion* fusions, const int* phases,
                       const uint16_t* const* xs, uint16_t* const* ys, int B, void* workspace, size_t workspace_bytes,
                       cudaStream_t stream) {
    if (!stream_gemv_supported(layers, n, B)) return EPTQ_ERR_UNSUPPORTED;
    if (workspace == nullptr || workspace_bytes < kPartialOffset) return EPTQ_ERR_WORKSPACE;
    const int n_sms = stream_sm_count();
    if (n_sms < 1) return EPTQ_ERR_LAUNCH;

    static StreamArgs args;                    // large: keep it off the stack; filled under a lock
    static std::mutex args_mutex;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> maps;
    std::lock_guard<std::mutex> lock(args_mutex);
    StreamArgs& a = args;
    a.use_lists = 1;
    for (int i = 0; i < n; ++i)
        if (layers[i].crit_ptr == nullptr || (layers[i].n_masked != 0 && (layers[i].crit_pos == nullptr || layers[i].crit_O == nullptr)) ||
            (layers[i].crit_O != nullptr && !aligned16(layers[i].crit_O)))
            a.use_lists = 0;
    {
        const int st = fill_group_args(a.g, layers, n, fusions, xs, ys, B, workspace, phases, a.use_lists != 0);
        if (st != EPTQ_OK) return st;
    }
    for (int i = 0; i < n; ++i) if (!aligned16(xs[i])) return EPTQ_ERR_ALIGN;
    const bool chained = a.g.n_phases > 1;
    if (chained) {
        // phase counters: the last 8 KB below the partial-sum region (the accumulators end far below it)
        if (static_cast<size_t>(a.g.total_tiles) * B * 128 * sizeof(float) > kPartialOffset - kCounterBytes - 8192)
            return EPTQ_ERR_UNSUPPORTED;
        a.g.done = reinterpret_cast<unsigned*>(reinterpret_cast<char*>(workspace) + kPartialOffset - 8192);
    }
    long long units = 0;
    int corr_units = 0;
    for (int i = 0; i < n; ++i) {
        units += static_cast<long long>(a.g.L[i].rt64) * a.g.L[i].cc128;
        corr_units += a.g.L[i].row_tiles * 4;
        const MapKey key{layers[i].Q, layers[i].M, layers[i].N};
        auto it = maps.find(key);
        if (it == maps.end()) {
            CUtensorMap m;
            if (!encode_q_map(layers[i].Q, layers[i].M, layers[i].N, &m)) return EPTQ_ERR_LAUNCH;
            if (maps.size() > 8192) maps.clear();
            it = maps.emplace(key, m).first;
        }
        a.maps[i] = it->second;
    }
    // the kernel cuts shares with 32-bit products units * blocks
    if (units * n_sms >= (1ll << 32)) return EPTQ_ERR_UNSUPPORTED;
    // Every phase is split over all blocks; a phase with fewer units than blocks leaves some without work in it.
    const int blocks = chained ? n_sms : (units < n_sms ? static_cast<int>(units) : n_sms);
    if (!chained) a.g.phase_units[0] = static_cast<int>(units);
    // Long shares of several layers: shifts of the even split (see CutTable); small enough to be int8 by construction.
    static StreamArgsT<kSmallGroup, true> cut_args;          // guarded by args_mutex
    bool use_cut = false;
    if (!chained && n >= 4 && n <= kSmallGroup && blocks <= kMaxCutBlocks && units >= 8ll * blocks) {
        int starts[kMaxGroupLayers], cut[kMaxCutBlocks + 1];
        for (int i = 0; i < n; ++i) starts[i] = a.g.L[i].unit0;
        balanced_cut(starts, n, static_cast<int>(units), blocks, cut);
        use_cut = true;
        for (int b = 0; b <= kMaxCutBlocks; ++b) {
            const long long even = b <= blocks ? units * b / blocks : units;
            const long long d = (b <= blocks ? cut[b] : static_cast<int>(units)) - even;
            if (d < -127 || d > 127) use_cut = false;
            cut_args.shift.cut[b] = static_cast<signed char>(b <= blocks ? d : 0);
        }
    }
    a.g.W = units;
    a.g.nw = blocks;
    a.g.corr_units = corr_units;
    a.g.n_corr_warps = blocks * kStreamCorrWarps;
    a.unit = layers[0].table8_scale;
    a.inv_unit = 1.0f / layers[0].table8_scale;
    a.status = reinterpret_cast<int*>(workspace) + (kMaxCounters - 1);
    a.zero = 0u;
    a.mul[0] = 128u; a.mul[1] = 1u << 16;
    a.wait_ns = 2000000000ull;

    static bool attr_done[64] = {};            // guarded by args_mutex
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return EPTQ_ERR_LAUNCH;
    if (!attr_done[dev]) {
        if (cudaFuncSetAttribute(gemv_stream_kernel<kMaxGroupLayers, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamSmemBytes) != cudaSuccess ||
            cudaFuncSetAttribute(gemv_stream_kernel<kSmallGroup, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamSmemBytes) != cudaSuccess ||
            cudaFuncSetAttribute(gemv_stream_kernel<kSmallGroup, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamSmemBytes) != cudaSuccess)
            return EPTQ_ERR_LAUNCH;
        attr_done[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(kStreamThreads);
    cfg.dynamicSmemBytes = kStreamSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (chained) {
        attr[0].id = cudaLaunchAttributeCooperative;
        attr[0].val.cooperative = 1;
    } else {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
    }
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t err;
    if (use_cut) {
        shrink_args(a, cut_args, n);
        err = cudaLaunchKernelEx(&cfg, gemv_stream_kernel<kSmallGroup, true>, cut_args);
    } else if (n <= kSmallGroup) {
        static StreamArgsT<kSmallGroup, false> small_args;     // guarded by args_mutex
        shrink_args(a, small_args, n);
        err = cudaLaunchKernelEx(&cfg, gemv_stream_kernel<kSmallGroup, false>, small_args);
    } else {
        err = cudaLaunchKernelEx(&cfg, gemv_stream_kernel<kMaxGroupLayers, false>, a);
    }
    count_launch(EPTQ_KERNEL_GEMV_STREAM);
    return err == cudaSuccess ? EPTQ_OK : EPTQ_ERR_LAUNCH;
}

}  // namespace eptq

#ifdef EPTQ_STREAM_TRACE
extern "C" int eptq_debug_set_stream_trace(unsigned long long* device_buffer) {
    return cudaMemcpyToSymbol(eptq::g_stream_trace, &device_buffer, sizeof(device_buffer)) == cudaSuccess ? 0 : 6;
}
#endif
