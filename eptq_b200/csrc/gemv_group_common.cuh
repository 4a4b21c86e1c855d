// Pieces shared by the persistent decode GEMVs (gemv_group.cu, gemv_stream.cu): the launch description,
// the fp32 accumulators in scratch with their arrival counters, the finalizing epilogue (g, bias, fused
// RMSNorm factor, residual add, rotary embedding, key/value cache stores) and the critical-block correction.
#pragma once

#include <cmath>

#include "common.cuh"

namespace eptq {

constexpr int kMaxGroupLayers = 32;
constexpr int kMaxCutBlocks = 160;           // blocks a host-made work split may name (streaming kernel, one phase)

struct GroupLayer {
    const int16_t* Q;
    const __half* g;
    const __half* h;
    const __half* x;
    const __half* O_vals;
    const int* O_col;
    const int* O_row_ptr;
    const __half* bias;
    __half* y;
    long long strip0;       // index of this layer's first strip in the global sequence
    long long acc_off;      // float offset of this layer's accumulators: [row tile][batch][128]
    int M, N;
    int ns;                 // strips per row tile = N / 32
    int row_tiles;          // ceil(M / 16)
    int tile0;              // index of this layer's first row tile (counters)
    int corr0;              // index of this layer's first correction unit (4 Q rows each)
    float x_scale;          // power of two, <= 1 / max|h|
    float x_inv_scale;
    // streaming kernel (gemv_stream.cu): units of 64 Q rows x 128 columns, row tile after row tile
    int unit0;              // index of this layer's first unit in the global sequence
    int rt64;               // ceil(M / 64)
    int cc128;              // ceil(N / 128)
    // chained launches (gemv_stream.cu): layers of a later phase read what earlier phases wrote
    int phase;
    int wait_tiles;         // tiles of the previous phase: x may be read once that many of them are finalized
                            // (16-row tiles, or 64-row tiles when the launch patches critical blocks from unit lists)
    int x_op;               // EPTQ_X_PLAIN, EPTQ_X_RMSNORM or EPTQ_X_SILU_MUL
    float norm_eps;
    const __half* x_aux;    // EPTQ_X_SILU_MUL: x = silu(x) * x_aux
    const int* crit_ptr;    // critical blocks per 64 x 128 unit (EptqLayer.crit_*), or null
    const unsigned* crit_pos;
    const __half* crit_O;
    // fused epilogue (EptqFusion): what the finalizing warp does with a finished row tile
    const __half* residual;     // EPTQ_Y_ADD_RESIDUAL
    const long long* position;  // rotary angle / cache row (device scalar)
    const float* inv_freq;      // 64 inverse frequencies
    int y_op;
    int max_len;
    float rope_scaling;
};

// MAXL: capacity of the layer table.  Kernel parameters are copied at every launch, so launches of a few layers
// use a small instantiation (half a microsecond per launch between 11 KB and 3 KB of parameters).
template <int MAXL>
struct GroupArgsT {
    GroupLayer L[MAXL];
    const uint2* table16;     // E8-D4: fp16 (512, 4)
    const unsigned* packed;   // E8: 65536 packed entries (see e8_decode)
    float* acc;             // zero on entry, zero again on exit
    unsigned* counters;
    long long W;            // total strips
    int n_layers;
    int B;
    int nw;                 // total main warps
    int corr_units;         // total correction units
    int n_corr_warps;
    int x_norm;             // EPTQ_X_RMSNORM on every layer, all reading one x: outputs are scaled by rsqrt(mean(x^2) + eps)
    float norm_eps;
    // phases of a chained launch: units and row tiles per phase, completion counter
    int n_phases;
    int total_tiles;
    unsigned* done;         // [phase][32] row tiles finalized in this launch, then one word of finished blocks; the
                            // last block to finish puts the zeros back.  Null when the launch has one phase.
    int phase_unit0[MAXL];
    int phase_units[MAXL];
};
using GroupArgs = GroupArgsT<kMaxGroupLayers>;

namespace groupdev {

__device__ __forceinline__ unsigned smem_addr(const void* p) {
    return static_cast<unsigned>(__cvta_generic_to_shared(p));
}
// Warp that owns global strip s when warp w owns [w*W/nw, (w+1)*W/nw).
// The host keeps W * nw below 2^32, so unsigned 32-bit arithmetic is exact.
__device__ __forceinline__ int owner_warp(long long s64, long long W64, int nw) {
    const unsigned s = static_cast<unsigned>(s64), W = static_cast<unsigned>(W64), n = static_cast<unsigned>(nw);
    unsigned w = (s * n) / W;
    while (w + 1 < n && ((w + 1) * W) / n <= s) ++w;
    while (w > 0 && (w * W) / n > s) --w;
    return static_cast<int>(w);
}
__device__ __forceinline__ void red_add4(float* p, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" :: "l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

struct Affine { float g[4]; float b[4]; };

__device__ __forceinline__ Affine load_affine(const GroupLayer& L, int rt, int lane) {
    Affine a;
#pragma unroll
    for (int i = 0; i < 4; ++i) { a.g[i] = 0.f; a.b[i] = 0.f; }
    const int row = rt * 16 + (lane >> 1);
    if (row < L.M) {
        const int o = row * 8 + (lane & 1) * 4;
        const uint2 graw = __ldg(reinterpret_cast<const uint2*>(L.g + o));
        const float2 g01 = __half22float2(*reinterpret_cast<const __half2*>(&graw.x));
        const float2 g23 = __half22float2(*reinterpret_cast<const __half2*>(&graw.y));
        a.g[0] = g01.x; a.g[1] = g01.y; a.g[2] = g23.x; a.g[3] = g23.y;
        if (L.bias != nullptr) {
            const uint2 braw = __ldg(reinterpret_cast<const uint2*>(L.bias + o));
            const float2 b01 = __half22float2(*reinterpret_cast<const __half2*>(&braw.x));
            const float2 b23 = __half22float2(*reinterpret_cast<const __half2*>(&braw.y));
            a.b[0] = b01.x; a.b[1] = b01.y; a.b[2] = b23.x; a.b[3] = b23.y;
        }
    }
    return a;
}

// The warp that took the last ticket of row tile rt: reads the tile's accumulators, puts the zeros (and the
// counter) back for the next launch, applies g, bias and the fused epilogue, writes y.
template <class GA>
__device__ __forceinline__ void finalize_tile(const GA& p, const GroupLayer& L, int rt, int lane,
                                              const Affine& aff, const float* inv_rms) {
    if (lane == 0) p.counters[L.tile0 + rt] = 0u;
    __syncwarp();      // lane 0's acquire (its ticket), then the warp barrier: every lane sees the other warps' adds
    const int row = rt * 16 + (lane >> 1);
    const int o = row * 8 + (lane & 1) * 4;
    const bool rope = L.y_op == EPTQ_Y_ROPE || L.y_op == EPTQ_Y_ROPE_TO_CACHE;
    const bool to_cache = L.y_op == EPTQ_Y_ROPE_TO_CACHE || L.y_op == EPTQ_Y_TO_CACHE;
    long long pos = 0;
    float cs[4] = {1.f, 1.f, 1.f, 1.f}, sn[4] = {0.f, 0.f, 0.f, 0.f};
    if (rope || to_cache) pos = *L.position;
    if (rope) {
        // A row tile is one head of 128: this lane holds dimensions 4*lane .. 4*lane+3, the rotation
        // partner (dimension +-64) sits 16 lanes away.  cos/sin rounded to fp16 as the model code does.
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float sv, cv;
            sincosf(static_cast<float>(pos) * L.inv_freq[(lane & 15) * 4 + c], &sv, &cv);
            cs[c] = __half2float(__float2half_rn(cv * L.rope_scaling));
            sn[c] = __half2float(__float2half_rn(sv * L.rope_scaling));
            if (lane < 16) sn[c] = -sn[c];
        }
    }
    for (int b = 0; b < p.B; ++b) {
        float* a = p.acc + L.acc_off + (static_cast<size_t>(rt) * p.B + b) * 128 + lane * 4;
        float4 s = __ldcg(reinterpret_cast<const float4*>(a));
        __stcg(reinterpret_cast<float4*>(a), make_float4(0.f, 0.f, 0.f, 0.f));
        if (inv_rms != nullptr) { const float r = inv_rms[b]; s.x *= r; s.y *= r; s.z *= r; s.w *= r; }
        __half2 o01 = __floats2half2_rn(fmaf(s.x, aff.g[0], aff.b[0]), fmaf(s.y, aff.g[1], aff.b[1]));
        __half2 o23 = __floats2half2_rn(fmaf(s.z, aff.g[2], aff.b[2]), fmaf(s.w, aff.g[3], aff.b[3]));
        if (rope) {                                       // every row of the tile exists (checked on the host)
            const float2 v01 = __half22float2(o01), v23 = __half22float2(o23);
            const float v[4] = {v01.x, v01.y, v23.x, v23.y};
            float r[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) r[c] = fmaf(v[c], cs[c], __shfl_xor_sync(0xffffffffu, v[c], 16) * sn[c]);
            o01 = __floats2half2_rn(r[0], r[1]);
            o23 = __floats2half2_rn(r[2], r[3]);
        }
        if (row >= L.M) continue;
        __half* dst = L.y + static_cast<size_t>(b) * 8 * L.M + o;
        if (to_cache) {
            const int heads = L.M >> 4;
            dst = L.y + ((static_cast<size_t>(b) * heads + rt) * L.max_len + pos) * 128 + lane * 4;
            if (pos < 0 || pos >= L.max_len) continue;
        }
        if (L.y_op == EPTQ_Y_ADD_RESIDUAL) {
            const uint2 rv = __ldcg(reinterpret_cast<const uint2*>(L.residual + static_cast<size_t>(b) * 8 * L.M + o));   // may be another block's store of this launch
            o01 = __hadd2(*reinterpret_cast<const __half2*>(&rv.x), o01);
            o23 = __hadd2(*reinterpret_cast<const __half2*>(&rv.y), o23);
        }
        uint2 outv;
        outv.x = *reinterpret_cast<const unsigned*>(&o01);
        outv.y = *reinterpret_cast<const unsigned*>(&o23);
        *reinterpret_cast<uint2*>(dst) = outv;
    }
    if (p.done != nullptr) {
        // Chained launch: count the finished tile of this phase (release: the stores above are visible to
        // whoever sees the count).  32 counters per phase, one 128-byte line, so that the tiles of a phase do not
        // queue on one address; a waiter sums the line.
        __syncwarp();
        if (lane == 0)
            asm volatile("red.release.gpu.global.add.u32 [%0], 1;" :: "l"(p.done + L.phase * 32 + ((L.tile0 + rt) & 31)) : "memory");
    }
}

// Take a ticket for row tile rt of layer L; the last of the expected arrivals (n_main GEMV partials and
// 4 correction quarters) reads the tile's accumulators, zeroes them for the next launch and writes y.
template <class GA>
__device__ __forceinline__ void arrive_and_finalize(const GA& p, const GroupLayer& L, int rt, int n_main,
                                                    int lane, const Affine& aff, const float* inv_rms) {
    __syncwarp();      // orders every lane's adds before lane 0's release below (release is cumulative)
    unsigned ticket = 0;
    unsigned* ctr = p.counters + L.tile0 + rt;
    if (lane == 0)
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(ticket) : "l"(ctr) : "memory");
    ticket = __shfl_sync(0xffffffffu, ticket, 0);
    if (ticket != static_cast<unsigned>(n_main) + 3u) return;
    finalize_tile(p, L, rt, lane, aff, inv_rms);
}

// Correction of 4 consecutive Q rows (8 lanes per row, 4 entries per lane and pass).
// Weight-side loads (row pointers, columns, O, h) are issued before `wait_dep`, x after.
template <class GA, typename WaitFn, typename ContribFn>
__device__ __forceinline__ void correction_unit(const GA& p, const GroupLayer& L, int qt, int lane,
                                                float cstar0, float cstar1, float cstar2, float cstar3,
                                                const float* inv_rms, WaitFn wait_dep, ContribFn contributors) {
    const int row = qt * 4 + (lane >> 3);
    const int sub = lane & 7;
    const int rt = qt >> 2;
    const Affine aff = load_affine(L, rt, lane);
    const float cstar[4] = {cstar0, cstar1, cstar2, cstar3};
    float acc[2][8];
#pragma unroll
    for (int b = 0; b < 2; ++b)
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[b][k] = 0.f;
    int lo = 0, hi = 0;
    if (row < L.M) {
        lo = __ldg(L.O_row_ptr + row);
        hi = __ldg(L.O_row_ptr + row + 1);
    }
    bool first = true;
    for (int i = lo + sub; __any_sync(0xffffffffu, i < hi) || first; i += 32) {
        int col[4];
        float hv[4];
        uint4 ov[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) col[j] = (i + 8 * j < hi) ? __ldg(L.O_col + i + 8 * j) : -1;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (col[j] >= 0) {
                hv[j] = __half2float(__ldg(L.h + col[j]));
                ov[j] = ldg128(L.O_vals + static_cast<size_t>(i + 8 * j) * 8);
            } else {
                hv[j] = 0.f;
                ov[j] = make_uint4(0, 0, 0, 0);
            }
        }
        if (first) { wait_dep(); first = false; }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float o8[8];
            unpack8(ov[j], o8);
#pragma unroll
            for (int k = 0; k < 8; ++k) o8[k] -= cstar[k & 3];
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                if (b < p.B) {
                    const float xv = (col[j] >= 0) ? hv[j] * __half2float(__ldg(L.x + static_cast<size_t>(b) * L.N + col[j])) : 0.f;
#pragma unroll
                    for (int k = 0; k < 8; ++k) acc[b][k] = fmaf(o8[k], xv, acc[b][k]);
                }
            }
        }
    }
#pragma unroll
    for (int b = 0; b < 2; ++b) {
        if (b < p.B) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                acc[b][k] += __shfl_xor_sync(0xffffffffu, acc[b][k], 1);
                acc[b][k] += __shfl_xor_sync(0xffffffffu, acc[b][k], 2);
                acc[b][k] += __shfl_xor_sync(0xffffffffu, acc[b][k], 4);
            }
            if (sub == 0 && lo < hi) {
                float* dst = p.acc + L.acc_off + (static_cast<size_t>(rt) * p.B + b) * 128 + ((qt & 3) * 4 + (lane >> 3)) * 8;
                red_add4(dst, acc[b][0], acc[b][1], acc[b][2], acc[b][3]);
                red_add4(dst + 4, acc[b][4], acc[b][5], acc[b][6], acc[b][7]);
            }
        }
    }
    arrive_and_finalize(p, L, rt, contributors(L, rt), lane, aff, inv_rms);
}

}  // namespace groupdev

// Host: fills the per-launch description from the C-ABI arguments (everything except the work split, which
// differs between the kernels: W, nw, corr_units, n_corr_warps).  Checks the fusion arguments.
inline int fill_group_args(GroupArgs& a, const EptqLayer* layers, int n, const EptqFusion* fusions,
                           const uint16_t* const* xs, uint16_t* const* ys, int B, void* workspace,
                           const int* phases = nullptr, bool tiles64 = false) {
    const bool e8 = layers[0].quantizer == EPTQ_E8;
    a.table16 = reinterpret_cast<const uint2*>(layers[0].table16);
    a.packed = e8 ? layers[0].table_packed : nullptr;
    a.counters = reinterpret_cast<unsigned*>(workspace);
    a.acc = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + kCounterBytes);
    a.n_layers = n;
    a.B = B;
    a.x_norm = 0;
    a.norm_eps = 0.f;
    a.n_phases = 1;
    a.total_tiles = 0;
    a.done = nullptr;
    if (fusions != nullptr) {
        // Fused RMSNorm without phases is a property of the launch: all layers or none, one shared input.
        int normed = 0;
        for (int i = 0; i < n; ++i) {
            if (fusions[i].x_op == EPTQ_X_RMSNORM) ++normed;
            else if (fusions[i].x_op == EPTQ_X_SILU_MUL) { if (phases == nullptr) return EPTQ_ERR_UNSUPPORTED; }
            else if (fusions[i].x_op != EPTQ_X_PLAIN) return EPTQ_ERR_UNSUPPORTED;
        }
        if (normed != 0 && phases == nullptr) {
            if (normed != n) return EPTQ_ERR_UNSUPPORTED;
            for (int i = 0; i < n; ++i)
                if (xs[i] != xs[0] || layers[i].N != layers[0].N || fusions[i].norm_eps != fusions[0].norm_eps)
                    return EPTQ_ERR_UNSUPPORTED;
            if (xs[0] == nullptr) return EPTQ_ERR_NULL;
            if (!aligned16(xs[0])) return EPTQ_ERR_ALIGN;
            a.x_norm = 1;
            a.norm_eps = fusions[0].norm_eps;
        }
    }
    if (phases != nullptr) {
        if (phases[0] != 0) return EPTQ_ERR_SHAPE;
        for (int i = 1; i < n; ++i)
            if (phases[i] != phases[i - 1] && phases[i] != phases[i - 1] + 1) return EPTQ_ERR_SHAPE;
        a.n_phases = phases[n - 1] + 1;
    }
    for (int k = 0; k < kMaxGroupLayers; ++k) { a.phase_unit0[k] = 0; a.phase_units[k] = 0; }
    long long strip0 = 0, poff = 0;
    int tile0 = 0, corr0 = 0, unit0 = 0;
    for (int i = 0; i < n; ++i) {
        const EptqLayer& L = layers[i];
        GroupLayer& G = a.L[i];
        if (xs[i] == nullptr || ys[i] == nullptr) return EPTQ_ERR_NULL;
        if (!aligned16(ys[i])) return EPTQ_ERR_ALIGN;
        G.Q = L.Q;
        G.g = reinterpret_cast<const __half*>(L.g);
        G.h = reinterpret_cast<const __half*>(L.h);
        G.x = reinterpret_cast<const __half*>(xs[i]);
        G.O_vals = reinterpret_cast<const __half*>(L.O_vals);
        G.O_col = L.O_col;
        G.O_row_ptr = L.O_row_ptr;
        G.bias = reinterpret_cast<const __half*>(L.bias);
        G.y = reinterpret_cast<__half*>(ys[i]);
        G.M = L.M; G.N = L.N;
        G.ns = L.N / 32;
        G.row_tiles = (L.M + 15) / 16;
        G.strip0 = strip0; G.acc_off = poff; G.tile0 = tile0; G.corr0 = corr0;
        G.rt64 = (L.M + 63) / 64;
        G.cc128 = (L.N + 127) / 128;
        G.unit0 = unit0;
        G.phase = phases != nullptr ? phases[i] : 0;
        G.wait_tiles = 0;
        if (G.phase > 0) {
            if (phases[i] != phases[i - 1]) {
                a.phase_unit0[G.phase] = unit0;
                int prev_tiles = 0;                          // row tiles of the previous phase
                for (int j = i - 1; j >= 0 && phases[j] == phases[i - 1]; --j)
                    prev_tiles += tiles64 ? a.L[j].rt64 : a.L[j].row_tiles;
                G.wait_tiles = prev_tiles;
            } else {
                G.wait_tiles = a.L[i - 1].wait_tiles;
            }
        }
        a.phase_units[G.phase] += G.rt64 * G.cc128;
        unit0 += G.rt64 * G.cc128;
        G.crit_ptr = L.crit_ptr;
        G.crit_pos = L.crit_pos;
        G.crit_O = reinterpret_cast<const __half*>(L.crit_O);
        G.x_op = fusions != nullptr ? fusions[i].x_op : EPTQ_X_PLAIN;
        G.norm_eps = fusions != nullptr ? fusions[i].norm_eps : 0.f;
        G.x_aux = fusions != nullptr ? reinterpret_cast<const __half*>(fusions[i].x_aux) : nullptr;
        if (G.x_op == EPTQ_X_SILU_MUL) {
            if (G.x_aux == nullptr) return EPTQ_ERR_NULL;
            if (!aligned16(G.x_aux)) return EPTQ_ERR_ALIGN;
        }
        int e = 0;
        std::frexp(L.h_absmax, &e);            // h_absmax = m * 2^e, m in [0.5, 1)  =>  2^-e <= 1/h_absmax
        G.x_scale = std::ldexp(1.0f, -e);
        G.x_inv_scale = std::ldexp(1.0f, e) * (e8 ? L.table_packed_scale : 1.0f);   // E8 entries are in lattice units
        G.residual = nullptr; G.position = nullptr; G.inv_freq = nullptr;
        G.y_op = EPTQ_Y_STORE; G.max_len = 0; G.rope_scaling = 1.f;
        if (fusions != nullptr) {
            const EptqFusion& F = fusions[i];
            G.y_op = F.y_op;
            switch (F.y_op) {
                case EPTQ_Y_STORE: break;
                case EPTQ_Y_ADD_RESIDUAL:
                    if (F.residual == nullptr) return EPTQ_ERR_NULL;
                    if ((reinterpret_cast<uintptr_t>(F.residual) & 7u) != 0) return EPTQ_ERR_ALIGN;
                    G.residual = reinterpret_cast<const __half*>(F.residual);
                    break;
                case EPTQ_Y_ROPE: case EPTQ_Y_ROPE_TO_CACHE: case EPTQ_Y_TO_CACHE:
                    if ((L.M % 16) != 0) return EPTQ_ERR_SHAPE;               // whole heads of 128 outputs
                    if (F.position == nullptr) return EPTQ_ERR_NULL;
                    if (F.y_op != EPTQ_Y_TO_CACHE && F.inv_freq == nullptr) return EPTQ_ERR_NULL;
                    if (F.y_op != EPTQ_Y_ROPE && F.max_len < 1) return EPTQ_ERR_SHAPE;
                    G.position = reinterpret_cast<const long long*>(F.position);
                    G.inv_freq = F.inv_freq;
                    G.max_len = F.max_len;
                    G.rope_scaling = F.rope_scaling;
                    break;
                default: return EPTQ_ERR_UNSUPPORTED;
            }
        }
        strip0 += static_cast<long long>(G.row_tiles) * G.ns;
        poff += static_cast<long long>(G.row_tiles) * B * 128;
        tile0 += G.row_tiles;
        corr0 += G.row_tiles * 4;
    }
    a.total_tiles = tile0;
    return EPTQ_OK;
}

}  // namespace eptq
