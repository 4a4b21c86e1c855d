// Small fused kernels between the quantized linears of a LLaMA-style decode step: residual add +
// RMSNorm, rotary embedding + key/value cache append, single-query attention over the cache,
// SiLU(gate) * up.  Each replaces a handful of elementwise launches of the HuggingFace forward the
// reference decodes through (bench_decode.py:44-71); all are trivially memory-bound, their purpose
// is to keep the number of launches per decoded token small.

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>

#include "../../include/eptq_b200.h"
#include "common.cuh"

namespace eptq {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum / max over up to 32 warps; `red` holds 33 floats.  `neutral` is 0 for the sum and a
// very negative number for the max.
template <bool kMax>
__device__ __forceinline__ float block_reduce(float v, float* red, float neutral) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = kMax ? warp_max(v) : warp_sum(v);
    __syncthreads();                                  // red may still be read from a previous call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? red[lane] : neutral;
        t = kMax ? warp_max(t) : warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// ---- residual add + RMSNorm ------------------------------------------------------------------
// One block per row.  x <- x + delta (fp16 rounding, as the reference's residual add), then
// out = w * fp16(x * rsqrt(mean(x^2) + eps)): the two roundings of the HuggingFace LlamaRMSNorm.
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(__half* __restrict__ x, const __half* __restrict__ delta,
                                                          const __half* __restrict__ w, __half* __restrict__ out,
                                                          int H, float eps) {
    __shared__ float red[33];
    // Programmatic dependent launch: let the next kernel of the stream start its own set-up now, and
    // wait for the previous kernel's results before touching any input.
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const size_t row = static_cast<size_t>(blockIdx.x) * H;
    float ss = 0.f;
    for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
        uint4 xv = *reinterpret_cast<const uint4*>(x + row + c);
        float f[8];
        unpack8(xv, f);
        if (delta != nullptr) {
            const uint4 dv = *reinterpret_cast<const uint4*>(delta + row + c);
            float d[8];
            unpack8(dv, d);
            __half2 r[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) r[i] = __floats2half2_rn(f[2 * i] + d[2 * i], f[2 * i + 1] + d[2 * i + 1]);
            xv = *reinterpret_cast<const uint4*>(r);
            *reinterpret_cast<uint4*>(x + row + c) = xv;
            unpack8(xv, f);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(f[i], f[i], ss);
    }
    const float total = block_reduce<false>(ss, red, 0.f);
    const float inv = rsqrtf(total / static_cast<float>(H) + eps);
    for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
        const uint4 xv = *reinterpret_cast<const uint4*>(x + row + c);      // own writes: same thread, same address
        const uint4 wv = *reinterpret_cast<const uint4*>(w + c);
        float f[8], g[8];
        unpack8(xv, f);
        unpack8(wv, g);
        __half2 r[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2 n = __floats2half2_rn(f[2 * i] * inv, f[2 * i + 1] * inv);
            const float2 nf = __half22float2(n);
            r[i] = __floats2half2_rn(g[2 * i] * nf.x, g[2 * i + 1] * nf.y);
        }
        *reinterpret_cast<uint4*>(out + row + c) = *reinterpret_cast<const uint4*>(r);
    }
}

// ---- SiLU(gate) * up ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) silu_mul_kernel(const __half* __restrict__ gate, const __half* __restrict__ up,
                                                       __half* __restrict__ out, size_t n8) {
    // Programmatic dependent launch: let the next kernel of the stream start its own set-up now, and
    // wait for the previous kernel's results before touching any input.
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n8;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const uint4 gv = reinterpret_cast<const uint4*>(gate)[i];
        const uint4 uv = reinterpret_cast<const uint4*>(up)[i];
        float g[8], u[8];
        unpack8(gv, g);
        unpack8(uv, u);
        __half2 r[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            // fp16 rounding after the activation and after the product, as two separate torch ops give
            const __half2 s = __floats2half2_rn(g[2 * k] / (1.f + __expf(-g[2 * k])), g[2 * k + 1] / (1.f + __expf(-g[2 * k + 1])));
            const float2 sf = __half22float2(s);
            r[k] = __floats2half2_rn(sf.x * u[2 * k], sf.y * u[2 * k + 1]);
        }
        reinterpret_cast<uint4*>(out)[i] = *reinterpret_cast<const uint4*>(r);
    }
}

// ---- rotary embedding + cache append -------------------------------------------------------------
// Grid (tokens, n_heads + 2 * n_kv_heads), hd/2 threads.  Token row r = b*T + t sits at cache position
// positions[t].  Heads [0, nh) rotate q in place; [nh, nh+nkv) rotate k into the key cache;
// the rest copy v into the value cache.  Pairing (i, i + hd/2) and cos/sin rounded to fp16 follow the
// HuggingFace LLaMA rotary embedding.
__global__ void rope_append_kernel(__half* __restrict__ q, const __half* __restrict__ k, const __half* __restrict__ v,
                                   __half* __restrict__ k_cache, __half* __restrict__ v_cache,
                                   const long long* __restrict__ positions, const float* __restrict__ inv_freq,
                                   int T, int nh, int nkv, int hd, int max_len, float scaling) {
    // Programmatic dependent launch: let the next kernel of the stream start its own set-up now, and
    // wait for the previous kernel's results before touching any input.
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int r = blockIdx.x, b = r / T, t = r - b * T;
    const int head = blockIdx.y;
    const int i = threadIdx.x, half = hd >> 1;
    const long long pos = positions[t];
    if (pos < 0 || pos >= max_len) return;                                   // out of the cache: leave untouched
    if (head >= nh + nkv) {                                                  // value: plain copy
        const int hv = head - nh - nkv;
        const __half* src = v + static_cast<size_t>(r) * nkv * hd + hv * hd;
        __half* dst = v_cache + ((static_cast<size_t>(b) * nkv + hv) * max_len + pos) * hd;
        dst[i] = src[i];
        dst[i + half] = src[i + half];
        return;
    }
    float s, c;
    sincosf(static_cast<float>(pos) * inv_freq[i], &s, &c);
    const float cf = __half2float(__float2half_rn(c * scaling)), sf = __half2float(__float2half_rn(s * scaling));
    if (head < nh) {
        __half* p = q + static_cast<size_t>(r) * nh * hd + head * hd;
        const float a = __half2float(p[i]), bb = __half2float(p[i + half]);
        p[i] = __float2half_rn(a * cf - bb * sf);
        p[i + half] = __float2half_rn(bb * cf + a * sf);
    } else {
        const int hk = head - nh;
        const __half* src = k + static_cast<size_t>(r) * nkv * hd + hk * hd;
        __half* dst = k_cache + ((static_cast<size_t>(b) * nkv + hk) * max_len + pos) * hd;
        const float a = __half2float(src[i]), bb = __half2float(src[i + half]);
        dst[i] = __float2half_rn(a * cf - bb * sf);
        dst[i + half] = __float2half_rn(bb * cf + a * sf);
    }
}

}  // namespace
}  // namespace eptq

namespace eptq {
namespace {

constexpr int kAttThreads = 128;
constexpr int kAttMaxChunk = 1024;       // keys one block scores at most (shared-memory score buffer)

// ---- attention of a few query tokens over the cache -------------------------------------------------
// Grid (n_heads, token rows, splits).  A block scores the keys [k0, k1) of its split (8 lanes per key,
// 128-byte coalesced segments), turns them into exp(score - max), accumulates the values, and writes
// (max, sum, accumulator) to scratch; the last block of a (row, head) to arrive merges the splits.
// Key/value cache layout: (batch, n_kv_heads, max_len, HD) fp16.  Token row r = b*T + t attends to the
// positions 0..positions[t].
template <int HD>
__global__ void __launch_bounds__(kAttThreads) decode_attention_kernel(
    const __half* __restrict__ q, const __half* __restrict__ k_cache, const __half* __restrict__ v_cache,
    const long long* __restrict__ positions, __half* __restrict__ out, float* __restrict__ partial,
    unsigned* __restrict__ counters, int T, int nh, int nkv, int max_len, float scale) {
    constexpr int LPR = HD / 8;                  // lanes per value row
    constexpr int KG = kAttThreads / LPR;        // value rows in flight
    __shared__ float sc[kAttMaxChunk];
    __shared__ float qs[HD];
    __shared__ float red[33];
    __shared__ float accs[KG][HD];
    __shared__ int is_last;
    // Programmatic dependent launch: let the next kernel of the stream start its own set-up now, and
    // wait for the previous kernel's results before touching any input.
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int tid = threadIdx.x;
    const int head = blockIdx.x, r = blockIdx.y, split = blockIdx.z, S = gridDim.z;
    const int b = r / T, t = r - b * T;
    long long pos = positions[t];
    const int n_keys = pos < 0 ? 0 : (pos + 1 > max_len ? max_len : static_cast<int>(pos + 1));
    const int chunk = (n_keys + S - 1) / S;
    const int k0 = split * chunk;
    const int k1 = min(n_keys, k0 + chunk);
    const int n = max(k1 - k0, 0);
    const int hk = head / (nh / nkv);
    const __half* Kb = k_cache + (static_cast<size_t>(b) * nkv + hk) * max_len * HD + static_cast<size_t>(k0) * HD;
    const __half* Vb = v_cache + (static_cast<size_t>(b) * nkv + hk) * max_len * HD + static_cast<size_t>(k0) * HD;

    for (int i = tid; i < HD; i += kAttThreads)
        qs[i] = __half2float(q[static_cast<size_t>(r) * nh * HD + head * HD + i]) * scale;
    __syncthreads();

    // Loads are issued in batches before any is used, so that a block pays about one memory round trip
    // per 64 keys instead of one per key row: 4 key rows per 8-lane group, and -- when the whole split
    // fits -- this thread's 8 value rows too, which then arrive under the softmax.
    constexpr int KPI = kAttThreads / 8;          // keys scored per pass of the block
    constexpr int SUB = 4;                        // passes batched
    constexpr int VSUB = 8;                       // value rows per thread batched
    const int kg = tid / LPR, jv = tid - kg * LPR;
    const bool small = n <= KG * VSUB;
    uint4 vreg[VSUB];
    {
        const int grp = tid >> 3, j = tid & 7;
        // The trip count is the same for every lane of a warp (the shuffles below name all 32 lanes);
        // a group past the end recomputes the last key and drops the result.
        for (int base = 0; base < n; base += KPI * SUB) {
            uint4 kreg[SUB][HD / 64];
#pragma unroll
            for (int it = 0; it < SUB; ++it) {
                const int kk = min(base + it * KPI + grp, n - 1);
#pragma unroll
                for (int c = 0; c < HD / 64; ++c) kreg[it][c] = ldg128(Kb + static_cast<size_t>(kk) * HD + c * 64 + j * 8);
            }
            if (small && base == 0) {
#pragma unroll
                for (int it = 0; it < VSUB; ++it) {
                    const int kk = kg + it * KG;
                    vreg[it] = kk < n ? ldg128(Vb + static_cast<size_t>(kk) * HD + jv * 8) : make_uint4(0, 0, 0, 0);
                }
            }
#pragma unroll
            for (int it = 0; it < SUB; ++it) {
                float d = 0.f;
#pragma unroll
                for (int c = 0; c < HD / 64; ++c) {
                    float f[8];
                    unpack8(kreg[it][c], f);
#pragma unroll
                    for (int i = 0; i < 8; ++i) d = fmaf(f[i], qs[c * 64 + j * 8 + i], d);
                }
                d += __shfl_xor_sync(0xffffffffu, d, 1);
                d += __shfl_xor_sync(0xffffffffu, d, 2);
                d += __shfl_xor_sync(0xffffffffu, d, 4);
                const int kk = base + it * KPI + grp;
                if (j == 0 && kk < n) sc[kk] = d;
            }
        }
    }
    __syncthreads();
    float m = -INFINITY;
    for (int kk = tid; kk < n; kk += kAttThreads) m = fmaxf(m, sc[kk]);
    m = block_reduce<true>(m, red, -INFINITY);
    float l = 0.f;
    for (int kk = tid; kk < n; kk += kAttThreads) {
        const float p = __expf(sc[kk] - m);
        sc[kk] = p;
        l += p;
    }
    l = block_reduce<false>(l, red, 0.f);           // its barriers also publish sc[]

    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    if (small) {
#pragma unroll
        for (int it = 0; it < VSUB; ++it) {
            const int kk = kg + it * KG;
            if (kk < n) {
                float f[8];
                unpack8(vreg[it], f);
                const float p = sc[kk];
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] = fmaf(p, f[i], acc[i]);
            }
        }
    } else {
        for (int base = 0; base < n; base += KG * VSUB) {
#pragma unroll
            for (int it = 0; it < VSUB; ++it) {
                const int kk = base + kg + it * KG;
                vreg[it] = kk < n ? ldg128(Vb + static_cast<size_t>(kk) * HD + jv * 8) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int it = 0; it < VSUB; ++it) {
                const int kk = base + kg + it * KG;
                if (kk < n) {
                    float f[8];
                    unpack8(vreg[it], f);
                    const float p = sc[kk];
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[i] = fmaf(p, f[i], acc[i]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) accs[kg][jv * 8 + i] = acc[i];
    __syncthreads();
    float mine = 0.f;
    if (tid < HD) {
#pragma unroll
        for (int gk = 0; gk < KG; ++gk) mine += accs[gk][tid];
    }
    const size_t slot = static_cast<size_t>(r) * nh + head;
    __half* dst = out + static_cast<size_t>(r) * nh * HD + head * HD;
    if (S == 1) {
        if (tid < HD) dst[tid] = __float2half_rn(l > 0.f ? mine / l : 0.f);
        return;
    }
    float* mypart = partial + (slot * S + split) * (HD + 2);
    if (tid < HD) __stcg(mypart + 2 + tid, mine);
    if (tid == 0) { __stcg(mypart, m); __stcg(mypart + 1, l); }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned ticket = atomicAdd(counters + slot, 1u);
        is_last = (ticket == static_cast<unsigned>(S - 1));
        if (is_last) counters[slot] = 0u;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (tid < HD) {
        const float* base = partial + slot * S * (HD + 2);
        float M = -INFINITY;
        for (int s = 0; s < S; ++s) M = fmaxf(M, __ldcg(base + static_cast<size_t>(s) * (HD + 2)));
        float L = 0.f, o = 0.f;
        for (int s = 0; s < S; ++s) {
            const float* ps = base + static_cast<size_t>(s) * (HD + 2);
            const float ms = __ldcg(ps);
            const float wgt = (ms == -INFINITY) ? 0.f : __expf(ms - M);
            L = fmaf(wgt, __ldcg(ps + 1), L);
            o = fmaf(wgt, __ldcg(ps + 2 + tid), o);
        }
        dst[tid] = __float2half_rn(L > 0.f ? o / L : 0.f);
    }
}

int attention_splits(int rows, int nh, int max_len) {
    const int need = (max_len + kAttMaxChunk - 1) / kAttMaxChunk;
    long long target = (2LL * 148 + static_cast<long long>(rows) * nh - 1) / (static_cast<long long>(rows) * nh);
    if (target > 64) target = 64;
    if (target > (max_len + 31) / 32) target = (max_len + 31) / 32;       // at least 32 keys per split
    int S = static_cast<int>(target);
    if (S < need) S = need;
    return S < 1 ? 1 : S;
}

// The arrival counters take a region of fixed size at the start of the scratch, so that calls of
// different shapes can share one buffer: every call leaves its counters at zero, and nothing else is
// ever written there.
constexpr size_t kAttCounterBytes = 65536;
constexpr long long kAttMaxCounters = kAttCounterBytes / sizeof(unsigned);

// Launch with the programmatic-stream-serialization attribute (the kernels above wait on their own).
template <typename... KArgs, typename... Args>
void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

int finish_launch() {
    count_launch(EPTQ_KERNEL_OTHER);
    return cudaGetLastError() == cudaSuccess ? EPTQ_OK : EPTQ_ERR_LAUNCH;
}

}  // namespace
}  // namespace eptq

using namespace eptq;

extern "C" int eptq_add_rmsnorm(uint16_t* x, const uint16_t* delta, const uint16_t* weight, uint16_t* out,
                                int rows, int H, float eps, void* stream) {
    if (x == nullptr || weight == nullptr || out == nullptr) return EPTQ_ERR_NULL;
    if (rows < 0 || H < 8 || (H % 8) != 0) return EPTQ_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(weight) || !aligned16(out) || (delta != nullptr && !aligned16(delta))) return EPTQ_ERR_ALIGN;
    if (rows == 0) return EPTQ_OK;
    launch_pdl(add_rmsnorm_kernel, dim3(rows), dim3(256), static_cast<cudaStream_t>(stream),
        reinterpret_cast<__half*>(x), reinterpret_cast<const __half*>(delta), reinterpret_cast<const __half*>(weight),
        reinterpret_cast<__half*>(out), H, eps);
    return finish_launch();
}

extern "C" int eptq_silu_mul(const uint16_t* gate, const uint16_t* up, uint16_t* out, size_t n, void* stream) {
    if (gate == nullptr || up == nullptr || out == nullptr) return EPTQ_ERR_NULL;
    if ((n % 8) != 0) return EPTQ_ERR_SHAPE;
    if (!aligned16(gate) || !aligned16(up) || !aligned16(out)) return EPTQ_ERR_ALIGN;
    if (n == 0) return EPTQ_OK;
    const size_t n8 = n / 8;
    const unsigned blocks = static_cast<unsigned>(n8 / 256 + 1 > 1184 ? 1184 : n8 / 256 + 1);
    launch_pdl(silu_mul_kernel, dim3(blocks), dim3(256), static_cast<cudaStream_t>(stream),
        reinterpret_cast<const __half*>(gate), reinterpret_cast<const __half*>(up), reinterpret_cast<__half*>(out), n8);
    return finish_launch();
}

extern "C" int eptq_rope_append(uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* k_cache,
                                uint16_t* v_cache, const int64_t* positions, const float* inv_freq, int B, int T,
                                int n_heads, int n_kv_heads, int head_dim, int max_len, float scaling, void* stream) {
    if (q == nullptr || k == nullptr || v == nullptr || k_cache == nullptr || v_cache == nullptr ||
        positions == nullptr || inv_freq == nullptr) return EPTQ_ERR_NULL;
    if (B < 0 || T < 0 || n_heads < 1 || n_kv_heads < 1 || head_dim < 2 || (head_dim % 2) != 0 || head_dim > 2048 ||
        max_len < 1 || static_cast<long long>(B) * T > 65535LL * 32768) return EPTQ_ERR_SHAPE;
    if (B == 0 || T == 0) return EPTQ_OK;
    const dim3 grid(static_cast<unsigned>(B) * T, n_heads + 2 * n_kv_heads);
    if (grid.y > 65535u) return EPTQ_ERR_SHAPE;
    launch_pdl(rope_append_kernel, grid, dim3(head_dim / 2), static_cast<cudaStream_t>(stream),
        reinterpret_cast<__half*>(q), reinterpret_cast<const __half*>(k), reinterpret_cast<const __half*>(v),
        reinterpret_cast<__half*>(k_cache), reinterpret_cast<__half*>(v_cache),
        reinterpret_cast<const long long*>(positions), inv_freq, T, n_heads, n_kv_heads, head_dim, max_len, scaling);
    return finish_launch();
}

extern "C" size_t eptq_attention_workspace_bytes(int rows, int n_heads, int head_dim, int max_len) {
    if (rows < 1 || n_heads < 1 || head_dim < 1 || max_len < 1) return 0;
    const int S = attention_splits(rows, n_heads, max_len);
    return kAttCounterBytes + static_cast<size_t>(rows) * n_heads * S * (head_dim + 2) * sizeof(float);
}

extern "C" int eptq_decode_attention(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache,
                                     const int64_t* positions, uint16_t* out, int B, int T, int n_heads,
                                     int n_kv_heads, int head_dim, int max_len, float scale, void* workspace,
                                     size_t workspace_bytes, void* stream) {
    if (q == nullptr || k_cache == nullptr || v_cache == nullptr || positions == nullptr || out == nullptr) return EPTQ_ERR_NULL;
    if (B < 0 || T < 0 || n_heads < 1 || n_kv_heads < 1 || (n_heads % n_kv_heads) != 0 || max_len < 1) return EPTQ_ERR_SHAPE;
    if (head_dim != 64 && head_dim != 128) return EPTQ_ERR_UNSUPPORTED;
    if (!aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache)) return EPTQ_ERR_ALIGN;
    if (B == 0 || T == 0) return EPTQ_OK;
    const long long rows_ll = static_cast<long long>(B) * T;
    if (rows_ll > 65535) return EPTQ_ERR_SHAPE;
    const int rows = static_cast<int>(rows_ll);
    const int S = attention_splits(rows, n_heads, max_len);
    if (S > 65535) return EPTQ_ERR_SHAPE;
    float* partial = nullptr;
    unsigned* counters = nullptr;
    if (S > 1) {
        if (static_cast<long long>(rows) * n_heads > kAttMaxCounters) return EPTQ_ERR_UNSUPPORTED;
        if (workspace == nullptr || workspace_bytes < eptq_attention_workspace_bytes(rows, n_heads, head_dim, max_len))
            return EPTQ_ERR_WORKSPACE;
        if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return EPTQ_ERR_ALIGN;
        counters = reinterpret_cast<unsigned*>(workspace);
        partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + kAttCounterBytes);
    }
    const dim3 grid(n_heads, rows, S);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const __half* qh = reinterpret_cast<const __half*>(q);
    const __half* kh = reinterpret_cast<const __half*>(k_cache);
    const __half* vh = reinterpret_cast<const __half*>(v_cache);
    const long long* ph = reinterpret_cast<const long long*>(positions);
    __half* oh = reinterpret_cast<__half*>(out);
    if (head_dim == 128)
        launch_pdl(decode_attention_kernel<128>, grid, dim3(kAttThreads), st, qh, kh, vh, ph, oh, partial, counters, T, n_heads, n_kv_heads, max_len, scale);
    else
        launch_pdl(decode_attention_kernel<64>, grid, dim3(kAttThreads), st, qh, kh, vh, ph, oh, partial, counters, T, n_heads, n_kv_heads, max_len, scale);
    return finish_launch();
}
