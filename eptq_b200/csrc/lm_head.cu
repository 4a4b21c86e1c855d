// Un-quantized output projection of a decoder-only model fused with the greedy pick: logits = lm_head(x),
// token = argmax.  The reference leaves lm_head in fp16 (quantize.py:86-90) and samples on the host side of a
// library GEMM (bench_decode.py:35-41); at batch 1 the projection is a 262 MB stream (Llama-2-7B), the next
// largest after the quantized linears, and the pick needs nothing but a running maximum.
//
// One warp per vocabulary row at a time (rows strided over all warps of a persistent grid), 128-bit loads with
// eight in flight per lane, the activations in shared memory, fp32 accumulation, the logit rounded to fp16 as a
// half-precision GEMM would return it.  Optionally the final RMSNorm of the model is applied to x on the way in
// (every block recomputes it: 8 KB).  Each block keeps (max, first index of the max); the last block to arrive
// (ticket in scratch, bounded by nothing: no block waits) merges the per-block results and writes the tokens.

#include "common.cuh"
#include <atomic>

namespace eptq {
namespace {

constexpr int kLmThreads = 512;
constexpr int kLmMaxBatch = 4;
constexpr int kLmMaxHidden = 8192;

struct LmArgs {
    const __half* W;          // (V, H)
    const __half* x;          // (B, H)
    const __half* norm_w;     // (H) or null
    __half* logits;           // (B, V) or null
    long long* tokens;        // (B)
    float* part_val;          // scratch: [blocks][B]
    int* part_idx;            // scratch: [blocks][B]
    unsigned* ticket;         // scratch: one counter, zero between calls
    int V, H, B;
    float eps;
};

// Order of the pick, as torch.argmax has it: a NaN ranks above every number, equal values (and NaNs among
// themselves) go to the lower index.  Any real candidate beats the start value (-inf, INT_MAX), so the result is a
// valid row whatever the logits are -- a token outside the vocabulary would fault the next embedding lookup.
__device__ __forceinline__ bool better_pick(float v, int i, float m, int mi) {
    const bool vn = v != v, mn = m != m;
    if (vn != mn) return vn;
    if (!vn && v != m) return v > m;
    return i < mi;
}

__global__ void __launch_bounds__(kLmThreads) lm_head_argmax_kernel(const LmArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    __half* xs = reinterpret_cast<__half*>(smem);                        // [B][H]
    __shared__ float red[kLmThreads / 32][kLmMaxBatch];
    __shared__ int redi[kLmThreads / 32][kLmMaxBatch];
    __shared__ float s_scale[kLmMaxBatch];
    __shared__ bool s_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // activations (and the fused norm) into shared memory
    for (int b = 0; b < a.B; ++b) {
        float ss = 0.f;
        for (int c = threadIdx.x * 8; c < a.H; c += kLmThreads * 8) {
            const uint4 v = __ldcg(reinterpret_cast<const uint4*>(a.x + static_cast<size_t>(b) * a.H + c));
            *reinterpret_cast<uint4*>(xs + b * a.H + c) = v;
            float f[8];
            unpack8(v, f);
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = fmaf(f[e], f[e], ss);
        }
        if (a.norm_w != nullptr) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) red[warp][0] = ss;
            __syncthreads();
            if (threadIdx.x == 0) {
                float tot = 0.f;
                for (int w = 0; w < kLmThreads / 32; ++w) tot += red[w][0];
                s_scale[b] = rsqrtf(tot / static_cast<float>(a.H) + a.eps);
            }
            __syncthreads();
            const float r = s_scale[b];
            // LlamaRMSNorm: round x * r to fp16, then multiply by the weight (fp16)
            for (int c = threadIdx.x; c < a.H; c += kLmThreads) {
                const __half n = __float2half_rn(__half2float(xs[b * a.H + c]) * r);
                xs[b * a.H + c] = __hmul(a.norm_w[c], n);
            }
        }
    }
    __syncthreads();

    float best[kLmMaxBatch];
    int best_i[kLmMaxBatch];
#pragma unroll
    for (int b = 0; b < kLmMaxBatch; ++b) { best[b] = -INFINITY; best_i[b] = 0x7fffffff; }
    const int total_warps = gridDim.x * (kLmThreads / 32);
    const int chunks = a.H / 256;                                  // 256 columns per warp pass (8 per lane)
    for (int row = blockIdx.x * (kLmThreads / 32) + warp; row < a.V; row += total_warps) {
        const __half* wr = a.W + static_cast<size_t>(row) * a.H + lane * 8;
        float acc[kLmMaxBatch] = {0.f, 0.f, 0.f, 0.f};
        for (int c0 = 0; c0 < chunks; c0 += 8) {
            uint4 w[8];
#pragma unroll
            for (int k = 0; k < 8; ++k)
                w[k] = (c0 + k < chunks) ? ldg128(wr + (c0 + k) * 256) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (c0 + k >= chunks) break;
                float wf[8];
                unpack8(w[k], wf);
#pragma unroll
                for (int b = 0; b < kLmMaxBatch; ++b) {
                    if (b >= a.B) break;
                    float xf[8];
                    unpack8(*reinterpret_cast<const uint4*>(xs + b * a.H + (c0 + k) * 256 + lane * 8), xf);
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[b] = fmaf(wf[e], xf[e], acc[b]);
                }
            }
        }
#pragma unroll
        for (int b = 0; b < kLmMaxBatch; ++b) {
            if (b >= a.B) break;
            float v = acc[b];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            const __half h = __float2half_rn(v);
            if (lane == 0 && a.logits != nullptr) a.logits[static_cast<size_t>(b) * a.V + row] = h;
            const float hv = __half2float(h);
            if (better_pick(hv, row, best[b], best_i[b])) { best[b] = hv; best_i[b] = row; }
        }
    }
    if (lane == 0) {
#pragma unroll
        for (int b = 0; b < kLmMaxBatch; ++b) { red[warp][b] = best[b]; redi[warp][b] = best_i[b]; }
    }
    __syncthreads();
    if (threadIdx.x < a.B) {
        const int b = threadIdx.x;
        float m = -INFINITY;
        int mi = 0x7fffffff;
        for (int w = 0; w < kLmThreads / 32; ++w)
            if (better_pick(red[w][b], redi[w][b], m, mi)) { m = red[w][b]; mi = redi[w][b]; }
        a.part_val[blockIdx.x * a.B + b] = m;
        a.part_idx[blockIdx.x * a.B + b] = mi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned t;
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(t) : "l"(a.ticket) : "memory");
        s_last = t == gridDim.x - 1;
        if (s_last) *a.ticket = 0u;
    }
    __syncthreads();
    if (s_last && threadIdx.x < a.B) {
        const int b = threadIdx.x;
        float m = -INFINITY;
        int mi = 0x7fffffff;
        for (unsigned k = 0; k < gridDim.x; ++k) {
            const float v = __ldcg(a.part_val + k * a.B + b);
            const int i = __ldcg(a.part_idx + k * a.B + b);
            if (better_pick(v, i, m, mi)) { m = v; mi = i; }
        }
        a.tokens[b] = (mi >= 0 && mi < a.V) ? mi : 0;
    }
}

}  // namespace
}  // namespace eptq

using namespace eptq;

extern "C" size_t eptq_lm_head_workspace_bytes(int B) {
    if (B < 1 || B > kLmMaxBatch) return 0;
    return 256 + static_cast<size_t>(1024) * B * 8;       // ticket, then (value, index) per block and batch row
}

extern "C" int eptq_lm_head_argmax(const uint16_t* W, const uint16_t* x, const uint16_t* norm_weight, float eps,
                                   uint16_t* logits, int64_t* tokens, int V, int H, int B, void* workspace,
                                   size_t workspace_bytes, void* stream) {
    if (W == nullptr || x == nullptr || tokens == nullptr || workspace == nullptr) return EPTQ_ERR_NULL;
    if (V < 1 || H < 256 || (H % 256) != 0 || H > kLmMaxHidden || B < 1 || B > kLmMaxBatch) return EPTQ_ERR_SHAPE;
    if (!aligned16(W) || !aligned16(x) || (norm_weight != nullptr && !aligned16(norm_weight)) ||
        (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return EPTQ_ERR_ALIGN;
    if (workspace_bytes < eptq_lm_head_workspace_bytes(B)) return EPTQ_ERR_WORKSPACE;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) return EPTQ_ERR_LAUNCH;
    const int rows_per_block = kLmThreads / 32;
    int blocks = sms * 2;
    if (blocks > (V + rows_per_block - 1) / rows_per_block) blocks = (V + rows_per_block - 1) / rows_per_block;
    if (blocks > 1024) blocks = 1024;
    LmArgs a;
    a.W = reinterpret_cast<const __half*>(W);
    a.x = reinterpret_cast<const __half*>(x);
    a.norm_w = reinterpret_cast<const __half*>(norm_weight);
    a.logits = reinterpret_cast<__half*>(logits);
    a.tokens = reinterpret_cast<long long*>(tokens);
    a.ticket = reinterpret_cast<unsigned*>(workspace);
    a.part_val = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + 256);
    a.part_idx = reinterpret_cast<int*>(reinterpret_cast<char*>(workspace) + 256 + static_cast<size_t>(1024) * B * 4);
    a.V = V; a.H = H; a.B = B; a.eps = eps;
    const size_t smem = static_cast<size_t>(B) * H * sizeof(__half);
    static std::atomic<bool> attr_done[64];       // setting the attribute twice is harmless; the flag itself must not race
    if (dev >= 0 && dev < 64 && !attr_done[dev] && smem > 48 * 1024) {
        if (cudaFuncSetAttribute(lm_head_argmax_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kLmMaxBatch * kLmMaxHidden * 2) != cudaSuccess)
            return EPTQ_ERR_LAUNCH;
        attr_done[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(kLmThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, lm_head_argmax_kernel, a);
    count_launch(EPTQ_KERNEL_OTHER);
    return err == cudaSuccess ? EPTQ_OK : EPTQ_ERR_LAUNCH;
}
