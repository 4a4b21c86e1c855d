// extern "C" surface of libeptq_b200: argument checks, kernel choice, status
// codes.  The functions here stand where the reference has `_run_forward`
// (csrc/eptq_kernels.cu:466-558) and the pybind module (csrc/binding.cpp:4-16).

#include <cmath>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.cuh"

extern "C" int eptq_prepare_d4_table8(const float* table, uint8_t* out, float* scale);

namespace eptq {

std::atomic<uint64_t> g_launches{0};
std::atomic<uint64_t> g_kernel_launches[EPTQ_KERNEL_COUNT];

int launch_dequant(const EptqLayer& L, uint16_t* W, cudaStream_t stream);
int launch_gemv_simt(const EptqLayer& L, const uint16_t* x, uint16_t* y, int B,
                     void* workspace, size_t workspace_bytes, cudaStream_t stream);
int simt_plan_splits(int M, int N, int B, int* cols_per_split);
bool mma_gemv_supported(const EptqLayer& L, int B);
size_t mma_workspace_bytes(int M, int N, int B);
int launch_gemv_mma(const EptqLayer& L, const uint16_t* x, uint16_t* y, int B,
                    void* workspace, size_t workspace_bytes, cudaStream_t stream);

bool gemm_supported(const EptqLayer& L, int T);
int launch_gemm_tcgen05(const EptqLayer& L, const uint16_t* x, uint16_t* y, int T, int* status, cudaStream_t stream);
bool gemm_ws_supported(const EptqLayer& L, const void* x, int T);
int launch_gemm_tcgen05_ws(const EptqLayer& L, const uint16_t* x, uint16_t* y, int T, int* status, cudaStream_t stream);
bool gemm_dense_supported(int T, int N, const void* x, const void* y, const void* bias);
int launch_gemm_dense(const uint16_t* W16, const uint16_t* x, uint16_t* y, const uint16_t* bias, int T, int out, int N,
                      int* status, cudaStream_t stream);
bool group_gemv_supported(const EptqLayer* layers, int n, int B);
size_t group_workspace_bytes(const EptqLayer* layers, int n, int B, int n_sms);
int launch_gemv_group(const EptqLayer* layers, int n, const EptqFusion* fusions, const uint16_t* const* xs,
                      uint16_t* const* ys, int B, void* workspace, size_t workspace_bytes, cudaStream_t stream);
bool stream_gemv_supported(const EptqLayer* layers, int n, int B);
int launch_gemv_stream(const EptqLayer* layers, int n, const EptqFusion* fusions, const int* phases,
                       const uint16_t* const* xs, uint16_t* const* ys, int B, void* workspace, size_t workspace_bytes,
                       cudaStream_t stream);

namespace {

int check_layer_common(const EptqLayer* L) {
    if (L == nullptr) return EPTQ_ERR_NULL;
    if (L->quantizer != EPTQ_E8 && L->quantizer != EPTQ_E8D4) return EPTQ_ERR_QUANTIZER;
    if (L->M <= 0 || L->N <= 0 || L->n_masked < -1) return EPTQ_ERR_SHAPE;
    if (L->Q == nullptr || L->g == nullptr || L->h == nullptr || L->O_row_ptr == nullptr) return EPTQ_ERR_NULL;
    if (L->n_masked != 0 && (L->O_vals == nullptr || L->O_col == nullptr)) return EPTQ_ERR_NULL;
    if (L->quantizer == EPTQ_E8D4 && L->table_rows != 512) return EPTQ_ERR_SHAPE;
    if (L->quantizer == EPTQ_E8 && (L->table_rows <= 0 || L->table_rows > 65535)) return EPTQ_ERR_SHAPE;
    if (L->S_group != nullptr) {
        if (L->qb_size <= 0 || (L->qb_size % 8) != 0 || ((8 * L->M) % L->qb_size) != 0) return EPTQ_ERR_SHAPE;
    }
    // 128-bit accesses: rows of Q / h / x / S_group start on 16 bytes when N % 8 == 0.
    if ((L->N % 8) == 0) {
        if (!aligned16(L->Q) || !aligned16(L->h)) return EPTQ_ERR_ALIGN;
        if (L->S_group != nullptr && !aligned16(L->S_group)) return EPTQ_ERR_ALIGN;
    }
    if (L->n_masked != 0 && !aligned16(L->O_vals)) return EPTQ_ERR_ALIGN;
    return EPTQ_OK;
}

// Bytes of the reconstructed fp16 weight (8M x N) behind the first MiB of scratch.
size_t dense_weight_bytes(int M, int N) {
    return (static_cast<size_t>(8) * M * N * sizeof(uint16_t) + 255) & ~static_cast<size_t>(255);
}

int forward_checked(const EptqLayer& L, const uint16_t* x, uint16_t* y, int B,
                    void* workspace, size_t workspace_bytes, void* stream) {
    int st = check_layer_common(&L);
    if (st != EPTQ_OK) return st;
    if (x == nullptr || y == nullptr || L.table16 == nullptr) return EPTQ_ERR_NULL;
    if (B <= 0) return EPTQ_ERR_SHAPE;
    if (!aligned16(L.table16)) return EPTQ_ERR_ALIGN;
    if ((L.N % 8) == 0 && !aligned16(x)) return EPTQ_ERR_ALIGN;
    if (workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return EPTQ_ERR_ALIGN;
    if (B > kGemmMinBatch && gemm_supported(L, B) && aligned16(y) && (L.bias == nullptr || aligned16(L.bias)) &&
        workspace != nullptr && workspace_bytes >= kCounterBytes) {
        int* status = reinterpret_cast<int*>(workspace) + (kMaxCounters - 1);     // last counter word: never a tile
        // Long prefill and a scratch buffer that holds the fp16 weight: reconstruct once, then a dense GEMM.
        if (gemm_dense_supported(B, L.N, x, y, L.bias) && workspace_bytes >= kPartialOffset + dense_weight_bytes(L.M, L.N)) {
            uint16_t* W16 = reinterpret_cast<uint16_t*>(reinterpret_cast<char*>(workspace) + kPartialOffset);
            st = launch_dequant(L, W16, static_cast<cudaStream_t>(stream));
            if (st != EPTQ_OK) return st;
            return launch_gemm_dense(W16, x, y, L.bias, B, 8 * L.M, L.N, status, static_cast<cudaStream_t>(stream));
        }
        if (gemm_ws_supported(L, x, B))
            return launch_gemm_tcgen05_ws(L, x, y, B, status, static_cast<cudaStream_t>(stream));
        return launch_gemm_tcgen05(L, x, y, B, status, static_cast<cudaStream_t>(stream));
    }
    if (stream_gemv_supported(&L, 1, B) && aligned16(y) && workspace != nullptr && workspace_bytes >= kPartialOffset) {
        const uint16_t* xs[1] = {x};
        uint16_t* ys[1] = {y};
        return launch_gemv_stream(&L, 1, nullptr, nullptr, xs, ys, B, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
    }
    // The E8 variant copies 219 KB of table into every block: not worth it for a small layer.
    const bool big_enough = L.quantizer != EPTQ_E8 || static_cast<long long>(L.M) * L.N >= (1LL << 20);
    if (big_enough && group_gemv_supported(&L, 1, B) && aligned16(y)) {
        const uint16_t* xs[1] = {x};
        uint16_t* ys[1] = {y};
        const size_t need = group_workspace_bytes(&L, 1, B, 0);
        if (need != 0 && workspace != nullptr && workspace_bytes >= need)
            return launch_gemv_group(&L, 1, nullptr, xs, ys, B, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
    }
    if (mma_gemv_supported(L, B) && aligned16(L.g) && (L.bias == nullptr || aligned16(L.bias)) && aligned16(y))
        return launch_gemv_mma(L, x, y, B, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
    return launch_gemv_simt(L, x, y, B, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

// E8-D4 tables seen by the reference-signature entry point, keyed by device pointer: the scale of the table as
// a multiple of the D4 lattice (0 = not such a multiple), found by reading the 4 KB table back once.
std::mutex g_codebook_mutex;
std::unordered_map<const void*, float> g_codebook_unit;
const uint8_t g_table8_marker[4] = {0, 0, 0, 0};     // non-null EptqLayer.table8: "table8_scale is valid"

float d4_unit_of(const uint16_t* codes, cudaStream_t stream) {
    {
        std::lock_guard<std::mutex> lock(g_codebook_mutex);
        auto it = g_codebook_unit.find(codes);
        if (it != g_codebook_unit.end()) return it->second;
    }
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return 0.f;   // no copy inside a capture
    std::vector<uint16_t> raw(2048);
    if (cudaMemcpy(raw.data(), codes, 4096, cudaMemcpyDeviceToHost) != cudaSuccess) return 0.f;
    std::vector<float> tab(2048);
    for (int i = 0; i < 2048; ++i) {
        const __half_raw hr = {raw[i]};
        tab[i] = __half2float(__half(hr));
    }
    std::vector<uint8_t> out(2048);
    float scale = 0.f;
    if (eptq_prepare_d4_table8(tab.data(), out.data(), &scale) != EPTQ_OK) scale = 0.f;
    std::lock_guard<std::mutex> lock(g_codebook_mutex);
    g_codebook_unit[codes] = scale;
    return scale;
}

}  // namespace
}  // namespace eptq

using namespace eptq;

extern "C" {

int eptq_abi_version(void) { return EPTQ_ABI_VERSION; }

const char* eptq_strerror(int status) {
    switch (status) {
        case EPTQ_OK: return "ok";
        case EPTQ_ERR_NULL: return "a required pointer is null";
        case EPTQ_ERR_SHAPE: return "shape argument out of range (M, N, B, qb_size or table size)";
        case EPTQ_ERR_ALIGN: return "pointer not aligned for 128-bit access";
        case EPTQ_ERR_QUANTIZER: return "unknown quantizer id";
        case EPTQ_ERR_WORKSPACE: return "workspace missing or too small (see eptq_workspace_bytes)";
        case EPTQ_ERR_LAUNCH: return "CUDA runtime rejected a kernel launch";
        case EPTQ_ERR_UNSUPPORTED: return "no kernel covers these arguments";
        case EPTQ_ERR_TIMEOUT: return "a bounded device-side wait ran out";
        default: return "unknown eptq status";
    }
}

uint64_t eptq_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

uint64_t eptq_kernel_launch_count(int kernel) {
    if (kernel < 0 || kernel >= EPTQ_KERNEL_COUNT) return 0;
    return g_kernel_launches[kernel].load(std::memory_order_relaxed);
}

size_t eptq_workspace_bytes(int M, int N, int B) {
    if (M <= 0 || N <= 0 || B <= 0) return 0;
    int cols = 0;
    const int splits = simt_plan_splits(M, N, B, &cols);
    size_t bytes = kPartialOffset;
    bytes += static_cast<size_t>(splits > 1 ? splits : 1) * B * 8u * M * sizeof(float);
    if (B <= 4 && (N % 32) == 0) {
        const size_t mma = mma_workspace_bytes(M, N, B);
        if (mma > bytes) bytes = mma;
    }
    if (B <= kGemmMinBatch && (N % 32) == 0) {
        EptqLayer shape = {};
        shape.M = M; shape.N = N;
        const size_t grp = group_workspace_bytes(&shape, 1, B, 0);
        if (grp > bytes) bytes = grp;
    }
    if (B >= kDenseMinTokens && (N % 8) == 0 && kPartialOffset + dense_weight_bytes(M, N) > bytes)
        bytes = kPartialOffset + dense_weight_bytes(M, N);
    return (bytes + 255) & ~static_cast<size_t>(255);
}

size_t eptq_layer_workspace_bytes(const EptqLayer* layer, int B) {
    if (layer == nullptr || B <= 0) return 0;
    // Above the GEMV batch limit a layer the tensor-core GEMM takes needs the counter block only.
    if (B > kGemmMinBatch && gemm_supported(*layer, B))
        return kPartialOffset + (B >= kDenseMinTokens ? dense_weight_bytes(layer->M, layer->N) : 0);
    return eptq_workspace_bytes(layer->M, layer->N, B);
}

size_t eptq_group_workspace_bytes(const EptqLayer* layers, int n_layers, int B) {
    if (stream_gemv_supported(layers, n_layers, B)) return kPartialOffset;
    if (!group_gemv_supported(layers, n_layers, B)) return 0;
    return (group_workspace_bytes(layers, n_layers, B, 0) + 255) & ~static_cast<size_t>(255);
}

int eptq_linear_forward_group_fused(const EptqLayer* layers, int n_layers, const EptqFusion* fusions,
                                    const uint16_t* const* xs, uint16_t* const* ys, int B,
                                    void* workspace, size_t workspace_bytes, void* stream) {
    if (layers == nullptr || xs == nullptr || ys == nullptr) return EPTQ_ERR_NULL;
    if (n_layers < 1 || B < 1) return EPTQ_ERR_SHAPE;
    for (int i = 0; i < n_layers; ++i) {
        const int st = check_layer_common(&layers[i]);
        if (st != EPTQ_OK) return st;
        if (xs[i] == nullptr || ys[i] == nullptr) return EPTQ_ERR_NULL;
        if (!aligned16(xs[i])) return EPTQ_ERR_ALIGN;
    }
    if (workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return EPTQ_ERR_ALIGN;
    if (stream_gemv_supported(layers, n_layers, B))
        return launch_gemv_stream(layers, n_layers, fusions, nullptr, xs, ys, B, workspace, workspace_bytes,
                                  static_cast<cudaStream_t>(stream));
    if (!group_gemv_supported(layers, n_layers, B)) return EPTQ_ERR_UNSUPPORTED;
    return launch_gemv_group(layers, n_layers, fusions, xs, ys, B, workspace, workspace_bytes,
                             static_cast<cudaStream_t>(stream));
}

int eptq_linear_forward_chain(const EptqLayer* layers, int n_layers, const EptqFusion* fusions, const int* phases,
                              const uint16_t* const* xs, uint16_t* const* ys, int B,
                              void* workspace, size_t workspace_bytes, void* stream) {
    if (layers == nullptr || xs == nullptr || ys == nullptr || phases == nullptr) return EPTQ_ERR_NULL;
    if (n_layers < 1 || B < 1) return EPTQ_ERR_SHAPE;
    for (int i = 0; i < n_layers; ++i) {
        const int st = check_layer_common(&layers[i]);
        if (st != EPTQ_OK) return st;
        if (xs[i] == nullptr || ys[i] == nullptr) return EPTQ_ERR_NULL;
        if (!aligned16(xs[i])) return EPTQ_ERR_ALIGN;
    }
    if (workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return EPTQ_ERR_ALIGN;
    if (!stream_gemv_supported(layers, n_layers, B)) return EPTQ_ERR_UNSUPPORTED;
    return launch_gemv_stream(layers, n_layers, fusions, phases, xs, ys, B, workspace, workspace_bytes,
                              static_cast<cudaStream_t>(stream));
}

// Status word of a scratch buffer (the last counter): EPTQ_OK, or EPTQ_ERR_TIMEOUT / EPTQ_ERR_LAUNCH left by a
// kernel whose bounded wait ran out.  Copies it to the host on `stream`, waits for the copy, clears the word.
int eptq_workspace_status(void* workspace, int* host_out, void* stream) {
    if (workspace == nullptr || host_out == nullptr) return EPTQ_ERR_NULL;
    int* word = reinterpret_cast<int*>(workspace) + (kMaxCounters - 1);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemcpyAsync(host_out, word, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess) return EPTQ_ERR_LAUNCH;
    if (cudaMemsetAsync(word, 0, sizeof(int), s) != cudaSuccess) return EPTQ_ERR_LAUNCH;
    return cudaStreamSynchronize(s) == cudaSuccess ? EPTQ_OK : EPTQ_ERR_LAUNCH;
}

int eptq_linear_forward_group(const EptqLayer* layers, int n_layers,
                              const uint16_t* const* xs, uint16_t* const* ys, int B,
                              void* workspace, size_t workspace_bytes, void* stream) {
    return eptq_linear_forward_group_fused(layers, n_layers, nullptr, xs, ys, B, workspace, workspace_bytes, stream);
}

int eptq_prepare_d4_table8(const float* table, uint8_t* out, float* scale) {
    if (table == nullptr || out == nullptr || scale == nullptr) return EPTQ_ERR_NULL;
    // Smallest non-zero magnitude is a coordinate 0.5 of the lattice.
    double amin = 0.0;
    for (int i = 0; i < 2048; ++i) {
        const double a = std::fabs(static_cast<double>(table[i]));
        if (a > 0.0 && (amin == 0.0 || a < amin)) amin = a;
    }
    if (amin == 0.0) return EPTQ_ERR_UNSUPPORTED;
    // Least-squares scale against the rounded half-integers.
    double num = 0.0, den = 0.0;
    for (int i = 0; i < 2048; ++i) {
        const double r = std::nearbyint(table[i] / amin) * 0.5;     // amin is the coordinate 0.5
        num += r * table[i];
        den += r * r;
    }
    if (den == 0.0) return EPTQ_ERR_UNSUPPORTED;
    const double sc = num / den;
    for (int i = 0; i < 2048; ++i) {
        const double r2 = table[i] / sc * 2.0;
        const double r = std::nearbyint(r2);
        if (std::fabs(r2 - r) > 2e-3 || std::fabs(r) > 127.0) return EPTQ_ERR_UNSUPPORTED;
        out[i] = static_cast<uint8_t>(static_cast<int8_t>(r));
    }
    *scale = static_cast<float>(sc * 0.5);
    return EPTQ_OK;
}

int eptq_e8_forward(const int16_t* Q, const uint16_t* codebook, int table_rows,
                    const uint16_t* g, const uint16_t* h, const uint16_t* x,
                    const uint16_t* O_vals, const int32_t* O_col,
                    const int32_t* O_row_ptr, const uint16_t* bias,
                    uint16_t* y, int M, int N, int B,
                    void* workspace, size_t workspace_bytes, void* stream) {
    EptqLayer L = {};
    L.quantizer = EPTQ_E8; L.M = M; L.N = N; L.table_rows = table_rows;
    L.n_masked = (O_vals != nullptr && O_col != nullptr) ? -1 : 0;   // count unknown: the CSR row pointers carry it
    L.Q = Q; L.table16 = codebook; L.g = g; L.h = h;
    L.O_vals = O_vals; L.O_col = O_col; L.O_row_ptr = O_row_ptr; L.bias = bias;
    return forward_checked(L, x, y, B, workspace, workspace_bytes, stream);
}

int eptq_e8d4_forward(const int16_t* Q, const uint16_t* codes,
                      const uint16_t* g, const uint16_t* h, const uint16_t* x,
                      const uint16_t* O_vals, const int32_t* O_col,
                      const int32_t* O_row_ptr, const uint16_t* bias,
                      uint16_t* y, int M, int N, int B,
                      void* workspace, size_t workspace_bytes, void* stream) {
    EptqLayer L = {};
    L.quantizer = EPTQ_E8D4; L.M = M; L.N = N; L.table_rows = 512;
    L.n_masked = (O_vals != nullptr && O_col != nullptr) ? -1 : 0;
    L.Q = Q; L.table16 = codes; L.g = g; L.h = h;
    L.O_vals = O_vals; L.O_col = O_col; L.O_row_ptr = O_row_ptr; L.bias = bias;
    if (codes != nullptr && B == 1) {                  // the streaming kernel needs the table as a lattice multiple
        const float unit = d4_unit_of(codes, static_cast<cudaStream_t>(stream));
        if (unit > 0.f) { L.table8 = g_table8_marker; L.table8_scale = unit; }
    }
    return forward_checked(L, x, y, B, workspace, workspace_bytes, stream);
}

void eptq_forget_codebook(const void* codes) {
    std::lock_guard<std::mutex> lock(g_codebook_mutex);
    if (codes == nullptr) g_codebook_unit.clear();
    else g_codebook_unit.erase(codes);
}

int eptq_linear_forward(const EptqLayer* layer, const uint16_t* x, uint16_t* y,
                        int B, void* workspace, size_t workspace_bytes, void* stream) {
    if (layer == nullptr) return EPTQ_ERR_NULL;
    return forward_checked(*layer, x, y, B, workspace, workspace_bytes, stream);
}

int eptq_dequantize(const EptqLayer* layer, uint16_t* W, void* stream) {
    int st = check_layer_common(layer);
    if (st != EPTQ_OK) return st;
    if (W == nullptr || layer->table32 == nullptr) return EPTQ_ERR_NULL;
    if (!aligned16(layer->table32)) return EPTQ_ERR_ALIGN;
    if ((layer->N % 8) == 0 && !aligned16(W)) return EPTQ_ERR_ALIGN;
    return launch_dequant(*layer, W, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
