// extern "C" surface of libeptq_b200: argument checks, kernel choice, status
// codes.  The functions here stand where the reference has `_run_forward`
// (csrc/eptq_kernels.cu:466-558) and the pybind module (csrc/binding.cpp:4-16).

#include "common.cuh"

namespace eptq {

std::atomic<uint64_t> g_launches{0};

int launch_dequant(const EptqLayer& L, uint16_t* W, cudaStream_t stream);
int launch_gemv_simt(const EptqLayer& L, const uint16_t* x, uint16_t* y, int B,
                     void* workspace, size_t workspace_bytes, cudaStream_t stream);
int simt_plan_splits(int M, int N, int B, int* cols_per_split);

namespace {

int check_layer_common(const EptqLayer* L) {
    if (L == nullptr) return EPTQ_ERR_NULL;
    if (L->quantizer != EPTQ_E8 && L->quantizer != EPTQ_E8D4) return EPTQ_ERR_QUANTIZER;
    if (L->M <= 0 || L->N <= 0 || L->n_masked < 0) return EPTQ_ERR_SHAPE;
    if (L->Q == nullptr || L->g == nullptr || L->h == nullptr || L->O_row_ptr == nullptr) return EPTQ_ERR_NULL;
    if (L->n_masked > 0 && (L->O_vals == nullptr || L->O_col == nullptr)) return EPTQ_ERR_NULL;
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
    if (L->n_masked > 0 && !aligned16(L->O_vals)) return EPTQ_ERR_ALIGN;
    return EPTQ_OK;
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
    return launch_gemv_simt(L, x, y, B, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
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

size_t eptq_workspace_bytes(int M, int N, int B) {
    if (M <= 0 || N <= 0 || B <= 0) return 0;
    int cols = 0;
    const int splits = simt_plan_splits(M, N, B, &cols);
    size_t bytes = kCounterBytes;
    bytes += static_cast<size_t>(splits > 1 ? splits : 1) * B * 8u * M * sizeof(float);
    return (bytes + 255) & ~static_cast<size_t>(255);
}

int eptq_e8_forward(const int16_t* Q, const uint16_t* codebook, int table_rows,
                    const uint16_t* g, const uint16_t* h, const uint16_t* x,
                    const uint16_t* O_vals, const int32_t* O_col,
                    const int32_t* O_row_ptr, const uint16_t* bias,
                    uint16_t* y, int M, int N, int B,
                    void* workspace, size_t workspace_bytes, void* stream) {
    EptqLayer L = {};
    L.quantizer = EPTQ_E8; L.M = M; L.N = N; L.table_rows = table_rows;
    L.n_masked = (O_vals != nullptr && O_col != nullptr) ? 1 : 0;   // only "present or not" matters here
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
    L.n_masked = (O_vals != nullptr && O_col != nullptr) ? 1 : 0;
    L.Q = Q; L.table16 = codes; L.g = g; L.h = h;
    L.O_vals = O_vals; L.O_col = O_col; L.O_row_ptr = O_row_ptr; L.bias = bias;
    return forward_checked(L, x, y, B, workspace, workspace_bytes, stream);
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
