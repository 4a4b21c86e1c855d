// eptq_linear_forward_static_scratch: the tensor-core E8-D4 GEMV for callers that
// cannot hand over a scratch buffer because they have no way to allocate one.
//
// Typical callers: an inference server that reserved all device memory for its
// own pools at start-up and forbids any later cudaMalloc; a plug-in living
// inside another runtime whose allocator it must not touch; a decode loop that
// has to stay free of allocator calls for latency reasons.  For them the
// partial-sum and arrival-counter scratch of the GEMV lives in a fixed array
// that is part of this library's device image.
//
// Consequences, all documented in the header as well:
//   * every GPU that loads the library holds kStaticScratchBytes until exit;
//   * shapes and batches whose scratch would not fit are refused;
//   * all calls on one device share the array, so calls that can overlap on the
//     GPU (different streams without ordering) race; the array keeps whatever
//     the last call left in it, and the kernel itself returns the counters it
//     needs at zero;
//   * the first call on a device looks the array's device address up; do that
//     first call before starting a stream capture.

#include <mutex>

#include "common.cuh"

namespace eptq {

bool mma_gemv_supported(const EptqLayer& L, int B);
size_t mma_workspace_bytes(int M, int N, int B);
int launch_gemv_mma(const EptqLayer& L, const uint16_t* x, uint16_t* y, int B,
                    void* workspace, size_t workspace_bytes, cudaStream_t stream);

namespace {

constexpr size_t kStaticScratchBytes = 4u << 20;       // 4 MiB

// Zero-initialised when the module is loaded onto a device.  In host code this
// name is only a handle for cudaGetSymbolAddress, never a usable pointer.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_ptr[kMaxDevices] = {};

// Device address of the array on the current device, looked up once per device.
int static_scratch_for_current_device(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return EPTQ_ERR_LAUNCH;
    if (dev < 0 || dev >= kMaxDevices) return EPTQ_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) return EPTQ_ERR_LAUNCH;
        g_scratch_ptr[dev] = ptr;
    }
    *out = g_scratch_ptr[dev];
    return EPTQ_OK;
}

}  // namespace
}  // namespace eptq

using namespace eptq;

extern "C" {

size_t eptq_static_scratch_bytes(void) { return kStaticScratchBytes; }

int eptq_linear_forward_static_scratch(const EptqLayer* layer, const uint16_t* x, uint16_t* y, int B, void* stream) {
    if (layer == nullptr || x == nullptr || y == nullptr) return EPTQ_ERR_NULL;
    if (layer->M <= 0 || layer->N <= 0 || B <= 0) return EPTQ_ERR_SHAPE;
    if (layer->Q == nullptr || layer->g == nullptr || layer->h == nullptr || layer->O_row_ptr == nullptr ||
        layer->table16 == nullptr)
        return EPTQ_ERR_NULL;
    if (layer->n_masked != 0 && (layer->O_vals == nullptr || layer->O_col == nullptr)) return EPTQ_ERR_NULL;
    if (!mma_gemv_supported(*layer, B)) return EPTQ_ERR_UNSUPPORTED;
    if (!aligned16(layer->g) || !aligned16(layer->h) || !aligned16(x) || !aligned16(y) ||
        (layer->bias != nullptr && !aligned16(layer->bias)) || (layer->n_masked != 0 && !aligned16(layer->O_vals)))
        return EPTQ_ERR_ALIGN;
    const size_t need = mma_workspace_bytes(layer->M, layer->N, B);
    if (need == 0 || need > kStaticScratchBytes) return EPTQ_ERR_WORKSPACE;   // beyond the fixed maximum
    void* scratch = nullptr;
    const int st = static_scratch_for_current_device(&scratch);
    if (st != EPTQ_OK) return st;
    return launch_gemv_mma(*layer, x, y, B, scratch, kStaticScratchBytes, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
