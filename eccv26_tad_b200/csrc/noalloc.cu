// Weight-gradient entry point for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc once they are running: inference servers that hand
// every byte of the device to their own arena at start-up, plugins whose host forbids allocation after
// initialisation, control loops that cannot afford the implicit synchronisation of an allocation.  svtad_conv_wgrad needs a workspace for its per-split
// fp32 partial sums, which such callers have nowhere to get from.  svtad_conv_wgrad_static is the same
// computation with that workspace taken from a fixed array that lives in the library's own device
// image, so the caller passes inputs and outputs only.
//
// The price: every GPU that loads the library holds SVTAD_STATIC_WS_BYTES of device memory until the
// process exits, problems whose workspace would be larger are refused, and all calls share the one
// array per device (see the header).
#include <mutex>

#include "common.cuh"

namespace svtad {

// In host code this name is only a handle for the runtime's symbol table, never a device address:
// the address the kernels get comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_ws[SVTAD_STATIC_WS_BYTES];

constexpr int MAX_DEVICES = 64;
static void* g_static_ws_ptr[MAX_DEVICES];
static std::mutex g_static_ws_mutex;

// Device address of the array on the current device; resolved once per device, with that device current.
static int static_ws_address(void** out) {
    int dev = 0;
    SV_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES)
        return set_error(SVTAD_ERR_UNSUPPORTED, "svtad_conv_wgrad_static: device ordinal %d is not supported", dev);
    std::lock_guard<std::mutex> lock(g_static_ws_mutex);
    if (g_static_ws_ptr[dev] == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_ws);
        if (e != cudaSuccess || p == nullptr)
            return set_error(SVTAD_ERR_CUDA, "svtad_conv_wgrad_static: cudaGetSymbolAddress failed: %s",
                             cudaGetErrorString(e));
        g_static_ws_ptr[dev] = p;
    }
    *out = g_static_ws_ptr[dev];
    return SVTAD_OK;
}

}  // namespace svtad

using namespace svtad;

extern "C" size_t svtad_static_workspace_bytes(void) { return SVTAD_STATIC_WS_BYTES; }

extern "C" int svtad_conv_wgrad_static(const void* gy, const void* x, const int32_t* nbr, void* gw, void* gb,
                                       int64_t n, int cin, int cout, int kk, int tokens_per_batch, int dtype,
                                       void* stream) {
    const size_t need = svtad_workspace_bytes(SVTAD_OP_WGRAD, n, cin, cout, kk, dtype);
    if (need > SVTAD_STATIC_WS_BYTES)
        return set_error(SVTAD_ERR_WORKSPACE,
                         "svtad_conv_wgrad_static: this problem needs a %zu-byte workspace, the built-in one holds "
                         "%zu bytes; use svtad_conv_wgrad with a caller-provided workspace",
                         need, (size_t)SVTAD_STATIC_WS_BYTES);
    void* ws = nullptr;
    if (need > 0) {
        int rc = static_ws_address(&ws);
        if (rc) return rc;
    }
    // nothing in the workspace has to start at zero: every split writes its whole partial before the
    // reduction reads it, so the previous call's contents are simply overwritten
    return svtad_conv_wgrad(gy, x, nbr, gw, gb, n, cin, cout, kk, tokens_per_batch, dtype, ws,
                            SVTAD_STATIC_WS_BYTES, stream);
}
