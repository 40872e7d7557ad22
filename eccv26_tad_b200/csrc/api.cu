// C ABI of the SparseConv2D ops: argument validation, path selection, workspace layout.
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace svtad {

static thread_local char g_err[512] = "";

int set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

// 0 = automatic, 1 = force CUDA-core kernels, 2 = force tensor-core kernels
static int forced_path() {
    const char* e = getenv("SVTAD_FORCE_PATH");
    if (e == nullptr || *e == 0) return 0;
    if (strcmp(e, "simt") == 0 || strcmp(e, "fp32") == 0) return 1;
    if (strcmp(e, "tc") == 0) return 2;
    return 0;
}

static bool use_tc(int op, int64_t n, int cin, int cout, int kk, int dtype) {
    int f = forced_path();
    if (f == 1) return false;
    return tc_supported(op, n, cin, cout, kk, dtype);
}

static int check_common(const char* who, int64_t n, int cin, int cout, int kk, int tpb, int dtype) {
    SV_CHECK_ARG(n >= 0 && n < (1ll << 31), "%s: n=%lld outside [0, 2^31)", who, (long long)n);
    SV_CHECK_ARG(cin > 0 && cout > 0, "%s: bad channel counts %d -> %d", who, cin, cout);
    SV_CHECK_ARG(kk > 0 && kk <= 49, "%s: kk=%d outside [1, 49]", who, kk);
    SV_CHECK_ARG(tpb >= 0, "%s: tokens_per_batch=%d is negative", who, tpb);
    SV_CHECK_ARG(dtype == SVTAD_F32 || dtype == SVTAD_BF16 || dtype == SVTAD_F16, "%s: unknown dtype %d", who, dtype);
    // same requirement as the reference wrapper (sparse_conv_layer.py:39-42)
    if (cin % 4 != 0)
        return set_error(SVTAD_ERR_UNSUPPORTED, "%s: C_in (%d) must be divisible by 4", who, cin);
    return SVTAD_OK;
}

static bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Per device: a stream of the library's own and two events, used to run the weight gradient next to the
// input gradient inside svtad_conv_bwd.  Created on first use, never destroyed (process lifetime).
struct SideLane {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
    std::mutex mu;     // one fork .. join sequence at a time per device (events are shared)
};
static constexpr int MAX_DEVICES = 64;
static SideLane g_lane[MAX_DEVICES];

static bool overlap_backward() {
    static const bool on = [] {
        const char* e = getenv("SVTAD_OVERLAP_BACKWARD");
        return !(e != nullptr && e[0] == '0');
    }();
    return on;
}

static int lane_ready(SideLane& l) {
    if (l.stream != nullptr) return SVTAD_OK;
    SV_CUDA(cudaStreamCreateWithFlags(&l.stream, cudaStreamNonBlocking));
    SV_CUDA(cudaEventCreateWithFlags(&l.fork, cudaEventDisableTiming));
    SV_CUDA(cudaEventCreateWithFlags(&l.join, cudaEventDisableTiming));
    return SVTAD_OK;
}

}  // namespace svtad

using namespace svtad;

extern "C" int svtad_version(void) { return 100; }

extern "C" const char* svtad_last_error_string(void) { return g_err; }

extern "C" int svtad_path_for(int op, int64_t n, int cin, int cout, int kk, int dtype) {
    return use_tc(op, n, cin, cout, kk, dtype) ? 1 : 0;
}

extern "C" int svtad_set_concurrency(int kernels) { return tc_set_share(kernels); }

extern "C" int svtad_get_concurrency(void) { return tc_get_share(); }

extern "C" int svtad_device_error(int32_t* code_out) {
    SV_CHECK_ARG(code_out != nullptr, "svtad_device_error: code_out is null");
    return tc_read_error(code_out);
}

extern "C" size_t svtad_workspace_bytes(int op, int64_t n, int cin, int cout, int kk, int dtype) {
    if (n <= 0 || cin <= 0 || cout <= 0 || kk <= 0) return 0;
    switch (op) {
        case SVTAD_OP_FWD: return 0;
        case SVTAD_OP_DGRAD: return align_up((size_t)n * cin * sizeof(float), 256);   // scatter form only
        case SVTAD_OP_WGRAD: {
            size_t a = simt_wgrad_ws_bytes(n, cin, cout, kk);
            size_t b = tc_supported(op, n, cin, cout, kk, dtype) ? tc_wgrad_ws_bytes(n, cin, cout, kk) : 0;
            return a > b ? a : b;
        }
        case SVTAD_OP_BWD:   // both halves run at the same time: the two workspaces sit side by side
            return align_up(svtad_workspace_bytes(SVTAD_OP_WGRAD, n, cin, cout, kk, dtype), 256) +
                   svtad_workspace_bytes(SVTAD_OP_DGRAD, n, cin, cout, kk, dtype);
    }
    return 0;
}

extern "C" int svtad_conv_fwd(const void* x, const int32_t* nbr, const void* w, const void* bias,
                              void* y, int64_t n, int cin, int cout, int kk, int tokens_per_batch,
                              int dtype, void* workspace, size_t workspace_bytes, void* stream) {
    (void)workspace; (void)workspace_bytes;
    int rc = check_common("svtad_conv_fwd", n, cin, cout, kk, tokens_per_batch, dtype);
    if (rc) return rc;
    if (n == 0) return SVTAD_OK;
    SV_CHECK_ARG(x && nbr && w && y, "svtad_conv_fwd: null pointer");
    SV_CHECK_ARG(aligned(x, 16) && aligned(w, 16) && aligned(y, 16) && aligned(nbr, 16) && aligned(bias, 16),
                 "svtad_conv_fwd: x, nbr, w, bias and y must be 16-byte aligned");
    ConvArgs p{x, nbr, w, bias, y, n, cin, cout, kk, tokens_per_batch, dtype};
    if (use_tc(SVTAD_OP_FWD, n, cin, cout, kk, dtype)) return tc_fwd(p, (cudaStream_t)stream);
    if (forced_path() == 2)
        return set_error(SVTAD_ERR_UNSUPPORTED, "svtad_conv_fwd: tensor-core path forced but shape/dtype unsupported");
    return simt_fwd(p, (cudaStream_t)stream);
}

extern "C" int svtad_conv_dgrad(const void* gy, const int32_t* nbr, const void* w, void* gx,
                                int64_t n, int cin, int cout, int kk, int tokens_per_batch,
                                int dtype, const int32_t* table_status, void* workspace,
                                size_t workspace_bytes, void* stream) {
    int rc = check_common("svtad_conv_dgrad", n, cin, cout, kk, tokens_per_batch, dtype);
    if (rc) return rc;
    if (n == 0) return SVTAD_OK;
    SV_CHECK_ARG(gy && nbr && w && gx, "svtad_conv_dgrad: null pointer");
    SV_CHECK_ARG(aligned(gy, 16) && aligned(w, 16) && aligned(gx, 16) && aligned(nbr, 16),
                 "svtad_conv_dgrad: gy, nbr, w and gx must be 16-byte aligned");
    if (cout % 4 != 0)
        return set_error(SVTAD_ERR_UNSUPPORTED, "svtad_conv_dgrad: C_out (%d) must be divisible by 4", cout);
    cudaStream_t s = (cudaStream_t)stream;
    ConvArgs p{gy, nbr, w, nullptr, gx, n, cin, cout, kk, tokens_per_batch, dtype};
    if (use_tc(SVTAD_OP_DGRAD, n, cin, cout, kk, dtype)) {
        rc = tc_dgrad(p, table_status, s);
    } else {
        if (forced_path() == 2)
            return set_error(SVTAD_ERR_UNSUPPORTED, "svtad_conv_dgrad: tensor-core path forced but shape/dtype unsupported");
        rc = simt_dgrad_gather(p, table_status, s);
    }
    if (rc) return rc;
    if (table_status != nullptr) {
        // asymmetric tables: the scatter form runs instead (both kernels read the status word)
        size_t need = svtad_workspace_bytes(SVTAD_OP_DGRAD, n, cin, cout, kk, dtype);
        if (workspace == nullptr || workspace_bytes < need)
            return set_error(SVTAD_ERR_WORKSPACE, "svtad_conv_dgrad: workspace %zu < %zu bytes", workspace_bytes, need);
        rc = simt_dgrad_scatter(p, table_status, static_cast<float*>(workspace), s);
    }
    return rc;
}

extern "C" int svtad_conv_wgrad(const void* gy, const void* x, const int32_t* nbr, void* gw, void* gb,
                                int64_t n, int cin, int cout, int kk, int tokens_per_batch,
                                int dtype, void* workspace, size_t workspace_bytes, void* stream) {
    int rc = check_common("svtad_conv_wgrad", n, cin, cout, kk, tokens_per_batch, dtype);
    if (rc) return rc;
    SV_CHECK_ARG(gw != nullptr, "svtad_conv_wgrad: gw is null");
    cudaStream_t s = (cudaStream_t)stream;
    if (n == 0) {
        SV_CUDA(cudaMemsetAsync(gw, 0, (size_t)kk * cin * cout * dtype_size(dtype), s));
        if (gb) SV_CUDA(cudaMemsetAsync(gb, 0, (size_t)cout * dtype_size(dtype), s));
        return SVTAD_OK;
    }
    SV_CHECK_ARG(gy && x && nbr, "svtad_conv_wgrad: null pointer");
    SV_CHECK_ARG(aligned(gy, 16) && aligned(x, 16) && aligned(gw, 16) && aligned(nbr, 16) && aligned(gb, 16),
                 "svtad_conv_wgrad: gy, x, nbr, gw and gb must be 16-byte aligned");
    SV_CHECK_ARG(workspace != nullptr && aligned(workspace, 256), "svtad_conv_wgrad: workspace is null or not 256-byte aligned");
    if (use_tc(SVTAD_OP_WGRAD, n, cin, cout, kk, dtype))
        return tc_wgrad(gy, x, nbr, gw, gb, n, cin, cout, kk, tokens_per_batch, dtype, workspace, workspace_bytes, s);
    if (forced_path() == 2)
        return set_error(SVTAD_ERR_UNSUPPORTED, "svtad_conv_wgrad: tensor-core path forced but shape/dtype unsupported");
    return simt_wgrad(gy, x, nbr, gw, gb, n, cin, cout, kk, tokens_per_batch, dtype, workspace, workspace_bytes, s);
}

extern "C" int svtad_conv_bwd(const void* gy, const void* x, const int32_t* nbr, const void* w, void* gx,
                              void* gw, void* gb, int64_t n, int cin, int cout, int kk,
                              int tokens_per_batch, int dtype, const int32_t* table_status,
                              void* workspace, size_t workspace_bytes, void* stream) {
    SV_CHECK_ARG(gx != nullptr || gw != nullptr, "svtad_conv_bwd: neither gx nor gw requested");
    SV_CHECK_ARG(gb == nullptr || gw != nullptr, "svtad_conv_bwd: gb needs gw");
    if (gw == nullptr)
        return svtad_conv_dgrad(gy, nbr, w, gx, n, cin, cout, kk, tokens_per_batch, dtype, table_status,
                                workspace, workspace_bytes, stream);
    if (gx == nullptr)
        return svtad_conv_wgrad(gy, x, nbr, gw, gb, n, cin, cout, kk, tokens_per_batch, dtype, workspace,
                                workspace_bytes, stream);
    // workspace = [weight-gradient part | input-gradient part (scatter form, only with a status word)]
    const size_t w_part = align_up(svtad_workspace_bytes(SVTAD_OP_WGRAD, n, cin, cout, kk, dtype), 256);
    const size_t d_part = table_status != nullptr ? svtad_workspace_bytes(SVTAD_OP_DGRAD, n, cin, cout, kk, dtype) : 0;
    if (n > 0 && (workspace == nullptr || workspace_bytes < w_part + d_part))
        return set_error(SVTAD_ERR_WORKSPACE, "svtad_conv_bwd: workspace %zu < %zu bytes", workspace_bytes,
                         w_part + d_part);
    void* ws_d = d_part ? static_cast<char*>(workspace) + w_part : nullptr;
    cudaStream_t s = (cudaStream_t)stream;
    int dev = 0;
    SV_CUDA(cudaGetDevice(&dev));
    if (!overlap_backward() || n == 0 || dev >= MAX_DEVICES) {
        int rc = svtad_conv_wgrad(gy, x, nbr, gw, gb, n, cin, cout, kk, tokens_per_batch, dtype, workspace, w_part, s);
        if (rc) return rc;
        return svtad_conv_dgrad(gy, nbr, w, gx, n, cin, cout, kk, tokens_per_batch, dtype, table_status, ws_d, d_part, s);
    }
    SideLane& lane = g_lane[dev];
    std::lock_guard<std::mutex> hold(lane.mu);
    int rc = lane_ready(lane);
    if (rc) return rc;
    // the two kernels share the GPU: each is planned for half of it unless the caller's hint already says more
    struct FloorGuard {
        int old;
        FloorGuard() : old(tc_set_share_floor(2)) {}
        ~FloorGuard() { tc_set_share_floor(old); }
    } floor_guard;
    // fork: the side stream starts where the caller's stream stands
    SV_CUDA(cudaEventRecord(lane.fork, s));
    SV_CUDA(cudaStreamWaitEvent(lane.stream, lane.fork, 0));
    int rc_w = svtad_conv_wgrad(gy, x, nbr, gw, gb, n, cin, cout, kk, tokens_per_batch, dtype, workspace, w_part,
                                lane.stream);
    int rc_d = svtad_conv_dgrad(gy, nbr, w, gx, n, cin, cout, kk, tokens_per_batch, dtype, table_status, ws_d,
                                d_part, s);
    // join, also after an error: whatever was launched on the side stream is ordered before the caller's next work
    cudaError_t e1 = cudaEventRecord(lane.join, lane.stream);
    cudaError_t e2 = cudaStreamWaitEvent(s, lane.join, 0);
    if (rc_w) return rc_w;
    if (rc_d) return rc_d;
    if (e1 != cudaSuccess || e2 != cudaSuccess)
        return set_error(SVTAD_ERR_CUDA, "svtad_conv_bwd: joining the side stream failed: %s",
                         cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
    return SVTAD_OK;
}
