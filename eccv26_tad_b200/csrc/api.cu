// C ABI of the SparseConv2D ops: argument validation, path selection, workspace layout.
#include <cstdlib>
#include <cstring>

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

}  // namespace svtad

using namespace svtad;

extern "C" int svtad_version(void) { return 100; }

extern "C" const char* svtad_last_error_string(void) { return g_err; }

extern "C" int svtad_path_for(int op, int64_t n, int cin, int cout, int kk, int dtype) {
    return use_tc(op, n, cin, cout, kk, dtype) ? 1 : 0;
}

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
    SV_CHECK_ARG(aligned(gy, 16) && aligned(x, 16) && aligned(gw, 16) && aligned(nbr, 16),
                 "svtad_conv_wgrad: gy, x, nbr and gw must be 16-byte aligned");
    SV_CHECK_ARG(workspace != nullptr && aligned(workspace, 256), "svtad_conv_wgrad: workspace is null or not 256-byte aligned");
    if (use_tc(SVTAD_OP_WGRAD, n, cin, cout, kk, dtype))
        return tc_wgrad(gy, x, nbr, gw, gb, n, cin, cout, kk, tokens_per_batch, dtype, workspace, workspace_bytes, s);
    if (forced_path() == 2)
        return set_error(SVTAD_ERR_UNSUPPORTED, "svtad_conv_wgrad: tensor-core path forced but shape/dtype unsupported");
    return simt_wgrad(gy, x, nbr, gw, gb, n, cin, cout, kk, tokens_per_batch, dtype, workspace, workspace_bytes, s);
}
