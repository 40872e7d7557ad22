// Shared host/device helpers of libsvtad.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/svtad.h"

namespace svtad {

// ---- host-side error reporting (thread-local text behind svtad_last_error_string) ----
int set_error(int code, const char* fmt, ...);
#define SV_CHECK_ARG(cond, ...) \
    do { if (!(cond)) return ::svtad::set_error(SVTAD_ERR_ARG, __VA_ARGS__); } while (0)
#define SV_CUDA(expr)                                                                         \
    do {                                                                                      \
        cudaError_t e__ = (expr);                                                             \
        if (e__ != cudaSuccess)                                                               \
            return ::svtad::set_error(SVTAD_ERR_CUDA, "%s failed: %s", #expr,                 \
                                      cudaGetErrorString(e__));                               \
    } while (0)
#define SV_LAUNCH_CHECK(name)                                                                 \
    do {                                                                                      \
        cudaError_t e__ = cudaGetLastError();                                                 \
        if (e__ != cudaSuccess)                                                               \
            return ::svtad::set_error(SVTAD_ERR_CUDA, "launch of %s failed: %s", name,        \
                                      cudaGetErrorString(e__));                               \
    } while (0)

inline size_t dtype_size(int dtype) { return dtype == SVTAD_F32 ? 4 : 2; }
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ---- launchers implemented in the other translation units ----
struct ConvArgs {
    const void* a;        // gathered operand: x (fwd) or gy (dgrad)
    const int32_t* nbr;
    const void* w;
    const void* bias;     // fwd only, may be null
    void* out;
    int64_t n;
    int cin, cout, kk, tpb, dtype;
};

// CUDA-core kernels (conv_simt.cu)
int simt_fwd(const ConvArgs& p, cudaStream_t s);
// fp32 forward tuned for the FFMA rate (conv_simt_fwd.cu)
bool simt_fwd_f32_supported(const ConvArgs& p);
int simt_fwd_f32(const ConvArgs& p, cudaStream_t s);
int simt_dgrad_gather(const ConvArgs& p, const int32_t* status, cudaStream_t s);
int simt_dgrad_scatter(const ConvArgs& p, const int32_t* status, float* ws, cudaStream_t s);
int simt_wgrad(const void* gy, const void* x, const int32_t* nbr, void* gw, void* gb, int64_t n,
               int cin, int cout, int kk, int tpb, int dtype, void* ws, size_t ws_bytes,
               cudaStream_t s);
size_t simt_wgrad_ws_bytes(int64_t n, int cin, int cout, int kk);
// shared pieces of the weight-gradient path (also used by the tensor-core path)
int bias_partial_launch(const void* gy, float* partial, int64_t n, int cout, int dtype, int splits,
                        cudaStream_t s);
int wgrad_finalize_launch(const float* ws_w, int splits_w, const float* ws_b, int splits_b,
                          void* gw, void* gb, int64_t n_w, int cout, int dtype, cudaStream_t s);
int bias_splits_for(int64_t n);

// tcgen05 kernels (conv_tc.cu)
bool tc_supported(int op, int64_t n, int cin, int cout, int kk, int dtype);
int tc_fwd(const ConvArgs& p, cudaStream_t s);
int tc_dgrad(const ConvArgs& p, const int32_t* status, cudaStream_t s);
int tc_wgrad(const void* gy, const void* x, const int32_t* nbr, void* gw, void* gb, int64_t n,
             int cin, int cout, int kk, int tpb, int dtype, void* ws, size_t ws_bytes,
             cudaStream_t s);
size_t tc_wgrad_ws_bytes(int64_t n, int cin, int cout, int kk);
int tc_read_error(int32_t* code_out);
int tc_set_share(int n);
int tc_get_share();
int tc_set_share_floor(int n);

// the single-CTA tensor-core kernels behind tc_* (conv_tc_hybrid.cu)
#define SV_DECLARE_TC_FAMILY(prefix)                                                                        \
    int prefix##_fwd(const ConvArgs& p, cudaStream_t s);                                                    \
    int prefix##_dgrad(const ConvArgs& p, const int32_t* status, cudaStream_t s);                           \
    int prefix##_wgrad(const void* gy, const void* x, const int32_t* nbr, void* gw, void* gb, int64_t n,    \
                       int cin, int cout, int kk, int tpb, int dtype, void* ws, size_t ws_bytes,            \
                       cudaStream_t s);
SV_DECLARE_TC_FAMILY(hybrid)
// forward / dgrad on CTA pairs (conv_tc_pair.cu)
int pair_fwd(const ConvArgs& p, cudaStream_t s);
int pair_dgrad(const ConvArgs& p, const int32_t* status, cudaStream_t s);

#ifdef __CUDACC__
// ---- device helpers ----
template <typename T> struct Cvt;
template <> struct Cvt<float> {
    static __device__ __forceinline__ float4 load4(const float* p) {
        return __ldg(reinterpret_cast<const float4*>(p));
    }
    static __device__ __forceinline__ float load1(const float* p) { return __ldg(p); }
    static __device__ __forceinline__ void store4(float* p, float4 v) {
        *reinterpret_cast<float4*>(p) = v;
    }
    static __device__ __forceinline__ void store1(float* p, float v) { *p = v; }
};
template <> struct Cvt<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
        uint2 r = __ldg(reinterpret_cast<const uint2*>(p));
        float4 v;
        v.x = __uint_as_float(r.x << 16);
        v.y = __uint_as_float(r.x & 0xffff0000u);
        v.z = __uint_as_float(r.y << 16);
        v.w = __uint_as_float(r.y & 0xffff0000u);
        return v;
    }
    static __device__ __forceinline__ float load1(const __nv_bfloat16* p) {
        return __bfloat162float(*p);
    }
    static __device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y);
        __nv_bfloat162 b = __floats2bfloat162_rn(v.z, v.w);
        uint2 r;
        r.x = *reinterpret_cast<uint32_t*>(&a);
        r.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = r;
    }
    static __device__ __forceinline__ void store1(__nv_bfloat16* p, float v) {
        *p = __float2bfloat16_rn(v);
    }
};
template <> struct Cvt<__half> {
    static __device__ __forceinline__ float4 load4(const __half* p) {
        uint2 r = __ldg(reinterpret_cast<const uint2*>(p));
        __half2 a = *reinterpret_cast<__half2*>(&r.x);
        __half2 b = *reinterpret_cast<__half2*>(&r.y);
        float2 fa = __half22float2(a), fb = __half22float2(b);
        return make_float4(fa.x, fa.y, fb.x, fb.y);
    }
    static __device__ __forceinline__ float load1(const __half* p) { return __half2float(*p); }
    static __device__ __forceinline__ void store4(__half* p, float4 v) {
        __half2 a = __floats2half2_rn(v.x, v.y);
        __half2 b = __floats2half2_rn(v.z, v.w);
        uint2 r;
        r.x = *reinterpret_cast<uint32_t*>(&a);
        r.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = r;
    }
    static __device__ __forceinline__ void store1(__half* p, float v) { *p = __float2half_rn(v); }
};
#endif  // __CUDACC__

}  // namespace svtad
