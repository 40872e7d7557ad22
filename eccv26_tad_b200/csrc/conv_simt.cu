// CUDA-core (FFMA) SparseConv2D kernels: fp32 tensors at any width, 16-bit tensors whose shape the
// tensor-core path does not take, and the asymmetric-table dgrad.  Strict fp32 FMA accumulation in
// (tap, channel) ascending order - the order of the reference's tiled forward
// (opentad/models/bricks/2d_sparse_v3.cu:574-629) - so fp32 results stay within 1e-5 relative.
//
// One gather-GEMM template serves three uses:
//   MODE_FWD      out[i,:]  = bias + sum_k  x[nbr[i,k]] . W[k]            (A = x,  B = W[k])
//   MODE_DGATHER  gx[j,:]   = sum_k' gy[nbr[j,k']] . W[KK-1-k']^T          (A = gy, B = W^T; symmetric tables)
//   MODE_DSCATTER gx[nbr[i,k],:] += gy[i] . W[k]^T  (fp32 atomics into a workspace; any table,
//                 the reference's own formulation, 2d_sparse_v3.cu:679-707)
#include <cstdlib>

#include "common.cuh"

namespace svtad {

enum { MODE_FWD = 0, MODE_DGATHER = 1, MODE_DSCATTER = 2 };
constexpr int BK = 16;
constexpr int MAX_KK = 49;

template <typename T, int BM, int BN, int MODE>
__global__ void __launch_bounds__((BM / 4) * (BN / 4))
conv_simt_kernel(const T* __restrict__ a, const int32_t* __restrict__ nbr, const T* __restrict__ w,
                 const T* __restrict__ bias, T* __restrict__ out, float* __restrict__ scatter_ws,
                 const int32_t* __restrict__ status, long n, int cred, int cn, int cin, int cout,
                 int kk, int tpb) {
    // cred = reduction width (channels of `a`), cn = output width
    constexpr int NT = (BM / 4) * (BN / 4);
    constexpr bool TRANS_B = (MODE != MODE_FWD);
    if (status != nullptr) {
        bool asym = (__ldg(status) & SVTAD_TABLE_ASYMMETRIC) != 0;
        if (MODE == MODE_DGATHER && asym) return;
        if (MODE == MODE_DSCATTER && !asym) return;
    }
    __shared__ __align__(16) float As[BK][BM + 4];
    __shared__ __align__(16) float Bs[BK][BN + 4];
    __shared__ int s_nbr[BM][MAX_KK];
    __shared__ int s_any[MAX_KK];

    const int tid = threadIdx.x;
    const int tx = tid % (BN / 4), ty = tid / (BN / 4);
    const long row0 = (long)blockIdx.y * BM;
    const int n0 = blockIdx.x * BN;

    for (int t = tid; t < kk; t += NT) s_any[t] = 0;
    __syncthreads();
    for (int e = tid; e < BM * kk; e += NT) {
        int r = e / kk, k = e - r * kk;
        long i = row0 + r;
        int v = -1;
        if (i < n) {
            if (MODE == MODE_DSCATTER) {
                v = (int)i;   // A rows are read in place; the table is used when scattering
            } else {
                int j = __ldg(nbr + i * kk + k);
                if (j != -1) {
                    long jj = (long)j + (tpb > 0 ? (i / tpb) * (long)tpb : 0);
                    if (jj >= 0 && jj < n) v = (int)jj;   // out-of-range entries read as zero
                }
            }
        }
        s_nbr[r][k] = v;
        if (v >= 0) s_any[k] = 1;
    }
    __syncthreads();

    // acc holds one tap's partial sum; tot collects the taps (shorter fp32 chains, smaller error)
    float acc[4][4], tot[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) { acc[i][j] = 0.f; tot[i][j] = 0.f; }

    for (int k = 0; k < kk; ++k) {
        if (!s_any[k]) continue;
        const int wtap = (MODE == MODE_DGATHER) ? (kk - 1 - k) : k;
        const T* wk = w + (long)wtap * cin * cout;
        for (int c0 = 0; c0 < cred; c0 += BK) {
            // A tile: BM rows x BK channels, stored transposed As[c][row]
            for (int g = tid; g < BM * (BK / 4); g += NT) {
                int r = g % BM, cg = g / BM;
                int c = c0 + cg * 4;
                int j = s_nbr[r][k];
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (j >= 0 && c < cred) v = Cvt<T>::load4(a + (long)j * cred + c);
                As[cg * 4 + 0][r] = v.x;
                As[cg * 4 + 1][r] = v.y;
                As[cg * 4 + 2][r] = v.z;
                As[cg * 4 + 3][r] = v.w;
            }
            if (!TRANS_B) {
                // B[c][nn] = W[k][c0+c][n0+nn]; rows of W are contiguous along nn
                for (int g = tid; g < BK * (BN / 4); g += NT) {
                    int c = g / (BN / 4), ng = g % (BN / 4);
                    int nn = n0 + ng * 4;
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (c0 + c < cred) {
                        const T* src = wk + (long)(c0 + c) * cout + nn;
                        if (nn + 3 < cn && (cout & 3) == 0) {
                            v = Cvt<T>::load4(src);
                        } else {
                            if (nn + 0 < cn) v.x = Cvt<T>::load1(src + 0);
                            if (nn + 1 < cn) v.y = Cvt<T>::load1(src + 1);
                            if (nn + 2 < cn) v.z = Cvt<T>::load1(src + 2);
                            if (nn + 3 < cn) v.w = Cvt<T>::load1(src + 3);
                        }
                    }
                    *reinterpret_cast<float4*>(&Bs[c][ng * 4]) = v;
                }
            } else {
                // B[c][nn] = W[wtap][n0+nn][c0+c]; contiguous along c (the reduction index)
                for (int g = tid; g < BN * (BK / 4); g += NT) {
                    int nn = g % BN, cg = g / BN;
                    int c = c0 + cg * 4;
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (n0 + nn < cn && c < cred) {
                        const T* src = wk + (long)(n0 + nn) * cout + c;
                        if ((cout & 3) == 0) {
                            v = Cvt<T>::load4(src);
                        } else {
                            v.x = Cvt<T>::load1(src + 0);
                            if (c + 1 < cred) v.y = Cvt<T>::load1(src + 1);
                            if (c + 2 < cred) v.z = Cvt<T>::load1(src + 2);
                            if (c + 3 < cred) v.w = Cvt<T>::load1(src + 3);
                        }
                    }
                    Bs[cg * 4 + 0][nn] = v.x;
                    Bs[cg * 4 + 1][nn] = v.y;
                    Bs[cg * 4 + 2][nn] = v.z;
                    Bs[cg * 4 + 3][nn] = v.w;
                }
            }
            __syncthreads();
#pragma unroll
            for (int c = 0; c < BK; ++c) {
                float4 av = *reinterpret_cast<const float4*>(&As[c][ty * 4]);
                float4 bv = *reinterpret_cast<const float4*>(&Bs[c][tx * 4]);
                float ar[4] = {av.x, av.y, av.z, av.w};
                float br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
            }
            __syncthreads();
        }
        if (MODE == MODE_DSCATTER) {
            // scatter this tap's contribution of rows i to rows nbr[i,k] (+off) and restart
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                long row = row0 + ty * 4 + i;
                if (row < n) {
                    int j = __ldg(nbr + row * kk + k);
                    long jj = (j == -1) ? -1 : (long)j + (tpb > 0 ? (row / tpb) * (long)tpb : 0);
                    if (jj >= 0 && jj < n) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            int col = n0 + tx * 4 + q;
                            if (col < cn) atomicAdd(scatter_ws + jj * cn + col, acc[i][q]);
                        }
                    }
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[i][q] = 0.f;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int q = 0; q < 4; ++q) { tot[i][q] += acc[i][q]; acc[i][q] = 0.f; }
        }
    }
    if (MODE == MODE_DSCATTER) return;

    const int col = n0 + tx * 4;
    float b4[4] = {0.f, 0.f, 0.f, 0.f};
    if (MODE == MODE_FWD && bias != nullptr) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (col + q < cn) b4[q] = Cvt<T>::load1(bias + col + q);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        long row = row0 + ty * 4 + i;
        if (row >= n) continue;
        T* dst = out + row * cn + col;
        if (col + 3 < cn && (cn & 3) == 0) {
            Cvt<T>::store4(dst, make_float4(tot[i][0] + b4[0], tot[i][1] + b4[1],
                                            tot[i][2] + b4[2], tot[i][3] + b4[3]));
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if (col + q < cn) Cvt<T>::store1(dst + q, tot[i][q] + b4[q]);
        }
    }
}

// In the DSCATTER mode the A rows are the tile's own rows, so every tap is visited and entries that
// are -1 or out of range are skipped when the tap's result is scattered.

template <typename T>
__global__ void cast_ws_kernel(const float* __restrict__ ws, T* __restrict__ out, long total,
                               const int32_t* __restrict__ status) {
    if (status != nullptr && (__ldg(status) & SVTAD_TABLE_ASYMMETRIC) == 0) return;
    long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (i < total) Cvt<T>::store1(out + i, ws[i]);
}

template <typename T, int MODE>
static int launch_conv_simt(const ConvArgs& p, const int32_t* status, float* ws, cudaStream_t s) {
    const bool fwd = (MODE == MODE_FWD);
    const int cred = fwd ? p.cin : p.cout;
    const int cn = fwd ? p.cout : p.cin;
    const T* a = static_cast<const T*>(p.a);
    const T* w = static_cast<const T*>(p.w);
    const T* bias = static_cast<const T*>(p.bias);
    T* out = static_cast<T*>(p.out);
    // small problems: 32-row tiles so that more SMs get work
    long tiles64 = ((p.n + 63) / 64) * ((cn + 63) / 64);
    if (tiles64 >= 2 * 148) {
        dim3 grid((cn + 63) / 64, (unsigned)((p.n + 63) / 64));
        conv_simt_kernel<T, 64, 64, MODE><<<grid, 256, 0, s>>>(a, p.nbr, w, bias, out, ws, status,
                                                               (long)p.n, cred, cn, p.cin, p.cout, p.kk, p.tpb);
    } else {
        dim3 grid((cn + 63) / 64, (unsigned)((p.n + 31) / 32));
        conv_simt_kernel<T, 32, 64, MODE><<<grid, 128, 0, s>>>(a, p.nbr, w, bias, out, ws, status,
                                                               (long)p.n, cred, cn, p.cin, p.cout, p.kk, p.tpb);
    }
    SV_LAUNCH_CHECK("conv_simt_kernel");
    return SVTAD_OK;
}

template <int MODE>
static int dispatch_conv_simt(const ConvArgs& p, const int32_t* status, float* ws, cudaStream_t s) {
    switch (p.dtype) {
        case SVTAD_F32: return launch_conv_simt<float, MODE>(p, status, ws, s);
        case SVTAD_BF16: return launch_conv_simt<__nv_bfloat16, MODE>(p, status, ws, s);
        case SVTAD_F16: return launch_conv_simt<__half, MODE>(p, status, ws, s);
    }
    return set_error(SVTAD_ERR_UNSUPPORTED, "unknown dtype %d", p.dtype);
}

int simt_fwd(const ConvArgs& p, cudaStream_t s) {
    if (simt_fwd_f32_supported(p) && getenv("SVTAD_SIMT_FWD_GENERIC") == nullptr) return simt_fwd_f32(p, s);
    return dispatch_conv_simt<MODE_FWD>(p, nullptr, nullptr, s);
}

int simt_dgrad_gather(const ConvArgs& p, const int32_t* status, cudaStream_t s) {
    return dispatch_conv_simt<MODE_DGATHER>(p, status, nullptr, s);
}

int simt_dgrad_scatter(const ConvArgs& p, const int32_t* status, float* ws, cudaStream_t s) {
    long total = (long)p.n * p.cin;
    SV_CUDA(cudaMemsetAsync(ws, 0, (size_t)total * sizeof(float), s));
    int rc = dispatch_conv_simt<MODE_DSCATTER>(p, status, ws, s);
    if (rc) return rc;
    unsigned grid = (unsigned)((total + 255) / 256);
    switch (p.dtype) {
        case SVTAD_F32: cast_ws_kernel<float><<<grid, 256, 0, s>>>(ws, (float*)p.out, total, status); break;
        case SVTAD_BF16: cast_ws_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(ws, (__nv_bfloat16*)p.out, total, status); break;
        default: cast_ws_kernel<__half><<<grid, 256, 0, s>>>(ws, (__half*)p.out, total, status); break;
    }
    SV_LAUNCH_CHECK("cast_ws_kernel");
    return SVTAD_OK;
}

// ------------------------------------------------------------------------------------------
// weight gradient: gW[k] (cin x cout) = sum_i x[nbr[i,k]]^T . gy[i]; split over tokens
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
wgrad_simt_kernel(const T* __restrict__ gy, const T* __restrict__ x, const int32_t* __restrict__ nbr,
                  float* __restrict__ ws, long n, int cin, int cout, int kk, int tpb,
                  long rows_per_split, int tiles_m, int tiles_n) {
    constexpr int BM = 64, BN = 64;
    __shared__ __align__(16) float As[BK][BM + 4];
    __shared__ __align__(16) float Bs[BK][BN + 4];
    __shared__ int s_j[BK];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    int tile = blockIdx.x;
    const int tn = tile % tiles_n; tile /= tiles_n;
    const int tm = tile % tiles_m;
    const int k = tile / tiles_m;
    const int m0 = tm * BM, n0 = tn * BN;
    const long i_begin = (long)blockIdx.y * rows_per_split;
    const long i_end = min(n, i_begin + rows_per_split);

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (long i0 = i_begin; i0 < i_end; i0 += BK) {
        if (tid < BK) {
            long i = i0 + tid;
            int v = -1;
            if (i < i_end) {
                int j = __ldg(nbr + i * kk + k);
                if (j != -1) {
                    long jj = (long)j + (tpb > 0 ? (i / tpb) * (long)tpb : 0);
                    if (jj >= 0 && jj < n) v = (int)jj;
                }
            }
            s_j[tid] = v;
        }
        __syncthreads();
        {   // 16 tokens x 16 float4 groups = 256 loads, one per thread, for A and for B
            int t = tid / 16, g = tid % 16;
            int j = s_j[t];
            float4 av = make_float4(0.f, 0.f, 0.f, 0.f), bv = av;
            int c = m0 + g * 4;
            if (j >= 0 && c < cin) av = Cvt<T>::load4(x + (long)j * cin + c);   // cin % 4 == 0
            *reinterpret_cast<float4*>(&As[t][g * 4]) = av;
            int cc = n0 + g * 4;
            if (j >= 0) {
                const T* src = gy + (i0 + t) * cout + cc;
                if (cc + 3 < cout && (cout & 3) == 0) {
                    bv = Cvt<T>::load4(src);
                } else {
                    if (cc + 0 < cout) bv.x = Cvt<T>::load1(src + 0);
                    if (cc + 1 < cout) bv.y = Cvt<T>::load1(src + 1);
                    if (cc + 2 < cout) bv.z = Cvt<T>::load1(src + 2);
                    if (cc + 3 < cout) bv.w = Cvt<T>::load1(src + 3);
                }
            }
            *reinterpret_cast<float4*>(&Bs[t][g * 4]) = bv;
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < BK; ++c) {
            float4 av = *reinterpret_cast<const float4*>(&As[c][ty * 4]);
            float4 bv = *reinterpret_cast<const float4*>(&Bs[c][tx * 4]);
            float ar[4] = {av.x, av.y, av.z, av.w};
            float br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
        }
        __syncthreads();
    }
    float* dst = ws + (long)blockIdx.y * kk * cin * cout + (long)k * cin * cout;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int ci = m0 + ty * 4 + i;
        if (ci >= cin) continue;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            int co = n0 + tx * 4 + q;
            if (co < cout) dst[(long)ci * cout + co] = acc[i][q];
        }
    }
}

// column sums of gy over a chunk of rows: partial[split][co]
template <typename T>
__global__ void __launch_bounds__(256)
bias_partial_kernel(const T* __restrict__ gy, float* __restrict__ partial, long n, int cout,
                    long rows_per_split) {
    __shared__ float s[4][64];
    const int tx = threadIdx.x % 64, ty = threadIdx.x / 64;
    const long i_begin = (long)blockIdx.x * rows_per_split;
    const long i_end = min(n, i_begin + rows_per_split);
    for (int c0 = 0; c0 < cout; c0 += 64) {
        int co = c0 + tx;
        float sum = 0.f;
        if (co < cout)
            for (long i = i_begin + ty; i < i_end; i += 4) sum += Cvt<T>::load1(gy + i * cout + co);
        s[ty][tx] = sum;
        __syncthreads();
        if (ty == 0 && co < cout)
            partial[(long)blockIdx.x * cout + co] = (s[0][tx] + s[1][tx]) + (s[2][tx] + s[3][tx]);
        __syncthreads();
    }
}

// fixed-order reduction of the per-split partials, one rounding to T
template <typename T>
__global__ void wgrad_finalize_kernel(const float* __restrict__ ws_w, int splits_w,
                                      const float* __restrict__ ws_b, int splits_b,
                                      T* __restrict__ gw, T* __restrict__ gb, long n_w, int cout) {
    long e = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (e < n_w) {
        float sum = 0.f;
        for (int s = 0; s < splits_w; ++s) sum += ws_w[(long)s * n_w + e];
        Cvt<T>::store1(gw + e, sum);
    } else if (gb != nullptr && e < n_w + cout) {
        int co = (int)(e - n_w);
        float sum = 0.f;
        for (int s = 0; s < splits_b; ++s) sum += ws_b[(long)s * cout + co];
        Cvt<T>::store1(gb + co, sum);
    }
}

int bias_splits_for(int64_t n) {
    long s = (n + 127) / 128;
    return (int)(s < 1 ? 1 : (s > 296 ? 296 : s));
}

int bias_partial_launch(const void* gy, float* partial, int64_t n, int cout, int dtype, int splits,
                        cudaStream_t s) {
    long rps = (n + splits - 1) / splits;
    if (rps < 1) rps = 1;
    switch (dtype) {
        case SVTAD_F32: bias_partial_kernel<float><<<splits, 256, 0, s>>>((const float*)gy, partial, (long)n, cout, rps); break;
        case SVTAD_BF16: bias_partial_kernel<__nv_bfloat16><<<splits, 256, 0, s>>>((const __nv_bfloat16*)gy, partial, (long)n, cout, rps); break;
        default: bias_partial_kernel<__half><<<splits, 256, 0, s>>>((const __half*)gy, partial, (long)n, cout, rps); break;
    }
    SV_LAUNCH_CHECK("bias_partial_kernel");
    return SVTAD_OK;
}

int wgrad_finalize_launch(const float* ws_w, int splits_w, const float* ws_b, int splits_b, void* gw,
                          void* gb, int64_t n_w, int cout, int dtype, cudaStream_t s) {
    long total = n_w + (gb ? cout : 0);
    unsigned grid = (unsigned)((total + 255) / 256);
    switch (dtype) {
        case SVTAD_F32: wgrad_finalize_kernel<float><<<grid, 256, 0, s>>>(ws_w, splits_w, ws_b, splits_b, (float*)gw, (float*)gb, (long)n_w, cout); break;
        case SVTAD_BF16: wgrad_finalize_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(ws_w, splits_w, ws_b, splits_b, (__nv_bfloat16*)gw, (__nv_bfloat16*)gb, (long)n_w, cout); break;
        default: wgrad_finalize_kernel<__half><<<grid, 256, 0, s>>>(ws_w, splits_w, ws_b, splits_b, (__half*)gw, (__half*)gb, (long)n_w, cout); break;
    }
    SV_LAUNCH_CHECK("wgrad_finalize_kernel");
    return SVTAD_OK;
}

static int simt_wgrad_splits(int64_t n, int cin, int cout, int kk) {
    long tiles = (long)kk * ((cin + 63) / 64) * ((cout + 63) / 64);
    long want = (2 * 148 + tiles - 1) / tiles;
    long max_by_rows = (n + 63) / 64;
    long s = want < max_by_rows ? want : max_by_rows;
    if (s < 1) s = 1;
    if (s > 64) s = 64;
    return (int)s;
}

size_t simt_wgrad_ws_bytes(int64_t n, int cin, int cout, int kk) {
    size_t w = (size_t)simt_wgrad_splits(n, cin, cout, kk) * kk * cin * cout * sizeof(float);
    size_t b = (size_t)bias_splits_for(n) * cout * sizeof(float);
    return align_up(w, 256) + align_up(b, 256);
}

int simt_wgrad(const void* gy, const void* x, const int32_t* nbr, void* gw, void* gb, int64_t n,
               int cin, int cout, int kk, int tpb, int dtype, void* ws, size_t ws_bytes,
               cudaStream_t s) {
    if (ws_bytes < simt_wgrad_ws_bytes(n, cin, cout, kk))
        return set_error(SVTAD_ERR_WORKSPACE, "svtad_conv_wgrad: workspace %zu < %zu bytes", ws_bytes,
                         simt_wgrad_ws_bytes(n, cin, cout, kk));
    const int splits = simt_wgrad_splits(n, cin, cout, kk);
    const long n_w = (long)kk * cin * cout;
    float* ws_w = static_cast<float*>(ws);
    float* ws_b = reinterpret_cast<float*>(static_cast<char*>(ws) + align_up((size_t)splits * n_w * sizeof(float), 256));
    const int tiles_m = (cin + 63) / 64, tiles_n = (cout + 63) / 64;
    long rps = ((n + splits - 1) / splits + BK - 1) / BK * BK;
    if (rps < BK) rps = BK;
    dim3 grid((unsigned)(kk * tiles_m * tiles_n), (unsigned)splits);
    switch (dtype) {
        case SVTAD_F32: wgrad_simt_kernel<float><<<grid, 256, 0, s>>>((const float*)gy, (const float*)x, nbr, ws_w, (long)n, cin, cout, kk, tpb, rps, tiles_m, tiles_n); break;
        case SVTAD_BF16: wgrad_simt_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)gy, (const __nv_bfloat16*)x, nbr, ws_w, (long)n, cin, cout, kk, tpb, rps, tiles_m, tiles_n); break;
        default: wgrad_simt_kernel<__half><<<grid, 256, 0, s>>>((const __half*)gy, (const __half*)x, nbr, ws_w, (long)n, cin, cout, kk, tpb, rps, tiles_m, tiles_n); break;
    }
    SV_LAUNCH_CHECK("wgrad_simt_kernel");
    int splits_b = 0;
    if (gb != nullptr) {
        splits_b = bias_splits_for(n);
        int rc = bias_partial_launch(gy, ws_b, n, cout, dtype, splits_b, s);
        if (rc) return rc;
    }
    return wgrad_finalize_launch(ws_w, splits, ws_b, splits_b, gw, gb, n_w, cout, dtype, s);
}

}  // namespace svtad
