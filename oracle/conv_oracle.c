/*
 * CPU oracle for SparseConv2D (TEST INFRASTRUCTURE, not product code).
 *
 * A plain-C restatement of the arithmetic of the reference's CUDA kernels, used only by
 * tests, the smoke check and the benchmark's CPU-baseline / reference legs:
 *
 *   forward   y[i,co]  = bias[co] + sum_k sum_ci x[nbr[i,k]+off(i), ci] * W[k,ci,co]
 *             (opentad/models/bricks/2d_sparse_v3.cu:574-629 for the (k, ci) order;
 *              implicit_gemm_v2.cu:63-77 for "-1 reads as zero" and :146-159 for
 *              "bias added in the accumulator type, one rounding")
 *   dgrad     gx[j,ci] = sum over (i,k) with nbr[i,k]+off(i)==j of sum_co gy[i,co]*W[k,ci,co]
 *             (2d_sparse_v3.cu:679-707; scatter form, valid for any table)
 *   wgrad     gW[k,ci,co] = sum_i [nbr[i,k]!=-1] x[nbr[i,k]+off(i), ci] * gy[i,co]
 *             (2d_sparse_v3.cu:733-744)
 *   bias grad gb[co] = sum_i gy[i,co]      (sparse_conv_layer.py:119-121)
 *
 *   off(i) = (i / tokens_per_batch) * tokens_per_batch when tokens_per_batch > 0, else 0
 *   (per row, as in 2d_sparse_v3.cu:674-677 and :728-731).
 *
 * Two flavours of every function: *_f32 accumulates in float like the reference (and is
 * the one that is timed as the CPU baseline, OpenMP over all host threads), *_f64
 * accumulates and returns double and is the ground truth the parity tests measure
 * errors against.  Inputs are always float arrays (bf16/fp16 tensors are widened
 * exactly by the caller).
 *
 * There is no CPU implementation of this op in the reference; parity of this file is
 * pinned by tests/golden/conv_*.npz (dense scatter -> conv2d -> gather identity computed
 * with torch on CPU) and, on a GPU box, by the reference's own CUDA extension.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#if defined(__x86_64__) && defined(__GNUC__)
#define SV_CLONES __attribute__((target_clones("avx512f", "avx2,fma", "default")))
#else
#define SV_CLONES
#endif

static inline int64_t sv_off(int64_t i, int tpb) { return tpb > 0 ? (i / tpb) * (int64_t)tpb : 0; }

#define ROWS_BLK 8

#define DEFINE_ORACLE(SUF, ACC)                                                                  \
    SV_CLONES void svtad_oracle_fwd_##SUF(const float* x, const int32_t* nbr, const float* w,  \
                                          const float* bias, ACC* y, int64_t n, int cin,      \
                                          int cout, int kk, int tpb) {                          \
        int64_t nblk = (n + ROWS_BLK - 1) / ROWS_BLK;                                            \
        _Pragma("omp parallel")                                                                  \
        {                                                                                        \
            ACC* acc = (ACC*)malloc(sizeof(ACC) * ROWS_BLK * (size_t)cout);                      \
            _Pragma("omp for schedule(dynamic, 4)")                                              \
            for (int64_t b = 0; b < nblk; ++b) {                                                 \
                int64_t i0 = b * ROWS_BLK;                                                       \
                int rows = (int)((n - i0) < ROWS_BLK ? (n - i0) : ROWS_BLK);                     \
                memset(acc, 0, sizeof(ACC) * ROWS_BLK * (size_t)cout);                           \
                for (int k = 0; k < kk; ++k) {                                                   \
                    const float* xr[ROWS_BLK];                                                   \
                    int any = 0;                                                                 \
                    for (int r = 0; r < rows; ++r) {                                             \
                        int32_t j = nbr[(i0 + r) * kk + k];                                      \
                        xr[r] = (j == -1) ? 0 : x + (j + sv_off(i0 + r, tpb)) * (int64_t)cin;    \
                        any |= (j != -1);                                                        \
                    }                                                                            \
                    if (!any) continue;                                                          \
                    for (int ci = 0; ci < cin; ++ci) {                                           \
                        const float* wr = w + ((int64_t)k * cin + ci) * cout;                    \
                        for (int r = 0; r < rows; ++r) {                                         \
                            if (!xr[r]) continue;                                                \
                            ACC a = (ACC)xr[r][ci];                                              \
                            ACC* ar = acc + (size_t)r * cout;                                    \
                            for (int co = 0; co < cout; ++co) ar[co] += a * (ACC)wr[co];         \
                        }                                                                        \
                    }                                                                            \
                }                                                                                \
                for (int r = 0; r < rows; ++r)                                                   \
                    for (int co = 0; co < cout; ++co)                                            \
                        y[(i0 + r) * (int64_t)cout + co] =                                       \
                            acc[(size_t)r * cout + co] + (bias ? (ACC)bias[co] : (ACC)0);        \
            }                                                                                    \
            free(acc);                                                                           \
        }                                                                                        \
    }                                                                                            \
                                                                                                 \
    SV_CLONES void svtad_oracle_dgrad_##SUF(const float* gy, const int32_t* nbr, const float* w,\
                                            ACC* gx, int64_t n, int cin, int cout, int kk,     \
                                            int tpb) {                                           \
        /* inverse lists: for every target row j the (i,k) pairs that read it, i ascending */   \
        int64_t* start = (int64_t*)calloc((size_t)n + 1, sizeof(int64_t));                       \
        for (int64_t i = 0; i < n; ++i)                                                          \
            for (int k = 0; k < kk; ++k) {                                                       \
                int32_t j = nbr[i * kk + k];                                                     \
                if (j != -1) start[j + sv_off(i, tpb) + 1]++;                                    \
            }                                                                                    \
        for (int64_t j = 0; j < n; ++j) start[j + 1] += start[j];                                \
        int64_t nnz = start[n];                                                                  \
        int64_t* fill = (int64_t*)malloc(sizeof(int64_t) * ((size_t)n + 1));                     \
        memcpy(fill, start, sizeof(int64_t) * ((size_t)n + 1));                                  \
        int64_t* src = (int64_t*)malloc(sizeof(int64_t) * (size_t)(nnz ? nnz : 1));              \
        for (int64_t i = 0; i < n; ++i)                                                          \
            for (int k = 0; k < kk; ++k) {                                                       \
                int32_t j = nbr[i * kk + k];                                                     \
                if (j != -1) src[fill[j + sv_off(i, tpb)]++] = i * kk + k;                       \
            }                                                                                    \
        _Pragma("omp parallel for schedule(dynamic, 16)")                                        \
        for (int64_t j = 0; j < n; ++j) {                                                        \
            ACC* out = gx + j * (int64_t)cin;                                                    \
            for (int ci = 0; ci < cin; ++ci) out[ci] = (ACC)0;                                   \
            for (int64_t e = start[j]; e < start[j + 1]; ++e) {                                  \
                int64_t i = src[e] / kk;                                                         \
                int k = (int)(src[e] % kk);                                                      \
                const float* g = gy + i * (int64_t)cout;                                         \
                for (int ci = 0; ci < cin; ++ci) {                                               \
                    const float* wr = w + ((int64_t)k * cin + ci) * cout;                        \
                    ACC s = (ACC)0;                                                              \
                    for (int co = 0; co < cout; ++co) s += (ACC)g[co] * (ACC)wr[co];             \
                    out[ci] += s;                                                                \
                }                                                                                \
            }                                                                                    \
        }                                                                                        \
        free(start); free(fill); free(src);                                                      \
    }                                                                                            \
                                                                                                 \
    SV_CLONES void svtad_oracle_wgrad_##SUF(const float* gy, const float* x, const int32_t* nbr,\
                                            ACC* gw, ACC* gb, int64_t n, int cin, int cout,     \
                                            int kk, int tpb) {                                   \
        const int CB = 8;                                                                        \
        int ncb = (cin + CB - 1) / CB;                                                           \
        _Pragma("omp parallel")                                                                  \
        {                                                                                        \
            ACC* acc = (ACC*)malloc(sizeof(ACC) * CB * (size_t)cout);                            \
            _Pragma("omp for schedule(dynamic, 1) collapse(2)")                                  \
            for (int k = 0; k < kk; ++k)                                                         \
                for (int cb = 0; cb < ncb; ++cb) {                                               \
                    int c0 = cb * CB;                                                            \
                    int nc = (cin - c0) < CB ? (cin - c0) : CB;                                  \
                    memset(acc, 0, sizeof(ACC) * CB * (size_t)cout);                             \
                    for (int64_t i = 0; i < n; ++i) {                                            \
                        int32_t j = nbr[i * kk + k];                                             \
                        if (j == -1) continue;                                                   \
                        const float* xr = x + (j + sv_off(i, tpb)) * (int64_t)cin + c0;          \
                        const float* g = gy + i * (int64_t)cout;                                 \
                        for (int c = 0; c < nc; ++c) {                                           \
                            ACC a = (ACC)xr[c];                                                  \
                            ACC* ar = acc + (size_t)c * cout;                                    \
                            for (int co = 0; co < cout; ++co) ar[co] += a * (ACC)g[co];          \
                        }                                                                        \
                    }                                                                            \
                    for (int c = 0; c < nc; ++c)                                                 \
                        memcpy(gw + ((int64_t)k * cin + c0 + c) * cout, acc + (size_t)c * cout,  \
                               sizeof(ACC) * (size_t)cout);                                      \
                }                                                                                \
            free(acc);                                                                           \
        }                                                                                        \
        if (gb) {                                                                                \
            for (int co = 0; co < cout; ++co) gb[co] = (ACC)0;                                   \
            for (int64_t i = 0; i < n; ++i)                                                      \
                for (int co = 0; co < cout; ++co) gb[co] += (ACC)gy[i * (int64_t)cout + co];     \
        }                                                                                        \
    }

DEFINE_ORACLE(f32, float)
DEFINE_ORACLE(f64, double)


/*
 * Row-subset flavour of the input gradient (double accumulate): gx_sel[r,:] = gx[sel[r],:] for the
 * `nsel` target rows listed in `sel`, computed from the same scatter-form definition as above
 * (2d_sparse_v3.cu:679-707) without evaluating the other rows.  Lets full-size problems be checked
 * on a sample of their rows in seconds.
 */
SV_CLONES void svtad_oracle_dgrad_rows_f64(const float* gy, const int32_t* nbr, const float* w, double* gx_sel,
                                           const int64_t* sel, int64_t nsel, int64_t n, int cin, int cout,
                                           int kk, int tpb) {
    /* position of every selected target row in `sel`, -1 for the rest */
    int64_t* pos = (int64_t*)malloc(sizeof(int64_t) * (size_t)(n ? n : 1));
    for (int64_t j = 0; j < n; ++j) pos[j] = -1;
    for (int64_t r = 0; r < nsel; ++r) pos[sel[r]] = r;
    int64_t* start = (int64_t*)calloc((size_t)nsel + 1, sizeof(int64_t));
    for (int64_t i = 0; i < n; ++i)
        for (int k = 0; k < kk; ++k) {
            int32_t j = nbr[i * kk + k];
            if (j != -1 && pos[j + sv_off(i, tpb)] >= 0) start[pos[j + sv_off(i, tpb)] + 1]++;
        }
    for (int64_t r = 0; r < nsel; ++r) start[r + 1] += start[r];
    int64_t nnz = start[nsel];
    int64_t* fill = (int64_t*)malloc(sizeof(int64_t) * ((size_t)nsel + 1));
    memcpy(fill, start, sizeof(int64_t) * ((size_t)nsel + 1));
    int64_t* src = (int64_t*)malloc(sizeof(int64_t) * (size_t)(nnz ? nnz : 1));
    for (int64_t i = 0; i < n; ++i)
        for (int k = 0; k < kk; ++k) {
            int32_t j = nbr[i * kk + k];
            if (j != -1 && pos[j + sv_off(i, tpb)] >= 0) src[fill[pos[j + sv_off(i, tpb)]]++] = i * kk + k;
        }
    _Pragma("omp parallel for schedule(dynamic, 4)")
    for (int64_t r = 0; r < nsel; ++r) {
        double* out = gx_sel + r * (int64_t)cin;
        for (int ci = 0; ci < cin; ++ci) out[ci] = 0.0;
        for (int64_t e = start[r]; e < start[r + 1]; ++e) {
            int64_t i = src[e] / kk;
            int k = (int)(src[e] % kk);
            const float* g = gy + i * (int64_t)cout;
            for (int ci = 0; ci < cin; ++ci) {
                const float* wr = w + ((int64_t)k * cin + ci) * cout;
                double s = 0.0;
                for (int co = 0; co < cout; ++co) s += (double)g[co] * (double)wr[co];
                out[ci] += s;
            }
        }
    }
    free(pos); free(start); free(fill); free(src);
}

int svtad_oracle_version(void) { return 3; }

/* Number of OpenMP threads the timed functions use (launchers such as torchrun export OMP_NUM_THREADS=1). */
#ifdef _OPENMP
#include <omp.h>
void svtad_oracle_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }
int svtad_oracle_get_threads(void) { return omp_get_max_threads(); }
#else
void svtad_oracle_set_threads(int n) { (void)n; }
int svtad_oracle_get_threads(void) { return 1; }
#endif
