// fp32 forward of SparseConv2D on the CUDA cores, built for the FFMA rate.
//
// fp32 tensors cannot go through the tensor cores without losing the 1e-5 the reference's fp32 path holds
// (opentad/models/bricks/2d_sparse_v3.cu:545-651, a 32 x 32 shared-memory tile kernel with two __syncthreads per
// 32-deep step; for C_in >= 128 the reference takes implicit_gemm_v2.cu:197-300, gather + cuBLAS SGEMM + reduce).
// This kernel is a gather-GEMM with
//   * 64 x 64 output tiles, 128 threads, 8 x 4 accumulators per thread (10.7 FMAs per shared-memory load),
//   * 32-deep K steps through a three-stage cp.async ring: gathered rows land as [row][channel] (16-byte copies,
//     -1 rows zero-filled without touching memory), weight rows as [channel][column],
//   * strict fp32 FMA accumulation in (tap, channel) ascending order inside a tap group,
//   * taps that no row of the tile uses are skipped,
//   * small problems: the K steps are split over the G CTAs of a thread-block cluster, which sum their tiles through
//     distributed shared memory in a fixed order (deterministic, no atomics) - so that a 784-row call still
//     spreads over the whole GPU.  The (tap, channel block) steps are dealt out evenly, whatever the tap count.
#include <cstdlib>

#include "common.cuh"

namespace svtad {

constexpr int F_BK = 32, F_STAGES = 3;
constexpr int F_ASTR = F_BK + 4;          // floats per gathered row in shared memory (144 B: 16-byte aligned, conflict-free)
constexpr int F_MAX_KK = 49;

__device__ __forceinline__ void f_cp16(uint32_t dst, const void* src, uint32_t bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}

template <int F_BM, int F_BN>
struct FwdSmem {
    float a[F_STAGES][F_BM * F_ASTR];
    float b[F_STAGES][F_BK * F_BN];
    int nbr[F_BM * F_MAX_KK];
    int any[F_MAX_KK];
    int n_act;
};

// G = CTAs of a cluster that share a tile's taps; the tile is F_BM x F_BN, every thread owns RPT rows x 4 columns of
// it (F_THREADS = F_BM * F_BN / (4 * RPT)): 8 rows for large calls (fewest shared-memory loads per FMA), 4 rows for
// small ones (twice the warps to hide latency with).
template <int G, int F_BM, int F_BN, int RPT>
__global__ void __launch_bounds__(F_BM * F_BN / (4 * RPT))
conv_fwd_f32_kernel(const float* __restrict__ x, const int32_t* __restrict__ nbr, const float* __restrict__ w,
                    const float* __restrict__ bias, float* __restrict__ out, long n, int cin, int cout, int kk,
                    int tpb, int tiles_n) {
    constexpr int F_THREADS = F_BM * F_BN / (4 * RPT);
    constexpr int TXN = F_BN / 4;                      // threads along the columns
    constexpr int TYN = F_THREADS / TXN;               // threads along the rows: thread ty owns rows ty + TYN * i
    constexpr int F_RSTR = F_BN + 4;                   // row stride of the tile parked for the cluster reduction
    extern __shared__ __align__(16) unsigned char f_smem_raw[];
    FwdSmem<F_BM, F_BN>& sm = *reinterpret_cast<FwdSmem<F_BM, F_BN>*>(f_smem_raw);
    const int tid = threadIdx.x;
    const int tx = tid % TXN, ty = tid / TXN;          // columns tx * 4 .. + 3, rows ty + TYN * i
    const int tile = blockIdx.x / G, grp = blockIdx.x % G;
    const long row0 = (long)(tile / tiles_n) * F_BM;
    const int n0 = (tile % tiles_n) * F_BN;

    for (int t = tid; t < kk; t += F_THREADS) sm.any[t] = 0;
    __syncthreads();
    for (int e = tid; e < F_BM * kk; e += F_THREADS) {
        const int r = e / kk, k = e - r * kk;
        const long i = row0 + r;
        int v = -1;
        if (i < n) {
            const int j = __ldg(nbr + i * kk + k);
            if (j != -1) {
                const long jj = (long)j + (tpb > 0 ? (i / tpb) * (long)tpb : 0);
                if (jj >= 0 && jj < n) v = (int)jj;
            }
        }
        sm.nbr[r * kk + k] = v;
        if (v >= 0) sm.any[k] = 1;
    }
    __syncthreads();

    // The K steps of the tile are (tap, 32-channel block) for every tap that some row uses, taps ascending; the G
    // CTAs of the cluster take equal contiguous shares of them (a share may start in the middle of a tap).
    const int cblk = (cin + F_BK - 1) / F_BK;
    if (tid == 0) {
        int m = 0;
        for (int k = 0; k < kk; ++k)
            if (sm.any[k]) sm.any[m++] = k;           // compacted in place: any[0 .. m) = the taps in use (m <= k always)
        sm.n_act = m;
    }
    __syncthreads();
    const int total_steps = sm.n_act * cblk;
    const int st_lo = (int)((long)grp * total_steps / G), st_hi = (int)((long)(grp + 1) * total_steps / G);
    const int steps = st_hi - st_lo;
    int ld_t = st_lo / cblk, ld_c = (st_lo % cblk) * F_BK;     // position of the loader: index into any[], channel
    auto load_stage = [&](int stage) {
        // A: F_BM rows x F_BK / 4 chunks of 16 B; B: F_BK channel rows x F_BN / 4 chunks of 16 B
        const uint32_t a_base = (uint32_t)__cvta_generic_to_shared(sm.a[stage]);
        const uint32_t b_base = (uint32_t)__cvta_generic_to_shared(sm.b[stage]);
        const int ld_k = sm.any[ld_t];
#pragma unroll
        for (int q = 0; q < (F_BM * F_BK / 4) / F_THREADS; ++q) {
            const int g = tid + q * F_THREADS;
            const int r = g / (F_BK / 4), ch = g % (F_BK / 4);
            const int c = ld_c + ch * 4;
            const int j = sm.nbr[r * kk + ld_k];
            const bool ok = j >= 0 && c < cin;
            f_cp16(a_base + (r * F_ASTR + ch * 4) * 4, ok ? x + (long)j * cin + c : x, ok ? 16u : 0u);
        }
#pragma unroll
        for (int q = 0; q < (F_BK * F_BN / 4) / F_THREADS; ++q) {
            const int g = tid + q * F_THREADS;
            const int cr = g / TXN, ch = g % TXN;
            const int c = ld_c + cr, nn = n0 + ch * 4;
            const bool ok = c < cin && nn < cout;
            f_cp16(b_base + (cr * F_BN + ch * 4) * 4, ok ? w + ((long)ld_k * cin + c) * cout + nn : w, ok ? 16u : 0u);
        }
        ld_c += F_BK;
        if (ld_c >= cin) { ld_c = 0; ++ld_t; }
    };

    float acc[RPT][4];
#pragma unroll
    for (int i = 0; i < RPT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    // prologue: F_STAGES - 1 steps in flight (one commit group per step, empty or not)
#pragma unroll
    for (int s = 0; s < F_STAGES - 1; ++s) {
        if (s < steps) load_stage(s);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int st = 0; st < steps; ++st) {
        asm volatile("cp.async.wait_group %0;" ::"n"(F_STAGES - 2) : "memory");
        if (F_THREADS == 32) __syncwarp(); else __syncthreads();   // step st has landed for every thread; the buffer refilled below is no longer read
        if (st + F_STAGES - 1 < steps) load_stage((st + F_STAGES - 1) % F_STAGES);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const float* as = sm.a[st % F_STAGES];
        const float* bs = sm.b[st % F_STAGES];
#pragma unroll
        for (int c4 = 0; c4 < F_BK; c4 += 4) {
            float4 av[RPT];
#pragma unroll
            for (int i = 0; i < RPT; ++i) av[i] = *reinterpret_cast<const float4*>(as + (ty + TYN * i) * F_ASTR + c4);
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                const float4 bv = *reinterpret_cast<const float4*>(bs + (c4 + cc) * F_BN + tx * 4);
#pragma unroll
                for (int i = 0; i < RPT; ++i) {
                    const float a = cc == 0 ? av[i].x : cc == 1 ? av[i].y : cc == 2 ? av[i].z : av[i].w;
                    acc[i][0] = fmaf(a, bv.x, acc[i][0]);
                    acc[i][1] = fmaf(a, bv.y, acc[i][1]);
                    acc[i][2] = fmaf(a, bv.z, acc[i][2]);
                    acc[i][3] = fmaf(a, bv.w, acc[i][3]);
                }
            }
        }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");

    const int col = n0 + tx * 4;
    if (G == 1) {
        float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (bias != nullptr && col < cout) b4 = __ldg(reinterpret_cast<const float4*>(bias + col));
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
            const long row = row0 + ty + TYN * i;
            if (row < n && col < cout)
                *reinterpret_cast<float4*>(out + row * cout + col) =
                    make_float4(acc[i][0] + b4.x, acc[i][1] + b4.y, acc[i][2] + b4.z, acc[i][3] + b4.w);
        }
        return;
    }
    // ---- the tap groups of a tile sum their partial tiles through distributed shared memory, group 0 first
    __syncthreads();                              // everyone is done with the stage ring: park the tile in it
    float* red = reinterpret_cast<float*>(f_smem_raw);
#pragma unroll
    for (int i = 0; i < RPT; ++i)
        *reinterpret_cast<float4*>(red + (ty + TYN * i) * F_RSTR + tx * 4) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    {
        constexpr int ROWS = F_BM / G;            // rows of the tile this CTA finishes
        const uint32_t local = (uint32_t)__cvta_generic_to_shared(red);
        for (int e = tid; e < ROWS * (F_BN / 4); e += F_THREADS) {
            const int r = grp * ROWS + e / (F_BN / 4), c4 = (e % (F_BN / 4)) * 4;
            const long row = row0 + r;
            const int cc = n0 + c4;
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int p = 0; p < G; ++p) {
                uint32_t peer;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer) : "r"(local + (r * F_RSTR + c4) * 4), "r"(p));
                float4 v;
                asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                             : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(peer) : "memory");
                s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
            }
            if (row < n && cc < cout) {
                float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
                if (bias != nullptr) b4 = __ldg(reinterpret_cast<const float4*>(bias + cc));
                *reinterpret_cast<float4*>(out + row * cout + cc) = make_float4(s.x + b4.x, s.y + b4.y, s.z + b4.z, s.w + b4.w);
            }
        }
    }
    // nobody leaves while a peer may still read its shared memory
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <int G, int F_BM, int F_BN, int RPT>
static int launch_fwd_f32(const ConvArgs& p, cudaStream_t s) {
    auto kern = conv_fwd_f32_kernel<G, F_BM, F_BN, RPT>;
    const int tiles_m = (int)((p.n + F_BM - 1) / F_BM), tiles_n = (p.cout + F_BN - 1) / F_BN;
    constexpr int F_THREADS = F_BM * F_BN / (4 * RPT);
    const size_t smem = sizeof(FwdSmem<F_BM, F_BN>);
    static bool attr_set[64] = {false};
    int dev = 0;
    SV_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        SV_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(tiles_m * tiles_n * G));
    cfg.blockDim = dim3(F_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = G;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = G > 1 ? 1 : 0;
    SV_CUDA(cudaLaunchKernelEx(&cfg, kern, (const float*)p.a, p.nbr, (const float*)p.w, (const float*)p.bias, (float*)p.out,
                               (long)p.n, p.cin, p.cout, p.kk, p.tpb, tiles_n));
    return SVTAD_OK;
}

bool simt_fwd_f32_supported(const ConvArgs& p) {
    auto al = [](const void* q) { return q == nullptr || (reinterpret_cast<uintptr_t>(q) % 16) == 0; };
    return p.dtype == SVTAD_F32 && p.cin % 4 == 0 && p.cout % 4 == 0 && p.kk <= F_MAX_KK && al(p.a) && al(p.w) &&
           al(p.bias) && al(p.out);
}

// fp32 forward; the caller has checked simt_fwd_f32_supported().
int simt_fwd_f32(const ConvArgs& p, cudaStream_t s) {
    const long tiles = ((p.n + 63) / 64) * ((p.cout + 63) / 64);
    if (tiles >= 2 * 148) return launch_fwd_f32<1, 64, 64, 8>(p, s);
    // small call: the K steps split over a cluster while that brings more SMs into play (148 on a B200, a few
    // CTAs each)
    int g = 1;
    while (g < 8 && tiles * g < 2 * 148) g *= 2;
    switch (g) {
        case 1: return launch_fwd_f32<1, 64, 64, 8>(p, s);
        case 2: return launch_fwd_f32<2, 64, 64, 8>(p, s);
        case 4: return launch_fwd_f32<4, 64, 64, 8>(p, s);
        default: return launch_fwd_f32<8, 64, 64, 8>(p, s);
    }
}

// ---------------------------------------------------------------------------------------------------------
// FFMA rate of the device: what the CUDA-core kernels are measured against
// ---------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) ffma_peak_kernel(float* out, int iters, float seed) {
    float a[8], b = seed, c = 1.0f - seed * 0.5f;
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = seed + i;
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
#pragma unroll
            for (int i = 0; i < 8; ++i) a[i] = fmaf(a[i], b, c);     // 8 independent chains per thread
        }
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += a[i];
    if (s == 123.456f) out[0] = s;     // never true; keeps the loop alive
}

}  // namespace svtad

using namespace svtad;

// Launches `launches` timing kernels of iters * 64 FMAs per thread on ctas * 256 threads.  The caller times the
// launch (events on `stream`) and divides: flops = 2 * 64 * iters * ctas * 256 per launch.
extern "C" int svtad_ffma_probe(int ctas, int iters, float* scratch, void* stream) {
    SV_CHECK_ARG(ctas > 0 && iters > 0 && scratch != nullptr, "svtad_ffma_probe: bad arguments");
    ffma_peak_kernel<<<ctas, 256, 0, (cudaStream_t)stream>>>(scratch, iters, 0.999f);
    SV_LAUNCH_CHECK("ffma_peak_kernel");
    return SVTAD_OK;
}
