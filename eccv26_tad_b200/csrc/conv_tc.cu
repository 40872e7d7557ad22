// Host side of the tcgen05 / TMEM SparseConv2D path: the device error word, tensor-map encoding, tile
// and split planning, and the dispatch between the kernel families
//   conv_tc_hybrid.cu   one CTA per tile: gathered rows by per-warp cp.async, weight / gy tiles by TMA
//   conv_tc_pair.cu     forward / dgrad on CTA pairs (cta_group::2) once row tiles outnumber the SMs
// They replace opentad/models/bricks/implicit_gemm_v2.cu:197-417 (gather kernel + cuBLAS batched GEMM +
// reduce kernel) and the atomic backward kernels opentad/models/bricks/2d_sparse_v3.cu:656-745.
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <map>
#include <mutex>
#include <utility>

#include "tc_common.cuh"

namespace svtad {

// Set (once, first code wins) by a bounded wait that gave up; read and cleared by svtad_device_error().
__device__ int g_tc_error = 0;

int* tc_error_ptr() {
    static thread_local int cached_dev = -1;
    static thread_local int* cached = nullptr;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    if (dev != cached_dev) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_tc_error) != cudaSuccess) return nullptr;
        cached = static_cast<int*>(p);
        cached_dev = dev;
    }
    return cached;
}

int tc_read_error(int32_t* code_out) {
    int v = 0;
    SV_CUDA(cudaDeviceSynchronize());
    SV_CUDA(cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int)));
    if (v != 0) {
        int zero = 0;
        SV_CUDA(cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int)));
    }
    *code_out = v;
    return SVTAD_OK;
}

// SM count of the current device (cached per device ordinal; a racing first call stores the same value)
int tc_num_sms() {
    constexpr int MAX_DEV = 64;
    static int cached[MAX_DEV] = {0};
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev >= 0 && dev < MAX_DEV && cached[dev] > 0) return cached[dev];
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    if (dev >= 0 && dev < MAX_DEV) cached[dev] = v;
    return v;
}

// How many kernels the caller expects to share the GPU (svtad_set_concurrency; SVTAD_CONCURRENCY for a start value).
// The planning below then counts on SMs / share multiprocessors per kernel: fewer, longer CTAs (wide column blocks,
// several row tiles per persistent CTA, fewer token splits), which costs a kernel latency when it runs alone but
// saves SM time - every CTA pays about 7 us of set-up, first-operand latency and epilogue whatever its share of the
// work - when the SMs are contended anyway.
static std::atomic<int>& tc_share_ref() {
    static std::atomic<int> v{[] {
        const char* e = getenv("SVTAD_CONCURRENCY");
        int x = (e != nullptr && *e) ? atoi(e) : 1;
        return x < 1 ? 1 : (x > 16 ? 16 : x);
    }()};
    return v;
}
int tc_set_share(int n) {
    if (n < 1) n = 1;
    if (n > 16) n = 16;
    return tc_share_ref().exchange(n);
}
int tc_get_share() { return tc_share_ref().load(); }
// a lower bound on the share for the calling thread's next launches (svtad_conv_bwd runs its two kernels side by
// side and plans each for half the GPU even when the caller gave no hint)
static thread_local int t_share_floor = 1;
int tc_set_share_floor(int n) {
    const int old = t_share_floor;
    t_share_floor = n < 1 ? 1 : n;
    return old;
}
int tc_plan_sms() {
    const int g = tc_share_ref().load();
    int v = tc_num_sms() / (g > t_share_floor ? g : t_share_floor);
    return v < 8 ? 8 : v;
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (kernel, device) instead of before every launch;
// the value only ever grows
int tc_ensure_smem(const void* kern, size_t bytes) {
    static std::mutex mu;
    static std::map<std::pair<const void*, int>, size_t> done;
    int dev = 0;
    SV_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> hold(mu);
    auto key = std::make_pair(kern, dev);
    auto it = done.find(key);
    if (it != done.end() && it->second >= bytes) return SVTAD_OK;
    SV_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    done[key] = bytes;
    return SVTAD_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

int tc_make_map(CUtensorMap* map, int rank, const void* base, const uint64_t* dims, const uint32_t* box, int fp16) {
    return tc_make_map_sw(map, rank, base, dims, box, fp16, 128);
}

int tc_make_map_sw(CUtensorMap* map, int rank, const void* base, const uint64_t* dims, const uint32_t* box, int fp16,
                   int swizzle_bytes) {
    // A descriptor depends only on (base, dims, box, element type, swizzle): a training step encodes the same few
    // again and again, so the last ones are kept per thread.
    struct Key { const void* base; uint64_t dims[3]; uint32_t box[3]; int rank, fp16, swz, dev; };
    struct Slot { Key key; CUtensorMap map; bool used; };
    constexpr int SLOTS = 32;
    static thread_local Slot cache[SLOTS];
    static thread_local unsigned next_slot = 0;
    Key key;
    memset(&key, 0, sizeof(key));
    key.base = base; key.rank = rank; key.fp16 = fp16; key.swz = swizzle_bytes;
    for (int i = 0; i < rank; ++i) { key.dims[i] = dims[i]; key.box[i] = box[i]; }
    if (cudaGetDevice(&key.dev) != cudaSuccess) key.dev = -1;
    for (int i = 0; i < SLOTS; ++i)
        if (cache[i].used && memcmp(&cache[i].key, &key, sizeof(Key)) == 0) { *map = cache[i].map; return SVTAD_OK; }
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return set_error(SVTAD_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    // the driver call needs this thread to hold the device's context (autograd worker threads may not yet)
    static thread_local int ctx_dev = -1;
    int dev = 0;
    SV_CUDA(cudaGetDevice(&dev));
    if (ctx_dev != dev) {
        SV_CUDA(cudaSetDevice(dev));   // binds the device's primary context to this thread; allocates nothing
        ctx_dev = dev;
    }
    cuuint64_t gdim[3], gstride[2];
    cuuint32_t bx[3], es[3] = {1, 1, 1};
    uint64_t stride = 2;
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bx[i] = box[i];
        stride *= dims[i];
        if (i < rank - 1) gstride[i] = stride;
    }
    CUresult r = fn(map, fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank,
                    const_cast<void*>(base), gdim, gstride, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(SVTAD_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    Slot& slot = cache[next_slot++ % SLOTS];
    slot.key = key; slot.map = *map; slot.used = true;
    return SVTAD_OK;
}

// One CTA runs per SM, so the cost of a column-block width is
// (waves over the SMs) x (bytes a CTA stages per K step: 16 KB of gathered rows + its weight tile).
int tc_pick_bn(int cn, long m_tiles) {
    const int cand[5] = {256, 192, 128, 96, 64};
    const char* e = getenv("SVTAD_TC_BN");
    if (e != nullptr && *e) {
        int v = atoi(e);
        for (int c : cand)
            if (v == c && cn % v == 0) return v;
    }
    const long sms = tc_plan_sms();
    int best = 0;
    long best_cost = 0;
    for (int c : cand) {
        if (cn % c != 0) continue;
        long ctas = m_tiles * (cn / c);
        long waves = (ctas + sms - 1) / sms;
        long cost = waves * (A_TILE_BYTES + b_tile_bytes_for(c));
        if (best == 0 || cost < best_cost) { best = c; best_cost = cost; }
    }
    return best;
}

// wgrad work split: (pairs of 64-channel blocks) x (column blocks of width BN) x (splits over tokens).
// One CTA runs per SM, so a candidate (BN, splits) costs
//   (waves over the SMs) x (64-token steps per CTA + fixed cost) x (cycles per step at that BN)
// plus the trip of the fp32 partials through memory (written by the main kernel, read by the reduction).
// Cycles per step and the partials' rate are what these kernels were measured at on a B200.
static WgradPlan wgrad_plan_for(int64_t n, int cin, int cout, int kk, long sms) {
    const int nblocks = kk * (cin / 64);
    long max_by_rows = (n + 2 * STAGE_K - 1) / (2 * STAGE_K);
    if (max_by_rows < 1) max_by_rows = 1;
    if (max_by_rows > 64) max_by_rows = 64;
    int forced_bn = 0;
    if (const char* e = getenv("SVTAD_TC_WGRAD_BN")) forced_bn = atoi(e);
    long forced_s = 0;
    if (const char* e = getenv("SVTAD_TC_WGRAD_SPLITS")) forced_s = atol(e);
    const int cand[4] = {256, 192, 128, 64};
    const double step_cycles[4] = {650.0, 584.0, 450.0, 400.0};
    // partials are written once and read once: from L2 while they fit beside the operands, else from memory
    const double partial_cycles_l2 = 2.0 * 1.9e9 / 12.0e12, partial_cycles_mem = 2.0 * 1.9e9 / 4.0e12;
    WgradPlan best;
    best.bn = 0;
    double best_cost = 0;
    for (int ci = 0; ci < 4; ++ci) {
        const int bn = cand[ci];
        if (cout % bn != 0) continue;
        if (bn < 192 && best.bn != 0 && forced_bn == 0) continue;      // narrow blocks only when no wide one divides cout
        if (forced_bn > 0 && bn != forced_bn && cout % forced_bn == 0) continue;
        WgradPlan pl;
        pl.bn = bn;
        pl.n_nblk = cout / bn;
        pl.n_pairs = (nblocks + 1) / 2;
        pl.ones_block = nblocks & 1;
        const long ctas = (long)pl.n_pairs * pl.n_nblk;
        for (long c = 1; c <= max_by_rows; ++c) {
            if (forced_s > 0 && c != (forced_s < max_by_rows ? forced_s : max_by_rows)) continue;
            const long tps = ((n + c - 1) / c + STAGE_K - 1) / STAGE_K * STAGE_K;
            const long splits = (n + tps - 1) / tps;
            const long waves = (ctas * splits + sms - 1) / sms;
            const double steps = (double)tps / STAGE_K + 12.0;          // + set-up, first operands, drain
            const double partial_bytes = (double)splits * kk * cin * cout * sizeof(float);
            const double cost = (double)waves * steps * step_cycles[ci] +
                                partial_bytes * (partial_bytes < 48e6 ? partial_cycles_l2 : partial_cycles_mem);
            if (best.bn == 0 || cost < best_cost * 0.98) {
                best = pl;
                best.tokens_per_split = tps;
                best.splits = (int)splits;
                best_cost = cost;
            }
        }
    }
    return best;
}

WgradPlan tc_wgrad_plan(int64_t n, int cin, int cout, int kk) { return wgrad_plan_for(n, cin, cout, kk, tc_plan_sms()); }

static size_t plan_bytes(const WgradPlan& pl, int64_t n, int cin, int cout, int kk) {
    size_t w = (size_t)pl.splits * kk * cin * cout * sizeof(float);
    int sb = pl.ones_block ? pl.splits : bias_splits_for(n);
    size_t b = (size_t)sb * cout * sizeof(float);
    return align_up(w, 256) + align_up(b, 256);
}

// Workspace of the plan in force at this moment (what a launch checks its workspace against) ...
size_t tc_wgrad_plan_ws_bytes(int64_t n, int cin, int cout, int kk) {
    return plan_bytes(tc_wgrad_plan(n, cin, cout, kk), n, cin, cout, kk);
}

// ... and what callers are told to provide: enough for the plan under every concurrency hint, so that a workspace
// sized once stays valid when the hint changes (a leaner plan usually has fewer token splits, but the waves'
// rounding can go the other way: 18 880 rows at C=192, 5x5 takes 3 splits planned for 148 SMs and 5 for 74).
size_t tc_wgrad_ws_bytes(int64_t n, int cin, int cout, int kk) {
    size_t need = 0;
    const int sms = tc_num_sms();
    for (int share = 1; share <= 16; ++share) {
        int v = sms / share;
        if (v < 8) v = 8;
        const size_t b = plan_bytes(wgrad_plan_for(n, cin, cout, kk, v), n, cin, cout, kk);
        if (b > need) need = b;
    }
    return need;
}


// fixed-order reduction of the per-split partials (4 elements per thread), one rounding
__global__ void __launch_bounds__(256)
wgrad_reduce4_kernel(const float* __restrict__ ws_w, int splits, const float* __restrict__ ws_b, int splits_b,
                     uint16_t* __restrict__ gw, uint16_t* __restrict__ gb, long n_w, int cout, int fp16) {
    long e = (blockIdx.x * (long)blockDim.x + threadIdx.x) * 4;
    const float* src;
    uint16_t* dst;
    long stride;
    int cnt;
    if (e < n_w) {
        src = ws_w + e; dst = gw + e; stride = n_w; cnt = splits;
    } else if (gb != nullptr && e - n_w < cout) {
        src = ws_b + (e - n_w); dst = gb + (e - n_w); stride = cout; cnt = splits_b;
    } else {
        return;
    }
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int s = 0; s < cnt; ++s) {
        float4 v = __ldcg(reinterpret_cast<const float4*>(src + (long)s * stride));
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    uint2 o;
    o.x = pack2(acc.x, acc.y, fp16 != 0);
    o.y = pack2(acc.z, acc.w, fp16 != 0);
    *reinterpret_cast<uint2*>(dst) = o;
}


int tc_wgrad_reduce_launch(const float* ws_w, int splits, const float* ws_b, int splits_b, void* gw, void* gb,
                           long n_w, int cout, int fp16, cudaStream_t s) {
    long total4 = (n_w + (gb ? cout : 0) + 3) / 4;
    SV_CUDA(tc_launch(wgrad_reduce4_kernel, dim3((unsigned)((total4 + 255) / 256)), dim3(256), 0, s, ws_w, splits, ws_b,
                      splits_b, (uint16_t*)gw, (uint16_t*)gb, n_w, cout, fp16));
    return SVTAD_OK;
}

bool tc_supported(int op, int64_t n, int cin, int cout, int kk, int dtype) {
    if (dtype != SVTAD_BF16 && dtype != SVTAD_F16) return false;
    if (n <= 0 || kk > 49) return false;
    if (cin % 64 != 0 || cout % 64 != 0) return false;
    (void)op;
    return true;
}

// Forward / dgrad on CTA pairs (tcgen05 cta_group::2) or on single CTAs.  Measured on B200 at C = 192: pairs win
// once there are more row tiles than SMs (918-941 vs 820-850 TFLOP/s at 226 560 rows); below that one CTA
// per (row tile, column block) starts sooner and uses narrower column blocks to fill the machine.
// SVTAD_TC_IMPL=pair / hybrid overrides the choice.
static bool use_pair(int64_t n) {
    const char* e = getenv("SVTAD_TC_IMPL");
    if (e != nullptr && *e) return e[0] == 'p';
    const long m_tiles = (n + TILE_M - 1) / TILE_M;
    return m_tiles > (long)tc_num_sms();
}

int tc_fwd(const ConvArgs& p, cudaStream_t s) {
    if (use_pair(p.n)) return pair_fwd(p, s);
    return hybrid_fwd(p, s);
}

int tc_dgrad(const ConvArgs& p, const int32_t* status, cudaStream_t s) {
    if (use_pair(p.n)) return pair_dgrad(p, status, s);
    return hybrid_dgrad(p, status, s);
}

int tc_wgrad(const void* gy, const void* x, const int32_t* nbr, void* gw, void* gb, int64_t n, int cin, int cout,
             int kk, int tpb, int dtype, void* ws, size_t ws_bytes, cudaStream_t s) {
    return hybrid_wgrad(gy, x, nbr, gw, gb, n, cin, cout, kk, tpb, dtype, ws, ws_bytes, s);
}

}  // namespace svtad
