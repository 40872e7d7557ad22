// Sum of the weight-gradient bucket over the ranks of one node: a two-shot all-reduce over peer-mapped memory
// in which every 8 bytes that cross NVLink carry their own "valid" flag.
//
// Data-parallel training of the reference all-reduces the adapters' gradients with torch DDP
// (src/eccv26_tad.py:288-300: one NCCL all-reduce per 25 MB bucket).  The bucket of this op is small (2 MB for
// three 192-channel layers), so the collective is pure latency: a protocol of "write, system fence, flag, wait"
// per phase costs four NVLink latencies plus two fences (measured on two B200s: 4.7 + 2.7 + 7.7 + 4.8 us for the
// two flag waits, the copies and the fence).  Here nothing waits for a fence or a separate flag.  Every rank's
// allocation holds the bucket and two staging areas in which a 16-byte unit of data occupies 32 bytes:
// (d0, e, d1, e | d2, e, d3, e), e = the number of the call.  8-byte stores are single-copy atomic, so a reader
// that sees e in a flag word sees the data word beside it.
//   1. rank r pushes its copy of slice p (p != r) into rank p's "in" staging area, row r;
//   2. rank p polls the rows of the other ranks unit by unit, adds them to its own copy in rank order 0 .. N-1
//      (fp32, one rounding: every rank ends up with bit-identical sums), writes the result into its own bucket
//      and pushes it into every other rank's "out" staging area;
//   3. every rank polls its "out" area for the other ranks' slices and copies them into its bucket.
// Plain stores and loads over NVLink only: no multicast, no NVLS, no TMA.  A thread only ever waits for data that
// another GPU pushes (never for a CTA of its own grid), so the grid needs no co-residency.  Every wait is bounded:
// when a peer does not show up within the limit the CTA records a code in the device error word
// (svtad_device_error), stops and returns; the bucket entries it had not reached stay as they were.  The call
// number lives in device memory and is advanced by the kernel itself, so a CUDA graph can replay the launch;
// flags are never reset (a stale unit carries an older number).
#include <cstdlib>
#include <mutex>
#include <set>
#include <utility>

#include "common.cuh"

namespace svtad {

int* tc_error_ptr();     // the library's device error word (conv_tc.cu)

// Small CTAs: four warps, one per SM sub-partition, so that a CTA fits into the registers a convolution CTA leaves
// free (a 9-warp CTA at 136 registers leaves 3 328 registers in its fullest sub-partition: one warp of this kernel).
constexpr int AR_THREADS = 128;
constexpr int AR_MAX_CTAS = 256;
constexpr int AR_MAX_RANKS = 16;
constexpr long long AR_DEFAULT_LIMIT = 2000000000ll;     // about a second

__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_volatile_v4(void* p, uint4 v) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ float2 widen2(uint32_t w, bool fp16) {
    if (fp16) {
        __half2 h = *reinterpret_cast<__half2*>(&w);
        return __half22float2(h);
    }
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
__device__ __forceinline__ uint32_t narrow2(float a, float b, bool fp16) {
    if (fp16) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void acc8(float (&acc)[8], uint4 q, bool fp16) {
    const float2 a = widen2(q.x, fp16), b = widen2(q.y, fp16), c = widen2(q.z, fp16), d = widen2(q.w, fp16);
    acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
    acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
}
// one 16-byte unit with its flags -> 32 bytes at `dst`
__device__ __forceinline__ void push_unit(void* dst, uint4 d, unsigned e) {
    st_volatile_v4(dst, make_uint4(d.x, e, d.y, e));
    st_volatile_v4(static_cast<char*>(dst) + 16, make_uint4(d.z, e, d.w, e));
}
// Waits (bounded) until the 32-byte unit at `src` carries call number e; false when the limit ran out.
// After a miss the thread sleeps (`backoff` ns, doubling up to 16x) before it looks again: the pollers read this
// GPU's own memory through L2, and thousands of them spinning flat out take bandwidth from the kernels that run
// beside the exchange.
__device__ __forceinline__ bool poll_unit(const void* src, unsigned e, uint4& d, long long limit, int* err, int code,
                                          volatile int* s_abort, unsigned backoff) {
    long long t0 = 0;
    unsigned nap = backoff;
    for (unsigned spin = 0;; ++spin) {
        const uint4 lo = ld_volatile_v4(src);
        const uint4 hi = ld_volatile_v4(static_cast<const char*>(src) + 16);
        if (lo.y == e && lo.w == e && hi.y == e && hi.w == e) {
            d = make_uint4(lo.x, lo.z, hi.x, hi.z);
            return true;
        }
        if (spin == 0) t0 = clock64();
        if (nap) {
            __nanosleep(nap);
            if (nap < backoff * 16u) nap *= 2u;
        }
        if ((spin & 7u) == 7u) {
            if (*s_abort) return false;
            if (clock64() - t0 > limit) {
                atomicCAS(err, 0, code);
                *s_abort = 1;
                return false;
            }
        }
    }
}

// One rank's part of the exchange.  `bufs[p]` is rank p's allocation as THIS rank addresses it:
// [bucket: n_unit * 16 B][in: world rows of n_unit / world units * 32 B][out: n_unit units * 32 B].
// Returns false when a wait ran out of time (the error word has been set).
__device__ bool ar_rank_body(void* const* bufs, int rank, int world, long n_unit, size_t stage_off, unsigned* epoch, int fp16_i,
                             long long limit, int* err, int cta, int n_ctas, volatile int* s_abort, unsigned backoff) {
    const int tid = threadIdx.x;
    const bool fp16 = fp16_i != 0;
    const unsigned e = epoch[cta] + 1u;          // number of this call; the same on every rank and CTA
    if (tid == 0) *s_abort = 0;
    __syncthreads();
    char* mine = static_cast<char*>(bufs[rank]);
    const long S = n_unit / world;               // units per slice
    const size_t in_off = stage_off, out_off = stage_off + (size_t)n_unit * 32;
    const long stride = (long)n_ctas * AR_THREADS;
    const long t = (long)cta * AR_THREADS + tid;
    // ---- 1. my copy of the other ranks' slices -> their "in" areas, row `rank`
    for (long u = t; u < n_unit; u += stride) {
        const int p = (int)(u / S);
        if (p == rank) continue;
        const uint4 d = *reinterpret_cast<const uint4*>(mine + u * 16);
        push_unit(static_cast<char*>(bufs[p]) + in_off + ((size_t)rank * S + (u - (long)p * S)) * 32, d, e);
    }
    // ---- 2. my slice: own copy + the rows the others pushed, in rank order; result to my bucket and their "out" areas
    bool ok = true;
    for (long j = t; j < S && ok; j += stride) {
        const long u = (long)rank * S + j;
        const uint4 own = *reinterpret_cast<const uint4*>(mine + u * 16);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int p = 0; p < world; ++p) {
            uint4 d = own;
            if (p != rank) ok = ok && poll_unit(mine + in_off + ((size_t)p * S + j) * 32, e, d, limit, err, 71, s_abort, backoff);
            if (!ok) break;
            acc8(acc, d, fp16);
        }
        if (!ok) break;
        uint4 o;
        o.x = narrow2(acc[0], acc[1], fp16); o.y = narrow2(acc[2], acc[3], fp16);
        o.z = narrow2(acc[4], acc[5], fp16); o.w = narrow2(acc[6], acc[7], fp16);
        *reinterpret_cast<uint4*>(mine + u * 16) = o;
        for (int q = 0; q < world; ++q)
            if (q != rank) push_unit(static_cast<char*>(bufs[q]) + out_off + (size_t)u * 32, o, e);
    }
    // ---- 3. the other ranks' slices: from my "out" area into my bucket
    for (long u = t; u < n_unit && ok; u += stride) {
        const int p = (int)(u / S);
        if (p == rank) continue;
        uint4 d;
        ok = poll_unit(mine + out_off + (size_t)u * 32, e, d, limit, err, 72, s_abort, backoff);
        if (ok) *reinterpret_cast<uint4*>(mine + u * 16) = d;
    }
    __syncthreads();
    const bool all_ok = *s_abort == 0;
    if (tid == 0 && all_ok) epoch[cta] = e;
    return all_ok;
}

struct ArPeers { void* p[AR_MAX_RANKS]; };

__global__ void __launch_bounds__(AR_THREADS, 8)
allreduce_twoshot_kernel(ArPeers peers, int rank, int world, long n_unit, size_t stage_off, unsigned* epoch, int fp16,
                         long long limit, int* err, unsigned backoff) {
    __shared__ int s_flag;
    ar_rank_body(peers.p, rank, world, n_unit, stage_off, epoch, fp16, limit, err, blockIdx.x, gridDim.x, &s_flag, backoff);
}

// All ranks in ONE launch on one GPU (blockIdx.y = rank): the same protocol with every "peer" buffer local.  The
// CTAs of different ranks wait for one another, so the launch is cooperative (all of them resident).  For tests on
// a machine with fewer GPUs than ranks.
__global__ void __launch_bounds__(AR_THREADS, 8)
allreduce_twoshot_emulated_kernel(ArPeers peers, int world, long n_unit, size_t stage_off, unsigned* epochs, int fp16,
                                  long long limit, int* err, unsigned backoff) {
    __shared__ int s_flag;
    const int rank = blockIdx.y;
    ar_rank_body(peers.p, rank, world, n_unit, stage_off, epochs + rank * AR_MAX_CTAS, fp16, limit, err, blockIdx.x,
                 gridDim.x, &s_flag, backoff);
}

static int ar_check(const char* who, void* const* peer_bufs, int rank, int world, int64_t n_elems, int dtype,
                    size_t stage_offset_bytes, void* epoch) {
    SV_CHECK_ARG(peer_bufs != nullptr && epoch != nullptr, "%s: null pointer", who);
    SV_CHECK_ARG(world >= 1 && world <= AR_MAX_RANKS, "%s: world size %d outside [1, %d]", who, world, AR_MAX_RANKS);
    SV_CHECK_ARG(rank >= 0 && rank < world, "%s: rank %d outside [0, %d)", who, rank, world);
    SV_CHECK_ARG(dtype == SVTAD_BF16 || dtype == SVTAD_F16, "%s: 16-bit buckets only (dtype %d)", who, dtype);
    SV_CHECK_ARG(n_elems >= 0 && n_elems % (8 * world) == 0,
                 "%s: the bucket must hold a multiple of 8 * world = %d elements (got %lld): pad it", who, 8 * world,
                 (long long)n_elems);
    SV_CHECK_ARG(stage_offset_bytes % 16 == 0 && stage_offset_bytes >= (size_t)n_elems * 2,
                 "%s: the staging areas must sit behind the bucket, 16-byte aligned", who);
    for (int p = 0; p < world; ++p)
        SV_CHECK_ARG(peer_bufs[p] != nullptr && reinterpret_cast<uintptr_t>(peer_bufs[p]) % 16 == 0,
                     "%s: peer pointer %d is null or not 16-byte aligned", who, p);
    return SVTAD_OK;
}

// SVTAD_ALLREDUCE_CTAS / SVTAD_ALLREDUCE_BACKOFF_NS, read once: every rank must run with the same values
static int ar_env(const char* name, int lo, int hi, int dflt) {
    const char* e = getenv(name);
    if (e == nullptr || !*e) return dflt;
    int v = atoi(e);
    return v < lo ? lo : (v > hi ? hi : v);
}
// Default 128 CTAs: measured beside the convolution kernels on two B200s, a 2 MB bucket's step took 0.1103 / 0.1093 /
// 0.1098 / 0.1136 ms with 256 / 128 / 64 / 32 CTAs.
static int ar_max_ctas() { static const int v = ar_env("SVTAD_ALLREDUCE_CTAS", 1, AR_MAX_CTAS, 128); return v; }
static unsigned ar_backoff() { static const int v = ar_env("SVTAD_ALLREDUCE_BACKOFF_NS", 0, 4096, 0); return (unsigned)v; }

// The exchange is meant to run beside the convolution kernels, whose CTAs take nearly all of an SM's shared memory.
// An SM runs kernels of one shared-memory / L1 split at a time, so this kernel asks for the same split (all shared)
// although it uses four bytes of it; otherwise its CTAs wait for SMs without a convolution CTA.  Once per device.
static int ar_prefer_shared(const void* kern) {
    static std::mutex mu;
    static std::set<std::pair<const void*, int>> done;
    int dev = 0;
    SV_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> hold(mu);
    if (done.count({kern, dev})) return SVTAD_OK;
    SV_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    done.insert({kern, dev});
    return SVTAD_OK;
}

static int ar_ctas(int64_t n_unit, int world) {
    // about four 16-byte units of the bucket per thread, within [1, the cap]
    (void)world;
    long c = (n_unit + 4 * AR_THREADS - 1) / (4 * AR_THREADS);
    if (c < 1) c = 1;
    if (c > ar_max_ctas()) c = ar_max_ctas();
    return (int)c;
}

}  // namespace svtad

using namespace svtad;

extern "C" size_t svtad_allreduce_stage_bytes(int64_t n_elems) { return n_elems > 0 ? (size_t)n_elems * 8 : 0; }

extern "C" size_t svtad_allreduce_epoch_bytes(void) { return (size_t)AR_MAX_RANKS * AR_MAX_CTAS * sizeof(unsigned); }

extern "C" int svtad_allreduce_sum(void* const* peer_bufs, int rank, int world, int64_t n_elems, int dtype,
                                   size_t stage_offset_bytes, void* epoch, int64_t wait_limit_cycles, void* stream) {
    int rc = ar_check("svtad_allreduce_sum", peer_bufs, rank, world, n_elems, dtype, stage_offset_bytes, epoch);
    if (rc) return rc;
    if (n_elems == 0 || world == 1) return SVTAD_OK;
    ArPeers peers;
    for (int p = 0; p < AR_MAX_RANKS; ++p) peers.p[p] = p < world ? peer_bufs[p] : nullptr;
    const long n_vec = (long)(n_elems / 8);
    const long long limit = wait_limit_cycles > 0 ? wait_limit_cycles : AR_DEFAULT_LIMIT;
    int* err = tc_error_ptr();
    SV_CHECK_ARG(err != nullptr, "svtad_allreduce_sum: no current CUDA device");
    rc = ar_prefer_shared(reinterpret_cast<const void*>(allreduce_twoshot_kernel));
    if (rc) return rc;
    allreduce_twoshot_kernel<<<ar_ctas(n_vec, world), AR_THREADS, 0, (cudaStream_t)stream>>>(
        peers, rank, world, n_vec, stage_offset_bytes, static_cast<unsigned*>(epoch), dtype == SVTAD_F16 ? 1 : 0, limit, err, ar_backoff());
    SV_LAUNCH_CHECK("allreduce_twoshot_kernel");
    return SVTAD_OK;
}

extern "C" int svtad_allreduce_sum_emulated(void* const* bufs, int world, int64_t n_elems, int dtype,
                                            size_t stage_offset_bytes, void* epochs, int64_t wait_limit_cycles,
                                            void* stream) {
    int rc = ar_check("svtad_allreduce_sum_emulated", bufs, 0, world, n_elems, dtype, stage_offset_bytes, epochs);
    if (rc) return rc;
    if (n_elems == 0) return SVTAD_OK;
    ArPeers peers;
    for (int p = 0; p < AR_MAX_RANKS; ++p) peers.p[p] = p < world ? bufs[p] : nullptr;
    long n_vec = (long)(n_elems / 8);
    size_t flag_off = stage_offset_bytes;
    unsigned* ep = static_cast<unsigned*>(epochs);
    int fp16 = dtype == SVTAD_F16 ? 1 : 0;
    long long limit = wait_limit_cycles > 0 ? wait_limit_cycles : AR_DEFAULT_LIMIT;
    int* err = tc_error_ptr();
    SV_CHECK_ARG(err != nullptr, "svtad_allreduce_sum_emulated: no current CUDA device");
    int ctas = ar_ctas(n_vec, world);
    if (ctas * world > 256) ctas = 256 / world;          // every CTA of every rank must be resident at once (148 SMs)
    unsigned backoff = ar_backoff();
    void* args[] = {&peers, &world, &n_vec, &flag_off, &ep, &fp16, &limit, &err, &backoff};
    SV_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(allreduce_twoshot_emulated_kernel),
                                        dim3((unsigned)ctas, (unsigned)world), dim3(AR_THREADS), args, 0,
                                        (cudaStream_t)stream));
    return SVTAD_OK;
}
