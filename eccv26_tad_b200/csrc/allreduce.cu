// Sum of the weight-gradient bucket over the ranks of one node: a two-shot all-reduce over peer-mapped memory.
//
// Data-parallel training of the reference all-reduces the adapters' gradients with torch DDP
// (src/eccv26_tad.py:288-300: one NCCL all-reduce per 25 MB bucket).  The bucket of this op is small (2 MB for
// three 192-channel layers), so the collective is pure latency.  Here every rank's bucket lives in memory that all
// ranks of the node have mapped (the caller sets that up and hands in the table of peer pointers); then
//   1. every rank tells every peer "my bucket is written" (one flag per peer and CTA),
//   2. rank r sums slice r of the bucket over all ranks with plain loads from the peers' memory, in rank order
//      0 .. N-1 (fixed order: all ranks end up with bit-identical sums), rounds once, and writes the result into
//      slice r of EVERY rank's bucket with plain stores,
//   3. every rank tells every peer "my slice is written everywhere" and waits for the same from all peers.
// Plain ld / st over NVLink only: no multicast, no NVLS, no TMA.  CTA c of every rank only ever waits for CTA c of
// the other ranks, never for a CTA of its own grid, so the grid needs no co-residency.  Every wait is bounded:
// when a peer does not show up within the limit the CTA records a code in the device error word
// (svtad_device_error), skips its work and returns.  Flags carry the number of the call (kept per CTA in device
// memory and advanced by the kernel itself, so a CUDA graph can replay the launch); nothing is ever reset.
#include "common.cuh"

namespace svtad {

int* tc_error_ptr();     // the library's device error word (conv_tc.cu)

constexpr int AR_THREADS = 512;
constexpr int AR_MAX_CTAS = 32;
constexpr int AR_MAX_RANKS = 16;
constexpr long long AR_DEFAULT_LIMIT = 2000000000ll;     // about a second

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_sys_v4(void* p, uint4 v) {
    asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
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

// Flag words of a rank: [phase 0 / 1][CTA][source rank], behind the bucket at byte offset `flag_off`.
__device__ __forceinline__ unsigned* ar_flag(void* buf, size_t flag_off, int phase, int cta, int src) {
    return reinterpret_cast<unsigned*>(static_cast<char*>(buf) + flag_off) + (phase * AR_MAX_CTAS + cta) * AR_MAX_RANKS + src;
}

// One rank's part of the exchange.  `bufs[p]` is rank p's bucket as THIS rank addresses it.
// Returns false when a wait ran out of time (the error word has been set).
__device__ bool ar_rank_body(void* const* bufs, int rank, int world, long n_vec, size_t flag_off, unsigned* epoch, int fp16,
                             long long limit, int* err, int cta, int n_ctas, volatile int* s_flag) {
    const int tid = threadIdx.x;
    const unsigned e = epoch[cta] + 1u;          // number of this call; the same on every rank
    void* mine = bufs[rank];
    if (tid == 0) *s_flag = 1;
    __syncthreads();
    // ---- 1. my bucket is complete (it was written by earlier work in this stream): tell every peer, wait for all
    if (tid < world) {
        st_release_sys(ar_flag(bufs[tid], flag_off, 0, cta, rank), e);
        const unsigned* f = ar_flag(mine, flag_off, 0, cta, tid);
        const long long t0 = clock64();
        for (unsigned spin = 1; (int)(ld_acquire_sys(f) - e) < 0; ++spin) {
            if ((spin & 15u) == 0u && clock64() - t0 > limit) {
                atomicCAS(err, 0, 71);
                *s_flag = 0;
                break;
            }
        }
    }
    __syncthreads();
    if (*s_flag == 0) return false;
    // ---- 2. slice `rank`, this CTA's share of it: sum over the ranks in rank order, write to every rank
    const long per_rank = n_vec / world;                       // 16-byte vectors per slice
    const long per_cta = (per_rank + n_ctas - 1) / n_ctas;
    const long v_lo = rank * per_rank + (long)cta * per_cta;
    long v_hi = v_lo + per_cta;
    if (v_hi > (rank + 1) * per_rank) v_hi = (rank + 1) * per_rank;
    for (long v = v_lo + tid; v < v_hi; v += AR_THREADS) {
        // all loads first (they cross NVLink: one latency, not `world` of them), then the sum in rank order
        uint4 q[AR_MAX_RANKS];
#pragma unroll
        for (int p = 0; p < AR_MAX_RANKS; ++p)
            if (p < world) q[p] = ld_relaxed_sys_v4(static_cast<const char*>(bufs[p]) + v * 16);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int p = 0; p < AR_MAX_RANKS; ++p) {
            if (p < world) {
                const float2 a = widen2(q[p].x, fp16 != 0), b = widen2(q[p].y, fp16 != 0), c = widen2(q[p].z, fp16 != 0),
                             d = widen2(q[p].w, fp16 != 0);
                acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
                acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
            }
        }
        uint4 o;
        o.x = narrow2(acc[0], acc[1], fp16 != 0); o.y = narrow2(acc[2], acc[3], fp16 != 0);
        o.z = narrow2(acc[4], acc[5], fp16 != 0); o.w = narrow2(acc[6], acc[7], fp16 != 0);
#pragma unroll
        for (int p = 0; p < AR_MAX_RANKS; ++p)
            if (p < world) st_relaxed_sys_v4(static_cast<char*>(bufs[p]) + v * 16, o);
    }
    __threadfence_system();       // this thread's stores to the peers are ordered before the flag that follows
    __syncthreads();
    // ---- 3. my share of slice `rank` is written everywhere: tell every peer, wait for the same from all
    if (tid < world) {
        st_release_sys(ar_flag(bufs[tid], flag_off, 1, cta, rank), e);
        const unsigned* f = ar_flag(mine, flag_off, 1, cta, tid);
        const long long t0 = clock64();
        for (unsigned spin = 1; (int)(ld_acquire_sys(f) - e) < 0; ++spin) {
            if ((spin & 15u) == 0u && clock64() - t0 > limit) {
                atomicCAS(err, 0, 72);
                *s_flag = 0;
                break;
            }
        }
    }
    __syncthreads();
    if (tid == 0 && *s_flag) epoch[cta] = e;
    return *s_flag != 0;
}

struct ArPeers { void* p[AR_MAX_RANKS]; };

__global__ void __launch_bounds__(AR_THREADS)
allreduce_twoshot_kernel(ArPeers peers, int rank, int world, long n_vec, size_t flag_off, unsigned* epoch, int fp16,
                         long long limit, int* err) {
    __shared__ int s_flag;
    ar_rank_body(peers.p, rank, world, n_vec, flag_off, epoch, fp16, limit, err, blockIdx.x, gridDim.x, &s_flag);
}

// All ranks in ONE launch on one GPU (blockIdx.y = rank): the same protocol with every "peer" buffer local.  The
// CTAs of different ranks wait for one another, so the launch is cooperative (all of them resident).  For tests on
// a machine with fewer GPUs than ranks.
__global__ void __launch_bounds__(AR_THREADS)
allreduce_twoshot_emulated_kernel(ArPeers peers, int world, long n_vec, size_t flag_off, unsigned* epochs, int fp16,
                                  long long limit, int* err) {
    __shared__ int s_flag;
    const int rank = blockIdx.y;
    ar_rank_body(peers.p, rank, world, n_vec, flag_off, epochs + rank * AR_MAX_CTAS, fp16, limit, err, blockIdx.x,
                 gridDim.x, &s_flag);
}

static int ar_check(const char* who, void* const* peer_bufs, int rank, int world, int64_t n_elems, int dtype,
                    size_t flag_offset_bytes, void* epoch) {
    SV_CHECK_ARG(peer_bufs != nullptr && epoch != nullptr, "%s: null pointer", who);
    SV_CHECK_ARG(world >= 1 && world <= AR_MAX_RANKS, "%s: world size %d outside [1, %d]", who, world, AR_MAX_RANKS);
    SV_CHECK_ARG(rank >= 0 && rank < world, "%s: rank %d outside [0, %d)", who, rank, world);
    SV_CHECK_ARG(dtype == SVTAD_BF16 || dtype == SVTAD_F16, "%s: 16-bit buckets only (dtype %d)", who, dtype);
    SV_CHECK_ARG(n_elems >= 0 && n_elems % (8 * world) == 0,
                 "%s: the bucket must hold a multiple of 8 * world = %d elements (got %lld): pad it", who, 8 * world,
                 (long long)n_elems);
    SV_CHECK_ARG(flag_offset_bytes % 16 == 0 && flag_offset_bytes >= (size_t)n_elems * 2,
                 "%s: the flag words must sit behind the bucket, 16-byte aligned", who);
    for (int p = 0; p < world; ++p)
        SV_CHECK_ARG(peer_bufs[p] != nullptr && reinterpret_cast<uintptr_t>(peer_bufs[p]) % 16 == 0,
                     "%s: peer pointer %d is null or not 16-byte aligned", who, p);
    return SVTAD_OK;
}

static int ar_ctas(int64_t n_vec, int world) {
    // about one 16-byte vector per thread and slice, within [1, AR_MAX_CTAS]
    long per_rank = n_vec / world;
    long c = (per_rank + AR_THREADS - 1) / AR_THREADS;
    if (c < 1) c = 1;
    if (c > AR_MAX_CTAS) c = AR_MAX_CTAS;
    return (int)c;
}

}  // namespace svtad

using namespace svtad;

extern "C" size_t svtad_allreduce_flag_bytes(void) { return (size_t)2 * AR_MAX_CTAS * AR_MAX_RANKS * sizeof(unsigned); }

extern "C" size_t svtad_allreduce_epoch_bytes(void) { return (size_t)AR_MAX_RANKS * AR_MAX_CTAS * sizeof(unsigned); }

extern "C" int svtad_allreduce_sum(void* const* peer_bufs, int rank, int world, int64_t n_elems, int dtype,
                                   size_t flag_offset_bytes, void* epoch, int64_t wait_limit_cycles, void* stream) {
    int rc = ar_check("svtad_allreduce_sum", peer_bufs, rank, world, n_elems, dtype, flag_offset_bytes, epoch);
    if (rc) return rc;
    if (n_elems == 0 || world == 1) return SVTAD_OK;
    ArPeers peers;
    for (int p = 0; p < AR_MAX_RANKS; ++p) peers.p[p] = p < world ? peer_bufs[p] : nullptr;
    const long n_vec = (long)(n_elems / 8);
    const long long limit = wait_limit_cycles > 0 ? wait_limit_cycles : AR_DEFAULT_LIMIT;
    int* err = tc_error_ptr();
    SV_CHECK_ARG(err != nullptr, "svtad_allreduce_sum: no current CUDA device");
    allreduce_twoshot_kernel<<<ar_ctas(n_vec, world), AR_THREADS, 0, (cudaStream_t)stream>>>(
        peers, rank, world, n_vec, flag_offset_bytes, static_cast<unsigned*>(epoch), dtype == SVTAD_F16 ? 1 : 0, limit, err);
    SV_LAUNCH_CHECK("allreduce_twoshot_kernel");
    return SVTAD_OK;
}

extern "C" int svtad_allreduce_sum_emulated(void* const* bufs, int world, int64_t n_elems, int dtype,
                                            size_t flag_offset_bytes, void* epochs, int64_t wait_limit_cycles,
                                            void* stream) {
    int rc = ar_check("svtad_allreduce_sum_emulated", bufs, 0, world, n_elems, dtype, flag_offset_bytes, epochs);
    if (rc) return rc;
    if (n_elems == 0) return SVTAD_OK;
    ArPeers peers;
    for (int p = 0; p < AR_MAX_RANKS; ++p) peers.p[p] = p < world ? bufs[p] : nullptr;
    long n_vec = (long)(n_elems / 8);
    size_t flag_off = flag_offset_bytes;
    unsigned* ep = static_cast<unsigned*>(epochs);
    int fp16 = dtype == SVTAD_F16 ? 1 : 0;
    long long limit = wait_limit_cycles > 0 ? wait_limit_cycles : AR_DEFAULT_LIMIT;
    int* err = tc_error_ptr();
    SV_CHECK_ARG(err != nullptr, "svtad_allreduce_sum_emulated: no current CUDA device");
    int ctas = ar_ctas(n_vec, world);
    if (ctas * world > 128) ctas = 128 / world;          // every CTA of every rank must be resident at once
    void* args[] = {&peers, &world, &n_vec, &flag_off, &ep, &fp16, &limit, &err};
    SV_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(allreduce_twoshot_emulated_kernel),
                                        dim3((unsigned)ctas, (unsigned)world), dim3(AR_THREADS), args, 0,
                                        (cudaStream_t)stream));
    return SVTAD_OK;
}
