// tcgen05 / TMEM SparseConv2D kernels for 16-bit tensors (bf16 / fp16 in, fp32 accumulate).
//
// One CTA owns a 128-row x BN-column output tile whose fp32 accumulator lives in tensor memory.
// Eight producer warps gather operand rows with 16-byte cp.async straight into the 128-byte-swizzled
// shared-memory layout that the UMMA descriptors describe (the gathered x / gy rows are never
// materialised in HBM), one elected thread issues tcgen05.mma, and the producer warps turn into the
// epilogue (tcgen05.ld -> +bias -> one rounding -> 16-byte stores).  A ring of mbarrier-guarded
// stages decouples the three roles.  Every wait is bounded: when it runs out the CTA records an
// error code in a device word, skips its stores, frees its tensor memory and returns.
//
//   forward   D[128, BN] += A(K-major: gathered x rows, 64 channels per stage) . B(MN-major: W[k] rows)
//   dgrad     same kernel, A = gathered gy rows through the mirrored table column, B = W[KK-1-k]
//             read K-major (i.e. transposed) - valid for symmetric tables
//   wgrad     D[128 = two 64-channel blocks of (tap, ci), BN] += A(MN-major: gathered x rows, 64 tokens
//             per stage) . B(MN-major: gy rows); split over tokens, fp32 partials to the workspace
//
// Replaces opentad/models/bricks/implicit_gemm_v2.cu:197-417 (gather kernel + cuBLAS batched GEMM +
// reduce kernel) and the atomic backward kernels opentad/models/bricks/2d_sparse_v3.cu:656-745.
#include <cstdlib>

#include "tc_common.cuh"

namespace svtad {

__device__ int g_tc_error = 0;

constexpr int TC_THREADS = 288;        // 4 A-producer warps, 4 B-producer warps, 1 MMA warp
constexpr int LAG = 2;                 // writer-fence protocol only: cp.async groups in flight per thread

struct TcSmemTail {            // lives after the stage ring in dynamic shared memory
    uint64_t full[8];
    uint64_t empty[8];
    uint64_t accum;
    uint32_t tmem_slot;
    int abort_flag;
    int any[52];
};

// ---------------------------------------------------------------------------------------------
// forward / dgrad
// ---------------------------------------------------------------------------------------------
template <int BN, bool DGRAD>
__global__ void __launch_bounds__(TC_THREADS, 1)
conv_tc_kernel(const uint16_t* __restrict__ a, const int32_t* __restrict__ nbr,
               const uint16_t* __restrict__ w, const uint16_t* __restrict__ bias,
               uint16_t* __restrict__ out, const int32_t* __restrict__ status, long n, int cred,
               int cn, int cin, int cout, int kk, int tpb, int nstage, int fp16, int writer_fence,
               int* __restrict__ err, int dbg) {
    if (DGRAD && status != nullptr && (__ldg(status) & SVTAD_TABLE_ASYMMETRIC)) return;
    constexpr int B_TILE_BYTES = b_tile_bytes_for(BN);
    constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
    constexpr int TM_COLS = tmem_cols_for(BN);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    TcSmemTail* tail = reinterpret_cast<TcSmemTail*>(smem + (size_t)nstage * STAGE_BYTES);
    float* s_bias = reinterpret_cast<float*>(tail + 1);
    int* s_nbr = reinterpret_cast<int*>(s_bias + BN);           // [TILE_M][kk]
    volatile int* s_abort = &tail->abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const long row0 = (long)blockIdx.x * TILE_M;
    const int n0 = blockIdx.y * BN;
    const uint32_t stage_base = smem_u32(smem);

    if (warp == 8) {
        tmem_alloc(smem_u32(&tail->tmem_slot), TM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        for (int s = 0; s < nstage; ++s) {
            mbar_init(smem_u32(&tail->full[s]), 256);
            mbar_init(smem_u32(&tail->empty[s]), 1);
        }
        mbar_init(smem_u32(&tail->accum), 1);
        tail->abort_flag = 0;
        fence_mbar_init();
    }
    for (int t = tid; t < kk; t += TC_THREADS) tail->any[t] = 0;
    for (int t = tid; t < BN; t += TC_THREADS)
        s_bias[t] = (!DGRAD && bias != nullptr) ? widen(bias[n0 + t], fp16 != 0) : 0.f;
    __syncthreads();
    for (int e = tid; e < TILE_M * kk; e += TC_THREADS) {
        int r = e / kk, k = e - r * kk;
        long i = row0 + r;
        int v = -1;
        if (i < n) {
            int j = __ldg(nbr + i * kk + k);
            if (j != -1) {
                long jj = (long)j + (tpb > 0 ? (i / tpb) * (long)tpb : 0);
                if (jj >= 0 && jj < n) v = (int)jj;
            }
        }
        s_nbr[e] = v;
        if (v >= 0) tail->any[k] = 1;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tail->tmem_slot;

    const int kchunks = cred / STAGE_K;
    int total_stages = 0;
    for (int k = 0; k < kk; ++k) total_stages += tail->any[k] ? kchunks : 0;

    if (warp < 8) {
        // ------------------------------------------------------------------ producers
        const int pt = tid & 127;
        int it = 0;
        bool alive = true;
        for (int k = 0; k < kk && alive; ++k) {
            if (!tail->any[k]) continue;
            const int wtap = DGRAD ? (kk - 1 - k) : k;
            const uint16_t* wk = w + (long)wtap * cin * cout;
            for (int kc = 0; kc < kchunks; ++kc, ++it) {
                const int s = it % nstage;
                if (!mbar_wait(smem_u32(&tail->empty[s]), ((it / nstage) & 1) ^ 1, s_abort, err, 1)) { alive = false; break; }
                const uint32_t a_tile = stage_base + (uint32_t)s * STAGE_BYTES;
                const uint32_t b_tile = a_tile + A_TILE_BYTES;
                const int c0 = kc * STAGE_K;
                if (dbg & 1) {
                    // timing experiment: no copies
                } else if (warp < 4) {
                    // A: 128 rows x 8 chunks of 16 B; 8 consecutive threads cover one row's 128 B
                    const int sub = pt & 7, rbase = pt >> 3;
                    const uint32_t dst0 = a_tile + rbase * 128 + ((sub ^ (rbase & 7)) << 4);
#pragma unroll
                    for (int itr = 0; itr < 8; ++itr) {
                        int r = itr * 16 + rbase;
                        int j = s_nbr[r * kk + k];
                        const uint16_t* src = a + (long)(j < 0 ? 0 : j) * cred + c0 + sub * 8;
                        cp_async16(dst0 + itr * 2048, src, j < 0 ? 0u : 16u);
                    }
                } else if (!DGRAD) {
                    // B (MN-major): 64 reduction rows x BN columns, 64-column blocks 8 KB apart
#pragma unroll
                    for (int itr = 0; itr < BN / 16; ++itr) {
                        int q = itr * 128 + pt;
                        int r = q / (BN / 8), cc = q % (BN / 8);
                        const uint16_t* src = wk + (long)(c0 + r) * cout + n0 + cc * 8;
                        uint32_t dst = b_tile + (cc >> 3) * 8192 + r * 128 + (((cc & 7) ^ (r & 7)) << 4);
                        cp_async16(dst, src, 16u);
                    }
                } else {
                    // B (K-major): BN output rows x 64 reduction elements, W[wtap][n0+nn][c0 ..]
#pragma unroll
                    for (int itr = 0; itr < BN / 16; ++itr) {
                        int q = itr * 128 + pt;
                        int nn = q >> 3, c = q & 7;
                        const uint16_t* src = wk + (long)(n0 + nn) * cout + c0 + c * 8;
                        uint32_t dst = b_tile + nn * 128 + ((c ^ (nn & 7)) << 4);
                        cp_async16(dst, src, 16u);
                    }
                }
                if (!writer_fence) {
                    cp_async_arrive_noinc(smem_u32(&tail->full[s]));
                } else {
                    cp_async_commit();
                    if (it >= LAG) {
                        cp_async_wait<LAG>();
                        fence_proxy_async();
                        mbar_arrive(smem_u32(&tail->full[(it - LAG) % nstage]));
                    }
                }
            }
        }
        if (writer_fence) {
            cp_async_wait<0>();
            fence_proxy_async();
            if (alive) {
                int first = total_stages - LAG < 0 ? 0 : total_stages - LAG;
                for (int j = first; j < total_stages; ++j) mbar_arrive(smem_u32(&tail->full[j % nstage]));
            }
        }

        // ------------------------------------------------------------------ epilogue
        bool have = alive;
        if (have && total_stages > 0) have = mbar_wait(smem_u32(&tail->accum), 0, s_abort, err, 3);
        tc_fence_after();
        if (have) {
            const int q = warp & 3, hsel = warp >> 2;
            const long row = row0 + q * 32 + lane;
            // warps w and w+4 share a lane quarter and alternate over the 16-column chunks
#pragma unroll 1
            for (int cbase = hsel * 16; cbase < BN; cbase += 32) {
                uint32_t v[16];
                if (total_stages > 0) {
                    tmem_ld16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + cbase, v);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = 0u;
                }
                if (row < n) {
                    uint4* dst = reinterpret_cast<uint4*>(out + row * cn + n0 + cbase);
#pragma unroll
                    for (int g = 0; g < 2; ++g) {
                        uint4 o;
                        o.x = pack2(__uint_as_float(v[g * 8 + 0]) + s_bias[cbase + g * 8 + 0],
                                    __uint_as_float(v[g * 8 + 1]) + s_bias[cbase + g * 8 + 1], fp16 != 0);
                        o.y = pack2(__uint_as_float(v[g * 8 + 2]) + s_bias[cbase + g * 8 + 2],
                                    __uint_as_float(v[g * 8 + 3]) + s_bias[cbase + g * 8 + 3], fp16 != 0);
                        o.z = pack2(__uint_as_float(v[g * 8 + 4]) + s_bias[cbase + g * 8 + 4],
                                    __uint_as_float(v[g * 8 + 5]) + s_bias[cbase + g * 8 + 5], fp16 != 0);
                        o.w = pack2(__uint_as_float(v[g * 8 + 6]) + s_bias[cbase + g * 8 + 6],
                                    __uint_as_float(v[g * 8 + 7]) + s_bias[cbase + g * 8 + 7], fp16 != 0);
                        dst[g] = o;
                    }
                }
            }
        }
    } else if (lane == 0) {
        // ------------------------------------------------------------------ MMA issuer
        const uint32_t idesc = make_idesc(fp16 ? 0 : 1, 0, DGRAD ? 0 : 1, TILE_M, BN);
        bool alive = true;
        for (int it = 0; it < total_stages; ++it) {
            const int s = it % nstage;
            if (!mbar_wait(smem_u32(&tail->full[s]), (it / nstage) & 1, s_abort, err, 2)) { alive = false; break; }
            fence_proxy_async();   // cp.async (generic proxy) writes -> tcgen05.mma (async proxy) reads
            tc_fence_after();
            const uint32_t a_tile = stage_base + (uint32_t)s * STAGE_BYTES;
            const uint32_t b_tile = a_tile + A_TILE_BYTES;
#pragma unroll
            for (int ks = 0; ks < STAGE_K / 16; ++ks) {
                uint64_t ad = make_smem_desc(a_tile + ks * 32, 0, 1024);
                uint64_t bd = DGRAD ? make_smem_desc(b_tile + ks * 32, 0, 1024)
                                    : make_smem_desc(b_tile + ks * 2048, 8192, 1024);
                if (!(dbg & 2)) umma_f16(tmem_base, ad, bd, idesc, (it | ks) != 0 ? 1u : 0u);
            }
            umma_commit(smem_u32(&tail->empty[s]));
        }
        if (alive && total_stages > 0) umma_commit(smem_u32(&tail->accum));
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, TM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
// wgrad
// ---------------------------------------------------------------------------------------------
template <int BN>
__global__ void __launch_bounds__(TC_THREADS, 1)
wgrad_tc_kernel(const uint16_t* __restrict__ gy, const uint16_t* __restrict__ x,
                const int32_t* __restrict__ nbr, float* __restrict__ ws, long n, int cin, int cout,
                int kk, int tpb, long tokens_per_split, int n_nblk, int nstage, int fp16,
                int writer_fence, int* __restrict__ err) {
    constexpr int B_TILE_BYTES = b_tile_bytes_for(BN);
    constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
    constexpr int TM_COLS = tmem_cols_for(BN);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    TcSmemTail* tail = reinterpret_cast<TcSmemTail*>(smem + (size_t)nstage * STAGE_BYTES);
    volatile int* s_abort = &tail->abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int pair = blockIdx.x / n_nblk;
    const int n0 = (blockIdx.x % n_nblk) * BN;
    const int cblocks = cin / 64;
    const int nblocks = kk * cblocks;
    const long i_begin = (long)blockIdx.y * tokens_per_split;
    const long i_end = min(n, i_begin + tokens_per_split);
    const int total_stages = i_end > i_begin ? (int)((i_end - i_begin + STAGE_K - 1) / STAGE_K) : 0;
    const uint32_t stage_base = smem_u32(smem);

    if (warp == 8) {
        tmem_alloc(smem_u32(&tail->tmem_slot), TM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        for (int s = 0; s < nstage; ++s) {
            mbar_init(smem_u32(&tail->full[s]), 256);
            mbar_init(smem_u32(&tail->empty[s]), 1);
        }
        mbar_init(smem_u32(&tail->accum), 1);
        tail->abort_flag = 0;
        fence_mbar_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tail->tmem_slot;

    if (warp < 8) {
        const int pt = tid & 127;
        bool alive = true;
        if (warp < 4) {
            // A: two 64-channel blocks (tap_h, chunk_h); block h holds 64 token rows of 128 B at h * 8 KB.
            const int sub = pt & 7, rbase = pt >> 3;
            int tap[2], ch0[2];
            bool real[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                int blk = pair * 2 + h;
                real[h] = blk < nblocks;
                tap[h] = real[h] ? blk / cblocks : 0;
                ch0[h] = real[h] ? (blk % cblocks) * 64 : 0;
            }
            // gather indices of the next stage are fetched while this stage's copies are issued
            int cur[8], nxt[8];
            auto fetch = [&](int stage_it, int (&dst)[8]) {
#pragma unroll
                for (int itr = 0; itr < 8; ++itr) {
                    const int h = itr >> 2;
                    long i = i_begin + (long)stage_it * STAGE_K + (itr & 3) * 16 + rbase;
                    int v = -1;
                    if (real[h] && i < i_end) {
                        int j = __ldg(nbr + i * kk + tap[h]);
                        if (j != -1) {
                            long jj = (long)j + (tpb > 0 ? (i / tpb) * (long)tpb : 0);
                            if (jj >= 0 && jj < n) v = (int)jj;
                        }
                    }
                    dst[itr] = v;
                }
            };
            if (total_stages > 0) fetch(0, cur);
            for (int it = 0; it < total_stages; ++it) {
                const int s = it % nstage;
                if (it + 1 < total_stages) fetch(it + 1, nxt);
                if (!mbar_wait(smem_u32(&tail->empty[s]), ((it / nstage) & 1) ^ 1, s_abort, err, 11)) { alive = false; break; }
                const uint32_t a_tile = stage_base + (uint32_t)s * STAGE_BYTES;
                const uint32_t dst0 = a_tile + rbase * 128 + ((sub ^ (rbase & 7)) << 4);
#pragma unroll
                for (int itr = 0; itr < 8; ++itr) {
                    const int h = itr >> 2;
                    int j = cur[itr];
                    const uint16_t* src = x + (long)(j < 0 ? 0 : j) * cin + ch0[h] + sub * 8;
                    cp_async16(dst0 + itr * 2048, src, j < 0 ? 0u : 16u);
                }
                if (!writer_fence) {
                    cp_async_arrive_noinc(smem_u32(&tail->full[s]));
                } else {
                    cp_async_commit();
                    if (it >= LAG) {
                        cp_async_wait<LAG>();
                        fence_proxy_async();
                        mbar_arrive(smem_u32(&tail->full[(it - LAG) % nstage]));
                    }
                }
#pragma unroll
                for (int itr = 0; itr < 8; ++itr) cur[itr] = nxt[itr];
            }
        } else {
            // B: 64 token rows x BN columns of gy, 64-column blocks 8 KB apart
            for (int it = 0; it < total_stages; ++it) {
                const int s = it % nstage;
                if (!mbar_wait(smem_u32(&tail->empty[s]), ((it / nstage) & 1) ^ 1, s_abort, err, 12)) { alive = false; break; }
                const uint32_t b_tile = stage_base + (uint32_t)s * STAGE_BYTES + A_TILE_BYTES;
                const long i0 = i_begin + (long)it * STAGE_K;
#pragma unroll
                for (int itr = 0; itr < BN / 16; ++itr) {
                    int q = itr * 128 + pt;
                    int r = q / (BN / 8), cc = q % (BN / 8);
                    long i = i0 + r;
                    bool ok = i < i_end;
                    const uint16_t* src = gy + (ok ? i : 0) * cout + n0 + cc * 8;
                    uint32_t dst = b_tile + (cc >> 3) * 8192 + r * 128 + (((cc & 7) ^ (r & 7)) << 4);
                    cp_async16(dst, src, ok ? 16u : 0u);
                }
                if (!writer_fence) {
                    cp_async_arrive_noinc(smem_u32(&tail->full[s]));
                } else {
                    cp_async_commit();
                    if (it >= LAG) {
                        cp_async_wait<LAG>();
                        fence_proxy_async();
                        mbar_arrive(smem_u32(&tail->full[(it - LAG) % nstage]));
                    }
                }
            }
        }
        if (writer_fence) {
            cp_async_wait<0>();
            fence_proxy_async();
            if (alive) {
                int first = total_stages - LAG < 0 ? 0 : total_stages - LAG;
                for (int j = first; j < total_stages; ++j) mbar_arrive(smem_u32(&tail->full[j % nstage]));
            }
        }

        // epilogue: fp32 partial tile -> workspace[split][(tap, ci)][co]
        bool have = alive;
        if (have && total_stages > 0) have = mbar_wait(smem_u32(&tail->accum), 0, s_abort, err, 13);
        tc_fence_after();
        if (have) {
            const int q = warp & 3, hsel = warp >> 2;
            const int blk = pair * 2 + (q >> 1);
            if (blk < nblocks) {
                const long grow = (long)(blk / cblocks) * cin + (blk % cblocks) * 64 + (q & 1) * 32 + lane;
                float* dstrow = ws + ((long)blockIdx.y * kk * cin + grow) * cout + n0;
#pragma unroll 1
                for (int cbase = hsel * 16; cbase < BN; cbase += 32) {
                    uint32_t v[16];
                    if (total_stages > 0) {
                        tmem_ld16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + cbase, v);
                        tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = 0u;
                    }
                    uint4* dst = reinterpret_cast<uint4*>(dstrow + cbase);
#pragma unroll
                    for (int g = 0; g < 4; ++g) dst[g] = make_uint4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
                }
            }
        }
    } else if (lane == 0) {
        const uint32_t idesc = make_idesc(fp16 ? 0 : 1, 1, 1, TILE_M, BN);
        bool alive = true;
        for (int it = 0; it < total_stages; ++it) {
            const int s = it % nstage;
            if (!mbar_wait(smem_u32(&tail->full[s]), (it / nstage) & 1, s_abort, err, 14)) { alive = false; break; }
            fence_proxy_async();
            tc_fence_after();
            const uint32_t a_tile = stage_base + (uint32_t)s * STAGE_BYTES;
            const uint32_t b_tile = a_tile + A_TILE_BYTES;
#pragma unroll
            for (int ks = 0; ks < STAGE_K / 16; ++ks) {
                uint64_t ad = make_smem_desc(a_tile + ks * 2048, 8192, 1024);
                uint64_t bd = make_smem_desc(b_tile + ks * 2048, 8192, 1024);
                umma_f16(tmem_base, ad, bd, idesc, (it | ks) != 0 ? 1u : 0u);
            }
            umma_commit(smem_u32(&tail->empty[s]));
        }
        if (alive && total_stages > 0) umma_commit(smem_u32(&tail->accum));
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, TM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
constexpr size_t SMEM_LIMIT = 227 * 1024;

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

static int num_sms() {
    static int cached = 0;
    if (cached == 0) {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0)
            cached = v;
        else
            cached = 148;
    }
    return cached;
}

// Operand feed of the tensor-core kernels: "tma" (conv_tc_tma.cu) or "cpasync" (this file).
static bool use_tma() {
    const char* e = getenv("SVTAD_TC_IMPL");
    if (e != nullptr && *e) return e[0] == 't';
    return true;
}

static bool writer_fence_mode() {
    const char* e = getenv("SVTAD_TC_WRITER_FENCE");
    return e != nullptr && *e == '1';
}

// Column-block width of a forward / dgrad CTA.  One CTA runs per SM, so the cost of a choice is
// (waves over the SMs) x (bytes a CTA stages per K step: 16 KB of gathered rows + its weight tile).
static int pick_bn(int cn, long m_tiles) {
    const int cand[5] = {256, 192, 128, 96, 64};
    const char* e = getenv("SVTAD_TC_BN");
    if (e != nullptr && *e) {
        int v = atoi(e);
        for (int c : cand)
            if (v == c && cn % v == 0) return v;
    }
    const long sms = num_sms();
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

static int stages_for(int bn, size_t extra) {
    size_t stage = A_TILE_BYTES + (size_t)b_tile_bytes_for(bn);
    size_t avail = SMEM_LIMIT - 1024 - sizeof(TcSmemTail) - extra;
    int s = (int)(avail / stage);
    return s > 8 ? 8 : s;
}

bool tc_supported(int op, int64_t n, int cin, int cout, int kk, int dtype) {
    if (dtype != SVTAD_BF16 && dtype != SVTAD_F16) return false;
    if (n <= 0 || kk > 49) return false;
    if (cin % 64 != 0 || cout % 64 != 0) return false;
    (void)op;
    return true;
}

template <int BN, bool DGRAD>
static int launch_conv_tc(const ConvArgs& p, const int32_t* status, cudaStream_t s) {
    const int cred = DGRAD ? p.cout : p.cin;
    const int cn = DGRAD ? p.cin : p.cout;
    size_t extra = (size_t)BN * sizeof(float) + (size_t)TILE_M * p.kk * sizeof(int);
    int nstage = stages_for(BN, extra);
    if (nstage < LAG + 2)
        return set_error(SVTAD_ERR_UNSUPPORTED, "tensor-core conv: not enough shared memory for BN=%d kk=%d", BN, p.kk);
    size_t smem = 1024 + (size_t)nstage * (A_TILE_BYTES + b_tile_bytes_for(BN)) + sizeof(TcSmemTail) + extra;
    auto kern = conv_tc_kernel<BN, DGRAD>;
    SV_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)((p.n + TILE_M - 1) / TILE_M), (unsigned)(cn / BN));
    kern<<<grid, TC_THREADS, smem, s>>>((const uint16_t*)p.a, p.nbr, (const uint16_t*)p.w,
                                        (const uint16_t*)p.bias, (uint16_t*)p.out, status, (long)p.n,
                                        cred, cn, p.cin, p.cout, p.kk, p.tpb, nstage,
                                        p.dtype == SVTAD_F16 ? 1 : 0, writer_fence_mode() ? 1 : 0, tc_error_ptr(),
                                        getenv("SVTAD_TC_DEBUG") ? atoi(getenv("SVTAD_TC_DEBUG")) : 0);
    SV_LAUNCH_CHECK("conv_tc_kernel");
    return SVTAD_OK;
}

template <bool DGRAD>
static int dispatch_conv_tc(const ConvArgs& p, const int32_t* status, cudaStream_t s) {
    const int cn = DGRAD ? p.cin : p.cout;
    int bn = pick_bn(cn, (p.n + TILE_M - 1) / TILE_M);
    switch (bn) {
        case 64: return launch_conv_tc<64, DGRAD>(p, status, s);
        case 96: return launch_conv_tc<96, DGRAD>(p, status, s);
        case 128: return launch_conv_tc<128, DGRAD>(p, status, s);
        case 192: return launch_conv_tc<192, DGRAD>(p, status, s);
        case 256: return launch_conv_tc<256, DGRAD>(p, status, s);
    }
    return set_error(SVTAD_ERR_UNSUPPORTED, "tensor-core conv: no column block for width %d", cn);
}

int tc_fwd(const ConvArgs& p, cudaStream_t s) {
    return use_tma() ? tma_fwd(p, s) : dispatch_conv_tc<false>(p, nullptr, s);
}
int tc_dgrad(const ConvArgs& p, const int32_t* status, cudaStream_t s) {
    return use_tma() ? tma_dgrad(p, status, s) : dispatch_conv_tc<true>(p, status, s);
}

struct WgradPlan {
    int bn, n_nblk, n_pairs, splits;
    long tokens_per_split;
};

static WgradPlan wgrad_plan(int64_t n, int cin, int cout, int kk) {
    WgradPlan pl;
    pl.bn = (cout <= 256) ? cout : (cout % 256 == 0 ? 256 : (cout % 192 == 0 ? 192 : (cout % 128 == 0 ? 128 : 64)));
    pl.n_nblk = cout / pl.bn;
    int nblocks = kk * (cin / 64);
    pl.n_pairs = (nblocks + 1) / 2;
    long ctas = (long)pl.n_pairs * pl.n_nblk;
    const long sms = num_sms();
    long max_by_rows = (n + 2 * STAGE_K - 1) / (2 * STAGE_K);
    if (max_by_rows < 1) max_by_rows = 1;
    if (max_by_rows > 64) max_by_rows = 64;
    // splits over tokens: minimise (waves over the SMs) x (tokens per split), ties to fewer splits
    long s = 1;
    double best = 0;
    for (long c = 1; c <= max_by_rows; ++c) {
        long waves = (ctas * c + sms - 1) / sms;
        double cost = (double)waves * (double)((n + c - 1) / c + 2 * STAGE_K);
        if (c == 1 || cost < best * 0.98) { best = cost; s = c; }
    }
    const char* e = getenv("SVTAD_TC_WGRAD_SPLITS");
    if (e != nullptr && *e && atoi(e) > 0) s = atoi(e) < max_by_rows ? atoi(e) : max_by_rows;
    long tps = ((n + s - 1) / s + STAGE_K - 1) / STAGE_K * STAGE_K;
    pl.tokens_per_split = tps;
    pl.splits = (int)((n + tps - 1) / tps);
    return pl;
}

static size_t cpasync_wgrad_ws_bytes(int64_t n, int cin, int cout, int kk) {
    WgradPlan pl = wgrad_plan(n, cin, cout, kk);
    size_t w = (size_t)pl.splits * kk * cin * cout * sizeof(float);
    size_t b = (size_t)bias_splits_for(n) * cout * sizeof(float);
    return align_up(w, 256) + align_up(b, 256);
}

size_t tc_wgrad_ws_bytes(int64_t n, int cin, int cout, int kk) {
    size_t a = cpasync_wgrad_ws_bytes(n, cin, cout, kk), b = tma_wgrad_ws_bytes(n, cin, cout, kk);
    return a > b ? a : b;
}

template <int BN>
static int launch_wgrad_tc(const void* gy, const void* x, const int32_t* nbr, float* ws, int64_t n,
                           int cin, int cout, int kk, int tpb, int dtype, const WgradPlan& pl,
                           cudaStream_t s) {
    int nstage = stages_for(BN, 0);
    size_t smem = 1024 + (size_t)nstage * (A_TILE_BYTES + b_tile_bytes_for(BN)) + sizeof(TcSmemTail);
    auto kern = wgrad_tc_kernel<BN>;
    SV_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)(pl.n_pairs * pl.n_nblk), (unsigned)pl.splits);
    kern<<<grid, TC_THREADS, smem, s>>>((const uint16_t*)gy, (const uint16_t*)x, nbr, ws, (long)n, cin,
                                        cout, kk, tpb, pl.tokens_per_split, pl.n_nblk, nstage,
                                        dtype == SVTAD_F16 ? 1 : 0, writer_fence_mode() ? 1 : 0, tc_error_ptr());
    SV_LAUNCH_CHECK("wgrad_tc_kernel");
    return SVTAD_OK;
}

int tc_wgrad(const void* gy, const void* x, const int32_t* nbr, void* gw, void* gb, int64_t n, int cin,
             int cout, int kk, int tpb, int dtype, void* ws, size_t ws_bytes, cudaStream_t s) {
    if (use_tma()) return tma_wgrad(gy, x, nbr, gw, gb, n, cin, cout, kk, tpb, dtype, ws, ws_bytes, s);
    size_t need = cpasync_wgrad_ws_bytes(n, cin, cout, kk);
    if (ws_bytes < need)
        return set_error(SVTAD_ERR_WORKSPACE, "svtad_conv_wgrad: workspace %zu < %zu bytes", ws_bytes, need);
    WgradPlan pl = wgrad_plan(n, cin, cout, kk);
    const long n_w = (long)kk * cin * cout;
    float* ws_w = static_cast<float*>(ws);
    float* ws_b = reinterpret_cast<float*>(static_cast<char*>(ws) + align_up((size_t)pl.splits * n_w * sizeof(float), 256));
    int rc;
    switch (pl.bn) {
        case 64: rc = launch_wgrad_tc<64>(gy, x, nbr, ws_w, n, cin, cout, kk, tpb, dtype, pl, s); break;
        case 128: rc = launch_wgrad_tc<128>(gy, x, nbr, ws_w, n, cin, cout, kk, tpb, dtype, pl, s); break;
        case 192: rc = launch_wgrad_tc<192>(gy, x, nbr, ws_w, n, cin, cout, kk, tpb, dtype, pl, s); break;
        case 256: rc = launch_wgrad_tc<256>(gy, x, nbr, ws_w, n, cin, cout, kk, tpb, dtype, pl, s); break;
        default: return set_error(SVTAD_ERR_UNSUPPORTED, "tensor-core wgrad: no column block for width %d", cout);
    }
    if (rc) return rc;
    int splits_b = 0;
    if (gb != nullptr) {
        splits_b = bias_splits_for(n);
        rc = bias_partial_launch(gy, ws_b, n, cout, dtype, splits_b, s);
        if (rc) return rc;
    }
    return wgrad_finalize_launch(ws_w, pl.splits, ws_b, splits_b, gw, gb, n_w, cout, dtype, s);
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

}  // namespace svtad
