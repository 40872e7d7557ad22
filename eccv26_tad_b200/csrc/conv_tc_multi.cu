// One persistent tcgen05 kernel over a LIST of SparseConv2D work items of mixed kinds.
//
// The single-purpose kernels (conv_tc_hybrid.cu) pay a fixed cost per launch that is as large as their main
// loop at the sizes a training step has: the trip to the neighbour table and then to the gathered rows before
// the first MMA can start, and the drain of the accumulator after the last one.  Here a CTA walks a list of
// items - forward tiles, input-gradient tiles and weight-gradient (block pair, token split) items of one or
// several problems - through ONE ring of shared-memory stages and two accumulators in tensor memory, so the
// next item's table and first operands arrive while the current item's MMAs run, and the current item's
// accumulator is drained while the next item's MMAs run.  The backward of a layer (input gradient + weight
// gradient, opentad/models/bricks/sparse_conv_layer.py:100-117, which the reference launches as two kernels
// after one another) becomes one launch plus the small fixed-order reduction of the weight-gradient partials.
//
// Item kinds and their operands (64-deep K steps, 128-byte swizzle everywhere):
//   forward   D[128 rows, BN] += A(K-major: gathered x rows) . B(MN-major: W[k] by TMA)
//   dgrad     D[128 rows, BN] += A(K-major: gathered gy rows) . B(K-major: W[KK-1-k] by TMA)      (gather form)
//   wgrad     D[2 x 64 (tap, ci) rows, BN] += A(MN-major: gathered x rows of 64 tokens) . B(MN-major: gy rows by TMA)
//             fp32 partial per token split to the workspace; an all-ones spare block yields the bias gradient
// Roles per CTA (288 threads): warps 0-3 produce (cp.async gathers; lane 0 of the owning warp issues the TMA),
// warp 4 lane 0 issues the MMAs, warps 5-8 drain accumulators.  A producer warp owns every fourth K step of the
// CTA's whole item sequence, so its turn continues seamlessly from one item into the next.
// Every mbarrier wait is bounded; on expiry the CTA records a code in the device error word, stops issuing,
// frees its tensor memory and returns.  No TMA load uses cluster multicast.
#include <cstdlib>
#include <cstring>

#include "tc_common.cuh"

namespace svtad {

constexpr int MU_THREADS = 288;
constexpr int MU_A_WARPS = 4;
constexpr int MU_A_THREADS = MU_A_WARPS * 32;
constexpr int MU_MAX_PROBLEMS = 6;

enum : int { MU_FWD = 0, MU_DGRAD = 1, MU_WGRAD = 2 };

struct MultiProblem {
    CUtensorMap map_b;          // forward / dgrad: the weight; wgrad: gy
    const uint16_t* a;          // gathered operand: x (forward, wgrad) or gy (dgrad)
    const int32_t* nbr;
    const uint16_t* bias;       // forward only, may be null
    uint16_t* out;              // forward: y, dgrad: gx
    float* ws_w;                // wgrad: per-split partials
    float* ws_b;                // wgrad: per-split bias partials (null = not wanted)
    long n;
    long tokens_per_split;      // wgrad
    int kind;
    int cred;                   // channels of the gathered operand
    int cn;                     // width of the output rows (forward: cout, dgrad: cin, wgrad: cout)
    int kk, tpb;
    int n_blks;                 // column blocks of width BN
    int first_item, n_items;
    int n_units;                // forward / dgrad: row tiles; wgrad: block pairs
    int splits;                 // wgrad
    int ones_block;             // wgrad: the block count is odd, the spare block carries the bias gradient
    int out_al32;
};

struct MultiParams {
    MultiProblem p[MU_MAX_PROBLEMS];
    int n_problems;
    int total_items;
    int nstage;
    int fp16;
    int kk_max;
    int* err;
};

struct MuItem {
    int prob;
    int kind;
    int steps;
    // forward / dgrad
    long row0;
    // wgrad
    int pair;
    int split;
    long i_begin, i_end;
    int n0;
};

__device__ __forceinline__ MuItem mu_decode(const MultiParams& P, int item) {
    MuItem it;
    int pi = 0;
#pragma unroll
    for (int q = 1; q < MU_MAX_PROBLEMS; ++q)
        if (q < P.n_problems && item >= P.p[q].first_item) pi = q;
    const MultiProblem& pr = P.p[pi];
    const int local = item - pr.first_item;
    it.prob = pi;
    it.kind = pr.kind;
    it.row0 = 0; it.pair = 0; it.split = 0; it.i_begin = 0; it.i_end = 0;
    if (pr.kind != MU_WGRAD) {
        it.row0 = (long)(local / pr.n_blks) * TILE_M;
        it.n0 = (local % pr.n_blks);
        it.steps = pr.kk * (pr.cred / STAGE_K);
    } else {
        const int per_split = pr.n_units * pr.n_blks;
        const int bx = local % per_split;
        it.split = local / per_split;
        it.pair = bx / pr.n_blks;
        it.n0 = bx % pr.n_blks;
        it.i_begin = (long)it.split * pr.tokens_per_split;
        it.i_end = pr.n < it.i_begin + pr.tokens_per_split ? pr.n : it.i_begin + pr.tokens_per_split;
        it.steps = it.i_end > it.i_begin ? (int)((it.i_end - it.i_begin + STAGE_K - 1) / STAGE_K) : 0;
    }
    return it;
}

__device__ __forceinline__ bool mu_warp_wait(uint32_t bar, uint32_t parity, volatile int* s_abort, int* err, int code,
                                             int lane) {
    int ok = 1;
    if (lane == 0) ok = mbar_wait(bar, parity, s_abort, err, code) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    __syncwarp();
    return ok != 0;
}

template <int BN>
__global__ void __launch_bounds__(MU_THREADS, 1)
conv_multi_kernel(const __grid_constant__ MultiParams P) {
    constexpr int B_TILE_BYTES = b_tile_bytes_for(BN);
    constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
    constexpr int TM_COLS = tmem_cols2_for(BN);
    constexpr int NC = BN / 32;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int nstage = P.nstage;
    TmaTail* tail = reinterpret_cast<TmaTail*>(smem + (size_t)nstage * STAGE_BYTES);
    const int tab_ints = TILE_M * P.kk_max;
    int* s_raw = reinterpret_cast<int*>(tail + 1);         // [128 * kk] raw table rows of the coming forward / dgrad tile
    int* s_xf = s_raw + tab_ints;                          // [kk][4][32] final row numbers of the current tile
    float* s_bias = reinterpret_cast<float*>(s_xf + tab_ints);                    // [2][256]
    int* s_wrows = reinterpret_cast<int*>(s_bias + 512);   // per producer warp: [2][128] raw entries + [128] final rows
    volatile int* s_abort = &tail->abort_flag;
    int* err = P.err;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t stage_base = smem_u32(smem);
    const int total_items = P.total_items;
    const int n_prod = nstage < MU_A_WARPS ? nstage : MU_A_WARPS;
    const bool fp16 = P.fp16 != 0;

    // ---- helpers of the producers -------------------------------------------------------------------------
    // raw table rows of a forward / dgrad tile -> s_raw (all producer threads), with an L2 prefetch of the rows
    // the tile will gather
    auto load_table = [&](const MultiProblem& pr, long row0) {
        const long rows = (pr.n - row0) < TILE_M ? (pr.n - row0) : TILE_M;
        const int valid_bytes = (int)rows * pr.kk * 4;
        const char* src = reinterpret_cast<const char*>(pr.nbr + row0 * pr.kk);
        const uint32_t dst = smem_u32(s_raw);
        for (int c = tid; c * 16 < TILE_M * pr.kk * 4; c += MU_A_THREADS) {
            int left = valid_bytes - c * 16;
            uint32_t nb = left >= 16 ? 16u : (left > 0 ? (uint32_t)left : 0u);
            cp_async16(dst + c * 16, nb ? src + c * 16 : src, nb);
        }
        if (tid == MU_A_THREADS - 1) l2_prefetch_rows(pr.a, row0 - 64, row0 + TILE_M + 64, pr.n, pr.cred);
    };
    // the two table entries (one per block of the pair) of each of the 64 tokens of a wgrad step -> this warp's
    // raw buffer `buf`; slot = block * 64 + token
    int* my_w = s_wrows + warp * 384;
    auto load_wrows = [&](const MultiProblem& pr, const MuItem& it, int st, int buf, bool pf) {
        const int cblocks = pr.cred / 64;
        const int nblocks = pr.kk * cblocks;
        const long i0 = it.i_begin + (long)st * STAGE_K;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int slot = lane * 4 + j;
            const int h = slot >> 6, t = slot & 63;
            const int blk = it.pair * 2 + h;
            const long i = i0 + t;
            const bool real = blk < nblocks && i < it.i_end;
            const int tap = real ? blk / cblocks : 0;
            const int32_t* src = pr.nbr + (real ? i * pr.kk + tap : 0);
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;"
                         ::"r"(smem_u32(my_w + buf * 128 + slot)), "l"(src), "r"(real ? 4u : 0u) : "memory");
        }
        if (lane == 31 && pf) l2_prefetch_rows(pr.a, i0 - 64, i0 + STAGE_K + 64, pr.n, pr.cred);
    };

    // ---- set-up ------------------------------------------------------------------------------------------
    // the first item's table starts its trip before anything else is set up
    MuItem first;
    if ((int)blockIdx.x < total_items) first = mu_decode(P, blockIdx.x);
    if (warp < MU_A_WARPS && (int)blockIdx.x < total_items) {
        const MultiProblem& pr = P.p[first.prob];
        if (first.kind != MU_WGRAD) {
            load_table(pr, first.row0);
        } else if (warp < n_prod && warp < first.steps) {
            load_wrows(pr, first, warp, 0, true);
        }
        cp_async_commit();
    }
    if (warp == MU_A_WARPS) {
        tmem_alloc(smem_u32(&tail->tmem_slot), TM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        for (int b = 0; b < nstage; ++b) {
            mbar_init(smem_u32(&tail->full[b]), 33);     // 32 copy arrivals + the TMA byte-count arrival
            mbar_init(smem_u32(&tail->empty[b]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&tail->accum_full[b]), 1);
            mbar_init(smem_u32(&tail->accum_empty[b]), 128);
        }
        tail->abort_flag = 0;
        fence_mbar_init();
        for (int q = 0; q < P.n_problems; ++q) tma_prefetch_map(&P.p[q].map_b);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tail->tmem_slot;

    if (warp < MU_A_WARPS) {
        // ================================================================== producers
        const int sub = lane & 7, rg = lane >> 3;
        bool alive = true;
        long g0 = 0;                      // global K-step index at which the current item starts
        long gw = warp;                   // this warp's next own global K step
        int s = warp % nstage;            // its ring buffer and the parity to wait for on its empty barrier
        uint32_t ph = ((warp / nstage) & 1) ^ 1;
        int wbuf = 0;                     // wgrad: which of this warp's raw-entry buffers holds its next own step
        MuItem it = first;
        for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
            const MultiProblem& pr = P.p[it.prob];
            const int next_item = item + gridDim.x;
            MuItem nx = it;
            if (next_item < total_items) nx = mu_decode(P, next_item);
            const bool fd = it.kind != MU_WGRAD;
            const int kchunks = pr.cred / STAGE_K;
            if (fd) {
                // this tile's raw table rows have landed; the barrier also says that every producer warp is done
                // reading the previous tile's row numbers
                cp_async_wait<0>();
                named_bar_sync(1, MU_A_THREADS);
                const int tints = TILE_M * pr.kk;
                for (int d = tid; d < tints; d += MU_A_THREADS) {
                    const int k = d >> 7, r = ((d & 31) << 2) | ((d >> 5) & 3);
                    const long i = it.row0 + r;
                    const int raw = s_raw[r * pr.kk + k];
                    const long jj = (long)raw + (pr.tpb > 0 ? (i / pr.tpb) * (long)pr.tpb : 0);
                    s_xf[d] = (i < pr.n && raw >= 0 && jj < pr.n) ? (int)jj : -1;
                }
                named_bar_sync(1, MU_A_THREADS);
                // the next tile's raw rows may now overwrite s_raw
                if (next_item < total_items && nx.kind != MU_WGRAD) {
                    load_table(P.p[nx.prob], nx.row0);
                    cp_async_commit();
                }
            } else {
                if (next_item < total_items && nx.kind != MU_WGRAD) {
                    // s_raw is free (its last reader was the transform of an earlier tile, two barriers ago)
                    load_table(P.p[nx.prob], nx.row0);
                    cp_async_commit();
                }
            }
            const long g_end = g0 + it.steps;
            if (alive && warp < n_prod) {
                const int cblocks = kchunks;
                const int nblocks = pr.kk * cblocks;
                const bool second_real = it.pair * 2 + 1 < nblocks;
                const bool ones_here = pr.ones_block && !second_real;
                int tap[2] = {0, 0}, ch0[2] = {0, 0};
                if (!fd) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int blk = it.pair * 2 + h;
                        if (blk < nblocks) { tap[h] = blk / cblocks; ch0[h] = (blk % cblocks) * 64; }
                    }
                }
                for (; gw < g_end; gw += n_prod) {
                    const int st = (int)(gw - g0);
                    const uint32_t a_tile = stage_base + (uint32_t)s * STAGE_BYTES;
                    const uint32_t b_tile = a_tile + A_TILE_BYTES;
                    const uint32_t bar = smem_u32(&tail->full[s]);
                    int jrow[32];
                    if (fd) {
                        const int k = st / kchunks;
                        const int4* trow = reinterpret_cast<const int4*>(s_xf + (k << 7) + (rg << 5));
#pragma unroll
                        for (int q4 = 0; q4 < 8; ++q4) {
                            const int4 v = trow[q4];
                            jrow[4 * q4] = v.x; jrow[4 * q4 + 1] = v.y; jrow[4 * q4 + 2] = v.z; jrow[4 * q4 + 3] = v.w;
                        }
                    } else {
                        // raw entries of this step (prefetched one own step ahead) -> final gather rows, shared
                        // through shared memory so that every lane holds the rows of the 32 slots it copies
                        cp_async_wait<0>();
                        __syncwarp();
                        const int* raw = my_w + wbuf * 128;
                        int* rows = my_w + 256;
                        const long i0 = it.i_begin + (long)st * STAGE_K;
                        int v4[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int slot = lane * 4 + j;
                            const int h = slot >> 6, t = slot & 63;
                            const long i = i0 + t;
                            int v = -1;
                            if ((h == 0 || second_real) && i < it.i_end) {
                                const int r = raw[slot];
                                const long jj = (long)r + (pr.tpb > 0 ? (i / pr.tpb) * (long)pr.tpb : 0);
                                if (r >= 0 && jj < pr.n) v = (int)jj;
                            }
                            v4[j] = v;
                        }
                        *reinterpret_cast<int4*>(rows + lane * 4) = make_int4(v4[0], v4[1], v4[2], v4[3]);
                        __syncwarp();
#pragma unroll
                        for (int itr = 0; itr < 32; ++itr) jrow[itr] = rows[itr * 4 + rg];
                        __syncwarp();
                        // this warp's next own step of this item: its entries start their trip now
                        if (gw + n_prod < g_end) {
                            load_wrows(pr, it, st + n_prod, wbuf ^ 1, false);
                            cp_async_commit();
                            wbuf ^= 1;
                        }
                    }
                    if (!mu_warp_wait(smem_u32(&tail->empty[s]), ph, s_abort, err, 61, lane)) { alive = false; break; }
                    if (fd) {
                        const int k = st / kchunks, kc = st - k * kchunks;
                        const int c0 = kc * STAGE_K;
                        const int n0 = it.n0 * BN;
                        if (lane == 0) {
                            const int wtap = it.kind == MU_DGRAD ? (pr.kk - 1 - k) : k;
                            if (it.kind == MU_FWD) {
                                mbar_expect_tx(bar, B_TILE_BYTES);
#pragma unroll
                                for (int b = 0; b < B_TILE_BYTES / 8192; ++b)
                                    tma_load_3d(b_tile + b * 8192, &pr.map_b, n0 + b * 64, c0, wtap, bar);
                            } else {
                                mbar_expect_tx(bar, BN * 128);
                                tma_load_3d(b_tile, &pr.map_b, c0, n0, wtap, bar);
                            }
                        }
                        const uint16_t* abase = pr.a + c0 + sub * 8;
#pragma unroll
                        for (int itr = 0; itr < 32; ++itr) {
                            const int j = jrow[itr];
                            const int r7 = ((itr & 1) << 2) | rg;
                            const uint32_t dst = a_tile + (itr * 4 + rg) * 128 + ((sub ^ r7) << 4);
                            cp_async16(dst, abase + (long)(j < 0 ? 0 : j) * pr.cred, j < 0 ? 0u : 16u);
                        }
                    } else {
                        const long i0 = it.i_begin + (long)st * STAGE_K;
                        const int n0 = it.n0 * BN;
                        if (lane == 0) {
                            mbar_expect_tx(bar, B_TILE_BYTES);
#pragma unroll
                            for (int b = 0; b < B_TILE_BYTES / 8192; ++b)
                                tma_load_2d(b_tile + b * 8192, &pr.map_b, n0 + b * 64, (int)i0, bar);
                        }
                        if (!second_real) {
                            // the pair's missing second block: all ones (its rows of D become sum_i gy[i,:], the bias
                            // gradient) or zeros; written by plain stores, made visible to the tensor core's reads
                            const uint32_t word = ones_here ? (fp16 ? 0x3C003C00u : 0x3F803F80u) : 0u;
#pragma unroll
                            for (int c = 0; c < 16; ++c)
                                asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};"
                                             ::"r"(a_tile + 8192 + (c * 32 + lane) * 16), "r"(word) : "memory");
                            fence_proxy_async();
                        }
                        const int rows_n = second_real ? 32 : 16;
#pragma unroll
                        for (int itr = 0; itr < 32; ++itr) {
                            if (itr < rows_n) {
                                const int r = itr * 4 + rg;
                                const int j = jrow[itr];
                                const int r7 = ((itr & 1) << 2) | rg;
                                const uint32_t dst = a_tile + r * 128 + ((sub ^ r7) << 4);
                                const uint16_t* src = pr.a + (long)(j < 0 ? 0 : j) * pr.cred + ch0[itr >> 4] + sub * 8;
                                cp_async16(dst, src, j < 0 ? 0u : 16u);
                            }
                        }
                    }
                    cp_async_arrive_noinc(bar);
                    s += n_prod;
                    while (s >= nstage) { s -= nstage; ph ^= 1u; }
                }
                // this warp's first own step of the next item, if that is a wgrad item: entries on their way
                if (alive && next_item < total_items && nx.kind == MU_WGRAD && gw < g_end + nx.steps) {
                    load_wrows(P.p[nx.prob], nx, (int)(gw - g_end), wbuf, true);
                    cp_async_commit();
                }
            }
            g0 = g_end;
            it = nx;
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
    } else if (warp == MU_A_WARPS) {
        // ================================================================== MMA issuer
        // the whole warp walks the loop and waits; one elected lane (the same every time) issues and commits
        {
            constexpr uint32_t desc_hi = smem_desc_hi(1024);
            bool alive = true;
            int local = 0, s = 0;
            uint32_t ph = 0;
            for (int item = blockIdx.x; item < total_items && alive; item += gridDim.x, ++local) {
                const MuItem it = mu_decode(P, item);
                const int buf = local & 1;
                if (!mbar_wait(smem_u32(&tail->accum_empty[buf]), ((local >> 1) & 1) ^ 1, s_abort, err, 62)) { alive = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                uint32_t idesc, a_or, b_or, a_inc, b_inc;
                if (it.kind == MU_FWD) {
                    idesc = make_idesc(fp16 ? 0 : 1, 0, 1, TILE_M, BN);
                    a_or = 0; b_or = smem_desc_lbo_bits(8192); a_inc = 2; b_inc = 128;
                } else if (it.kind == MU_DGRAD) {
                    idesc = make_idesc(fp16 ? 0 : 1, 0, 0, TILE_M, BN);
                    a_or = 0; b_or = 0; a_inc = 2; b_inc = 2;
                } else {
                    idesc = make_idesc(fp16 ? 0 : 1, 1, 1, TILE_M, BN);
                    a_or = smem_desc_lbo_bits(8192); b_or = smem_desc_lbo_bits(8192); a_inc = 128; b_inc = 128;
                }
                for (int st = 0; st < it.steps; ++st) {
                    if (!mbar_wait(smem_u32(&tail->full[s]), ph, s_abort, err, 63)) { alive = false; break; }
                    fence_proxy_async();   // cp.async (generic proxy) writes -> tcgen05.mma (async proxy) reads
                    tc_fence_after();
                    const uint32_t a_tile = stage_base + (uint32_t)s * STAGE_BYTES;
                    if (elect_one_sync()) {
                        const uint32_t a_lo = ((a_tile & 0x3FFFFu) >> 4) | a_or;
                        const uint32_t b_lo = (((a_tile + A_TILE_BYTES) & 0x3FFFFu) >> 4) | b_or;
                        umma_f16_lh(d_tmem, a_lo, desc_hi, b_lo, desc_hi, idesc, st != 0 ? 1u : 0u);
#pragma unroll
                        for (int ks = 1; ks < STAGE_K / 16; ++ks)
                            umma_f16_lh_acc(d_tmem, a_lo + ks * a_inc, desc_hi, b_lo + ks * b_inc, desc_hi, idesc);
                        umma_commit(smem_u32(&tail->empty[s]));
                    }
                    __syncwarp();
                    if (++s == nstage) { s = 0; ph ^= 1u; }
                }
                if (!alive) break;
                if (elect_one_sync()) umma_commit(smem_u32(&tail->accum_full[buf]));
                __syncwarp();
            }
        }
    } else {
        // ================================================================== epilogue (warps 5..8)
        const int q = warp & 3;
        const int et = tid - (MU_A_WARPS + 1) * 32;
        int local = 0;
        for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++local) {
            const MuItem it = mu_decode(P, item);
            const MultiProblem& pr = P.p[it.prob];
            const int buf = local & 1;
            const int n0 = it.n0 * BN;
            float* sb = s_bias + buf * 256;
            if (it.kind != MU_WGRAD) {
                for (int t = et; t < BN; t += 128)
                    sb[t] = (it.kind == MU_FWD && pr.bias != nullptr) ? widen(__ldg(pr.bias + n0 + t), fp16) : 0.f;
            }
            named_bar_sync(2, 128);
            if (!mu_warp_wait(smem_u32(&tail->accum_full[buf]), (local >> 1) & 1, s_abort, err, 64, lane)) break;
            tc_fence_after();
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
            uint32_t va[32], vb[32];
            if (it.kind != MU_WGRAD) {
                const long row = it.row0 + q * 32 + lane;
                uint16_t* orow = pr.out + row * pr.cn + n0;
                tmem_ld32(t_addr, va);
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    uint32_t (&v)[32] = (c & 1) ? vb : va;
                    tmem_ld_wait();
                    if (c + 1 < NC) tmem_ld32(t_addr + (c + 1) * 32, (c & 1) ? va : vb);
                    if (row < pr.n) store_row_chunk32(orow + c * 32, v, sb + c * 32, fp16, pr.out_al32 != 0);
                }
            } else {
                const int cblocks = pr.cred / 64;
                const int nblocks = pr.kk * cblocks;
                const int blk = it.pair * 2 + (q >> 1);
                const bool ones_here = pr.ones_block && !(it.pair * 2 + 1 < nblocks);
                float* dstrow = nullptr;
                if (blk < nblocks) {
                    const long grow = (long)(blk / cblocks) * pr.cred + (blk % cblocks) * 64 + (q & 1) * 32 + lane;
                    dstrow = pr.ws_w + ((long)it.split * pr.kk * pr.cred + grow) * pr.cn + n0;
                } else if (ones_here && q == 2 && lane == 0 && pr.ws_b != nullptr) {
                    dstrow = pr.ws_b + (long)it.split * pr.cn + n0;
                }
                tmem_ld32(t_addr, va);
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    uint32_t (&v)[32] = (c & 1) ? vb : va;
                    tmem_ld_wait();
                    if (c + 1 < NC) tmem_ld32(t_addr + (c + 1) * 32, (c & 1) ? va : vb);
                    if (dstrow != nullptr) {
                        float* dst = dstrow + c * 32;
#pragma unroll
                        for (int g = 0; g < 4; ++g) st_global_v8(dst + g * 8, &v[g * 8]);
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(smem_u32(&tail->accum_empty[buf]));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == MU_A_WARPS) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, TM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------
static int multi_bn_for(int width) {
    const int cand[4] = {256, 192, 128, 64};
    for (int c : cand)
        if (width % c == 0) return c;
    return 0;
}

// The backward of one layer as one launch: input-gradient tiles and weight-gradient items in one work list.
// Returns SVTAD_ERR_UNSUPPORTED (without touching the error text's meaning for the caller's fallback) when the
// shapes do not fit this kernel; the caller then uses the single-purpose kernels.
bool multi_bwd_supported(int64_t n, int cin, int cout, int kk) {
    if (cin % 64 != 0 || cout % 64 != 0 || n <= 0) return false;
    const int bn = multi_bn_for(cin);
    if (bn == 0 || bn != multi_bn_for(cout) || cout > 256 * 64) return false;
    const char* e = getenv("SVTAD_TC_FUSED_BWD");
    if (e != nullptr && e[0] == '0') return false;
    // more row tiles than SMs: the CTA-pair kernels are the faster input gradient
    const long m_tiles = (n + TILE_M - 1) / TILE_M;
    if (m_tiles > (long)tc_num_sms() && !(e != nullptr && e[0] == '1')) return false;
    const size_t stage = A_TILE_BYTES + b_tile_bytes_for(bn);
    const size_t extra = sizeof(TmaTail) + 2 * (size_t)TILE_M * kk * sizeof(int) + 512 * sizeof(float) +
                         (size_t)MU_A_WARPS * 384 * sizeof(int);
    return (TC_SMEM_LIMIT - 1024 - extra) / stage >= 3;
}

template <int BN>
static int launch_multi(MultiParams& P, cudaStream_t s) {
    const size_t stage = A_TILE_BYTES + b_tile_bytes_for(BN);
    const size_t extra = sizeof(TmaTail) + 2 * (size_t)TILE_M * P.kk_max * sizeof(int) + 512 * sizeof(float) +
                         (size_t)MU_A_WARPS * 384 * sizeof(int);
    int nstage = (int)((TC_SMEM_LIMIT - 1024 - extra) / stage);
    if (nstage > 8) nstage = 8;
    if (nstage < 3)
        return set_error(SVTAD_ERR_UNSUPPORTED, "tensor-core work-list kernel: not enough shared memory for BN=%d kk=%d", BN, P.kk_max);
    P.nstage = nstage;
    const size_t smem = 1024 + nstage * stage + extra;
    auto kern = conv_multi_kernel<BN>;
    { int rc_s = tc_ensure_smem(reinterpret_cast<const void*>(kern), smem); if (rc_s) return rc_s; }
    const int sms = tc_num_sms();
    const int grid = P.total_items < sms ? P.total_items : sms;
    SV_CUDA(tc_launch(kern, dim3(grid), dim3(MU_THREADS), smem, s, P));
    return SVTAD_OK;
}

// weight-gradient split of the one-launch backward: the items of both kinds together fill whole rounds of the SMs
WgradPlan multi_bwd_plan(int64_t n, int cin, int cout, int kk) {
    const int bn = multi_bn_for(cin);
    const long m_tiles = (n + TILE_M - 1) / TILE_M;
    return tc_wgrad_plan_with(n, cin, cout, kk, bn, m_tiles * (cin / bn), kk * (cout / STAGE_K));
}

bool tc_bwd_fused_supported(int64_t n, int cin, int cout, int kk, int dtype) {
    return (dtype == SVTAD_BF16 || dtype == SVTAD_F16) && kk <= 49 && multi_bwd_supported(n, cin, cout, kk);
}

int tc_bwd_fused(const void* gy, const void* x, const int32_t* nbr, const void* w, void* gx, void* gw, void* gb, int64_t n,
                 int cin, int cout, int kk, int tpb, int dtype, void* ws, size_t ws_bytes, cudaStream_t s) {
    const int fp16 = dtype == SVTAD_F16 ? 1 : 0;
    const int bn = multi_bn_for(cin);
    const long m_tiles = (n + TILE_M - 1) / TILE_M;
    WgradPlan pl = multi_bwd_plan(n, cin, cout, kk);
    const long n_w = (long)kk * cin * cout;
    const int sb = pl.ones_block ? pl.splits : bias_splits_for(n);
    const size_t need = align_up((size_t)pl.splits * n_w * sizeof(float), 256) + align_up((size_t)sb * cout * sizeof(float), 256);
    if (ws_bytes < need)
        return set_error(SVTAD_ERR_WORKSPACE, "svtad_conv_bwd: workspace %zu < %zu bytes", ws_bytes, need);
    float* ws_w = static_cast<float*>(ws);
    float* ws_b = reinterpret_cast<float*>(static_cast<char*>(ws) + align_up((size_t)pl.splits * n_w * sizeof(float), 256));
    const bool bias_in_kernel = gb != nullptr && pl.ones_block;

    MultiParams P;
    memset(&P, 0, sizeof(P));
    P.n_problems = 2;
    P.fp16 = fp16;
    P.kk_max = kk;
    P.err = tc_error_ptr();
    // problem 0: weight gradient (its items come first: they are the ones the reduction kernel waits for)
    {
        MultiProblem& q = P.p[0];
        uint64_t dims[2] = {(uint64_t)cout, (uint64_t)n};
        uint32_t box[2] = {64, 64};
        int rc = tc_make_map(&q.map_b, 2, gy, dims, box, fp16);
        if (rc) return rc;
        q.kind = MU_WGRAD;
        q.a = static_cast<const uint16_t*>(x);
        q.nbr = nbr;
        q.ws_w = ws_w;
        q.ws_b = bias_in_kernel ? ws_b : nullptr;
        q.n = n;
        q.tokens_per_split = pl.tokens_per_split;
        q.cred = cin; q.cn = cout; q.kk = kk; q.tpb = tpb;
        q.n_blks = cout / bn;
        q.n_units = pl.n_pairs;
        q.splits = pl.splits;
        q.ones_block = pl.ones_block;
        q.first_item = 0;
        q.n_items = pl.n_pairs * q.n_blks * pl.splits;
    }
    // problem 1: input gradient (gather form)
    {
        MultiProblem& q = P.p[1];
        uint64_t dims[3] = {(uint64_t)cout, (uint64_t)cin, (uint64_t)kk};
        uint32_t box[3] = {64, (uint32_t)bn, 1};
        int rc = tc_make_map(&q.map_b, 3, w, dims, box, fp16);
        if (rc) return rc;
        q.kind = MU_DGRAD;
        q.a = static_cast<const uint16_t*>(gy);
        q.nbr = nbr;
        q.out = static_cast<uint16_t*>(gx);
        q.n = n;
        q.cred = cout; q.cn = cin; q.kk = kk; q.tpb = tpb;
        q.n_blks = cin / bn;
        q.n_units = (int)m_tiles;
        q.first_item = P.p[0].n_items;
        q.n_items = (int)m_tiles * q.n_blks;
        q.out_al32 = (reinterpret_cast<uintptr_t>(gx) % 32 == 0) ? 1 : 0;
    }
    P.total_items = P.p[0].n_items + P.p[1].n_items;
    if (const char* only = getenv("SVTAD_X_MULTI_ONLY")) {       // timing experiment: one kind of item only
        if (only[0] == 'w') { P.n_problems = 1; P.total_items = P.p[0].n_items; }
        if (only[0] == 'd') { P.p[0] = P.p[1]; P.p[0].first_item = 0; P.n_problems = 1; P.total_items = P.p[0].n_items; }
    }
    int rc;
    switch (bn) {
        case 64: rc = launch_multi<64>(P, s); break;
        case 128: rc = launch_multi<128>(P, s); break;
        case 192: rc = launch_multi<192>(P, s); break;
        case 256: rc = launch_multi<256>(P, s); break;
        default: return set_error(SVTAD_ERR_UNSUPPORTED, "tensor-core work-list kernel: no column block for width %d", cin);
    }
    if (rc) return rc;
    int splits_b = 0;
    if (gb != nullptr) {
        if (bias_in_kernel) {
            splits_b = pl.splits;
        } else {
            splits_b = bias_splits_for(n);
            rc = bias_partial_launch(gy, ws_b, n, cout, dtype, splits_b, s);
            if (rc) return rc;
        }
    }
    return tc_wgrad_reduce_launch(ws_w, pl.splits, ws_b, splits_b, gw, gb, n_w, cout, fp16, s);
}

}  // namespace svtad
