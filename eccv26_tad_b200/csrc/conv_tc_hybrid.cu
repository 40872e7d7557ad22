// Default tcgen05 / TMEM SparseConv2D kernels for 16-bit tensors (bf16 / fp16 in, fp32 accumulate).
//
//   forward   D[128 rows, BN] += A(K-major: gathered x rows, 64 channels per stage) . B(MN-major: W[k])
//   dgrad     same kernel, A = gathered gy rows through the table, B = W[KK-1-k] read K-major (i.e.
//             transposed) - the gather form of the input gradient, valid for symmetric tables
//   wgrad     D[128 = two 64-channel blocks of (tap, ci), BN] += A(MN-major: gathered x rows, 64 tokens
//             per stage) . B(MN-major: gy rows); split over tokens, fp32 partials to the workspace;
//             an all-ones spare block turns the bias gradient into one more row of D
//
// Operand feed.  Gathered rows are irregular, so four producer warps copy them with 16-byte cp.async
// straight into the 128-byte-swizzled layout the UMMA descriptors describe (nothing gathered is ever
// materialised in HBM); each warp owns every fourth pipeline stage, so a stage costs 32 barrier
// arrivals instead of one per thread.  Regular tiles (weights, gy) come through TMA, issued by lane 0
// of the warp that owns the stage.  One elected thread issues tcgen05.mma; four warps drain the
// accumulator (tcgen05.ld -> +bias -> one rounding -> 16-byte stores).
//
// Forward / dgrad CTAs are persistent over (row tile, column block) work items with two accumulators in
// tensor memory, so a tile's epilogue overlaps the next tile's main loop; the tile's table rows are
// prefetched into shared memory one tile ahead (with an L2 prefetch of the rows it will gather) and rewritten
// there as final row numbers in the order the producer lanes read them.  Where at least three rounds fit in
// shared memory, two 64-deep buffers share one full / empty barrier pair, so the issuing thread's per-round
// work is spent once per eight MMAs.  At most min(producer warps, buffers) warps produce: a warp waits for the
// consumer only on its own steps, and with more warps than buffers it could lap the consumer by two rounds,
// which the barrier's phase parity cannot tell from "free".  No TMA load uses cluster multicast.  Every
// mbarrier wait is bounded: when it runs out the CTA records a code in the device error word, stops, frees its
// tensor memory and returns.  Inputs whose row tiles outnumber the SMs go to the CTA-pair kernels instead
// (conv_tc_pair.cu).
#include <cstdlib>

#include "tc_common.cuh"

namespace svtad {

constexpr int HY_THREADS = 288;    // warps 0-3 producers, warp 4 MMA + TMEM owner, warps 5-8 epilogue
constexpr int A_WARPS = 4;
constexpr int A_THREADS = A_WARPS * 32;
// forward / dgrad: producer warps, then the MMA warp, then four epilogue warps
#ifndef SV_FW_A_WARPS
#define SV_FW_A_WARPS 4
#endif
constexpr int FW_A_WARPS = SV_FW_A_WARPS;
// warps that share the fill of one buffer
#ifndef SV_FW_NPW
#define SV_FW_NPW 1
#endif
constexpr int FW_NPW = SV_FW_NPW;
constexpr int FW_GROUPS = FW_A_WARPS / FW_NPW;
constexpr int FW_ITR = 32 / FW_NPW;          // 4-row copy iterations per lane and buffer
constexpr int FW_A_THREADS = FW_A_WARPS * 32;
constexpr int FW_THREADS = (FW_A_WARPS + 5) * 32;

// lane 0 waits (bounded), the whole warp learns the outcome
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* s_abort, int* err, int code,
                                          int lane) {
    int ok = 1;
    if (lane == 0) ok = mbar_wait(bar, parity, s_abort, err, code) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    __syncwarp();
    return ok != 0;
}

// ---------------------------------------------------------------------------------------------
// forward / dgrad
// ---------------------------------------------------------------------------------------------
// RB = 64-deep buffers per barrier round (1 or 2).
template <int BN, bool DGRAD, int RB>
__global__ void __launch_bounds__(FW_THREADS, 1)
conv_hybrid_kernel(const __grid_constant__ CUtensorMap map_w, const uint16_t* __restrict__ a,
                   const int32_t* __restrict__ nbr, const uint16_t* __restrict__ bias,
                   uint16_t* __restrict__ out, const int32_t* __restrict__ status, long n, int cred, int cn,
                   int kk, int tpb, int nstage, int fp16, int m_tiles, int n_blks, int out_al32, int* __restrict__ err) {
    if (DGRAD && status != nullptr && (__ldg(status) & SVTAD_TABLE_ASYMMETRIC)) return;
    constexpr int B_TILE_BYTES = b_tile_bytes_for(BN);
    constexpr int B_TX_BYTES = DGRAD ? BN * 128 : B_TILE_BYTES;
    constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
    constexpr int TM_COLS = tmem_cols2_for(BN);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    TmaTail* tail = reinterpret_cast<TmaTail*>(smem + (size_t)nstage * STAGE_BYTES);
    // [TILE_M * kk] raw table rows of the next tile (landing zone of the prefetch), then [kk][4][32] the
    // current tile's final row numbers in the order the producer lanes read them (16-byte loads)
    int* s_tab = reinterpret_cast<int*>(tail + 1);
    volatile int* s_abort = &tail->abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t stage_base = smem_u32(smem);
    const int tiles_total = m_tiles * n_blks;
    const int kchunks = cred / STAGE_K;
    const int stages_per_tile = kk * kchunks;
    // With RB = 2, two 64-deep buffers form one barrier round (a 128-deep K step): the MMA thread's per-round
    // work (wait, fences, commit) is spent once per eight instructions instead of once per four - worth it when
    // at least three rounds fit in shared memory.  A tile with an odd number of 64-deep steps gets an empty last
    // half: its owner only arrives on the barrier.
    const int sp_pad = RB == 2 ? ((stages_per_tile + 1) & ~1) : stages_per_tile;
    const int nbig = nstage / RB;             // nstage (number of 64-deep buffers) is a multiple of RB
    constexpr int RSH = RB == 2 ? 1 : 0;      // buffer -> barrier round
    const int tab_ints = TILE_M * kk;

    // raw table rows of a tile -> s_tab, by the producer threads, one tile ahead.  Behind them goes an L2 prefetch
    // of the rows the tile will gather: for tables built on a grid they lie within a few dozen rows of the tile's
    // own, so the gathers that follow the table's trip to memory do not have to make a second one.
    auto load_table = [&](int tile) {
        const long row0 = (long)(tile / n_blks) * TILE_M;
        const long rows = (n - row0) < TILE_M ? (n - row0) : TILE_M;
        const int valid_bytes = (int)rows * kk * 4;
        const char* src = reinterpret_cast<const char*>(nbr + row0 * kk);
        const uint32_t dst = smem_u32(s_tab);
        for (int c = tid; c * 16 < tab_ints * 4; c += FW_A_THREADS) {
            int left = valid_bytes - c * 16;
            uint32_t nb = left >= 16 ? 16u : (left > 0 ? (uint32_t)left : 0u);
            cp_async16(dst + c * 16, nb ? src + c * 16 : src, nb);
        }
        cp_async_commit();
        if (tid == FW_A_THREADS - 1) l2_prefetch_rows(a, row0 - 64, row0 + TILE_M + 64, n, cred);
    };
    // the first tile's rows start their trip before anything else is set up
    if (warp < FW_A_WARPS && (int)blockIdx.x < tiles_total) load_table(blockIdx.x);
    if (warp == FW_A_WARPS) {
        tmem_alloc(smem_u32(&tail->tmem_slot), TM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        for (int b = 0; b < nbig; ++b) {
            mbar_init(smem_u32(&tail->full[b]), (FW_NPW * 32 + 1) * RB);    // per buffer: the copies of the lanes that fill it + the TMA byte-count arrival
            mbar_init(smem_u32(&tail->empty[b]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&tail->accum_full[b]), 1);
            mbar_init(smem_u32(&tail->accum_empty[b]), 128);
        }
        tail->abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_map(&map_w);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tail->tmem_slot;

    if (warp < FW_A_WARPS) {
        // ------------------------------------------------------------------ producers
        const int sub = lane & 7, rg = lane >> 3;
        bool alive = true;
        // FW_NPW warps share the fill of one buffer (each a FW_ITR * 4-row slice of it); the FW_A_WARPS / FW_NPW
        // groups take turns on the K steps.  Never more groups than buffers: a group waits for the consumer only on
        // its own steps, so with more groups than buffers one of them could run two rounds ahead of the consumer,
        // where the parity of the empty barrier looks the same as "free", and refill a buffer in use.
        const int grp = warp / FW_NPW, part = warp % FW_NPW;
        const int n_own = nstage < FW_GROUPS ? nstage : FW_GROUPS;
        int local = 0;
        for (int tile = blockIdx.x; tile < tiles_total; tile += gridDim.x, ++local) {
            const long row0 = (long)(tile / n_blks) * TILE_M;
            const int n0 = (tile % n_blks) * BN;
            int* xf = s_tab + tab_ints;
            // this tile's table rows have landed (only table copies are ever committed to a group); the first
            // barrier also says that every producer warp is done reading the previous tile's row numbers
            cp_async_wait<0>();
            named_bar_sync(1, FW_A_THREADS);
            // entries become final row numbers: batch offset folded in, -1 for anything that reads as zero;
            // stored as [tap][row & 3][row >> 2], the order in which a lane group walks a stage's rows
            for (int d = tid; d < tab_ints; d += FW_A_THREADS) {
                const int k = d >> 7, r = ((d & 31) << 2) | ((d >> 5) & 3);
                long i = row0 + r;
                int raw = s_tab[r * kk + k];
                long jj = (long)raw + (tpb > 0 ? (i / tpb) * (long)tpb : 0);
                xf[d] = (i < n && raw >= 0 && jj < n) ? (int)jj : -1;
            }
            named_bar_sync(1, FW_A_THREADS);
            if (tile + (int)gridDim.x < tiles_total) load_table(tile + gridDim.x);
            if (!alive || grp >= n_own) continue;   // keep taking part in the barriers above
            const int it0 = local * sp_pad;
            // first step of this tile that this warp's group owns; then every n_own-th one.  Buffer, phase and
            // (tap, chunk) advance incrementally: no division in the loop.
            int st = ((grp - it0) % n_own + n_own) % n_own;
            int s = (it0 + st) % nstage;                         // 64-deep buffer; its barrier round is s >> RSH
            uint32_t ph = (((it0 + st) / nstage) & 1) ^ 1;
            int k = st / kchunks, kc = st - k * kchunks;
            for (; st < sp_pad; st += n_own) {
                if (!warp_wait(smem_u32(&tail->empty[s >> RSH]), ph, s_abort, err, 41, lane)) { alive = false; break; }
                const uint32_t a_tile = stage_base + (uint32_t)s * STAGE_BYTES;
                const uint32_t bar = smem_u32(&tail->full[s >> RSH]);
                const bool tma_turn = lane == 0 && part == 0;
                if (RB == 2 && st >= stages_per_tile) {
                    // the empty half of the tile's last round: same number of arrivals, nothing to copy
                    mbar_arrive(bar);
                    if (tma_turn) mbar_arrive(bar);
                } else {
                    const int c0 = kc * STAGE_K;
                    if (tma_turn) {
                        const uint32_t b_tile = a_tile + A_TILE_BYTES;
                        const int wtap = DGRAD ? (kk - 1 - k) : k;
                        mbar_expect_tx(bar, B_TX_BYTES);
                        if (!DGRAD) {
#pragma unroll
                            for (int b = 0; b < B_TILE_BYTES / 8192; ++b)
                                tma_load_3d(b_tile + b * 8192, &map_w, n0 + b * 64, c0, wtap, bar);
                        } else {
                            tma_load_3d(b_tile, &map_w, c0, n0, wtap, bar);
                        }
                    }
                    // this warp's rows are (FW_ITR * part + itr) * 4 + rg: all row numbers first (16-byte loads, the
                    // same for the 8 lanes of a row group), then the copies back to back
                    const int4* trow = reinterpret_cast<const int4*>(xf + (k << 7) + (rg << 5) + FW_ITR * part);
                    int jrow[FW_ITR];
#pragma unroll
                    for (int q4 = 0; q4 < FW_ITR / 4; ++q4) {
                        const int4 v = trow[q4];
                        jrow[4 * q4] = v.x; jrow[4 * q4 + 1] = v.y; jrow[4 * q4 + 2] = v.z; jrow[4 * q4 + 3] = v.w;
                    }
                    // A: 8 consecutive lanes cover one row's 128 B (8 chunks of 16 B)
                    const uint16_t* abase = a + c0 + sub * 8;
#pragma unroll
                    for (int itr = 0; itr < FW_ITR; ++itr) {
                        const int j = jrow[itr];
                        const int r7 = ((itr & 1) << 2) | rg;            // (row & 7) for row = (FW_ITR * part + itr) * 4 + rg
                        const uint32_t dst = a_tile + ((FW_ITR * part + itr) * 4 + rg) * 128 + ((sub ^ r7) << 4);
                        cp_async16(dst, abase + (long)(j < 0 ? 0 : j) * cred, j < 0 ? 0u : 16u);
                    }
                    cp_async_arrive_noinc(bar);
                }
                s += n_own;
                while (s >= nstage) { s -= nstage; ph ^= 1u; }
                kc += n_own;
                while (kc >= kchunks) { kc -= kchunks; if (++k == kk) k = 0; }
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
    } else if (warp == FW_A_WARPS) {
        // ------------------------------------------------------------------ MMA issuer
        // The whole warp walks the loop and waits; one elected lane (the same one every time) issues the MMAs and
        // the commits.  Measured on B200 in a loop without data movement: 422 cycles per 64-deep step at BN = 192
        // against 487 when a single diverged lane runs the loop by itself (the tensor pipe needs 384).
        {
            const uint32_t idesc = make_idesc(fp16 ? 0 : 1, 0, DGRAD ? 0 : 1, TILE_M, BN);
            constexpr uint32_t desc_hi = smem_desc_hi(1024);
            bool alive = true;
            int local = 0, s = 0;
            uint32_t ph = 0;
            for (int tile = blockIdx.x; tile < tiles_total && alive; tile += gridDim.x, ++local) {
                const int buf = local & 1;
                if (!mbar_wait(smem_u32(&tail->accum_empty[buf]), ((local >> 1) & 1) ^ 1, s_abort, err, 42)) { alive = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int st = 0; st < sp_pad; st += RB) {
                    if (!mbar_wait(smem_u32(&tail->full[s]), ph, s_abort, err, 43)) { alive = false; break; }
                    fence_proxy_async();   // cp.async (generic proxy) writes -> tcgen05.mma (async proxy) reads
                    tc_fence_after();
                    const uint32_t a_tile = stage_base + (uint32_t)(RB * s) * STAGE_BYTES;
                    const int halves = (RB == 2 && st + 1 < stages_per_tile) ? 2 : 1;
                    if (elect_one_sync()) {
                        // descriptor low words: start address >> 4 (shared memory is below 256 KB, so adding a K step's
                        // offset never carries into the LBO field above it)
                        uint32_t a_lo = (a_tile & 0x3FFFFu) >> 4;
                        for (int h = 0; h < halves; ++h) {
                            const uint32_t b_lo = (a_lo + (A_TILE_BYTES >> 4)) | (DGRAD ? 0u : smem_desc_lbo_bits(8192));
                            umma_f16_lh(d_tmem, a_lo, desc_hi, b_lo, desc_hi, idesc, (st | h) != 0 ? 1u : 0u);
#pragma unroll
                            for (int ks = 1; ks < STAGE_K / 16; ++ks)
                                umma_f16_lh_acc(d_tmem, a_lo + ks * 2, desc_hi, b_lo + ks * (DGRAD ? 2 : 128), desc_hi, idesc);
                            a_lo += STAGE_BYTES >> 4;
                        }
                        umma_commit(smem_u32(&tail->empty[s]));
                    }
                    __syncwarp();
                    if (++s == nbig) { s = 0; ph ^= 1u; }
                }
                if (!alive) break;
                if (elect_one_sync()) umma_commit(smem_u32(&tail->accum_full[buf]));
                __syncwarp();
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 5..8)
        constexpr int NC = BN / 32;
        const int q = warp & 3;
        const int et = tid - (FW_A_WARPS + 1) * 32;          // 0..127 among the epilogue threads
        float* s_bias = reinterpret_cast<float*>(s_tab + 2 * tab_ints);   // [2][256]
        int local = 0;
        for (int tile = blockIdx.x; tile < tiles_total; tile += gridDim.x, ++local) {
            const int buf = local & 1;
            const long row = (long)(tile / n_blks) * TILE_M + q * 32 + lane;
            const int n0 = (tile % n_blks) * BN;
            // the tile's bias goes to shared memory while the main loop is still running
            float* sb = s_bias + buf * 256;
            for (int t = et; t < BN; t += 128)
                sb[t] = (!DGRAD && bias != nullptr) ? widen(__ldg(bias + n0 + t), fp16 != 0) : 0.f;
            named_bar_sync(2, 128);
            if (!warp_wait(smem_u32(&tail->accum_full[buf]), (local >> 1) & 1, s_abort, err, 44, lane)) break;
            tc_fence_after();
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
            uint16_t* orow = out + row * cn + n0;
            // two 32-column chunks in flight: the next tcgen05.ld runs while this chunk is converted and stored
            uint32_t va[32], vb[32];
            tmem_ld32(t_addr, va);
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                uint32_t (&v)[32] = (c & 1) ? vb : va;
                tmem_ld_wait();
                if (c + 1 < NC) tmem_ld32(t_addr + (c + 1) * 32, (c & 1) ? va : vb);
                if (row < n) store_row_chunk32(orow + c * 32, v, sb + c * 32, fp16 != 0, out_al32 != 0);
            }
            tc_fence_before();
            mbar_arrive(smem_u32(&tail->accum_empty[buf]));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == FW_A_WARPS) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, TM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
// wgrad
// ---------------------------------------------------------------------------------------------
template <int BN>
__global__ void __launch_bounds__(HY_THREADS, 1)
wgrad_hybrid_kernel(const __grid_constant__ CUtensorMap map_gy, const uint16_t* __restrict__ x,
                    const int32_t* __restrict__ nbr, float* __restrict__ ws_w, float* __restrict__ ws_b,
                    long n, int cin, int cout, int kk, int tpb, long tokens_per_split, int n_nblk,
                    int nstage, int fp16, int ones_block, int* __restrict__ err) {
    constexpr int B_TILE_BYTES = b_tile_bytes_for(BN);
    constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
    constexpr int TM_COLS = tmem_cols_for(BN);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    TmaTail* tail = reinterpret_cast<TmaTail*>(smem + (size_t)nstage * STAGE_BYTES);
    int* s_idx = reinterpret_cast<int*>(tail + 1);                 // per producer warp: a ring of [2][128] table entries
    volatile int* s_abort = &tail->abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int pair = blockIdx.x / n_nblk;
    const int n0 = (blockIdx.x % n_nblk) * BN;
    const int cblocks = cin / 64;
    const int nblocks = kk * cblocks;
    const long i_begin = (long)blockIdx.y * tokens_per_split;
    const long i_end = n < i_begin + tokens_per_split ? n : i_begin + tokens_per_split;
    const int total_stages = i_end > i_begin ? (int)((i_end - i_begin + STAGE_K - 1) / STAGE_K) : 0;
    const uint32_t stage_base = smem_u32(smem);
    const bool second_real = pair * 2 + 1 < nblocks;
    // second block of the last pair when the block count is odd: all ones, so its rows of D are sum_i gy[i,:]
    const bool ones_here = ones_block && !second_real;

    // A producer warp owns every n_prod-th 64-token step.  The A tile of a step has 128 slots (slot = block * 64 +
    // token); each lane looks up the table entry nbr[token, tap(block)] of the four slots lane + 32 * j.  The
    // entries travel WG_PF own steps ahead of their use through a small ring in shared memory (4-byte cp.async,
    // one commit group per own step).
    constexpr int WG_PF = 2;
    int* my_ent = s_idx + warp * (WG_PF * 128);         // [WG_PF][128] raw entries of this warp's coming steps
    // CTAs of different block pairs walk the token range from different starting points; `src_stage` is the
    // 64-token step that pipeline step `it` carries
    const int rot = total_stages > 0 ? (int)(((long)blockIdx.x * 5) % total_stages) : 0;
    auto src_stage = [&](int it) { int v = it + rot; return v >= total_stages ? v - total_stages : v; };
    // never more producer warps than buffers (see the forward kernel)
    const int n_prod = nstage < A_WARPS ? nstage : A_WARPS;
    int tap[2], ch0[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int blk = pair * 2 + h;
        const bool real = blk < nblocks;
        tap[h] = real ? blk / cblocks : 0;
        ch0[h] = real ? (blk % cblocks) * 64 : 0;
    }
    // entries of own step number `own` (pipeline step warp + own * n_prod) -> ring slot own % WG_PF
    auto load_entries = [&](int own) {
        const int it = warp + own * n_prod;
        if (it < total_stages) {
            const long i0 = i_begin + (long)src_stage(it) * STAGE_K;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int slot = lane + 32 * j;
                const int h = j >> 1, t = slot & 63;
                const long i = i0 + t;
                const bool ok = (h == 0 || second_real) && i < i_end;
                const int32_t* src = nbr + (ok ? i * kk + tap[h] : 0);
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;"
                             ::"r"(smem_u32(my_ent + (own % WG_PF) * 128 + slot)), "l"(src), "r"(ok ? 4u : 0u) : "memory");
            }
        }
        cp_async_commit();     // one group per own step, empty or not: the wait below counts groups
    };
    // the first steps' entries start their trip before anything else is set up
    if (warp < n_prod) {
#pragma unroll
        for (int own = 0; own < WG_PF; ++own) load_entries(own);
        if (lane == 31 && warp < total_stages) {
            const long i0 = i_begin + (long)src_stage(warp) * STAGE_K;
            l2_prefetch_rows(x, i0 - 64, i0 + STAGE_K + 64, n, cin);
        }
    }
    if (warp == 4) {
        tmem_alloc(smem_u32(&tail->tmem_slot), TM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        for (int s = 0; s < nstage; ++s) {
            mbar_init(smem_u32(&tail->full[s]), 33);     // the owning warp's 32 copy arrivals + the TMA byte count
            mbar_init(smem_u32(&tail->empty[s]), 1);
        }
        mbar_init(smem_u32(&tail->accum_full[0]), 1);
        tail->abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_map(&map_gy);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tail->tmem_slot;

    if (warp < A_WARPS) {
        // ------------------------------------------------------------------ producers
        if (!second_real) {
            // the missing second block of every stage is written once: ones (bias row) or zeros
            const uint32_t word = ones_here ? (fp16 ? 0x3C003C00u : 0x3F803F80u) : 0u;
            for (int s = 0; s < nstage; ++s) {
                uint32_t base = stage_base + (uint32_t)s * STAGE_BYTES + 8192;
                for (int c = tid; c < 512; c += A_THREADS)
                    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(base + c * 16), "r"(word) : "memory");
            }
            fence_proxy_async();
            named_bar_sync(1, A_THREADS);
        }
        const int sub = lane & 7, rg = lane >> 3;
        int s = warp % nstage;
        uint32_t ph = ((warp / nstage) & 1) ^ 1;
        const int rows_n = second_real ? 32 : 16;            // slots 64..127 belong to the second block
        int own = 0;
        for (int it = warp; it < total_stages && warp < n_prod; it += n_prod, ++own) {
            // this own step's entries have landed (the WG_PF - 1 younger groups may still be in flight)
            cp_async_wait<WG_PF - 1>();
            const long i0 = i_begin + (long)src_stage(it) * STAGE_K;
            int v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int slot = lane + 32 * j;
                const int h = j >> 1, t = slot & 63;
                const long i = i0 + t;
                v[j] = -1;
                if ((h == 0 || second_real) && i < i_end) {
                    const int raw = my_ent[(own % WG_PF) * 128 + slot];
                    const long jj = (long)raw + (tpb > 0 ? (i / tpb) * (long)tpb : 0);
                    if (raw >= 0 && jj < n) v[j] = (int)jj;
                }
            }
            load_entries(own + WG_PF);       // the ring slot just read is free again (each lane reads only what it copied)
            // the rows this lane copies: slot itr * 4 + rg is held by lane (itr & 7) * 4 + rg in v[itr >> 3]
            int jrow[32];
#pragma unroll
            for (int itr = 0; itr < 32; ++itr) jrow[itr] = __shfl_sync(0xffffffffu, v[itr >> 3], (itr & 7) * 4 + rg);
            if (!warp_wait(smem_u32(&tail->empty[s]), ph, s_abort, err, 51, lane)) break;
            const uint32_t a_tile = stage_base + (uint32_t)s * STAGE_BYTES;
            const uint32_t bar = smem_u32(&tail->full[s]);
            if (lane == 0) {
                const uint32_t b_tile = a_tile + A_TILE_BYTES;
                mbar_expect_tx(bar, B_TILE_BYTES);
#pragma unroll
                for (int b = 0; b < B_TILE_BYTES / 8192; ++b)
                    tma_load_2d(b_tile + b * 8192, &map_gy, n0 + b * 64, (int)i0, bar);
            }
#pragma unroll
            for (int itr = 0; itr < 32; ++itr) {
                if (itr < rows_n) {
                    const int r = itr * 4 + rg;
                    const int j = jrow[itr];
                    const int r7 = ((itr & 1) << 2) | rg;
                    const uint32_t dst = a_tile + r * 128 + ((sub ^ r7) << 4);
                    const uint16_t* src = x + (long)(j < 0 ? 0 : j) * cin + ch0[itr >> 4] + sub * 8;
                    cp_async16(dst, src, j < 0 ? 0u : 16u);
                }
            }
            cp_async_arrive_noinc(bar);
            s += n_prod;
            while (s >= nstage) { s -= nstage; ph ^= 1u; }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
    } else if (warp == 4) {
        // the whole warp walks the loop and waits; one elected lane issues the MMAs and the commits
        const uint32_t idesc = make_idesc(fp16 ? 0 : 1, 1, 1, TILE_M, BN);
        bool alive = true;
        int s = 0;
        uint32_t ph = 0;
        for (int it = 0; it < total_stages; ++it) {
            if (!mbar_wait(smem_u32(&tail->full[s]), ph, s_abort, err, 52)) { alive = false; break; }
            fence_proxy_async();
            tc_fence_after();
            const uint32_t a_tile = stage_base + (uint32_t)s * STAGE_BYTES;
            if (elect_one_sync()) {
                // both operands MN-major: 16 K rows per step = 2048 B, 64-element blocks 8192 B apart
                const uint32_t a_lo = ((a_tile & 0x3FFFFu) >> 4) | smem_desc_lbo_bits(8192);
                const uint32_t b_lo = a_lo + (A_TILE_BYTES >> 4);
                umma_f16_lh(tmem_base, a_lo, smem_desc_hi(1024), b_lo, smem_desc_hi(1024), idesc, it != 0 ? 1u : 0u);
#pragma unroll
                for (int ks = 1; ks < STAGE_K / 16; ++ks)
                    umma_f16_lh_acc(tmem_base, a_lo + ks * 128, smem_desc_hi(1024), b_lo + ks * 128, smem_desc_hi(1024), idesc);
                umma_commit(smem_u32(&tail->empty[s]));
            }
            __syncwarp();
            if (++s == nstage) { s = 0; ph ^= 1u; }
        }
        if (alive && total_stages > 0 && elect_one_sync()) umma_commit(smem_u32(&tail->accum_full[0]));
        __syncwarp();
    } else {
        // epilogue: fp32 partial tile -> ws_w[split][(tap, ci)][co]; the all-ones block -> ws_b[split][co]
        bool have = true;
        if (total_stages > 0) have = mbar_wait(smem_u32(&tail->accum_full[0]), 0, s_abort, err, 53);
        tc_fence_after();
        if (have) {
            const int q = warp & 3;
            const int blk = pair * 2 + (q >> 1);
            float* dstrow = nullptr;
            if (blk < nblocks) {
                const long grow = (long)(blk / cblocks) * cin + (blk % cblocks) * 64 + (q & 1) * 32 + lane;
                dstrow = ws_w + ((long)blockIdx.y * kk * cin + grow) * cout + n0;
            } else if (ones_here && q == 2 && lane == 0 && ws_b != nullptr) {
                dstrow = ws_b + (long)blockIdx.y * cout + n0;
            }
            constexpr int NC = BN / 32;
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
            uint32_t va[32], vb[32];
            if (total_stages > 0) tmem_ld32(t_addr, va);
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                uint32_t (&v)[32] = (c & 1) ? vb : va;
                if (total_stages > 0) {
                    tmem_ld_wait();
                    if (c + 1 < NC) tmem_ld32(t_addr + (c + 1) * 32, (c & 1) ? va : vb);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0u;
                }
                if (dstrow != nullptr) {
                    // 32 bytes (one whole sector) per store: the workspace is 256-byte aligned, rows are cout * 4 bytes
                    float* dst = dstrow + c * 32;
#pragma unroll
                    for (int g = 0; g < 4; ++g) st_global_v8(dst + g * 8, &v[g * 8]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, TM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
template <int BN, bool DGRAD>
static int launch_conv_hybrid(const ConvArgs& p, const int32_t* status, cudaStream_t s) {
    const int cred = DGRAD ? p.cout : p.cin;
    const int cn = DGRAD ? p.cin : p.cout;
    const int fp16 = p.dtype == SVTAD_F16 ? 1 : 0;
    CUtensorMap map_w;
    {
        uint64_t dims[3] = {(uint64_t)p.cout, (uint64_t)p.cin, (uint64_t)p.kk};
        uint32_t box[3] = {64, (uint32_t)(DGRAD ? BN : 64), 1};
        int rc = tc_make_map(&map_w, 3, p.w, dims, box, fp16);
        if (rc) return rc;
    }
    const size_t stage = A_TILE_BYTES + b_tile_bytes_for(BN);
    const size_t extra = sizeof(TmaTail) + 2 * (size_t)TILE_M * p.kk * sizeof(int) + 2 * 256 * sizeof(float);
    int nstage = (int)((TC_SMEM_LIMIT - 1024 - extra) / stage);
    if (nstage > 16) nstage = 16;
    if (nstage < 2)
        return set_error(SVTAD_ERR_UNSUPPORTED, "tensor-core conv: not enough shared memory for BN=%d kk=%d", BN, p.kk);
    // rounds of two buffers once three rounds fit (narrow column blocks); otherwise one buffer per round
    const bool two = nstage >= 6;
    if (two) nstage &= ~1;
    const size_t smem = 1024 + nstage * stage + extra;
    auto kern = two ? conv_hybrid_kernel<BN, DGRAD, 2> : conv_hybrid_kernel<BN, DGRAD, 1>;
    { int rc_s = tc_ensure_smem(reinterpret_cast<const void*>(kern), smem); if (rc_s) return rc_s; }
    const int m_tiles = (int)((p.n + TILE_M - 1) / TILE_M);
    const int n_blks = cn / BN;
    long tiles = (long)m_tiles * n_blks;
    // persistent CTAs.  (Evening the tiles out - 135 tiles as 45 CTAs of 3 instead of 49 CTAs of 3 or 2 - was
    // measured slower inside a step of concurrent kernels: 0.0907 against 0.0858 ms.)
    const long plan = tc_plan_sms();
    int grid = (int)(tiles < plan ? tiles : plan);
    SV_CUDA(tc_launch(kern, dim3(grid), dim3(FW_THREADS), smem, s, map_w, (const uint16_t*)p.a, p.nbr,
                      (const uint16_t*)p.bias, (uint16_t*)p.out, status, (long)p.n, cred, cn, p.kk, p.tpb, nstage, fp16,
                      m_tiles, n_blks, (reinterpret_cast<uintptr_t>(p.out) % 32 == 0) ? 1 : 0, tc_error_ptr()));
    return SVTAD_OK;
}

template <bool DGRAD>
static int dispatch_conv_hybrid(const ConvArgs& p, const int32_t* status, cudaStream_t s) {
    const int cn = DGRAD ? p.cin : p.cout;
    int bn = tc_pick_bn(cn, (p.n + TILE_M - 1) / TILE_M);
    switch (bn) {
        case 64: return launch_conv_hybrid<64, DGRAD>(p, status, s);
        case 96: return launch_conv_hybrid<96, DGRAD>(p, status, s);
        case 128: return launch_conv_hybrid<128, DGRAD>(p, status, s);
        case 192: return launch_conv_hybrid<192, DGRAD>(p, status, s);
        case 256: return launch_conv_hybrid<256, DGRAD>(p, status, s);
    }
    return set_error(SVTAD_ERR_UNSUPPORTED, "tensor-core conv: no column block for width %d", cn);
}


int hybrid_fwd(const ConvArgs& p, cudaStream_t s) { return dispatch_conv_hybrid<false>(p, nullptr, s); }
int hybrid_dgrad(const ConvArgs& p, const int32_t* status, cudaStream_t s) { return dispatch_conv_hybrid<true>(p, status, s); }

template <int BN>
static int launch_wgrad_hybrid(const void* gy, const void* x, const int32_t* nbr, float* ws_w, float* ws_b, int64_t n, int cin, int cout, int kk, int tpb, int fp16,
                               const WgradPlan& pl, cudaStream_t s) {
    CUtensorMap map_gy;
    {
        uint64_t dims[2] = {(uint64_t)cout, (uint64_t)n};
        uint32_t box[2] = {64, 64};
        int rc = tc_make_map(&map_gy, 2, gy, dims, box, fp16);
        if (rc) return rc;
    }
    const size_t stage = A_TILE_BYTES + b_tile_bytes_for(BN);
    const size_t extra = sizeof(TmaTail) + (size_t)A_WARPS * 2 * 128 * sizeof(int);
    int nstage = (int)((TC_SMEM_LIMIT - 1024 - extra) / stage);
    if (nstage > 8) nstage = 8;
    if (nstage < 2)
        return set_error(SVTAD_ERR_UNSUPPORTED, "tensor-core wgrad: not enough shared memory for BN=%d kk=%d", BN, kk);
    const size_t smem = 1024 + nstage * stage + extra;
    dim3 grid((unsigned)(pl.n_pairs * pl.n_nblk), (unsigned)pl.splits);
    auto kern = wgrad_hybrid_kernel<BN>;
    { int rc_s = tc_ensure_smem(reinterpret_cast<const void*>(kern), smem); if (rc_s) return rc_s; }
    SV_CUDA(tc_launch(kern, grid, dim3(HY_THREADS), smem, s, map_gy, (const uint16_t*)x, nbr, ws_w, ws_b, (long)n, cin, cout, kk, tpb, pl.tokens_per_split,
                      pl.n_nblk, nstage, fp16, pl.ones_block, tc_error_ptr()));
    return SVTAD_OK;
}

int hybrid_wgrad(const void* gy, const void* x, const int32_t* nbr, void* gw, void* gb, int64_t n, int cin, int cout,
                 int kk, int tpb, int dtype, void* ws, size_t ws_bytes, cudaStream_t s) {
    size_t need = tc_wgrad_plan_ws_bytes(n, cin, cout, kk);
    if (ws_bytes < need)
        return set_error(SVTAD_ERR_WORKSPACE, "svtad_conv_wgrad: workspace %zu < %zu bytes", ws_bytes, need);
    WgradPlan pl = tc_wgrad_plan(n, cin, cout, kk);
    const int fp16 = dtype == SVTAD_F16 ? 1 : 0;
    const long n_w = (long)kk * cin * cout;
    float* ws_w = static_cast<float*>(ws);
    float* ws_b = reinterpret_cast<float*>(static_cast<char*>(ws) + align_up((size_t)pl.splits * n_w * sizeof(float), 256));
    const bool bias_in_kernel = gb != nullptr && pl.ones_block;
    float* kb = bias_in_kernel ? ws_b : nullptr;
    int rc;
    switch (pl.bn) {
        case 64: rc = launch_wgrad_hybrid<64>(gy, x, nbr, ws_w, kb, n, cin, cout, kk, tpb, fp16, pl, s); break;
        case 128: rc = launch_wgrad_hybrid<128>(gy, x, nbr, ws_w, kb, n, cin, cout, kk, tpb, fp16, pl, s); break;
        case 192: rc = launch_wgrad_hybrid<192>(gy, x, nbr, ws_w, kb, n, cin, cout, kk, tpb, fp16, pl, s); break;
        case 256: rc = launch_wgrad_hybrid<256>(gy, x, nbr, ws_w, kb, n, cin, cout, kk, tpb, fp16, pl, s); break;
        default: return set_error(SVTAD_ERR_UNSUPPORTED, "tensor-core wgrad: no column block for width %d", cout);
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
