// Forward / dgrad of SparseConv2D on CTA pairs: tcgen05.mma.cta_group::2, M = 256 per instruction.
//
// Two CTAs of a thread-block cluster (two SMs) work on two neighbouring 128-row tiles.  Each CTA gathers its
// own rows (A operand, as in the one-CTA kernels) but stages only HALF of the weight tile: the instruction
// reads columns [0, BN/2) of B from the even CTA's shared memory and [BN/2, BN) from the odd CTA's, and writes
// each CTA's 128 rows of D into that CTA's tensor memory.  Per CTA and K step the shared-memory traffic of the
// weight tile is halved (12 KB written + 12 KB read instead of 24 + 24 at BN = 192), which is what bounds the
// one-CTA kernels, and a problem of m row tiles needs m CTAs whatever BN is.
//
// Roles per CTA (288 threads): warps 0-3 producers (cp.async gathers + lane 0's TMA of the B half, arriving on
// the CTA's own full barrier), warp 4: in the even CTA the MMA issuer, in the odd CTA a relay that forwards
// "my stage is full" to the even CTA's barrier; warps 5-8 epilogue of the CTA's own accumulator.
// The even CTA's MMA thread commits to the empty / accumulator barriers of both CTAs.  No TMA load uses
// cluster multicast.  Every wait is bounded (device error word), and both CTAs meet at a cluster barrier before
// tensor memory is freed, so neither leaves while the other may still read its shared memory.
//
// Layouts: A K-major, 128-byte swizzle (gathered rows of 64 channels).  dgrad B: K-major, 128-byte swizzle,
// BN/2 rows.  forward B: MN-major; BN/2 columns are not a whole number of 64-column swizzle atoms at BN = 192,
// so the forward uses the 64-byte swizzle (32-column atoms of 64 rows x 64 B = 4 KB).
#include <cstdlib>

#include "tc_common.cuh"

namespace svtad {

constexpr int PR_THREADS = 288;
constexpr int PR_A_WARPS = 4;
constexpr int PR_A_THREADS = PR_A_WARPS * 32;

__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait on a barrier that a thread of the other CTA arrives on
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* s_abort, int* err, int code) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if ((spin & 31u) == 0u) {
            if (*s_abort) return false;
            if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                *s_abort = 1;
                atomicCAS(err, 0, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// tcgen05.mma over the CTA pair; descriptors as (low word, high word)
__device__ __forceinline__ void umma_pair_f16_lh(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                                 uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
}
// arrival on a barrier of either CTA (cluster address) once every MMA issued so far by this thread has finished
__device__ __forceinline__ void umma_pair_commit(uint32_t cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
}
// lane 0 waits (bounded), the whole warp learns the outcome
__device__ __forceinline__ bool warp_wait_pair(uint32_t bar, uint32_t parity, volatile int* s_abort, int* err, int code,
                                               int lane) {
    int ok = 1;
    if (lane == 0) ok = mbar_wait(bar, parity, s_abort, err, code) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    __syncwarp();
    return ok != 0;
}

struct alignas(16) PairTail {   // barriers are per round of two 64-deep buffers
    uint64_t full[8];          // per half 32 copy arrivals + TMA; the even CTA's also counts the odd CTA's relay
    uint64_t empty[8];         // one arrival: the even CTA's tcgen05.commit
    uint64_t accum_full[2];    // one arrival: the even CTA's tcgen05.commit
    uint64_t accum_empty[2];   // even CTA only: one arrival per epilogue warp of both CTAs
    uint32_t tmem_slot;
    int abort_flag;
};

template <int BN, bool DGRAD>
__global__ void __launch_bounds__(PR_THREADS, 1)
conv_pair_kernel(const __grid_constant__ CUtensorMap map_w, const uint16_t* __restrict__ a,
                 const int32_t* __restrict__ nbr, const uint16_t* __restrict__ bias,
                 uint16_t* __restrict__ out, const int32_t* __restrict__ status, long n, int cred, int cn,
                 int kk, int tpb, int nstage, int fp16, int m_pairs, int n_blks, int out_al32, int* __restrict__ err) {
    // uniform over the whole grid, so both CTAs of a pair leave together
    if (DGRAD && status != nullptr && (__ldg(status) & SVTAD_TABLE_ASYMMETRIC)) return;
    constexpr int HALF = BN / 2;                  // columns of B this CTA stages
    constexpr int B_BYTES = HALF * 128;           // 64 K x HALF columns x 2 bytes, either layout
    constexpr int STAGE_BYTES = A_TILE_BYTES + B_BYTES;
    constexpr int TM_COLS = tmem_cols2_for(BN);
    constexpr int NC = BN / 32;

    extern __shared__ uint8_t smem_raw[];
    // same offset in both CTAs: the dynamic segment starts at the same shared-memory address in every CTA
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    PairTail* tail = reinterpret_cast<PairTail*>(smem + (size_t)nstage * STAGE_BYTES);
    int* s_tab = reinterpret_cast<int*>(tail + 1);        // [TILE_M * kk] raw rows of the next tile, then [kk][4][32] row numbers
    volatile int* s_abort = &tail->abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_cta_rank();             // 0 = even CTA (issues the MMAs), 1 = odd CTA
    const int cid = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    const uint32_t stage_base = smem_u32(smem);
    const int items_total = m_pairs * n_blks;
    const int kchunks = cred / STAGE_K;
    const int stages_per_tile = kk * kchunks;
    // Two 64-deep buffers form one barrier round (a 128-deep K step): the MMA thread's per-round work (wait,
    // fences, commits) is spent once per eight instructions instead of once per four.  A tile with an odd
    // number of 64-deep steps gets an empty last half: its owner only arrives on the barrier.
    const int sp_pad = (stages_per_tile + 1) & ~1;
    const int nbig = nstage >> 1;             // nstage (number of 64-deep buffers) is even
    // never more producer warps than buffers: a warp that is not held back by its own previous use of a buffer
    // could run two rounds ahead of the consumer, where the empty barrier's parity reads as "free"
    const int n_prod = nstage < PR_A_WARPS ? nstage : PR_A_WARPS;
    const int tab_ints = TILE_M * kk;
    float* s_bias = reinterpret_cast<float*>(s_tab + 2 * tab_ints);   // [2][256]

    auto load_table = [&](int item) {
        const long row0 = ((long)(item / n_blks) * 2 + rank) * TILE_M;
        long rows = n - row0;
        rows = rows < 0 ? 0 : (rows < TILE_M ? rows : TILE_M);
        const int valid_bytes = (int)rows * kk * 4;
        const char* src = reinterpret_cast<const char*>(nbr + (rows > 0 ? row0 : 0) * kk);
        const uint32_t dst = smem_u32(s_tab);
        for (int c = tid; c * 16 < tab_ints * 4; c += PR_A_THREADS) {
            int left = valid_bytes - c * 16;
            uint32_t nb = left >= 16 ? 16u : (left > 0 ? (uint32_t)left : 0u);
            cp_async16(dst + c * 16, nb ? src + c * 16 : src, nb);
        }
        cp_async_commit();
        // L2 prefetch of the rows this tile will gather (see the one-CTA kernel)
        if (tid == PR_A_THREADS - 1) l2_prefetch_rows(a, row0 - 64, row0 + TILE_M + 64, n, cred);
    };
    // the first tile's rows start their trip before anything else is set up
    if (warp < PR_A_WARPS && cid < items_total) load_table(cid);
    if (warp == 4) {
        tmem_alloc_pair(smem_u32(&tail->tmem_slot), TM_COLS);
        tmem_relinquish_pair();
    }
    if (tid == 0) {
        for (int b = 0; b < nbig; ++b) {
            mbar_init(smem_u32(&tail->full[b]), rank == 0 ? 67 : 66);   // two halves x (32 copies + TMA), + the relay
            mbar_init(smem_u32(&tail->empty[b]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&tail->accum_full[b]), 1);
            mbar_init(smem_u32(&tail->accum_empty[b]), 8);
        }
        tail->abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_map(&map_w);
    }
    tc_fence_before();
    __syncthreads();
    cluster_barrier();          // both CTAs' barriers exist before anyone arrives on the other's
    tc_fence_after();
    const uint32_t tmem_base = tail->tmem_slot;

    if (warp < PR_A_WARPS) {
        // ------------------------------------------------------------------ producers (both CTAs)
        const int sub = lane & 7, rg = lane >> 3;
        bool alive = true;
        int local = 0;
        for (int item = cid; item < items_total; item += n_clusters, ++local) {
            const long row0 = ((long)(item / n_blks) * 2 + rank) * TILE_M;
            const int n0 = (item % n_blks) * BN + (int)rank * HALF;      // first column of this CTA's half of B
            int* xf = s_tab + tab_ints;
            cp_async_wait<0>();
            named_bar_sync(1, PR_A_THREADS);
            for (int d = tid; d < tab_ints; d += PR_A_THREADS) {
                const int k = d >> 7, r = ((d & 31) << 2) | ((d >> 5) & 3);
                long i = row0 + r;
                int raw = s_tab[r * kk + k];
                long jj = (long)raw + (tpb > 0 ? (i / tpb) * (long)tpb : 0);
                xf[d] = (i < n && raw >= 0 && jj < n) ? (int)jj : -1;
            }
            named_bar_sync(1, PR_A_THREADS);
            if (item + n_clusters < items_total) load_table(item + n_clusters);
            if (!alive || warp >= n_prod) continue;
            const int it0 = local * sp_pad;
            int st = ((warp - it0) % n_prod + n_prod) % n_prod;
            int s = (it0 + st) % nstage;                         // 64-deep buffer; its barrier round is s >> 1
            uint32_t ph = (((it0 + st) / nstage) & 1) ^ 1;
            int k = st / kchunks, kc = st - k * kchunks;
            for (; st < sp_pad; st += n_prod) {
                if (!warp_wait_pair(smem_u32(&tail->empty[s >> 1]), ph, s_abort, err, 51, lane)) { alive = false; break; }
                const uint32_t a_tile = stage_base + (uint32_t)s * STAGE_BYTES;
                const uint32_t bar = smem_u32(&tail->full[s >> 1]);
                if (st >= stages_per_tile) {
                    // the empty half of the tile's last round: same number of arrivals, nothing to copy
                    mbar_arrive(bar);
                    if (lane == 0) mbar_arrive(bar);
                } else {
                    const int c0 = kc * STAGE_K;
                    if (lane == 0) {
                        const uint32_t b_tile = a_tile + A_TILE_BYTES;
                        const int wtap = DGRAD ? (kk - 1 - k) : k;
                        mbar_expect_tx(bar, B_BYTES);
                        if (!DGRAD) {
#pragma unroll
                            for (int b = 0; b < HALF / 32; ++b)
                                tma_load_3d(b_tile + b * 4096, &map_w, n0 + b * 32, c0, wtap, bar);
                        } else {
                            tma_load_3d(b_tile, &map_w, c0, n0, wtap, bar);
                        }
                    }
                    const uint16_t* abase = a + c0 + sub * 8;
                    const int4* trow = reinterpret_cast<const int4*>(xf + (k << 7) + (rg << 5));
                    int jrow[32];
#pragma unroll
                    for (int q4 = 0; q4 < 8; ++q4) {
                        const int4 v = trow[q4];
                        jrow[4 * q4] = v.x; jrow[4 * q4 + 1] = v.y; jrow[4 * q4 + 2] = v.z; jrow[4 * q4 + 3] = v.w;
                    }
#pragma unroll
                    for (int itr = 0; itr < 32; ++itr) {
                        const int j = jrow[itr];
                        const int r7 = ((itr & 1) << 2) | rg;
                        const uint32_t dst = a_tile + (itr * 4 + rg) * 128 + ((sub ^ r7) << 4);
                        cp_async16(dst, abase + (long)(j < 0 ? 0 : j) * cred, j < 0 ? 0u : 16u);
                    }
                    cp_async_arrive_noinc(bar);
                }
                s += n_prod;
                while (s >= nstage) { s -= nstage; ph ^= 1u; }
                kc += n_prod;
                while (kc >= kchunks) { kc -= kchunks; if (++k == kk) k = 0; }
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
    } else if (warp == 4) {
        if (rank == 0) {
            // ------------------------------------------------------------------ MMA issuer (even CTA)
            // the whole warp walks the loop and waits; one elected lane (the same every time) issues and commits
            const uint32_t idesc = make_idesc(fp16 ? 0 : 1, 0, DGRAD ? 0 : 1, 2 * TILE_M, BN);
            bool alive = true;
            int local = 0, s = 0;
            uint32_t ph = 0;
            // distance from one of this CTA's shared-memory addresses to the same location in the odd CTA
            const uint32_t to_peer = map_to_cta(stage_base, 1) - stage_base;
            for (int item = cid; item < items_total && alive; item += n_clusters, ++local) {
                const int buf = local & 1;
                if (!mbar_wait(smem_u32(&tail->accum_empty[buf]), ((local >> 1) & 1) ^ 1, s_abort, err, 52)) { alive = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int st = 0; st < sp_pad; st += 2) {
                    if (!mbar_wait(smem_u32(&tail->full[s]), ph, s_abort, err, 53)) { alive = false; break; }
                    fence_proxy_async();
                    tc_fence_after();
                    const uint32_t a_tile = stage_base + (uint32_t)(2 * s) * STAGE_BYTES;
                    const int halves = (st + 1 < stages_per_tile) ? 2 : 1;
                    if (elect_one_sync()) {
                        // descriptor low words (start address >> 4, LBO field); the high words are constants.
                        // forward B: 16 K rows of 64 B per step (1024 B), 8-row groups 512 B apart, 32-column atoms
                        // 4 KB apart, 64-byte swizzle (layout code 4)
                        uint32_t a_lo = (a_tile & 0x3FFFFu) >> 4;
                        constexpr uint32_t a_hi = smem_desc_hi(1024);
                        constexpr uint32_t b_hi = DGRAD ? smem_desc_hi(1024) : (((512u >> 4) & 0x3FFFu) | (1u << 14) | (4u << 29));
                        for (int h = 0; h < halves; ++h) {
                            const uint32_t b_lo = (a_lo + (A_TILE_BYTES >> 4)) | (DGRAD ? 0u : smem_desc_lbo_bits(4096));
#pragma unroll
                            for (int ks = 0; ks < STAGE_K / 16; ++ks)
                                umma_pair_f16_lh(d_tmem, a_lo + ks * 2, a_hi, b_lo + ks * (DGRAD ? 2 : 64), b_hi, idesc,
                                                 ks != 0 ? 1u : ((st | h) != 0 ? 1u : 0u));
                            a_lo += STAGE_BYTES >> 4;
                        }
                        const uint32_t e_local = smem_u32(&tail->empty[s]);
                        umma_pair_commit(e_local);
                        umma_pair_commit(e_local + to_peer);
                    }
                    __syncwarp();
                    if (++s == nbig) { s = 0; ph ^= 1u; }
                }
                if (!alive) break;
                if (elect_one_sync()) {
                    const uint32_t f_local = smem_u32(&tail->accum_full[buf]);
                    umma_pair_commit(f_local);
                    umma_pair_commit(f_local + to_peer);
                }
                __syncwarp();
            }
        } else if (lane == 0) {
            // ------------------------------------------------------------------ relay (odd CTA)
            bool alive = true;
            int s = 0;
            uint32_t ph = 0;
            for (int item = cid; item < items_total && alive; item += n_clusters) {
                for (int st = 0; st < sp_pad; st += 2) {
                    if (!mbar_wait(smem_u32(&tail->full[s]), ph, s_abort, err, 54)) { alive = false; break; }
                    fence_proxy_async();      // this CTA's cp.async writes -> the even CTA's tcgen05.mma reads
                    mbar_arrive_cluster(map_to_cta(smem_u32(&tail->full[s]), 0));
                    if (++s == nbig) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 5..8, both CTAs)
        const int q = warp & 3;
        const int et = tid - (PR_A_WARPS + 1) * 32;
        int local = 0;
        for (int item = cid; item < items_total; item += n_clusters, ++local) {
            const int buf = local & 1;
            const long row = ((long)(item / n_blks) * 2 + rank) * TILE_M + q * 32 + lane;
            const int n0 = (item % n_blks) * BN;
            float* sb = s_bias + buf * 256;
            for (int t = et; t < BN; t += 128)
                sb[t] = (!DGRAD && bias != nullptr) ? widen(__ldg(bias + n0 + t), fp16 != 0) : 0.f;
            named_bar_sync(2, 128);
            if (!warp_wait_pair(smem_u32(&tail->accum_full[buf]), (local >> 1) & 1, s_abort, err, 55, lane)) break;
            tc_fence_after();
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
            uint16_t* orow = out + row * cn + n0;
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
            __syncwarp();
            if (lane == 0) {
                const uint32_t e = smem_u32(&tail->accum_empty[buf]);
                mbar_arrive_cluster(map_to_cta(e, 0));
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_barrier();          // nobody frees tensor memory or leaves while the other CTA's work may still touch it
    if (warp == 4) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
template <int BN, bool DGRAD>
static int launch_conv_pair(const ConvArgs& p, const int32_t* status, cudaStream_t s) {
    const int cred = DGRAD ? p.cout : p.cin;
    const int cn = DGRAD ? p.cin : p.cout;
    const int fp16 = p.dtype == SVTAD_F16 ? 1 : 0;
    constexpr int HALF = BN / 2;
    CUtensorMap map_w;
    {
        uint64_t dims[3] = {(uint64_t)p.cout, (uint64_t)p.cin, (uint64_t)p.kk};
        // dgrad: rows of 64 output channels (K), HALF input-channel rows per CTA, 128-byte swizzle;
        // forward: 32 output channels (N) x 64 input-channel rows (K) per box, 64-byte swizzle
        uint32_t box_d[3] = {64, (uint32_t)HALF, 1};
        uint32_t box_f[3] = {32, 64, 1};
        int rc = tc_make_map_sw(&map_w, 3, p.w, dims, DGRAD ? box_d : box_f, fp16, DGRAD ? 128 : 64);
        if (rc) return rc;
    }
    const size_t stage = A_TILE_BYTES + (size_t)HALF * 128;
    const size_t extra = sizeof(PairTail) + 2 * (size_t)TILE_M * p.kk * sizeof(int) + 2 * 256 * sizeof(float);
    int nstage = (int)((TC_SMEM_LIMIT - 1024 - extra) / stage);
    if (nstage > 16) nstage = 16;
    nstage &= ~1;      // two 64-deep buffers per barrier round
    if (nstage < 4)
        return set_error(SVTAD_ERR_UNSUPPORTED, "tensor-core conv (CTA pairs): not enough shared memory for BN=%d kk=%d", BN, p.kk);
    const size_t smem = 1024 + nstage * stage + extra;
    auto kern = conv_pair_kernel<BN, DGRAD>;
    { int rc_s = tc_ensure_smem(reinterpret_cast<const void*>(kern), smem); if (rc_s) return rc_s; }
    const long m_tiles = (p.n + TILE_M - 1) / TILE_M;
    const int m_pairs = (int)((m_tiles + 1) / 2);
    const int n_blks = cn / BN;
    const long items = (long)m_pairs * n_blks;
    const long max_clusters = tc_num_sms() / 2;
    const int clusters = (int)(items < max_clusters ? items : max_clusters);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * clusters));
    cfg.blockDim = dim3(PR_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    SV_CUDA(cudaLaunchKernelEx(&cfg, kern, map_w, (const uint16_t*)p.a, p.nbr, (const uint16_t*)p.bias,
                               (uint16_t*)p.out, status, (long)p.n, cred, cn, p.kk, p.tpb, nstage, fp16, m_pairs,
                               n_blks, (reinterpret_cast<uintptr_t>(p.out) % 32 == 0) ? 1 : 0, tc_error_ptr()));
    return SVTAD_OK;
}

// widest column block that divides the output width (a pair needs one CTA per row tile whatever the width)
static int pair_pick_bn(int cn) {
    const int cand[4] = {256, 192, 128, 64};
    const char* e = getenv("SVTAD_TC_BN");
    if (e != nullptr && *e) {
        int v = atoi(e);
        for (int c : cand)
            if (v == c && cn % v == 0) return v;
    }
    for (int c : cand)
        if (cn % c == 0) return c;
    return 0;
}

template <bool DGRAD>
static int dispatch_conv_pair(const ConvArgs& p, const int32_t* status, cudaStream_t s) {
    const int cn = DGRAD ? p.cin : p.cout;
    switch (pair_pick_bn(cn)) {
        case 64: return launch_conv_pair<64, DGRAD>(p, status, s);
        case 128: return launch_conv_pair<128, DGRAD>(p, status, s);
        case 192: return launch_conv_pair<192, DGRAD>(p, status, s);
        case 256: return launch_conv_pair<256, DGRAD>(p, status, s);
    }
    return set_error(SVTAD_ERR_UNSUPPORTED, "tensor-core conv (CTA pairs): no column block for width %d", cn);
}

int pair_fwd(const ConvArgs& p, cudaStream_t s) { return dispatch_conv_pair<false>(p, nullptr, s); }
int pair_dgrad(const ConvArgs& p, const int32_t* status, cudaStream_t s) { return dispatch_conv_pair<true>(p, status, s); }

}  // namespace svtad
