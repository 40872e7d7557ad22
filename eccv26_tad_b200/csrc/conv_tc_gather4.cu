// All-TMA variant of the tcgen05 SparseConv2D kernels (selected with SVTAD_TC_IMPL=gather4).
//
// Same math and tile shapes as conv_tc_hybrid.cu, but every operand reaches shared memory through the
// tensor-memory-accelerator.  Measured slower than the hybrid feed on B200 (one gather4 moves only
// 512 bytes), kept as a validated alternative:
//   * gathered rows (x for forward / wgrad, gy for dgrad): cp.async.bulk.tensor tile::gather4 - one
//     instruction fetches four arbitrary rows x 64 channels and writes them 128-byte-swizzled; a row
//     index past the end of the tensor reads as zeros, which is how -1 table entries are served;
//   * weights / gy tiles: plain tiled TMA boxes.
// One warp produces (each lane issues one gather4 per stage), one thread issues the MMAs, four warps
// drain the accumulator.  Forward / dgrad CTAs are persistent over output tiles with two accumulators
// in tensor memory so that a tile's epilogue overlaps the next tile's main loop.  No TMA load here
// uses cluster multicast.  Every mbarrier wait is bounded (see tc_common.cuh).
#include <cstdlib>

#include "tc_common.cuh"

namespace svtad {

constexpr int TMA_THREADS = 192;   // warp 0 producer, warp 1 MMA + TMEM owner, warps 2-5 epilogue

// ---------------------------------------------------------------------------------------------
// forward / dgrad, persistent over (row tile, column block)
// ---------------------------------------------------------------------------------------------
template <int BN, bool DGRAD>
__global__ void __launch_bounds__(TMA_THREADS, 1)
conv_tma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                const int32_t* __restrict__ nbr, const uint16_t* __restrict__ bias,
                uint16_t* __restrict__ out, const int32_t* __restrict__ status, long n, int cred, int cn,
                int kk, int tpb, int nstage, int fp16, int m_tiles, int n_blks, int* __restrict__ err) {
    if (DGRAD && status != nullptr && (__ldg(status) & SVTAD_TABLE_ASYMMETRIC)) return;
    constexpr int B_TILE_BYTES = b_tile_bytes_for(BN);
    constexpr int B_TX_BYTES = DGRAD ? BN * 128 : B_TILE_BYTES;
    constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
    constexpr int TM_COLS = tmem_cols2_for(BN);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    TmaTail* tail = reinterpret_cast<TmaTail*>(smem + (size_t)nstage * STAGE_BYTES);
    int* s_tab = reinterpret_cast<int*>(tail + 1);                 // [2][TILE_M * kk] raw table rows
    volatile int* s_abort = &tail->abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t stage_base = smem_u32(smem);
    const int tiles_total = m_tiles * n_blks;
    const int kchunks = cred / STAGE_K;
    const int stages_per_tile = kk * kchunks;
    const int tab_ints = TILE_M * kk;

    if (warp == 1) {
        tmem_alloc(smem_u32(&tail->tmem_slot), TM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        for (int s = 0; s < nstage; ++s) {
            mbar_init(smem_u32(&tail->full[s]), 1);
            mbar_init(smem_u32(&tail->empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&tail->accum_full[b]), 1);
            mbar_init(smem_u32(&tail->accum_empty[b]), 128);
        }
        tail->abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_map(&map_a);
        tma_prefetch_map(&map_w);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tail->tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        // raw table rows of a tile -> s_tab[buf] with 16-byte async copies (rows past n read as zero bytes)
        auto load_table = [&](int tile, int buf) {
            const long row0 = (long)(tile / n_blks) * TILE_M;
            const long rows = (n - row0) < TILE_M ? (n - row0) : TILE_M;
            const int valid_bytes = (int)rows * kk * 4;
            const char* src = reinterpret_cast<const char*>(nbr + row0 * kk);
            const uint32_t dst = smem_u32(s_tab + buf * tab_ints);
            for (int c = lane; c * 16 < tab_ints * 4; c += 32) {
                int left = valid_bytes - c * 16;
                uint32_t nb = left >= 16 ? 16u : (left > 0 ? (uint32_t)left : 0u);
                cp_async16(dst + c * 16, nb ? src + c * 16 : src, nb);
            }
        };
        bool alive = true;
        int it = 0;
        if ((int)blockIdx.x < tiles_total) load_table(blockIdx.x, 0);
        int local = 0;
        for (int tile = blockIdx.x; tile < tiles_total && alive; tile += gridDim.x, ++local) {
            const int buf = local & 1;
            const long row0 = (long)(tile / n_blks) * TILE_M;
            const int n0 = (tile % n_blks) * BN;
            asm volatile("cp.async.wait_all;" ::: "memory");
            __syncwarp();
            if (tile + (int)gridDim.x < tiles_total) load_table(tile + gridDim.x, buf ^ 1);
            long off[4];
            bool rowok[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                long i = row0 + lane * 4 + j;
                rowok[j] = i < n;
                off[j] = tpb > 0 ? (i / tpb) * (long)tpb : 0;
            }
            const int* tab = s_tab + buf * tab_ints + lane * 4 * kk;
            for (int k = 0; k < kk && alive; ++k) {
                int idx[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    int raw = tab[j * kk + k];
                    long jj = (long)raw + off[j];
                    idx[j] = (rowok[j] && raw >= 0 && jj < n) ? (int)jj : (int)n;   // row n is out of bounds: zeros
                }
                const int wtap = DGRAD ? (kk - 1 - k) : k;
                for (int kc = 0; kc < kchunks; ++kc, ++it) {
                    const int s = it % nstage;
                    if (!mbar_wait(smem_u32(&tail->empty[s]), ((it / nstage) & 1) ^ 1, s_abort, err, 21)) { alive = false; break; }
                    const uint32_t a_tile = stage_base + (uint32_t)s * STAGE_BYTES;
                    const uint32_t b_tile = a_tile + A_TILE_BYTES;
                    const uint32_t bar = smem_u32(&tail->full[s]);
                    const int c0 = kc * STAGE_K;
                    if (lane == 0) {
                        mbar_expect_tx(bar, A_TILE_BYTES + B_TX_BYTES);
                        if (!DGRAD) {
#pragma unroll
                            for (int b = 0; b < B_TILE_BYTES / 8192; ++b)
                                tma_load_3d(b_tile + b * 8192, &map_w, n0 + b * 64, c0, wtap, bar);
                        } else {
                            tma_load_3d(b_tile, &map_w, c0, n0, wtap, bar);
                        }
                    }
                    __syncwarp();   // the stage's byte count is posted before any lane's copy can complete
                    tma_gather4(a_tile + lane * 512, &map_a, c0, idx[0], idx[1], idx[2], idx[3], bar);
                }
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = make_idesc(fp16 ? 0 : 1, 0, DGRAD ? 0 : 1, TILE_M, BN);
            bool alive = true;
            int it = 0, local = 0;
            for (int tile = blockIdx.x; tile < tiles_total && alive; tile += gridDim.x, ++local) {
                const int buf = local & 1;
                if (!mbar_wait(smem_u32(&tail->accum_empty[buf]), ((local >> 1) & 1) ^ 1, s_abort, err, 22)) { alive = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int st = 0; st < stages_per_tile; ++st, ++it) {
                    const int s = it % nstage;
                    if (!mbar_wait(smem_u32(&tail->full[s]), (it / nstage) & 1, s_abort, err, 23)) { alive = false; break; }
                    tc_fence_after();
                    const uint32_t a_tile = stage_base + (uint32_t)s * STAGE_BYTES;
                    const uint32_t b_tile = a_tile + A_TILE_BYTES;
#pragma unroll
                    for (int ks = 0; ks < STAGE_K / 16; ++ks) {
                        uint64_t ad = make_smem_desc(a_tile + ks * 32, 0, 1024);
                        uint64_t bd = DGRAD ? make_smem_desc(b_tile + ks * 32, 0, 1024)
                                            : make_smem_desc(b_tile + ks * 2048, 8192, 1024);
                        umma_f16(d_tmem, ad, bd, idesc, (st | ks) != 0 ? 1u : 0u);
                    }
                    umma_commit(smem_u32(&tail->empty[s]));
                }
                if (alive) umma_commit(smem_u32(&tail->accum_full[buf]));
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int q = warp & 3;
        bool alive = true;
        int local = 0;
        for (int tile = blockIdx.x; tile < tiles_total && alive; tile += gridDim.x, ++local) {
            const int buf = local & 1;
            const long row = (long)(tile / n_blks) * TILE_M + q * 32 + lane;
            const int n0 = (tile % n_blks) * BN;
            if (!mbar_wait(smem_u32(&tail->accum_full[buf]), (local >> 1) & 1, s_abort, err, 24)) { alive = false; break; }
            tc_fence_after();
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
#pragma unroll 1
            for (int cbase = 0; cbase < BN; cbase += 32) {
                uint32_t v[32];
                tmem_ld32(t_addr + cbase, v);
                tmem_ld_wait();
                if (row < n) {
                    uint4* dst = reinterpret_cast<uint4*>(out + row * cn + n0 + cbase);
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        float b8[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            b8[e] = (!DGRAD && bias != nullptr) ? widen(__ldg(bias + n0 + cbase + g * 8 + e), fp16 != 0) : 0.f;
                        uint4 o;
                        o.x = pack2(__uint_as_float(v[g * 8 + 0]) + b8[0], __uint_as_float(v[g * 8 + 1]) + b8[1], fp16 != 0);
                        o.y = pack2(__uint_as_float(v[g * 8 + 2]) + b8[2], __uint_as_float(v[g * 8 + 3]) + b8[3], fp16 != 0);
                        o.z = pack2(__uint_as_float(v[g * 8 + 4]) + b8[4], __uint_as_float(v[g * 8 + 5]) + b8[5], fp16 != 0);
                        o.w = pack2(__uint_as_float(v[g * 8 + 6]) + b8[6], __uint_as_float(v[g * 8 + 7]) + b8[7], fp16 != 0);
                        dst[g] = o;
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(smem_u32(&tail->accum_empty[buf]));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, TM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
// wgrad: D[128 = two 64-channel blocks of (tap, ci), BN] += gathered x^T . gy over a token range
// ---------------------------------------------------------------------------------------------
template <int BN>
__global__ void __launch_bounds__(TMA_THREADS, 1)
wgrad_tma_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_gy,
                 const int32_t* __restrict__ nbr, float* __restrict__ ws_w, float* __restrict__ ws_b,
                 long n, int cin, int cout, int kk, int tpb, long tokens_per_split, int n_nblk,
                 int nstage, int fp16, int ones_block, int* __restrict__ err) {
    constexpr int B_TILE_BYTES = b_tile_bytes_for(BN);
    constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
    constexpr int TM_COLS = tmem_cols_for(BN);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    TmaTail* tail = reinterpret_cast<TmaTail*>(smem + (size_t)nstage * STAGE_BYTES);
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
    // second block of the last pair when the block count is odd: all ones, so its rows of D are sum_i gy[i,:]
    const bool ones_here = ones_block && (pair * 2 + 1 == nblocks);

    if (warp == 1) {
        tmem_alloc(smem_u32(&tail->tmem_slot), TM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        for (int s = 0; s < nstage; ++s) {
            mbar_init(smem_u32(&tail->full[s]), 1);
            mbar_init(smem_u32(&tail->empty[s]), 1);
        }
        mbar_init(smem_u32(&tail->accum_full[0]), 1);
        tail->abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_map(&map_x);
        tma_prefetch_map(&map_gy);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tail->tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        const int h = lane >> 4;                      // which 64-channel block this lane gathers for
        const int blk = pair * 2 + h;
        const bool real = blk < nblocks;
        const int tap = real ? blk / cblocks : 0;
        const int ch0 = real ? (blk % cblocks) * 64 : 0;
        const bool gather = real;                     // lanes of a missing / all-ones block issue nothing
        if (!real) {
            // fill this block of every stage once: ones (bias row trick) or zeros
            const uint32_t word = ones_here ? (fp16 ? 0x3C003C00u : 0x3F803F80u) : 0u;
            for (int s = 0; s < nstage; ++s) {
                uint32_t base = stage_base + (uint32_t)s * STAGE_BYTES + 8192;
                for (int c = (lane & 15); c < 512; c += 16)
                    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(base + c * 16), "r"(word) : "memory");
            }
            fence_proxy_async();
        }
        __syncwarp();
        const uint32_t a_bytes = (pair * 2 + 1 < nblocks) ? A_TILE_BYTES : A_TILE_BYTES / 2;
        auto fetch = [&](int stage_it, int (&dst)[4]) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                long i = i_begin + (long)stage_it * STAGE_K + (lane & 15) * 4 + j;
                int v = (int)n;
                if (gather && i < i_end) {
                    int raw = __ldg(nbr + i * kk + tap);
                    long jj = (long)raw + (tpb > 0 ? (i / tpb) * (long)tpb : 0);
                    if (raw >= 0 && jj < n) v = (int)jj;
                }
                dst[j] = v;
            }
        };
        int cur[4], nxt[4] = {0, 0, 0, 0};
        if (total_stages > 0) fetch(0, cur);
        for (int it = 0; it < total_stages; ++it) {
            const int s = it % nstage;
            if (it + 1 < total_stages) fetch(it + 1, nxt);
            if (!mbar_wait(smem_u32(&tail->empty[s]), ((it / nstage) & 1) ^ 1, s_abort, err, 31)) break;
            const uint32_t a_tile = stage_base + (uint32_t)s * STAGE_BYTES;
            const uint32_t b_tile = a_tile + A_TILE_BYTES;
            const uint32_t bar = smem_u32(&tail->full[s]);
            if (lane == 0) {
                mbar_expect_tx(bar, a_bytes + B_TILE_BYTES);
                const int i0 = (int)(i_begin + (long)it * STAGE_K);
#pragma unroll
                for (int b = 0; b < B_TILE_BYTES / 8192; ++b)
                    tma_load_2d(b_tile + b * 8192, &map_gy, n0 + b * 64, i0, bar);
            }
            __syncwarp();
            if (gather) tma_gather4(a_tile + lane * 512, &map_x, ch0, cur[0], cur[1], cur[2], cur[3], bar);
#pragma unroll
            for (int j = 0; j < 4; ++j) cur[j] = nxt[j];
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = make_idesc(fp16 ? 0 : 1, 1, 1, TILE_M, BN);
            bool alive = true;
            for (int it = 0; it < total_stages; ++it) {
                const int s = it % nstage;
                if (!mbar_wait(smem_u32(&tail->full[s]), (it / nstage) & 1, s_abort, err, 32)) { alive = false; break; }
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
            if (alive && total_stages > 0) umma_commit(smem_u32(&tail->accum_full[0]));
        }
    } else {
        // epilogue: fp32 partial tile -> ws_w[split][(tap, ci)][co]; the all-ones block -> ws_b[split][co]
        bool have = true;
        if (total_stages > 0) have = mbar_wait(smem_u32(&tail->accum_full[0]), 0, s_abort, err, 33);
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
#pragma unroll 1
            for (int cbase = 0; cbase < BN; cbase += 32) {
                uint32_t v[32];
                if (total_stages > 0) {
                    tmem_ld32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + cbase, v);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0u;
                }
                if (dstrow != nullptr) {
                    uint4* dst = reinterpret_cast<uint4*>(dstrow + cbase);
#pragma unroll
                    for (int g = 0; g < 8; ++g) dst[g] = make_uint4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, TM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
template <int BN, bool DGRAD>
static int launch_conv_tma(const ConvArgs& p, const int32_t* status, cudaStream_t s) {
    const int cred = DGRAD ? p.cout : p.cin;
    const int cn = DGRAD ? p.cin : p.cout;
    const int fp16 = p.dtype == SVTAD_F16 ? 1 : 0;
    CUtensorMap map_a, map_w;
    {
        uint64_t dims[2] = {(uint64_t)cred, (uint64_t)p.n};
        uint32_t box[2] = {64, 1};
        int rc = tc_make_map(&map_a, 2, p.a, dims, box, fp16);
        if (rc) return rc;
    }
    {
        uint64_t dims[3] = {(uint64_t)p.cout, (uint64_t)p.cin, (uint64_t)p.kk};
        uint32_t box[3] = {64, (uint32_t)(DGRAD ? BN : 64), 1};
        int rc = tc_make_map(&map_w, 3, p.w, dims, box, fp16);
        if (rc) return rc;
    }
    const size_t stage = A_TILE_BYTES + b_tile_bytes_for(BN);
    const size_t extra = sizeof(TmaTail) + 2 * (size_t)TILE_M * p.kk * sizeof(int);
    int nstage = (int)((TC_SMEM_LIMIT - 1024 - extra) / stage);
    if (nstage > 8) nstage = 8;
    if (nstage < 2)
        return set_error(SVTAD_ERR_UNSUPPORTED, "tensor-core conv: not enough shared memory for BN=%d kk=%d", BN, p.kk);
    const size_t smem = 1024 + nstage * stage + extra;
    auto kern = conv_tma_kernel<BN, DGRAD>;
    SV_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int m_tiles = (int)((p.n + TILE_M - 1) / TILE_M);
    const int n_blks = cn / BN;
    long tiles = (long)m_tiles * n_blks;
    int grid = (int)(tiles < tc_num_sms() ? tiles : tc_num_sms());
    kern<<<grid, TMA_THREADS, smem, s>>>(map_a, map_w, p.nbr, (const uint16_t*)p.bias, (uint16_t*)p.out, status,
                                         (long)p.n, cred, cn, p.kk, p.tpb, nstage, fp16, m_tiles, n_blks,
                                         tc_error_ptr());
    SV_LAUNCH_CHECK("conv_tma_kernel");
    return SVTAD_OK;
}

template <bool DGRAD>
static int dispatch_conv_tma(const ConvArgs& p, const int32_t* status, cudaStream_t s) {
    const int cn = DGRAD ? p.cin : p.cout;
    int bn = tc_pick_bn(cn, (p.n + TILE_M - 1) / TILE_M);
    switch (bn) {
        case 64: return launch_conv_tma<64, DGRAD>(p, status, s);
        case 96: return launch_conv_tma<96, DGRAD>(p, status, s);
        case 128: return launch_conv_tma<128, DGRAD>(p, status, s);
        case 192: return launch_conv_tma<192, DGRAD>(p, status, s);
        case 256: return launch_conv_tma<256, DGRAD>(p, status, s);
    }
    return set_error(SVTAD_ERR_UNSUPPORTED, "tensor-core conv: no column block for width %d", cn);
}

int gather4_fwd(const ConvArgs& p, cudaStream_t s) { return dispatch_conv_tma<false>(p, nullptr, s); }
int gather4_dgrad(const ConvArgs& p, const int32_t* status, cudaStream_t s) { return dispatch_conv_tma<true>(p, status, s); }

template <int BN>
static int launch_wgrad_tma(const void* gy, const void* x, const int32_t* nbr, float* ws_w, float* ws_b, int64_t n,
                            int cin, int cout, int kk, int tpb, int fp16, const WgradPlan& pl, cudaStream_t s) {
    CUtensorMap map_x, map_gy;
    {
        uint64_t dims[2] = {(uint64_t)cin, (uint64_t)n};
        uint32_t box[2] = {64, 1};
        int rc = tc_make_map(&map_x, 2, x, dims, box, fp16);
        if (rc) return rc;
    }
    {
        uint64_t dims[2] = {(uint64_t)cout, (uint64_t)n};
        uint32_t box[2] = {64, 64};
        int rc = tc_make_map(&map_gy, 2, gy, dims, box, fp16);
        if (rc) return rc;
    }
    const size_t stage = A_TILE_BYTES + b_tile_bytes_for(BN);
    int nstage = (int)((TC_SMEM_LIMIT - 1024 - sizeof(TmaTail)) / stage);
    if (nstage > 8) nstage = 8;
    const size_t smem = 1024 + nstage * stage + sizeof(TmaTail);
    auto kern = wgrad_tma_kernel<BN>;
    SV_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)(pl.n_pairs * pl.n_nblk), (unsigned)pl.splits);
    kern<<<grid, TMA_THREADS, smem, s>>>(map_x, map_gy, nbr, ws_w, ws_b, (long)n, cin, cout, kk, tpb,
                                         pl.tokens_per_split, pl.n_nblk, nstage, fp16, pl.ones_block,
                                         tc_error_ptr());
    SV_LAUNCH_CHECK("wgrad_tma_kernel");
    return SVTAD_OK;
}

int gather4_wgrad(const void* gy, const void* x, const int32_t* nbr, void* gw, void* gb, int64_t n, int cin, int cout,
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
    int rc;
    switch (pl.bn) {
        case 64: rc = launch_wgrad_tma<64>(gy, x, nbr, ws_w, bias_in_kernel ? ws_b : nullptr, n, cin, cout, kk, tpb, fp16, pl, s); break;
        case 128: rc = launch_wgrad_tma<128>(gy, x, nbr, ws_w, bias_in_kernel ? ws_b : nullptr, n, cin, cout, kk, tpb, fp16, pl, s); break;
        case 192: rc = launch_wgrad_tma<192>(gy, x, nbr, ws_w, bias_in_kernel ? ws_b : nullptr, n, cin, cout, kk, tpb, fp16, pl, s); break;
        case 256: rc = launch_wgrad_tma<256>(gy, x, nbr, ws_w, bias_in_kernel ? ws_b : nullptr, n, cin, cout, kk, tpb, fp16, pl, s); break;
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
