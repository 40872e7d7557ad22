// Neighbor-table kernels: full-grid init, fused top-k + compaction + table build, remap, check.
//
// Semantics follow the torch code of the reference backbone
// (opentad/models/backbones/vit_sparse_adapter_poguise.py: :1623-1670 init, :785-787 selection,
// :913-977 gather + remap); the algorithms do not: selection is an exact k-th-key search on
// order-preserving integer keys, compaction is a ballot/popc prefix scan, and the table is
// emitted straight from the kept set without materialising the old-to-new map in HBM.
#include "common.cuh"

namespace svtad {

// float -> uint32 key with the same order as "a > b" on floats; every NaN maps to the largest
// key (torch.topk ranks NaN above all numbers); -0.0 and +0.0 map to the same key.
__device__ __forceinline__ uint32_t score_key(float f) {
    if (f != f) return 0xFFFFFFFFu;
    if (f == 0.0f) f = 0.0f;
    uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// ------------------------------------------------------------------------------------------
// init
// ------------------------------------------------------------------------------------------
__global__ void table_init_kernel(int32_t* __restrict__ table, long total, int hw, int h, int w,
                                  int ksize, int kk) {
    long f0 = (long)(blockIdx.x * (long)blockDim.x + threadIdx.x) * 4;
    if (f0 >= total) return;
    int r = ksize >> 1;
    int32_t v[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        long f = f0 + e;
        long row = f / kk;
        int tap = (int)(f - row * kk);
        int p = (int)(row % hw);
        int y = p / w, x = p - y * w;
        int dy = tap / ksize - r, dx = tap % ksize - r;
        int yy = y + dy, xx = x + dx;
        v[e] = ((unsigned)yy < (unsigned)h && (unsigned)xx < (unsigned)w)
                   ? (int32_t)(row + dy * w + dx) : -1;
    }
    if (f0 + 3 < total && (reinterpret_cast<uintptr_t>(table) & 15) == 0) {
        *reinterpret_cast<int4*>(table + f0) = make_int4(v[0], v[1], v[2], v[3]);
    } else {
        for (int e = 0; e < 4 && f0 + e < total; ++e) table[f0 + e] = v[e];
    }
}

// ------------------------------------------------------------------------------------------
// build: one warp per segment (seg_len <= 32 * ITEMS)
// ------------------------------------------------------------------------------------------
template <int KS>
__device__ __forceinline__ void tap_to_dydx(int tap, int ksize, int& dy, int& dx) {
    if constexpr (KS > 0) {
        dy = tap / KS - KS / 2;
        dx = tap % KS - KS / 2;
    } else {
        dy = tap / ksize - ksize / 2;
        dx = tap % ksize - ksize / 2;
    }
}

// floor(e / d) for e < 65536 with the host-computed multiplier ceil(2^32 / d)
__device__ __forceinline__ int div_magic(int e, uint32_t magic) { return (int)__umulhi((uint32_t)e, magic); }

template <int ITEMS, int KS>
__global__ void __launch_bounds__(256)
table_build_warp_kernel(const float* __restrict__ scores, int n_seg, int L, int k, int h, int w,
                        int ksize, uint32_t magic_w, uint32_t magic_hw, int32_t* __restrict__ kept_idx,
                        int32_t* __restrict__ table, int64_t* __restrict__ idx64) {
    constexpr int WARPS = 8;
    constexpr int CAP = ITEMS * 32;
    constexpr int KKMAX = (KS > 0) ? KS * KS : 49;
    __shared__ int16_t s_rank[WARPS][CAP];
    __shared__ uint32_t s_pos[WARPS][CAP];
    constexpr int RR = (KS > 0 && KS <= 5) ? 32 : 8;   // kept tokens whose rows are staged per round
    __shared__ int32_t s_out[WARPS][RR * KKMAX];     // staged table rows, written out with coalesced stores
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int seg = blockIdx.x * WARPS + wid;
    if (seg >= n_seg) return;
    const unsigned lt = (1u << lane) - 1u;
    const float* sc = scores + (long)seg * L;

    uint32_t key[ITEMS];
#pragma unroll
    for (int j = 0; j < ITEMS; ++j) {
        int e = j * 32 + lane;
        key[j] = (e < L) ? score_key(__ldg(sc + e)) : 0u;   // 0 is below every real key
    }
    // Threshold search, bit by bit from the top: T grows while count(key >= T) >= k.  As soon as the count
    // is exactly k the kept set {key >= T} is decided and the remaining bits are skipped; if it never is
    // (ties at the boundary) all 32 bits are walked and T ends as the k-th largest key.
    uint32_t T = 0;
    if (L != k) {
#pragma unroll 1
        for (int bit = 31; bit >= 0; --bit) {
            uint32_t cand = T | (1u << bit);
            int c = 0;
#pragma unroll
            for (int j = 0; j < ITEMS; ++j) c += (key[j] >= cand);
            c = __reduce_add_sync(0xffffffffu, c);
            if (c >= k) {
                T = cand;
                if (c == k) break;
            }
        }
    }
    int gt = 0;
#pragma unroll
    for (int j = 0; j < ITEMS; ++j) gt += (key[j] > T);
    gt = __reduce_add_sync(0xffffffffu, gt);
    const int need_ties = k - gt;   // >= 1 ties at the threshold are kept, lowest index first

    const int hw = h * w;
    int run_tie = 0, run_keep = 0;
#pragma unroll
    for (int j = 0; j < ITEMS; ++j) {
        int e = j * 32 + lane;
        bool valid = e < L;
        bool eq = valid && key[j] == T;
        bool g = valid && key[j] > T;
        unsigned eqm = __ballot_sync(0xffffffffu, eq);
        int tie_rank = run_tie + __popc(eqm & lt);
        bool keep = g || (eq && tie_rank < need_ties);
        unsigned km = __ballot_sync(0xffffffffu, keep);
        int rank = run_keep + __popc(km & lt);
        if (valid) s_rank[wid][e] = keep ? (int16_t)rank : (int16_t)-1;
        if (keep) {
            int p = (hw == 1) ? 0 : e - div_magic(e, magic_hw) * hw;
            int y = (w == 1) ? p : div_magic(p, magic_w), x = p - y * w;
            s_pos[wid][rank] = (uint32_t)e | ((uint32_t)y << 16) | ((uint32_t)x << 24);
        }
        run_tie += __popc(eqm);
        run_keep += __popc(km);
    }
    __syncwarp();

    const long base = (long)seg * k;
    if (kept_idx != nullptr)
        for (int r = lane; r < k; r += 32) kept_idx[base + r] = (int32_t)(s_pos[wid][r] & 0xFFFFu);
    if (idx64 != nullptr)
        for (int r = lane; r < k; r += 32) idx64[base + r] = (int64_t)(s_pos[wid][r] & 0xFFFFu);
    if (table == nullptr) return;

    // one lane per kept token computes its K*K entries into shared memory; the warp then writes the
    // staged rows (contiguous in the table) with 16-byte stores
    const int KK = (KS > 0) ? KS * KS : ksize * ksize;
    int32_t* so = s_out[wid];
    for (int r0 = 0; r0 < k; r0 += RR) {
        const int r = r0 + lane;
        if (lane < RR && r < k) {
            const uint32_t pk = s_pos[wid][r];
            const int p = (int)(pk & 0xFFFFu), y = (int)((pk >> 16) & 0xFFu), x = (int)(pk >> 24);
            if (KS > 0) {
#pragma unroll
                for (int tap = 0; tap < KS * KS; ++tap) {
                    const int dy = tap / KS - KS / 2, dx = tap % KS - KS / 2;
                    int32_t v = -1;
                    if ((unsigned)(y + dy) < (unsigned)h && (unsigned)(x + dx) < (unsigned)w) {
                        int rk = s_rank[wid][p + dy * w + dx];
                        if (rk >= 0) v = (int32_t)(base + rk);
                    }
                    so[lane * KK + tap] = v;
                }
            } else {
                for (int tap = 0; tap < KK; ++tap) {
                    const int dy = tap / ksize - ksize / 2, dx = tap % ksize - ksize / 2;
                    int32_t v = -1;
                    if ((unsigned)(y + dy) < (unsigned)h && (unsigned)(x + dx) < (unsigned)w) {
                        int rk = s_rank[wid][p + dy * w + dx];
                        if (rk >= 0) v = (int32_t)(base + rk);
                    }
                    so[lane * KK + tap] = v;
                }
            }
        }
        __syncwarp();
        const int rows = (k - r0) < RR ? (k - r0) : RR;
        const int cnt = rows * KK;
        const long g0 = (base + r0) * KK;                  // first table element of this round
        int32_t* out = table + g0;
        int lead = (int)((4 - (g0 & 3)) & 3);              // scalars up to the next 16-byte boundary
        if (lead > cnt) lead = cnt;
        if ((reinterpret_cast<uintptr_t>(table) & 15) != 0) lead = cnt;   // unaligned table: all scalar
        if (lane < lead) out[lane] = so[lane];
        const int nvec = (cnt - lead) >> 2;
        for (int v = lane; v < nvec; v += 32) {
            const int o = lead + 4 * v;
            *reinterpret_cast<int4*>(out + o) = make_int4(so[o], so[o + 1], so[o + 2], so[o + 3]);
        }
        for (int o = lead + 4 * nvec + lane; o < cnt; o += 32) out[o] = so[o];
        __syncwarp();
    }
}

// ------------------------------------------------------------------------------------------
// build: one CTA per segment (any seg_len whose rank array fits in shared memory)
// ------------------------------------------------------------------------------------------
constexpr int BLK = 1024;

__device__ __forceinline__ int block_excl_scan_flag(bool flag, int* s_w, int& total) {
    // exclusive prefix count of `flag` over the block in thread order; all threads call it
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    unsigned m = __ballot_sync(0xffffffffu, flag);
    __syncthreads();               // s_w free for reuse
    if (lane == 0) s_w[wid] = __popc(m);
    __syncthreads();
    int before = 0, all = 0;
#pragma unroll
    for (int i = 0; i < BLK / 32; ++i) {
        int c = s_w[i];
        before += (i < wid) ? c : 0;
        all += c;
    }
    total = all;
    return before + __popc(m & ((1u << lane) - 1u));
}

__global__ void __launch_bounds__(BLK)
table_build_block_kernel(const float* __restrict__ scores, int n_seg, int L, int k, int h, int w,
                         int ksize, int32_t* __restrict__ kept_idx, int32_t* __restrict__ table,
                         int64_t* __restrict__ idx64, const int32_t* __restrict__ table_in, int kk_in) {
    extern __shared__ int32_t s_rank[];          // [L]
    __shared__ int s_hist[256];
    __shared__ int s_w[BLK / 32];
    __shared__ uint32_t s_prefix;
    __shared__ int s_need;
    const int seg = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const float* sc = scores + (long)seg * L;

    // (1) radix select of the k-th largest key, one byte per pass, most significant first
    if (tid == 0) { s_prefix = 0; s_need = k; }
    uint32_t mask = 0;
    for (int pass = 3; pass >= 0; --pass) {
        if (tid < 256) s_hist[tid] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix;
        for (int e = tid; e < L; e += BLK) {
            uint32_t key = score_key(__ldg(sc + e));
            if ((key & mask) == prefix) atomicAdd(&s_hist[(key >> (8 * pass)) & 255], 1);
        }
        __syncthreads();
        if (wid == 0) {
            // lane l owns bins 255-8l .. 248-8l (descending); find the bin holding the need-th key
            int need = s_need;
            int cnt[8], sum = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) { cnt[i] = s_hist[255 - 8 * lane - i]; sum += cnt[i]; }
            int incl = sum;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                int t = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += t;
            }
            unsigned hit = __ballot_sync(0xffffffffu, incl >= need);
            int owner = __ffs(hit) - 1;      // always found: total matching keys >= need
            if (lane == owner) {
                int above = incl - sum;      // keys in strictly higher bins
                int i = 0;
                while (i < 7 && above + cnt[i] < need) { above += cnt[i]; ++i; }
                s_prefix = prefix | ((uint32_t)(255 - 8 * lane - i) << (8 * pass));
                s_need = need - above;
            }
        }
        mask |= 0xFFu << (8 * pass);
        __syncthreads();
    }
    const uint32_t T = s_prefix;
    const int need_ties = s_need;

    // (2) ordered compaction: tie ranks, keep flags, new ranks
    int32_t* pos_out = kept_idx + (long)seg * k;      // kept positions, read back in (3)
    int run_tie = 0, run_keep = 0;
    for (int c0 = 0; c0 < L; c0 += BLK) {
        int e = c0 + tid;
        bool valid = e < L;
        uint32_t key = valid ? score_key(__ldg(sc + e)) : 0u;
        bool eq = valid && key == T;
        bool g = valid && key > T;
        int tot_tie, tot_keep;
        int tie_rank = run_tie + block_excl_scan_flag(eq, s_w, tot_tie);
        bool keep = g || (eq && tie_rank < need_ties);
        int rank = run_keep + block_excl_scan_flag(keep, s_w, tot_keep);
        if (valid) s_rank[e] = keep ? rank : -1;
        if (keep) {
            if (kept_idx != nullptr) pos_out[rank] = e;
            if (idx64 != nullptr) idx64[(long)seg * k + rank] = e;
        }
        run_tie += tot_tie;
        run_keep += tot_keep;
    }
    __syncthreads();
    if (table == nullptr) return;

    const long base = (long)seg * k;
    if (table_in != nullptr) {
        // (3') later pruning round: the kept rows of the previous table, renumbered through the rank array
        const long total_in = (long)k * kk_in;
        const long seg0 = (long)seg * L;
        int32_t* out_r = table + base * kk_in;
        for (long f = tid; f < total_in; f += BLK) {
            int r = (int)(f / kk_in);
            int tap = (int)(f - (long)r * kk_in);
            int p = __ldcg(pos_out + r);
            int32_t old = __ldg(table_in + (seg0 + p) * kk_in + tap);
            int32_t v = -1;
            long loc = (long)old - seg0;
            if (old >= 0 && loc >= 0 && loc < L) {
                int rk = s_rank[loc];
                if (rk >= 0) v = (int32_t)(base + rk);
            }
            out_r[f] = v;
        }
        return;
    }

    // (3) emit table rows
    const int KK = ksize * ksize, hw = h * w, r0 = ksize >> 1;
    int32_t* out = table + base * KK;
    const long total = (long)k * KK;
    for (long f = tid; f < total; f += BLK) {
        int r = (int)(f / KK);
        int tap = (int)(f - (long)r * KK);
        int dy = tap / ksize - r0, dx = tap % ksize - r0;
        int p = __ldcg(pos_out + r);
        int q = p % hw;
        int y = q / w, x = q - y * w;
        int yy = y + dy, xx = x + dx;
        int32_t v = -1;
        if ((unsigned)yy < (unsigned)h && (unsigned)xx < (unsigned)w) {
            int rk = s_rank[p + dy * w + dx];
            if (rk >= 0) v = (int32_t)(base + rk);
        }
        out[f] = v;
    }
}

// ------------------------------------------------------------------------------------------
// remap
// ------------------------------------------------------------------------------------------
__global__ void remap_scatter_kernel(const int64_t* __restrict__ idx, int32_t* __restrict__ map,
                                     int B, int n_prev, int n_new) {
    long t = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (t >= (long)B * n_new) return;
    int b = (int)(t / n_new);
    int64_t p = idx[t];
    if (p < 0 || p >= n_prev) return;       // ignored, never written out of range
    map[(long)b * n_prev + p] = (int32_t)t;  // t == b*n_new + j
}

__global__ void remap_gather_kernel(const int32_t* __restrict__ table_in,
                                    const int64_t* __restrict__ idx,
                                    const int32_t* __restrict__ map, int32_t* __restrict__ out,
                                    int B, int n_prev, int n_new, int kk) {
    long f = blockIdx.x * (long)blockDim.x + threadIdx.x;
    long total = (long)B * n_new * kk;
    if (f >= total) return;
    long row = f / kk;
    int tap = (int)(f - row * kk);
    int b = (int)(row / n_new);
    int64_t p = idx[row];
    int32_t v = -1;
    if (p >= 0 && p < n_prev) {
        int32_t old = __ldg(table_in + ((long)b * n_prev + p) * kk + tap);
        if (old >= 0 && (long)old < (long)B * n_prev) v = map[old];
    }
    out[f] = v;
}

// ------------------------------------------------------------------------------------------
// check
// ------------------------------------------------------------------------------------------
__global__ void table_check_kernel(const int32_t* __restrict__ nbr, long n, int kk, int tpb,
                                   int32_t* __restrict__ status) {
    long f = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (f >= n * kk) return;
    long i = f / kk;
    int k = (int)(f - i * kk);
    int32_t j = __ldg(nbr + f);
    if (j == -1) return;
    long off = tpb > 0 ? (i / tpb) * (long)tpb : 0;
    long jj = (long)j + off;
    int bad = 0;
    if (j < -1 || jj < 0 || jj >= n) {
        bad = SVTAD_TABLE_OUT_OF_RANGE | SVTAD_TABLE_ASYMMETRIC;
    } else {
        int32_t back = __ldg(nbr + jj * kk + (kk - 1 - k));
        long off2 = tpb > 0 ? (jj / tpb) * (long)tpb : 0;
        if (back == -1 || (long)back + off2 != i) bad = SVTAD_TABLE_ASYMMETRIC;
    }
    if (bad && ((*reinterpret_cast<volatile int32_t*>(status)) & bad) != bad) atomicOr(status, bad);
}

}  // namespace svtad

using namespace svtad;

// ------------------------------------------------------------------------------------------
// C ABI
// ------------------------------------------------------------------------------------------
extern "C" int svtad_table_init(int B, int T, int h, int w, int ksize, int32_t* table,
                                void* stream) {
    SV_CHECK_ARG(B >= 0 && T >= 0 && h > 0 && w > 0, "svtad_table_init: bad grid %d x %d x %d x %d", B, T, h, w);
    SV_CHECK_ARG(ksize >= 1 && (ksize & 1), "svtad_table_init: ksize must be odd, got %d", ksize);
    long rows = (long)B * T * h * w;
    SV_CHECK_ARG(rows < (1l << 31), "svtad_table_init: %ld rows do not fit int32 indices", rows);
    if (rows == 0) return SVTAD_OK;
    SV_CHECK_ARG(table != nullptr, "svtad_table_init: table is null");
    long total = rows * ksize * ksize;
    long threads = (total + 3) / 4;
    table_init_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        table, total, h * w, h, w, ksize, ksize * ksize);
    SV_LAUNCH_CHECK("table_init_kernel");
    return SVTAD_OK;
}

static int table_build_impl(const float* scores, int n_seg, int seg_len, int k, int h, int w,
                            int ksize, int32_t* kept_idx, int32_t* table, int64_t* idx64,
                            void* stream, const char* who) {
    SV_CHECK_ARG(n_seg >= 0 && seg_len > 0, "%s: bad n_seg=%d seg_len=%d", who, n_seg, seg_len);
    SV_CHECK_ARG(k >= 0 && k <= seg_len, "%s: k_keep=%d outside [0, %d]", who, k, seg_len);
    if (table != nullptr) {
        SV_CHECK_ARG(h > 0 && w > 0 && seg_len % (h * w) == 0,
                     "%s: seg_len=%d is not a multiple of h*w=%d*%d", who, seg_len, h, w);
        SV_CHECK_ARG(ksize >= 1 && (ksize & 1) && ksize <= 15, "%s: ksize must be odd and <= 15, got %d", who, ksize);
        SV_CHECK_ARG(h < 256 && w < 256, "%s: grid side must be < 256", who);
    } else {
        h = seg_len; w = 1; ksize = 1;
    }
    SV_CHECK_ARG((long)n_seg * k < (1l << 31), "%s: n_seg*k_keep does not fit int32 indices", who);
    if (n_seg == 0 || k == 0) return SVTAD_OK;
    SV_CHECK_ARG(scores != nullptr, "%s: scores is null", who);
    cudaStream_t s = (cudaStream_t)stream;
    if (seg_len <= 256) {
        unsigned grid = (unsigned)((n_seg + 7) / 8);
        const uint32_t mw = (uint32_t)((0x100000000ull + w - 1) / w), mhw = (uint32_t)((0x100000000ull + h * w - 1) / (h * w));
        if (ksize == 3)
            table_build_warp_kernel<8, 3><<<grid, 256, 0, s>>>(scores, n_seg, seg_len, k, h, w, ksize, mw, mhw, kept_idx, table, idx64);
        else if (ksize == 5)
            table_build_warp_kernel<8, 5><<<grid, 256, 0, s>>>(scores, n_seg, seg_len, k, h, w, ksize, mw, mhw, kept_idx, table, idx64);
        else
            table_build_warp_kernel<8, 0><<<grid, 256, 0, s>>>(scores, n_seg, seg_len, k, h, w, ksize, mw, mhw, kept_idx, table, idx64);
        SV_LAUNCH_CHECK("table_build_warp_kernel");
        return SVTAD_OK;
    }
    // CTA-per-segment path needs the kept positions in global memory between its phases
    SV_CHECK_ARG(table == nullptr || kept_idx != nullptr, "%s: kept_idx is required with a table", who);
    size_t smem = (size_t)seg_len * sizeof(int32_t);
    if (smem > 200 * 1024)
        return set_error(SVTAD_ERR_UNSUPPORTED, "%s: seg_len=%d exceeds the %d-token segment limit", who, seg_len, 200 * 1024 / 4);
    static thread_local int attr_dev = -1;
    int dev = 0;
    SV_CUDA(cudaGetDevice(&dev));
    if (attr_dev != dev) {
        SV_CUDA(cudaFuncSetAttribute(table_build_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_dev = dev;
    }
    table_build_block_kernel<<<n_seg, BLK, smem, s>>>(scores, n_seg, seg_len, k, h, w, ksize, kept_idx, table, idx64, nullptr, 0);
    SV_LAUNCH_CHECK("table_build_block_kernel");
    return SVTAD_OK;
}

extern "C" int svtad_table_build(const float* scores, int n_seg, int seg_len, int k_keep, int h,
                                 int w, int ksize, int32_t* kept_idx, int32_t* table,
                                 void* stream) {
    SV_CHECK_ARG(k_keep >= 0 && k_keep <= seg_len, "svtad_table_build: k_keep=%d outside [0, %d]", k_keep, seg_len);
    SV_CHECK_ARG(n_seg <= 0 || k_keep == 0 || (kept_idx != nullptr && table != nullptr),
                 "svtad_table_build: kept_idx / table is null");
    return table_build_impl(scores, n_seg, seg_len, k_keep, h, w, ksize, kept_idx, table, nullptr,
                            stream, "svtad_table_build");
}

extern "C" int svtad_topk_select(const float* scores, int n_seg, int seg_len, int k_keep,
                                 int64_t* idx, void* stream) {
    SV_CHECK_ARG(n_seg == 0 || k_keep == 0 || idx != nullptr, "svtad_topk_select: idx is null");
    return table_build_impl(scores, n_seg, seg_len, k_keep, 0, 0, 0, nullptr, nullptr, idx, stream,
                            "svtad_topk_select");
}

extern "C" int svtad_table_select_remap(const float* scores, const int32_t* table_in, int B, int n_prev,
                                        int k_keep, int kk, int32_t* kept_idx, int64_t* idx, int32_t* table_out,
                                        void* stream) {
    SV_CHECK_ARG(B >= 0 && n_prev > 0 && kk > 0, "svtad_table_select_remap: bad sizes");
    SV_CHECK_ARG(k_keep >= 0 && k_keep <= n_prev, "svtad_table_select_remap: k_keep=%d outside [0, %d]", k_keep, n_prev);
    SV_CHECK_ARG((long)B * n_prev < (1l << 31), "svtad_table_select_remap: row count does not fit int32 indices");
    if (B == 0 || k_keep == 0) return SVTAD_OK;
    SV_CHECK_ARG(scores && table_in && kept_idx && table_out, "svtad_table_select_remap: null pointer");
    size_t smem = (size_t)n_prev * sizeof(int32_t);
    if (smem > 200 * 1024)
        return set_error(SVTAD_ERR_UNSUPPORTED, "svtad_table_select_remap: n_prev=%d exceeds the %d-token limit", n_prev, 200 * 1024 / 4);
    SV_CUDA(cudaFuncSetAttribute(table_build_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    table_build_block_kernel<<<B, BLK, smem, (cudaStream_t)stream>>>(scores, B, n_prev, k_keep, n_prev, 1, 1, kept_idx,
                                                                     table_out, idx, table_in, kk);
    SV_LAUNCH_CHECK("table_build_block_kernel");
    return SVTAD_OK;
}

extern "C" int svtad_table_remap(const int32_t* table_in, const int64_t* idx, int B, int n_prev,
                                 int n_new, int kk, int32_t* scratch, int32_t* table_out,
                                 void* stream) {
    SV_CHECK_ARG(B >= 0 && n_prev >= 0 && n_new >= 0 && kk > 0, "svtad_table_remap: bad sizes");
    SV_CHECK_ARG((long)B * n_prev < (1l << 31) && (long)B * n_new < (1l << 31),
                 "svtad_table_remap: row count does not fit int32 indices");
    if (B == 0 || n_new == 0) return SVTAD_OK;
    SV_CHECK_ARG(table_in && idx && scratch && table_out, "svtad_table_remap: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    SV_CUDA(cudaMemsetAsync(scratch, 0xFF, (size_t)B * n_prev * sizeof(int32_t), s));
    long rows = (long)B * n_new;
    remap_scatter_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, s>>>(idx, scratch, B, n_prev, n_new);
    SV_LAUNCH_CHECK("remap_scatter_kernel");
    long total = rows * kk;
    remap_gather_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(table_in, idx, scratch, table_out, B, n_prev, n_new, kk);
    SV_LAUNCH_CHECK("remap_gather_kernel");
    return SVTAD_OK;
}

extern "C" int svtad_table_check(const int32_t* nbr, int64_t n, int kk, int tokens_per_batch,
                                 int32_t* status, void* stream) {
    SV_CHECK_ARG(n >= 0 && kk > 0 && tokens_per_batch >= 0, "svtad_table_check: bad sizes");
    SV_CHECK_ARG(status != nullptr, "svtad_table_check: status is null");
    cudaStream_t s = (cudaStream_t)stream;
    SV_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t), s));
    if (n == 0) return SVTAD_OK;
    SV_CHECK_ARG(nbr != nullptr, "svtad_table_check: nbr is null");
    long total = (long)n * kk;
    table_check_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(nbr, (long)n, kk, tokens_per_batch, status);
    SV_LAUNCH_CHECK("table_check_kernel");
    return SVTAD_OK;
}
