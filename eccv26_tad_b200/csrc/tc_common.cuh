// PTX wrappers and descriptor builders shared by the tcgen05 kernels.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace svtad {

// device address of the library's error word (set by bounded waits that give up); see conv_tc.cu
int* tc_error_ptr();

constexpr int TILE_M = 128;
constexpr int STAGE_K = 64;            // 64 x 16-bit = one 128-byte swizzle row
constexpr int A_TILE_BYTES = TILE_M * 128;
constexpr long long WAIT_LIMIT_CYCLES = 4000000000ll;   // about two seconds

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// non-blocking probe of a phase
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the CTA is aborting (this or another wait ran out of time).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* s_abort, int* err, int code) {
    if (mbar_test_wait(bar, parity)) return true;
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
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
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// Arrival on `bar` that fires when all cp.async copies issued so far by this thread have landed; the
// barrier's expected count already includes it (.noinc), so the issuing thread never blocks.
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// one lane of the (converged) warp returns true - the same lane every time for a full mask
__device__ __forceinline__ bool elect_one_sync() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// same with the two shared-memory descriptors given as (low word, high word): the low word is the only part that
// changes from one K step to the next (start address >> 4, and the LBO field), so the issuing thread adds a
// constant instead of rebuilding 64-bit values
__device__ __forceinline__ void umma_f16_lh(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                            uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
}
// accumulating form (D += A.B) with the predicate set once, for every K step but a tile's first
__device__ __forceinline__ void umma_f16_lh_acc(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                                uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.eq.b32 p, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc) : "memory");
}
// high word of a 128-byte-swizzle descriptor (SBO, version 1, layout code 2) and the LBO bits of the low word
__host__ __device__ constexpr uint32_t smem_desc_hi(uint32_t sbo) { return ((sbo >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29); }
__host__ __device__ constexpr uint32_t smem_desc_lbo_bits(uint32_t lbo) { return ((lbo >> 4) & 0x3FFFu) << 16; }
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
// 32-byte store (one whole sector per lane and instruction); `p` must be 32-byte aligned
__device__ __forceinline__ void st_global_v8(void* p, const uint32_t* v) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle (layout code 2), descriptor version 1.
// K-major operand:  rows at 128 B, 8-row groups `sbo` apart, `lbo` unused (0).
// MN-major operand: 64-element (128 B) runs along M/N, `sbo` between 8-row groups along K,
//                   `lbo` between successive 64-element blocks along M/N.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
// Instruction descriptor of tcgen05.mma kind::f16: fp32 accumulate, A/B format (0 = f16, 1 = bf16),
// operand majors (0 = K-major, 1 = MN-major), N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc(int fmt, int a_mn_major, int b_mn_major, int m, int n) {
    return (1u << 4) | (static_cast<uint32_t>(fmt) << 7) | (static_cast<uint32_t>(fmt) << 10) |
           (static_cast<uint32_t>(a_mn_major) << 15) | (static_cast<uint32_t>(b_mn_major) << 16) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi, bool fp16) {
    if (fp16) {
        __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&b);
}
__device__ __forceinline__ float widen(uint16_t v, bool fp16) {
    if (fp16) return __half2float(__ushort_as_half(v));
    return __uint_as_float(static_cast<uint32_t>(v) << 16);
}

// 32 accumulator columns of one output row: + bias (fp32), one rounding, 64 bytes to `dst` - as two whole 32-byte
// sectors when the row is 32-byte aligned, else as four 16-byte stores
__device__ __forceinline__ void store_row_chunk32(uint16_t* dst, const uint32_t (&v)[32], const float* bias32, bool fp16,
                                                  bool al32) {
    const float4* b4 = reinterpret_cast<const float4*>(bias32);
    uint32_t o[16];
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        const float4 ba = b4[g];
        o[2 * g] = pack2(__uint_as_float(v[g * 4 + 0]) + ba.x, __uint_as_float(v[g * 4 + 1]) + ba.y, fp16);
        o[2 * g + 1] = pack2(__uint_as_float(v[g * 4 + 2]) + ba.z, __uint_as_float(v[g * 4 + 3]) + ba.w, fp16);
    }
    if (al32) {
        st_global_v8(dst, &o[0]);
        st_global_v8(dst + 16, &o[8]);
    } else {
        uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
        for (int g = 0; g < 4; ++g) d4[g] = make_uint4(o[4 * g], o[4 * g + 1], o[4 * g + 2], o[4 * g + 3]);
    }
}

// bytes of one B stage: MN-major tiles are whole 64-column blocks of 8 KB, K-major tiles BN rows of 128 B
constexpr int b_tile_bytes_for(int bn) { return ((bn + 63) / 64) * 8192; }
constexpr int tmem_cols_for(int bn) { return bn <= 32 ? 32 : bn <= 64 ? 64 : bn <= 128 ? 128 : 256; }


__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
// hint: bring `bytes` (multiple of 16) starting at the 16-byte aligned `p` into L2; no completion to wait for
__device__ __forceinline__ void l2_prefetch_bulk(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
// rows [row_lo, row_hi) of a row-major 16-bit matrix with `cols` columns, clipped to [0, n)
__device__ __forceinline__ void l2_prefetch_rows(const uint16_t* base, long row_lo, long row_hi, long n, int cols) {
    if (row_lo < 0) row_lo = 0;
    if (row_hi > n) row_hi = n;
    if (row_hi > row_lo) l2_prefetch_bulk(base + row_lo * cols, (uint32_t)((row_hi - row_lo) * cols * 2));
}
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

struct alignas(16) TmaTail {   // 16-byte multiple: the table buffers behind it are filled by 16-byte copies
    uint64_t full[8];
    uint64_t empty[8];
    uint64_t accum_full[2];
    uint64_t accum_empty[2];
    uint32_t tmem_slot;
    int abort_flag;
};

constexpr int tmem_cols2_for(int bn) { return 2 * bn <= 64 ? 64 : 2 * bn <= 128 ? 128 : 2 * bn <= 256 ? 256 : 512; }


// ---- host helpers shared by the tensor-core translation units (defined in conv_tc.cu) ----
template <typename... KArgs, typename... Args>
inline cudaError_t tc_launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
constexpr size_t TC_SMEM_LIMIT = 227 * 1024;
int tc_num_sms();
int tc_plan_sms();          // SMs a kernel is planned for: all of them divided by the caller's concurrency hint
int tc_set_share(int n);    // sets the hint, returns the previous one
int tc_get_share();
int tc_set_share_floor(int n);   // per calling thread; returns the previous floor
int tc_ensure_smem(const void* kern, size_t bytes);
// 16-bit tensor map with 128-byte swizzle and zero fill outside the tensor; dims[0] is the contiguous one
int tc_make_map(CUtensorMap* map, int rank, const void* base, const uint64_t* dims, const uint32_t* box, int fp16);
// same with a 64- or 128-byte swizzle
int tc_make_map_sw(CUtensorMap* map, int rank, const void* base, const uint64_t* dims, const uint32_t* box, int fp16,
                   int swizzle_bytes);
// column-block width of a forward / dgrad CTA for an output of `cn` columns and `m_tiles` row tiles
int tc_pick_bn(int cn, long m_tiles);
struct WgradPlan {
    int bn, n_nblk, n_pairs, splits, ones_block;
    long tokens_per_split;
};
WgradPlan tc_wgrad_plan(int64_t n, int cin, int cout, int kk);
size_t tc_wgrad_plan_ws_bytes(int64_t n, int cin, int cout, int kk);

// fixed-order reduction of per-split fp32 partials into the 16-bit gradient tensors
int tc_wgrad_reduce_launch(const float* ws_w, int splits, const float* ws_b, int splits_b, void* gw, void* gb,
                           long n_w, int cout, int fp16, cudaStream_t s);

}  // namespace svtad
