/*
 * svtad.h - C ABI of libsvtad.so: SparseConv2D (SV-TAD) for NVIDIA B200 (sm_100a).
 *
 * This is the whole drop-in boundary of the library.  Every function takes plain device
 * pointers and sizes, launches on the CUDA stream handed in, never allocates and never
 * synchronises the host; inputs, outputs and workspaces belong to the caller.  Every
 * function returns 0 on success or one of the SVTAD_ERR_* codes below, in which case
 * svtad_last_error_string() describes the problem (thread-local).  Bad arguments are
 * rejected on the host; nothing on the device asserts or traps.
 *
 * Conventions shared by all entry points
 *   nbr      int32 [n, kk]   neighbor table; column k = (dy+r)*K + (dx+r), r = K/2, dy outer;
 *                            entry = row index of that neighbor in the SAME [n, C] tensor, or -1
 *   w        [kk, cin, cout] weight, pre-permuted layout of the reference module
 *   dtype    SVTAD_F32 / SVTAD_BF16 / SVTAD_F16 - type of every floating tensor of the call;
 *            products and sums are always fp32, one rounding at the end
 *   tokens_per_batch  > 0: table entries are local to blocks of that many rows and
 *            off(i) = (i / tokens_per_batch) * tokens_per_batch is added per row; 0: global
 *   stream   a cudaStream_t (passed as void* so that C callers need no CUDA headers)
 *
 * Reference interfaces replaced (paths inside pcr-upm/eccv26_tad):
 *   the pybind module opentad_sparse_ops, opentad/models/bricks/2d_sparse_v3_bind.cpp:8-14,
 *   and the torch-op table code of opentad/models/backbones/vit_sparse_adapter_poguise.py.
 */
#ifndef SVTAD_H_
#define SVTAD_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SVTAD_OK 0
#define SVTAD_ERR_ARG 1          /* null pointer, negative size, misaligned pointer ...        */
#define SVTAD_ERR_UNSUPPORTED 2  /* shape / dtype outside what the kernels implement            */
#define SVTAD_ERR_WORKSPACE 3    /* workspace smaller than svtad_workspace_bytes() says         */
#define SVTAD_ERR_CUDA 4         /* a CUDA runtime call or a kernel launch reported an error    */

#define SVTAD_F32 0
#define SVTAD_BF16 1
#define SVTAD_F16 2

#define SVTAD_OP_FWD 0
#define SVTAD_OP_DGRAD 1
#define SVTAD_OP_WGRAD 2
#define SVTAD_OP_BWD 3   /* svtad_conv_bwd: both gradients in one call */

/* Bits of the device status word written by svtad_table_check(). */
#define SVTAD_TABLE_OUT_OF_RANGE 1
#define SVTAD_TABLE_ASYMMETRIC 2

int svtad_version(void);

/* Text of the last error raised on the calling thread ("" if none). */
const char* svtad_last_error_string(void);

/*
 * Full-grid table: table[b, t*h*w + y*w + x, k] = global index of (b, t, y+dy, x+dx) or -1
 * outside the h x w grid.  table: int32 [B, T*h*w, ksize*ksize].
 * Replaces get_initial_neighbor_indices, vit_sparse_adapter_poguise.py:1623-1670.
 */
int svtad_table_init(int B, int T, int h, int w, int ksize, int32_t* table, void* stream);

/*
 * Fused selection + table for one pruning round that starts from the full grid.
 * scores: float32 [n_seg, seg_len], seg_len a multiple of h*w (a segment is a slice or a clip).
 * Keeps the k_keep largest scores of every segment (ties: lower index wins; NaN is largest),
 * writes kept_idx int32 [n_seg, k_keep] (ascending positions inside the segment) and
 * table int32 [n_seg*k_keep, ksize*ksize] (global indices seg*k_keep + rank, or -1).
 * Replaces torch.topk + sort (vit_sparse_adapter_poguise.py:785-787) followed by the
 * gather + remap of :913-977 applied to the table of :1623-1670.
 */
int svtad_table_build(const float* scores, int n_seg, int seg_len, int k_keep, int h, int w,
                      int ksize, int32_t* kept_idx, int32_t* table, void* stream);

/*
 * Selection alone: idx int64 [n_seg, k_keep], ascending, same tie / NaN rule as above.
 * Replaces torch.topk + sort, vit_sparse_adapter_poguise.py:785-787.
 */
int svtad_topk_select(const float* scores, int n_seg, int seg_len, int k_keep, int64_t* idx,
                      void* stream);

/*
 * One pruning round on an existing table.  table_in int32 [B, n_prev, kk] (global over
 * B*n_prev), idx int64 [B, n_new] kept positions per batch row, scratch int32 [B*n_prev]
 * (overwritten), table_out int32 [B, n_new, kk] (global over B*n_new).
 * Replaces the gather + remap in Block._inner_forward, vit_sparse_adapter_poguise.py:913-977;
 * scratch is that code's global_mapping_buffer (:1713-1717).
 */
int svtad_table_remap(const int32_t* table_in, const int64_t* idx, int B, int n_prev, int n_new,
                      int kk, int32_t* scratch, int32_t* table_out, void* stream);

/*
 * Selection and remap of a later pruning round in one kernel: per batch row, the k_keep largest of
 * scores float32 [B, n_prev] (tie / NaN rule as above) give kept_idx int32 [B, k_keep] and, if idx is not
 * NULL, the same positions as int64 [B, k_keep]; table_out int32 [B, k_keep, kk] holds the kept rows of
 * table_in int32 [B, n_prev, kk] renumbered to B*k_keep global indices.  n_prev <= 51200.
 * Replaces torch.topk + sort (vit_sparse_adapter_poguise.py:785-787) plus the gather + remap block
 * (:913-977) of one Block._inner_forward call; needs no mapping buffer.
 */
int svtad_table_select_remap(const float* scores, const int32_t* table_in, int B, int n_prev, int k_keep,
                             int kk, int32_t* kept_idx, int64_t* idx, int32_t* table_out, void* stream);

/*
 * Validates a table on the device: ORs SVTAD_TABLE_OUT_OF_RANGE / SVTAD_TABLE_ASYMMETRIC into
 * status[0] (int32, device memory, cleared by this call first).  "Symmetric" means
 * nbr[nbr[i,k]+off, kk-1-k]+off == i for every valid entry, which every table produced by the
 * functions above satisfies.  Counterpart of the debug validator
 * opentad/models/backbones/internvideo_next.py:41-70, but it reports instead of asserting.
 */
int svtad_table_check(const int32_t* nbr, int64_t n, int kk, int tokens_per_batch,
                      int32_t* status, void* stream);

/* Workspace size (bytes) that the given op needs for the given problem (0 for the forward). */
size_t svtad_workspace_bytes(int op, int64_t n, int cin, int cout, int kk, int dtype);

/*
 * y[i,co] = bias[co] + sum_k sum_ci x[nbr[i,k]+off(i), ci] * w[k,ci,co]; bias may be NULL.
 * Replaces fwd, implicit_gemm_fwd_v2 and implicit_gemm_fwd_v2_chunked
 * (2d_sparse_v3.cu:751-822, implicit_gemm_v2.cu:197-300, :306-417).
 */
int svtad_conv_fwd(const void* x, const int32_t* nbr, const void* w, const void* bias, void* y,
                   int64_t n, int cin, int cout, int kk, int tokens_per_batch, int dtype,
                   void* workspace, size_t workspace_bytes, void* stream);

/*
 * gx[j,ci] = sum over (i,k) with nbr[i,k]+off(i)==j of sum_co gy[i,co] * w[k,ci,co].
 * table_status: NULL when the caller guarantees a symmetric table (the gather form is used);
 * otherwise the device word written by svtad_table_check() - the kernels read it on the
 * device and take the scatter form (fp32 atomics into the workspace) for asymmetric tables.
 * Replaces bwd_in, 2d_sparse_v3.cu:824-835 (kernel :656-709).
 */
int svtad_conv_dgrad(const void* gy, const int32_t* nbr, const void* w, void* gx, int64_t n,
                     int cin, int cout, int kk, int tokens_per_batch, int dtype,
                     const int32_t* table_status, void* workspace, size_t workspace_bytes,
                     void* stream);

/*
 * gw[k,ci,co] = sum_i [nbr[i,k]!=-1] x[nbr[i,k]+off(i), ci] * gy[i,co]; gb[co] = sum_i gy[i,co]
 * (gb may be NULL).  Deterministic: split over tokens into the workspace, then a fixed-order
 * reduction.  Replaces bwd_w, 2d_sparse_v3.cu:837-850 (kernel :714-745) and the bias-grad
 * reduction sparse_conv_layer.py:119-121.
 */
int svtad_conv_wgrad(const void* gy, const void* x, const int32_t* nbr, void* gw, void* gb,
                     int64_t n, int cin, int cout, int kk, int tokens_per_batch, int dtype,
                     void* workspace, size_t workspace_bytes, void* stream);

/*
 * The whole backward of one layer in one call: gx as svtad_conv_dgrad, gw / gb as svtad_conv_wgrad
 * (any of gx, gw may be NULL; gb needs gw).  When both are asked for, the weight gradient runs on a
 * stream owned by the library next to the input gradient on `stream`, forked and joined with events, so
 * for the caller everything is ordered on `stream`; SVTAD_OVERLAP_BACKWARD=0 keeps both on `stream`.
 * Workspace: svtad_workspace_bytes(SVTAD_OP_BWD, ...), 256-byte aligned.
 * Replaces the backward of SparseConv2dFunction, sparse_conv_layer.py:92-123 (bwd_in, then bwd_w, then
 * the bias sum, one after the other).  The first call on a device creates the stream and two events.
 */
int svtad_conv_bwd(const void* gy, const void* x, const int32_t* nbr, const void* w, void* gx, void* gw,
                   void* gb, int64_t n, int cin, int cout, int kk, int tokens_per_batch, int dtype,
                   const int32_t* table_status, void* workspace, size_t workspace_bytes, void* stream);

/*
 * svtad_conv_wgrad for callers that cannot allocate device memory (no counterpart in the reference).
 * Who needs it: hosts that must not call cudaMalloc once they are running - servers that gave all
 * device memory to their own arena, plugins whose host forbids allocation after start-up, loops that
 * cannot afford the implicit synchronisation of an allocation.  The per-split partial sums go to an array
 * of SVTAD_STATIC_WS_BYTES that is part of the library's device image, so every GPU that loads the
 * library holds that much memory until the process exits.  The call itself allocates nothing
 * (no cudaMalloc / cudaFree, no allocating library routine).
 *   - Limit: problems with svtad_workspace_bytes(SVTAD_OP_WGRAD, ...) > SVTAD_STATIC_WS_BYTES are
 *     refused with SVTAD_ERR_WORKSPACE (C = 192 and 256 at 3x3 fit; C = 1024 does not).
 *   - "Allocates nothing" holds from the second call of a kind on.  The first call on a device looks the
 *     array's address up (cudaGetSymbolAddress, with that device current), and the first launch of each
 *     kernel variant (one per column-block width and dtype family, plus the reduction) makes the CUDA
 *     runtime load it, which may allocate inside the driver.  So make one call per shape and dtype that
 *     will be used during start-up, before the phase in which nothing may allocate.
 *   - All calls on a device share the array and it keeps the previous call's contents.  Nothing in
 *     it needs clearing between calls, but two calls that overlap on the GPU (different streams)
 *     race on it: keep them on one stream or order them with events.
 * Arguments and results as svtad_conv_wgrad, minus the workspace.
 */
#define SVTAD_STATIC_WS_BYTES (32u << 20)
size_t svtad_static_workspace_bytes(void);
int svtad_conv_wgrad_static(const void* gy, const void* x, const int32_t* nbr, void* gw, void* gb,
                            int64_t n, int cin, int cout, int kk, int tokens_per_batch, int dtype,
                            void* stream);

/*
 * Sum of a 16-bit gradient bucket over the `world` ranks (GPUs) of one node, in place, by a two-shot exchange
 * over peer-mapped memory: every rank pushes its copy of slice p to rank p, rank p adds the copies up (rank order
 * 0..world-1, fp32, one rounding: all ranks get bit-identical sums) and pushes the result back to everyone.  What
 * crosses NVLink are plain 16-byte stores in which every 8 bytes carry their own flag word (the number of the
 * call), so no phase waits for a system fence or a separate flag.  Replaces the
 * bucket all-reduce torch DDP issues for the adapters' gradients in the reference's training loop
 * (src/eccv26_tad.py:288-300); there the collective is NCCL's.
 *   peer_bufs   HOST array of `world` device pointers: rank p's allocation as THIS rank can address it (its own
 *               at index `rank`).  The caller maps the memory (CUDA IPC, cuMem, torch symmetric memory).
 *   n_elems     elements of the bucket (the start of the allocation), a multiple of 8 * world (pad with zeros)
 *   stage_offset_bytes   where, behind the bucket in the same allocation, svtad_allreduce_stage_bytes(n_elems)
 *               bytes of staging space live; they must be zero before the first call and belong to this function
 *               afterwards
 *   epoch       svtad_allreduce_epoch_bytes() bytes of LOCAL device memory, zero before the first call; it holds
 *               one call counter per CTA, so it (and the staging space) belongs to ONE bucket of one size: the
 *               launch shape follows from n_elems, and a counter array used with buckets of different sizes
 *               would let its counters drift apart
 *   wait_limit_cycles   how long a CTA waits for a peer (SM clock cycles; 0 = about one second).  When the limit
 *               runs out the CTA records code 71 / 72 in the device error word (svtad_device_error), leaves the
 *               bucket as it is and returns; nothing hangs and the context stays usable.
 * Every rank must make the same sequence of calls.  The launch can be captured into a CUDA graph (the call
 * number that the flags carry is kept on the device).  No multicast, no NVLS.  The kernel is built to run beside
 * the convolution kernels: up to 128 CTAs (SVTAD_ALLREDUCE_CTAS) of 128 threads, no dynamic shared memory, the
 * same shared-memory / L1 split as the convolution kernels, so its CTAs fit into what a convolution CTA leaves
 * free on an SM.  To hide it behind other work, put it (and the weight gradients it waits for) on a stream of
 * higher priority than the rest.
 * svtad_allreduce_sum_emulated runs all ranks' parts in one cooperative launch on the current device (`bufs` are
 * then `world` local buffers, `epochs` holds svtad_allreduce_epoch_bytes()): for tests on machines with fewer GPUs than ranks.
 */
size_t svtad_allreduce_stage_bytes(int64_t n_elems);
size_t svtad_allreduce_epoch_bytes(void);
int svtad_allreduce_sum(void* const* peer_bufs, int rank, int world, int64_t n_elems, int dtype,
                        size_t stage_offset_bytes, void* epoch, int64_t wait_limit_cycles, void* stream);
int svtad_allreduce_sum_emulated(void* const* bufs, int world, int64_t n_elems, int dtype,
                                 size_t stage_offset_bytes, void* epochs, int64_t wait_limit_cycles, void* stream);

/*
 * Concurrency hint (no counterpart in the reference): how many of this library's kernels the caller expects to
 * share the GPU at a time - independent layers on streams of their own, forward next to backward.  The default, 1,
 * plans every kernel for the whole GPU, which gives a kernel that runs alone its shortest latency.  With a hint of
 * k the tensor-core kernels are planned for (SMs / k) multiprocessors each: wide column blocks, persistent CTAs
 * that take several row tiles in turn, fewer token splits in the weight gradient.  Every CTA pays a few
 * microseconds of set-up, first-operand latency and epilogue whatever its share of the work, so fewer and longer
 * CTAs cost a lone kernel latency but save SM time when the SMs are contended anyway (three layers' passes in one
 * step on a B200: 0.110 ms with the default, 0.086 ms with a hint of 3).  Results do not depend on the hint beyond
 * the summation order of the weight gradient's partials.  The hint is process-wide and read at launch time;
 * svtad_workspace_bytes does not depend on it (it covers the plan under every hint), so a workspace sized once
 * stays valid when the hint changes.  svtad_conv_bwd, whose two
 * kernels run side by side, plans them for half the GPU each even under the default.
 * svtad_set_concurrency returns the previous value (values are clamped to [1, 16]); SVTAD_CONCURRENCY in the
 * environment gives the start value.
 */
int svtad_set_concurrency(int kernels);
int svtad_get_concurrency(void);

/*
 * Reads (and clears) the device-side error word of the current device: non-zero means a bounded
 * wait inside a kernel gave up and that launch's output is invalid.  Synchronises
 * the device.  No reference counterpart.
 */
int svtad_device_error(int32_t* code_out);

/*
 * Measurement aid: launches one kernel of `ctas` x 256 threads that does nothing but iters * 64 dependent-chain
 * FMAs per thread (8 independent chains), i.e. 2 * 64 * iters * ctas * 256 flops.  Timed by the caller with events
 * on `stream`, it gives the FFMA rate the CUDA-core (fp32) kernels are measured against.  `scratch` is one float
 * of device memory (never written).  No reference counterpart.
 */
int svtad_ffma_probe(int ctas, int iters, float* scratch, void* stream);

/*
 * Which implementation the given problem dispatches to: 0 = CUDA-core (SIMT) kernels,
 * 1 = tcgen05 tensor-core kernels.  Honours the SVTAD_FORCE_PATH=simt|tc environment override.
 */
int svtad_path_for(int op, int64_t n, int cin, int cout, int kk, int dtype);

#ifdef __cplusplus
}
#endif
#endif /* SVTAD_H_ */
