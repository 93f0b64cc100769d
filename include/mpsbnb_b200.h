/*
 * mpsbnb_b200 — C ABI of the B200 (sm_100a) quantize / dequantize / fused dequant-matmul
 * library.  Every function takes raw DEVICE pointers, sizes, and a CUDA stream
 * (cudaStream_t passed as void*; NULL = legacy default stream), enqueues work on that
 * stream WITHOUT synchronising, and returns a status code.  The library never allocates
 * or frees tensor memory: outputs and workspaces are supplied by the caller.
 *
 * Each entry point names the function of the reference (mps-bitsandbytes v0.7.0) it
 * stands in for: the Python function in mps_bitsandbytes/functional.py whose result it
 * must reproduce, and — where one exists — the pybind11 binding of the reference's
 * native extension, mps_bitsandbytes/csrc/mps_bitsandbytes.mm, that a maintainer would
 * re-point at this symbol.
 *
 * Layouts are the reference's, unchanged:
 *   packed 4-bit weights  uint8 [N, Kp/2], low nibble = even k, high nibble = odd k,
 *                         Kp = K rounded up to a multiple of blocksize (functional.py:219-251)
 *   absmax                fp32 [N, Kp/blocksize]; or, double-quantised, int8 of the same
 *                         shape plus fp32 absmax2 [ceil(N*nb/256)] (functional.py:288-292)
 */
#ifndef MPSBNB_B200_H
#define MPSBNB_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes (0 = success, negative = failure) */
#define MPSBNB_OK 0
#define MPSBNB_ERR_INVALID_ARG (-1)   /* null pointer, bad enum, bad size                    */
#define MPSBNB_ERR_UNSUPPORTED (-2)   /* shape / dtype combination this build cannot run     */
#define MPSBNB_ERR_CUDA (-3)          /* a CUDA call failed: see mpsbnb_last_cuda_error()    */
#define MPSBNB_ERR_WORKSPACE (-4)     /* workspace too small: see the *_workspace_bytes call */
#define MPSBNB_ERR_TOO_LARGE (-5)     /* size beyond a documented fixed limit                */
#define MPSBNB_ERR_NO_DEVICE (-6)     /* no sm_100 device is current                         */

/* element types */
#define MPSBNB_F16 0
#define MPSBNB_BF16 1
#define MPSBNB_F32 2
/* 4-bit codebooks: functional.py:21-32 */
#define MPSBNB_NF4 0
#define MPSBNB_FP4 1

const char *mpsbnb_status_string(int status);
/* cudaError_t (as int) and text of the most recent failing CUDA call on this thread */
int mpsbnb_last_cuda_error(void);
const char *mpsbnb_last_cuda_error_string(void);
/* ABI version: bumped on any signature change */
int mpsbnb_abi_version(void);

/* ---------------------------------------------------------------------------------------
 * 4-bit blockwise quantise / dequantise
 * ------------------------------------------------------------------------------------- */

/* functional.py:163-303 quantize_4bit (2-D row-wise path :216-255; the flat path
 * :257-286 is rows = 1, cols = numel).  Binding replaced: _C.quantize_nf4 /
 * _C.quantize_fp4 (mps_bitsandbytes.mm:2738, 2746).
 *   A          [rows, cols] row-major, a_dtype in {F16, BF16, F32}
 *   absmax_in  optional fp32 [rows, nb]: use these block maxima instead of computing them
 *   packed     out uint8 [rows, Kp/2]
 *   absmax_out out fp32  [rows, nb]   (nb = Kp / blocksize); may be NULL if absmax_in given
 * Bit-exact with the reference CPU path.  NaN inputs are not supported. */
int mpsbnb_quantize_4bit(const void *A, int a_dtype, int64_t rows, int64_t cols, int blocksize,
                         int quant_type, const float *absmax_in, uint8_t *packed,
                         float *absmax_out, void *stream);

/* functional.py:306-416 dequantize_4bit, with the double-quant expansion of :335-337
 * folded in.  Binding replaced: _C.dequantize_nf4 / _C.dequantize_fp4
 * (mps_bitsandbytes.mm:2739-2740, 2747-2748).
 *   absmax   fp32 [rows, nb] when absmax2 == NULL, else int8 [rows, nb]
 *   absmax2  NULL, or fp32 [ceil(rows*nb/256)] second-level maxima
 *   out      [rows, cols] in out_dtype
 * Bit-exact with the reference CPU path. */
int mpsbnb_dequantize_4bit(const uint8_t *packed, const void *absmax, const float *absmax2,
                           int64_t rows, int64_t cols, int blocksize, int quant_type, void *out,
                           int out_dtype, void *stream);

/* functional.py:469-539 quantize_blockwise (flat int8, used with blocksize 256 for the
 * double quantisation of absmax, :291).  Binding replaced: _C.double_quant
 * (mps_bitsandbytes.mm:2762) — but with the Python semantics (signed, 127/absmax).
 *   A [n] a_dtype; absmax_in optional fp32 [nblk]; q out int8 [n]; absmax_out fp32 [nblk] */
int mpsbnb_quantize_blockwise(const void *A, int a_dtype, int64_t n, int blocksize,
                              const float *absmax_in, int8_t *q, float *absmax_out, void *stream);

/* functional.py:542-600 dequantize_blockwise: out[i] = float(q[i]) * (absmax[i/bs] / 127). */
int mpsbnb_dequantize_blockwise(const int8_t *q, const float *absmax, int64_t n, int blocksize,
                                void *out, int out_dtype, void *stream);

/* ---------------------------------------------------------------------------------------
 * 4-bit fused dequantise-matmul:  y[M,N] = x[M,K] . W[N,K]^T (+ bias)
 * functional.py:680-773 matmul_4bit / matmul_nf4 / matmul_fp4.
 * Bindings replaced: _C.matmul_nf4 / _C.matmul_fp4 (mps_bitsandbytes.mm:2741-2743,
 * 2749-2751; host wrappers :1956-2032, :2099-2151).
 * x, bias in x_dtype (F16 or BF16); y in y_dtype; fp32 accumulation.
 * ------------------------------------------------------------------------------------- */

/* Decode shapes (M <= mpsbnb_gemv_4bit_max_m() = 32): weights streamed once from HBM.
 * Needs blocksize 64 (any K; Kp/2 bytes per row).  No workspace.
 * M <= 8: TMA ring + table expansion + dot products / mma.sync; 9 <= M <= 32: TMA ring + expansion
 * into tensor memory + tcgen05.mma (packed rows must be 16-byte aligned for both; otherwise, and
 * for unaligned rows, a direct-load kernel). */
int mpsbnb_gemv_4bit_max_m(void);
int mpsbnb_gemv_4bit(const void *x, int x_dtype, int64_t M, const uint8_t *packed,
                     const void *absmax, const float *absmax2, int64_t N, int64_t K,
                     int blocksize, int quant_type, const void *bias, void *y, int y_dtype,
                     void *stream);

/* Grouped decode GEMV: several 4-bit linears (block size 64, batch M <= mpsbnb_gemv_4bit_group_max_m()) in ONE launch of
 * a persistent kernel, e.g. the seven projections of a decoder layer.  Replaces a sequence
 * of _C.matmul_nf4 / _C.matmul_fp4 calls (mps_bitsandbytes.mm:2741-2751), which the
 * reference issues one Metal dispatch at a time.
 *   x        [M, x_ld] activations; column k of the product reads x[m, k mod x_period]
 *            (x_period = 0 means K: no wrap)
 *   y / acc  results are stored to y [M, N] (y_dtype), or — when acc != NULL — atomically
 *            added to the fp32 matrix acc [M, N] (several linears may share one acc; long
 *            K is then split across CTAs).  The caller zeroes acc.
 * A plan (device memory supplied by the caller, 256-byte aligned, size from
 * mpsbnb_gemv_4bit_group_plan_bytes) is built once and run any number of times. */
typedef struct mpsbnb_linear4_desc {
    const void *x;
    int64_t x_ld, x_period;
    const uint8_t *packed;
    const void *absmax;
    const float *absmax2;
    const void *bias;
    void *y;
    float *acc;
    int64_t N, K;
    int64_t segment;          /* 0, 1, 2 ...: linears of segment g + 1 read what the closing step of segment g wrote
                               * (several decoder layers in ONE launch); all 0 for an ordinary group */
} mpsbnb_linear4_desc;

/* Two kernels implement the decode path, chosen by the batch alone.  M <= 8: TMA ring, table
 * expansion, dot products (M <= 2) or mma.sync in the consumer warps.  9 <= M <= 32: TMA ring, table
 * expansion into tensor memory, tcgen05.mma with fp32 accumulators in tensor memory, stream-K work
 * split (a 16-column and a 32-column instance).  No reference counterpart. */
/* Largest batch M a group plan accepts (32). */
int mpsbnb_gemv_4bit_group_max_m(void);

/* Optional closing step of a grouped launch, run inside the kernel by the CTA that finishes last (so no
 * separate boundary kernel is needed): h_shard = alpha * acc (acc: fp32 [M, hs], re-armed to zero) is
 * stored into columns [rank * hs, (rank + 1) * hs) of every peer_h[r] ([M, H] in the activation dtype,
 * r < nranks; a device array of pointers, own buffer included; nranks = 1, hs = H on a single GPU), and
 * then, if peer_flags is not NULL, peer_flags[r][rank] = (*step) * mul + add for every r.
 * counter: a device int that is zero between launches.  acc == NULL: no closing step.
 * tile_cnt != NULL selects the streamed form instead: every 32-row tile of acc is converted, stored and
 * re-armed as soon as the last of its tile_expect contributions (plan.acc_parts: the units of all linears
 * that add into acc) has arrived — tile_cnt: hs / 32 device ints, zero between launches — and the flags
 * are raised after the last tile.  Linears with an accumulator are scheduled first in a launch, so this
 * happens early and the exchange hides behind the rest of the launch.  Because h of the NEXT layer is
 * then written while THIS layer is still reading its own h, peer_h must not be the buffer the launch reads
 * x from (rotate three buffers when ranks may run more than a layer apart; when all segments run in ONE launch and
 * some linears feed nothing that is waited for, give every segment its own buffer: a CTA may lag several segments).
 * Several segments in one launch (mpsbnb_linear4_desc.segment; streamed form only): the closing step of
 * segment g stores into buffer (g + 1) % nbuf — peer_h is then an array of nbuf * nranks pointers,
 * [buffer][rank] — and raises the flags to (*step) * mul + add + g; linears of segment g >= 1 wait
 * (plan.wait_*) until all flags are >= (*wait_step) * wait_mul + wait_add + g.  One accumulator and one
 * tile_cnt serve all segments (segment g + 1 cannot add before segment g is closed).  Such a launch is
 * cooperative: all its CTAs are resident, because CTAs wait for each other's closing steps. */
typedef struct mpsbnb_group_epilogue {
    float *acc;
    void *const *peer_h;
    int *const *peer_flags;
    const int *step;
    int *counter;
    int *tile_cnt;
    float alpha;
    int M, hs, H, rank, nranks, mul, add, tile_expect;
    int nbuf;                 /* buffers peer_h rotates over (0 or 1: a single one) */
    int count_tiles;          /* streamed closing step: 0 = the CTA that closes the shard's last tile SETS every rank's flag to
                               * step * mul + add + segment; 1 = every closed tile ADDS 1 to every rank's flag (no counter,
                               * no second fence: waiters then expect a multiple of the tiles per shard, see wait_seg_mul);
                               * 2 = no flags at all: peer_h are TAGGED buffers (8-byte entries {two values, tag}, tag =
                               * step * mul + add + segment) and every linear of the plan reads its x in that form, expecting
                               * the tag (*wait_step) * wait_mul + wait_add + segment * wait_seg_mul.  A linear then starts as
                               * soon as ITS columns carry the tag, so segments overlap: acc holds TWO accumulators
                               * [2][M][hs] and tile_cnt two sets of counts [2][ceil(hs / 32)], indexed by segment parity,
                               * and the accumulating linears of segment s point their acc at copy s & 1 */
} mpsbnb_group_epilogue;

typedef struct mpsbnb_group_plan {
    void *dev;
    int64_t units_offset;
    int n_linears, n_units, M, x_dtype, quant_type;
    int flags;               /* set by the caller before a run: MPSBNB_GROUP_PDL or 0 */
    int64_t aux_offset;      /* filled by the plan call: per-CTA table inside the plan memory */
    int grid, impl;          /* filled by the plan call: CTAs to launch, kernel family */
    /* Optional, set by the caller before a run (zero = off): before its first read of x the kernel waits,
     * for at most about a second, until each of the wait_n ints at wait_flags (memory of this GPU) is
     * >= (*wait_step) * wait_mul + wait_add.  Used with mpsbnb_stack_boundary_push on the other GPUs. */
    const int *wait_flags;
    const int *wait_step;
    int wait_n, wait_mul, wait_add;
    int acc_parts;            /* filled by the plan call: units per 32-row tile and segment that add into an accumulator */
    int n_segments;           /* filled by the plan call */
    int wait_seg_mul;         /* set by the caller: linears of segment g wait for (*wait_step) * wait_mul + wait_add + g * wait_seg_mul
                               * (0 is read as 1) */
    mpsbnb_group_epilogue ep; /* optional, set by the caller before a run (default kernel only) */
} mpsbnb_group_plan;

/* Launch with programmatic dependent launch: the kernel may start (build its tables, fetch
 * weights) while the previous kernel in the stream is still finishing, and waits for that
 * kernel before it reads x or writes results.  Use when the previous kernel produces x. */
#define MPSBNB_GROUP_PDL 1

size_t mpsbnb_gemv_4bit_group_plan_bytes(const mpsbnb_linear4_desc *descs, int n_linears);
/* Builds the plan (synchronises the stream once: it uploads the tables). */
int mpsbnb_gemv_4bit_group_plan(const mpsbnb_linear4_desc *descs, int n_linears, int64_t M, int x_dtype,
                                int y_dtype, int quant_type, void *plan_dev, size_t plan_bytes,
                                mpsbnb_group_plan *plan_out, void *stream);
int mpsbnb_gemv_4bit_group_run(const mpsbnb_group_plan *plan, void *stream);

/* Layer boundary of the synthetic decoder-layer stack used by the decode benchmark:
 *   h[m, j] = alpha * (o[m, j] + d[m, j])  for j < H,   e[m, j] = h[m, j mod H]  for j < F
 * (h: next layer's input; e: F-wide input of its down projection; e may be NULL).
 * No reference counterpart: the reference ships no model, only the linear layers. */
int mpsbnb_stack_boundary(const void *o, const void *d, int dtype, float alpha, int64_t M, int64_t H,
                          int64_t F, void *h, void *e, void *stream);

/* Boundary for the grouped path, where o and down were atomically accumulated into one fp32
 * matrix: h[i] = alpha * acc[i] (i < n, rounded to dtype) and acc[i] = 0.
 * No reference counterpart. */
int mpsbnb_stack_boundary_acc(float *acc, float alpha, int64_t n, void *h, int dtype, int flags,
                              void *stream);   /* flags: MPSBNB_GROUP_PDL or 0 */

/* Layer-boundary exchange of the N-sharded stack without a collective call (one process per GPU).
 * No reference counterpart (the reference is single-device).
 *  - mpsbnb_ipc_export / _open / _close: CUDA IPC plumbing for a buffer the CALLER allocated: export
 *    gives the 64-byte handle of the allocation containing dev_ptr and dev_ptr's offset in it; a peer
 *    process opens the handle (base address in its own address space, peer access enabled) and closes
 *    it when done.  A process cannot open its own handle.
 *  - mpsbnb_stack_boundary_push: h_shard = alpha * acc (acc: fp32 [M, hs], re-armed to zero) is stored
 *    into columns [rank * hs, (rank + 1) * hs) of peer_h[r] ([M, H], r = 0 .. nranks-1, own buffer
 *    included; device array of pointers) and then peer_flags[r][rank] = (*step) * mul + add for every r
 *    (device array of pointers to each rank's int[nranks] flag array).  One small kernel; hs % 8 == 0.
 *  - mpsbnb_flags_wait: a kernel that waits (bounded, status 502 on time-out) until flags[0..n) >=
 *    (*step) * mul + add: put it at the end of a step so that the host reads a complete h.
 *  - mpsbnb_flags_push: peer_flags[r][rank] = (*step) * mul + add for every r, without data (the
 *    end-of-step acknowledgement: "my h buffers may be overwritten again").
 *  - mpsbnb_counter_add: *counter += value on the stream (the step counter, inside a CUDA graph). */
int mpsbnb_ipc_export(const void *dev_ptr, void *handle64, int64_t *offset_out);
int mpsbnb_ipc_open(const void *handle64, void **base_out);
int mpsbnb_ipc_close(void *base);
int mpsbnb_stack_boundary_push(float *acc, float alpha, int64_t M, int64_t hs, int64_t H, int rank, int nranks,
                               void *const *peer_h, int *const *peer_flags, const int *step, int mul, int add,
                               int dtype, int flags, void *stream);
int mpsbnb_flags_wait(const int *flags, int n, const int *step, int mul, int add, int pdl, void *stream);
int mpsbnb_flags_push(int *const *peer_flags, int rank, int nranks, const int *step, int mul, int add, void *stream);
int mpsbnb_counter_add(int *counter, int value, void *stream);
/* Tagged form of a 16-bit matrix [M, H] (H even): 8-byte entries {columns 2p and 2p+1, tag}, what the decode kernel's
 * closing step exchanges when ep.count_tiles == 2 (an aligned 8-byte store arrives whole, so a reader that sees the tag has
 * the data: no fence, no flag).  mpsbnb_tagged_write converts a plain matrix with tag (*step) * mul + add (a stack's input);
 * mpsbnb_tagged_read waits - bounded, then device status 502 - until every entry carries that tag and returns the plain
 * matrix (a stack's result).  No reference counterpart. */
int mpsbnb_tagged_write(const void *x, int64_t M, int64_t H, void *tagged, const int *step, int mul, int add, void *stream);
int mpsbnb_tagged_read(const void *tagged, int64_t M, int64_t H, void *out, const int *step, int mul, int add, void *stream);

/* Multi-GPU form of the boundary: G[r][m][c] holds the all-gathered per-rank shards of the
 * new h (c < H / nranks); writes h[m, r*H/nranks + c] = G[r][m][c] and e as above.
 * No reference counterpart (the reference is single-device). */
int mpsbnb_stack_expand(const void *G, int dtype, int64_t nranks, int64_t M, int64_t H, int64_t F,
                        void *h, void *e, void *stream);

/* functional.py:680-773 matmul_4bit on prefill shapes (any M); the reference's Metal analogue
 * dequantises inside the GEMM's K loop (nf4_matmul_large, mps_bitsandbytes.mm:567-696).
 * Block size 64 (packed 16-byte aligned): ONE fused kernel - packed bytes by TMA, expanded in
 * shared memory, tcgen05 MMA; no 16-bit copy of the weight exists.  The workspace then only
 * holds a re-pitched copy of x when K % 8 != 0 or x is not 16-byte aligned.  Other block sizes:
 * W is dequantised into the workspace in x_dtype and multiplied by the plain tcgen05 GEMM.
 * workspace must hold mpsbnb_gemm_4bit_workspace_bytes(...) bytes, 256-B aligned, non-NULL. */
size_t mpsbnb_gemm_4bit_workspace_bytes(int64_t M, int64_t N, int64_t K, int blocksize);
int mpsbnb_gemm_4bit(const void *x, int x_dtype, int64_t M, const uint8_t *packed,
                     const void *absmax, const float *absmax2, int64_t N, int64_t K,
                     int blocksize, int quant_type, const void *bias, void *y, int y_dtype,
                     void *workspace, size_t workspace_bytes, void *stream);

/* mpsbnb_gemm_4bit without a workspace argument and without any allocation: the expanded
 * weight goes into a fixed 32 MiB array inside the library's device image, shared by all
 * calls on a device.  No counterpart in the reference (whose wrappers allocate from the
 * PyTorch allocator on every call); it exists for hosts that own all device memory
 * themselves and cannot provide a workspace.
 *  - Limit: mpsbnb_gemm_4bit_static_bytes(x, M, N, K) <= mpsbnb_gemm_4bit_static_max_bytes()
 *    (N * roundup8(K) * 2 bytes, plus M * roundup8(K) * 2 when K % 8 != 0 or x is not
 *    16-byte aligned); larger problems return MPSBNB_ERR_TOO_LARGE and enqueue nothing.
 *  - The first call on each device resolves the array's address (set-up, not a stream
 *    operation): make it before any stream capture that will hold later calls.
 *  - Calls that may overlap in time on different streams of one device race on the array;
 *    same-stream calls are ordered.  Nothing in the array needs to start at zero.
 *  - The resolved address is cached per device.  After cudaDeviceReset() the context it
 *    belonged to is gone: call mpsbnb_gemm_4bit_static_forget() so that the next call
 *    resolves it again.
 * The weight is expanded into the array and multiplied by the plain tcgen05 GEMM; results agree
 * with mpsbnb_gemm_4bit within the matmul tolerance (1e-2; measured ~5e-4) and repeat exactly. */
void mpsbnb_gemm_4bit_static_forget(void);
size_t mpsbnb_gemm_4bit_static_max_bytes(void);
size_t mpsbnb_gemm_4bit_static_bytes(const void *x, int64_t M, int64_t N, int64_t K);
int mpsbnb_gemm_4bit_static(const void *x, int x_dtype, int64_t M, const uint8_t *packed,
                            const void *absmax, const float *absmax2, int64_t N, int64_t K,
                            int blocksize, int quant_type, const void *bias, void *y,
                            int y_dtype, void *stream);

/* Dense tensor-core GEMM y[M,N] = a[M,K] . b[N,K]^T (+ bias), both operands K-major in
 * ab_dtype (F16/BF16) with leading dimensions lda / ldb in elements (multiples of 8, bases
 * 16-byte aligned: TMA row pitches), fp32 accumulation in tensor memory.  Building block of
 * the prefill paths above and below; stands for torch.nn.functional.linear at
 * functional.py:767, 806, 944.  Optional epilogue: y = acc * row_scale[m] * col_scale[n] + bias[n]
 * (bias in ab_dtype).  K must be > 0. */
int mpsbnb_gemm_f16(const void *a, int64_t lda, const void *b, int64_t ldb, int ab_dtype, int64_t M,
                    int64_t N, int64_t K, const float *row_scale, const float *col_scale,
                    const void *bias, void *y, int y_dtype, void *stream);

/* Device-side status word of the current device: 0, or the code of the bounded wait that
 * ran out inside a kernel (kernels never trap or spin forever; they record and return).
 * Synchronises the device.  reset != 0 clears the word.  No reference counterpart: the
 * reference reports Metal pipeline failures as exceptions (mps_bitsandbytes.mm:1739-1771). */
int mpsbnb_device_status(int *status_out, int reset);

/* ---------------------------------------------------------------------------------------
 * INT8 row-wise, col+row, LLM.int8 statistics
 * ------------------------------------------------------------------------------------- */

/* functional.py:607-625 quantize_rowwise: q int8 [rows, cols], scales fp32 [rows] = row absmax. */
int mpsbnb_quantize_rowwise(const void *x, int x_dtype, int64_t rows, int64_t cols, int8_t *q,
                            float *scales, void *stream);
/* functional.py:628-636 dequantize_rowwise: out = float(q) * (scales[row] / 127). */
int mpsbnb_dequantize_rowwise(const int8_t *q, const float *scales, int64_t rows, int64_t cols,
                              void *out, int out_dtype, void *stream);
/* functional.py:814-863 double_quant: row- and column-quantised int8 copies with their
 * statistics.  row_stats_in / col_stats_in optional (else computed and written to *_out). */
int mpsbnb_double_quant(const void *A, int a_dtype, int64_t rows, int64_t cols,
                        const float *row_stats_in, const float *col_stats_in, int8_t *out_row,
                        int8_t *out_col, float *row_stats_out, float *col_stats_out, void *stream);
/* functional.py:866-889 dequant_absmax (tensor form): out[r, b] = float(q[r, b]) * scales[r, b / blocksize],
 * q int8 [rows, nblk], scales fp32 [rows, ndq] with ndq >= ceil(nblk / blocksize), out fp32 [rows, nblk].
 * (No division by 127: the reference multiplies by the stored scale as it is.) */
int mpsbnb_dequant_absmax(const int8_t *q, const float *scales, int64_t rows, int64_t nblk, int64_t ndq,
                          int blocksize, float *out, void *stream);
/* functional.py:896-924 quantize_colrow: q = round(W * 127 / sqrt(r[n] c[k])). */
int mpsbnb_quantize_colrow(const void *W, int w_dtype, int64_t rows, int64_t cols, int8_t *q,
                           float *row_absmax, float *col_absmax, void *stream);
/* functional.py:927-932 dequantize_colrow. */
int mpsbnb_dequantize_colrow(const int8_t *q, const float *row_scales, const float *col_scales,
                             int64_t rows, int64_t cols, void *out, int out_dtype, void *stream);

/* functional.py:788-793 matmul_int8; binding replaced: _C.matmul_int8
 * (mps_bitsandbytes.mm:2730-2732, kernel int8_matmul_dequant :155-196).
 *   A int8 [M,K] with a_scales [M]; B int8 [K,N] (N contiguous) with b_scales [N];
 *   y [M,N] = sum_k A B * a_scales[m] * b_scales[n] / 127^2, in y_dtype.
 * workspace: mpsbnb_matmul_int8_workspace_bytes(M,N,K) bytes. */
size_t mpsbnb_matmul_int8_workspace_bytes(int64_t M, int64_t N, int64_t K);
int mpsbnb_matmul_int8(const int8_t *A, const int8_t *B, const float *a_scales,
                       const float *b_scales, int64_t M, int64_t N, int64_t K, void *y,
                       int y_dtype, void *workspace, size_t workspace_bytes, void *stream);

/* functional.py:935-945 matmul_colrow and nn/linear8bit.py:91-102 (W8A16 with col_scales
 * == NULL: plain row-wise weights); binding replaced: _C.linear_int8
 * (mps_bitsandbytes.mm:2733-2735).  x [M,K] x_dtype, W int8 [N,K]. */
size_t mpsbnb_linear_int8_workspace_bytes(int64_t M, int64_t N, int64_t K);
int mpsbnb_linear_int8(const void *x, int x_dtype, int64_t M, const int8_t *W,
                       const float *row_scales, const float *col_scales, int64_t N, int64_t K,
                       const void *bias, void *y, int y_dtype, void *workspace,
                       size_t workspace_bytes, void *stream);

/* nn/outlier_aware.py:84-146 OutlierAwareLinear.forward (LLM.int8 mixed-precision decomposition):
 *   y = deq(quantize_rowwise(x_main)) . deq(W_main)^T + x_outlier . outlier_w^T + bias
 * with x_main / W_main the columns NOT listed in outlier_idx, both dequantised as
 * q.to(op) * (scale / 127).to(op) (:118-119, :138-139).  The reference has no native binding for
 * it (three Python matmuls); here the re-quantised x, the dequantised W and the 16-bit outlier
 * columns form the two operands of ONE tcgen05 GEMM over the full K.
 *   x           [M, K] in x_dtype (F16, BF16 or F32)
 *   W, w_scales int8 [N, K] (entries in outlier columns are ignored), fp32 [N] row maxima
 *   outlier_idx int64 [n_outliers] distinct column numbers (may be NULL when n_outliers == 0:
 *               the pure INT8 path, :112-121); outlier_w [N, n_outliers] in op_dtype
 *   bias        NULL or [N] in op_dtype; op_dtype F16 or BF16 (the module's compute_dtype)
 *   y           [M, N] in y_dtype
 * workspace: mpsbnb_outlier_linear_workspace_bytes(M, N, K) bytes, 256-byte aligned. */
size_t mpsbnb_outlier_linear_workspace_bytes(int64_t M, int64_t N, int64_t K);
int mpsbnb_outlier_linear(const void *x, int x_dtype, int64_t M, const int8_t *W, const float *w_scales,
                          const int64_t *outlier_idx, int64_t n_outliers, const void *outlier_w,
                          int64_t N, int64_t K, const void *bias, int op_dtype, void *y, int y_dtype,
                          void *workspace, size_t workspace_bytes, void *stream);

/* ---------------------------------------------------------------------------------------
 * Quantised embedding look-ups (gather + dequantise in one pass)
 * ------------------------------------------------------------------------------------- */

/* nn/embedding.py:78-139 Embedding4bit.forward; bindings replaced: _C.embedding_4bit_nf4 /
 * _C.embedding_4bit_fp4 (:94-101).  out[t, :] = code[nibble] * absmax[row, k / blocksize] for
 * row = indices[t], computed in fp32 and rounded once (functional.py:388-416 on one row).
 *   indices   int32 (index_bytes 4) or int64 (index_bytes 8) [n_indices]
 *   packed    uint8 [num_embeddings, packed_ld] (packed_ld >= dim / 2 bytes per row; dim even)
 *   absmax    fp32 [num_embeddings, ceil(dim / blocksize)]
 *   padding_idx  rows with this index give zeros (:135-137); negative = none
 *   out       [n_indices, dim] in out_dtype
 * An index outside [0, num_embeddings) gives a zero row (the kernel neither faults nor raises;
 * the Python path of the reference raises IndexError). */
int mpsbnb_embedding_4bit(const void *indices, int index_bytes, int64_t n_indices, const uint8_t *packed,
                          int64_t packed_ld, const float *absmax, int64_t num_embeddings, int64_t dim,
                          int blocksize, int quant_type, int64_t padding_idx, void *out, int out_dtype,
                          void *stream);
/* nn/embedding.py:244-275 Embedding8bit.forward; binding replaced: _C.embedding_8bit (:252-256).
 * out[t, k] = T(q[row, k]) * T(scales[row] / 127), the scale rounded to out_dtype first (:269).
 *   q int8 [num_embeddings, dim], scales fp32 [num_embeddings]; other arguments as above. */
int mpsbnb_embedding_8bit(const void *indices, int index_bytes, int64_t n_indices, const int8_t *q,
                          const float *scales, int64_t num_embeddings, int64_t dim, int64_t padding_idx,
                          void *out, int out_dtype, void *stream);

/* ---------------------------------------------------------------------------------------
 * FP8 E4M3 (row-scaled)
 * ------------------------------------------------------------------------------------- */

/* functional.py:643-663 -> :1086-1163; binding replaced: _C.quantize_fp8_e4m3
 * (mps_bitsandbytes.mm:2754), with the Python encoder's rounding (not the Metal one). */
int mpsbnb_quantize_fp8_e4m3(const void *x, int x_dtype, int64_t rows, int64_t cols,
                             uint8_t *codes, float *scales, void *stream);
/* functional.py:666-673 -> :1166-1216; binding replaced: _C.dequantize_fp8_e4m3 (:2755-2756). */
int mpsbnb_dequantize_fp8_e4m3(const uint8_t *codes, const float *scales, int64_t rows,
                               int64_t cols, void *out, int out_dtype, void *stream);
/* functional.py:796-807 matmul_fp8_e4m3; binding replaced: _C.matmul_fp8_e4m3 (:2757-2759). */
size_t mpsbnb_linear_fp8_workspace_bytes(int64_t M, int64_t N, int64_t K);
int mpsbnb_linear_fp8_e4m3(const void *x, int x_dtype, int64_t M, const uint8_t *codes,
                           const float *scales, int64_t N, int64_t K, const void *bias, void *y,
                           int y_dtype, void *workspace, size_t workspace_bytes, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* MPSBNB_B200_H */
