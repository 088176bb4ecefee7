/*
 * b200fp8 — C ABI of the B200 (sm_100a) block-FP8 hot path.
 *
 * The library replaces the device side of the reference package
 * finegrained-fp8-helion (AmesingFlank/hf_kernels_helion):
 *
 *   finegrained-fp8-helion/finegrained-fp8-helion/torch-ext/finegrained_fp8_helion/fp8.py:19-39
 *       the Helion kernel `_w8a8_block_fp8_matmul`            -> b200fp8_gemm
 *   .../torch-ext/finegrained_fp8_helion/__init__.py:14
 *       the separate `.to(output_dtype)` pass                 -> folded into b200fp8_gemm (out_dtype)
 *   per-token-group activation quantiser (absent from the reference, defined by
 *       the benchmark configuration text: scale = group amax / 448, e4m3 cast) -> b200fp8_quant_act
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless the name says host;
 *   - leading dimensions (ld*) are in ELEMENTS of the tensor they belong to;
 *   - no function allocates, frees or synchronises; kernels are enqueued on
 *     `stream` (a cudaStream_t passed as void*, NULL = legacy default stream);
 *   - every function returns a b200fp8_status (0 = ok) and never throws;
 *   - `status_word` (may be NULL) is a device uint32 the kernels write a non-zero
 *     code into when a bounded device-side wait gives up; the caller reads it
 *     after synchronising the stream.
 */
#ifndef B200FP8_H_
#define B200FP8_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum b200fp8_status {
  B200FP8_OK = 0,
  B200FP8_ERR_NULL = 1,       /* a required pointer is NULL */
  B200FP8_ERR_SHAPE = 2,      /* M, N or K is negative, or a leading dimension is too small */
  B200FP8_ERR_ALIGN = 3,      /* pointer or leading dimension breaks a 16-byte rule */
  B200FP8_ERR_DTYPE = 4,      /* out_dtype is not one of B200FP8_OUT_* */
  B200FP8_ERR_VARIANT = 5,    /* unknown variant, or variant cannot run this shape */
  B200FP8_ERR_WORKSPACE = 6,  /* workspace missing or smaller than b200fp8_gemm_workspace_bytes */
  B200FP8_ERR_ARCH = 7,       /* current device is not compute capability 10.x */
  B200FP8_ERR_DRIVER = 8,     /* cuTensorMapEncodeTiled unavailable or rejected the tensor */
  B200FP8_ERR_LAUNCH = 9,     /* the CUDA runtime refused the launch (see cudaGetLastError) */
  B200FP8_ERR_TOO_LARGE = 10  /* request exceeds a fixed capacity of the entry point */
} b200fp8_status;

/* out_dtype of b200fp8_gemm */
#define B200FP8_OUT_BF16 0
#define B200FP8_OUT_FP32 1

/* variant of b200fp8_gemm */
#define B200FP8_VARIANT_AUTO 0    /* pick by shape */
#define B200FP8_VARIANT_TILE128 1 /* persistent tcgen05 kernel, 128x128 output tiles */
#define B200FP8_VARIANT_TILE256 2 /* persistent tcgen05 kernel, 128x256 output tiles */
#define B200FP8_VARIANT_STREAMK 3 /* swap-AB stream-K kernel for M <= 256 (decode shapes) */
#define B200FP8_VARIANT_TILE256_SK 4 /* 128x256 tiles; the tiles of the last, partly empty wave are split along K over the idle SMs */
#define B200FP8_VARIANT_PAIR256 5 /* 256x256 tiles on CTA pairs (tcgen05 cta_group::2), each SM holds half of the B tile */
#define B200FP8_VARIANT_PAIR256_SPLIT 6 /* same, every K block issued and promoted as two 128-column halves */
#define B200FP8_VARIANT_PAIR256_SPLIT_SK 7 /* same as 6, the pair tiles of the last, partly empty wave split along K over the idle pairs */

/* codes a kernel may leave in *status_word */
#define B200FP8_DEV_OK 0u
#define B200FP8_DEV_WAIT_TIMEOUT 1u /* an mbarrier wait exceeded its time limit; output is invalid */

/* Library version, major*10000 + minor*100 + patch. */
int b200fp8_version(void);

/* Static English description of a status code. Never NULL. */
const char* b200fp8_strerror(int status);

/*
 * Per-token-group activation quantiser (no counterpart function in the reference;
 * it is the producer of the A / As arguments of
 * torch-ext/finegrained_fp8_helion/__init__.py:7-11).
 *
 *   x  [M, K] bf16, row stride ldx          (read)
 *   q  [M, K] float8_e4m3fn, row stride ldq (written)
 *   s  [M, ceil(K/128)] fp32, row stride lds (written)
 *
 * For every row and every 128-wide group along K:
 *   amax = max |x|, s = amax / 448 (fp32 IEEE division), q = e4m3_rne(x / s);
 *   an all-zero group gives s = 0 and q = 0. A ragged last group (K % 128 != 0)
 *   takes its amax over the elements that exist.
 * Requires K % 8 == 0, ldx % 8 == 0, ldq % 8 == 0 and x, q 16- and 8-byte aligned.
 */
int b200fp8_quant_act(const void* x, void* q, float* s,
                      int64_t M, int64_t K,
                      int64_t ldx, int64_t ldq, int64_t lds,
                      void* stream);

/*
 * 128x128-block weight quantiser (generator side of the path; no counterpart in
 * the reference, whose callers receive B / Bs ready-made:
 * torch-ext/finegrained_fp8_helion/__init__.py:9-11).
 *
 *   w  [N, K] bf16, row stride ldw            (read)
 *   q  [N, K] float8_e4m3fn, row stride ldq   (written)
 *   s  [ceil(N/128), ceil(K/128)] fp32, row stride lds (written)
 * Same arithmetic as b200fp8_quant_act with the amax taken over a 128x128 block.
 */
int b200fp8_quant_weight(const void* w, void* q, float* s,
                         int64_t N, int64_t K,
                         int64_t ldw, int64_t ldq, int64_t lds,
                         void* stream);

/*
 * Block-FP8 W8A8 GEMM, C = A . B^T with per-block fp32 scales
 * (replaces torch-ext/finegrained_fp8_helion/fp8.py:19-39 and the dtype cast of
 * torch-ext/finegrained_fp8_helion/__init__.py:14).
 *
 *   A  [M, K] float8_e4m3fn, row stride lda        B  [N, K] float8_e4m3fn, row stride ldb
 *   As [M, ceil(K/128)] fp32, row stride ld_as     Bs [ceil(N/128), ceil(K/128)] fp32, row stride ld_bs
 *   C  [M, N] bf16 (B200FP8_OUT_BF16) or fp32 (B200FP8_OUT_FP32), row stride ldc
 *
 *   C[m, n] = sum over 128-wide K blocks kb of
 *             dot(A[m, kb], B[n, kb]) * As[m, kb] * Bs[n / 128, kb]       (fp32 accumulate)
 *
 * Requires lda % 16 == 0, ldb % 16 == 0, A and B 16-byte aligned (TMA rules);
 * M, N, K otherwise arbitrary (ragged edges are masked). M == 0 or N == 0 is a
 * no-op; K == 0 writes zeros.
 *
 * `workspace` holds per-call scratch (a K-block-major copy of As for every variant, plus
 * the fp32 partial tiles of B200FP8_VARIANT_STREAMK); size it with
 * b200fp8_gemm_workspace_bytes for the same (M, N, K, variant), align it to 256 bytes. Its
 * contents need no initialisation.
 */
int b200fp8_gemm(const void* A, const void* B, const float* As, const float* Bs, void* C,
                 int64_t M, int64_t N, int64_t K,
                 int64_t lda, int64_t ldb, int64_t ld_as, int64_t ld_bs, int64_t ldc,
                 int out_dtype, int variant,
                 void* workspace, size_t workspace_bytes,
                 uint32_t* status_word, void* stream);

/*
 * b200fp8_gemm writing the same [M, N] result into n_dst (1..8) buffers, C_dst[0] being the
 * caller's own. No counterpart in the reference (which has no multi-GPU code); it is the
 * compute + exchange step of the N-sharded layout derived from
 * torch-ext/finegrained_fp8_helion/fp8.py:30-36: every GPU computes its column slice and
 * stores it straight into the full-width output buffer of every GPU of the node, so that no
 * separate all-gather pass is needed. C_dst[d] points at the first element of THIS call's
 * column slice inside destination d (a peer buffer opened with b200fp8_ipc_open, plus the
 * slice's column offset), ldc_dst[d] is that buffer's row pitch in elements.
 * Each finished 32-row x 128-byte box is staged in shared memory and sent to every
 * destination with an asynchronous TMA store (remote ones cross NVLink) while the following
 * tiles compute; no TMA load ever touches peer memory. Every C_dst[d] must be 16-byte aligned, ldc_dst[d] and N multiples
 * of 16 bytes worth of elements; only the tile variants (or AUTO resolving to one) are
 * allowed. The stores are complete when the kernel is; the caller synchronises the GPUs
 * (stream order + a barrier between ranks) before any of them reads its buffer.
 */
int b200fp8_gemm_scatter(const void* A, const void* B, const float* As, const float* Bs,
                         int n_dst, void* const* C_dst, const int64_t* ldc_dst,
                         int64_t M, int64_t N, int64_t K,
                         int64_t lda, int64_t ldb, int64_t ld_as, int64_t ld_bs,
                         int out_dtype, int variant,
                         void* workspace, size_t workspace_bytes,
                         uint32_t* status_word, void* stream);

/*
 * The same GEMM with one B scale per ROW of B and K block: Bs_row is [N, ceil(K/128)] fp32
 * (row pitch ld_bs), everything else as b200fp8_gemm. This is the operand layout of the
 * reference's second block-FP8 kernel, deep-gemm-helion
 * (deep-gemm-helion/deep-gemm-helion/torch-ext/deep_gemm_helion/fp8.py:13-29:
 * acc += dot(a, b^T) * sA[m, kb][:, None] * sB[n, kb][None, :], bf16 result;
 * torch-ext/deep_gemm_helion/op.py:7-10). Runs on the 128 x 128 tile kernel; the promotion
 * multiplies every accumulator column by its own scale (one multiply more per element than
 * the block-scaled form). Workspace: b200fp8_gemm_rowscale_workspace_bytes(M, N, K) bytes,
 * 256-byte aligned (both scale sets re-laid K-block-major).
 */
int b200fp8_gemm_rowscale(const void* A, const void* B, const float* As, const float* Bs_row, void* C,
                          int64_t M, int64_t N, int64_t K,
                          int64_t lda, int64_t ldb, int64_t ld_as, int64_t ld_bs, int64_t ldc,
                          int out_dtype,
                          void* workspace, size_t workspace_bytes,
                          uint32_t* status_word, void* stream);
int64_t b200fp8_gemm_rowscale_workspace_bytes(int64_t M, int64_t N, int64_t K);

/*
 * Quantise-then-multiply in one call: C = e4m3_quant(x) . B^T with the activations given as
 * bf16 [M, K] (row pitch ldx elements). The caller of the reference quantises its activations
 * before the op (scripts/rebench_llm.py:130-133 builds A and As first); here the first launch
 * quantises x with the arithmetic of b200fp8_quant_act and leaves the e4m3 rows and the
 * K-block-major scales directly in the layout the GEMM kernel reads (inside `workspace`), the
 * GEMM follows with programmatic dependent launch. Two launches instead of three, no
 * separate q / scale tensors, and the result is bit-identical to b200fp8_quant_act followed
 * by b200fp8_gemm. K must be a multiple of 128, x 16-byte aligned, ldx a multiple of 8; only
 * the tile variants (or AUTO). Workspace: b200fp8_linear_workspace_bytes(M, N, K, variant)
 * bytes (about M*K + 4*M*K/128), 256-byte aligned.
 */
int b200fp8_linear(const void* x_bf16, const void* B, const float* Bs, void* C,
                   int64_t M, int64_t N, int64_t K,
                   int64_t ldx, int64_t ldb, int64_t ld_bs, int64_t ldc,
                   int out_dtype, int variant,
                   void* workspace, size_t workspace_bytes,
                   uint32_t* status_word, void* stream);
int64_t b200fp8_linear_workspace_bytes(int64_t M, int64_t N, int64_t K, int variant);

/*
 * b200fp8_gemm whose result goes to a multimem (NVLink multicast) address: C_multimem is the
 * multicast view of one buffer that exists on every GPU of a multicast group (cuMulticast* /
 * torch symmetric memory rendezvous), offset to the first element of THIS call's column
 * slice; ldc is the buffer's row pitch in elements. Each 128-byte row segment of a finished
 * tile is written once with multimem.st and the NVSwitch replicates it into all GPUs' copies,
 * this GPU's included, so a GPU sends its slice once instead of once per peer. No counterpart
 * in the reference. Same alignment rules, variants and completion semantics as
 * b200fp8_gemm_scatter; the library cannot check that the address is a multimem address.
 */
int b200fp8_gemm_multicast(const void* A, const void* B, const float* As, const float* Bs,
                           void* C_multimem,
                           int64_t M, int64_t N, int64_t K,
                           int64_t lda, int64_t ldb, int64_t ld_as, int64_t ld_bs, int64_t ldc,
                           int out_dtype, int variant,
                           void* workspace, size_t workspace_bytes,
                           uint32_t* status_word, void* stream);

/*
 * Barrier between the n (<= 8) GPUs of a node that follow a b200fp8_gemm_scatter with one another's
 * reads: flag_arrays[p] is GPU p's array of n 32-bit flags (zero at start; the caller's own
 * for p == rank, the others mapped with b200fp8_ipc_open), epoch a number that grows by one
 * per barrier, the same on every GPU. The kernel (one warp, enqueued on `stream` behind the GEMM)
 * publishes `epoch` to every GPU and waits until every GPU has published it; work enqueued
 * behind it may read the buffers the peers wrote. The wait is bounded (about 10 s); on expiry
 * B200FP8_DEV_WAIT_TIMEOUT is set in the status word. Each GPU of the group must run its own
 * process's call on its own device: the kernels wait for one another. No counterpart in the
 * reference.
 */
int b200fp8_peer_barrier(uint32_t* const* flag_arrays, int n, int rank, uint32_t epoch,
                         uint32_t* status_word, void* stream);

/*
 * The same barrier with the caller's own bound on the wait, in SM clocks (>= 1): for callers that
 * know their ranks are in step and want a lost peer reported within milliseconds, and for testing
 * the time-out path without a peer (n = 2 with both flag arrays local and the second slot never
 * published: the kernel returns after `limit_clocks` with B200FP8_DEV_WAIT_TIMEOUT in the status
 * word; nothing faults). No counterpart in the reference.
 */
int b200fp8_peer_barrier_limited(uint32_t* const* flag_arrays, int n, int rank, uint32_t epoch,
                                 int64_t limit_clocks, uint32_t* status_word, void* stream);

/*
 * CUDA IPC helpers for b200fp8_gemm_scatter (no counterpart in the reference). export: a
 * 64-byte handle of the device allocation that contains ptr, and ptr's byte offset inside it;
 * the handle travels to the other process by any host channel. open: maps that allocation
 * into the calling process with the CURRENT device as the accessing GPU (peer access is
 * enabled on demand) and returns its base; close unmaps it.
 */
int b200fp8_ipc_export(const void* ptr, void* handle_out_64, int64_t* offset_out);
int b200fp8_ipc_open(const void* handle_64, void** base_out);
int b200fp8_ipc_close(void* base);

/* Bytes of workspace b200fp8_gemm needs for this call (0 when none). Negative = error status, negated. */
int64_t b200fp8_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int variant);

/* The variant B200FP8_VARIANT_AUTO resolves to for this shape on the current device. */
int b200fp8_gemm_pick_variant(int64_t M, int64_t N, int64_t K);

/*
 * How many CTA pairs (clusters of two, one CTA per SM) of the B200FP8_VARIANT_PAIR256* kernels the
 * current device can hold at once: the persistent grid of those kernels. 0 = the device cannot run
 * them. (The reference's counterpart is the `num_sm_multiplier` / persistent-grid choice inside its
 * tuned Helion configs, torch-ext/finegrained_fp8_helion/_helion_aot_fp8_cuda_sm100.py:13-28.)
 */
int b200fp8_gemm_pair_clusters(void);

/*
 * Decode-shape GEMM for callers that must not allocate device memory. No counterpart in the
 * reference (there every call allocates through torch).
 *
 * Who needs it: code that runs where cudaMalloc is off limits - an inference server that
 * handed all of HBM to its own pool at start-up, a real-time loop that cannot afford the
 * device-wide synchronisation cudaMalloc/cudaFree imply, or a host layer that simply has no
 * allocator to give this library a workspace from. b200fp8_gemm's stream-K variant needs an
 * fp32 workspace from its caller; this entry point runs the same three kernels with the
 * workspace in a fixed array inside the library image instead.
 *
 * Same arguments and result as b200fp8_gemm(..., variant = B200FP8_VARIANT_STREAMK) without
 * the workspace pair. It calls no cudaMalloc, cudaFree or other allocating routine.
 *
 * Limits and rules:
 *   - the array is B200FP8_STATIC_SCRATCH_BYTES (4 MiB) per GPU that loads the library, held
 *     until the process exits; a call whose workspace need
 *     (b200fp8_gemm_workspace_bytes(M, N, K, B200FP8_VARIANT_STREAMK)) is larger returns
 *     B200FP8_ERR_TOO_LARGE - once N * K is large enough to occupy all 148 SMs of a B200 that
 *     means M <= 16 tokens (smaller problems with more tokens fit as well);
 *     K == 0 is rejected with B200FP8_ERR_SHAPE;
 *   - the first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current); make that first call outside any
 *     stream capture;
 *   - all calls on a device share the one array, which keeps the previous call's contents
 *     (nothing in it needs zeroing, every word read is written earlier in the same call):
 *     two calls whose kernels can overlap on the GPU - different streams, no dependency -
 *     race on it. Keep calls on one stream or order them with events.
 */
#define B200FP8_STATIC_SCRATCH_BYTES (4u << 20)
int b200fp8_gemm_decode_static(const void* A, const void* B, const float* As, const float* Bs, void* C,
                               int64_t M, int64_t N, int64_t K,
                               int64_t lda, int64_t ldb, int64_t ld_as, int64_t ld_bs, int64_t ldc,
                               int out_dtype, uint32_t* status_word, void* stream);

/*
 * Work partition of the stream-K variant, exposed for tests and tools (no counterpart
 * in the reference). `total` (weight tile, K block) units are spread over `grid` CTAs in
 * contiguous ranges: CTA c owns units [first_unit(c), first_unit(c + 1)).
 * b200fp8_streamk_grid returns the CTA count b200fp8_gemm would use on the current device
 * (or on a 148-SM B200 when no device is present).
 */
int64_t b200fp8_streamk_first_unit(int64_t cta, int64_t total, int64_t grid);
int64_t b200fp8_streamk_owner(int64_t unit, int64_t total, int64_t grid);
int64_t b200fp8_streamk_grid(int64_t M, int64_t N, int64_t K);

#ifdef __cplusplus
}
#endif
#endif /* B200FP8_H_ */
