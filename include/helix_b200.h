/*
 * helix_b200.h -- C ABI of libhelix_b200.so.
 *
 * The Helix reference has no FFI: its host<->kernel boundary is "spawn an nvcc
 * built executable with `M N K` on argv and parse one stdout line"
 * (scripts/Ampere_FP16/Ampere_FP16_gemm.py:432-441, src_template/Ampere_FP16/
 * gemm.cu:661-692).  Each entry point below replaces one of those executables
 * (or the Python loop around it) with an in-process call; the comment above
 * every declaration names the reference interface it stands in for.
 *
 * Conventions
 *   - every function returns HELIX_OK (0) or a negative helix_status_t; nothing
 *     throws, exits or traps the GPU;
 *   - the caller owns every buffer (inputs, outputs, workspace and the optional
 *     4-byte device status word); pointers are device pointers unless the name
 *     says host;
 *   - work is queued on the current CUDA device and on the stream passed as
 *     `stream` (a cudaStream_t cast to void*; NULL = default stream), and is
 *     asynchronous except for the helix_time_* and helix_*_host functions;
 *   - `status_dev`, when not NULL, points to a zero-initialised int in device
 *     memory; a kernel whose bounded wait ran out stores HELIX_ERR_TIMEOUT
 *     there and returns instead of spinning for ever.
 */
#ifndef HELIX_B200_H_
#define HELIX_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum helix_status {
  HELIX_OK = 0,
  HELIX_ERR_INVALID = -1,     /* bad argument (negative extent, NULL pointer, unknown op) */
  HELIX_ERR_ALIGN = -2,       /* pointer or leading dimension violates the 16-byte rule   */
  HELIX_ERR_WORKSPACE = -3,   /* workspace missing or smaller than helix_workspace_bytes  */
  HELIX_ERR_CUDA = -4,        /* a CUDA runtime / driver call failed                      */
  HELIX_ERR_TIMEOUT = -5,     /* a bounded device-side wait ran out (status word only)    */
  HELIX_ERR_UNSUPPORTED = -6, /* configuration not built into the library                 */
  HELIX_ERR_NODEVICE = -7,    /* no sm_100 device is current                              */
  HELIX_ERR_CAPACITY = -8     /* problem larger than a fixed built-in buffer can hold     */
} helix_status_t;

typedef enum helix_op {
  HELIX_OP_GEMM_F16 = 0, /* tcgen05 tensor-core GEMM, fp16 in, fp32 accumulate, fp16 out  */
  HELIX_OP_GEMV_F16 = 1, /* memory-bound SIMT GEMV for 1..8 right-hand sides              */
  HELIX_OP_CONV_F16 = 2, /* implicit-GEMM NHWC convolution on the same tensor-core path   */
  HELIX_OP_GEMM_F32 = 3, /* SIMT FFMA GEMM, true fp32                                     */
  HELIX_OP_CONV_F32 = 4, /* true-fp32 NHWC convolution: column matrix + the FFMA GEMM      */
  HELIX_OP_GEMV_F32 = 5  /* true-fp32 memory-bound GEMV for 1..8 right-hand sides          */
} helix_op_t;

/* Replaces the queried-nowhere literal `108` (A100 SM count) of the reference's
 * cost models (scripts/Ampere_FP16/Ampere_FP16_gemm.py:425 and 11 more sites). */
typedef struct helix_devinfo {
  int sm_count;
  int cc_major, cc_minor;
  int clock_khz, mem_clock_khz;
  int64_t l2_bytes;
  int64_t smem_per_sm;
  int64_t smem_per_block_optin;
  int64_t total_mem;
  char name[64];
} helix_devinfo_t;

/* One point of the search space.  Stands in for the `-D` macro tuple that names a
 * reference executable: (K_STAGE, BLOCK_ROWS, BLOCK_COLS, WARP_ROWS, WARP_COLS,
 * splitK) for fp16 (scripts/Ampere_FP16/build_Ampere_FP16.py:41-62) and
 * (BM, BN, BK, TM, TN, ...) for fp32 (scripts/Ampere_FP32/build_Ampere_FP32.py:37-63).
 * A zeroed struct (tile_m == 0) asks the library to choose. */
typedef struct helix_cfg {
  int op;        /* helix_op_t                                                       */
  int tile_m;    /* CTA tile rows   (GEMM_F16/CONV: 128; GEMM_F32: 32..128)          */
  int tile_n;    /* CTA tile cols   (GEMM_F16/CONV: 16..256, multiple of 16)         */
  int tile_k;    /* K slab per stage (GEMM_F16/CONV: 64; GEMM_F32: 8 or 16)          */
  int stages;    /* shared-memory ring depth (0 = as many as fit)                    */
  int cta_group; /* 1 = one CTA per tile, 2 = CTA pair sharing one 256-row tile      */
  int split_k;   /* >= 1; > 1 needs a workspace (it needs no clearing: the arrival counters in it are
                    tagged per launch); the K slices of a tile are summed in slice order by the CTA
                    that completes the tile last                                        */
  int swap_ab;   /* 1 = put N on the 128-row UMMA axis (skinny M)                    */
  int raster;    /* M-blocks per rasterisation group (L2 reuse), 0 = default         */
  int thread_m;  /* GEMM_F32: per-thread register block rows                         */
  int thread_n;  /* GEMM_F32: per-thread register block cols                         */
  int load_group;/* GEMM_F16/CONV: warps per CTA that issue TMA loads, consecutive K slabs going to
                    different warps (0 = 2; at most 3, never more than stages);
                    GEMV_F16: 16-byte loads in flight per thread and row (0 = default)  */
  int stream_k;  /* GEMM_F16/CONV: 1 = whole waves of tiles round-robin, the K slabs of the
                    remaining tiles dealt evenly to all CTAs or CTA pairs (needs a workspace);
                    overrides split_k                                                    */
  int conv_gather; /* CONV_F16: 0 = activations arrive through an im2col tensor map wherever the
                      geometry allows it (C a multiple of 64, tensor of 128 KiB or more), else
                      through gathering producer warps; 1 = always gather (cp.async);
                      3 = window-resident kernel (stride 1, C a multiple of 64, W + 2*pad <= 256);
                      4 = row-pair kernel (3 x 3, stride 1, pad 1, 64 -> 64 channels, W <= 62: pixels on
                      the accumulator rows, window and all weights resident; the library's own choice
                      for that geometry when W >= 46 and there are at least three row pairs per SM).
                      With swap_ab = 1 (im2col geometries only) the output channels take the
                      128-row axis and tile_n pixels the other one                          */
  int max_ctas;  /* > 0: the launch spreads over at most this many SMs (also honoured when the rest of
                    the struct is zero, i.e. with the library's own choice): lets two independent
                    launches on two streams share the machine, each with longer-lived CTAs      */
  int probe;     /* tuning instrument, 0 in normal use.  GEMM_F16 / CONV_F16 through a tensor map: bit 0 = the
                    issuing thread skips its tcgen05.mma instructions, bit 1 = the A-side operand is not
                    loaded, bit 2 = the B-side operand is not loaded.  Timing such a launch separates
                    operand delivery from tensor-core time; its output is meaningless.  Bit 3 = every ring
                    stage is released on its own (no pairing of stages per commit); bits 4-6, when not zero,
                    fix how many ring stages share one arrival barrier; bit 7 = two warps issue the MMAs
                    of alternate K slabs (one-CTA kernel with at most two loading warps; measured 4-8 %
                    faster on tiles up to 128 wide, not a default); bit 8 = swapped tiles with at most 64
                    rows keep M = 128 MMAs instead of M = 64; bit 9 = the pair kernel (cta_group 2) issues its
                    MMAs from one warp (two warps alternating K slabs are its default with at most two
                    loading warps); results are not affected by these                                     */
} helix_cfg_t;

/* A fully described launch; the tagged union the timing entry point iterates. */
typedef struct helix_launch {
  int op;            /* helix_op_t */
  helix_cfg_t cfg;   /* cfg.tile_m == 0: library default */
  const void* a;     /* GEMM: A[M,K]   GEMV (f16 and f32): W[rows=N,K]   CONV: x[N,H,W,C]   */
  const void* b;     /* GEMM: B[N,K] (f16) / B[K,N] (f32)  GEMV: X[m=M,K]  CONV: w[KO,R,S,C] */
  void* c;           /* GEMM: C[M,N]   GEMV: Y             CONV: y[N,Ho,Wo,KO] */
  int64_t lda, ldb, ldc; /* leading dimensions in elements (0 = packed)        */
  int M, N, K;
  int batch;             /* strided-batch count (GEMM_F16), >= 1               */
  int64_t stride_a, stride_b, stride_c; /* batch strides in elements           */
  int conv[9];           /* CONV: N, H, W, C, KO, R, S, stride, pad            */
  int trans_a;           /* GEMM_F32: 1 = A is handed over as K x M            */
  int64_t ldc_inner;     /* GEMV: element stride between rows of W in Y (0 = 1) */
  void* ws;              /* workspace or NULL                                   */
  size_t ws_bytes;
  uint32_t flags;        /* HELIX_LAUNCH_* bits                                 */
} helix_launch_t;

/* The caller asserts that nothing this launch reads or writes is written by the kernel queued just
 * before it on the same stream (independent shapes of a sweep).  The kernel then does not wait for
 * that kernel to finish before it loads operands, so consecutive launches overlap at their edges.
 * Without the flag only the set-up phase overlaps.  Ignored for launches that use a workspace.
 * A flagged kernel still waits for its predecessor before it exits, so it never completes first: a
 * later launch that is ordered after the flagged one is ordered after everything queued before it. */
#define HELIX_LAUNCH_INDEPENDENT 1u
/* GEMV: the caller asserts that operand `a` (the matrix W: weights) is not written by the kernel
 * queued just before this launch, while X may be.  The kernel issues its first batch of W loads,
 * then waits for that kernel, then reads X: launch latency and ramp-up hide behind its tail. */
#define HELIX_LAUNCH_STATIC_A 2u

/* Library version (major*100 + minor). */
int helix_version(void);
/* Human-readable text of a status code. */
const char* helix_status_string(int status);

/* Device facts for the cost model; replaces the literal 108 (see helix_devinfo_t). */
int helix_device_info(int dev, helix_devinfo_t* out);

/* Enumerate the configurations compiled into the library.  Replaces listing
 * build/bin_fp16/gemm_<K_STAGE>_<BR>_<BC>_<WR>_<WC> and build/bin_fp32/sgemm_*
 * (scripts/Ampere_FP16/build_Ampere_FP16.py:41-70, scripts/Ampere_FP32/
 * build_Ampere_FP32.py:37-63). */
int helix_num_configs(int op);
int helix_get_config(int op, int idx, helix_cfg_t* out);

/* The configuration the library would pick for `launch` when launch->cfg is zeroed: the built-in
 * analytic stand-in for cost_model() (scripts/Ampere_FP16/Ampere_FP16_gemm.py:420-430), used when
 * no profiled dictionary is at hand. */
int helix_default_config(const helix_launch_t* launch, helix_cfg_t* out);

/* Bytes of workspace a launch needs (0 when none). */
size_t helix_workspace_bytes(const helix_launch_t* launch);

/* Queue one launch.  Generic form of the four typed entry points below. */
int helix_launch(const helix_launch_t* launch, void* status_dev, void* stream);

/* C[M,N] (fp16) = A[M,K] (fp16, row-major) * B[N,K]^T (fp16, row-major = column-major KxN),
 * fp32 accumulate.  Replaces build/bin_fp16/gemm_* and gemm_splitK_*
 * (src_template/Ampere_FP16/gemm.cu:120-558, gemm_splitK.cu:120-531) as invoked by
 * get_Ampere_FP16_gemm_Helix_result (scripts/Ampere_FP16/Ampere_FP16_gemm.py:432-441).
 * No host-side padding of M and N is needed.  lda/ldb multiples of 8, 16-byte aligned bases. */
int helix_gemm_f16(const helix_cfg_t* cfg, const void* A, int64_t lda, const void* B, int64_t ldb,
                   void* C, int64_t ldc, int M, int N, int K,
                   int batch, int64_t stride_a, int64_t stride_b, int64_t stride_c,
                   void* ws, size_t ws_bytes, void* status_dev, void* stream);

/* Y[i,r] (fp16) = sum_k W[r,k] * X[i,k], i < m <= 8, fp32 accumulate; element (i,r) is
 * stored at Y[i*ldy + r*ldy_inner].  Replaces build/bin_fp16/gemv and gemv_splitK
 * (src_template/Ampere_FP16/gemv.cu:151-252, gemv_splitK.cu:153-260). */
int helix_gemv_f16(const helix_cfg_t* cfg, const void* W, int64_t ldw, const void* X, int64_t ldx,
                   void* Y, int64_t ldy, int64_t ldy_inner, int rows, int K, int m,
                   void* ws, size_t ws_bytes, void* status_dev, void* stream);

/* y[N,Ho,Wo,KO] = conv2d(x[N,H,W,C], w[KO,R,S,C]), zero padding, fp32 accumulate, fp16 in/out,
 * as one implicit GEMM with M = N*Ho*Wo, N = KO, K = R*S*C.  Replaces the im2col executable plus
 * GEMM executable pair of get_Ampere_FP16_conv_Helix_result (scripts/Ampere_FP16/
 * Ampere_FP16_conv.py:431-446, src_template/Ampere_FP16/im2col.cu:37-97).  C a multiple of 8 (16-byte pixels), or
 * C = 4 (an RGB image stored with one zero channel) for the first-layer geometry: stride 2, 2 <= R <= 8, pad < R,
 * S + (pad odd) <= 8, W even and at most 128 output pixels per row, KO = 64 or 128; that case runs its own kernel,
 * needs no workspace, and reads of an explicit cfg only the probe bits (bit 0 no MMAs, bit 1 no row copies, bit 2
 * no output stores).  Any other C = 4 call returns HELIX_ERR_UNSUPPORTED. */
int helix_conv2d_f16_nhwc(const helix_cfg_t* cfg, const void* x, const void* w, void* y,
                          int N, int H, int W, int C, int KO, int R, int S, int stride, int pad,
                          void* ws, size_t ws_bytes, void* status_dev, void* stream);

/* C[M,N] = A * B in true fp32 (FFMA only, k ascending, no TF32).  B is K x N row-major; A is
 * M x K row-major (trans_a = 0, the x86 template's layout, scripts/x86_CPU/profile_x86_CPU.py:27-29)
 * or K x M (trans_a = 1, what src_template/Ampere_FP32/sgemm.cu:138 is handed).  Replaces
 * build/bin_fp32/sgemm_* (sgemm.cu:97-350; scripts/Ampere_FP32/Ampere_FP32_gemm.py:101-107). */
int helix_gemm_f32(const helix_cfg_t* cfg, const float* A, int64_t lda, int trans_a,
                   const float* B, int64_t ldb, float* C, int64_t ldc, int M, int N, int K,
                   void* status_dev, void* stream);

/* Y[i,r] = sum_k W[r,k] * X[i,k] in true fp32 (FFMA only), i < m <= 8; element (i,r) is stored at
 * Y[i*ldy + r*ldy_inner].  K and the leading dimensions are multiples of 4 floats, bases 16-byte aligned.
 * Each output is the shuffle-tree sum (xor 16, 8, 4, 2, 1) of 32 lane chains, lane l adding the elements
 * 4l..4l+3 of every 128-element stretch of K in ascending order: a fixed order, so results repeat bit for
 * bit.  cfg: tile_n = rows per warp (1, 2), load_group = loads in flight (2, 4, 8), split_k; NULL = library
 * choice.  Stands in for the reference's fp32 GEMV template, which none of its scripts builds
 * (src_template/Ampere_FP32/gemv_template_fp32.cu:153-218). */
int helix_gemv_f32(const helix_cfg_t* cfg, const float* W, int64_t ldw, const float* X, int64_t ldx, float* Y,
                   int64_t ldy, int64_t ldy_inner, int rows, int K, int m, void* ws, size_t ws_bytes,
                   void* status_dev, void* stream);

/* y[N,Ho,Wo,KO] = conv2d(x[N,H,W,C], w[KO,R,S,C]) in true fp32, zero padding: a column matrix
 * col[N*Ho*Wo][R*S*C] and the transposed weights are written into the caller's workspace
 * (helix_workspace_bytes; 256-byte aligned), then the FFMA GEMM of helix_gemm_f32 runs on them, so
 * every output is one fmaf chain over (r, s, c) ascending.  Replaces the im2col executable plus
 * sgemm executable pair of get_Ampere_FP32_conv_Helix_result
 * (scripts/Ampere_FP32/Ampere_FP32_conv.py:101-113, src_template/Ampere_FP32/im2col.cu:37-97).
 * A 1x1, stride-1, unpadded convolution needs no column matrix.  cfg: a HELIX_OP_GEMM_F32
 * configuration or NULL. */
int helix_conv2d_f32_nhwc(const helix_cfg_t* cfg, const float* x, const float* w, float* y,
                          int N, int H, int W, int C, int KO, int R, int S, int stride, int pad,
                          void* ws, size_t ws_bytes, void* status_dev, void* stream);

/* Time `count` launches round-robin: `warmup` untimed rounds, then `iters` timed rounds between
 * two CUDA events on a private stream; *avg_s is seconds per launch.  Distinct buffers per
 * entry give the rotating-operand protocol for memory-bound shapes.  Replaces the cudaEvent
 * loops of the reference harnesses (gemm.cu:622-660: 10 warm-up + 10 timed launches).
 * use_graph != 0 captures one round into a CUDA graph first (for kernels of a few microseconds). */
int helix_time_launches(const helix_launch_t* list, int count, int warmup, int iters, int use_graph,
                        double* avg_s, double* min_round_s, double* max_round_s);

/* Host-buffer convenience wrappers (synchronous: H2D copy, launch, D2H copy).  They are what the
 * end-to-end benchmark leg times and what a caller without device memory of its own would bind. */
int helix_gemm_f16_host(const void* A, const void* B, void* C, int M, int N, int K);
int helix_gemv_f16_host(const void* W, const void* X, void* Y, int rows, int K, int m);
int helix_gemm_f32_host(const float* A, const float* B, float* C, int M, int N, int K);
int helix_conv2d_f16_nhwc_host(const void* x, const void* w, void* y, int N, int H, int W, int C,
                               int KO, int R, int S, int stride, int pad);

/* Split-K GEMV (same result as helix_gemv_f16 with cfg.split_k = split_k) that never touches the
 * device allocator: the fp32 partial sums go to a 4 MiB array compiled into the library instead
 * of a caller workspace, so split_k * m * rows may not exceed HELIX_GEMV_STATIC_FLOATS, else
 * HELIX_ERR_CAPACITY (split_k as used: a split that would leave fewer than 256 elements of K per slice runs
 * as split_k = 1, and a single-pass GEMV never touches the array, so it is never rejected for size).  It has no counterpart in the reference.  Meant for callers that cannot
 * allocate when they need the product, e.g. a decode loop that has given all HBM to its own
 * pool.  The first call on each device looks up the array's device address (the set-up), so
 * make that first call before any stream capture begins.  The array is shared by all calls and keeps the last call's partials; a call overwrites every slot before
 * reading it, so nothing needs clearing, but calls that can overlap on the GPU (different
 * streams) corrupt each other and must be ordered by the caller. */
#define HELIX_GEMV_STATIC_FLOATS (1u << 20)
int helix_gemv_f16_static(const void* W, int64_t ldw, const void* X, int64_t ldx, void* Y, int64_t ldy,
                          int64_t ldy_inner, int rows, int K, int m, int split_k, void* stream);

/* Timeline capture for tuning the fp16 GEMM / convolution kernels, one-CTA and CTA-pair (the
 * reference has only whole-kernel cudaEvent times, gemm.cu:622-660).  While a device buffer is
 * set, each such launch whose grid fits writes helix_trace_words_per_cta() 64-bit words per CTA
 * into it: [0] globaltimer and [1] clock64 at CTA start, [2] clock64 when global memory may first
 * be touched, [3] clock64 and [4] globaltimer at teardown; (one-CTA kernel) [5]..[7] the MMA-issuing thread's
 * cycles summed over its K slabs, two 32-bit sums per word: barrier waits | fence and descriptors, the four MMAs |
 * the commit, slab count | everything between a commit and the next wait; from word 8 on, for each of the first
 * 20 work items of the CTA, six clock64 stamps: first / last load request, MMA issue start / end,
 * epilogue start / end; then, for the CTA's first 32 K slabs, the clock64 at which each was
 * requested (32 words) and at which the MMA issuer found it loaded (32 words).  Later launches
 * overwrite earlier ones.  Pass NULL to switch capture off (the default). */
int helix_trace_buffer(void* device_buf, size_t bytes);
int helix_trace_words_per_cta(void);

/* Self-test of the bounded device-side wait (no reference counterpart: the reference's kernels have no
 * waits that can fail).  One thread waits on a barrier that nothing arrives at; after `limit_ns`
 * nanoseconds (at most one second) the wait gives up, HELIX_ERR_TIMEOUT appears in *status_dev and the
 * kernel returns normally.  This is the path every kernel of the library takes when a pipeline stage
 * never completes; the caller reads the status word after synchronising. */
int helix_selftest_bounded_wait(uint64_t limit_ns, void* status_dev, void* stream);

/* Number of kernel launches this process has queued through the library (all ops). */
int64_t helix_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* HELIX_B200_H_ */
