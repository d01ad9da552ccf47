/*
 * tuna_b200 — C ABI of the B200 (sm_100a) FP16 x 4-bit(codebook) GEMM.
 *
 * Drop-in boundary for the two host launchers behind TryForefront/tuna's torch
 * extension (extension.cpp:22-24).  Plain pointers and sizes only; every
 * pointer is DEVICE memory owned by the caller unless stated otherwise; every
 * call is enqueued on `stream` (a cudaStream_t passed as void*) and returns
 * without synchronising.  All entry points return TUNA_OK (0) or a negative
 * tuna_status; nothing is launched when the status is negative.
 *
 * Names follow the reference: m = output features (rows of W), n = tokens,
 * k = reduction length.  Layouts (reference file:line):
 *   x       fp16  [n, k]          row-major activations        (test.py:76)
 *   q       u8    [m/8, k/8, 32]  packed 4-bit codes; byte j of tile (mt,kt)
 *                                 holds W[8mt+j/4, 8kt+2(j%4)] in its HIGH and
 *                                 W[.., 8kt+2(j%4)+1] in its LOW nibble
 *                                 (test.py:55-65, kernel.cu:3171,3221-3228)
 *   absmax  fp32  [m]             one scale per output row     (test.py:16-18)
 *   code    fp32  [16]            codebook, passed per call    (test.py:19-40)
 *   o       fp16  [n, m]          row-major output             (test.py:79)
 */
#ifndef TUNA_B200_H
#define TUNA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum tuna_status {
    TUNA_OK = 0,
    TUNA_ERR_NULL_POINTER = -1,    /* a required pointer is NULL                        */
    TUNA_ERR_BAD_SHAPE = -2,       /* m, k not positive multiples of 8, or n < 1        */
    TUNA_ERR_MISALIGNED = -3,      /* a pointer misses its required alignment           */
    TUNA_ERR_WORKSPACE = -4,       /* workspace NULL/too small for this shape           */
    TUNA_ERR_BAD_CONFIG = -5,      /* explicit launch config is inconsistent            */
    TUNA_ERR_LAUNCH = -6,          /* the CUDA runtime refused the launch               */
    TUNA_ERR_NO_DEVICE = -7,       /* no sm_100 device / kernel image not loadable      */
    TUNA_ERR_DEVICE_TIMEOUT = -8,  /* a bounded in-kernel wait ran out (status word)    */
    TUNA_ERR_TOO_LARGE = -9        /* beyond a documented size limit                    */
} tuna_status;

/* Which kernel family a launch uses.  AUTO lets the shape table decide. */
typedef enum tuna_path {
    TUNA_PATH_AUTO = 0,
    TUNA_PATH_STREAM = 1, /* register-streaming mma.sync kernel, small token counts       */
    TUNA_PATH_UMMA = 2,   /* tcgen05/TMEM kernel: TMA-staged, dequant into TMEM       */
    TUNA_PATH_TSTREAM = 3 /* tcgen05 weight-streaming kernel: ld.global -> table ->   *
                           * tcgen05.st fragments, small token counts                 */
} tuna_path;

/* Launch configuration, the Blackwell counterpart of the reference's
 * KernelConfig (configs.cu:12-54).  Produced by the shape table generated from
 * param_map.json, or filled by hand (tuner, tests).  Zero means "default". */
typedef struct tuna_config {
    int32_t path;          /* tuna_path                                               */
    int32_t tile_tok;      /* tokens per pass: stream 8|16|32; tstream 16|32|64|128;  *
                            * umma 16|32|64|128|256                                   */
    int32_t rows_per_warp; /* stream: 32-row blocks per warp (1|2)                    */
    int32_t warps_m;       /* stream: consumer warps along output rows (power of 2)   */
    int32_t warps_k;       /* stream: consumer warps along K (power of 2, m*k <= 16)  */
    int32_t k_steps;       /* stream: 32-column steps per warp per unit (8|16|32|64); *
                            * tstream: 32-column steps per slot (4|8)                 */
    int32_t ctas;          /* persistent CTAs (0 = one per SM)                        */
    int32_t stages_w;      /* umma: packed-weight ring depth (64-column stages)       */
    int32_t stages_x;      /* umma: unit stages (activation tile + A-operand slots)   */
    int32_t dequant_warps; /* umma: warps converting codes into TMEM (mult of 4)      */
    int32_t row_blocks;    /* umma, tstream: 128-row blocks per CTA tile (1|2|4)      */
    int32_t stages_a;      /* umma: derived (stages_x * row_blocks TMEM operand slots) */
    int32_t k_accs;        /* umma: accumulators per row block along K (1|2|4)        */
    int32_t reserved[3];
} tuna_config;

/*
 * o[n, m] = x[n, k] * dequant(q)[m, k]^T, fp16 operands, fp32 accumulation,
 * one fp16 rounding.  Replaces `wrapper` (kernel.cu:3009-3156) and keeps its
 * argument order (q, x, code, absmax, o — extension.cpp:29-33 reorders the
 * Python arguments into it).  Differences, all supersets of the reference:
 * `o` is overwritten (no pre-zeroing needed, a pre-zeroed `o` is also fine);
 * every (m % 8 == 0, k % 8 == 0, n >= 1) shape runs instead of only the 14
 * tabulated ones; results are bit-identical from run to run.
 * `workspace` holds split-K partial sums (a region whose size depends only on
 * the device: about 58 MB on a 148-SM part) followed by arrival counters; its
 * first tuna_matmul_workspace_bytes() bytes must be ZERO before the first call.
 * Every call leaves the counters zero and the counters of any shape lie beyond
 * the partial-sum region, so ONE zero-initialised allocation (sized for the
 * largest shape) serves consecutive calls of any shapes on one stream; calls
 * that overlap on the device need separate workspaces.  Alignment: q, x, o,
 * workspace 16 bytes; absmax, code 4 bytes (absmax may be a slice of a larger
 * scale buffer).
 */
int tuna_matmul(const void *q, const void *x, const void *code, const void *absmax, void *o,
                int m, int n, int k, void *workspace, size_t workspace_bytes, void *stream);

/* As tuna_matmul, with an explicit launch configuration (tuner, tests). */
int tuna_matmul_cfg(const void *q, const void *x, const void *code, const void *absmax, void *o,
                    int m, int n, int k, void *workspace, size_t workspace_bytes, void *stream,
                    const tuna_config *cfg);

/* Upper bound, over every configuration the table can pick for this shape, of
 * the workspace tuna_matmul needs.  Host-only arithmetic, no CUDA call. */
size_t tuna_matmul_workspace_bytes(int m, int n, int k);

/* The configuration tuna_matmul would use for (m, n, k) on the current device:
 * exact table entry if param_map.json had one for the shape and token bucket,
 * otherwise a heuristic.  Replaces the 122-arm if-chain of kernel.cu:3022-3155;
 * unlike it, an unknown shape is never a silent no-op. */
int tuna_lookup_config(int m, int n, int k, tuna_config *out);

/*
 * o[m, k] (fp16) = fp16_rn(fp32(code[nibble]) * fp32(absmax[row])).  Replaces
 * `dequantize_wrapper` (kernel.cu:3243-3253) and is bit-exact to its kernel
 * (kernel.cu:3218-3229).  Works for any m % 8 == 0, k % 8 == 0 (the reference
 * needs multiples of 64).
 */
int tuna_dequant(const void *q, const void *absmax, const void *code, void *o,
                 int m, int k, void *stream);

/* Reads and clears the device status word of the last tcgen05 launch on the
 * current device (synchronises `stream`).  TUNA_OK, or
 * TUNA_ERR_DEVICE_TIMEOUT if a bounded mbarrier wait gave up. */
int tuna_check_device_status(void *stream);

/* Self-test of the bounded in-kernel waits: enqueues a one-warp kernel that waits, with a limit of
 * about a millisecond, on a barrier nothing arrives at.  The wait gives up, the kernel returns, and
 * the next tuna_check_device_status() reports TUNA_ERR_DEVICE_TIMEOUT (and clears the word).  The
 * GPU is neither hung nor faulted by it. */
int tuna_selftest_bounded_wait(void *stream);

/*
 * The GEMM for callers that cannot allocate device memory.  It has no counterpart in the
 * reference.  Some hosts of this library run inside a region where cudaMalloc is off limits: an
 * inference server that hands all device memory to its own pool at start-up, or code that runs
 * between the nodes of a latency-critical serving loop where an allocation would synchronise the
 * device.  For them this entry point takes no workspace: the scratch of the small-token-count
 * kernel (tile counters and split-K partial tiles) and its status word are file-scope device
 * arrays of the library, TUNA_NOALLOC_SCRATCH_BYTES in total, which every GPU that loads the
 * library keeps until the process exits.  It never calls cudaMalloc, cudaFree or an allocating
 * library routine.
 *  - Same arguments, layouts and result as tuna_matmul (mma.sync streaming kernel, any n; more than
 *    32 tokens run as several passes).  A shape whose scratch would exceed the array returns
 *    TUNA_ERR_TOO_LARGE.  The scratch is 64 bytes of counters per row tile (a row tile is 32 to
 *    1024 rows, chosen with the configuration) plus two partial tiles per CTA, at most 18.5 MiB
 *    on a 148-SM part; with the largest partial tiles about 24 000 row tiles still fit.
 *  - The first call on a device looks up the arrays' device addresses (cudaGetSymbolAddress) and
 *    opts the kernel into large shared memory.
 *  - All calls share the one array per device and it keeps the previous call's contents (the part
 *    that must start at zero is cleared on the stream by every call): calls that overlap on the
 *    same GPU, on different streams, race.  Use tuna_matmul with separate workspaces for that.
 */
#define TUNA_NOALLOC_SCRATCH_BYTES (20u << 20)
int tuna_matmul_noalloc(const void *q, const void *x, const void *code, const void *absmax, void *o,
                        int m, int n, int k, void *stream);

/*
 * `batch` independent GEMMs of one shape in one call: matrix b uses q + b*q_stride,
 * x + b*x_stride (0 = the same activations for all), absmax + b*absmax_stride and writes
 * o + b*o_stride (strides in bytes, multiples of 16; `code` is shared).  For token counts of the
 * streaming kernel (n <= 32) this is ONE launch whose work split runs across the matrices, so
 * the fixed cost per launch is paid once: the Mixtral expert projections (8 GEMMs of
 * 14336 -> 4096, per-expert activations) or the reference's "combined" 14336 -> 32768 GEMM
 * (make_configs.py:105-106, README.md:18: x_stride = 0).  Larger n: one launch per matrix.
 * Workspace: tuna_matmul_batched_workspace_bytes (zero before the first use, left clean).
 */
int tuna_matmul_batched(const void *q, const void *x, const void *code, const void *absmax, void *o,
                        int m, int n, int k, int batch, size_t q_stride, size_t x_stride, size_t absmax_stride,
                        size_t o_stride, void *workspace, size_t workspace_bytes, void *stream);
size_t tuna_matmul_batched_workspace_bytes(int m, int n, int k, int batch);

/*
 * `count` independent GEMMs - every x, q, absmax ready when the call is enqueued, every o written by
 * it, one shared codebook - in ONE persistent launch: the units of all the GEMMs form one sequence
 * that is cut evenly across the SMs, so small GEMMs (a Mistral attention projection is 1.3 us of
 * HBM time) neither pay a launch each nor leave SMs idle, and the exchange of split-K partial sums
 * of one GEMM overlaps with the streaming of the next.  This is how a layer's or a model's
 * weight-streaming GEMMs are meant to be issued when their inputs do not depend on each other
 * (QKV and gate+up of a layer, the experts of a mixture, a benchmark sweep); the reference has no
 * counterpart (its README sums single-GEMM times, README.md:25-27).  Shapes, layouts and results
 * as tuna_matmul; token counts up to 64 run in the sequence kernel (64 GEMMs per launch), a
 * sequence with a larger token count is issued GEMM by GEMM.  Every GEMM has its own token
 * count n, so this is also the grouped GEMM of a mixture of experts with a per-expert token
 * list (the step the reference fakes with one combined GEMM over all experts,
 * make_configs.py:105-106): one entry per expert, x and o pointing at that expert's rows, n its
 * number of routed tokens; n = 0 (an expert without tokens) is skipped.  Workspace:
 * tuna_matmul_sequence_workspace_bytes (zero before the first use, left clean).
 */
typedef struct tuna_gemm_desc {
    const void *q;      /* u8   [m/8, k/8, 32] */
    const void *x;      /* fp16 [n, k]         */
    const void *absmax; /* fp32 [m]            */
    void *o;            /* fp16 [n, m]         */
    int32_t m, n, k;
    int32_t flags;      /* 0, or TUNA_GEMM_PARTIAL in a tuna_matmul_sequence_reduce call */
} tuna_gemm_desc;
int tuna_matmul_sequence(const tuna_gemm_desc *gemms, int count, const void *code, void *workspace, size_t workspace_bytes,
                         void *stream);
size_t tuna_matmul_sequence_workspace_bytes(const tuna_gemm_desc *gemms, int count);

/*
 * K-split (row-parallel) GEMMs fused with the sum of their partial outputs over the GPUs of one
 * node.  No counterpart in the reference (it has no multi-GPU path; a tensor-parallel caller runs
 * its `matmul` per rank and all-reduces the fp16 outputs).  Every rank calls
 * tuna_matmul_sequence_reduce with the same list of shapes, token counts (1..64) and flags; a GEMM
 * with flags = TUNA_GEMM_PARTIAL gets this rank's K slice (q repacked for the slice, x columns of
 * the slice) and, when the stream work is done, every rank's o holds the sum over ranks, added in
 * rank order in fp32 (identical on all ranks); a GEMM with flags = 0 is an ordinary one that
 * shares the launch (e.g. the column-parallel GEMMs of the same layers).  The GEMM kernel's epilogue stores finished rows straight into every rank's
 * exchange buffer (peer memory, ordinary stores), a small kernel per launch raises this rank's
 * flag on every peer, waits for all flags - at most about a second, then the device status word
 * reports TUNA_ERR_DEVICE_TIMEOUT through tuna_check_device_status - and sums.  Two launches
 * (GEMMs, reduce) per 64 GEMMs, capturable in a CUDA graph (the exchange number lives in device
 * memory).  Calls on one exchange must be issued in the same order on every rank, on one stream
 * per rank.
 *   tuna_exchange_bytes    size every rank's buffer needs for the largest call it will make
 *   tuna_exchange_create   allocates and zero-fills this rank's buffer (cudaMalloc) and returns
 *                          a TUNA_IPC_HANDLE_BYTES-byte handle other processes can open
 *   tuna_exchange_open     maps a peer's buffer from its handle (cudaIpcOpenMemHandle)
 *   tuna_exchange_close / tuna_exchange_destroy   undo open / create; a buffer may be destroyed only
 *                          after every peer has closed its mapping of it
 * tuna_exchange.buffer[] holds the buffers of all ranks in rank order (own buffer at [rank]);
 * world = 1 is valid (the sum of one slab).
 */
#define TUNA_GEMM_PARTIAL 1 /* tuna_gemm_desc.flags: a K-split GEMM whose output is summed over the ranks */
#define TUNA_MAX_PEERS 8
#define TUNA_IPC_HANDLE_BYTES 64
typedef struct tuna_exchange {
    int32_t rank, world;
    void *buffer[TUNA_MAX_PEERS];
    size_t bytes; /* of each buffer */
} tuna_exchange;
size_t tuna_exchange_bytes(const tuna_gemm_desc *gemms, int count, int world);
int tuna_exchange_create(size_t bytes, void **buffer, void *ipc_handle);
int tuna_exchange_open(const void *ipc_handle, void **buffer);
int tuna_exchange_close(void *peer_buffer);
int tuna_exchange_destroy(void *buffer);
int tuna_matmul_sequence_reduce(const tuna_gemm_desc *gemms, int count, const void *code, void *workspace, size_t workspace_bytes,
                                const tuna_exchange *exchange, void *stream);

/*
 * Quantizer: w fp16 [m, k] row-major -> packed codes q [m/8, k/8, 32] + absmax fp32 [m], for the
 * codebook `code` fp32 [16].  Replaces the reference's quantize_blockwise_dynamic_4bit(w,
 * block_size = k, preprocess = True) (test.py:7-68, a chain of torch kernels) with two kernels;
 * bit-identical results: absmax = max |w| per row, code = first index of the nearest codebook
 * entry to fp32(w) / absmax (fp32 division).  m and k multiples of 8; w and q 16-byte aligned.
 */
int tuna_quantize(const void *w, const void *code, void *q, void *absmax, int m, int k, void *stream);

const char *tuna_status_string(int status);

/* Library / table identification: ABI version and number of table entries. */
int tuna_abi_version(void);
int tuna_config_table_size(void);

/* Status of the calling thread's last wrapper() / dequantize_wrapper() call (below). */
int tuna_last_wrapper_status(void);

#ifdef __cplusplus
}

/*
 * The reference's own two native entry points, with their C++ linkage and parameter lists
 * (declared in extension.cpp:22-24, defined in kernel.cu:3009 and kernel.cu:3243), so that the
 * reference's pybind module links against this library unchanged.  `wrapper` takes its scratch
 * from an allocation cached inside the library per (device, stream), so calls on different
 * streams may overlap as they may in the reference.  The first call on a stream (and a call
 * that needs a larger scratch than any before it) allocates: make it outside stream capture -
 * during capture such a call fails with TUNA_ERR_WORKSPACE.  Buffers are never freed while the
 * process lives (a captured graph may refer to them).  Neither function reports errors (the
 * reference's do not either): read tuna_last_wrapper_status() after the call.
 */
struct CUstream_st;
void wrapper(void *q, void *x, void *c, void *s, void *o, int m, int n, int k, CUstream_st *stream);
void dequantize_wrapper(void *q, void *a, void *c, void *o, const int m, const int k, CUstream_st *stream);
#endif
#endif /* TUNA_B200_H */
