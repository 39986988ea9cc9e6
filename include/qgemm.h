/*
 * qgemm.h -- C-ABI of the B200 (sm_100a) quantized-GEMM library (libqgemm.so).
 *
 * This is the drop-in boundary under the C++ API of include/gemm.h: plain pointers and sizes, no
 * C++ or framework types. Every pointer is a DEVICE pointer owned by the caller, exactly as in the
 * reference harness (tests/includes/test_config.h:245-262). All entry points return a
 * qgemm_status_t and are asynchronous with respect to the host unless stated otherwise; work is
 * enqueued on `stream` (0 = the default stream, which is what the reference always uses, e.g.
 * src/gemm/sm80_gemm_kernel_v4.cu:344-349).
 *
 * There is no CPU fallback: on a machine without an sm_100 GPU the compute entry points fail with
 * QGEMM_ERR_CUDA / QGEMM_ERR_UNSUPPORTED.
 */
#ifndef QGEMM_H_
#define QGEMM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    QGEMM_OK = 0,
    QGEMM_ERR_INVALID_ARG = 1,    /* null pointer, ld smaller than the row length, bad enum */
    QGEMM_ERR_UNSUPPORTED = 2,    /* dtype combination or device not supported */
    QGEMM_ERR_ALIGNMENT = 3,      /* operand base not 16-byte aligned or ld*sizeof(T) not a multiple of 16 */
    QGEMM_ERR_CUDA = 4,           /* a CUDA runtime/driver call failed */
    QGEMM_ERR_WORKSPACE = 5,      /* scratch memory could not be provided */
    QGEMM_ERR_DEVICE_TIMEOUT = 6  /* a kernel abandoned a bounded wait; see qgemm_device_status */
} qgemm_status_t;

typedef enum {
    QGEMM_DTYPE_BF16 = 0,
    QGEMM_DTYPE_FP16 = 1,
    QGEMM_DTYPE_INT8 = 2,
    QGEMM_DTYPE_FP8_E4M3 = 3, /* OCP e4m3 (max 448), the CUDA-side FP8 type of include/gpu_type.h:7 */
    QGEMM_DTYPE_FP32 = 4,
    QGEMM_DTYPE_INT32 = 5,
    QGEMM_DTYPE_INT4 = 6 /* signed 4-bit (-8..7), two per byte, element 2i in the low nibble of byte i: the "Int4" of
                            the reference's roadmap (develop.md:9-12), which has no code for it. Input type of the
                            GEMM entry points (A [M,K] and B [N,K], K-major only, K and the leading dimensions even
                            and counted in elements) and output type of qgemm_quantize. The tensor cores have no
                            4-bit integer kind: the operands are widened to int8 in scratch and multiplied by the
                            int8 kernel, so results are the exact int32 sums, as for INT8. */
} qgemm_dtype_t;

/* How the K x N operand B is laid out in memory. */
typedef enum {
    QGEMM_B_ROW_MAJOR = 0, /* B[k*ldb + n]: the layout of GEMM_kernel_v1..v5 (src/include/gemm_utils.cuh:108) */
    QGEMM_B_K_MAJOR = 1    /* B[n*ldb + k]: "col-major [K,N]", the operand form of GEMM_kernel_v3_1 / v4_1
                              (src/include/gemm_utils.cuh:263-273) and of fp8_mm
                              (src/mix_gemm/hip_mix_gemm_kernel.cpp:425-439, 508-516) */
} qgemm_b_layout_t;

typedef struct CUstream_st* qgemm_stream_t; /* == cudaStream_t */

/* Optional tuning overrides; zero in a field means "library heuristic". */
typedef struct {
    int tile_n;  /* 64, 128 or 256 */
    int split_k; /* number of K splits (>= 1) */
    int group_m; /* tile rows per scheduling group */
    int max_ctas; /* cap on the persistent grid (testing) */
    int cta_pair; /* 1 = pair two CTAs on 256x256 tiles (tcgen05 cta_group::2), 2 = pair them on 512x256 tiles,
                     -1 = never, 0 = heuristic */
    int relayout_b; /* row-major B: 1 = always relay it out to K-major with the transpose kernel first,
                       0 = read it in place (MN-major tensor-core operand) when its base and ldb are 16-byte aligned */
} qgemm_tuning_t;

/*
 * C = A x B.  Replaces GEMM_kernel_v1..v5<typeIn,typeOut> (include/gemm.h:25-66; specialisations
 * e.g. src/gemm/sm80_gemm_kernel_v4.cu:366-378) and, with QGEMM_B_K_MAJOR, the operand form of
 * GEMM_kernel_v3_1 / v4_1.
 *   A: [M,K] row-major, leading dimension lda (elements).   B: see qgemm_b_layout_t, ldb.
 *   C: [M,N] row-major, ldc.   in_dtype x out_dtype: {BF16,FP16} -> {FP32,BF16,FP16} (fp32
 *   accumulate), INT8 -> INT32 (exact).
 * A, and B when K-major, need a 16-byte aligned base and ld*sizeof(T) % 16 == 0 (the reference
 * needs the same for its float4 / cp.async loads). A row-major B that is aligned the same way is read in
 * place as an MN-major tensor-core operand; one that is not (or when qgemm_tuning_t.relayout_b / the
 * environment variable QGEMM_RELAYOUT_B=1 asks for it) is first relaid out to K-major in library scratch
 * by the transpose kernel.
 */
int qgemm_gemm(int in_dtype, int out_dtype, int b_layout, const void* A, size_t lda, const void* B, size_t ldb,
               void* C, size_t ldc, size_t M, size_t N, size_t K, qgemm_stream_t stream);

/*
 * Mixed-precision GEMM C = (A o Q_A) x (B o Q_B) (README.md:5-7) with per-matrix scalar
 * coefficients: out = cast(scale_a * scale_b * acc). Argument order follows the reference's
 * (a, b, as, bs, c) (src/mix_gemm/hip_mix_gemm_kernel.cpp:508-516; src/gemm/sm80_gemm_kernel.cu:4-22).
 *   in_dtype: INT8 (int32 accumulate, exact) or FP8_E4M3 (fp32 accumulate); BF16/FP16 also accepted.
 *   out_dtype: BF16, FP16 or FP32.   scale_a / scale_b: DEVICE pointers to one float each, or NULL (= 1).
 */
int qgemm_mix_gemm(int in_dtype, int out_dtype, int b_layout, const void* A, size_t lda, const void* B, size_t ldb,
                   const float* scale_a, const float* scale_b, void* C, size_t ldc, size_t M, size_t N, size_t K,
                   qgemm_stream_t stream);

/* Both of the above with explicit tuning (tuning may be NULL). scale_a/scale_b may be NULL. */
int qgemm_gemm_ex(int in_dtype, int out_dtype, int b_layout, const void* A, size_t lda, const void* B, size_t ldb,
                  const float* scale_a, const float* scale_b, void* C, size_t ldc, size_t M, size_t N, size_t K,
                  const qgemm_tuning_t* tuning, qgemm_stream_t stream);

/* How the M x K operand A is laid out in memory (block-scaled entry point only). */
typedef enum {
    QGEMM_A_ROW_MAJOR = 0, /* A[m*lda + k] */
    QGEMM_A_COL_MAJOR = 1  /* A[m + k*lda]: how fp8_mm receives a (src/mix_gemm/hip_mix_gemm_kernel.cpp:96, 425-439) */
} qgemm_a_layout_t;

/*
 * FP8 e4m3 GEMM with block scales. Replaces fp8_mm / FP8_GEMM_kernel, the one mixed kernel the reference
 * implements (AMD only; src/mix_gemm/hip_mix_gemm_kernel.cpp:249-378, entry :508-516):
 *   C[m,n] = sum_kb ( sum_{k in block kb} A[m,k] B[k,n] ) * a_scale[kb*M + m] * b_scale[kb*ceil(N/128) + n/128]
 * with 128-wide K blocks (a_scale: one per row and block, "[m, k/128] col-major"; b_scale: one per 128 x 128
 * block of B, "[k/128, n/128] row-major"; :124-169, :425-439), fp32 accumulation, one rounding to out_dtype
 * (BF16 as the reference, or FP16 / FP32). A: see qgemm_a_layout_t; B: qgemm_b_layout_t (the reference passes
 * a col-major A and a row-major [K,N] B; both are relaid out to K-major scratch by the transpose kernel, K-major
 * operands are used in place and need 16-byte alignment). The FP8 format is OCP e4m3 (include/gpu_type.h:7).
 * Any M, N, K > 0 (the reference needs all three divisible by 32, :442-505).
 */
int qgemm_fp8_block_scaled_gemm(int out_dtype, int a_layout, int b_layout, const void* A, size_t lda, const void* B,
                                size_t ldb, const float* a_scale, const float* b_scale, void* C, size_t ldc, size_t M,
                                size_t N, size_t K, qgemm_stream_t stream);

/*
 * out[c*ld_out + r] = in[r*ld_in + c] for 1- or 2-byte elements. Replaces matrix_transpose<T>
 * (src/include/matrix_transpose.h:3-4; src/transpose/transpose.cu:60-77). Any rows, cols >= 0;
 * ld_in >= cols, ld_out >= rows (elements). in and out must not overlap.
 */
int qgemm_transpose(const void* in, void* out, size_t rows, size_t cols, size_t ld_in, size_t ld_out,
                    size_t elem_bytes, qgemm_stream_t stream);

/*
 * Per-matrix quantisation, the step in front of qgemm_mix_gemm (the reference's roadmap names it,
 * develop.md:9-12, README.md:1, but has no kernel for it):
 *   *amax_out = max |in|;  *scale_out = amax / qmax (qmax = 448 for FP8_E4M3, 127 for INT8, 7 for INT4; 1 if
 *   amax == 0);  out[r*ld_out + c] = round_to_nearest_even(in[r*ld_in + c] / scale), saturated to +-qmax.
 * in: FP32 or BF16 [rows, cols]; out: FP8_E4M3, INT8 or INT4 (packed, cols and ld_out even), same shape. scale_out and amax_out are DEVICE pointers
 * to one float each (amax_out doubles as the reduction's scratch); pass scale_out as scale_a / scale_b of
 * qgemm_mix_gemm. Everything stays on `stream`; nothing is read back to the host.
 */
int qgemm_quantize(int in_dtype, int out_dtype, const void* in, size_t ld_in, void* out, size_t ld_out,
                   float* scale_out, float* amax_out, size_t rows, size_t cols, qgemm_stream_t stream);

/*
 * Library-owned scratch of the current device (relaid-out B, split-K partial sums). It grows on
 * demand (a growth step synchronises the device and allocates); reserve it up front to keep
 * allocation out of timed or captured regions. The reference API has no workspace argument
 * (include/gemm.h:25-66), hence the internal buffer.
 */
int qgemm_workspace_reserve(size_t bytes);
size_t qgemm_workspace_bytes(void);

/* Bytes of scratch a call with these arguments would use at most (row-major B counted as relaid out). */
size_t qgemm_workspace_query(int in_dtype, int b_layout, size_t M, size_t N, size_t K, const qgemm_tuning_t* tuning);

/*
 * Which kernel configuration a GEMM of this shape would get on the current device (the same planning the entry
 * points run; alignment-dependent fall-backs, e.g. a C that TMA cannot address, are decided at call time and not
 * reflected): out6 = { tile rows, tile columns, CTAs per tile (1, or 2 = tcgen05 cta_group::2 pair), K splits,
 * tiles of the last wave whose K range is sliced (0 = none), slices }. No counterpart in the reference.
 */
int qgemm_plan_query(int in_dtype, int out_dtype, int b_layout, size_t M, size_t N, size_t K,
                     const qgemm_tuning_t* tuning, int* out6);

/*
 * qgemm_plan_query with more fields: writes min(n_out, QGEMM_PLAN_FIELDS) of
 *   [0..5] as qgemm_plan_query;
 *   [6] tile columns of the balanced tiling, 0 = equal tiles. With QGEMM_BALANCE=1 in the environment a problem with
 *       fewer equal tiles than SMs (small M) gets the sixteen-column units of N dealt out over as many tile columns as
 *       there are SMs per tile row, so that every SM pulls an equal share of B (off by default: measured, it does not
 *       pay on B200); [1] is then the widest tile the kernel is built for and
 *   [7] the narrowest tile's width in columns (the widest is 16 more when N / 16 does not divide evenly);
 *   [8] rows of A loaded per pipeline stage; [9] CTAs launched;
 *   [10] CTAs per cluster when the K slices of [3] are added up inside one launch through distributed shared memory
 *        (2, 4 or 8; with [2] == 2 the slices run on CTA pairs and the cluster has twice as many CTAs), 0 when they go
 *        through scratch and a second kernel. QGEMM_KCLUSTER=0 in the environment turns the one-launch form off,
 *        QGEMM_KCLUSTER=1 its CTA-pair variant only;
 *   [11] K blocks (128 bytes of K each) brought in by one TMA instruction: 2 with the 64-wide tile when K is a whole
 *        number of blocks and both operands are K-major in memory, else 1 (QGEMM_KGROUP overrides).
 */
#define QGEMM_PLAN_FIELDS 12
int qgemm_plan_query_ex(int in_dtype, int out_dtype, int b_layout, size_t M, size_t N, size_t K,
                        const qgemm_tuning_t* tuning, int* out, int n_out);

/*
 * Synchronises the current device and copies its four status words to out4:
 * [0] error code (0 = none, 1 = a bounded wait ran out), [1] CTA, [2] role (1 producer, 2 MMA,
 * 3 epilogue), [3] position. Returns QGEMM_ERR_DEVICE_TIMEOUT if [0] != 0. Clears the words.
 * The words of qgemm_mix_gemm_splitk_static (which keeps its own, inside the loaded module) are read and
 * cleared as well and reported when the ordinary ones are clean. Allocates nothing: on a device where no
 * GEMM has run yet there is nothing to read.
 */
int qgemm_device_status(int* out4);

/*
 * The QGEMM_* environment variables (tuning overrides for experiments: QGEMM_TILE_N, QGEMM_SPLIT_K,
 * QGEMM_GROUP_M, QGEMM_CTA_PAIR, QGEMM_RELAYOUT_B, QGEMM_MAX_CTAS, QGEMM_DIRECT_STORE, QGEMM_FULL_A_TILE,
 * QGEMM_TAIL_SPLIT, QGEMM_BALANCE, QGEMM_PREFETCH, QGEMM_KCLUSTER, QGEMM_KGROUP, QGEMM_EARLY_GROUPS, QGEMM_ONE_TILE, QGEMM_EVEN_RUNS, QGEMM_HOST_BANDS, QGEMM_HOST_BANDS_N) are
 * read once, when the library is
 * loaded; this reads them again. Not meant to run concurrently with GEMM calls of other threads.
 */
int qgemm_reload_env(void);

/*
 * Test hook for failure detection without a GPU fault: the NEXT GEMM this process launches leaves out the TMA
 * loads of 128-byte K block `k_block` in every CTA, so that the consumer's bounded wait runs out after about a
 * second, the kernel returns by itself and qgemm_device_status reports where it gave up. One-shot (the launch
 * that consumes it disarms it); k_block < 0 disarms. Nothing in the library arms it by itself.
 */
int qgemm_test_arm_skip_load(int k_block);

/*
 * Split-K mixed GEMM that allocates nothing. It has no counterpart in the reference; it exists for
 * callers that cannot allocate device memory where they need the product -- real-time loops that must not
 * risk the device-wide synchronisation an allocation can imply, embedders whose memory budget is fixed at
 * start-up, and processes in which another allocator already owns all of the GPU's memory so that a
 * cudaMalloc made here would fail. Same result as qgemm_gemm_ex with
 * tuning {tile_n = 128, split_k}, bit for bit, but the partial sums live in a fixed array inside the
 * loaded module (QGEMM_STATIC_SCRATCH_BYTES, held by every GPU that loads the library until the process
 * exits) instead of the library's growable scratch, and no cudaMalloc / cudaFree or other allocating
 * routine is called.
 *   A [M,K] and B [N,K] (K-major only), both 16-byte aligned with 16-byte-multiple leading dimensions;
 *   dtypes as qgemm_mix_gemm, plus INT8 -> INT32 with both scales NULL; 2 <= split_k <= ceil(K*sizeof(T)/128).
 *   Needs split_k * M * round_up(N,4) * 4 bytes of the fixed array: a larger problem is rejected with
 *   QGEMM_ERR_WORKSPACE before anything is launched.
 * The first call on a device resolves the array's device address (cudaGetSymbolAddress) and configures the
 * kernel; make that first call before starting any stream capture. All calls on a device share the one
 * array, which keeps the previous call's partial sums (none of them needs clearing: each call overwrites
 * what it later reads), so calls that overlap on the GPU (for example on different streams with no
 * ordering between them) race with each other and must be serialised by the caller. A bounded wait that runs out in
 * its kernels is reported by qgemm_device_status like any other, which allocates nothing either.
 */
#define QGEMM_STATIC_SCRATCH_BYTES (32u << 20)
int qgemm_mix_gemm_splitk_static(int in_dtype, int out_dtype, const void* A, size_t lda, const void* B, size_t ldb,
                                 const float* scale_a, const float* scale_b, void* C, size_t ldc, size_t M, size_t N,
                                 size_t K, int split_k, qgemm_stream_t stream);

/*
 * C = cast(scale_a * scale_b * (A x B)) with A, B and C in HOST memory: what the reference's harness does around
 * every kernel -- copy the operands to the device, launch, copy C back (tests/includes/test_config.h:239-286) --
 * as one pipelined call. A goes up in row bands and B in column bands, alternately; each arriving band is
 * followed by one GEMM over the blocks of C it completes and by their download on a second copy engine, so the
 * PCIe link stays busy in both directions and only a thin strip is left after the last byte has arrived.
 *   A_host [M,K], B_host ([K,N] row-major or [N,K] K-major), C_host [M,N]; leading dimensions in elements, no
 *   alignment requirement on the host side. Pin the host buffers (cudaHostAlloc / cudaHostRegister): with
 *   pageable memory the copies still work but do not overlap.
 *   scale_a_host / scale_b_host: HOST pointers to one float each, read during the call; NULL = 1.0.
 *   dtypes as qgemm_gemm_ex (BF16/FP16 -> FP32/BF16/FP16; INT8 -> INT32 exact, or scaled; FP8 scaled).
 * Device buffers for the three matrices are kept inside the library between calls (freed by qgemm_shutdown).
 * The work is ordered after everything already enqueued on `stream`, and on return `stream` has been made to
 * wait for the last download: C_host is complete once `stream` is synchronised. Calls on one device are
 * serialised against each other.
 */
int qgemm_gemm_host(int in_dtype, int out_dtype, int b_layout, const void* A_host, size_t lda, const void* B_host,
                    size_t ldb, const float* scale_a_host, const float* scale_b_host, void* C_host, size_t ldc,
                    size_t M, size_t N, size_t K, qgemm_stream_t stream);

/*
 * qgemm_gemm_host with A already in DEVICE memory (A_dev [M,K], 16-byte aligned base and lda * sizeof(T) a multiple
 * of 16; everything else as above): only B is uploaded, in column bands, and every arriving band is followed by the
 * GEMM and the download of the column strip of C it completes. For the ranks of a column-sharded product, which all
 * multiply the same A: each uploads a share of A's rows, they exchange the shares over NVLink (an all-gather), and
 * A crosses PCIe once per box instead of once per GPU. A_dev is read by work ordered after `stream`. No
 * counterpart in the reference (single GPU, tests/includes/test_config.h:239-286).
 */
int qgemm_gemm_host_resident_a(int in_dtype, int out_dtype, int b_layout, const void* A_dev, size_t lda,
                               const void* B_host, size_t ldb, const float* scale_a_host, const float* scale_b_host,
                               void* C_host, size_t ldc, size_t M, size_t N, size_t K, qgemm_stream_t stream);

/*
 * The bands qgemm_gemm_host cuts an extent (the rows of A with shrink != 0, the columns of B with shrink == 0)
 * into: about `bands` (0 = the default, 8) equal bands of whole 256-wide tiles; with `shrink` the last of them is
 * halved repeatedly down to 256. Writes up to max_bands pairs {lo, hi} to edges_out (may be NULL) and returns the
 * number of bands. Pure host arithmetic: callers use it to count the launches and copies of a qgemm_gemm_host
 * call. No counterpart in the reference.
 */
int qgemm_host_band_schedule(size_t extent, int bands, int shrink, size_t* edges_out, int max_bands);

/*
 * GEMM whose result is stored to several buffers by the same kernel: C_dsts[0..n_dsts-1] each receive the
 * identical M x N block (same ldc, same out_dtype). No counterpart in the reference, which is single-GPU; it
 * serves the column-sharded configuration: rank r passes, for every GPU of the box, the address of columns
 * [n0, n1) of that GPU's full [M, N_total] matrix (its own first, the others mapped with qgemm_peer_open), and
 * when all ranks' calls have completed every GPU holds the whole C -- the all-gather happens as tile stores
 * over NVLink from the GEMM's epilogue while later tiles are still being multiplied. Only stores cross to other
 * GPUs; nothing is loaded from them. Arguments as qgemm_mix_gemm (scales may be NULL; INT8 -> INT32 with both
 * NULL); 1 <= n_dsts <= QGEMM_MAX_DSTS; every destination 16-byte aligned and ldc * sizeof(out) a multiple of
 * 16 (QGEMM_ERR_ALIGNMENT otherwise). The call only enqueues work on `stream`; a destination on another GPU is
 * complete once this call's stream work has finished, and the ranks still need their own barrier before they
 * read what the others wrote.
 */
#define QGEMM_MAX_DSTS 8
int qgemm_gemm_multi_dst(int in_dtype, int out_dtype, int b_layout, const void* A, size_t lda, const void* B,
                         size_t ldb, const float* scale_a, const float* scale_b, void* const* C_dsts, int n_dsts,
                         size_t ldc, size_t M, size_t N, size_t K, qgemm_stream_t stream);

/*
 * Inter-process sharing of a device buffer between the ranks of one box (CUDA IPC memory handles), so that
 * qgemm_gemm_multi_dst can be given the other ranks' matrices. No counterpart in the reference.
 *   qgemm_peer_export  fills handle_out[QGEMM_PEER_HANDLE_BYTES] for the device allocation that contains ptr
 *                      and *offset_out with ptr's byte offset inside it; the allocation must come from
 *                      cudaMalloc (not from a virtual-memory pool). Send both to the other processes by any means.
 *   qgemm_peer_open    maps an exported allocation into this process (a different process from the exporter)
 *                      and enables peer access; *base_out + offset is the buffer.
 *   qgemm_peer_close   unmaps it; call before the exporting process frees the allocation.
 */
#define QGEMM_PEER_HANDLE_BYTES 64
/* A device allocation of its own (cudaMalloc) for a buffer that will be exported: an exported handle covers the
 * whole allocation that contains the buffer, so a buffer carved out of a framework's caching allocator would expose
 * its neighbours in the same block to every process that maps it. Free with qgemm_peer_free after every peer has
 * closed its mapping. */
int qgemm_peer_alloc(size_t bytes, void** ptr_out);
int qgemm_peer_free(void* ptr);
int qgemm_peer_export(const void* ptr, void* handle_out, size_t* offset_out);
int qgemm_peer_open(const void* handle, void** base_out);
int qgemm_peer_close(void* base);

/* Frees the scratch and cached descriptors of every device (blas::blas_destroy() calls this). */
int qgemm_shutdown(void);

const char* qgemm_status_string(int status);
int qgemm_version(void);

#ifdef __cplusplus
}
#endif
#endif /* QGEMM_H_ */
