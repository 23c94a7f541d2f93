/*
 * b200s — Strassen / Strassen-Winograd / dense matrix multiplication for NVIDIA B200 (sm_100a).
 *
 * C ABI of libb200s.so. Plain pointers and sizes only; every pointer named "device" is a CUDA
 * device pointer of the current device, every stream is a cudaStream_t passed as void*.
 * All functions return a b200s_status (0 = success, negative = error); none throws, aborts
 * or synchronises the device unless its comment says so.
 *
 * The reference project (vmad18/strassen-triton) is pure Python and has no FFI of its own:
 * its boundary for this path is a set of module-level functions taking torch tensors. Each
 * entry point below names the reference function(s) whose arithmetic it carries; the Python
 * modules of the same names in this repository bind these entry points with ctypes.
 */
#ifndef B200S_H_
#define B200S_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum b200s_status {
  B200S_OK = 0,
  B200S_ERR_NULL_POINTER = -1,
  B200S_ERR_BAD_SHAPE = -2,     /* non-positive extent, or extent not divisible as the depth needs */
  B200S_ERR_BAD_STRIDE = -3,    /* leading dimension too small or not a multiple of 16 bytes */
  B200S_ERR_BAD_ALIGNMENT = -4, /* base pointer not 16-byte aligned */
  B200S_ERR_BAD_DTYPE = -5,
  B200S_ERR_BAD_ALGO = -6,
  B200S_ERR_BAD_DEPTH = -7,     /* depth outside 0..4 (b200s_preadd / b200s_combine / b200s_matmul_static: 1..2) */
  B200S_ERR_WORKSPACE_TOO_SMALL = -8,
  B200S_ERR_CUDA = -9,          /* a CUDA runtime/driver call failed; see b200s_last_cuda_error */
  B200S_ERR_NO_DEVICE = -10,    /* no sm_100 device is current */
  B200S_ERR_DEVICE_TIMEOUT = -11, /* a kernel gave up on a bounded wait (read by b200s_device_status) */
  B200S_ERR_TUNER_IO = -12,
  B200S_ERR_TOO_LARGE = -13     /* problem exceeds the fixed capacity of a no-allocation entry point */
} b200s_status;

typedef enum b200s_dtype { B200S_BF16 = 0, B200S_FP16 = 1, B200S_FP32 = 2 } b200s_dtype;

/* Which operand dimension is contiguous in memory. */
typedef enum b200s_major {
  B200S_K_MAJOR = 0, /* the contraction dimension K is contiguous: A stored M x K, B stored N x K */
  B200S_MN_MAJOR = 1 /* the outer dimension is contiguous: A stored K x M, B stored K x N */
} b200s_major;

typedef enum b200s_algo {
  B200S_ALGO_AUTO = 0,    /* tuner table decides algorithm and depth */
  B200S_ALGO_DENSE = 1,   /* plain tensor-core GEMM, depth ignored */
  B200S_ALGO_CLASSIC = 2, /* Strassen's 7 products, 10 pre-additions, 8 post-additions */
  B200S_ALGO_WINOGRAD = 3 /* Strassen-Winograd form: 7 products, 8 + 7 additions */
} b200s_algo;

/* How fp32 inputs reach the tensor cores. */
typedef enum b200s_precision {
  B200S_PREC_TF32 = 0,  /* one TF32 pass (10-bit mantissa operands), what torch does with allow_tf32 */
  B200S_PREC_3XTF32 = 1 /* split each operand into hi+lo TF32 parts, three passes: operands keep their fp32
                           mantissa, error ~1e-5 at K = 1024 (left by the tensor core's fp32 accumulation) */
} b200s_precision;

/*
 * One matrix product C[b] (+)= A[b] . B[b], b = 0..batch-1, with A logically M x K and
 * B logically K x N. Leading dimensions and batch strides are in ELEMENTS.
 *   a_major == K_MAJOR : A[b](m,k) = A[b*strideA + m*lda + k]     (row-major M x K)
 *   a_major == MN_MAJOR: A[b](m,k) = A[b*strideA + k*lda + m]     (row-major K x M, e.g. X.T)
 *   b_major == MN_MAJOR: B[b](k,n) = B[b*strideB + k*ldb + n]     (row-major K x N)
 *   b_major == K_MAJOR : B[b](k,n) = B[b*strideB + n*ldb + k]     (row-major N x K, e.g. weight.T)
 *   C[b](m,n) = C[b*strideC + m*ldc + n], always row-major.
 */
typedef struct b200s_problem {
  int64_t M, N, K;
  int64_t batch;
  int64_t lda, ldb, ldc;
  int64_t strideA, strideB, strideC;
  int32_t a_major;    /* b200s_major */
  int32_t b_major;    /* b200s_major */
  int32_t in_dtype;   /* b200s_dtype of A and B */
  int32_t out_dtype;  /* b200s_dtype of C */
  int32_t algo;       /* b200s_algo */
  int32_t depth;      /* recursion levels 0..4, or -1 = tuner table decides. Up to two levels run as one
                         pre-add / grouped GEMM / recombination pipeline; levels beyond that wrap it in
                         host-side recursion (one outer level around seven products of one level less,
                         operand sums rounded at each outer level as in the reference's recursion) */
  int32_t beta;       /* 0: C = A.B   1: C += A.B */
  int32_t prod_dtype; /* dtype the 7^depth sub-products are stored in between the GEMM and the
                         recombination: B200S_FP32, or the input dtype (the reference's rounding
                         point: torch.mm returns the input dtype). -1 = same as in_dtype */
  int32_t precision;  /* b200s_precision, used when in_dtype is fp32 */
  int32_t tile_variant; /* GEMM tile shape: 0 = library default, 1 = one CTA per 128x256 tile,
                         2 = a CTA pair per 256x256 tile (tcgen05 cta_group::2, accumulators
                         double-buffered), 3 = a CTA pair per 256x512 tile */
  int32_t pipeline;   /* how the Strassen passes are scheduled: 0 = library decides, 1 = pipelined
                         (operand sums and recombination run on side streams beside the products,
                         outer group by outer group), 2 = sequential on the caller's stream */
  int32_t b_blocks_ready; /* 1: the operand blocks of B already sit in `workspace` from an earlier call with
                         the same B, extents, dtype, algo, depth and schedule (and the same workspace):
                         skip forming them. Used when one B multiplies several row panels of A. */
  int32_t fuse;       /* whether the operand sums and the recombination run inside the product kernel:
                         0 = library decides, 1 = fused (one persistent kernel multiplies all 7^depth blocks
                         while extra warps of every CTA form the later groups' operand blocks and recombine
                         each quadrant of C as soon as its products are stored), 2 = separate passes (then
                         `pipeline` picks their schedule), 3 = fused, but the last quadrant of C is
                         recombined by a full-width launch after the kernel. Fused needs batch 1, depth 1-2,
                         16-bit operands with prod_dtype equal to them, tile_variant 0 or 3; an explicit
                         1 or 3 that cannot be met returns B200S_ERR_BAD_SHAPE */
} b200s_problem;

/* Library version, major*10000 + minor*100 + patch. */
int b200s_version(void);

/* Static, human-readable text for a status code. */
const char* b200s_status_string(int status);

/* Text of the last CUDA error seen by the calling host thread ("" if none). */
const char* b200s_last_cuda_error(void);

/*
 * Bytes of device scratch b200s_matmul needs for this problem after algo/depth resolution
 * (0 for a dense product). Scratch holds the 7^depth pre-added operand blocks of A and B and the
 * 7^depth sub-products: the temporaries S1..S10 and M1..M7 of
 * fixed_strassen_fp32_agg.py:87-113 and :38-44.
 */
int b200s_workspace_bytes(const b200s_problem* p, size_t* bytes_out);

/*
 * C (+)= A . B on `stream`. Replaces, on the device, the arithmetic of
 *   fixed_strassen_fp32_agg.py:13-56   _strassen_base                (algo classic, depth 1)
 *   fixed_strassen_fp32_agg.py:59-125  strassen_matmul_n_layers      (classic, depth 2)
 *   fixed_strassen.py:12-126           the same-dtype twins
 *   strassen.py:697-812                _strassen_base / strassen_matmul_two_layers
 *   strassen.py:66-88,195-213,674-693  run_matmul_fp32_accum / run_strassen / run_strassen2 (beta = 1)
 *   strassen_2_layer.py:7-15           run_strassen_2_layer_fp32_accum (beta = 1, depth 2)
 *   strassen_no_tuning.py:536-556      run_winograd_strassen          (algo winograd, beta = 1)
 * Operand blocks are summed in fp32 from the original blocks and rounded once to the input
 * dtype; products accumulate in fp32 on the tensor cores; recombination across all levels sums
 * in fp32 and rounds once to out_dtype.
 * `workspace` may be NULL when b200s_workspace_bytes reports 0. Asynchronous: returns after
 * enqueuing the kernels.
 */
int b200s_matmul(const b200s_problem* p, const void* A_device, const void* B_device, void* C_device,
                 void* workspace_device, size_t workspace_bytes, void* stream);

/*
 * C (+)= A . B + bias: b200s_matmul with a row vector of N elements of out_dtype added to every row
 * of the product in fp32, before the one rounding to out_dtype - the `x @ W.T + b` of the reference's
 * LinearStrassen (model/layers.py:271-272) without a separate pass over the output. A dense product
 * adds it in the GEMM epilogue, a one- or two-level Strassen product in its recombination kernel
 * (the sequential schedule is used; more than two levels return B200S_ERR_BAD_DEPTH).
 */
int b200s_matmul_bias(const b200s_problem* p, const void* A_device, const void* B_device, const void* bias_device,
                      void* C_device, void* workspace_device, size_t workspace_bytes, void* stream);

/*
 * C (+)= A . B like b200s_matmul, for callers that cannot hand over scratch memory. (No counterpart
 * in the reference: it is an addition of this library.)
 *
 * Who needs it: code that runs where device allocation is off the table - a real-time or
 * safety-certified control loop that must not call an allocator after start-up, a plug-in hosted by
 * an application that owns all device memory and gives its guests none, a callback that runs inside
 * someone else's stream-ordered pipeline and may not synchronise or allocate. Such callers pass only
 * the operands and the result; the blocks that b200s_matmul keeps in `workspace` live here in a
 * fixed 64 MiB array that is part of the library image (so every GPU that loads the library carries
 * those 64 MiB until the process exits). The function calls no cudaMalloc / cudaFree and no
 * allocating library routine.
 *
 * Limit: b200s_workspace_bytes(p) must not exceed 64 MiB (for bf16: depth 1 up to about 2048^3,
 * depth 2 up to about 1792^3; at depth 0 any size of 16-bit operands, while fp32 operands given
 * MN-major need their K-major copy to fit, i.e. M*K*4 and K*N*4 bytes); larger problems return
 * B200S_ERR_TOO_LARGE and launch nothing. Always the sequential schedule on `stream`; `pipeline`,
 * `fuse` and `b_blocks_ready` are ignored. fp32 operands run as one TF32 pass: a problem that asks
 * for B200S_PREC_3XTF32 is refused with B200S_ERR_BAD_DTYPE rather than silently run at lower
 * precision.
 *
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress) and the
 * device's properties; make that first call outside any stream capture. All calls share the one
 * array: it still holds the previous call's blocks when a call starts, every byte a call reads it
 * has written first, so nothing needs clearing - but two calls whose kernels can overlap on the GPU
 * (different streams, or several host threads) overwrite each other's blocks and give wrong
 * results. Serialise them on one stream. A wait that gives up inside this call is recorded in
 * status words of the library image, not in those b200s_device_status reads: b200s_static_status
 * reads (and clears) them the same way, device -> host on `stream`, again without allocating.
 */
int b200s_matmul_static(const b200s_problem* p, const void* A_device, const void* B_device, void* C_device,
                        void* stream);
int b200s_static_status(void* stream, int32_t* status_out, int32_t* detail_out);

/*
 * The algorithm and depth b200s_matmul will use for p (resolves AUTO / -1 through the tuner
 * table; clamps depth to what the extents allow). Replaces the hand-chosen `depth=` arguments and
 * the triton.autotune config lists of strassen.py:9-30,93-114,218-236.
 */
int b200s_resolve(const b200s_problem* p, int32_t* algo_out, int32_t* depth_out);

/*
 * Tuner table: measured (M,N,K,in_dtype) -> (algo, depth, schedule) entries; lookups pick the entry
 * nearest in log-extents and fall back to a dense product below the smallest recorded crossover.
 * The schedule is a b200s_problem.fuse value (0 = none recorded: the built-in rule applies) and is
 * used when the caller leaves `fuse` and `pipeline` at 0. The table is process-wide, guarded by a
 * mutex. File format: one entry per line, "M N K in_dtype algo depth [fuse]".
 */
int b200s_tuner_clear(void);
int b200s_tuner_record(int64_t M, int64_t N, int64_t K, int32_t in_dtype, int32_t algo, int32_t depth);
int b200s_tuner_load(const char* path);
int b200s_tuner_save(const char* path);
int b200s_tuner_lookup(int64_t M, int64_t N, int64_t K, int32_t in_dtype, int32_t* algo_out,
                       int32_t* depth_out);
int b200s_tuner_record_schedule(int64_t M, int64_t N, int64_t K, int32_t in_dtype, int32_t algo, int32_t depth,
                                int32_t fuse);
int b200s_tuner_lookup_schedule(int64_t M, int64_t N, int64_t K, int32_t in_dtype, int32_t* algo_out,
                                int32_t* depth_out, int32_t* fuse_out);

/*
 * Reads (device -> host, synchronising `stream`) and clears the per-device status word that
 * kernels set when a bounded wait ran out. *status_out is B200S_OK or B200S_ERR_DEVICE_TIMEOUT,
 * *detail_out the role code of the waiter that gave up.
 */
int b200s_device_status(void* stream, int32_t* status_out, int32_t* detail_out);

/*
 * Self-test of the bounded device-side waits: launches a one-thread kernel that waits limit_ns
 * (1 .. 10^9) on a barrier nobody signals, gives up, and reports it in the status words exactly as
 * a stalled GEMM role would. Afterwards b200s_device_status returns B200S_ERR_DEVICE_TIMEOUT with
 * detail 7 once, then B200S_OK again. The kernel owns no TMA transfer and no tensor memory, so
 * nothing is left in flight when it returns. No counterpart in the reference.
 */
int b200s_wait_probe(uint64_t limit_ns, void* stream);

/*
 * Stage timing of b200s_matmul calls (the per-kernel rows the reference reads from torch.profiler in
 * its profiling scripts, main_profiling.py:197-229 for the totals). Between _begin and _end every
 * call that runs the sequential or the fused schedule on the current device records an event on its
 * stream at each stage boundary, for at most max_calls (1..4096) calls. _end waits for the recorded
 * calls, writes the mean duration in milliseconds of the four stages to stage_ms_out[0..3] - operand
 * blocks of A, operand blocks of B, products, recombination; in the fused schedule: blocks of A of the
 * first group, blocks of B of the first group, the fused kernel, the recombination left after it -
 * and the number of calls measured to *calls_out. A dense product counts entirely as "products";
 * the multi-stream pipelined schedule and products of more than two levels record nothing. One
 * collection at a time, process-wide.
 */
int b200s_profile_begin(int max_calls);
int b200s_profile_end(float* stage_ms_out, int32_t* calls_out);

/* Number of kernels this library has launched in the calling process (for benchmarks' accounting). */
int64_t b200s_launch_count(void);

/*
 * Stand-alone passes of the Strassen pipeline, exposed for tests and profiling.
 * b200s_preadd: writes the 7^depth operand blocks of one side (side 0 = A, 1 = B) into `out`
 *   (block p at out + p * rows_blk * cols_blk elements, same major as the input).
 * b200s_combine: reads 7^depth product blocks (Mb x Nb each, row-major, prod_dtype) and writes
 *   or accumulates C.
 * They carry the additions of fixed_strassen_fp32_agg.py:87-96 and :115-118.
 */
int b200s_preadd(const b200s_problem* p, int side, const void* X_device, void* out_device, void* stream);
int b200s_combine(const b200s_problem* p, const void* products_device, void* C_device, void* stream);

/*
 * b200s_combine writing the finished M x N product to n_dst (1..8) destinations at once: C_list[i]
 * is the device address of element (0,0) of the product inside destination i, all with leading
 * dimension p->ldc. Destinations may be memory of other GPUs mapped into this process (peer or
 * symmetric memory): the stores are plain global stores, so a row-sharded product lands in every
 * GPU's copy of C without a separate all-gather. beta must be 0 and batch 1. The reference has no
 * multi-GPU product; this carries the exchange step of a row-sharded product.
 */
int b200s_combine_peers(const b200s_problem* p, const void* products_device, void* const* C_list, int n_dst,
                        void* stream);

/*
 * b200s_matmul whose result goes to n_dst (1..8) destinations at once: C_list[i] is the device address
 * of element (0,0) of the product inside destination i, all with leading dimension p->ldc; beta must
 * be 0 and batch 1. A dense product stores every finished tile to all destinations from the GEMM's
 * epilogue: C_list[0] (put this GPU's own copy there) by TMA, the others by ordinary 16-byte stores
 * of the same staged tile, so the exchange of a row-sharded product rides on the product kernel, tile
 * by tile (it needs C rows that are multiples of 16 bytes); a one- or two-level Strassen product runs
 * its sequential schedule and ends in b200s_combine_peers. Destinations may be other GPUs' memory mapped
 * into this process; only stores go there, every load reads this GPU's memory. The reference has no
 * multi-GPU product: this is the per-rank step of the row-sharded one.
 */
int b200s_matmul_peers(const b200s_problem* p, const void* A_device, const void* B_device, void* const* C_list,
                       int n_dst, void* workspace_device, size_t workspace_bytes, void* stream);

/*
 * The dense row-sharded step with the exchange done by the NVSwitch: C_local is this GPU's copy of
 * the rows (written by TMA as in b200s_matmul), C_multicast the NVLS multicast address of the same
 * rows (an address bound to every GPU's copy of C, e.g. the multicast pointer of a symmetric-memory
 * allocation). Every finished tile is stored once more with multimem.st to C_multicast and the
 * switch replicates it into all GPUs' memory: each GPU sends its rows once instead of once per peer.
 * Dense products only (B200S_ERR_BAD_ALGO otherwise), beta 0, batch 1, rows of C multiples of 16
 * bytes. No counterpart in the reference.
 */
int b200s_matmul_multicast(const b200s_problem* p, const void* A_device, const void* B_device, void* C_local,
                           void* C_multicast, void* workspace_device, size_t workspace_bytes, void* stream);

/*
 * Barrier number `epoch` among `world` (1..8) GPUs on `stream`: pads[r] is rank r's pad of at least
 * `world` 32-bit slots, zero before the first barrier, reachable from this GPU. The kernel stores
 * `epoch` into slot `rank` of every pad and waits until all slots of pads[rank] have reached it; use
 * epochs 1, 2, 3, ... The wait is bounded by limit_ns: when it runs out the kernel reports
 * B200S_ERR_DEVICE_TIMEOUT with detail 8 through b200s_device_status and returns - it does not trap,
 * so a rank that died between steps costs its peers one limit, not their context. No counterpart in
 * the reference.
 */
int b200s_peer_barrier(void* const* pads, int rank, int world, uint32_t epoch, uint64_t limit_ns, void* stream);

/*
 * Copies `bytes` (a multiple of 16, both ends 16-byte aligned) from src_device to n_dst (1..8)
 * destinations, typically the same rows of C in the other GPUs' symmetric memory. The kernel keeps
 * one small block per SM (no shared memory, few registers) so that it can run beside a resident
 * GEMM CTA: the exchange of a finished row panel overlaps the products of the next one. No
 * counterpart in the reference (it has no multi-GPU product).
 */
int b200s_push_rows(const void* src_device, void* const* dst_list, int n_dst, size_t bytes, void* stream);

/*
 * Exchange beside the products. b200s_set_product_sms(n) makes every product kernel launched
 * afterwards by this process occupy at most n SMs (0 = all; returns the previous setting), which
 * leaves the others to kernels of other streams. b200s_push_panel copies `bytes` (a multiple of 16,
 * both ends 16-byte aligned) of finished rows with at most max_blocks blocks of 512 threads: to the
 * n_dst (1..8) peer copies in dst_list, or, when mc_dst is given, once to that NVLS multicast address
 * of the same rows (the NVSwitch writes every GPU's copy; dst_list and n_dst are ignored). A
 * row-sharded product computes row panel i+1 on most SMs while a few SMs send panel i. No counterpart
 * in the reference (it has no multi-GPU product).
 */
int b200s_set_product_sms(int n);
/*
 * b200s_set_sender_sms(n): a dense product with several destinations (b200s_matmul_peers,
 * b200s_matmul_multicast) launched afterwards by this process gives n (even, 0..64; 0 = none; returns
 * the previous setting) of its CTAs to sending instead of multiplying: they wait until a block of
 * columns of C is finished, read it from this GPU's copy and store it to the other copies, so the
 * epilogue warps of the multiplying CTAs store locally only. One kernel, one launch.
 */
int b200s_set_sender_sms(int n);
int b200s_push_panel(const void* src_device, void* const* dst_list, int n_dst, void* mc_dst, size_t bytes,
                     int max_blocks, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* B200S_H_ */
