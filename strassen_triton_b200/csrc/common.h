// Internal declarations shared by the translation units of libb200s.so.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/b200s.h"

namespace b200s {

// ---- host-side bookkeeping (api.cu) -------------------------------------------------------
void note_cuda_error(cudaError_t e, const char* where);
void count_launch(int n = 1);
// Device status words (2 x uint32) of the current device, allocated on first use. nullptr on failure.
uint32_t* device_status_words();
int sm_count();
// SMs the product kernels may occupy: sm_count() unless b200s_set_product_sms lowered it.
int product_sm_count();
// Counters (kSendUnits 32-bit words per device) the sending CTAs of a row-sharded product wait on.
constexpr int kSendUnits = 4000;
uint32_t* device_send_counters();
// SMs a product with several destinations gives to sending CTAs (b200s_set_sender_sms; 0 = none).
int sender_sm_count();

#define B200S_CUDA_OK(expr)                          \
  do {                                               \
    cudaError_t e__ = (expr);                        \
    if (e__ != cudaSuccess) {                        \
      ::b200s::note_cuda_error(e__, #expr);          \
      return B200S_ERR_CUDA;                         \
    }                                                \
  } while (0)

inline size_t dtype_size(int dt) { return dt == B200S_FP32 ? 4 : 2; }

// ---- GEMM (gemm_sm100.cu) -----------------------------------------------------------------
// C[b] (+)= A[b] . B[b] for b < batch; all operands on the device. Leading dimensions and
// batch strides in elements. in_dtype fp32 runs as TF32.
struct GemmArgs {
  const void* A;
  const void* B;
  void* C;
  int64_t M, N, K, batch;
  int64_t lda, ldb, ldc;
  int64_t strideA, strideB, strideC;
  int a_major, b_major;
  int in_dtype, out_dtype;
  int beta;
  int cta_group;  // tile variant of b200s_problem: 0 = default, 1..3 = force
  // Optional: device status words and SM count supplied by the caller instead of the per-device
  // state of api.cu (nullptr / 0 = use that state).
  uint32_t* status = nullptr;
  int sms = 0;
  // Optional: n_dst > 0 stores C to C_list[0 .. n_dst) instead of C (same ldc everywhere; needs the
  // TMA-store epilogue: beta 0, 16-byte aligned rows). Destinations may be peer GPUs' memory.
  int n_dst = 0;
  void* const* C_list = nullptr;
  // Optional: a row vector of N elements of out_dtype added to every row of the product before the
  // result is rounded (the bias of a Linear layer).
  const void* bias = nullptr;
  // Optional: an NVLS multicast address of C(0,0) that maps to every GPU's copy. C (or C_list[0])
  // is then this GPU's own copy, written by TMA, and every tile is also stored once to mc_dst.
  void* mc_dst = nullptr;
  // Optional, with several destinations: the last send_sms CTAs of the launch do the remote stores
  // (block of columns by block of columns, as C gets finished) instead of the epilogue warps.
  int send_sms = 0;
};
int launch_gemm(const GemmArgs& g, cudaStream_t stream);
// One-thread kernel that waits `limit_ns` on a barrier nobody signals and reports the give-up in the
// device status words (the self-test behind b200s_wait_probe).
int launch_wait_probe(uint64_t limit_ns, cudaStream_t stream);

// ---- fused Strassen kernel (gemm_sm100.cu) ------------------------------------------------
// One persistent launch that runs the grouped product over all 7^depth operand blocks while four
// extra warps per CTA ("adders") form the operand blocks of the later outer groups and recombine
// each outer quadrant of C as soon as the groups feeding it are done. Groups are laid out in
// scratch in processing order: group i holds outer product order[i] (7 blocks at two levels, 1 at one).
struct FusedArgs {
  GemmArgs gemm;             // A = operand blocks of A, B = those of B, C = product blocks, batch = 7^depth
  int algo, depth;           // classic / winograd, 1 or 2 levels
  const void* A;             // original operands and how their blocks are stored (as PreaddArgs)
  const void* B;
  int64_t lda, ldb;
  int64_t a_rows_blk, a_cols_blk, b_rows_blk, b_cols_blk;
  int a_transposed, b_transposed;
  void* C;                   // result, row-major
  int64_t Mb, Nb, ldc;
  int out_dtype, beta;
  int order[7];              // outer products in processing order
  int groups_formed;         // leading groups whose operand blocks were formed before this launch (>= 1)
  int b_formed;              // 1: every block of B is in place already
  int quads_inside;          // bit r set: outer quadrant r of C is recombined by this launch
  uint32_t* flags;           // 16 words, zero when the kernel starts: counters the CTAs share
};
int launch_fused(const FusedArgs& f, cudaStream_t stream);

// ---- fp32 operand re-layout (transpose.cu) -----------------------------------------------
// out[c][r] = in[r][c] for a rows x cols fp32 matrix per batch item.
int launch_transpose_f32(const void* in, void* out, int64_t rows, int64_t cols, int64_t ld_in, int64_t ld_out,
                         int64_t batch, int64_t stride_in, int64_t stride_out, cudaStream_t stream);

// Three-pass TF32: out = rows x 3*cols with K segments [hi|lo|hi] (side 0) or [hi|hi|lo] (side 1).
int launch_split3_f32(const void* in, void* out, int64_t rows, int64_t cols, int64_t ld_in, int64_t batch,
                      int64_t stride_in, int side, cudaStream_t stream);

// ---- Strassen schedule (schedule.h) and its passes (preadd.cu, combine.cu) ----------------
struct PreaddArgs {
  const void* X;   // one operand, storage rows x cols with the contiguous dimension last
  void* out;       // 7^depth blocks, block p at out + p * rows_blk * cols_blk
  int64_t rows_blk, cols_blk;  // extents of one block in storage orientation
  int64_t ld;                  // elements between storage rows of X
  int64_t batch, strideX;      // batch stride of X in elements; output batch stride is 7^depth blocks
  int transposed;  // storage rows run along the logical column index of the operand
  int side;        // 0 = A (table U), 1 = B (table V)
  int algo, depth, dtype;
};
int launch_preadd(const PreaddArgs& a, cudaStream_t stream);

struct CombineArgs {
  const void* products;  // 7^depth blocks of Mb x Nb, row-major, block p at p * Mb * Nb
  void* C;
  int64_t Mb, Nb, ldc;
  int64_t batch, strideC;
  int algo, depth, prod_dtype, out_dtype, beta;
  const void* bias = nullptr;  // optional: N = 2^depth * Nb elements of out_dtype, added to every row before the rounding
};
int launch_combine(const CombineArgs& a, cudaStream_t stream);
// The same recombination written to n_dst (<= 8) copies of C at once (a.C and a.beta are ignored).
int launch_combine_peers(const CombineArgs& a, void* const* dst, int n_dst, cudaStream_t stream);
// Barrier number `epoch` among `world` GPUs over pads of 32-bit slots (peer.cu); bounded by limit_ns.
int launch_peer_barrier(void* const* pads, int rank, int world, uint32_t epoch, uint64_t limit_ns,
                        cudaStream_t stream);
// Contiguous copy of `bytes` (a multiple of 16) from src to n_dst (<= 8) destinations, small SM footprint.
int launch_push_rows(const void* src, void* const* dst, int n_dst, size_t bytes, cudaStream_t stream);
// The same copy by at most max_blocks blocks of 512 threads, to n_dst peer copies or, when mc_dst is
// given, once to a multicast address (peer.cu).
int launch_push_panel(const void* src, void* const* dst, int n_dst, void* mc_dst, size_t bytes, int max_blocks,
                      cudaStream_t stream);


// Outer-group forms used by the pipelined driver (api.cu): operand blocks of a few outer products,
// and recombination of a few outer quadrants of C. Block positions in scratch are given
// explicitly so the driver can lay groups out in processing order.
struct PreaddOuterArgs {
  const void* X;
  void* out;
  int64_t rows_blk, cols_blk;  // extents of one finest block in storage orientation
  int64_t ld, batch, strideX;
  int transposed, side, algo, depth, dtype;
  int n_groups;
  int groups[7];      // outer product indices p1 to form
  int out_block0[7];  // first output block of each
};
int launch_preadd_outer(const PreaddOuterArgs& a, cudaStream_t stream);

struct CombineOuterArgs {
  const void* products;
  void* C;
  int64_t Mb, Nb, ldc, batch, strideC;
  int algo, depth, prod_dtype, out_dtype, beta;
  int n_quads;
  int quads[4];         // outer quadrants of C to write
  int group_block0[7];  // first product block of outer product p1
};
int launch_combine_outer(const CombineOuterArgs& a, cudaStream_t stream);

}  // namespace b200s
