// Operand pre-addition pass of the Strassen pipeline.
//
// One pass over an operand: each thread loads the 4^depth quadrant values at one 16-byte
// position, forms all 7^depth signed sums in fp32 and writes them, rounded once to the operand
// dtype, as 7^depth dense blocks that the grouped GEMM reads as its batch. The operand is read
// exactly once; reads and writes are 128-bit and coalesced along the contiguous dimension.
//
// It carries the additions the reference makes before its products:
// fixed_strassen_fp32_agg.py:26-44 (one level, quadrants widened to fp32, sums rounded to
// base_dtype) and :77-96 (S1..S10 of the outer level); at two levels the reference rounds S1..S10
// before forming the inner sums, here both levels are summed in fp32 and rounded once.

#include <cuda_runtime.h>

#include <utility>

#include "common.h"
#include "preadd_device.cuh"
#include "schedule.h"

namespace b200s {

namespace {

using namespace pre;

struct PreaddKernelParams {
  const void* X;
  void* out;
  int64_t rows_blk, cols_vec;  // block rows, 16-byte vectors per block row
  int64_t ld;                  // elements
  int64_t strideX;             // elements
  int32_t transposed;
};

template <int DEPTH, typename T>
struct PreaddVec {
  static constexpr int N = DEPTH == 2 ? 4 : Vec16<T>::N;
};

template <int DEPTH, int ALGO, int SIDE, typename T>
__global__ void __launch_bounds__(256, DEPTH == 2 ? 2 : 1) preadd_kernel(const PreaddKernelParams p) {
  using PA = Preadd<DEPTH, ALGO, SIDE, T, PreaddVec<DEPTH, T>::N>;
  constexpr int NQ = PA::NQ, NP = PA::NP, VEC = PA::VEC;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= p.rows_blk * p.cols_vec) return;
  const int64_t row = idx / p.cols_vec;
  const int64_t cv = idx - row * p.cols_vec;
  const int64_t cols_blk = p.cols_vec * VEC;
  const T* X = static_cast<const T*>(p.X) + static_cast<int64_t>(blockIdx.y) * p.strideX;

  float x[NQ][VEC];
#pragma unroll
  for (int q = 0; q < NQ; ++q) {
    const int lr = sched::block_row(DEPTH, q), lc = sched::block_col(DEPTH, q);
    const int sr = p.transposed ? lc : lr;
    const int sc = p.transposed ? lr : lc;
    load_n<T, VEC>(X + (sr * p.rows_blk + row) * p.ld + sc * cols_blk + cv * VEC, x[q]);
  }
  const int64_t blk_elems = p.rows_blk * cols_blk;
  T* out = static_cast<T*>(p.out) + static_cast<int64_t>(blockIdx.y) * NP * blk_elems + row * cols_blk + cv * VEC;
  PA::all_products(x, out, blk_elems, std::make_integer_sequence<int, NP>{});
}

template <int DEPTH, int ALGO, int SIDE, typename T>
int launch_one(const PreaddArgs& a, cudaStream_t stream) {
  constexpr int VEC = PreaddVec<DEPTH, T>::N;
  PreaddKernelParams kp;
  kp.X = a.X;
  kp.out = a.out;
  kp.rows_blk = a.rows_blk;
  kp.cols_vec = a.cols_blk / VEC;
  kp.ld = a.ld;
  kp.strideX = a.strideX;
  kp.transposed = a.transposed;
  const int64_t total = kp.rows_blk * kp.cols_vec;
  const int64_t blocks = (total + 255) / 256;
  if (blocks > INT32_MAX || a.batch > 65535) return B200S_ERR_BAD_SHAPE;
  dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(a.batch));
  preadd_kernel<DEPTH, ALGO, SIDE, T><<<grid, 256, 0, stream>>>(kp);
  B200S_CUDA_OK(cudaGetLastError());
  count_launch();
  return B200S_OK;
}

template <int DEPTH, int ALGO, int SIDE>
int launch_dtype(const PreaddArgs& a, cudaStream_t stream) {
  switch (a.dtype) {
    case B200S_BF16:
      return launch_one<DEPTH, ALGO, SIDE, __nv_bfloat16>(a, stream);
    case B200S_FP16:
      return launch_one<DEPTH, ALGO, SIDE, __half>(a, stream);
    case B200S_FP32:
      return launch_one<DEPTH, ALGO, SIDE, float>(a, stream);
  }
  return B200S_ERR_BAD_DTYPE;
}

template <int DEPTH, int ALGO>
int launch_side(const PreaddArgs& a, cudaStream_t stream) {
  return a.side == 0 ? launch_dtype<DEPTH, ALGO, sched::kSideA>(a, stream)
                     : launch_dtype<DEPTH, ALGO, sched::kSideB>(a, stream);
}

// ---- outer-group form ----------------------------------------------------------------------
// One launch forms the operand blocks of a few outer products p1 only (7 blocks each at two
// levels, 1 at one level), so the pipelined driver can start the products of the first group
// while the later groups' operands are still being formed. The outer row of the table is a
// run-time argument; the inner level stays compile-time.

template <int INNER, int ALGO, int SIDE, typename T>
// (two blocks per SM for the two-level Winograd table, whose sums need more than the 85 registers three would leave)
__global__ void __launch_bounds__(256, (INNER == 1 && ALGO == sched::kWinograd) ? 2 : 3)
    preadd_outer_kernel(const PreaddOuterParams p) {
  using OP = OuterPosition<INNER, ALGO, SIDE, T>;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= p.rows_blk * p.cols_vec) return;
  typename OP::Raw raw;
  float t[OP::NQ2][OP::VEC];
  const typename OP::Where w = OP::locate(p, idx);
  OP::fetch(p, blockIdx.y, blockIdx.z, w, raw);
  OP::reduce(p, blockIdx.y, raw, t);
  OP::store(p, blockIdx.y, blockIdx.z, w, t);
}

template <int INNER, int ALGO, int SIDE, typename T>
int launch_outer_one(const PreaddOuterArgs& a, cudaStream_t stream) {
  constexpr int VEC = Vec16<T>::N;
  PreaddOuterParams kp;
  kp.X = a.X;
  kp.out = a.out;
  kp.rows_blk = a.rows_blk;
  kp.cols_vec = a.cols_blk / VEC;
  kp.ld = a.ld;
  kp.strideX = a.strideX;
  kp.out_batch_blocks = sched::ipow(7, INNER + 1);
  kp.transposed = a.transposed;
  for (int g = 0; g < a.n_groups; ++g) {
    set_outer_terms(kp, g, ALGO, SIDE, a.groups[g]);
    kp.out_block0[g] = a.out_block0[g];
  }
  const int64_t total = kp.rows_blk * kp.cols_vec;
  const int64_t blocks = (total + 255) / 256;
  if (total > INT32_MAX || a.batch > 65535) return B200S_ERR_BAD_SHAPE;
  dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(a.n_groups), static_cast<unsigned>(a.batch));
  preadd_outer_kernel<INNER, ALGO, SIDE, T><<<grid, 256, 0, stream>>>(kp);
  B200S_CUDA_OK(cudaGetLastError());
  count_launch();
  return B200S_OK;
}

template <int INNER, int ALGO, int SIDE>
int launch_outer_dtype(const PreaddOuterArgs& a, cudaStream_t stream) {
  switch (a.dtype) {
    case B200S_BF16:
      return launch_outer_one<INNER, ALGO, SIDE, __nv_bfloat16>(a, stream);
    case B200S_FP16:
      return launch_outer_one<INNER, ALGO, SIDE, __half>(a, stream);
    case B200S_FP32:
      return launch_outer_one<INNER, ALGO, SIDE, float>(a, stream);
  }
  return B200S_ERR_BAD_DTYPE;
}

template <int INNER, int ALGO>
int launch_outer_side(const PreaddOuterArgs& a, cudaStream_t stream) {
  return a.side == 0 ? launch_outer_dtype<INNER, ALGO, sched::kSideA>(a, stream)
                     : launch_outer_dtype<INNER, ALGO, sched::kSideB>(a, stream);
}

}  // namespace

int launch_preadd(const PreaddArgs& a, cudaStream_t stream) {
  const size_t es = dtype_size(a.dtype);
  const int vec = static_cast<int>(16 / es);
  if (a.rows_blk <= 0 || a.cols_blk <= 0 || a.batch <= 0) return B200S_ERR_BAD_SHAPE;
  if (a.cols_blk % vec) return B200S_ERR_BAD_SHAPE;
  if ((a.ld * es) % 16 || (a.batch > 1 && (a.strideX * es) % 16)) return B200S_ERR_BAD_STRIDE;
  if ((reinterpret_cast<uintptr_t>(a.X) & 15u) || (reinterpret_cast<uintptr_t>(a.out) & 15u))
    return B200S_ERR_BAD_ALIGNMENT;
  const bool wino = a.algo == B200S_ALGO_WINOGRAD;
  if (!wino && a.algo != B200S_ALGO_CLASSIC) return B200S_ERR_BAD_ALGO;
  if (a.depth == 1)
    return wino ? launch_side<1, sched::kWinograd>(a, stream) : launch_side<1, sched::kClassic>(a, stream);
  if (a.depth == 2)
    return wino ? launch_side<2, sched::kWinograd>(a, stream) : launch_side<2, sched::kClassic>(a, stream);
  return B200S_ERR_BAD_DEPTH;
}

}  // namespace b200s

namespace b200s {

int launch_preadd_outer(const PreaddOuterArgs& a, cudaStream_t stream) {
  const size_t es = dtype_size(a.dtype);
  const int vec = static_cast<int>(16 / es);
  if (a.rows_blk <= 0 || a.cols_blk <= 0 || a.batch <= 0 || a.n_groups <= 0 || a.n_groups > 7)
    return B200S_ERR_BAD_SHAPE;
  if (a.cols_blk % vec) return B200S_ERR_BAD_SHAPE;
  if ((a.ld * es) % 16 || (a.batch > 1 && (a.strideX * es) % 16)) return B200S_ERR_BAD_STRIDE;
  if ((reinterpret_cast<uintptr_t>(a.X) & 15u) || (reinterpret_cast<uintptr_t>(a.out) & 15u))
    return B200S_ERR_BAD_ALIGNMENT;
  const bool wino = a.algo == B200S_ALGO_WINOGRAD;
  if (!wino && a.algo != B200S_ALGO_CLASSIC) return B200S_ERR_BAD_ALGO;
  if (a.depth == 1)
    return wino ? launch_outer_side<0, sched::kWinograd>(a, stream) : launch_outer_side<0, sched::kClassic>(a, stream);
  if (a.depth == 2)
    return wino ? launch_outer_side<1, sched::kWinograd>(a, stream) : launch_outer_side<1, sched::kClassic>(a, stream);
  return B200S_ERR_BAD_DEPTH;
}

}  // namespace b200s
