// Recombination pass of the Strassen pipeline.
//
// Each thread reads one position (a 16-byte vector; a pair of 16-bit products in the two-level
// pass) of all 7^depth product blocks, accumulates the 4^depth signed output sums in fp32
// registers (all levels at once) and writes, or adds into, the 4^depth blocks of C, rounding once
// to the output dtype. Every product element is read exactly once and every element of C written
// exactly once; a warp's accesses are contiguous.
//
// It carries the post-additions and the quadrant assembly of the reference:
// fixed_strassen_fp32_agg.py:47-56 and :115-123 (products widened to fp32, summed, rounded to
// base_dtype, vstack/hstack). With beta = 1 it adds into C as the reference's run_* launchers do
// (strassen.py:184-192).

#include <cuda_runtime.h>

#include <mutex>
#include <utility>

#include "combine_device.cuh"
#include "common.h"
#include "schedule.h"

namespace b200s {

namespace {

using namespace comb;

struct CombineKernelParams {
  const void* products;
  void* C;
  int64_t Mb, nb_vec;  // block rows, positions (Combine::VEC elements each) per block row
  int64_t ldc, strideC;
  int32_t out_dtype, beta, vec_ok;
  const void* bias;
};

__device__ __forceinline__ float bias_at(const void* bias, int out_dtype, int64_t col) {
  if (out_dtype == B200S_BF16) return __bfloat162float(__ldg(static_cast<const __nv_bfloat16*>(bias) + col));
  if (out_dtype == B200S_FP16) return __half2float(__ldg(static_cast<const __half*>(bias) + col));
  return __ldg(static_cast<const float*>(bias) + col);
}

template <int DEPTH, int ALGO, typename TP>
__global__ void __launch_bounds__(256, DEPTH == 2 && sizeof(TP) == 4 ? 2 : 3) combine_kernel(const CombineKernelParams p) {
  using CB = Combine<DEPTH, ALGO, TP>;
  constexpr int NQ = CB::NQ, NP = CB::NP, VEC = CB::VEC;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= p.Mb * p.nb_vec) return;
  const int64_t row = idx / p.nb_vec;
  const int64_t cv = idx - row * p.nb_vec;
  const int64_t Nb = p.nb_vec * VEC;
  const int64_t blk_elems = p.Mb * Nb;

  float acc[NQ][VEC];
#pragma unroll
  for (int r = 0; r < NQ; ++r)
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[r][i] = 0.f;

  const TP* prod0 =
      static_cast<const TP*>(p.products) + static_cast<int64_t>(blockIdx.y) * NP * blk_elems + row * Nb + cv * VEC;
  CB::all_products(prod0, blk_elems, acc, std::make_integer_sequence<int, NP>{});

#pragma unroll
  for (int r = 0; r < NQ; ++r) {
    const int64_t crow = sched::block_row(DEPTH, r) * p.Mb + row;
    const int64_t ccol = sched::block_col(DEPTH, r) * Nb + cv * VEC;
    if (p.bias != nullptr) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[r][i] += bias_at(p.bias, p.out_dtype, ccol + i);
    }
    const int64_t off = static_cast<int64_t>(blockIdx.y) * p.strideC + crow * p.ldc + ccol;
    if (p.out_dtype == B200S_BF16)
      store_out<__nv_bfloat16, VEC>(static_cast<__nv_bfloat16*>(p.C) + off, acc[r], p.beta != 0, p.vec_ok != 0);
    else if (p.out_dtype == B200S_FP16)
      store_out<__half, VEC>(static_cast<__half*>(p.C) + off, acc[r], p.beta != 0, p.vec_ok != 0);
    else
      store_out<float, VEC>(static_cast<float*>(p.C) + off, acc[r], p.beta != 0, p.vec_ok != 0);
  }
}

template <int DEPTH, int ALGO, typename TP>
int launch_one(const CombineArgs& a, cudaStream_t stream) {
  constexpr int VEC = Combine<DEPTH, ALGO, TP>::VEC;
  CombineKernelParams kp;
  kp.products = a.products;
  kp.C = a.C;
  kp.Mb = a.Mb;
  kp.nb_vec = a.Nb / VEC;
  kp.ldc = a.ldc;
  kp.strideC = a.strideC;
  kp.out_dtype = a.out_dtype;
  kp.beta = a.beta;
  kp.bias = a.bias;
  const size_t oes = dtype_size(a.out_dtype);
  kp.vec_ok = ((reinterpret_cast<uintptr_t>(a.C) & 15u) == 0) && ((a.ldc * oes) % 16 == 0) &&
              ((a.Nb * oes) % 16 == 0) && (a.batch == 1 || (a.strideC * oes) % 16 == 0);
  if (a.Nb % VEC) return B200S_ERR_BAD_SHAPE;
  const int64_t total = kp.Mb * kp.nb_vec;
  const int64_t blocks = (total + 255) / 256;
  if (blocks > INT32_MAX || a.batch > 65535) return B200S_ERR_BAD_SHAPE;
  dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(a.batch));
  combine_kernel<DEPTH, ALGO, TP><<<grid, 256, 0, stream>>>(kp);
  B200S_CUDA_OK(cudaGetLastError());
  count_launch();
  return B200S_OK;
}

template <int DEPTH, int ALGO>
int launch_dtype(const CombineArgs& a, cudaStream_t stream) {
  switch (a.prod_dtype) {
    case B200S_BF16:
      return launch_one<DEPTH, ALGO, __nv_bfloat16>(a, stream);
    case B200S_FP16:
      return launch_one<DEPTH, ALGO, __half>(a, stream);
    case B200S_FP32:
      return launch_one<DEPTH, ALGO, float>(a, stream);
  }
  return B200S_ERR_BAD_DTYPE;
}

// ---- recombination fused with the exchange of a row-sharded product ------------------------------
// Same arithmetic as combine_kernel, but every output vector is stored to several destinations:
// this GPU's copy of C and the copies of its peers, reached through peer-mapped pointers (plain
// st.global over NVLink). The all-gather of a row-sharded product then costs no separate pass: the
// finished rows leave the SM straight for every GPU's memory.
struct CombinePeersParams {
  const void* products;
  void* dst[8];
  int32_t n_dst;
  int64_t Mb, nb_vec;
  int64_t ldc;
  int32_t out_dtype, vec_ok;
};

template <int DEPTH, int ALGO, typename TP>
__global__ void __launch_bounds__(256, DEPTH == 2 && sizeof(TP) == 4 ? 2 : 3) combine_peers_kernel(const CombinePeersParams p) {
  using CB = Combine<DEPTH, ALGO, TP>;
  constexpr int NQ = CB::NQ, NP = CB::NP, VEC = CB::VEC;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= p.Mb * p.nb_vec) return;
  const int64_t row = idx / p.nb_vec;
  const int64_t cv = idx - row * p.nb_vec;
  const int64_t Nb = p.nb_vec * VEC;
  const int64_t blk_elems = p.Mb * Nb;
  float acc[NQ][VEC];
#pragma unroll
  for (int r = 0; r < NQ; ++r)
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[r][i] = 0.f;
  const TP* prod0 = static_cast<const TP*>(p.products) + row * Nb + cv * VEC;
  CB::all_products(prod0, blk_elems, acc, std::make_integer_sequence<int, NP>{});
#pragma unroll
  for (int r = 0; r < NQ; ++r) {
    const int64_t off = (sched::block_row(DEPTH, r) * p.Mb + row) * p.ldc + sched::block_col(DEPTH, r) * Nb + cv * VEC;
#pragma unroll 1
    for (int d = 0; d < p.n_dst; ++d) {
      if (p.out_dtype == B200S_BF16)
        store_out<__nv_bfloat16, VEC>(static_cast<__nv_bfloat16*>(p.dst[d]) + off, acc[r], false, p.vec_ok != 0);
      else if (p.out_dtype == B200S_FP16)
        store_out<__half, VEC>(static_cast<__half*>(p.dst[d]) + off, acc[r], false, p.vec_ok != 0);
      else
        store_out<float, VEC>(static_cast<float*>(p.dst[d]) + off, acc[r], false, p.vec_ok != 0);
    }
  }
}

template <int DEPTH, int ALGO, typename TP>
int launch_peers_one(const CombineArgs& a, void* const* dst, int n_dst, cudaStream_t stream) {
  constexpr int VEC = Combine<DEPTH, ALGO, TP>::VEC;
  CombinePeersParams kp;
  kp.products = a.products;
  kp.n_dst = n_dst;
  const size_t oes = dtype_size(a.out_dtype);
  bool vec_ok = ((a.ldc * oes) % 16 == 0) && ((a.Nb * oes) % 16 == 0);
  for (int d = 0; d < 8; ++d) {
    kp.dst[d] = d < n_dst ? dst[d] : nullptr;
    if (d < n_dst && (reinterpret_cast<uintptr_t>(dst[d]) & 15u)) vec_ok = false;
  }
  kp.Mb = a.Mb;
  kp.nb_vec = a.Nb / VEC;
  kp.ldc = a.ldc;
  kp.out_dtype = a.out_dtype;
  kp.vec_ok = vec_ok;
  if (a.Nb % VEC) return B200S_ERR_BAD_SHAPE;
  const int64_t blocks = (kp.Mb * kp.nb_vec + 255) / 256;
  if (blocks > INT32_MAX) return B200S_ERR_BAD_SHAPE;
  combine_peers_kernel<DEPTH, ALGO, TP><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(kp);
  B200S_CUDA_OK(cudaGetLastError());
  count_launch();
  return B200S_OK;
}

template <int DEPTH, int ALGO>
int launch_peers_dtype(const CombineArgs& a, void* const* dst, int n_dst, cudaStream_t stream) {
  switch (a.prod_dtype) {
    case B200S_BF16:
      return launch_peers_one<DEPTH, ALGO, __nv_bfloat16>(a, dst, n_dst, stream);
    case B200S_FP16:
      return launch_peers_one<DEPTH, ALGO, __half>(a, dst, n_dst, stream);
    case B200S_FP32:
      return launch_peers_one<DEPTH, ALGO, float>(a, dst, n_dst, stream);
  }
  return B200S_ERR_BAD_DTYPE;
}

// ---- outer-quadrant form --------------------------------------------------------------------
// One launch writes a few outer quadrants of C only, reading just the product groups that feed
// them, so the pipelined driver can recombine a quadrant as soon as its last group is done.

template <int INNER, int ALGO, typename TP>
__global__ void __launch_bounds__(256, 3) combine_outer_kernel(const CombineOuterParams p) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= p.Mb * p.nb_vec) return;
  outer_position<INNER, ALGO, TP>(p, blockIdx.y, blockIdx.z, idx);
}

template <int INNER, int ALGO, typename TP>
int launch_outer_one(const CombineOuterArgs& a, cudaStream_t stream) {
  constexpr int VEC = PVec<TP>::N;
  CombineOuterParams kp;
  kp.products = a.products;
  kp.C = a.C;
  kp.Mb = a.Mb;
  kp.nb_vec = a.Nb / VEC;
  kp.ldc = a.ldc;
  kp.strideC = a.strideC;
  kp.batch_blocks = sched::ipow(7, INNER + 1);
  kp.out_dtype = a.out_dtype;
  kp.beta = a.beta;
  const size_t oes = dtype_size(a.out_dtype);
  kp.vec_ok = ((reinterpret_cast<uintptr_t>(a.C) & 15u) == 0) && ((a.ldc * oes) % 16 == 0) &&
              ((a.Nb * oes) % 16 == 0) && (a.batch == 1 || (a.strideC * oes) % 16 == 0);
  for (int e = 0; e < a.n_quads; ++e) {
    kp.quad[e] = static_cast<int8_t>(a.quads[e]);
    for (int p1 = 0; p1 < 7; ++p1) kp.coef[e][p1] = static_cast<int8_t>(sched::w1(ALGO, a.quads[e], p1));
  }
  for (int p1 = 0; p1 < 7; ++p1) kp.group_block0[p1] = a.group_block0[p1];
  const int64_t total = kp.Mb * kp.nb_vec;
  const int64_t blocks = (total + 255) / 256;
  if (total > INT32_MAX || a.batch > 65535) return B200S_ERR_BAD_SHAPE;
  dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(a.n_quads), static_cast<unsigned>(a.batch));
  combine_outer_kernel<INNER, ALGO, TP><<<grid, 256, 0, stream>>>(kp);
  B200S_CUDA_OK(cudaGetLastError());
  count_launch();
  return B200S_OK;
}

template <int INNER, int ALGO>
int launch_outer_dtype(const CombineOuterArgs& a, cudaStream_t stream) {
  switch (a.prod_dtype) {
    case B200S_BF16:
      return launch_outer_one<INNER, ALGO, __nv_bfloat16>(a, stream);
    case B200S_FP16:
      return launch_outer_one<INNER, ALGO, __half>(a, stream);
    case B200S_FP32:
      return launch_outer_one<INNER, ALGO, float>(a, stream);
  }
  return B200S_ERR_BAD_DTYPE;
}

}  // namespace

int launch_combine(const CombineArgs& a, cudaStream_t stream) {
  const size_t pes = dtype_size(a.prod_dtype);
  const int vec = static_cast<int>(16 / pes);
  if (a.Mb <= 0 || a.Nb <= 0 || a.batch <= 0) return B200S_ERR_BAD_SHAPE;
  if (a.Nb % vec) return B200S_ERR_BAD_SHAPE;
  if (reinterpret_cast<uintptr_t>(a.products) & 15u) return B200S_ERR_BAD_ALIGNMENT;
  const bool wino = a.algo == B200S_ALGO_WINOGRAD;
  if (!wino && a.algo != B200S_ALGO_CLASSIC) return B200S_ERR_BAD_ALGO;
  if (a.depth == 1)
    return wino ? launch_dtype<1, sched::kWinograd>(a, stream) : launch_dtype<1, sched::kClassic>(a, stream);
  if (a.depth == 2)
    return wino ? launch_dtype<2, sched::kWinograd>(a, stream) : launch_dtype<2, sched::kClassic>(a, stream);
  return B200S_ERR_BAD_DEPTH;
}

}  // namespace b200s

namespace b200s {

int launch_combine_outer(const CombineOuterArgs& a, cudaStream_t stream) {
  const size_t pes = dtype_size(a.prod_dtype);
  const int vec = static_cast<int>(16 / pes);
  if (a.Mb <= 0 || a.Nb <= 0 || a.batch <= 0 || a.n_quads <= 0 || a.n_quads > 4) return B200S_ERR_BAD_SHAPE;
  if (a.Nb % vec) return B200S_ERR_BAD_SHAPE;
  if (reinterpret_cast<uintptr_t>(a.products) & 15u) return B200S_ERR_BAD_ALIGNMENT;
  const bool wino = a.algo == B200S_ALGO_WINOGRAD;
  if (!wino && a.algo != B200S_ALGO_CLASSIC) return B200S_ERR_BAD_ALGO;
  if (a.depth == 1)
    return wino ? launch_outer_dtype<0, sched::kWinograd>(a, stream) : launch_outer_dtype<0, sched::kClassic>(a, stream);
  if (a.depth == 2)
    return wino ? launch_outer_dtype<1, sched::kWinograd>(a, stream) : launch_outer_dtype<1, sched::kClassic>(a, stream);
  return B200S_ERR_BAD_DEPTH;
}

}  // namespace b200s

namespace b200s {

int launch_combine_peers(const CombineArgs& a, void* const* dst, int n_dst, cudaStream_t stream) {
  const size_t pes = dtype_size(a.prod_dtype);
  if (a.Mb <= 0 || a.Nb <= 0 || a.batch != 1 || n_dst < 1 || n_dst > 8 || !dst) return B200S_ERR_BAD_SHAPE;
  if (a.Nb % static_cast<int>(16 / pes)) return B200S_ERR_BAD_SHAPE;
  if (reinterpret_cast<uintptr_t>(a.products) & 15u) return B200S_ERR_BAD_ALIGNMENT;
  for (int d = 0; d < n_dst; ++d)
    if (!dst[d]) return B200S_ERR_NULL_POINTER;
  const bool wino = a.algo == B200S_ALGO_WINOGRAD;
  if (!wino && a.algo != B200S_ALGO_CLASSIC) return B200S_ERR_BAD_ALGO;
  if (a.depth == 1)
    return wino ? launch_peers_dtype<1, sched::kWinograd>(a, dst, n_dst, stream)
                : launch_peers_dtype<1, sched::kClassic>(a, dst, n_dst, stream);
  if (a.depth == 2)
    return wino ? launch_peers_dtype<2, sched::kWinograd>(a, dst, n_dst, stream)
                : launch_peers_dtype<2, sched::kClassic>(a, dst, n_dst, stream);
  return B200S_ERR_BAD_DEPTH;
}

}  // namespace b200s

namespace b200s {

namespace {
// Copies a contiguous byte range to several destinations (other GPUs' memory mapped into this
// process). One 256-thread block per SM with a handful of registers and no shared memory, so it
// runs beside a resident GEMM CTA: the rows of a finished panel cross NVLink while the tensor
// cores work on the next panel.
struct PushParams {
  const uint4* src;
  uint4* dst[8];
  int32_t n_dst;
  int64_t n_vec;
};

__global__ void __launch_bounds__(256) push_rows_kernel(const PushParams p) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < p.n_vec; i += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = __ldcs(p.src + i + u * stride);
#pragma unroll 1
    for (int d = 0; d < p.n_dst; ++d)
#pragma unroll
      for (int u = 0; u < 4; ++u) p.dst[d][i + u * stride] = v[u];
  }
  for (; i < p.n_vec; i += stride) {
    const uint4 v = __ldcs(p.src + i);
    for (int d = 0; d < p.n_dst; ++d) p.dst[d][i] = v;
  }
}
}  // namespace

int launch_push_rows(const void* src, void* const* dst, int n_dst, size_t bytes, cudaStream_t stream) {
  if (!src || !dst) return B200S_ERR_NULL_POINTER;
  if (n_dst < 1 || n_dst > 8 || bytes == 0 || bytes % 16) return B200S_ERR_BAD_SHAPE;
  if (reinterpret_cast<uintptr_t>(src) & 15u) return B200S_ERR_BAD_ALIGNMENT;
  PushParams kp;
  kp.src = static_cast<const uint4*>(src);
  kp.n_dst = n_dst;
  kp.n_vec = static_cast<int64_t>(bytes / 16);
  for (int d = 0; d < 8; ++d) {
    kp.dst[d] = d < n_dst ? static_cast<uint4*>(dst[d]) : nullptr;
    if (d < n_dst && (!dst[d] || (reinterpret_cast<uintptr_t>(dst[d]) & 15u))) return B200S_ERR_BAD_ALIGNMENT;
  }
  const int sms = sm_count();
  if (sms <= 0) return B200S_ERR_NO_DEVICE;
  int64_t blocks = (kp.n_vec + 255) / 256;
  if (blocks > sms) blocks = sms;
  // Ask for the same shared-memory carve-out the GEMM CTAs run with, so that an SM does not have
  // to drain before it can host a block of this kernel beside one of them.
  static std::once_flag carve;
  std::call_once(carve, [] {
    cudaFuncSetAttribute(push_rows_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  });
  push_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(kp);
  B200S_CUDA_OK(cudaGetLastError());
  count_launch();
  return B200S_OK;
}

}  // namespace b200s
