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

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <utility>

#include "common.h"
#include "schedule.h"

namespace b200s {

namespace {

struct PreaddKernelParams {
  const void* X;
  void* out;
  int64_t rows_blk, cols_vec;  // block rows, 16-byte vectors per block row
  int64_t ld;                  // elements
  int64_t strideX;             // elements
  int32_t transposed;
};

template <typename T>
struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
};

template <typename T>
__device__ __forceinline__ void load_vec(const T* ptr, float (&f)[Vec16<T>::N]);
template <>
__device__ __forceinline__ void load_vec<float>(const float* ptr, float (&f)[4]) {
  const float4 v = __ldg(reinterpret_cast<const float4*>(ptr));
  f[0] = v.x, f[1] = v.y, f[2] = v.z, f[3] = v.w;
}
template <>
__device__ __forceinline__ void load_vec<__nv_bfloat16>(const __nv_bfloat16* ptr, float (&f)[8]) {
  const uint4 v = __ldg(reinterpret_cast<const uint4*>(ptr));
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void load_vec<__half>(const __half* ptr, float (&f)[8]) {
  const uint4 v = __ldg(reinterpret_cast<const uint4*>(ptr));
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    f[2 * i] = t.x, f[2 * i + 1] = t.y;
  }
}

template <typename T>
__device__ __forceinline__ void store_vec(T* ptr, const float (&f)[Vec16<T>::N]);
template <>
__device__ __forceinline__ void store_vec<float>(float* ptr, const float (&f)[4]) {
  *reinterpret_cast<float4*>(ptr) = make_float4(f[0], f[1], f[2], f[3]);
}
template <>
__device__ __forceinline__ void store_vec<__nv_bfloat16>(__nv_bfloat16* ptr, const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 t = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&t);
  }
  *reinterpret_cast<uint4*>(ptr) = make_uint4(w[0], w[1], w[2], w[3]);
}
template <>
__device__ __forceinline__ void store_vec<__half>(__half* ptr, const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 t = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&t);
  }
  *reinterpret_cast<uint4*>(ptr) = make_uint4(w[0], w[1], w[2], w[3]);
}

// 8-byte forms for four 16-bit elements: the depth-2 single-pass kernel holds 16 x 4 inputs
// instead of 16 x 8, so three times as many threads are resident and keep loads in flight.
__device__ __forceinline__ void load_vec4(const __nv_bfloat16* ptr, float (&f)[4]) {
  const uint2 v = __ldg(reinterpret_cast<const uint2*>(ptr));
  f[0] = __uint_as_float(v.x << 16), f[1] = __uint_as_float(v.x & 0xffff0000u);
  f[2] = __uint_as_float(v.y << 16), f[3] = __uint_as_float(v.y & 0xffff0000u);
}
__device__ __forceinline__ void load_vec4(const __half* ptr, float (&f)[4]) {
  const uint2 v = __ldg(reinterpret_cast<const uint2*>(ptr));
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
  f[0] = a.x, f[1] = a.y, f[2] = b.x, f[3] = b.y;
}
__device__ __forceinline__ void load_vec4(const float* ptr, float (&f)[4]) { load_vec<float>(ptr, f); }
__device__ __forceinline__ void store_vec4(__nv_bfloat16* ptr, const float (&f)[4]) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
  *reinterpret_cast<uint2*>(ptr) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}
__device__ __forceinline__ void store_vec4(__half* ptr, const float (&f)[4]) {
  const __half2 a = __floats2half2_rn(f[0], f[1]), b = __floats2half2_rn(f[2], f[3]);
  *reinterpret_cast<uint2*>(ptr) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}
__device__ __forceinline__ void store_vec4(float* ptr, const float (&f)[4]) { store_vec<float>(ptr, f); }

template <typename T, int N>
__device__ __forceinline__ void load_n(const T* ptr, float (&f)[N]) {
  if constexpr (N == Vec16<T>::N)
    load_vec<T>(ptr, f);
  else
    load_vec4(ptr, f);
}
template <typename T, int N>
__device__ __forceinline__ void store_n(T* ptr, const float (&f)[N]) {
  if constexpr (N == Vec16<T>::N)
    store_vec<T>(ptr, f);
  else
    store_vec4(ptr, f);
}

template <int DEPTH, int ALGO, int SIDE, typename T, int VEC_ = Vec16<T>::N>
struct Preadd {
  static constexpr int NQ = sched::ipow(4, DEPTH);
  static constexpr int NP = sched::ipow(7, DEPTH);
  static constexpr int VEC = VEC_;

  template <int P, int Q>
  static __device__ __forceinline__ void add_term(const float (&x)[NQ][VEC], float (&acc)[VEC], bool& first) {
    constexpr int c = sched::uv(ALGO, SIDE, DEPTH, P, Q);
    if constexpr (c != 0) {
      if (first) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] = c > 0 ? x[Q][i] : -x[Q][i];
        first = false;
      } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] = c > 0 ? acc[i] + x[Q][i] : acc[i] - x[Q][i];
      }
    }
  }

  template <int P, int... Qs>
  static __device__ __forceinline__ void one_product(const float (&x)[NQ][VEC], T* out_blk0, int64_t blk_elems,
                                                     std::integer_sequence<int, Qs...>) {
    float acc[VEC];
    bool first = true;
    (add_term<P, Qs>(x, acc, first), ...);
    store_n<T, VEC>(out_blk0 + P * blk_elems, acc);
  }

  template <int... Ps>
  static __device__ __forceinline__ void all_products(const float (&x)[NQ][VEC], T* out_blk0, int64_t blk_elems,
                                                      std::integer_sequence<int, Ps...>) {
    (one_product<Ps>(x, out_blk0, blk_elems, std::make_integer_sequence<int, NQ>{}), ...);
  }
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

struct PreaddOuterParams {
  const void* X;
  void* out;
  int64_t rows_blk, cols_vec;  // finest block rows, 16-byte vectors per finest block row
  int64_t ld, strideX;
  int64_t out_batch_blocks;    // blocks per batch item in `out` (7^depth)
  int32_t transposed;
  int8_t coef[7][4];           // [listed group][outer quadrant]
  int32_t out_block0[7];       // first output block of each listed group
};

template <int INNER, int ALGO, int SIDE, typename T>
__global__ void __launch_bounds__(256, 3) preadd_outer_kernel(const PreaddOuterParams p) {
  constexpr int VEC = Vec16<T>::N;
  constexpr int NQ2 = INNER ? 4 : 1;
  constexpr int NP2 = INNER ? 7 : 1;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= p.rows_blk * p.cols_vec) return;
  const int64_t row = idx / p.cols_vec;
  const int64_t cv = idx - row * p.cols_vec;
  const int64_t cols_blk = p.cols_vec * VEC;
  const int g = blockIdx.y;
  const T* X = static_cast<const T*>(p.X) + static_cast<int64_t>(blockIdx.z) * p.strideX;

  float t[NQ2][VEC];
#pragma unroll
  for (int q2 = 0; q2 < NQ2; ++q2) {
    bool first = true;
#pragma unroll
    for (int q1 = 0; q1 < 4; ++q1) {
      const int c = p.coef[g][q1];
      if (c != 0) {
        // position of (outer q1, inner q2) in the block grid, in storage orientation
        const int lr = INNER ? 2 * (q1 >> 1) + (q2 >> 1) : (q1 >> 1);
        const int lc = INNER ? 2 * (q1 & 1) + (q2 & 1) : (q1 & 1);
        const int sr = p.transposed ? lc : lr;
        const int sc = p.transposed ? lr : lc;
        float x[VEC];
        load_vec<T>(X + (sr * p.rows_blk + row) * p.ld + sc * cols_blk + cv * VEC, x);
        if (first) {
#pragma unroll
          for (int i = 0; i < VEC; ++i) t[q2][i] = c > 0 ? x[i] : -x[i];
          first = false;
        } else {
#pragma unroll
          for (int i = 0; i < VEC; ++i) t[q2][i] = c > 0 ? t[q2][i] + x[i] : t[q2][i] - x[i];
        }
      }
    }
  }
  const int64_t blk_elems = p.rows_blk * cols_blk;
  T* out = static_cast<T*>(p.out) +
           (static_cast<int64_t>(blockIdx.z) * p.out_batch_blocks + p.out_block0[g]) * blk_elems + row * cols_blk +
           cv * VEC;
  if constexpr (INNER) {
    // the inner level: the same compile-time table walk as the single-pass kernel at depth 1
    Preadd<1, ALGO, SIDE, T>::all_products(t, out, blk_elems, std::make_integer_sequence<int, NP2>{});
  } else {
    store_vec<T>(out, t[0]);
  }
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
    for (int q = 0; q < 4; ++q) kp.coef[g][q] = static_cast<int8_t>(sched::uv1(ALGO, SIDE, a.groups[g], q));
    kp.out_block0[g] = a.out_block0[g];
  }
  const int64_t total = kp.rows_blk * kp.cols_vec;
  const int64_t blocks = (total + 255) / 256;
  if (blocks > INT32_MAX || a.batch > 65535) return B200S_ERR_BAD_SHAPE;
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
