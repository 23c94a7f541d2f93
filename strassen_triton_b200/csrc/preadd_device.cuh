// Device code of the operand pre-addition, shared by the stand-alone passes (preadd.cu) and by the
// adder warps of the fused Strassen kernel (gemm_sm100.cu): vector loads/stores with fp32 widening,
// the compile-time walk over the coefficient tables, and the per-position body of the outer-group
// form. Both users run the very same arithmetic, so their results are bit-identical.
//
// The additions are those of fixed_strassen_fp32_agg.py:26-44 (one level) and :77-96 (S1..S10).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <utility>

#include "mem_hints.cuh"
#include "schedule.h"

namespace b200s {
namespace pre {

template <typename T>
struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
};

// 16 bytes of T widened to fp32.
template <typename T>
__device__ __forceinline__ void unpack_vec(const uint4& v, float (&f)[Vec16<T>::N]);
template <>
__device__ __forceinline__ void unpack_vec<float>(const uint4& v, float (&f)[4]) {
  f[0] = __uint_as_float(v.x), f[1] = __uint_as_float(v.y), f[2] = __uint_as_float(v.z), f[3] = __uint_as_float(v.w);
}
template <>
__device__ __forceinline__ void unpack_vec<__nv_bfloat16>(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void unpack_vec<__half>(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    f[2 * i] = t.x, f[2 * i + 1] = t.y;
  }
}

// fp32 values rounded to T (to nearest even) and packed into 16 bytes.
template <typename T>
__device__ __forceinline__ uint4 pack_vec(const float (&f)[Vec16<T>::N]);
template <>
__device__ __forceinline__ uint4 pack_vec<float>(const float (&f)[4]) {
  return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
}
template <>
__device__ __forceinline__ uint4 pack_vec<__nv_bfloat16>(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 t = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&t);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
template <>
__device__ __forceinline__ uint4 pack_vec<__half>(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 t = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&t);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

template <typename T, class A = mem::Plain>
__device__ __forceinline__ void load_vec(const T* ptr, float (&f)[Vec16<T>::N], const A& acc = A{}) {
  unpack_vec<T>(mem::ld16_readonly(ptr, acc), f);
}
template <typename T, class A = mem::Plain>
__device__ __forceinline__ void store_vec(T* ptr, const float (&f)[Vec16<T>::N], const A& acc = A{}) {
  mem::st16(ptr, pack_vec<T>(f), acc);
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
template <typename T, int N, class A = mem::Plain>
__device__ __forceinline__ void store_n(T* ptr, const float (&f)[N], const A& acc = A{}) {
  if constexpr (N == Vec16<T>::N)
    store_vec<T>(ptr, f, acc);
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

  template <int P, class A, int... Qs>
  static __device__ __forceinline__ void one_product(const float (&x)[NQ][VEC], T* out_blk0, int64_t blk_elems,
                                                     const A& access, std::integer_sequence<int, Qs...>) {
    float acc[VEC];
    bool first = true;
    (add_term<P, Qs>(x, acc, first), ...);
    store_n<T, VEC>(out_blk0 + P * blk_elems, acc, access);
  }

  template <class A = mem::Plain, int... Ps>
  static __device__ __forceinline__ void all_products(const float (&x)[NQ][VEC], T* out_blk0, int64_t blk_elems,
                                                      std::integer_sequence<int, Ps...>, const A& access = A{}) {
    (one_product<Ps>(x, out_blk0, blk_elems, access, std::make_integer_sequence<int, NQ>{}), ...);
  }
};


// ---- outer-group form ----------------------------------------------------------------------
// Operand blocks of a few outer products p1 only (7 blocks each at two levels, 1 at one level).
// The outer row of the table is a run-time argument (a list of signed quadrants); the inner level
// stays compile-time.

struct PreaddOuterParams {
  const void* X;
  void* out;
  int64_t rows_blk, cols_vec;  // finest block rows, 16-byte vectors per finest block row
  int64_t ld, strideX;
  int64_t out_batch_blocks;    // blocks per batch item in `out` (7^depth)
  int32_t transposed;
  int8_t n_terms[7];           // [listed group]: non-zero entries of its outer table row
  int8_t term_quad[7][4];      // their outer quadrants, ascending
  int8_t term_sign[7][4];      // +1 / -1
  int32_t out_block0[7];       // first output block of each listed group
};

// Fills the term list of listed group g from row p1 of the outer table.
inline void set_outer_terms(PreaddOuterParams& p, int g, int algo, int side, int p1) {
  int n = 0;
  for (int q = 0; q < 4; ++q) {
    const int c = sched::uv1(algo, side, p1, q);
    if (c != 0) {
      p.term_quad[g][n] = static_cast<int8_t>(q);
      p.term_sign[g][n] = static_cast<int8_t>(c);
      ++n;
    }
  }
  p.n_terms[g] = static_cast<int8_t>(n);
}

// One 16-byte position `idx` (< rows_blk * cols_vec) of listed group g of batch item z, in three
// steps so that a caller can keep the loads of the next position in flight while it finishes this
// one: fetch (the raw 16-byte loads), reduce (the level-1 sum of the outer quadrants in fp32) and
// store (the inner level's seven sums, each rounded once).
template <int INNER, int ALGO, int SIDE, typename T>
struct OuterPosition {
  static constexpr int VEC = Vec16<T>::N;
  static constexpr int NQ2 = INNER ? 4 : 1;
  static constexpr int NP2 = INNER ? 7 : 1;
  static constexpr int MAXT = ALGO == sched::kClassic ? 2 : 4;  // most non-zeros in a row of U or V
  struct Raw {
    uint4 v[MAXT][NQ2];
  };

  // Where position idx sits inside one block: element offset in the operand (row * ld + column) and in
  // an output block (row * cols_blk + column). Positions per block fit 32 bits (the launchers check).
  struct Where {
    int64_t in_off, out_off;
  };
  static __device__ __forceinline__ Where locate(const PreaddOuterParams& p, int64_t idx) {
    const uint32_t cols_vec = static_cast<uint32_t>(p.cols_vec);
    const uint32_t row = static_cast<uint32_t>(idx) / cols_vec;
    const uint32_t cv = static_cast<uint32_t>(idx) - row * cols_vec;
    Where w;
    w.in_off = static_cast<int64_t>(row) * p.ld + static_cast<int64_t>(cv) * VEC;
    w.out_off = (static_cast<int64_t>(row) * cols_vec + cv) * VEC;
    return w;
  }

  template <class A = mem::Plain>
  static __device__ __forceinline__ void fetch(const PreaddOuterParams& p, int g, int z, const Where& w, Raw& raw,
                                               const A& access = A{}) {
    const int64_t cols_blk = p.cols_vec * VEC;
    const T* X = static_cast<const T*>(p.X) + static_cast<int64_t>(z) * p.strideX + w.in_off;
    const int nt = p.n_terms[g];
#pragma unroll
    for (int j = 0; j < MAXT; ++j) {
      if (j < nt) {
        const int q1 = p.term_quad[g][j];
#pragma unroll
        for (int q2 = 0; q2 < NQ2; ++q2) {
          // position of (outer q1, inner q2) in the block grid, in storage orientation
          const int lr = INNER ? 2 * (q1 >> 1) + (q2 >> 1) : (q1 >> 1);
          const int lc = INNER ? 2 * (q1 & 1) + (q2 & 1) : (q1 & 1);
          const int sr = p.transposed ? lc : lr;
          const int sc = p.transposed ? lr : lc;
          raw.v[j][q2] = mem::ld16_readonly(X + sr * p.rows_blk * p.ld + sc * cols_blk, access);
        }
      }
    }
  }

  static __device__ __forceinline__ void reduce(const PreaddOuterParams& p, int g, const Raw& raw,
                                                float (&t)[NQ2][VEC]) {
    const int nt = p.n_terms[g];
#pragma unroll
    for (int j = 0; j < MAXT; ++j) {
      if (j < nt) {
        const bool plus = p.term_sign[g][j] > 0;
#pragma unroll
        for (int q2 = 0; q2 < NQ2; ++q2) {
          float x[VEC];
          unpack_vec<T>(raw.v[j][q2], x);
          if (j == 0) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) t[q2][i] = plus ? x[i] : -x[i];
          } else {
#pragma unroll
            for (int i = 0; i < VEC; ++i) t[q2][i] = plus ? t[q2][i] + x[i] : t[q2][i] - x[i];
          }
        }
      }
    }
  }

  template <class A = mem::Plain>
  static __device__ __forceinline__ void store(const PreaddOuterParams& p, int g, int z, const Where& w,
                                               const float (&t)[NQ2][VEC], const A& access = A{}) {
    const int64_t blk_elems = p.rows_blk * p.cols_vec * VEC;
    T* out = static_cast<T*>(p.out) + (static_cast<int64_t>(z) * p.out_batch_blocks + p.out_block0[g]) * blk_elems +
             w.out_off;
    if constexpr (INNER) {
      // the inner level: the same compile-time table walk as the single-pass kernel at depth 1
      Preadd<1, ALGO, SIDE, T>::all_products(t, out, blk_elems, std::make_integer_sequence<int, NP2>{}, access);
    } else {
      store_vec<T>(out, t[0], access);
    }
  }
};

}  // namespace pre
}  // namespace b200s
