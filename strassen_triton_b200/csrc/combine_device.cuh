// Device code of the recombination, shared by the stand-alone passes (combine.cu) and by the adder
// warps of the fused Strassen kernel (gemm_sm100.cu): product loads with fp32 widening, the
// compile-time walk over the recombination table, output stores, and the per-position body of the
// outer-quadrant form. Both users run the very same arithmetic, so their results are bit-identical.
//
// The additions are those of fixed_strassen_fp32_agg.py:47-56 and :115-123.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <utility>

#include "../../include/b200s.h"
#include "mem_hints.cuh"
#include "preadd_device.cuh"
#include "schedule.h"

namespace b200s {
namespace comb {

template <typename T>
struct PVec {
  static constexpr int N = 16 / sizeof(T);
};

// Two 16-bit products packed in one 32-bit word, widened to fp32.
__device__ __forceinline__ void unpack_pair(uint32_t w, const __nv_bfloat16*, float (&f)[2]) {
  f[0] = __uint_as_float(w << 16), f[1] = __uint_as_float(w & 0xffff0000u);
}
__device__ __forceinline__ void unpack_pair(uint32_t w, const __half*, float (&f)[2]) {
  const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&w));
  f[0] = v.x, f[1] = v.y;
}

// 16 bytes of products widened to fp32; read once.
template <typename T, class A = mem::Plain>
__device__ __forceinline__ void load_pvec(const T* ptr, float (&f)[PVec<T>::N], const A& access = A{}) {
  pre::unpack_vec<T>(mem::ld16_once(ptr, access), f);
}

template <typename OutT>
__device__ __forceinline__ OutT cvt(float v);
template <>
__device__ __forceinline__ float cvt<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ __nv_bfloat16 cvt<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ __half cvt<__half>(float v) {
  return __float2half_rn(v);
}
__device__ __forceinline__ float widen(float v) { return v; }
__device__ __forceinline__ float widen(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float widen(__half v) { return __half2float(v); }

// Writes N consecutive output elements, as 16-byte vectors when aligned.
template <typename OutT, int N, class A = mem::Plain>
__device__ __forceinline__ void store_out(OutT* dst, const float (&f)[N], bool beta, bool vec_ok, const A& access = A{}) {
  constexpr int kPer = 16 / sizeof(OutT);
  if constexpr (N >= kPer) {
    if (vec_ok) {
#pragma unroll
      for (int v = 0; v < N / kPer; ++v) {
        union {
          uint4 u;
          OutT e[kPer];
        } pack;
        if (beta) {
          pack.u = *reinterpret_cast<const uint4*>(dst + v * kPer);
#pragma unroll
          for (int i = 0; i < kPer; ++i) pack.e[i] = cvt<OutT>(widen(pack.e[i]) + f[v * kPer + i]);
        } else {
#pragma unroll
          for (int i = 0; i < kPer; ++i) pack.e[i] = cvt<OutT>(f[v * kPer + i]);
        }
        mem::st16(dst + v * kPer, pack.u, access);
      }
      return;
    }
  }
  if constexpr (N * sizeof(OutT) == 4) {
    if (vec_ok) {
      union {
        uint32_t u;
        OutT e[N];
      } pack;
      if (beta) {
        pack.u = *reinterpret_cast<const uint32_t*>(dst);
#pragma unroll
        for (int i = 0; i < N; ++i) pack.e[i] = cvt<OutT>(widen(pack.e[i]) + f[i]);
      } else {
#pragma unroll
        for (int i = 0; i < N; ++i) pack.e[i] = cvt<OutT>(f[i]);
      }
      *reinterpret_cast<uint32_t*>(dst) = pack.u;
      return;
    }
  }
  if constexpr (N * sizeof(OutT) == 8) {
    if (vec_ok) {
      union {
        uint2 u;
        OutT e[N];
      } pack;
      if (beta) {
        pack.u = *reinterpret_cast<const uint2*>(dst);
#pragma unroll
        for (int i = 0; i < N; ++i) pack.e[i] = cvt<OutT>(widen(pack.e[i]) + f[i]);
      } else {
#pragma unroll
        for (int i = 0; i < N; ++i) pack.e[i] = cvt<OutT>(f[i]);
      }
      *reinterpret_cast<uint2*>(dst) = pack.u;
      return;
    }
  }
#pragma unroll
  for (int i = 0; i < N; ++i) dst[i] = cvt<OutT>(beta ? widen(dst[i]) + f[i] : f[i]);
}

// A position is one 16-byte vector of products, except in the two-level single pass over 16-bit
// products, where it is one pair (4 bytes): 16 x 2 accumulators and 49 words of products then fit
// some 75 registers, so all 49 loads of a thread are issued before its first addition and three
// blocks of 256 threads are resident per SM. With wider positions the accumulators crowd the loads
// out of the register file, they go out in batches, and the pass is bound by memory latency
// (measured at 16384^2: 0.36 ms against 0.47 ms with 8-byte positions, 0.62 ms with 16-byte ones).
template <int DEPTH, int ALGO, typename TP>
struct Combine {
  static constexpr int NQ = sched::ipow(4, DEPTH);
  static constexpr int NP = sched::ipow(7, DEPTH);
  static constexpr bool kPairs = DEPTH == 2 && sizeof(TP) == 2;
  static constexpr int VEC = kPairs ? 2 : PVec<TP>::N;

  template <int P, int R>
  static __device__ __forceinline__ void add_term(const float (&x)[VEC], float (&acc)[NQ][VEC]) {
    constexpr int c = sched::w(ALGO, DEPTH, R, P);
    if constexpr (c != 0) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[R][i] = c > 0 ? acc[R][i] + x[i] : acc[R][i] - x[i];
    }
  }

  template <int P, class A, int... Rs>
  static __device__ __forceinline__ void one_product(const TP* prod0, int64_t blk_elems, float (&acc)[NQ][VEC],
                                                     const A& access, std::integer_sequence<int, Rs...>) {
    float x[VEC];
    load_pvec<TP>(prod0 + P * blk_elems, x, access);
    (add_term<P, Rs>(x, acc), ...);
  }

  template <int P, int... Rs>
  static __device__ __forceinline__ void one_pair(uint32_t raw, float (&acc)[NQ][VEC], std::integer_sequence<int, Rs...>) {
    float x[VEC];
    unpack_pair(raw, static_cast<const TP*>(nullptr), x);
    (add_term<P, Rs>(x, acc), ...);
  }

  template <class A = mem::Plain, int... Ps>
  static __device__ __forceinline__ void all_products(const TP* prod0, int64_t blk_elems, float (&acc)[NQ][VEC],
                                                      std::integer_sequence<int, Ps...>, const A& access = A{}) {
    if constexpr (kPairs) {
      // every load first (read once: streaming), then the additions in table order
      uint32_t raw[NP];
      ((raw[Ps] = __ldcs(reinterpret_cast<const uint32_t*>(prod0 + Ps * blk_elems))), ...);
      (one_pair<Ps>(raw[Ps], acc, std::make_integer_sequence<int, NQ>{}), ...);
    } else {
      (one_product<Ps>(prod0, blk_elems, acc, access, std::make_integer_sequence<int, NQ>{}), ...);
    }
  }
};


// ---- outer-quadrant form --------------------------------------------------------------------
// A few outer quadrants of C only, reading just the product groups that feed them, so a quadrant
// can be recombined as soon as its last group is done.

struct CombineOuterParams {
  const void* products;
  void* C;
  int64_t Mb, nb_vec;       // finest block rows, 16-byte product vectors per finest block row
  int64_t ldc, strideC;
  int64_t batch_blocks;     // product blocks per batch item (7^depth)
  int32_t out_dtype, beta, vec_ok;
  int8_t quad[4];           // outer quadrant of each listed entry
  int8_t coef[4][7];        // [listed entry][outer product p1]
  int32_t group_block0[7];  // first product block of outer product p1
};

// One 16-byte position `idx` (< Mb * nb_vec) of listed entry e of batch item z: the inner level's
// recombination of every feeding group, summed over the groups in fp32, rounded once.
template <int INNER, int ALGO, typename TP, class A = mem::Plain>
__device__ __forceinline__ void outer_position(const CombineOuterParams& p, int e, int z, int64_t idx,
                                               const A& access = A{}) {
  constexpr int VEC = PVec<TP>::N;
  constexpr int NQ2 = INNER ? 4 : 1;
  constexpr int NP2 = INNER ? 7 : 1;
  // positions per block fit 32 bits (the launchers check)
  const int64_t row = static_cast<uint32_t>(idx) / static_cast<uint32_t>(p.nb_vec);
  const int64_t cv = idx - row * p.nb_vec;
  const int64_t Nb = p.nb_vec * VEC;
  const int64_t blk_elems = p.Mb * Nb;

  float acc[NQ2][VEC];
#pragma unroll
  for (int r = 0; r < NQ2; ++r)
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[r][i] = 0.f;

  const TP* prod = static_cast<const TP*>(p.products) + static_cast<int64_t>(z) * p.batch_blocks * blk_elems +
                   row * Nb + cv * VEC;
#pragma unroll 1
  for (int p1 = 0; p1 < 7; ++p1) {
    const int c = p.coef[e][p1];
    if (c == 0) continue;
    const TP* g0 = prod + static_cast<int64_t>(p.group_block0[p1]) * blk_elems;
    if constexpr (INNER) {
      float part[NQ2][VEC];
#pragma unroll
      for (int r = 0; r < NQ2; ++r)
#pragma unroll
        for (int i = 0; i < VEC; ++i) part[r][i] = 0.f;
      Combine<1, ALGO, TP>::all_products(g0, blk_elems, part, std::make_integer_sequence<int, NP2>{}, access);
#pragma unroll
      for (int r = 0; r < NQ2; ++r)
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[r][i] = c > 0 ? acc[r][i] + part[r][i] : acc[r][i] - part[r][i];
    } else {
      float x[VEC];
      load_pvec<TP>(g0, x, access);
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[0][i] = c > 0 ? acc[0][i] + x[i] : acc[0][i] - x[i];
    }
  }

  const int r1 = p.quad[e];
#pragma unroll
  for (int r2 = 0; r2 < NQ2; ++r2) {
    const int br = INNER ? 2 * (r1 >> 1) + (r2 >> 1) : (r1 >> 1);
    const int bc = INNER ? 2 * (r1 & 1) + (r2 & 1) : (r1 & 1);
    const int64_t off = static_cast<int64_t>(z) * p.strideC + (br * p.Mb + row) * p.ldc + bc * Nb + cv * VEC;
    if (p.out_dtype == B200S_BF16)
      store_out<__nv_bfloat16, VEC>(static_cast<__nv_bfloat16*>(p.C) + off, acc[r2], p.beta != 0, p.vec_ok != 0, access);
    else if (p.out_dtype == B200S_FP16)
      store_out<__half, VEC>(static_cast<__half*>(p.C) + off, acc[r2], p.beta != 0, p.vec_ok != 0, access);
    else
      store_out<float, VEC>(static_cast<float*>(p.C) + off, acc[r2], p.beta != 0, p.vec_ok != 0, access);
  }
}

}  // namespace comb
}  // namespace b200s
