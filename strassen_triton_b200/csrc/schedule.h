// Coefficient tables of the two bilinear <2,2,2;7> algorithms, in the form
//   M_p = (sum_q U[p][q] A_q) . (sum_q V[p][q] B_q),   C_r = sum_p W[r][p] M_p
// with quadrants ordered q, r = 0..3 for (11, 12, 21, 22).
//
// Classic: products M1..M7 in the order of fixed_strassen_fp32_agg.py:38-44 (= strassen.py:722-728),
// recombination of :47-50.
// Winograd: the Strassen-Winograd form (S1=A21+A22, S2=S1-A11, S3=A11-A21, S4=A12-S2, T1=B12-B11,
// T2=B22-T1, T3=B22-B12, T4=T2-B21; P1=A11.B11, P2=A12.B21, P3=S4.B22, P4=A22.T4, P5=S1.T1,
// P6=S2.T2, P7=S3.T3; C11=P1+P2, C12=P1+P6+P5+P3, C21=P1+P6+P7-P4, C22=P1+P6+P7+P5) with the
// shared sub-expressions expanded, so every operand block is one sum of original quadrants.
//
// Two levels are the Kronecker squares: product p = 7*p1 + p2, quadrant q = 4*q1 + q2 where
// index 1 is the outer (level-1) and index 2 the inner (level-2) split.
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define B200S_HD __host__ __device__
#else
#define B200S_HD
#endif

namespace b200s {
namespace sched {

enum { kClassic = 0, kWinograd = 1 };
enum { kSideA = 0, kSideB = 1 };

// U (side 0) or V (side 1) entry for product p, quadrant q at one level.
B200S_HD constexpr int uv1(int algo, int side, int p, int q) {
  constexpr int8_t t[2][2][7][4] = {
      {// classic
       {{1, 0, 0, 1}, {0, 0, 1, 1}, {1, 0, 0, 0}, {0, 0, 0, 1}, {1, 1, 0, 0}, {-1, 0, 1, 0}, {0, 1, 0, -1}},
       {{1, 0, 0, 1}, {1, 0, 0, 0}, {0, 1, 0, -1}, {-1, 0, 1, 0}, {0, 0, 0, 1}, {1, 1, 0, 0}, {0, 0, 1, 1}}},
      {// winograd
       {{1, 0, 0, 0}, {0, 1, 0, 0}, {1, 1, -1, -1}, {0, 0, 0, 1}, {0, 0, 1, 1}, {-1, 0, 1, 1}, {1, 0, -1, 0}},
       {{1, 0, 0, 0}, {0, 0, 1, 0}, {0, 0, 0, 1}, {1, -1, -1, 1}, {-1, 1, 0, 0}, {1, -1, 0, 1}, {0, -1, 0, 1}}}};
  return t[algo][side][p][q];
}

// W entry: contribution of product p to output quadrant r at one level.
B200S_HD constexpr int w1(int algo, int r, int p) {
  constexpr int8_t t[2][4][7] = {
      {{1, 0, 0, 1, -1, 0, 1}, {0, 0, 1, 0, 1, 0, 0}, {0, 1, 0, 1, 0, 0, 0}, {1, -1, 1, 0, 0, 1, 0}},
      {{1, 1, 0, 0, 0, 0, 0}, {1, 0, 1, 0, 1, 1, 0}, {1, 0, 0, -1, 0, 1, 1}, {1, 0, 0, 0, 1, 1, 1}}};
  return t[algo][r][p];
}

B200S_HD constexpr int ipow(int b, int e) { return e == 0 ? 1 : b * ipow(b, e - 1); }

// Entry of the depth-level U/V table (depth 1 or 2).
B200S_HD constexpr int uv(int algo, int side, int depth, int p, int q) {
  return depth == 1 ? uv1(algo, side, p, q) : uv1(algo, side, p / 7, q / 4) * uv1(algo, side, p % 7, q % 4);
}
B200S_HD constexpr int w(int algo, int depth, int r, int p) {
  return depth == 1 ? w1(algo, r, p) : w1(algo, r / 4, p / 7) * w1(algo, r % 4, p % 7);
}

// Position of quadrant index q (depth levels) in the 2^depth x 2^depth block grid.
B200S_HD constexpr int block_row(int depth, int q) {
  return depth == 1 ? (q >> 1) : 2 * ((q / 4) >> 1) + ((q % 4) >> 1);
}
B200S_HD constexpr int block_col(int depth, int q) {
  return depth == 1 ? (q & 1) : 2 * ((q / 4) & 1) + ((q % 4) & 1);
}

}  // namespace sched
}  // namespace b200s
