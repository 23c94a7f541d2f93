// Out-of-place transpose of fp32 operands.
//
// tcgen05.mma reads 32-bit (TF32) operands from shared memory only in K-major form with the
// plain 128-byte swizzle this library's TMA maps use, so an fp32 operand whose outer dimension is
// contiguous (for example B of a row-major A @ B) is first rewritten K-major into scratch.
// 16-bit operands never take this path: the tensor core reads both of their majors directly.
//
// Also here: the hi/lo split of fp32 operands for the three-pass TF32 mode (B200S_PREC_3XTF32).

#include <cuda_runtime.h>

#include "common.h"

namespace b200s {

namespace {

// in: rows x cols (ld_in), out: cols x rows (ld_out); one 32x32 tile per block, 32x8 threads.
__global__ void __launch_bounds__(256) transpose32_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                          int64_t rows, int64_t cols, int64_t ld_in, int64_t ld_out,
                                                          int64_t stride_in, int64_t stride_out) {
  __shared__ float tile[32][33];
  in += static_cast<int64_t>(blockIdx.z) * stride_in;
  out += static_cast<int64_t>(blockIdx.z) * stride_out;
  const int64_t c0 = static_cast<int64_t>(blockIdx.x) * 32, r0 = static_cast<int64_t>(blockIdx.y) * 32;
#pragma unroll
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int64_t r = r0 + j, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = in[r * ld_in + c];
  }
  __syncthreads();
#pragma unroll
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int64_t c = c0 + j, r = r0 + threadIdx.x;
    if (r < rows && c < cols) out[c * ld_out + r] = tile[threadIdx.x][j];
  }
}

// hi = x rounded to TF32 (10-bit mantissa), lo = x - hi rounded to TF32. x.y ~ hi.hi' + lo.hi' + hi.lo'
// with the dropped lo.lo' term about 2^-22 of the product.
__device__ __forceinline__ float tf32_round(float x) {
  return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u);
}

// in: rows x cols fp32 (ld_in); out: rows x 3*cols, three K segments per row:
// side 0 (A): [hi | lo | hi], side 1 (B): [hi | hi | lo].
__global__ void __launch_bounds__(256) split3_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t rows,
                                                     int64_t cols4, int64_t ld_in, int64_t stride_in, int side) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= rows * cols4) return;
  const int64_t r = idx / cols4, c4 = idx - r * cols4;
  const int64_t cols = cols4 * 4;
  const float4 x = *reinterpret_cast<const float4*>(in + static_cast<int64_t>(blockIdx.y) * stride_in + r * ld_in + c4 * 4);
  float4 hi, lo;
  hi.x = tf32_round(x.x), hi.y = tf32_round(x.y), hi.z = tf32_round(x.z), hi.w = tf32_round(x.w);
  lo.x = tf32_round(x.x - hi.x), lo.y = tf32_round(x.y - hi.y), lo.z = tf32_round(x.z - hi.z), lo.w = tf32_round(x.w - hi.w);
  float* o = out + (static_cast<int64_t>(blockIdx.y) * rows + r) * (3 * cols) + c4 * 4;
  *reinterpret_cast<float4*>(o) = hi;
  *reinterpret_cast<float4*>(o + cols) = side == 0 ? lo : hi;
  *reinterpret_cast<float4*>(o + 2 * cols) = side == 0 ? hi : lo;
}

}  // namespace

int launch_split3_f32(const void* in, void* out, int64_t rows, int64_t cols, int64_t ld_in, int64_t batch,
                      int64_t stride_in, int side, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || batch <= 0 || batch > 65535 || cols % 4) return B200S_ERR_BAD_SHAPE;
  if ((ld_in * 4) % 16 || (reinterpret_cast<uintptr_t>(in) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u))
    return B200S_ERR_BAD_ALIGNMENT;
  const int64_t blocks = (rows * (cols / 4) + 255) / 256;
  if (blocks > INT32_MAX) return B200S_ERR_BAD_SHAPE;
  dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(batch));
  split3_kernel<<<grid, 256, 0, stream>>>(static_cast<const float*>(in), static_cast<float*>(out), rows, cols / 4, ld_in,
                                          stride_in, side);
  B200S_CUDA_OK(cudaGetLastError());
  count_launch();
  return B200S_OK;
}

int launch_transpose_f32(const void* in, void* out, int64_t rows, int64_t cols, int64_t ld_in, int64_t ld_out,
                         int64_t batch, int64_t stride_in, int64_t stride_out, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || batch <= 0 || batch > 65535) return B200S_ERR_BAD_SHAPE;
  const int64_t gx = (cols + 31) / 32, gy = (rows + 31) / 32;
  if (gx > INT32_MAX || gy > 65535) return B200S_ERR_BAD_SHAPE;
  dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy), static_cast<unsigned>(batch));
  transpose32_kernel<<<grid, dim3(32, 8), 0, stream>>>(static_cast<const float*>(in), static_cast<float*>(out), rows,
                                                       cols, ld_in, ld_out, stride_in, stride_out);
  B200S_CUDA_OK(cudaGetLastError());
  count_launch();
  return B200S_OK;
}

}  // namespace b200s
