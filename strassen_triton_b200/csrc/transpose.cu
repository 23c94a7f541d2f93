// Out-of-place transpose of fp32 operands.
//
// tcgen05.mma reads 32-bit (TF32) operands from shared memory only in K-major form with the
// plain 128-byte swizzle this library's TMA maps use, so an fp32 operand whose outer dimension is
// contiguous (for example B of a row-major A @ B) is first rewritten K-major into scratch.
// 16-bit operands never take this path: the tensor core reads both of their majors directly.

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

}  // namespace

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
