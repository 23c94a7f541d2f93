// Device-side barrier among the GPUs of a row-sharded product.
//
// Every rank owns a pad of 32-bit slots in memory all ranks can reach (peer-mapped or symmetric
// memory), one slot per rank. To pass barrier number `epoch` a rank stores `epoch` into its slot of
// every rank's pad, then waits until every slot of its own pad has reached `epoch`. Slots only grow, so
// a pad is never cleared and consecutive barriers cannot be confused. The wait is bounded: when the
// limit runs out (a peer died, or never entered the call) the kernel records that in the device
// status words and returns; nothing traps and the context stays usable.
//
// The reference has no multi-GPU product; this orders the exchange of a row-sharded product.

#include <cuda_runtime.h>

#include "common.h"
#include "ptx_sm100.cuh"

namespace b200s {

namespace {

struct BarrierParams {
  uint32_t* pad[8];  // pad of rank r (device address valid on this GPU)
  int32_t rank, world;
  uint32_t epoch;
  uint64_t limit_ns;
  uint32_t* status;
};

constexpr uint32_t kWhoPeerBarrier = 8;

__global__ void __launch_bounds__(32) peer_barrier_kernel(const BarrierParams p) {
  const int r = threadIdx.x;
  if (r >= p.world) return;
  // everything this GPU wrote before (its stores into the peers' C) is ordered before the signal
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.pad[r] + p.rank), "r"(p.epoch) : "memory");
  const uint32_t* mine = p.pad[p.rank] + r;
  const uint64_t start = ptx::global_timer_ns();
  for (uint32_t it = 0;; ++it) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    // slots only grow; the comparison survives the counter wrapping around
    if (static_cast<int32_t>(v - p.epoch) >= 0) break;
    __nanosleep(200);
    if ((it & 0x3fu) == 0x3fu && ptx::global_timer_ns() - start > p.limit_ns) {
      atomicExch(&p.status[0], 1u);
      atomicExch(&p.status[1], kWhoPeerBarrier);
      break;
    }
  }
}

// Copy of finished rows of C to the other GPUs' copies, on a handful of SMs: the product kernel of
// the next row panel is launched on the remaining SMs (b200s_set_product_sms) and runs beside it.
// With a multicast address every 16 bytes leave this GPU once and the NVSwitch writes them to all
// copies (this GPU's own included, with the values it already holds); without one they are stored
// to every peer in turn. Loads read local memory only.
struct PushPanelParams {
  const uint4* src;
  uint8_t* mc;       // multicast address of the same bytes, or nullptr
  uint4* dst[8];     // else: n_dst peer copies
  int32_t n_dst;
  int64_t n_vec;
};

__global__ void __launch_bounds__(512) push_panel_kernel(const PushPanelParams p) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < p.n_vec; i += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = __ldcs(p.src + i + u * stride);
    if (p.mc != nullptr) {
#pragma unroll
      for (int u = 0; u < 4; ++u) ptx::multimem_st_v4(p.mc + (i + u * stride) * 16, v[u]);
    } else {
#pragma unroll 1
      for (int d = 0; d < p.n_dst; ++d)
#pragma unroll
        for (int u = 0; u < 4; ++u) p.dst[d][i + u * stride] = v[u];
    }
  }
  for (; i < p.n_vec; i += stride) {
    const uint4 v = __ldcs(p.src + i);
    if (p.mc != nullptr) {
      ptx::multimem_st_v4(p.mc + i * 16, v);
    } else {
      for (int d = 0; d < p.n_dst; ++d) p.dst[d][i] = v;
    }
  }
}

}  // namespace

int launch_peer_barrier(void* const* pads, int rank, int world, uint32_t epoch, uint64_t limit_ns,
                        cudaStream_t stream) {
  if (!pads) return B200S_ERR_NULL_POINTER;
  if (world < 1 || world > 8 || rank < 0 || rank >= world || limit_ns == 0) return B200S_ERR_BAD_SHAPE;
  BarrierParams kp;
  for (int r = 0; r < 8; ++r) {
    kp.pad[r] = r < world ? static_cast<uint32_t*>(pads[r]) : nullptr;
    if (r < world && (!pads[r] || (reinterpret_cast<uintptr_t>(pads[r]) & 3u))) return B200S_ERR_BAD_ALIGNMENT;
  }
  kp.rank = rank, kp.world = world, kp.epoch = epoch, kp.limit_ns = limit_ns;
  kp.status = device_status_words();
  if (!kp.status) return B200S_ERR_NO_DEVICE;
  peer_barrier_kernel<<<1, 32, 0, stream>>>(kp);
  B200S_CUDA_OK(cudaGetLastError());
  count_launch();
  return B200S_OK;
}

int launch_push_panel(const void* src, void* const* dst, int n_dst, void* mc_dst, size_t bytes, int max_blocks,
                      cudaStream_t stream) {
  if (!src || (!mc_dst && !dst)) return B200S_ERR_NULL_POINTER;
  if (bytes == 0 || bytes % 16 || max_blocks < 1) return B200S_ERR_BAD_SHAPE;
  if (!mc_dst && (n_dst < 1 || n_dst > 8)) return B200S_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(src) & 15u) || (reinterpret_cast<uintptr_t>(mc_dst) & 15u)) return B200S_ERR_BAD_ALIGNMENT;
  PushPanelParams kp;
  kp.src = static_cast<const uint4*>(src);
  kp.mc = static_cast<uint8_t*>(mc_dst);
  kp.n_dst = mc_dst ? 0 : n_dst;
  kp.n_vec = static_cast<int64_t>(bytes / 16);
  for (int d = 0; d < 8; ++d) {
    kp.dst[d] = (!mc_dst && d < n_dst) ? static_cast<uint4*>(dst[d]) : nullptr;
    if (!mc_dst && d < n_dst && (!dst[d] || (reinterpret_cast<uintptr_t>(dst[d]) & 15u))) return B200S_ERR_BAD_ALIGNMENT;
  }
  const int sms = sm_count();
  if (sms <= 0) return B200S_ERR_NO_DEVICE;
  int64_t blocks = (kp.n_vec + 511) / 512;
  if (blocks > max_blocks) blocks = max_blocks;
  if (blocks > sms) blocks = sms;
  push_panel_kernel<<<static_cast<unsigned>(blocks), 512, 0, stream>>>(kp);
  B200S_CUDA_OK(cudaGetLastError());
  count_launch();
  return B200S_OK;
}

}  // namespace b200s
