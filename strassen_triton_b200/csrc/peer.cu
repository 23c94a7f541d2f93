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

}  // namespace b200s
