// Thin inline-PTX wrappers for the sm_100a features the GEMM kernels use:
// mbarrier, TMA tiled copies (cp.async.bulk.tensor), tensor memory (TMEM)
// allocation, tcgen05.mma / commit / ld, and the proxy fences between them.
//
// Every wait in this file is bounded: mbar_wait() gives up after a wall-clock
// limit, records that in a shared abort word and returns false so that the
// caller can leave its loop, release TMEM and return.
#pragma once

#include <cuda.h>
#include <cstdint>

namespace b200s {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// ---------------------------------------------------------------- mbarrier

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Arrive on the barrier at the same shared-memory offset in CTA `cta` of this cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar, uint32_t cta) {
  asm volatile(
      "{\n"
      " .reg .b32 remote;\n"
      " mapa.shared::cluster.u32 remote, %0, %1;\n"
      " mbarrier.arrive.release.cluster.shared::cluster.b64 _, [remote];\n"
      "}\n" ::"r"(bar),
      "r"(cta)
      : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

// Upper bound, in nanoseconds, for how long the hardware may keep a waiting thread suspended
// inside one try_wait before it returns false; a long hint keeps waiting warps off the issue
// ports (and off the power budget) instead of spinning.
constexpr uint32_t kSuspendHintNs = 10000000u;

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      " selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
      : "memory");
  return ok != 0;
}

__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n"
      " selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
      : "memory");
  return ok != 0;
}

// Wall-clock limit of one wait. A healthy kernel never waits longer than a
// few milliseconds on any barrier; the limit only bounds a broken pipeline.
constexpr uint64_t kWaitLimitNs = 2000000000ull;

// Waits for the phase with the given parity. Returns false (and sets *abort_word,
// a word in shared memory that all roles of the CTA poll) when `limit_ns` of wall clock run out
// or when another role has already given up.
// kBackoffNs > 0 sleeps that long between polls: for waits that normally last a whole main loop.
template <bool kClusterScope = false, int kBackoffNs = 0>
__device__ __forceinline__ bool mbar_wait_limit(uint32_t bar, uint32_t parity, volatile uint32_t* abort_word,
                                                uint32_t who, uint64_t limit_ns) {
  uint64_t start = 0;
  for (uint32_t it = 0;; ++it) {
    bool ok = kClusterScope ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity);
    if (ok) return true;
    if constexpr (kBackoffNs > 0) __nanosleep(kBackoffNs);
    if ((it & 0xfu) == 0xfu) {
      if (*abort_word != 0) return false;
      uint64_t now = global_timer_ns();
      if (start == 0) {
        start = now;
      } else if (now - start > limit_ns) {
        *abort_word = who;
        return false;
      }
    }
  }
}
template <bool kClusterScope = false, int kBackoffNs = 0>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity,
                                          volatile uint32_t* abort_word, uint32_t who) {
  return mbar_wait_limit<kClusterScope, kBackoffNs>(bar, parity, abort_word, who, kWaitLimitNs);
}

// Waits for a phase without the abort protocol, until `deadline_ns` of the global timer at the
// latest: what a CTA that is already giving up uses to let its own copies in flight land.
__device__ __forceinline__ bool mbar_wait_until(uint32_t bar, uint32_t parity, uint64_t deadline_ns) {
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() > deadline_ns) return false;
    __nanosleep(64);
  }
}

// ---- register reallocation between warpgroups --------------------------------------------------
// All four warps of a warpgroup execute these together. A kernel launched with R registers per
// thread may hand registers of its light warpgroups (dec) to its heavy ones (inc); the sum over the
// warpgroups must stay within the register file.
template <int kRegs>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs));
}
template <int kRegs>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs));
}

// Barrier `id` (1..15) among `nthreads` threads of the CTA (whole warps).
__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Orders this thread's generic-proxy accesses with async-proxy accesses (TMA) to the same memory, in
// both directions: before publishing data that a TMA load elsewhere will read, and before reading
// with ordinary loads what a completed TMA store wrote.
__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

// ---- counters in global memory shared by the CTAs of one launch ---------------------------------
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* ptr) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}
// Publishes everything this thread (and, through a preceding CTA barrier, its CTA) wrote before it.
__device__ __forceinline__ void red_release_gpu_add(uint32_t* ptr, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(ptr), "r"(v) : "memory");
}

// Waits until *ctr >= target, with the same wall-clock limit and abort protocol as mbar_wait.
__device__ __forceinline__ bool wait_counter(const uint32_t* ctr, uint32_t target, volatile uint32_t* abort_word,
                                             uint32_t who) {
  uint64_t start = 0;
  for (uint32_t it = 0;; ++it) {
    if (ld_acquire_gpu(ctr) >= target) return true;
    __nanosleep(256);
    if ((it & 0x3fu) == 0x3fu) {
      if (*abort_word != 0) return false;
      uint64_t now = global_timer_ns();
      if (start == 0) {
        start = now;
      } else if (now - start > kWaitLimitNs) {
        *abort_word = who;
        return false;
      }
    }
  }
}

// ---------------------------------------------------------------- fences

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- TMA

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

// Tiled 3-D load global -> this CTA's shared memory, completion on an mbarrier of this CTA.
// c0 is the innermost coordinate: c0 * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int c0,
                                            int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// Same copy issued from either CTA of a CTA pair: the data lands in the issuing
// CTA's shared memory, the transaction bytes are counted on the barrier whose
// (cluster-mapped) address is given, which may live in the peer CTA.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* m,
                                                 uint32_t bar_cluster_addr, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// Tiled 3-D store shared -> global (bulk async group).
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, uint32_t src, int c0, int c1,
                                             int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(src), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
// Same store with an L2 eviction-priority hint (a policy word from make_evict_first_policy).
__device__ __forceinline__ void tma_store_3d_hint(const CUtensorMap* m, uint32_t src, int c0, int c1, int c2,
                                                  uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3, %4}], [%1], %5;" ::"l"(
          reinterpret_cast<uint64_t>(m)),
      "r"(src), "r"(c0), "r"(c1), "r"(c2), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t make_evict_first_policy() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int kPending>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
template <int kPending>
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(kPending) : "memory");
}

// ---------------------------------------------------------------- shared-memory stores, packing

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
// 16-byte store to an NVLS multicast address: the NVSwitch writes the bytes into the same offset of
// every GPU's memory bound to the multicast object. A plain store as far as this GPU is concerned -
// nothing is loaded or reduced and nothing is waited for.
__device__ __forceinline__ void multimem_st_v4(void* mc_ptr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_ptr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
// Two floats -> two bf16 / f16 (round to nearest even) in one 32-bit word, `lo` in the low half.
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// ---------------------------------------------------------------- TMEM

// Whole-warp calls. `slot` is a shared-memory word that receives the TMEM base address.
template <int kCtaGroup>
__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t ncols) {
  if constexpr (kCtaGroup == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot),
                 "r"(ncols)
                 : "memory");
  } else {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot),
                 "r"(ncols)
                 : "memory");
  }
}
template <int kCtaGroup>
__device__ __forceinline__ void tmem_relinquish() {
  if constexpr (kCtaGroup == 1) {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  } else {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
}
template <int kCtaGroup>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if constexpr (kCtaGroup == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
  } else {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
  }
}

// ---------------------------------------------------------------- tcgen05.mma

// Shared-memory matrix descriptor (64-bit) for a tile whose rows are 128 bytes
// wide and stored with the 128-byte swizzle, as a TMA box with
// CU_TENSOR_MAP_SWIZZLE_128B writes it.
//   bits [0,14)  start address >> 4
//   bits [16,30) leading-dimension byte offset >> 4
//   bits [32,46) stride-dimension byte offset >> 4
//   bits [46,48) descriptor version (1 on sm_100)
//   bits [61,64) layout type (2 = 128-byte swizzle)
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

// Instruction descriptor (32-bit) for kind::f16 / kind::tf32 with fp32 accumulation.
//   bits [4,6)   accumulator format (1 = f32)
//   bits [7,10)  A format, bits [10,13) B format (0 = f16, 1 = bf16, 2 = tf32)
//   bit 13 / 14  negate A / B
//   bit 15 / 16  A / B major (0 = K-major, 1 = MN-major)
//   bits [17,23) N >> 3
//   bits [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_instr_desc(uint32_t fmt, uint32_t a_mn_major,
                                                       uint32_t b_mn_major, uint32_t m, uint32_t n) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (a_mn_major << 15) | (b_mn_major << 16) |
         ((n >> 3) << 17) | ((m >> 4) << 24);
}

template <int kCtaGroup, bool kTf32>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                     uint32_t accumulate) {
  if constexpr (kCtaGroup == 1) {
    if constexpr (kTf32) {
      asm volatile(
          "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
          " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
          "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
          : "memory");
    } else {
      asm volatile(
          "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
          " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
          "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
          : "memory");
    }
  } else {
    if constexpr (kTf32) {
      asm volatile(
          "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
          " tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
          "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
          : "memory");
    } else {
      asm volatile(
          "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
          " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
          "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
          : "memory");
    }
  }
}

// Makes the mbarrier (a cluster-mapped shared address) complete one arrival when
// all tcgen05 operations issued so far by this thread have finished.
template <int kCtaGroup>
__device__ __forceinline__ void umma_commit(uint32_t bar_cluster_addr) {
  if constexpr (kCtaGroup == 1) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     bar_cluster_addr)
                 : "memory");
  } else {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     bar_cluster_addr)
                 : "memory");
  }
}

__device__ __forceinline__ uint32_t mapa_cluster(uint32_t saddr, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(cta));
  return r;
}

// ---------------------------------------------------------------- tcgen05.ld

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives lane
// (lane_base + i), columns [col, col+32).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

}  // namespace ptx
}  // namespace b200s
