// 16-byte global accesses with or without an L2 eviction hint.
//
// The add passes touch every byte once. When they run as warps of the fused Strassen kernel, beside
// tensor-core tiles whose operands live in L2, their lines must leave L2 first: the hinted forms carry
// an evict-first cache policy (and skip L1). The stand-alone passes use the plain forms. The
// arithmetic around an access is the same either way.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace b200s {
namespace mem {

// How a pass accesses memory: kHint selects the hinted forms, `policy` is the cache-policy word.
template <bool kHint_>
struct Access {
  static constexpr bool kHint = kHint_;
  uint64_t policy = 0;
};
using Plain = Access<false>;
using Streaming = Access<true>;

__device__ __forceinline__ Streaming make_streaming() {
  Streaming s;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(s.policy));
  return s;
}

// Data nobody writes while the kernel runs.
template <class A>
__device__ __forceinline__ uint4 ld16_readonly(const void* ptr, const A& a) {
  if constexpr (A::kHint) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(ptr), "l"(a.policy));
    return v;
  } else {
    return __ldg(reinterpret_cast<const uint4*>(ptr));
  }
}

// Data read once that another CTA of the same launch may have written: through L2, never the
// non-coherent path.
template <class A>
__device__ __forceinline__ uint4 ld16_once(const void* ptr, const A& a) {
  if constexpr (A::kHint) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(ptr), "l"(a.policy)
                 : "memory");
    return v;
  } else {
    return __ldcs(reinterpret_cast<const uint4*>(ptr));
  }
}

template <class A>
__device__ __forceinline__ void st16(void* ptr, const uint4& v, const A& a) {
  if constexpr (A::kHint) {
    asm volatile("st.global.L2::cache_hint.v4.b32 [%0], {%1, %2, %3, %4}, %5;" ::"l"(ptr), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w), "l"(a.policy)
                 : "memory");
  } else {
    *reinterpret_cast<uint4*>(ptr) = v;
  }
}

}  // namespace mem
}  // namespace b200s
