// Batched / grouped dense GEMM for sm_100a: C[b] (+)= A[b] . B[b].
//
// One persistent, warp-specialised kernel:
//   warp 0      TMA producer: cp.async.bulk.tensor loads of 128-byte-swizzled operand tiles
//               into a ring of shared-memory stages
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (fp32 accumulators in TMEM)
//   warps 2..5  epilogue: tcgen05.ld of a finished accumulator, conversion, stores to C
// The accumulator is double-buffered in TMEM so the epilogue of tile i overlaps the main loop
// of tile i+1. With kCtaGroup == 2 two CTAs of a cluster share one 256-row tile
// (tcgen05.mma.cta_group::2): each CTA loads its own 128 rows of A and its half of the B tile,
// the leader CTA issues the MMAs for both.
//
// The 7 or 49 sub-products of a Strassen step are one launch of this kernel: the batch
// coordinate of the 3-D tensor maps selects the product, tiles are ordered product-major so one
// product's operands stay in L2 while its tiles run.
//
// It stands where the reference calls torch.mm (cuBLAS) for its sub-products:
// fixed_strassen_fp32_agg.py:38-44, fixed_strassen.py:39-45, strassen.py:722-728, and where it
// launches its dense Triton kernel, strassen.py:31-88.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <mutex>

#include "combine_device.cuh"
#include "common.h"
#include "preadd_device.cuh"
#include "ptx_sm100.cuh"
#include "schedule.h"

namespace b200s {

namespace {

constexpr int kBM = 128;          // accumulator rows per CTA (TMEM lanes)
constexpr int kRowBytes = 128;    // bytes of one swizzled smem row = one K block of a K-major tile

struct GemmKernelParams {
  int32_t M, N;               // extents of one C[b]
  int32_t m_tiles, n_tiles;   // tiles per batch item
  int32_t k_blocks;
  int32_t total_tiles;
  int32_t raster_group;       // m-tiles that share a band of n-tiles in the tile order
  int32_t wave_tiles;         // tiles the whole device works on at a time (its SMs / CTAs per tile)
  int32_t a_mn, b_mn;
  int32_t fmt;                // operand format field of the instruction descriptor
  int32_t out_dtype, beta;
  int32_t tma_store;          // 1: the epilogue stages tiles in shared memory and stores them with TMA
  int32_t n_dst;              // copies of C the TMA-store epilogue writes (1 unless the product is exchanged)
  uint8_t* dst[8];            // their (0,0) elements; copy 0 is stored by TMA, the others by ordinary stores
  const void* bias;           // optional row vector (N elements of out_dtype) added before the rounding
  uint8_t* mc;                // or: one NVLS multicast address that reaches every GPU's copy (then n_dst == 2)
  int32_t send_ctas;          // > 0: the last send_ctas CTAs of the grid multiply nothing; they send finished blocks of
                              // columns of C to dst[1..] / mc while the others multiply (the epilogue then stores locally only)
  uint32_t* send_counters;    // one counter per (band of m-tiles, n-tile): epilogue warps done with a tile of it
  int32_t stagger;            // 1: clusters hold their remote stores back by different shares of the tile period
                              // (per-peer stores at 4 GPUs, 32768^3: 15.0 -> 14.4 ms a step; no gain with multicast)
  int64_t ldc, strideC;
  void* C;
  uint32_t* status;
};

// Role codes stored in the abort word / device status when a wait runs out.
enum : uint32_t {
  kWhoProducer = 1,
  kWhoMma = 2,
  kWhoMmaAcc = 3,
  kWhoEpilogue = 4,
  kWhoProducerGroup = 5,  // fused kernel: the producer waiting for a group's operand blocks
  kWhoAdder = 6,          // fused kernel: an adder warp waiting for a group's products
  kWhoProbe = 7,          // wait_probe_kernel: the self-test of the bounded wait
  kWhoSender = 11         // a sending CTA waiting for a block of columns of C to be complete
};

// How long a CTA that gives up waits for its producer's outstanding TMA loads to land.
constexpr uint64_t kDrainLimitNs = 20ull * 1000 * 1000;

// ---- fused Strassen kernel: what the adder warps do ----------------------------------------------
// Phase 1: the operand blocks of every outer group still to be formed, in processing order; warps 0-1
// of the adder warpgroup take side A, warps 2-3 side B (all four side A when B's blocks exist already).
// Phase 2: the quadrants of C, each once the groups feeding it are stored. Every CTA takes the
// positions first, first + stride, ... of every task. The two sides and the two phases are separate
// loops on purpose: the compiler then allocates registers for one body at a time.
constexpr int kAdderThreads = 128;

struct FusedKernelParams {
  pre::PreaddOuterParams pre[2];  // listed group i = group at processing position i
  comb::CombineOuterParams comb;  // listed entry e = outer quadrant e
  uint32_t* flags;                // [0, 8): adder teams done with the operand blocks of group i; [8, 16): epilogue
                                  // warps done with a tile of group i
  uint32_t ready_target;          // value of a ready counter once every team of every CTA has signalled
  uint32_t done_target;           // value of a done counter once every tile of a group is stored
  int32_t np2;                    // product blocks per outer group
  int32_t groups_formed;          // leading groups whose operand blocks existed before the launch
  int32_t b_formed;               // all of B's blocks existed before the launch
  int32_t n_comb;                 // quadrants of C recombined by the adders
  int8_t comb_quad[4];            // in the order in which their groups complete
  int8_t comb_wait[4];            // leading groups whose products the quadrant needs
};

struct NoFuse {
  static constexpr bool kOn = false, kSend = false;
  struct Params {};
};
// The plain product kernel whose last CTAs send finished blocks of C to other GPUs (run_sender).
struct WithSenders {
  static constexpr bool kOn = false, kSend = true;
  struct Params {};
};
template <int INNER, int ALGO, typename T>
struct Fuse {
  static constexpr bool kOn = true, kSend = false;
  static constexpr int kInner = INNER, kAlgo = ALGO;
  using Elem = T;
  using Params = FusedKernelParams;
};

// The adders' loads and stores carry an evict-first L2 policy: what they stream through once must not
// push the operand tiles of the products out of L2.
template <int INNER, int ALGO, int SIDE, typename T>
__device__ __forceinline__ void adder_preadd(const pre::PreaddOuterParams& p, int g, int64_t first, int64_t stride) {
  using OP = pre::OuterPosition<INNER, ALGO, SIDE, T>;
  const int64_t total = p.rows_blk * p.cols_vec;
  const mem::Streaming access = mem::make_streaming();
#pragma unroll 1
  for (int64_t idx = first; idx < total; idx += stride) {
    const typename OP::Where w = OP::locate(p, idx);
    typename OP::Raw raw;
    float t[OP::NQ2][OP::VEC];
    OP::fetch(p, g, 0, w, raw, access);
    OP::reduce(p, g, raw, t);
    OP::store(p, g, 0, w, t, access);
  }
}

template <int INNER, int ALGO, typename TP>
__device__ __forceinline__ void adder_combine(const comb::CombineOuterParams& p, int e, int64_t first, int64_t stride) {
  const int64_t total = p.Mb * p.nb_vec;
  const mem::Streaming access = mem::make_streaming();
#pragma unroll 1
  for (int64_t idx = first; idx < total; idx += stride) comb::outer_position<INNER, ALGO, TP>(p, e, 0, idx, access);
}

// A team of `nthreads` adder threads (barrier `bar`) finished the operand blocks of group i: the blocks
// will be read by TMA loads of other CTAs.
__device__ __forceinline__ void adder_signal(uint32_t* ready, uint32_t bar, uint32_t nthreads, bool leader) {
  ptx::fence_proxy_async_all();
  ptx::named_bar_sync(bar, nthreads);
  if (leader) {
    __threadfence();
    ptx::red_release_gpu_add(ready, 1u);
  }
}

template <class F>
__device__ __forceinline__ void run_adders(const FusedKernelParams& fz, volatile uint32_t* abort_word,
                                           volatile uint32_t* go_word, int tid) {
  constexpr int INNER = F::kInner, ALGO = F::kAlgo;
  using T = typename F::Elem;
  // ---- phase 1: operand blocks
  if (fz.b_formed || tid < 64) {
    const int team = fz.b_formed ? kAdderThreads : 64;
    const int64_t first = static_cast<int64_t>(blockIdx.x) * team + tid;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * team;
#pragma unroll 1
    for (int i = fz.groups_formed; i < 7; ++i) {
      adder_preadd<INNER, ALGO, sched::kSideA, T>(fz.pre[0], i, first, stride);
      adder_signal(fz.flags + i, 2, team, tid == 0);
    }
  } else {
    const int64_t first = static_cast<int64_t>(blockIdx.x) * 64 + (tid - 64);
    const int64_t stride = static_cast<int64_t>(gridDim.x) * 64;
#pragma unroll 1
    for (int i = fz.groups_formed; i < 7; ++i) {
      adder_preadd<INNER, ALGO, sched::kSideB, T>(fz.pre[1], i, first, stride);
      adder_signal(fz.flags + i, 3, 64, tid == 64);
    }
  }
  // ---- phase 2: quadrants of C
  const int64_t first = static_cast<int64_t>(blockIdx.x) * kAdderThreads + tid;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kAdderThreads;
#pragma unroll 1
  for (int t = 0; t < fz.n_comb; ++t) {
    // the products of the first comb_wait[t] groups must all be in global memory
    if (tid == 0) {
      const int nwait = fz.comb_wait[t];
      for (int j = 0; j < nwait; ++j)
        if (!ptx::wait_counter(fz.flags + 8 + j, fz.done_target, abort_word, kWhoAdder)) break;
      ptx::fence_proxy_async_all();  // they were written by TMA stores
      *go_word = *abort_word == 0 ? 1u : 0u;
    }
    // One thread decides for the team: the abort word can change at any moment (another role giving
    // up), and threads that read it themselves could part ways and leave the rest at the barrier.
    ptx::named_bar_sync(1, kAdderThreads);
    const bool go = *go_word != 0;
    ptx::named_bar_sync(1, kAdderThreads);  // all have read the decision before it is written again
    if (!go) break;
    adder_combine<INNER, ALGO, T>(fz.comb, fz.comb_quad[t], first, stride);
  }
}

// ---- sending CTAs of a row-sharded dense product -----------------------------------------------
// The tile order walks the m-tiles of a band, then moves to the next n-tile, so C is finished one
// block of columns (all rows of a band x the columns of one n-tile) after the other. Every epilogue
// warp counts its part of a tile on the counter of that block once its TMA stores have reached
// global memory; a sending CTA waits for a block's counter, reads the block from this GPU's C and
// writes it to the other copies: one multimem store per 16 bytes when a multicast address is given,
// else one store per peer. The wait is bounded like every other; all loads read local memory.
template <int kThreads>
__device__ __forceinline__ void run_sender(const GemmKernelParams& p, int sender, int n_senders, int tile_m, int tile_n,
                                           int parts_per_tile, volatile uint32_t* abort_word, volatile uint32_t* go_word) {
  const int n_bands = (p.m_tiles + p.raster_group - 1) / p.raster_group;
  const int units = n_bands * p.n_tiles;
  const int64_t row_bytes = p.ldc * 2;
  for (int u = sender; u < units; u += n_senders) {
    const int g = u / p.n_tiles, nt = u - g * p.n_tiles;
    const int gsz = min(p.raster_group, p.m_tiles - g * p.raster_group);
    if (threadIdx.x == 0) {
      const bool ok = ptx::wait_counter(p.send_counters + u, static_cast<uint32_t>(gsz * parts_per_tile), abort_word, kWhoSender);
      ptx::fence_proxy_async_all();   // the block was written by TMA stores
      *go_word = ok ? 1u : 0u;
    }
    __syncthreads();
    const bool go = *go_word != 0;
    __syncthreads();                  // all have read the decision before it is written again
    if (!go) break;
    const int r0 = g * p.raster_group * tile_m;
    const int nrows = min(gsz * tile_m, p.M - r0);
    const int c0 = nt * tile_n;
    const int vpr = (min(tile_n, p.N - c0) * 2) / 16;   // 16-byte vectors per row of the block
    const int total = nrows * vpr;
    const uint8_t* src = p.dst[0] + static_cast<int64_t>(r0) * row_bytes + static_cast<int64_t>(c0) * 2;
    const int64_t dst_off = static_cast<int64_t>(r0) * row_bytes + static_cast<int64_t>(c0) * 2;
    for (int i0 = threadIdx.x; i0 < total; i0 += 4 * kThreads) {
      uint4 v[4];
      int64_t off[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int i = i0 + k * kThreads;
        const int row = i / vpr, c = i - row * vpr;
        off[k] = static_cast<int64_t>(row) * row_bytes + c * 16;
        if (i < total) v[k] = __ldcg(reinterpret_cast<const uint4*>(src + off[k]));
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (i0 + k * kThreads < total) {
          if (p.mc != nullptr) {
            ptx::multimem_st_v4(p.mc + dst_off + off[k], v[k]);
          } else {
            for (int d = 1; d < p.n_dst; ++d) *reinterpret_cast<uint4*>(p.dst[d] + dst_off + off[k]) = v[k];
          }
        }
      }
    }
  }
}

__device__ __forceinline__ void decode_tile(const GemmKernelParams& p, int tile, int& b, int& mt,
                                            int& nt) {
  const int kGroup = p.raster_group;
  const int per_batch = p.m_tiles * p.n_tiles;
  b = tile / per_batch;
  int t = tile - b * per_batch;
  const int per_group = kGroup * p.n_tiles;
  const int g = t / per_group;
  const int first_m = g * kGroup;
  const int gsz = min(kGroup, p.m_tiles - first_m);
  t -= g * per_group;
  mt = first_m + t % gsz;
  nt = t / gsz;
}

template <typename OutT>
__device__ __forceinline__ OutT cvt_out(float v);
template <>
__device__ __forceinline__ float cvt_out<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ __nv_bfloat16 cvt_out<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ __half cvt_out<__half>(float v) {
  return __float2half_rn(v);
}
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }

// Adds the bias entries of columns [col, col + 32) (those below N) to 32 fp32 accumulator words.
__device__ __forceinline__ void add_bias32(uint32_t (&r)[32], const void* bias, int out_dt, int col, int N) {
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    if (col + j < N) {
      float b;
      if (out_dt == B200S_BF16)
        b = __bfloat162float(__ldg(static_cast<const __nv_bfloat16*>(bias) + col + j));
      else if (out_dt == B200S_FP16)
        b = __half2float(__ldg(static_cast<const __half*>(bias) + col + j));
      else
        b = __ldg(static_cast<const float*>(bias) + col + j);
      r[j] = __float_as_uint(__uint_as_float(r[j]) + b);
    }
  }
}

// Writes 32 consecutive columns of one row. `ncols` (<= 32) of them are inside the matrix.
template <typename OutT>
__device__ __forceinline__ void store_row32(OutT* dst, const uint32_t (&r)[32], int ncols,
                                            bool vec_ok, bool beta) {
  constexpr int kPerVec = 16 / sizeof(OutT);
  if (vec_ok && ncols == 32) {
#pragma unroll
    for (int v = 0; v < 32 / kPerVec; ++v) {
      union {
        uint4 u;
        OutT e[kPerVec];
      } pack;
      if (beta) {
        pack.u = *reinterpret_cast<const uint4*>(dst + v * kPerVec);
#pragma unroll
        for (int i = 0; i < kPerVec; ++i)
          pack.e[i] = cvt_out<OutT>(to_f32(pack.e[i]) + __uint_as_float(r[v * kPerVec + i]));
      } else {
#pragma unroll
        for (int i = 0; i < kPerVec; ++i) pack.e[i] = cvt_out<OutT>(__uint_as_float(r[v * kPerVec + i]));
      }
      *reinterpret_cast<uint4*>(dst + v * kPerVec) = pack.u;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if (i < ncols) {
        float v = __uint_as_float(r[i]);
        if (beta) v += to_f32(dst[i]);
        dst[i] = cvt_out<OutT>(v);
      }
    }
  }
}

// Destinations of C. A row-sharded product stores every finished tile into each GPU's copy of C (peer
// memory mapped into this process): the exchange is part of the epilogue, tile by tile, over NVLink.
// Copy 0 (this GPU's own) is written by TMA through a tensor map, the others by ordinary stores.
// Stores only - every load of this kernel reads this GPU's own memory.
constexpr int kMaxDst = 8;
struct CMaps {
  CUtensorMap m[1];
};

// kNH = number of 256-column accumulator halves one tile owns.
//   kNH == 1: tile N = 256, two accumulators used alternately, so the epilogue of tile i overlaps
//             the main loop of tile i+1; 4 epilogue warps.
//   kNH == 2: tile N = 512 (CTA pair: 256 x 512), both halves share each A block, which cuts the
//             shared-memory fill traffic per flop by a quarter; the single accumulator set is
//             drained by 8 epilogue warps before the next tile's first MMA.
//
// With F::kOn (the fused Strassen kernel, 256 x 512 tiles only) the CTA has four warpgroups: warps
// 0-3 producer, MMA issuer and two idle warps; warps 4-11 epilogue; warps 12-15 adders, which form
// operand blocks and recombine finished quadrants of C (run_adders) beside the products. The
// producer waits for a group's operand blocks before its first tile of that group, the epilogue
// warps count every stored tile so that the adders know when a group's products are complete.
// Registers move from the first warpgroup to the epilogue warpgroups (setmaxnreg).
template <int kCtaGroup, int kNH, int kStages, bool kTf32, class F>
__global__ void __launch_bounds__(F::kOn ? 512 : 64 + 128 * kNH, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CMaps tmC, const GemmKernelParams p,
            const __grid_constant__ typename F::Params fz) {
  static_assert(!F::kOn || (kCtaGroup == 2 && kNH == 2 && !kTf32), "the fused kernel exists for 256 x 512 tiles of 16-bit operands");
  constexpr int kEpiWarp0 = F::kOn ? 4 : 2;      // first epilogue warp
  constexpr int ES = kTf32 ? 4 : 2;              // operand element size
  constexpr int BKE = kRowBytes / ES;            // K elements per stage
  constexpr int BNH = 256;                       // columns of one accumulator half (one tcgen05.mma N)
  constexpr int BN_TILE = BNH * kNH;             // columns of C one tile covers
  constexpr int BNH_CTA = BNH / kCtaGroup;       // rows of one B half this CTA loads
  constexpr int A_BYTES = kBM * kRowBytes;
  constexpr int BH_BYTES = BNH_CTA * kRowBytes;  // one B half in this CTA's shared memory
  constexpr int STAGE_BYTES = A_BYTES + kNH * BH_BYTES;
  constexpr int CHUNK_E = kRowBytes / ES;        // MN elements per 128-byte row of an MN-major tile
  constexpr int CHUNK_BYTES = BKE * kRowBytes;   // one MN-major chunk: BKE k-rows of 128 bytes
  constexpr int UMMA_K = 32 / ES;                // K elements per tcgen05.mma
  constexpr int K_STEPS = BKE / UMMA_K;          // = 4
  constexpr int ACC_BUFS = kNH == 1 ? 2 : 1;     // accumulator sets in TMEM
  constexpr int EPI_WARPS = 4 * kNH;
  constexpr int STG_BUFS = kNH == 1 ? 2 : 1;     // 4 KB staging buffers per epilogue warp
  constexpr uint32_t TMEM_COLS = 512;
  constexpr int STAGING_BYTES = EPI_WARPS * STG_BUFS * 4096;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw);

  // Stages, then the epilogue staging buffers, then the barriers.
  const uint32_t staging_base = base + kStages * STAGE_BYTES;
  const uint32_t bar_base = staging_base + STAGING_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };
  volatile uint32_t* tmem_slot =
      reinterpret_cast<volatile uint32_t*>(gbase + kStages * STAGE_BYTES + STAGING_BYTES + 8 * (2 * kStages + 4));
  volatile uint32_t* abort_word = tmem_slot + 1;
  [[maybe_unused]] volatile uint32_t* go_word = tmem_slot + 2;  // go / stop decision of the adders (fused kernel) or of a sending CTA

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = (kCtaGroup == 2) ? ptx::cluster_ctarank() : 0u;
  const int cluster_id = blockIdx.x / kCtaGroup;
  // clusters that multiply; the sending CTAs of a row-sharded product come after them in the grid
  const int num_clusters = (static_cast<int>(gridDim.x) - (F::kSend ? p.send_ctas : 0)) / kCtaGroup;
  [[maybe_unused]] const bool is_sender = F::kSend && cluster_id >= num_clusters;

  if (threadIdx.x == 0) {
    *abort_word = 0;
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(tfull_bar(b), 1);
      ptx::mbar_init(tempty_bar(b), EPI_WARPS * kCtaGroup);
    }
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tmA);
    ptx::prefetch_tensormap(&tmB);
    if (p.tma_store) ptx::prefetch_tensormap(&tmC.m[0]);
  }
  if (warp == 1) {
    ptx::tmem_alloc<kCtaGroup>(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    ptx::tmem_relinquish<kCtaGroup>();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if constexpr (kCtaGroup == 2) {
    ptx::cluster_arrive();
    ptx::cluster_wait();
  }
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // Fused kernel: 512 threads start with 128 registers each and re-divide them by warpgroup,
  // 40 (producer, MMA issuer) + 168 + 168 (epilogue) + 136 (adders) per thread.
  if (is_sender) {
    if constexpr (F::kSend) {
      constexpr int kThreadsAll = 64 + 128 * kNH;
      run_sender<kThreadsAll>(p, (cluster_id - num_clusters) * kCtaGroup + static_cast<int>(cta_rank), p.send_ctas,
                              kBM * kCtaGroup, BN_TILE, EPI_WARPS * kCtaGroup, abort_word, go_word);
    }
  } else if (warp < kEpiWarp0) {
  if constexpr (F::kOn) ptx::setmaxnreg_dec<40>();
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool alive = true;
      [[maybe_unused]] int group_ready = 0;
      if constexpr (F::kOn) group_ready = fz.groups_formed;
      int it = 0;
      for (int tile = cluster_id; alive && tile < p.total_tiles; tile += num_clusters, ++it) {
        int b, mt, nt;
        decode_tile(p, tile, b, mt, nt);
        // Every other wave of tiles walks K backwards: a cluster then starts its next tile with the K
        // slices its neighbours touched last, which are the ones still in L2 (walking forwards every
        // time is the cyclic pattern an LRU cache serves worst). A wave is counted in tiles of the
        // whole device, not of this launch's grid, so the order of the additions along K, and with
        // it every bit of the result, is the same on any number of SMs.
        const bool k_reversed = ((tile / p.wave_tiles) & 1) != 0;
        if constexpr (F::kOn) {
          // first tile of a new outer group: every CTA's adders must have stored its operand blocks
          const int g = b / fz.np2;
          if (g >= group_ready) {
            if (!ptx::wait_counter(fz.flags + g, fz.ready_target * gridDim.x, abort_word, kWhoProducerGroup)) {
              alive = false;
              break;
            }
            ptx::fence_proxy_async_all();
            group_ready = g + 1;
          }
        }
        const int m0 = mt * (kBM * kCtaGroup) + static_cast<int>(cta_rank) * kBM;
        const int n0 = nt * BN_TILE + static_cast<int>(cta_rank) * BNH_CTA;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!ptx::mbar_wait<kCtaGroup == 2>(empty_bar(stage), phase ^ 1u, abort_word, kWhoProducer)) {
            alive = false;
            break;
          }
          const uint32_t sA = base + stage * STAGE_BYTES;
          const uint32_t sB = sA + A_BYTES;
          const int k0 = (k_reversed ? p.k_blocks - 1 - kb : kb) * BKE;
          // With a CTA pair both CTAs' bytes are counted on the leader's barrier.
          uint32_t fb = full_bar(stage);
          if constexpr (kCtaGroup == 2) fb = ptx::mapa_cluster(fb, 0);
          if (cta_rank == 0) ptx::mbar_expect_tx(full_bar(stage), kCtaGroup * STAGE_BYTES);
          auto load = [&](uint32_t dst, const CUtensorMap* m, int c0, int c1) {
            if constexpr (kCtaGroup == 2)
              ptx::tma_load_3d_pair(dst, m, fb, c0, c1, b);
            else
              ptx::tma_load_3d(dst, m, fb, c0, c1, b);
          };
          if (!p.a_mn) {
            load(sA, &tmA, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < kBM / CHUNK_E; ++j) load(sA + j * CHUNK_BYTES, &tmA, m0 + j * CHUNK_E, k0);
          }
#pragma unroll
          for (int h = 0; h < kNH; ++h) {
            const uint32_t sBh = sB + h * BH_BYTES;
            const int nh = n0 + h * BNH;
            if (!p.b_mn) {
              load(sBh, &tmB, k0, nh);
            } else {
#pragma unroll
              for (int j = 0; j < BNH_CTA / CHUNK_E; ++j) load(sBh + j * CHUNK_BYTES, &tmB, nh + j * CHUNK_E, k0);
            }
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!alive && cta_rank == 0) {
        // (The second CTA of a pair cannot poll these barriers; the cluster barrier of the teardown
        // holds it until this CTA is past this point.)
        // Giving up with copies possibly still in flight into this CTA's (and, in a pair, the
        // peer's) shared memory: only the last kStages loads can be outstanding, and their bytes are
        // counted on this CTA's full barriers. Let them land, within a limit, before the teardown
        // lets any CTA of the cluster leave. Stages below `stage` were armed in the current pass
        // over the ring, the others in the pass before (a barrier never armed reads as complete).
        const uint64_t deadline = ptx::global_timer_ns() + kDrainLimitNs;
        for (uint32_t s = 0; s < static_cast<uint32_t>(kStages); ++s)
          if (!ptx::mbar_wait_until(full_bar(static_cast<int>(s)), s < stage ? phase : phase ^ 1u, deadline)) break;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && cta_rank == 0) {
      const uint32_t idesc =
          ptx::make_instr_desc(static_cast<uint32_t>(p.fmt), p.a_mn, p.b_mn, kBM * kCtaGroup, BNH);
      // K-major: 8-row groups 1024 bytes apart, K advances 32 bytes inside the swizzled row.
      // MN-major: 8-k-row groups 1024 bytes apart (SBO), 128-byte MN chunks CHUNK_BYTES apart (LBO).
      const uint32_t a_lbo = p.a_mn ? CHUNK_BYTES : 16u, b_lbo = p.b_mn ? CHUNK_BYTES : 16u;
      const uint32_t a_adv = p.a_mn ? (UMMA_K / 8) * 1024u : 32u;
      const uint32_t b_adv = p.b_mn ? (UMMA_K / 8) * 1024u : 32u;
      const uint64_t a_desc0 = ptx::make_smem_desc(base, a_lbo, 1024u);
      const uint64_t b_desc0 = ptx::make_smem_desc(base + A_BYTES, b_lbo, 1024u);
      uint32_t stage = 0, phase = 0;
      int it = 0;
      bool alive = true;
      for (int tile = cluster_id; alive && tile < p.total_tiles; tile += num_clusters, ++it) {
        const int buf = it % ACC_BUFS;
        const uint32_t aphase = (it / ACC_BUFS) & 1u;
        if (!ptx::mbar_wait<kCtaGroup == 2>(tempty_bar(buf), aphase ^ 1u, abort_word, kWhoMmaAcc)) {
          alive = false;
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t acc = tmem_base + static_cast<uint32_t>(buf * BN_TILE);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!ptx::mbar_wait<kCtaGroup == 2>(full_bar(stage), phase, abort_word, kWhoMma)) {
            alive = false;
            break;
          }
          ptx::tc_fence_after_sync();
          // descriptors differ from the stage-0 ones only in the (16-byte granular) start address
          const uint32_t soff = stage * (STAGE_BYTES >> 4);
          const uint32_t accf = kb != 0 ? 1u : 0u;
#pragma unroll
          for (int h = 0; h < kNH; ++h) {
#pragma unroll
            for (int k = 0; k < K_STEPS; ++k) {
              const uint64_t ad = a_desc0 + (soff + k * (a_adv >> 4));
              const uint64_t bd = b_desc0 + (soff + h * (BH_BYTES >> 4) + k * (b_adv >> 4));
              ptx::umma<kCtaGroup, kTf32>(acc + h * BNH, ad, bd, idesc, k == 0 ? accf : 1u);
            }
          }
          // Frees the stage (in both CTAs) once the MMAs above have read it.
          ptx::umma_commit<kCtaGroup>(empty_bar(stage));
          if constexpr (kCtaGroup == 2) ptx::umma_commit<kCtaGroup>(ptx::mapa_cluster(empty_bar(stage), 1));
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!alive) break;
        ptx::umma_commit<kCtaGroup>(tfull_bar(buf));
        if constexpr (kCtaGroup == 2) ptx::umma_commit<kCtaGroup>(ptx::mapa_cluster(tfull_bar(buf), 1));
      }
    }
    __syncwarp();
  }
  } else if (warp < kEpiWarp0 + EPI_WARPS) {
    // ------------------------------------------------------------ epilogue
    if constexpr (F::kOn) ptx::setmaxnreg_inc<168>();
    const int ew = warp - kEpiWarp0;  // epilogue warp index
    const int lane_group = warp & 3;  // TMEM lanes [32*lane_group, +32) belong to this warp
    const int half = ew >> 2;         // which 256-column half of the tile this warp drains
    const int out_dt = p.out_dtype;
    const size_t out_es = (out_dt == B200S_FP32) ? 4 : 2;
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.C) & 15u) == 0) && ((p.ldc * out_es) % 16 == 0) &&
                        ((p.strideC * out_es) % 16 == 0);
    const uint32_t stg = staging_base + static_cast<uint32_t>(ew * STG_BUFS) * 4096u;
    const uint32_t sw = static_cast<uint32_t>(lane & 7);
    // C is not read again by this kernel: let its lines leave L2 before the operand tiles do
    const uint64_t store_policy = ptx::make_evict_first_policy();
    int it = 0;
    int stage_flip = 0;
    // Several destinations: the tiles of a wave finish together, and with them come the remote stores
    // of all CTAs of all GPUs in one burst. The epilogue is not needed again before the next tile is
    // done, so every cluster holds its stores back by its own share of the tile period it observed
    // last: the bursts become a steady stream.
    uint32_t tile_seen_ns = 0, hold_ns = 0;
    for (int tile = cluster_id; tile < p.total_tiles; tile += num_clusters, ++it) {
      int b, mt, nt;
      decode_tile(p, tile, b, mt, nt);
      const int buf = it % ACC_BUFS;
      const uint32_t aphase = (it / ACC_BUFS) & 1u;
      // one lane waits, the warp follows
      int ok = 1;
      if (lane == 0) ok = ptx::mbar_wait<kCtaGroup == 2, 64>(tfull_bar(buf), aphase, abort_word, kWhoEpilogue) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (p.n_dst > 1 && p.stagger && !F::kSend) {
        const uint32_t now = static_cast<uint32_t>(ptx::global_timer_ns());  // differences survive the wrap
        if (it > 0) {
          const uint32_t period = now - tile_seen_ns;
          // clusters 0 .. n-1 spread over 60 % of the period; nothing for periods under 20 us or over 50 ms
          hold_ns = (period > 20000u && period < 50000000u)
                        ? (period / 10u * 6u) * static_cast<uint32_t>(cluster_id) / static_cast<uint32_t>(num_clusters)
                        : 0u;   // at most 3e7 x 73: fits 32 bits
        }
        tile_seen_ns = now;
      }
      ptx::tc_fence_after_sync();
      const int row_warp = mt * (kBM * kCtaGroup) + static_cast<int>(cta_rank) * kBM + lane_group * 32;
      const int row = row_warp + lane;
      const int col0 = nt * BN_TILE + half * BNH;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) +
                             static_cast<uint32_t>(buf * BN_TILE + half * BNH);
      bool released = false;
      auto release_accumulator = [&]() {
        // every tcgen05.ld of this warp has completed: hand the accumulator back to the MMA warp
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (kCtaGroup == 2)
            ptx::mbar_arrive_cluster(tempty_bar(buf), 0);
          else
            ptx::mbar_arrive(tempty_bar(buf));
        }
        released = true;
      };
      auto stage_and_store = [&](const uint32_t (&h)[32], int gc) {
        const uint32_t sbuf = stg + static_cast<uint32_t>(stage_flip) * 4096u;
        const uint32_t srow = sbuf + static_cast<uint32_t>(lane) * 128u;
        // the store that last read this staging buffer must be done with it
        if (lane == 0) ptx::tma_store_wait_read<STG_BUFS - 1>();
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j)
          ptx::st_shared_v4(srow + ((static_cast<uint32_t>(j) ^ sw) << 4), h[4 * j], h[4 * j + 1], h[4 * j + 2],
                            h[4 * j + 3]);
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          ptx::tma_store_3d_hint(&tmC.m[0], sbuf, col0 + gc, row_warp, b, store_policy);
          ptx::tma_store_commit();
        }
        if (p.n_dst > 1 && !F::kSend) {
          // The other copies of C (peer GPUs' memory) get the same box through ordinary 16-byte
          // stores, whole 128-byte rows per quarter warp. They travel through the load/store unit, so
          // a slow NVLink write never sits in the TMA queue in front of the next operand loads.
          const int rr = lane >> 3, cc = lane & 7;
          const int64_t byte_col = static_cast<int64_t>(col0 + gc) * static_cast<int64_t>(out_es) + cc * 16;
          const bool col_ok = byte_col < static_cast<int64_t>(p.N) * static_cast<int64_t>(out_es);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = 4 * i + rr;
            const uint4 v = ptx::ld_shared_v4(sbuf + static_cast<uint32_t>(r) * 128u +
                                              ((static_cast<uint32_t>(cc) ^ static_cast<uint32_t>(r & 7)) << 4));
            const int grow = row_warp + r;
            if (col_ok && grow < p.M) {
              const int64_t off = (static_cast<int64_t>(b) * p.strideC + static_cast<int64_t>(grow) * p.ldc) *
                                      static_cast<int64_t>(out_es) + byte_col;
              if (p.mc != nullptr) {
                ptx::multimem_st_v4(p.mc + off, v);   // one store, replicated to every GPU by the NVSwitch
              } else {
                for (int d = 1; d < p.n_dst; ++d) *reinterpret_cast<uint4*>(p.dst[d] + off) = v;
              }
            }
          }
          __syncwarp();
        }
        if constexpr (STG_BUFS == 2) stage_flip ^= 1;
      };
      if (p.tma_store && out_es == 2) {
        // 128-byte row groups of 64 columns: tcgen05.ld -> convert -> swizzled st.shared -> one TMA
        // store of a 32-row x 128-byte box. The loads of group g+1 are in flight while group g is
        // staged and stored.
        // First the whole accumulator goes to registers (converted, 128 packed words per thread) and
        // is handed back, then the staging and the stores run while the MMA warp already works on
        // the next tile.
        constexpr int kChunks = BNH / 32;
        uint32_t hp[kChunks * 16];
        uint32_t r[32];
        ptx::tmem_ld_32x32(taddr, r);
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
          ptx::tmem_ld_wait();
          if (p.bias != nullptr) add_bias32(r, p.bias, out_dt, col0 + c * 32, p.N);
          if (out_dt == B200S_BF16) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              hp[c * 16 + j] = ptx::pack_bf16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              hp[c * 16 + j] = ptx::pack_f16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
          }
          if (c + 1 < kChunks) ptx::tmem_ld_32x32(taddr + (c + 1) * 32, r);
        }
        release_accumulator();
        if (hold_ns != 0) {
          // bounded by construction: at most 60 % of a period of at most 50 ms, in short sleeps
          const uint32_t t0 = static_cast<uint32_t>(ptx::global_timer_ns());
          while (static_cast<uint32_t>(ptx::global_timer_ns()) - t0 < hold_ns) __nanosleep(1000);
        }
#pragma unroll
        for (int g = 0; g < kChunks / 2; ++g) {
          uint32_t h[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) h[j] = hp[g * 32 + j];
          stage_and_store(h, g * 64);
        }
        if constexpr (F::kOn) {
          // count this warp's part of the tile once its stores have reached global memory
          if (lane == 0) {
            ptx::tma_store_wait_all<0>();
            ptx::fence_proxy_async_all();
            __threadfence();
            ptx::red_release_gpu_add(fz.flags + 8 + b / fz.np2, 1u);
          }
          __syncwarp();
        }
        if constexpr (F::kSend) {
          if (p.send_ctas > 0) {
            // the same for the sending CTAs: this warp's part of the block of columns is in global memory
            if (lane == 0) {
              ptx::tma_store_wait_all<0>();
              ptx::fence_proxy_async_all();
              __threadfence();
              ptx::red_release_gpu_add(p.send_counters + (mt / p.raster_group) * p.n_tiles + nt, 1u);
            }
            __syncwarp();
          }
        }
      } else if (p.tma_store) {
#pragma unroll 1
        for (int gc = 0; gc < BNH; gc += 32) {
          uint32_t h[32];
          ptx::tmem_ld_32x32(taddr + gc, h);
          ptx::tmem_ld_wait();
          if (p.bias != nullptr) add_bias32(h, p.bias, out_dt, col0 + gc, p.N);
          stage_and_store(h, gc);
        }
      } else {
        uint8_t* crow = static_cast<uint8_t*>(p.C) +
                        (static_cast<int64_t>(b) * p.strideC + static_cast<int64_t>(row) * p.ldc) * out_es;
#pragma unroll 1
        for (int c = 0; c < BNH / 32; ++c) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(taddr + c * 32, r);
          ptx::tmem_ld_wait();
          const int col = col0 + c * 32;
          const int ncols = min(32, p.N - col);
          if (p.bias != nullptr) add_bias32(r, p.bias, out_dt, col, p.N);
          if (row < p.M && ncols > 0) {
            if (out_dt == B200S_BF16)
              store_row32(reinterpret_cast<__nv_bfloat16*>(crow) + col, r, ncols, vec_ok, p.beta != 0);
            else if (out_dt == B200S_FP16)
              store_row32(reinterpret_cast<__half*>(crow) + col, r, ncols, vec_ok, p.beta != 0);
            else
              store_row32(reinterpret_cast<float*>(crow) + col, r, ncols, vec_ok, p.beta != 0);
          }
        }
      }
      if (!released) release_accumulator();
    }
    if (p.tma_store && lane == 0) ptx::tma_store_wait_all<0>();  // shared memory must outlive the stores
    __syncwarp();
  } else {
    // ------------------------------------------------------------ adders (fused kernel only)
    if constexpr (F::kOn) {
      ptx::setmaxnreg_inc<136>();
      run_adders<F>(fz, abort_word, go_word, static_cast<int>(threadIdx.x) - 32 * (kEpiWarp0 + EPI_WARPS));
    }
  }

  // ------------------------------------------------------------ teardown
  ptx::tc_fence_before_sync();
  __syncthreads();
  if constexpr (kCtaGroup == 2) {
    // Neither CTA may leave while its peer can still signal its barriers or read its tiles.
    ptx::cluster_arrive();
    ptx::cluster_wait();
  }
  if (threadIdx.x == 0 && *abort_word != 0) {
    atomicExch(&p.status[0], 1u);
    atomicExch(&p.status[1], *abort_word);
  }
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc<kCtaGroup>(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(f);
  });
  return fn;
}

// Tensor map over an operand stored as [batch][rows][cols], cols contiguous, with a box of
// box_rows x (128 bytes of cols) and the 128-byte swizzle.
int make_operand_map(CUtensorMap* map, const void* ptr, int dtype, int64_t rows, int64_t cols, int64_t ld,
                     int64_t batch, int64_t batch_stride, int box_rows, bool for_store = false) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return B200S_ERR_CUDA;
  const size_t es = dtype_size(dtype);
  CUtensorMapDataType dt = dtype == B200S_BF16   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : dtype == B200S_FP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows),
                        static_cast<cuuint64_t>(batch)};
  // A single batch item still needs a legal (multiple of 16 bytes) outer stride.
  int64_t bs = batch > 1 ? batch_stride : rows * ld;
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * es, static_cast<cuuint64_t>(bs) * es};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(kRowBytes / es), static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, dt, 3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, for_store ? CU_TENSOR_MAP_L2_PROMOTION_NONE : CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    note_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
    return B200S_ERR_CUDA;
  }
  return B200S_OK;
}

// m-tiles that share a band of n-tiles in the tile order. Consecutive waves of a band re-read the
// band's rows of A: with 8 m-tiles those rows stay in L2 between waves as long as K is moderate
// (8 x 256 rows x K elements within a good half of L2: K = 16384 in bf16 still qualifies); for longer K nothing survives between waves
// anyway and a taller band wins because one wave then touches fewer distinct operand bytes.
// Measured on B200, bf16: 16384^3 6.3 ms with 8 against 6.9 ms with 16; 16384 x 32768 x 32768
// 28.5 ms with 8 against 25.3 ms with 16 (cuBLAS 24.8 ms).
constexpr int kRasterGroup = 8;
constexpr int kRasterGroupLongK = 16;
constexpr double kBandBytesInL2 = 72.0 * 1024 * 1024;

template <int kCtaGroup, int kNH, int kStages, bool kTf32, class F>
int launch_variant(const CUtensorMap& tmA, const CUtensorMap& tmB, const CMaps& tmC, GemmKernelParams kp,
                   const typename F::Params& fz, int sms, int all_sms, cudaStream_t stream) {
  constexpr int kThreadsV = F::kOn ? 512 : 64 + 128 * kNH;
  constexpr int STAGE_BYTES = kBM * kRowBytes + kNH * (256 / kCtaGroup) * kRowBytes;
  constexpr int STAGING_BYTES = 4 * kNH * (kNH == 1 ? 2 : 1) * 4096;
  constexpr int SMEM = kStages * STAGE_BYTES + STAGING_BYTES + 8 * (2 * kStages + 4) + 16 + 1024;
  static_assert(SMEM <= 227 * 1024, "shared memory budget");
  auto kernel = gemm_kernel<kCtaGroup, kNH, kStages, kTf32, F>;

  // Per-device one-time setup: opt in to the shared-memory size and find out how many
  // clusters can be resident at once (static tile striding needs all of them co-resident).
  static std::mutex mu;
  static int max_clusters[64] = {0};
  int dev = 0;
  B200S_CUDA_OK(cudaGetDevice(&dev));
  int resident;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= 64) return B200S_ERR_NO_DEVICE;
    if (max_clusters[dev] == 0) {
      B200S_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
      // all_sms: the capacity of the device, whatever share of it this call may use
      int n = all_sms / kCtaGroup;
      if (kCtaGroup == 2) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(all_sms / 2 * 2);
        cfg.blockDim = dim3(kThreadsV);
        cfg.dynamicSmemBytes = SMEM;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2;
        at[0].val.clusterDim.y = 1;
        at[0].val.clusterDim.z = 1;
        cfg.attrs = at;
        cfg.numAttrs = 1;
        int q = 0;
        B200S_CUDA_OK(cudaOccupancyMaxActiveClusters(&q, kernel, &cfg));
        if (q < 1) return B200S_ERR_CUDA;
        if (q < n) n = q;
      }
      max_clusters[dev] = n;
    }
    resident = max_clusters[dev];
  }
  if (sms / kCtaGroup < resident) resident = sms / kCtaGroup;

  // sending CTAs (a row-sharded product) come on top of the clusters that multiply
  const int send_clusters = F::kSend ? kp.send_ctas / kCtaGroup : 0;
  int clusters = resident - send_clusters;
  if (clusters < 1) return B200S_ERR_BAD_SHAPE;
  if (kp.total_tiles < clusters) clusters = kp.total_tiles;
  clusters += send_clusters;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(clusters * kCtaGroup);
  cfg.blockDim = dim3(kThreadsV);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = kCtaGroup;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  B200S_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, tmA, tmB, tmC, kp, fz));
  count_launch();
  return B200S_OK;
}

struct Prepared {
  CUtensorMap tmA, tmB;
  CMaps tmC;
  GemmKernelParams kp;
  int variant, sms;
  int all_sms;          // SMs of the device (sms may be a share of them)
  bool tf32;
  int send_units = 0;   // counters the sending CTAs wait on (0: no sending CTAs)
};

// Validates the product, picks the tile variant (forced_variant > 0 overrides), builds the tensor
// maps and the kernel parameters.
int prepare_gemm(const GemmArgs& g, int forced_variant, Prepared* out) {
  if (g.M <= 0 || g.N <= 0 || g.K <= 0 || g.batch <= 0) return B200S_ERR_BAD_SHAPE;
  if (g.M > INT32_MAX || g.N > INT32_MAX || g.K > INT32_MAX) return B200S_ERR_BAD_SHAPE;
  const bool tf32 = g.in_dtype == B200S_FP32;
  const size_t es = dtype_size(g.in_dtype);
  if ((reinterpret_cast<uintptr_t>(g.A) & 15u) || (reinterpret_cast<uintptr_t>(g.B) & 15u))
    return B200S_ERR_BAD_ALIGNMENT;
  if ((g.lda * es) % 16 || (g.ldb * es) % 16) return B200S_ERR_BAD_STRIDE;
  if (g.batch > 1 && ((g.strideA * es) % 16 || (g.strideB * es) % 16)) return B200S_ERR_BAD_STRIDE;

  uint32_t* status = g.status ? g.status : device_status_words();
  if (!status) return B200S_ERR_CUDA;
  const int sms = g.sms > 0 ? g.sms : product_sm_count();
  if (sms < 2) return B200S_ERR_NO_DEVICE;

  // Tile variant: 1 = one CTA, 128 x 256 tiles; 2 = CTA pair, 256 x 256 tiles, double-buffered
  // accumulators; 3 = CTA pair, 256 x 512 tiles. Wide outputs default to 3, narrow ones to 2.
  int variant = forced_variant > 0 ? forced_variant : g.cta_group;
  if (variant == 0) variant = (g.N >= 1024 && g.M >= 256) ? 3 : 2;
  const int cta_group = variant == 1 ? 1 : 2;
  const int nh = variant == 3 ? 2 : 1;
  const int BN = 256 * nh;
  const int bke = kRowBytes / static_cast<int>(es);

  int rc;
  // K-major operands are stored [rows = M or N][cols = K]; MN-major ones [rows = K][cols = M or N].
  if (g.a_major == B200S_K_MAJOR)
    rc = make_operand_map(&out->tmA, g.A, g.in_dtype, g.M, g.K, g.lda, g.batch, g.strideA, kBM);
  else
    rc = make_operand_map(&out->tmA, g.A, g.in_dtype, g.K, g.M, g.lda, g.batch, g.strideA, bke);
  if (rc) return rc;
  const int bn_cta = 256 / cta_group;  // rows of one B half this CTA loads
  if (g.b_major == B200S_K_MAJOR)
    rc = make_operand_map(&out->tmB, g.B, g.in_dtype, g.N, g.K, g.ldb, g.batch, g.strideB, bn_cta);
  else
    rc = make_operand_map(&out->tmB, g.B, g.in_dtype, g.K, g.N, g.ldb, g.batch, g.strideB, bke);
  if (rc) return rc;

  // The epilogue stores through TMA when C can be described by a tensor map and is overwritten.
  const size_t oes = dtype_size(g.out_dtype);
  const bool tma_store = g.beta == 0 && (reinterpret_cast<uintptr_t>(g.C) & 15u) == 0 && (g.ldc * oes) % 16 == 0 &&
                         (g.batch == 1 || (g.strideC * oes) % 16 == 0);
  const int n_dst = g.n_dst > 0 ? g.n_dst : 1;
  if (n_dst > kMaxDst) return B200S_ERR_BAD_SHAPE;
  if (n_dst > 1 && !tma_store) return B200S_ERR_BAD_ALIGNMENT;  // several destinations exist only for the TMA-store epilogue
  if (n_dst > 1 && (g.N * oes) % 16) return B200S_ERR_BAD_STRIDE;  // the extra copies are written in whole 16-byte pieces
  out->tmC.m[0] = out->tmA;  // never dereferenced unless built below
  out->kp.mc = nullptr;
  if (g.mc_dst) {
    if (n_dst != 1 || !tma_store) return B200S_ERR_BAD_SHAPE;  // one local copy by TMA plus the multicast address
    if (reinterpret_cast<uintptr_t>(g.mc_dst) & 15u) return B200S_ERR_BAD_ALIGNMENT;
    if ((g.N * oes) % 16) return B200S_ERR_BAD_STRIDE;
    out->kp.mc = static_cast<uint8_t*>(g.mc_dst);
  }
  for (int d = 0; d < kMaxDst; ++d) {
    out->kp.dst[d] = nullptr;
    if (tma_store && d < n_dst) {
      void* dst = g.n_dst > 0 ? g.C_list[d] : g.C;
      if (!dst) return B200S_ERR_NULL_POINTER;
      if (reinterpret_cast<uintptr_t>(dst) & 15u) return B200S_ERR_BAD_ALIGNMENT;
      out->kp.dst[d] = static_cast<uint8_t*>(dst);
      if (d == 0) {
        rc = make_operand_map(&out->tmC.m[0], dst, g.out_dtype, g.M, g.N, g.ldc, g.batch, g.strideC, 32, true);
        if (rc) return rc;
      }
    }
  }

  GemmKernelParams& kp = out->kp;
  kp.bias = g.bias;
  kp.tma_store = tma_store ? 1 : 0;
  kp.n_dst = kp.mc ? 2 : n_dst;
  kp.stagger = (kp.n_dst > 1 && kp.mc == nullptr) ? 1 : 0;  // measured: helps per-peer stores, nothing for multicast
  kp.M = static_cast<int32_t>(g.M);
  kp.N = static_cast<int32_t>(g.N);
  const int tile_m = kBM * cta_group;
  kp.m_tiles = static_cast<int32_t>((g.M + tile_m - 1) / tile_m);
  kp.n_tiles = static_cast<int32_t>((g.N + BN - 1) / BN);
  kp.k_blocks = static_cast<int32_t>((g.K + bke - 1) / bke);
  const int64_t total = static_cast<int64_t>(kp.m_tiles) * kp.n_tiles * g.batch;
  if (total > INT32_MAX) return B200S_ERR_BAD_SHAPE;
  kp.total_tiles = static_cast<int32_t>(total);
  const double band_bytes = static_cast<double>(kRasterGroup) * tile_m * static_cast<double>(g.K) * static_cast<double>(es);
  kp.raster_group = band_bytes <= kBandBytesInL2 ? kRasterGroup : kRasterGroupLongK;
  const int all_sms = g.sms > 0 ? g.sms : sm_count();
  kp.wave_tiles = all_sms / cta_group > 0 ? all_sms / cta_group : 1;
  out->all_sms = all_sms;
  kp.send_ctas = 0;
  kp.send_counters = nullptr;
  if (g.send_sms >= 2 && kp.n_dst > 1) {
    // Sending CTAs exist for the 256x512 CTA-pair variant with 16-bit output through the TMA-store
    // epilogue; any other product keeps the exchange in its epilogue.
    const int64_t units = static_cast<int64_t>((kp.m_tiles + kp.raster_group - 1) / kp.raster_group) * kp.n_tiles;
    const int send = (g.send_sms & ~1);
    if (variant == 3 && !tf32 && tma_store && oes == 2 && g.batch == 1 && units <= kSendUnits && sms - send >= 2) {
      kp.send_counters = device_send_counters();
      if (!kp.send_counters) return B200S_ERR_NO_DEVICE;
      kp.send_ctas = send;
      out->send_units = static_cast<int>(units);
    }
  }
  kp.a_mn = g.a_major == B200S_MN_MAJOR;
  kp.b_mn = g.b_major == B200S_MN_MAJOR;
  kp.fmt = tf32 ? 2 : (g.in_dtype == B200S_BF16 ? 1 : 0);
  kp.out_dtype = g.out_dtype;
  kp.beta = g.beta;
  kp.ldc = g.ldc;
  kp.strideC = g.strideC;
  kp.C = g.C;
  kp.status = status;
  out->variant = variant;
  out->sms = sms;
  out->tf32 = tf32;
  return B200S_OK;
}

template <int INNER, int ALGO>
int launch_fused_dtype(const Prepared& pr, const FusedKernelParams& fz, int dtype, cudaStream_t stream) {
  if (dtype == B200S_BF16)
    return launch_variant<2, 2, 4, false, Fuse<INNER, ALGO, __nv_bfloat16>>(pr.tmA, pr.tmB, pr.tmC, pr.kp, fz, pr.sms, pr.all_sms, stream);
  if (dtype == B200S_FP16)
    return launch_variant<2, 2, 4, false, Fuse<INNER, ALGO, __half>>(pr.tmA, pr.tmB, pr.tmC, pr.kp, fz, pr.sms, pr.all_sms, stream);
  return B200S_ERR_BAD_DTYPE;
}

// ---- self-test of the bounded wait ---------------------------------------------------------------
// One thread waits on an mbarrier that nobody ever arrives on, with the caller's limit instead of the
// kernels' two seconds, and reports the give-up exactly as the GEMM roles do: abort word, then the
// device status words. Nothing else runs in the CTA (no TMA, no tensor memory), so running out of
// time leaves nothing in flight.
__global__ void __launch_bounds__(32) wait_probe_kernel(uint64_t limit_ns, uint32_t* status) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t abort_word;
  if (threadIdx.x == 0) {
    abort_word = 0;
    ptx::mbar_init(ptx::smem_u32(&bar), 1);
    ptx::fence_mbar_init();
    const bool ok = ptx::mbar_wait_limit<false, 64>(ptx::smem_u32(&bar), 0u, &abort_word, kWhoProbe, limit_ns);
    if (!ok) {
      atomicExch(&status[0], 1u);
      atomicExch(&status[1], abort_word);
    }
  }
}

}  // namespace

int launch_wait_probe(uint64_t limit_ns, cudaStream_t stream) {
  uint32_t* status = device_status_words();
  if (!status) return B200S_ERR_NO_DEVICE;
  wait_probe_kernel<<<1, 32, 0, stream>>>(limit_ns, status);
  B200S_CUDA_OK(cudaGetLastError());
  count_launch();
  return B200S_OK;
}

int launch_gemm(const GemmArgs& g, cudaStream_t stream) {
  Prepared pr;
  int rc = prepare_gemm(g, 0, &pr);
  if (rc) return rc;
  const NoFuse::Params none{};
  if (pr.kp.send_ctas > 0) {
    const WithSenders::Params none_s{};
    B200S_CUDA_OK(cudaMemsetAsync(pr.kp.send_counters, 0, sizeof(uint32_t) * static_cast<size_t>(pr.send_units), stream));
    return launch_variant<2, 2, 4, false, WithSenders>(pr.tmA, pr.tmB, pr.tmC, pr.kp, none_s, pr.sms, pr.all_sms, stream);
  }
  if (pr.variant == 3) {
    if (pr.tf32) return launch_variant<2, 2, 4, true, NoFuse>(pr.tmA, pr.tmB, pr.tmC, pr.kp, none, pr.sms, pr.all_sms, stream);
    return launch_variant<2, 2, 4, false, NoFuse>(pr.tmA, pr.tmB, pr.tmC, pr.kp, none, pr.sms, pr.all_sms, stream);
  }
  if (pr.variant == 2) {
    if (pr.tf32) return launch_variant<2, 1, 6, true, NoFuse>(pr.tmA, pr.tmB, pr.tmC, pr.kp, none, pr.sms, pr.all_sms, stream);
    return launch_variant<2, 1, 6, false, NoFuse>(pr.tmA, pr.tmB, pr.tmC, pr.kp, none, pr.sms, pr.all_sms, stream);
  }
  if (pr.tf32) return launch_variant<1, 1, 4, true, NoFuse>(pr.tmA, pr.tmB, pr.tmC, pr.kp, none, pr.sms, pr.all_sms, stream);
  return launch_variant<1, 1, 4, false, NoFuse>(pr.tmA, pr.tmB, pr.tmC, pr.kp, none, pr.sms, pr.all_sms, stream);
}

int launch_fused(const FusedArgs& f, cudaStream_t stream) {
  const GemmArgs& g = f.gemm;
  const bool wino = f.algo == B200S_ALGO_WINOGRAD;
  if (!wino && f.algo != B200S_ALGO_CLASSIC) return B200S_ERR_BAD_ALGO;
  if (f.depth != 1 && f.depth != 2) return B200S_ERR_BAD_DEPTH;
  if (g.in_dtype != B200S_BF16 && g.in_dtype != B200S_FP16) return B200S_ERR_BAD_DTYPE;
  if (g.out_dtype != g.in_dtype || g.beta != 0) return B200S_ERR_BAD_DTYPE;  // products are stored in the operand dtype
  if (!f.flags || !f.A || !f.B || !f.C) return B200S_ERR_NULL_POINTER;
  if (f.groups_formed < 1 || f.groups_formed > 7) return B200S_ERR_BAD_SHAPE;
  const int np2 = f.depth == 2 ? 7 : 1;
  if (g.batch != 7 * np2) return B200S_ERR_BAD_SHAPE;
  const int sa = wino ? sched::kWinograd : sched::kClassic;

  Prepared pr;
  int rc = prepare_gemm(g, 3, &pr);
  if (rc) return rc;
  if (!pr.kp.tma_store) return B200S_ERR_BAD_ALIGNMENT;

  const size_t es = dtype_size(g.in_dtype);
  const int vec = static_cast<int>(16 / es);
  if (f.a_cols_blk % vec || f.b_cols_blk % vec || f.Nb % vec) return B200S_ERR_BAD_SHAPE;
  if ((f.lda * es) % 16 || (f.ldb * es) % 16) return B200S_ERR_BAD_STRIDE;
  if ((reinterpret_cast<uintptr_t>(f.A) & 15u) || (reinterpret_cast<uintptr_t>(f.B) & 15u))
    return B200S_ERR_BAD_ALIGNMENT;

  FusedKernelParams fz = {};
  int pos[7];
  for (int i = 0; i < 7; ++i) pos[f.order[i]] = i;
  for (int side = 0; side < 2; ++side) {
    pre::PreaddOuterParams& pp = fz.pre[side];
    pp.X = side == 0 ? f.A : f.B;
    pp.out = const_cast<void*>(side == 0 ? g.A : g.B);
    pp.rows_blk = side == 0 ? f.a_rows_blk : f.b_rows_blk;
    pp.cols_vec = (side == 0 ? f.a_cols_blk : f.b_cols_blk) / vec;
    pp.ld = side == 0 ? f.lda : f.ldb;
    pp.strideX = 0;
    pp.out_batch_blocks = 7 * np2;
    pp.transposed = side == 0 ? f.a_transposed : f.b_transposed;
    for (int i = 0; i < 7; ++i) {
      pre::set_outer_terms(pp, i, sa, side, f.order[i]);
      pp.out_block0[i] = i * np2;
    }
  }
  comb::CombineOuterParams& cp = fz.comb;
  cp.products = g.C;
  cp.C = f.C;
  cp.Mb = f.Mb;
  cp.nb_vec = f.Nb / vec;
  cp.ldc = f.ldc;
  cp.strideC = 0;
  cp.batch_blocks = 7 * np2;
  cp.out_dtype = f.out_dtype;
  cp.beta = f.beta;
  const size_t oes = dtype_size(f.out_dtype);
  cp.vec_ok = ((reinterpret_cast<uintptr_t>(f.C) & 15u) == 0) && ((f.ldc * oes) % 16 == 0) && ((f.Nb * oes) % 16 == 0);
  for (int e = 0; e < 4; ++e) {
    cp.quad[e] = static_cast<int8_t>(e);
    for (int p1 = 0; p1 < 7; ++p1) cp.coef[e][p1] = static_cast<int8_t>(sched::w1(sa, e, p1));
  }
  for (int p1 = 0; p1 < 7; ++p1) cp.group_block0[p1] = pos[p1] * np2;

  fz.flags = f.flags;
  fz.np2 = np2;
  fz.groups_formed = f.groups_formed;
  fz.b_formed = f.b_formed ? 1 : 0;
  fz.ready_target = f.b_formed ? 1u : 2u;  // adder teams per CTA (times the CTAs, in the kernel)
  fz.done_target = static_cast<uint32_t>(np2) * pr.kp.m_tiles * pr.kp.n_tiles * 2u * 8u;  // 2 CTAs x 8 epilogue warps per tile
  // The quadrants of C in the order in which the groups feeding them complete.
  int n = 0;
  for (int last = 0; last < 7; ++last) {
    for (int r = 0; r < 4; ++r) {
      if (!(f.quads_inside & (1 << r))) continue;
      int lp = 0;
      for (int p1 = 0; p1 < 7; ++p1)
        if (sched::w1(sa, r, p1) != 0 && pos[p1] > lp) lp = pos[p1];
      if (lp != last) continue;
      fz.comb_quad[n] = static_cast<int8_t>(r);
      fz.comb_wait[n] = static_cast<int8_t>(lp + 1);
      ++n;
    }
  }
  fz.n_comb = n;

  if (f.depth == 2)
    return wino ? launch_fused_dtype<1, sched::kWinograd>(pr, fz, g.in_dtype, stream)
                : launch_fused_dtype<1, sched::kClassic>(pr, fz, g.in_dtype, stream);
  return wino ? launch_fused_dtype<0, sched::kWinograd>(pr, fz, g.in_dtype, stream)
              : launch_fused_dtype<0, sched::kClassic>(pr, fz, g.in_dtype, stream);
}

}  // namespace b200s
