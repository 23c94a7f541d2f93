// C ABI of libb200s.so: argument validation, algorithm/depth resolution through the tuner
// table, workspace layout, and the launch sequence pre-add(A), pre-add(B), grouped GEMM,
// recombination. Nothing here touches host copies of the matrices; there is no CPU path.

#include <cuda_runtime.h>

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "common.h"
#include "schedule.h"

namespace b200s {

namespace {

thread_local char g_cuda_error[512] = "";
std::atomic<int64_t> g_launches{0};

// ---- stage timing (b200s_profile_begin / _end) ----------------------------------------------
// While collection is on, the sequential and the fused schedule of b200s_matmul record an event on
// the caller's stream at every stage boundary: start, after the operand blocks of A, after those of
// B, after the products (the fused kernel, in the fused schedule), after the recombination.
constexpr int kProfMarks = 5;
std::mutex g_prof_mu;
bool g_prof_on = false;
int g_prof_max = 0, g_prof_calls = 0;
std::vector<cudaEvent_t> g_prof_ev;

// Returns the slot of a new call (or -1 when collection is off or full).
int prof_new_call() {
  std::lock_guard<std::mutex> lock(g_prof_mu);
  if (!g_prof_on || g_prof_calls >= g_prof_max) return -1;
  return g_prof_calls++;
}
void prof_mark(int slot, int k, cudaStream_t stream) {
  if (slot < 0) return;
  cudaEventRecord(g_prof_ev[static_cast<size_t>(slot) * kProfMarks + k], stream);
}

struct DeviceState {
  bool ready = false;
  bool ok = false;
  int sms = 0;
  uint32_t* status = nullptr;
  // Pipelined driver: side streams and events, created on the first pipelined call.
  std::mutex pipe_mu;
  bool pipe_ready = false;
  cudaStream_t s_add = nullptr, s_gemm = nullptr;
  cudaEvent_t ev_start = nullptr, ev_end = nullptr, ev_pre[7] = {}, ev_done[7] = {};
};
std::mutex g_dev_mu;
DeviceState g_dev[64];

DeviceState* current_device_state() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_dev_mu);
  DeviceState& s = g_dev[dev];
  if (!s.ready) {
    s.ready = true;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return &s;
    if (prop.major != 10) return &s;  // tcgen05 / TMEM kernels: sm_100 only
    s.sms = prop.multiProcessorCount;
    // two status words, then (64 bytes on) the counters of the sending CTAs
    void* ptr = nullptr;
    const size_t bytes = 64 + sizeof(uint32_t) * kSendUnits;
    if (cudaMalloc(&ptr, bytes) != cudaSuccess) return &s;
    if (cudaMemset(ptr, 0, bytes) != cudaSuccess) return &s;
    s.status = static_cast<uint32_t*>(ptr);
    s.ok = true;
  }
  return &s;
}

// ---- tuner table ---------------------------------------------------------------------------
struct TunerEntry {
  int64_t M, N, K;
  int32_t in_dtype, algo, depth;
  int32_t fuse;  // schedule of a Strassen entry: 0 = built-in default, else the b200s_problem.fuse value
};
std::mutex g_tuner_mu;
std::vector<TunerEntry> g_tuner;

double log_volume(int64_t M, int64_t N, int64_t K) {
  return std::log2(static_cast<double>(M)) + std::log2(static_cast<double>(N)) + std::log2(static_cast<double>(K));
}

// Built-in choice when the table holds nothing for the dtype: a dense product below a cube of
// kDefaultCrossover, two Strassen levels from there on (measured on B200, bf16: up to 12288^3 the
// dense kernel wins, at 16384^3 and 32768^3 two levels win over one level and over dense).
constexpr int64_t kDefaultCrossover = 14336;

void default_choice(int64_t M, int64_t N, int64_t K, int32_t* algo, int32_t* depth) {
  const double v = log_volume(M, N, K);
  const double c1 = 3.0 * std::log2(static_cast<double>(kDefaultCrossover));
  if (v < c1) {
    *algo = B200S_ALGO_DENSE, *depth = 0;
  } else {
    *algo = B200S_ALGO_CLASSIC, *depth = 2;
  }
}

bool valid_dtype(int d) { return d == B200S_BF16 || d == B200S_FP16 || d == B200S_FP32; }

// Largest depth <= want for which every extent splits into 2^depth blocks whose contiguous
// runs are whole 16-byte vectors.
// Levels beyond two run as host-side recursion: one outer level of pre-addition and recombination
// around seven products of one level less (see run_deep).
constexpr int kMaxDepth = 4;

int feasible_depth(const b200s_problem& p, int want) {
  int d = want;
  while (d > 0) {
    const int64_t q = (int64_t{1} << d) * 8;
    if (p.M % q == 0 && p.N % q == 0 && p.K % q == 0) break;
    --d;
  }
  return d;
}

struct Plan {
  int algo, depth, prod_dtype;
  int table_fuse;           // schedule the tuner table holds for this shape (0 = none recorded)
  int64_t np;               // 7^depth
  int64_t Mb, Nb, Kb;       // block extents
  size_t sa_bytes, sb_bytes, mp_bytes;
  size_t ta_bytes, tb_bytes;  // K-major copies of fp32 operands given MN-major
  size_t a3_bytes, b3_bytes;  // hi/lo split operands of the three-pass TF32 mode
  size_t deep_bytes;          // scratch of the recursion for more than two levels
  size_t flag_bytes;          // counters the CTAs of the fused kernel share (last bytes of the scratch)
  bool split3;
  size_t total_bytes;
};

constexpr size_t kFlagBytes = 256;

size_t round256(size_t x) { return (x + 255) & ~size_t{255}; }

int make_plan(const b200s_problem* p, Plan* plan) {
  if (!p) return B200S_ERR_NULL_POINTER;
  if (p->M <= 0 || p->N <= 0 || p->K <= 0 || p->batch <= 0) return B200S_ERR_BAD_SHAPE;
  if (!valid_dtype(p->in_dtype) || !valid_dtype(p->out_dtype)) return B200S_ERR_BAD_DTYPE;
  if (p->a_major != B200S_K_MAJOR && p->a_major != B200S_MN_MAJOR) return B200S_ERR_BAD_STRIDE;
  if (p->b_major != B200S_K_MAJOR && p->b_major != B200S_MN_MAJOR) return B200S_ERR_BAD_STRIDE;
  if (p->algo < B200S_ALGO_AUTO || p->algo > B200S_ALGO_WINOGRAD) return B200S_ERR_BAD_ALGO;
  if (p->depth < -1 || p->depth > kMaxDepth) return B200S_ERR_BAD_DEPTH;
  if (p->beta != 0 && p->beta != 1) return B200S_ERR_BAD_SHAPE;
  if (p->pipeline < 0 || p->pipeline > 2) return B200S_ERR_BAD_SHAPE;
  if (p->fuse < 0 || p->fuse > 3) return B200S_ERR_BAD_SHAPE;
  if (p->precision != B200S_PREC_TF32 && p->precision != B200S_PREC_3XTF32) return B200S_ERR_BAD_DTYPE;
  if (p->b_blocks_ready != 0 && p->b_blocks_ready != 1) return B200S_ERR_BAD_SHAPE;
  const int64_t a_cols = p->a_major == B200S_K_MAJOR ? p->K : p->M;
  const int64_t b_cols = p->b_major == B200S_K_MAJOR ? p->K : p->N;
  if (p->lda < a_cols || p->ldb < b_cols || p->ldc < p->N) return B200S_ERR_BAD_STRIDE;

  int32_t algo = p->algo, depth = p->depth;
  {
    int32_t ta, td, tf = 0;
    b200s_tuner_lookup_schedule(p->M, p->N, p->K, p->in_dtype, &ta, &td, &tf);
    plan->table_fuse = tf;
  }
  if (algo == B200S_ALGO_AUTO || depth < 0) {
    int32_t ta, td;
    b200s_tuner_lookup(p->M, p->N, p->K, p->in_dtype, &ta, &td);
    if (algo == B200S_ALGO_AUTO) {
      algo = ta;
      if (depth < 0) depth = td;
    } else if (depth < 0) {
      depth = (algo == B200S_ALGO_DENSE) ? 0 : (td > 0 ? td : 1);
    }
    if (algo == B200S_ALGO_DENSE) depth = 0;
    if (algo != B200S_ALGO_DENSE && depth == 0) algo = B200S_ALGO_DENSE;
  }
  if (algo == B200S_ALGO_DENSE) depth = 0;
  if (algo != B200S_ALGO_DENSE) {
    if (p->algo != B200S_ALGO_AUTO && p->depth > 0) {
      // An explicit request must be met exactly.
      if (feasible_depth(*p, depth) != depth) return B200S_ERR_BAD_SHAPE;
    } else {
      depth = feasible_depth(*p, depth);
    }
    if (depth == 0) algo = B200S_ALGO_DENSE;
  }

  plan->algo = algo;
  plan->depth = depth;
  int pd = p->prod_dtype < 0 ? p->in_dtype : p->prod_dtype;
  if (!valid_dtype(pd)) return B200S_ERR_BAD_DTYPE;
  if (p->in_dtype == B200S_FP32) pd = B200S_FP32;
  plan->prod_dtype = pd;
  plan->np = sched::ipow(7, depth);
  const int64_t div = int64_t{1} << depth;
  plan->Mb = p->M / div;
  plan->Nb = p->N / div;
  plan->Kb = p->K / div;
  plan->ta_bytes = plan->tb_bytes = 0;
  if (p->in_dtype == B200S_FP32) {
    const size_t b = static_cast<size_t>(p->batch);
    if (p->a_major == B200S_MN_MAJOR) plan->ta_bytes = round256(b * p->M * p->K * 4);
    if (p->b_major == B200S_MN_MAJOR) plan->tb_bytes = round256(b * p->K * p->N * 4);
  }
  plan->a3_bytes = plan->b3_bytes = 0;
  plan->split3 = p->in_dtype == B200S_FP32 && p->precision == B200S_PREC_3XTF32;
  if (plan->split3) {
    if (p->K % 4) return B200S_ERR_BAD_SHAPE;
    const size_t nb3 = static_cast<size_t>(p->batch) * static_cast<size_t>(plan->np);
    plan->a3_bytes = round256(nb3 * plan->Mb * plan->Kb * 3 * 4);
    plan->b3_bytes = round256(nb3 * plan->Nb * plan->Kb * 3 * 4);
  }
  plan->deep_bytes = 0;
  plan->flag_bytes = 0;
  if (depth > 2) {
    if (p->batch != 1) return B200S_ERR_BAD_SHAPE;
    // scratch of every outer level (7 operand blocks of each side, 7 products) plus the scratch of
    // one two-level product of the innermost extents, reused by all sub-products in turn
    const size_t es3 = dtype_size(p->in_dtype), ps3 = dtype_size(pd);
    size_t total = 0;
    int64_t m = p->M, n = p->N, k = p->K;
    for (int d = depth; d > 2; --d) {
      m /= 2, n /= 2, k /= 2;
      total += round256(7 * m * k * es3) + round256(7 * k * n * es3) + round256(7 * m * n * ps3);
    }
    b200s_problem inner = *p;
    inner.M = m, inner.N = n, inner.K = k;
    inner.a_major = inner.b_major = B200S_K_MAJOR;  // extents only matter here
    inner.lda = k, inner.ldb = k, inner.ldc = n;
    if (p->in_dtype != B200S_FP32) {
      inner.a_major = p->a_major, inner.b_major = p->b_major;
      inner.lda = p->a_major == B200S_K_MAJOR ? k : m;
      inner.ldb = p->b_major == B200S_K_MAJOR ? k : n;
    }
    inner.algo = algo, inner.depth = 2, inner.out_dtype = pd, inner.beta = 0;
    Plan ip;
    int rc = make_plan(&inner, &ip);
    if (rc) return rc;
    plan->deep_bytes = total + ip.total_bytes;
    plan->a3_bytes = plan->b3_bytes = 0;
    plan->sa_bytes = plan->sb_bytes = plan->mp_bytes = 0;
    plan->total_bytes = plan->ta_bytes + plan->tb_bytes + plan->deep_bytes;
    return B200S_OK;
  }
  if (depth == 0) {
    plan->sa_bytes = plan->sb_bytes = plan->mp_bytes = 0;
    plan->total_bytes = plan->ta_bytes + plan->tb_bytes + plan->a3_bytes + plan->b3_bytes;
    return B200S_OK;
  }
  const size_t es = dtype_size(p->in_dtype), ps = dtype_size(pd);
  const size_t nb = static_cast<size_t>(p->batch) * static_cast<size_t>(plan->np);
  plan->sa_bytes = round256(nb * plan->Mb * plan->Kb * es);
  plan->sb_bytes = round256(nb * plan->Kb * plan->Nb * es);
  plan->mp_bytes = round256(nb * plan->Mb * plan->Nb * ps);
  plan->flag_bytes = kFlagBytes;
  plan->total_bytes = plan->sa_bytes + plan->sb_bytes + plan->mp_bytes + plan->ta_bytes + plan->tb_bytes +
                      plan->a3_bytes + plan->b3_bytes + plan->flag_bytes;
  return B200S_OK;
}

// Order in which the outer products are formed and multiplied, chosen so that the outer quadrants
// of C complete one after another (classic: C11 after 4 groups, then C12, C21, C22).
const int kOrderClassic[7] = {0, 3, 4, 6, 2, 1, 5};
const int kOrderWinograd[7] = {0, 1, 4, 5, 2, 6, 3};

int ensure_pipe(DeviceState* ds) {
  if (ds->pipe_ready) return B200S_OK;
  int lo = 0, hi = 0;
  B200S_CUDA_OK(cudaDeviceGetStreamPriorityRange(&lo, &hi));
  B200S_CUDA_OK(cudaStreamCreateWithPriority(&ds->s_gemm, cudaStreamNonBlocking, hi));
  B200S_CUDA_OK(cudaStreamCreateWithPriority(&ds->s_add, cudaStreamNonBlocking, lo));
  B200S_CUDA_OK(cudaEventCreateWithFlags(&ds->ev_start, cudaEventDisableTiming));
  B200S_CUDA_OK(cudaEventCreateWithFlags(&ds->ev_end, cudaEventDisableTiming));
  for (int i = 0; i < 7; ++i) {
    B200S_CUDA_OK(cudaEventCreateWithFlags(&ds->ev_pre[i], cudaEventDisableTiming));
    B200S_CUDA_OK(cudaEventCreateWithFlags(&ds->ev_done[i], cudaEventDisableTiming));
  }
  ds->pipe_ready = true;
  return B200S_OK;
}

// Strassen with the outer level software-pipelined over three streams: the bandwidth-bound
// operand sums of group i+1.. and the recombination of finished quadrants run beside the
// tensor-core-bound products of group i. Scratch blocks are laid out in processing order.
int run_pipelined(const b200s_problem* p, const Plan& plan, const void* A, const void* B, void* C, void* Sa, void* Sb,
                  void* Mp, cudaStream_t user) {
  DeviceState* ds = current_device_state();
  if (!ds || !ds->ok) return B200S_ERR_NO_DEVICE;
  std::lock_guard<std::mutex> lock(ds->pipe_mu);
  int rc = ensure_pipe(ds);
  if (rc) return rc;
  const bool wino = plan.algo == B200S_ALGO_WINOGRAD;
  const int* order = wino ? kOrderWinograd : kOrderClassic;
  const int sa = wino ? sched::kWinograd : sched::kClassic;
  const int np2 = static_cast<int>(plan.np / 7);  // products per outer group
  int pos[7];
  for (int i = 0; i < 7; ++i) pos[order[i]] = i;
  const size_t es = dtype_size(p->in_dtype), ps = dtype_size(plan.prod_dtype);
  const bool a_k = p->a_major == B200S_K_MAJOR, b_k = p->b_major == B200S_K_MAJOR;

  B200S_CUDA_OK(cudaEventRecord(ds->ev_start, user));
  B200S_CUDA_OK(cudaStreamWaitEvent(ds->s_add, ds->ev_start, 0));
  B200S_CUDA_OK(cudaStreamWaitEvent(ds->s_gemm, ds->ev_start, 0));

  for (int i = 0; i < 7; ++i) {
    PreaddOuterArgs pa;
    pa.batch = 1;
    pa.algo = plan.algo, pa.depth = plan.depth, pa.dtype = p->in_dtype;
    pa.n_groups = 1;
    pa.groups[0] = order[i];
    pa.out_block0[0] = i * np2;
    pa.X = A, pa.out = Sa, pa.side = 0;
    pa.rows_blk = a_k ? plan.Mb : plan.Kb, pa.cols_blk = a_k ? plan.Kb : plan.Mb;
    pa.ld = p->lda, pa.strideX = 0, pa.transposed = !a_k;
    rc = launch_preadd_outer(pa, ds->s_add);
    if (rc) return rc;
    if (!p->b_blocks_ready) {
      pa.X = B, pa.out = Sb, pa.side = 1;
      pa.rows_blk = b_k ? plan.Nb : plan.Kb, pa.cols_blk = b_k ? plan.Kb : plan.Nb;
      pa.ld = p->ldb, pa.transposed = b_k;
      rc = launch_preadd_outer(pa, ds->s_add);
      if (rc) return rc;
    }
    B200S_CUDA_OK(cudaEventRecord(ds->ev_pre[i], ds->s_add));
  }

  int last_pos[4];
  for (int r = 0; r < 4; ++r) {
    last_pos[r] = 0;
    for (int p1 = 0; p1 < 7; ++p1)
      if (sched::w1(sa, r, p1) != 0 && pos[p1] > last_pos[r]) last_pos[r] = pos[p1];
  }

  for (int i = 0; i < 7; ++i) {
    B200S_CUDA_OK(cudaStreamWaitEvent(ds->s_gemm, ds->ev_pre[i], 0));
    GemmArgs g;
    g.cta_group = p->tile_variant;
    g.in_dtype = p->in_dtype, g.a_major = p->a_major, g.b_major = p->b_major;
    g.A = static_cast<const uint8_t*>(Sa) + static_cast<size_t>(i) * np2 * plan.Mb * plan.Kb * es;
    g.B = static_cast<const uint8_t*>(Sb) + static_cast<size_t>(i) * np2 * plan.Kb * plan.Nb * es;
    g.C = static_cast<uint8_t*>(Mp) + static_cast<size_t>(i) * np2 * plan.Mb * plan.Nb * ps;
    g.M = plan.Mb, g.N = plan.Nb, g.K = plan.Kb, g.batch = np2;
    g.lda = a_k ? plan.Kb : plan.Mb, g.ldb = b_k ? plan.Kb : plan.Nb, g.ldc = plan.Nb;
    g.strideA = plan.Mb * plan.Kb, g.strideB = plan.Kb * plan.Nb, g.strideC = plan.Mb * plan.Nb;
    g.out_dtype = plan.prod_dtype, g.beta = 0;
    rc = launch_gemm(g, ds->s_gemm);
    if (rc) return rc;
    B200S_CUDA_OK(cudaEventRecord(ds->ev_done[i], ds->s_gemm));

    CombineOuterArgs ca;
    ca.n_quads = 0;
    for (int r = 0; r < 4; ++r)
      if (last_pos[r] == i) ca.quads[ca.n_quads++] = r;
    if (ca.n_quads == 0) continue;
    ca.products = Mp, ca.C = C;
    ca.Mb = plan.Mb, ca.Nb = plan.Nb, ca.ldc = p->ldc, ca.batch = 1, ca.strideC = 0;
    ca.algo = plan.algo, ca.depth = plan.depth, ca.prod_dtype = plan.prod_dtype, ca.out_dtype = p->out_dtype;
    ca.beta = p->beta;
    for (int p1 = 0; p1 < 7; ++p1) ca.group_block0[p1] = pos[p1] * np2;
    // the products stream is in order, so this event also covers every earlier group
    B200S_CUDA_OK(cudaStreamWaitEvent(ds->s_add, ds->ev_done[i], 0));
    rc = launch_combine_outer(ca, ds->s_add);
    if (rc) return rc;
  }
  B200S_CUDA_OK(cudaEventRecord(ds->ev_end, ds->s_add));
  B200S_CUDA_OK(cudaStreamWaitEvent(user, ds->ev_end, 0));
  return B200S_OK;
}

// Can the fused kernel carry this product? One product (no batch), one or two levels, 16-bit operands
// with the products stored in the same type, 256 x 512 tiles, blocks small enough for 32-bit positions.
bool fused_eligible(const b200s_problem* p, const Plan& plan) {
  if (p->batch != 1 || plan.depth < 1 || plan.depth > 2 || plan.split3) return false;
  if (p->in_dtype != B200S_BF16 && p->in_dtype != B200S_FP16) return false;
  if (plan.prod_dtype != p->in_dtype) return false;
  if (p->tile_variant != 0 && p->tile_variant != 3) return false;
  const int64_t lim = int64_t{1} << 31;
  return plan.Mb * plan.Kb / 8 < lim && plan.Kb * plan.Nb / 8 < lim && plan.Mb * plan.Nb / 8 < lim;
}

// Strassen as one persistent launch (launch_fused): the operand blocks of the first outer group are
// formed by the stand-alone pass, then the fused kernel multiplies all groups while its adder warps
// form the later groups' blocks and recombine every quadrant of C whose groups are done. With
// tail_outside the quadrant(s) that need the last group are left to a full-width recombination
// launch after the kernel instead of to the adder warps.
int run_fused(const b200s_problem* p, const Plan& plan, const void* A, const void* B, void* C, void* Sa, void* Sb,
              void* Mp, uint32_t* flags, bool tail_outside, cudaStream_t stream) {
  const bool wino = plan.algo == B200S_ALGO_WINOGRAD;
  const int* order = wino ? kOrderWinograd : kOrderClassic;
  const int sa = wino ? sched::kWinograd : sched::kClassic;
  const int np2 = static_cast<int>(plan.np / 7);
  int pos[7];
  for (int i = 0; i < 7; ++i) pos[order[i]] = i;
  const bool a_k = p->a_major == B200S_K_MAJOR, b_k = p->b_major == B200S_K_MAJOR;
  const int prof = prof_new_call();
  prof_mark(prof, 0, stream);

  B200S_CUDA_OK(cudaMemsetAsync(flags, 0, 64, stream));

  PreaddOuterArgs pa;
  pa.batch = 1, pa.strideX = 0;
  pa.algo = plan.algo, pa.depth = plan.depth, pa.dtype = p->in_dtype;
  pa.n_groups = 1;
  pa.groups[0] = order[0];
  pa.out_block0[0] = 0;
  pa.X = A, pa.out = Sa, pa.side = 0;
  pa.rows_blk = a_k ? plan.Mb : plan.Kb, pa.cols_blk = a_k ? plan.Kb : plan.Mb;
  pa.ld = p->lda, pa.transposed = !a_k;
  int rc = launch_preadd_outer(pa, stream);
  if (rc) return rc;
  prof_mark(prof, 1, stream);
  PreaddOuterArgs pb = pa;
  pb.X = B, pb.out = Sb, pb.side = 1;
  pb.rows_blk = b_k ? plan.Nb : plan.Kb, pb.cols_blk = b_k ? plan.Kb : plan.Nb;
  pb.ld = p->ldb, pb.transposed = b_k;
  if (!p->b_blocks_ready) {
    rc = launch_preadd_outer(pb, stream);
    if (rc) return rc;
  }
  prof_mark(prof, 2, stream);
  int last_pos[4], tail_mask = 0;
  for (int r = 0; r < 4; ++r) {
    last_pos[r] = 0;
    for (int p1 = 0; p1 < 7; ++p1)
      if (sched::w1(sa, r, p1) != 0 && pos[p1] > last_pos[r]) last_pos[r] = pos[p1];
    if (tail_outside && last_pos[r] == 6) tail_mask |= 1 << r;
  }

  FusedArgs f;
  GemmArgs& g = f.gemm;
  g.cta_group = 3;
  g.in_dtype = p->in_dtype, g.a_major = p->a_major, g.b_major = p->b_major;
  g.A = Sa, g.B = Sb, g.C = Mp;
  g.M = plan.Mb, g.N = plan.Nb, g.K = plan.Kb, g.batch = plan.np;
  g.lda = a_k ? plan.Kb : plan.Mb, g.ldb = b_k ? plan.Kb : plan.Nb, g.ldc = plan.Nb;
  g.strideA = plan.Mb * plan.Kb, g.strideB = plan.Kb * plan.Nb, g.strideC = plan.Mb * plan.Nb;
  g.out_dtype = plan.prod_dtype, g.beta = 0;
  f.algo = plan.algo, f.depth = plan.depth;
  f.A = A, f.B = B, f.lda = p->lda, f.ldb = p->ldb;
  f.a_rows_blk = pa.rows_blk, f.a_cols_blk = pa.cols_blk, f.a_transposed = pa.transposed;
  f.b_rows_blk = pb.rows_blk, f.b_cols_blk = pb.cols_blk, f.b_transposed = pb.transposed;
  f.C = C, f.Mb = plan.Mb, f.Nb = plan.Nb, f.ldc = p->ldc, f.out_dtype = p->out_dtype, f.beta = p->beta;
  for (int i = 0; i < 7; ++i) f.order[i] = order[i];
  f.groups_formed = 1;
  f.b_formed = p->b_blocks_ready ? 1 : 0;
  f.quads_inside = 0xf & ~tail_mask;
  f.flags = flags;
  rc = launch_fused(f, stream);
  if (rc) return rc;
  prof_mark(prof, 3, stream);

  if (tail_mask) {
    CombineOuterArgs ca;
    ca.n_quads = 0;
    for (int r = 0; r < 4; ++r)
      if (tail_mask & (1 << r)) ca.quads[ca.n_quads++] = r;
    ca.products = Mp, ca.C = C;
    ca.Mb = plan.Mb, ca.Nb = plan.Nb, ca.ldc = p->ldc, ca.batch = 1, ca.strideC = 0;
    ca.algo = plan.algo, ca.depth = plan.depth, ca.prod_dtype = plan.prod_dtype, ca.out_dtype = p->out_dtype;
    ca.beta = p->beta;
    for (int p1 = 0; p1 < 7; ++p1) ca.group_block0[p1] = pos[p1] * np2;
    rc = launch_combine_outer(ca, stream);
    if (rc) return rc;
  }
  prof_mark(prof, 4, stream);
  return B200S_OK;
}

// More than two levels: one outer level here (operand sums rounded to the operand dtype, as the
// reference's recursion rounds S1..S10 at every level, fixed_strassen_fp32_agg.py:87-96), seven
// products of one level less through b200s_matmul, one outer recombination in fp32.
int run_deep(const b200s_problem* p, const Plan& plan, const void* A, const void* B, void* C, uint8_t* ws,
             cudaStream_t stream) {
  const size_t es = dtype_size(p->in_dtype), ps = dtype_size(plan.prod_dtype);
  const int64_t Mb = p->M / 2, Nb = p->N / 2, Kb = p->K / 2;
  const bool a_k = p->a_major == B200S_K_MAJOR, b_k = p->b_major == B200S_K_MAJOR;
  uint8_t* Sa = ws;
  uint8_t* Sb = Sa + round256(7 * Mb * Kb * es);
  uint8_t* Mp = Sb + round256(7 * Kb * Nb * es);
  uint8_t* inner = Mp + round256(7 * Mb * Nb * ps);

  PreaddArgs pa;
  pa.batch = 1, pa.strideX = 0, pa.algo = plan.algo, pa.depth = 1, pa.dtype = p->in_dtype;
  pa.X = A, pa.out = Sa, pa.side = 0;
  pa.rows_blk = a_k ? Mb : Kb, pa.cols_blk = a_k ? Kb : Mb, pa.ld = p->lda, pa.transposed = !a_k;
  int rc = launch_preadd(pa, stream);
  if (rc) return rc;
  pa.X = B, pa.out = Sb, pa.side = 1;
  pa.rows_blk = b_k ? Nb : Kb, pa.cols_blk = b_k ? Kb : Nb, pa.ld = p->ldb, pa.transposed = b_k;
  rc = launch_preadd(pa, stream);
  if (rc) return rc;

  b200s_problem q = *p;
  q.M = Mb, q.N = Nb, q.K = Kb, q.batch = 1;
  q.lda = a_k ? Kb : Mb, q.ldb = b_k ? Kb : Nb, q.ldc = Nb;
  q.strideA = q.strideB = q.strideC = 0;
  q.algo = plan.algo, q.depth = plan.depth - 1;
  q.out_dtype = plan.prod_dtype, q.beta = 0, q.pipeline = 2, q.b_blocks_ready = 0;
  size_t need = 0;
  rc = b200s_workspace_bytes(&q, &need);
  if (rc) return rc;
  for (int i = 0; i < 7; ++i) {
    rc = b200s_matmul(&q, Sa + static_cast<size_t>(i) * Mb * Kb * es, Sb + static_cast<size_t>(i) * Kb * Nb * es,
                      Mp + static_cast<size_t>(i) * Mb * Nb * ps, inner, need, stream);
    if (rc) return rc;
  }
  CombineArgs c;
  c.products = Mp, c.C = C;
  c.Mb = Mb, c.Nb = Nb, c.ldc = p->ldc, c.batch = 1, c.strideC = 0;
  c.algo = plan.algo, c.depth = 1, c.prod_dtype = plan.prod_dtype, c.out_dtype = p->out_dtype, c.beta = p->beta;
  return launch_combine(c, stream);
}

}  // namespace

void note_cuda_error(cudaError_t e, const char* where) {
  std::snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s (%s)", where, cudaGetErrorName(e),
                cudaGetErrorString(e));
}
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
uint32_t* device_status_words() {
  DeviceState* s = current_device_state();
  return (s && s->ok) ? s->status : nullptr;
}
int sm_count() {
  DeviceState* s = current_device_state();
  return (s && s->ok) ? s->sms : 0;
}

uint32_t* device_send_counters() {
  DeviceState* s = current_device_state();
  return (s && s->ok) ? s->status + 16 : nullptr;
}

static std::atomic<int> g_sender_sms{0};    // 0 = the exchange stays in the epilogue
int sender_sm_count() { return g_sender_sms.load(std::memory_order_relaxed); }

static std::atomic<int> g_product_sms{0};   // 0 = no limit
int product_sm_count() {
  const int all = sm_count();
  const int lim = g_product_sms.load(std::memory_order_relaxed);
  return (lim > 0 && lim < all) ? lim : all;
}

}  // namespace b200s

using namespace b200s;

extern "C" {

int b200s_version(void) { return 100; }

const char* b200s_status_string(int status) {
  switch (status) {
    case B200S_OK: return "ok";
    case B200S_ERR_NULL_POINTER: return "null pointer argument";
    case B200S_ERR_BAD_SHAPE: return "bad shape: non-positive extent, or extents not divisible as the requested depth needs";
    case B200S_ERR_BAD_STRIDE: return "bad stride or major: leading dimension too small or not a multiple of 16 bytes";
    case B200S_ERR_BAD_ALIGNMENT: return "base pointer not 16-byte aligned";
    case B200S_ERR_BAD_DTYPE: return "unsupported dtype";
    case B200S_ERR_BAD_ALGO: return "unknown algorithm";
    case B200S_ERR_BAD_DEPTH: return "depth out of range (0..4, or -1 for the tuner table)";
    case B200S_ERR_WORKSPACE_TOO_SMALL: return "workspace too small";
    case B200S_ERR_CUDA: return "CUDA call failed";
    case B200S_ERR_NO_DEVICE: return "current device is not an sm_100 GPU";
    case B200S_ERR_DEVICE_TIMEOUT: return "a kernel gave up on a bounded wait";
    case B200S_ERR_TUNER_IO: return "tuner table file could not be read or written";
    case B200S_ERR_TOO_LARGE: return "problem exceeds the fixed capacity of this entry point";
  }
  return "unknown status";
}

const char* b200s_last_cuda_error(void) { return g_cuda_error; }

int64_t b200s_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int b200s_resolve(const b200s_problem* p, int32_t* algo_out, int32_t* depth_out) {
  if (!p || !algo_out || !depth_out) return B200S_ERR_NULL_POINTER;
  Plan plan;
  int rc = make_plan(p, &plan);
  if (rc) return rc;
  *algo_out = plan.algo;
  *depth_out = plan.depth;
  return B200S_OK;
}

int b200s_workspace_bytes(const b200s_problem* p, size_t* bytes_out) {
  if (!p || !bytes_out) return B200S_ERR_NULL_POINTER;
  Plan plan;
  int rc = make_plan(p, &plan);
  if (rc) return rc;
  *bytes_out = plan.total_bytes;
  return B200S_OK;
}

int b200s_preadd(const b200s_problem* p, int side, const void* X, void* out, void* stream) {
  if (!p || !X || !out) return B200S_ERR_NULL_POINTER;
  if (side != 0 && side != 1) return B200S_ERR_BAD_SHAPE;
  Plan plan;
  int rc = make_plan(p, &plan);
  if (rc) return rc;
  if (plan.depth == 0) return B200S_ERR_BAD_DEPTH;
  PreaddArgs a;
  a.X = X;
  a.out = out;
  a.batch = p->batch;
  a.side = side;
  a.algo = plan.algo;
  a.depth = plan.depth;
  a.dtype = p->in_dtype;
  if (side == 0) {
    const bool kmaj = p->a_major == B200S_K_MAJOR;
    a.rows_blk = kmaj ? plan.Mb : plan.Kb;
    a.cols_blk = kmaj ? plan.Kb : plan.Mb;
    a.ld = p->lda;
    a.strideX = p->strideA;
    a.transposed = !kmaj;
  } else {
    const bool kmaj = p->b_major == B200S_K_MAJOR;
    a.rows_blk = kmaj ? plan.Nb : plan.Kb;
    a.cols_blk = kmaj ? plan.Kb : plan.Nb;
    a.ld = p->ldb;
    a.strideX = p->strideB;
    a.transposed = kmaj;
  }
  if (!device_status_words()) return B200S_ERR_NO_DEVICE;
  return launch_preadd(a, static_cast<cudaStream_t>(stream));
}

static int combine_with_bias(const b200s_problem* p, const void* products, void* C, const void* bias, void* stream);

int b200s_combine(const b200s_problem* p, const void* products, void* C, void* stream) {
  return combine_with_bias(p, products, C, nullptr, stream);
}

static int combine_with_bias(const b200s_problem* p, const void* products, void* C, const void* bias, void* stream) {
  if (!p || !products || !C) return B200S_ERR_NULL_POINTER;
  Plan plan;
  int rc = make_plan(p, &plan);
  if (rc) return rc;
  if (plan.depth == 0) return B200S_ERR_BAD_DEPTH;
  CombineArgs c;
  c.products = products;
  c.C = C;
  c.Mb = plan.Mb;
  c.Nb = plan.Nb;
  c.ldc = p->ldc;
  c.batch = p->batch;
  c.strideC = p->strideC;
  c.algo = plan.algo;
  c.depth = plan.depth;
  c.prod_dtype = plan.prod_dtype;
  c.out_dtype = p->out_dtype;
  c.beta = p->beta;
  c.bias = bias;
  if (!device_status_words()) return B200S_ERR_NO_DEVICE;
  return launch_combine(c, static_cast<cudaStream_t>(stream));
}

int b200s_combine_peers(const b200s_problem* p, const void* products, void* const* C_list, int n_dst, void* stream) {
  if (!p || !products || !C_list) return B200S_ERR_NULL_POINTER;
  Plan plan;
  int rc = make_plan(p, &plan);
  if (rc) return rc;
  if (plan.depth == 0) return B200S_ERR_BAD_DEPTH;
  if (p->batch != 1 || p->beta != 0) return B200S_ERR_BAD_SHAPE;
  CombineArgs c;
  c.products = products, c.C = nullptr;
  c.Mb = plan.Mb, c.Nb = plan.Nb, c.ldc = p->ldc, c.batch = 1, c.strideC = 0;
  c.algo = plan.algo, c.depth = plan.depth, c.prod_dtype = plan.prod_dtype, c.out_dtype = p->out_dtype;
  c.beta = 0;
  if (!device_status_words()) return B200S_ERR_NO_DEVICE;
  return launch_combine_peers(c, C_list, n_dst, static_cast<cudaStream_t>(stream));
}

int b200s_set_product_sms(int n) {
  if (n < 0) return B200S_ERR_BAD_SHAPE;
  if (n == 1) n = 2;                         // a CTA pair needs two
  return g_product_sms.exchange(n & ~1, std::memory_order_relaxed);
}

int b200s_set_sender_sms(int n) {
  if (n < 0 || n > 64) return B200S_ERR_BAD_SHAPE;
  return g_sender_sms.exchange(n & ~1, std::memory_order_relaxed);
}

int b200s_push_panel(const void* src, void* const* dst_list, int n_dst, void* mc_dst, size_t bytes, int max_blocks,
                     void* stream) {
  return launch_push_panel(src, dst_list, n_dst, mc_dst, bytes, max_blocks, static_cast<cudaStream_t>(stream));
}

int b200s_push_rows(const void* src, void* const* dst_list, int n_dst, size_t bytes, void* stream) {
  if (!device_status_words()) return B200S_ERR_NO_DEVICE;
  return launch_push_rows(src, dst_list, n_dst, bytes, static_cast<cudaStream_t>(stream));
}

// C (+)= A . B into C, or (n_dst > 0, beta 0, one product) into every destination of dst_list.
static int run_matmul(const b200s_problem* p_in, const void* A, const void* B, void* C, void* const* dst_list,
                      int n_dst, void* workspace, size_t workspace_bytes, void* stream_v, void* mc_dst = nullptr,
                      const void* bias = nullptr) {
  if (!p_in || !A || !B || (!C && n_dst == 0)) return B200S_ERR_NULL_POINTER;
  Plan plan;
  int rc = make_plan(p_in, &plan);
  if (rc) return rc;
  b200s_problem local = *p_in;
  b200s_problem* p = &local;
  if (plan.total_bytes > 0) {
    if (!workspace) return B200S_ERR_NULL_POINTER;
    if (workspace_bytes < plan.total_bytes) return B200S_ERR_WORKSPACE_TOO_SMALL;
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return B200S_ERR_BAD_ALIGNMENT;
  }
  if (!device_status_words()) return B200S_ERR_NO_DEVICE;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

  uint8_t* ws = static_cast<uint8_t*>(workspace);
  if (plan.ta_bytes) {
    // fp32 A given K x M: rewrite it M x K
    void* At = ws + plan.sa_bytes + plan.sb_bytes + plan.mp_bytes;
    rc = launch_transpose_f32(A, At, p->K, p->M, p->lda, p->K, p->batch, p->strideA, p->M * p->K, stream);
    if (rc) return rc;
    A = At;
    p->a_major = B200S_K_MAJOR, p->lda = p->K, p->strideA = p->M * p->K;
  }
  const bool b_reused = p->b_blocks_ready && plan.depth > 0;
  if (plan.tb_bytes && b_reused) {
    p->b_major = B200S_K_MAJOR, p->ldb = p->K, p->strideB = p->K * p->N;  // blocks were formed from the K-major copy
  } else if (plan.tb_bytes) {
    // fp32 B given K x N: rewrite it N x K
    void* Bt = ws + plan.sa_bytes + plan.sb_bytes + plan.mp_bytes + plan.ta_bytes;
    rc = launch_transpose_f32(B, Bt, p->K, p->N, p->ldb, p->K, p->batch, p->strideB, p->K * p->N, stream);
    if (rc) return rc;
    B = Bt;
    p->b_major = B200S_K_MAJOR, p->ldb = p->K, p->strideB = p->K * p->N;
  }

  if (plan.depth > 2) {
    if (n_dst > 0 || bias) return B200S_ERR_BAD_DEPTH;  // several destinations or a bias: dense, or one pipeline of up to two levels
    return run_deep(p, plan, A, B, C, ws + plan.ta_bytes + plan.tb_bytes, stream);
  }

  GemmArgs g;
  g.cta_group = p->tile_variant;
  if (g.cta_group < 0 || g.cta_group > 3) return B200S_ERR_BAD_SHAPE;
  g.in_dtype = p->in_dtype;
  g.a_major = p->a_major;
  g.b_major = p->b_major;
  uint8_t* A3 = ws + plan.sa_bytes + plan.sb_bytes + plan.mp_bytes + plan.ta_bytes + plan.tb_bytes;
  uint8_t* B3 = A3 + plan.a3_bytes;
  if (plan.depth == 0) {
    g.A = A, g.B = B, g.C = C;
    g.n_dst = n_dst, g.C_list = dst_list, g.mc_dst = mc_dst, g.bias = bias;
    g.send_sms = (n_dst > 1 || mc_dst) ? sender_sm_count() : 0;
    g.M = p->M, g.N = p->N, g.K = p->K, g.batch = p->batch;
    g.lda = p->lda, g.ldb = p->ldb, g.ldc = p->ldc;
    g.strideA = p->strideA, g.strideB = p->strideB, g.strideC = p->strideC;
    g.out_dtype = p->out_dtype;
    g.beta = p->beta;
    if (plan.split3) {
      // both operands are K-major here; the product runs over the three K segments
      rc = launch_split3_f32(A, A3, p->M, p->K, p->lda, p->batch, p->strideA, 0, stream);
      if (rc) return rc;
      rc = launch_split3_f32(B, B3, p->N, p->K, p->ldb, p->batch, p->strideB, 1, stream);
      if (rc) return rc;
      g.A = A3, g.B = B3, g.K = 3 * p->K;
      g.lda = g.ldb = 3 * p->K;
      g.strideA = p->M * 3 * p->K, g.strideB = p->N * 3 * p->K;
    }
    const int prof = prof_new_call();
    for (int k = 0; k < 3; ++k) prof_mark(prof, k, stream);
    rc = launch_gemm(g, stream);
    for (int k = 3; k < kProfMarks; ++k) prof_mark(prof, k, stream);
    return rc;
  }

  void* Sa = ws;
  void* Sb = ws + plan.sa_bytes;
  void* Mp = ws + plan.sa_bytes + plan.sb_bytes;

  const double volume = static_cast<double>(p->M) * static_cast<double>(p->N) * static_cast<double>(p->K);
  int fuse = p->fuse;
  if (fuse == 0 && p->pipeline == 0) {
    // The caller left the schedule open: the tuner table's entry for this shape, else separate passes.
    // (Measured on B200: under the 1000 W power cap the fused kernel lowers the SM clock for the whole
    // product and costs more energy than it hides time, so it is nobody's default.)
    fuse = plan.table_fuse != 0 ? plan.table_fuse : 2;
  }
  if (n_dst == 0 && !bias && (fuse == 1 || fuse == 3)) {
    if (fused_eligible(p, plan)) {
      uint32_t* flags = reinterpret_cast<uint32_t*>(ws + plan.total_bytes - plan.flag_bytes);
      return run_fused(p, plan, A, B, C, Sa, Sb, Mp, flags, fuse == 3, stream);
    }
    if (p->fuse != 0) return B200S_ERR_BAD_SHAPE;  // an explicit request must be met
  }
  // Large single products run the pipelined driver unless the caller chose otherwise.
  const bool pipelined = p->pipeline == 1 || (p->pipeline == 0 && volume >= 24576.0 * 24576.0 * 24576.0);
  if (n_dst == 0 && !bias && p->batch == 1 && pipelined && !plan.split3) return run_pipelined(p, plan, A, B, C, Sa, Sb, Mp, stream);

  const int prof = prof_new_call();
  prof_mark(prof, 0, stream);
  rc = b200s_preadd(p, 0, A, Sa, stream_v);
  if (rc) return rc;
  prof_mark(prof, 1, stream);
  if (!p->b_blocks_ready) {
    rc = b200s_preadd(p, 1, B, Sb, stream_v);
    if (rc) return rc;
  }
  prof_mark(prof, 2, stream);

  const bool a_k = p->a_major == B200S_K_MAJOR, b_k = p->b_major == B200S_K_MAJOR;
  g.A = Sa, g.B = Sb, g.C = Mp;
  g.M = plan.Mb, g.N = plan.Nb, g.K = plan.Kb;
  g.batch = p->batch * plan.np;
  g.lda = a_k ? plan.Kb : plan.Mb;
  g.ldb = b_k ? plan.Kb : plan.Nb;
  g.ldc = plan.Nb;
  g.strideA = plan.Mb * plan.Kb;
  g.strideB = plan.Kb * plan.Nb;
  g.strideC = plan.Mb * plan.Nb;
  g.out_dtype = plan.prod_dtype;
  g.beta = 0;
  if (plan.split3) {
    // operand blocks are K-major fp32: split every block row into its three K segments
    const int64_t nblk = p->batch * plan.np;
    rc = launch_split3_f32(Sa, A3, nblk * plan.Mb, plan.Kb, plan.Kb, 1, 0, 0, stream);
    if (rc) return rc;
    if (!p->b_blocks_ready) {
      rc = launch_split3_f32(Sb, B3, nblk * plan.Nb, plan.Kb, plan.Kb, 1, 0, 1, stream);
      if (rc) return rc;
    }
    g.A = A3, g.B = B3, g.K = 3 * plan.Kb;
    g.lda = g.ldb = 3 * plan.Kb;
    g.strideA = plan.Mb * 3 * plan.Kb, g.strideB = plan.Nb * 3 * plan.Kb;
  }
  rc = launch_gemm(g, stream);
  if (rc) return rc;
  prof_mark(prof, 3, stream);

  if (n_dst > 0 && bias) return B200S_ERR_BAD_SHAPE;  // the multi-destination recombination carries no bias
  rc = n_dst > 0 ? b200s_combine_peers(p, Mp, dst_list, n_dst, stream_v) : combine_with_bias(p, Mp, C, bias, stream_v);
  prof_mark(prof, 4, stream);
  return rc;
}

int b200s_matmul(const b200s_problem* p, const void* A, const void* B, void* C, void* workspace,
                 size_t workspace_bytes, void* stream) {
  if (!C) return B200S_ERR_NULL_POINTER;
  return run_matmul(p, A, B, C, nullptr, 0, workspace, workspace_bytes, stream);
}

int b200s_matmul_bias(const b200s_problem* p, const void* A, const void* B, const void* bias, void* C, void* workspace,
                      size_t workspace_bytes, void* stream) {
  if (!C || !bias) return B200S_ERR_NULL_POINTER;
  if (p && p->out_dtype != B200S_FP32 && (reinterpret_cast<uintptr_t>(bias) & 1u)) return B200S_ERR_BAD_ALIGNMENT;
  return run_matmul(p, A, B, C, nullptr, 0, workspace, workspace_bytes, stream, nullptr, bias);
}

int b200s_matmul_peers(const b200s_problem* p, const void* A, const void* B, void* const* C_list, int n_dst,
                       void* workspace, size_t workspace_bytes, void* stream) {
  if (!p || !C_list) return B200S_ERR_NULL_POINTER;
  if (n_dst < 1 || n_dst > 8 || p->batch != 1 || p->beta != 0) return B200S_ERR_BAD_SHAPE;
  for (int d = 0; d < n_dst; ++d)
    if (!C_list[d]) return B200S_ERR_NULL_POINTER;
  return run_matmul(p, A, B, nullptr, C_list, n_dst, workspace, workspace_bytes, stream);
}

int b200s_matmul_multicast(const b200s_problem* p, const void* A, const void* B, void* C_local, void* C_multicast,
                           void* workspace, size_t workspace_bytes, void* stream) {
  if (!p || !C_local || !C_multicast) return B200S_ERR_NULL_POINTER;
  if (p->batch != 1 || p->beta != 0) return B200S_ERR_BAD_SHAPE;
  int32_t algo = 0, depth = 0;
  int rc = b200s_resolve(p, &algo, &depth);
  if (rc) return rc;
  if (depth != 0) return B200S_ERR_BAD_ALGO;  // the multicast store lives in the dense product's epilogue
  return run_matmul(p, A, B, C_local, nullptr, 0, workspace, workspace_bytes, stream, C_multicast);
}

int b200s_peer_barrier(void* const* pads, int rank, int world, uint32_t epoch, uint64_t limit_ns, void* stream) {
  return launch_peer_barrier(pads, rank, world, epoch, limit_ns, static_cast<cudaStream_t>(stream));
}

// ---- product with built-in scratch ---------------------------------------------------------------
//
// Scratch for b200s_matmul_static lives in the library image instead of in memory the caller
// allocates: a fixed array in device global memory, present on every GPU that loads the library for
// as long as the process lives. In host code the array's name stands for the symbol, not for a
// device address, so its address is asked from the runtime once per device (cudaGetSymbolAddress,
// with that device current) and only that pointer is handed to kernels.
constexpr size_t kStaticScratchBytes = size_t{64} << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static __device__ __align__(256) uint32_t g_static_status[2];  // zero at load; set only when a wait gives up

namespace {
struct StaticState {
  bool ready = false;
  void* scratch = nullptr;
  uint32_t* status = nullptr;
  int sms = 0;
};
std::mutex g_static_mu;
StaticState g_static[64];

// Set-up of the calling thread's current device: queries only, no allocation.
int static_state(StaticState** out) {
  int dev = -1;
  B200S_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return B200S_ERR_NO_DEVICE;
  std::lock_guard<std::mutex> lock(g_static_mu);
  StaticState& s = g_static[dev];
  if (!s.ready) {
    int major = 0, sms = 0;
    B200S_CUDA_OK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    B200S_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (major != 10) return B200S_ERR_NO_DEVICE;
    void* scratch = nullptr;
    void* status = nullptr;
    B200S_CUDA_OK(cudaGetSymbolAddress(&scratch, g_static_scratch));
    B200S_CUDA_OK(cudaGetSymbolAddress(&status, g_static_status));
    s.scratch = scratch;
    s.status = static_cast<uint32_t*>(status);
    s.sms = sms;
    s.ready = true;
  }
  *out = &s;
  return B200S_OK;
}
}  // namespace

int b200s_matmul_static(const b200s_problem* p_in, const void* A, const void* B, void* C, void* stream_v) {
  if (!p_in || !A || !B || !C) return B200S_ERR_NULL_POINTER;
  // fp32 operands run as one TF32 pass here; the three-pass mode needs more scratch than this entry has
  if (p_in->in_dtype == B200S_FP32 && p_in->precision == B200S_PREC_3XTF32) return B200S_ERR_BAD_DTYPE;
  Plan plan;
  int rc = make_plan(p_in, &plan);
  if (rc) return rc;
  if (plan.depth > 2) return B200S_ERR_BAD_DEPTH;  // the recursion for deeper levels is not offered here
  if (plan.total_bytes > kStaticScratchBytes) return B200S_ERR_TOO_LARGE;
  StaticState* st = nullptr;
  rc = static_state(&st);
  if (rc) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  b200s_problem local = *p_in;
  b200s_problem* p = &local;
  uint8_t* ws = static_cast<uint8_t*>(st->scratch);

  // Same sequence as the sequential schedule of b200s_matmul, every pass on the caller's stream.
  if (plan.ta_bytes) {
    void* At = ws + plan.sa_bytes + plan.sb_bytes + plan.mp_bytes;
    rc = launch_transpose_f32(A, At, p->K, p->M, p->lda, p->K, p->batch, p->strideA, p->M * p->K, stream);
    if (rc) return rc;
    A = At;
    p->a_major = B200S_K_MAJOR, p->lda = p->K, p->strideA = p->M * p->K;
  }
  if (plan.tb_bytes) {
    void* Bt = ws + plan.sa_bytes + plan.sb_bytes + plan.mp_bytes + plan.ta_bytes;
    rc = launch_transpose_f32(B, Bt, p->K, p->N, p->ldb, p->K, p->batch, p->strideB, p->K * p->N, stream);
    if (rc) return rc;
    B = Bt;
    p->b_major = B200S_K_MAJOR, p->ldb = p->K, p->strideB = p->K * p->N;
  }
  const bool a_k = p->a_major == B200S_K_MAJOR, b_k = p->b_major == B200S_K_MAJOR;

  GemmArgs g;
  g.status = st->status;
  g.sms = st->sms;
  g.cta_group = p->tile_variant;
  if (g.cta_group < 0 || g.cta_group > 3) return B200S_ERR_BAD_SHAPE;
  g.in_dtype = p->in_dtype, g.a_major = p->a_major, g.b_major = p->b_major;
  if (plan.depth == 0) {
    g.A = A, g.B = B, g.C = C;
    g.M = p->M, g.N = p->N, g.K = p->K, g.batch = p->batch;
    g.lda = p->lda, g.ldb = p->ldb, g.ldc = p->ldc;
    g.strideA = p->strideA, g.strideB = p->strideB, g.strideC = p->strideC;
    g.out_dtype = p->out_dtype, g.beta = p->beta;
    return launch_gemm(g, stream);
  }
  void* Sa = ws;
  void* Sb = ws + plan.sa_bytes;
  void* Mp = ws + plan.sa_bytes + plan.sb_bytes;

  PreaddArgs pa;
  pa.batch = p->batch, pa.algo = plan.algo, pa.depth = plan.depth, pa.dtype = p->in_dtype;
  pa.X = A, pa.out = Sa, pa.side = 0;
  pa.rows_blk = a_k ? plan.Mb : plan.Kb, pa.cols_blk = a_k ? plan.Kb : plan.Mb;
  pa.ld = p->lda, pa.strideX = p->strideA, pa.transposed = !a_k;
  rc = launch_preadd(pa, stream);
  if (rc) return rc;
  pa.X = B, pa.out = Sb, pa.side = 1;
  pa.rows_blk = b_k ? plan.Nb : plan.Kb, pa.cols_blk = b_k ? plan.Kb : plan.Nb;
  pa.ld = p->ldb, pa.strideX = p->strideB, pa.transposed = b_k;
  rc = launch_preadd(pa, stream);
  if (rc) return rc;

  g.A = Sa, g.B = Sb, g.C = Mp;
  g.M = plan.Mb, g.N = plan.Nb, g.K = plan.Kb, g.batch = p->batch * plan.np;
  g.lda = a_k ? plan.Kb : plan.Mb, g.ldb = b_k ? plan.Kb : plan.Nb, g.ldc = plan.Nb;
  g.strideA = plan.Mb * plan.Kb, g.strideB = plan.Kb * plan.Nb, g.strideC = plan.Mb * plan.Nb;
  g.out_dtype = plan.prod_dtype, g.beta = 0;
  rc = launch_gemm(g, stream);
  if (rc) return rc;

  CombineArgs c;
  c.products = Mp, c.C = C;
  c.Mb = plan.Mb, c.Nb = plan.Nb, c.ldc = p->ldc, c.batch = p->batch, c.strideC = p->strideC;
  c.algo = plan.algo, c.depth = plan.depth, c.prod_dtype = plan.prod_dtype, c.out_dtype = p->out_dtype;
  c.beta = p->beta;
  return launch_combine(c, stream);
}

int b200s_wait_probe(uint64_t limit_ns, void* stream) {
  if (limit_ns == 0 || limit_ns > 1000000000ull) return B200S_ERR_BAD_SHAPE;  // at most one second
  if (!device_status_words()) return B200S_ERR_NO_DEVICE;
  return launch_wait_probe(limit_ns, static_cast<cudaStream_t>(stream));
}

int b200s_static_status(void* stream, int32_t* status_out, int32_t* detail_out) {
  if (!status_out) return B200S_ERR_NULL_POINTER;
  StaticState* st = nullptr;
  int rc = static_state(&st);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint32_t host[2] = {0, 0};
  B200S_CUDA_OK(cudaMemcpyAsync(host, st->status, sizeof(host), cudaMemcpyDeviceToHost, s));
  B200S_CUDA_OK(cudaStreamSynchronize(s));
  if (host[0] != 0) {
    B200S_CUDA_OK(cudaMemsetAsync(st->status, 0, sizeof(host), s));
    B200S_CUDA_OK(cudaStreamSynchronize(s));
  }
  *status_out = host[0] ? B200S_ERR_DEVICE_TIMEOUT : B200S_OK;
  if (detail_out) *detail_out = static_cast<int32_t>(host[1]);
  return B200S_OK;
}

int b200s_device_status(void* stream, int32_t* status_out, int32_t* detail_out) {
  if (!status_out) return B200S_ERR_NULL_POINTER;
  uint32_t* words = device_status_words();
  if (!words) return B200S_ERR_NO_DEVICE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint32_t host[2] = {0, 0};
  B200S_CUDA_OK(cudaMemcpyAsync(host, words, sizeof(host), cudaMemcpyDeviceToHost, s));
  B200S_CUDA_OK(cudaStreamSynchronize(s));
  if (host[0] != 0) {
    B200S_CUDA_OK(cudaMemsetAsync(words, 0, sizeof(host), s));
    B200S_CUDA_OK(cudaStreamSynchronize(s));
  }
  *status_out = host[0] ? B200S_ERR_DEVICE_TIMEOUT : B200S_OK;
  if (detail_out) *detail_out = static_cast<int32_t>(host[1]);
  return B200S_OK;
}

// ---- stage timing ------------------------------------------------------------------------------

int b200s_profile_begin(int max_calls) {
  if (max_calls < 1 || max_calls > 4096) return B200S_ERR_BAD_SHAPE;
  std::lock_guard<std::mutex> lock(g_prof_mu);
  for (cudaEvent_t e : g_prof_ev) cudaEventDestroy(e);
  g_prof_ev.assign(static_cast<size_t>(max_calls) * kProfMarks, nullptr);
  for (auto& e : g_prof_ev) B200S_CUDA_OK(cudaEventCreate(&e));
  g_prof_max = max_calls, g_prof_calls = 0, g_prof_on = true;
  return B200S_OK;
}

int b200s_profile_end(float* stage_ms_out, int32_t* calls_out) {
  if (!stage_ms_out || !calls_out) return B200S_ERR_NULL_POINTER;
  std::lock_guard<std::mutex> lock(g_prof_mu);
  g_prof_on = false;
  for (int k = 0; k + 1 < kProfMarks; ++k) stage_ms_out[k] = 0.f;
  *calls_out = g_prof_calls;
  int rc = B200S_OK;
  for (int c = 0; c < g_prof_calls && rc == B200S_OK; ++c) {
    cudaEvent_t* ev = &g_prof_ev[static_cast<size_t>(c) * kProfMarks];
    if (cudaEventSynchronize(ev[kProfMarks - 1]) != cudaSuccess) rc = B200S_ERR_CUDA;
    for (int k = 0; k + 1 < kProfMarks && rc == B200S_OK; ++k) {
      float ms = 0.f;
      if (cudaEventElapsedTime(&ms, ev[k], ev[k + 1]) != cudaSuccess) rc = B200S_ERR_CUDA;
      stage_ms_out[k] += ms;
    }
  }
  if (rc == B200S_OK && g_prof_calls > 0)
    for (int k = 0; k + 1 < kProfMarks; ++k) stage_ms_out[k] /= static_cast<float>(g_prof_calls);
  for (cudaEvent_t e : g_prof_ev) cudaEventDestroy(e);
  g_prof_ev.clear();
  g_prof_max = g_prof_calls = 0;
  return rc;
}

// ---- tuner -----------------------------------------------------------------------------------

int b200s_tuner_clear(void) {
  std::lock_guard<std::mutex> lock(g_tuner_mu);
  g_tuner.clear();
  return B200S_OK;
}

int b200s_tuner_record_schedule(int64_t M, int64_t N, int64_t K, int32_t in_dtype, int32_t algo, int32_t depth,
                                int32_t fuse) {
  if (M <= 0 || N <= 0 || K <= 0) return B200S_ERR_BAD_SHAPE;
  if (!valid_dtype(in_dtype)) return B200S_ERR_BAD_DTYPE;
  if (algo < B200S_ALGO_DENSE || algo > B200S_ALGO_WINOGRAD) return B200S_ERR_BAD_ALGO;
  if (depth < 0 || depth > kMaxDepth) return B200S_ERR_BAD_DEPTH;
  if (fuse < 0 || fuse > 3) return B200S_ERR_BAD_SHAPE;
  if (algo == B200S_ALGO_DENSE) depth = 0, fuse = 0;
  std::lock_guard<std::mutex> lock(g_tuner_mu);
  for (auto& e : g_tuner) {
    if (e.M == M && e.N == N && e.K == K && e.in_dtype == in_dtype) {
      e.algo = algo, e.depth = depth, e.fuse = fuse;
      return B200S_OK;
    }
  }
  g_tuner.push_back({M, N, K, in_dtype, algo, depth, fuse});
  return B200S_OK;
}

int b200s_tuner_record(int64_t M, int64_t N, int64_t K, int32_t in_dtype, int32_t algo, int32_t depth) {
  return b200s_tuner_record_schedule(M, N, K, in_dtype, algo, depth, 0);
}

int b200s_tuner_lookup_schedule(int64_t M, int64_t N, int64_t K, int32_t in_dtype, int32_t* algo_out,
                                int32_t* depth_out, int32_t* fuse_out) {
  if (!algo_out || !depth_out || !fuse_out) return B200S_ERR_NULL_POINTER;
  if (M <= 0 || N <= 0 || K <= 0) return B200S_ERR_BAD_SHAPE;
  std::lock_guard<std::mutex> lock(g_tuner_mu);
  const TunerEntry* best = nullptr;
  double best_d = 0;
  const double lm = std::log2(static_cast<double>(M)), ln = std::log2(static_cast<double>(N)),
               lk = std::log2(static_cast<double>(K));
  for (const auto& e : g_tuner) {
    if (e.in_dtype != in_dtype) continue;
    const double dm = lm - std::log2(static_cast<double>(e.M)), dn = ln - std::log2(static_cast<double>(e.N)),
                 dk = lk - std::log2(static_cast<double>(e.K));
    const double d = dm * dm + dn * dn + dk * dk;
    if (!best || d < best_d) best = &e, best_d = d;
  }
  if (!best) {
    default_choice(M, N, K, algo_out, depth_out);
    *fuse_out = 0;
    return B200S_OK;
  }
  *algo_out = best->algo;
  *depth_out = best->depth;
  *fuse_out = best->fuse;
  return B200S_OK;
}

int b200s_tuner_lookup(int64_t M, int64_t N, int64_t K, int32_t in_dtype, int32_t* algo_out, int32_t* depth_out) {
  int32_t fuse = 0;
  return b200s_tuner_lookup_schedule(M, N, K, in_dtype, algo_out, depth_out, &fuse);
}

int b200s_tuner_load(const char* path) {
  if (!path) return B200S_ERR_NULL_POINTER;
  std::FILE* f = std::fopen(path, "r");
  if (!f) return B200S_ERR_TUNER_IO;
  std::vector<TunerEntry> entries;
  char line[256];
  bool bad = false;
  while (std::fgets(line, sizeof(line), f)) {
    if (line[0] == '#' || line[0] == '\n' || line[0] == '\0') continue;
    long long m, n, k;
    int dt, algo, depth, fuse = 0;
    const int got = std::sscanf(line, "%lld %lld %lld %d %d %d %d", &m, &n, &k, &dt, &algo, &depth, &fuse);
    if (got < 6 || m <= 0 || n <= 0 || k <= 0 || !valid_dtype(dt) || algo < B200S_ALGO_DENSE ||
        algo > B200S_ALGO_WINOGRAD || depth < 0 || depth > kMaxDepth || fuse < 0 || fuse > 3) {
      bad = true;
      break;
    }
    const bool dense = algo == B200S_ALGO_DENSE;
    entries.push_back({m, n, k, dt, algo, dense ? 0 : depth, dense ? 0 : fuse});
  }
  std::fclose(f);
  if (bad) return B200S_ERR_TUNER_IO;  // a corrupt file leaves the current table untouched
  std::lock_guard<std::mutex> lock(g_tuner_mu);
  g_tuner.swap(entries);
  return B200S_OK;
}

int b200s_tuner_save(const char* path) {
  if (!path) return B200S_ERR_NULL_POINTER;
  std::FILE* f = std::fopen(path, "w");
  if (!f) return B200S_ERR_TUNER_IO;
  std::lock_guard<std::mutex> lock(g_tuner_mu);
  std::fprintf(f, "# M N K in_dtype algo depth fuse\n");
  for (const auto& e : g_tuner)
    std::fprintf(f, "%lld %lld %lld %d %d %d %d\n", static_cast<long long>(e.M), static_cast<long long>(e.N),
                 static_cast<long long>(e.K), e.in_dtype, e.algo, e.depth, e.fuse);
  std::fclose(f);
  return B200S_OK;
}

}  // extern "C"
