// C ABI of libsage_b200: argument validation, scratch carving and kernel dispatch.
//
// The checks mirror the ones the reference performs before launching
// (csrc/bindings.cpp:13-48 of the reference): positive N, K divisible by 128, a
// 64/128/256-entry codebook, 4-byte aligned grid and codebook, rows <= 65535.
// Errors come back as negative status codes instead of C++ exceptions.
#include "../../include/sage_b200.h"
#include "../../include/sage_b200_debug.h"

#include <atomic>
#include <climits>
#include <cstring>
#include <mutex>

#include "sage_common.cuh"
#include "sage_kernels.h"

namespace sageb200 {
// bit 0: the packed-linear kernels; bit 1: every glue kernel (measured slower: most have nothing to
// do before their wait); bit 2: the attention step alone, which requests its first cache rows
// before the wait (measured +0.5 % on the one-sequence step)
int g_sageb200_pdl = 5;
unsigned long long g_sageb200_glue_launches = 0;
namespace {

constexpr int kMaxDevices = 64;
constexpr int kVersion = 100;  // 0.1.0

struct DeviceState {
  std::atomic<int> ready{0};
  int sm_count = 0;
  int major = 0;
  int *status = nullptr;       // device-visible address of the word the kernels write on a timed-out wait
  volatile int *status_host = nullptr;  // the same word as the host reads it
};

// One page of host memory per device for the status word.  It is static storage pinned and
// mapped with cudaHostRegister at set-up, so that no entry point of the library allocates
// memory; only where the platform refuses to pin static storage does set-up fall back to
// one pinned word from cudaHostAlloc.
struct alignas(4096) StatusPage {
  int word;
  char pad[4096 - sizeof(int)];
};
StatusPage g_status_pages[64];
std::mutex g_setup_mutex;  // first-time set-up of a device may be raced by several host threads

// Activation rows from which the tcgen05 prefill GEMM takes over from 16-row skinny passes.
constexpr int kGemmMinRows = 33;
DeviceState g_devices[kMaxDevices];
Tuning g_tuning{0, 0, 0, 0};
std::atomic<unsigned long long> g_launches{0};
long long *g_trace = nullptr;  // profiling aid, see sageb200_debug_trace
int g_trace_launch = 0;        // launches traced since the buffer was set

size_t align256(size_t bytes) { return (bytes + 255) / 256 * 256; }

constexpr size_t kStageSharedLimit = 96 * 1024;  // rows up to 49152 channels
cudaError_t configure_stage_rows();  // (defined after the kernel)

// Per-device one-time set-up on the calling thread's current device.
int device_state(DeviceState **out) {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) {
    cudaGetLastError();
    return SAGEB200_ERR_NO_DEVICE;
  }
  if (device < 0 || device >= kMaxDevices) return SAGEB200_ERR_NO_DEVICE;
  DeviceState &state = g_devices[device];
  if (!state.ready.load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!state.ready.load(std::memory_order_acquire)) {
      int sms = 0, major = 0;
      if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
          cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) {
        cudaGetLastError();
        return SAGEB200_ERR_CUDA;
      }
      if (major != 10) return SAGEB200_ERR_NO_DEVICE;  // built for sm_100a only
      if (configure_skinny() != cudaSuccess || configure_gemm_tc() != cudaSuccess ||
          configure_stage_rows() != cudaSuccess) {
        cudaGetLastError();
        return SAGEB200_ERR_CUDA;
      }
      // the status word: this device's static page, pinned and mapped in place
      StatusPage &page = g_status_pages[device];
      page.word = 0;
      void *device_view = nullptr;
      if (cudaHostRegister(&page, sizeof(page), cudaHostRegisterMapped | cudaHostRegisterPortable) == cudaSuccess &&
          cudaHostGetDevicePointer(&device_view, &page.word, 0) == cudaSuccess && device_view) {
        state.status = static_cast<int *>(device_view);
        state.status_host = &page.word;
      } else {
        cudaGetLastError();
        int *word = nullptr;
        if (cudaHostAlloc(reinterpret_cast<void **>(&word), sizeof(int), cudaHostAllocMapped) != cudaSuccess) {
          cudaGetLastError();
          return SAGEB200_ERR_CUDA;
        }
        *word = 0;
        state.status = word;
        state.status_host = word;
      }
      state.sm_count = sms;
      state.major = major;
      state.ready.store(1, std::memory_order_release);
    }
  }
  *out = &state;
  // a kernel of an earlier call reported a timed-out wait
  // (it stays recorded until sageb200_clear_status)
  if (*state.status_host != 0) return SAGEB200_ERR_TIMEOUT;
  return SAGEB200_OK;
}

int planning_sm_count() {
  DeviceState *state = nullptr;
  if (device_state(&state) == SAGEB200_OK) return state->sm_count;
  return 148;
}

int check_shape(int rows, int n, int k, int entries) {
  if (n <= 0 || k <= 0 || (k % 128) != 0 || rows < 0) return SAGEB200_ERR_INVALID_ARGUMENT;
  if (direction_bits_of(entries) < 0) return SAGEB200_ERR_INVALID_ARGUMENT;
  if (rows > 65535) return SAGEB200_ERR_RANGE;
  if (static_cast<long long>((n + 15) / 16) * (k / 128) * 16 > INT_MAX) return SAGEB200_ERR_RANGE;
  return SAGEB200_OK;
}

int check_buffers(const void *codes, const void *radii, const void *grid, const void *book) {
  if (!codes || !radii || !grid || !book) return SAGEB200_ERR_INVALID_ARGUMENT;
  // grid and codebook: 4 bytes as in the reference; codes/radii (and grid, for the bulk
  // copies of the decode kernel) additionally 16 bytes, which any allocator provides
  if ((reinterpret_cast<uintptr_t>(grid) & 15) || (reinterpret_cast<uintptr_t>(book) & 3) ||
      (reinterpret_cast<uintptr_t>(radii) & 15) || (reinterpret_cast<uintptr_t>(codes) & 15))
    return SAGEB200_ERR_ALIGNMENT;
  return SAGEB200_OK;
}

// Scratch layout: a FIXED counter region at the front (arrival counters, zero between
// launches) followed by split-K partial sums.  The counter region never holds anything
// else, so one buffer can serve calls of different shapes one after another.
constexpr size_t kCounterRegionBytes = 64 * 1024;
constexpr int kCounterCapacity = static_cast<int>(kCounterRegionBytes / sizeof(unsigned));

// Scratch one problem needs at `rows` <= 16: partial pieces, then (rows > 1 with a
// permutation) the gathered activations.
// (a fused producer of several rows gives every problem its own staged copy)
size_t gather_bytes(int rows, int k, bool permuted) {
  return rows > 1 && permuted ? align256(static_cast<size_t>(rows) * k * 2) : 0;
}
size_t plan_bytes(const SkinnyPlan &plan) { return align256(plan.partial_bytes); }

// Shares of the device for the problems of a grouped launch: CTAs in proportion to the
// (tile, group) units of each problem, so the launch is one resident wave.
void cta_budgets(const sageb200_problem *problems, int count, const DeviceState &device, int *budgets) {
  for (int i = 0; i < count; ++i) budgets[i] = 0;
  int live = 0;
  double total = 0;
  for (int i = 0; i < count; ++i)
    if (problems[i].rows > 0) {
      ++live;
      total += static_cast<double>((problems[i].n + 15) / 16) * (problems[i].k / 128);
    }
  if (live <= 1) return;  // a single problem plans for the whole device
  const int per_sm = g_tuning.ctas_per_sm > 0 ? g_tuning.ctas_per_sm : 1;
  const int resident = device.sm_count * per_sm;
  for (int i = 0; i < count; ++i) {
    if (problems[i].rows == 0) continue;
    const double units = static_cast<double>((problems[i].n + 15) / 16) * (problems[i].k / 128);
    int share = static_cast<int>(resident * units / total);
    budgets[i] = share < 1 ? 1 : share;
  }
}

// Scratch bytes (after the counter region) the problems need together.
// `fits` (optional): whether the plans' shared-memory needs - the launch reserves the largest of
// each kind over its problems - fit one launch together.
size_t grouped_scratch_bytes(const sageb200_problem *problems, int count, const DeviceState &device,
                             int act_kind = 0, bool *fits = nullptr) {
  int budgets[kMaxGrouped];
  cta_budgets(problems, count, device, budgets);
  size_t bytes = 0;
  size_t x_bytes = 0, lin_bytes = 0;
  int unit_capacity = 0, warps = 0, warp_segments = 0, column_blocks = 1;
  bool ring = false;
  for (int i = 0; i < count; ++i) {
    const sageb200_problem &in = problems[i];
    if (in.rows == 0) continue;
    const SkinnyPlan plan =
        plan_skinny(in.rows, in.n, in.k, in.entries, device.sm_count, g_tuning, budgets[i], in.rows == 1 ? act_kind : 0);
    bytes += align256(plan.partial_bytes) + gather_bytes(in.rows, in.k, in.perm != nullptr || act_kind != 0);
    if (plan.x_bytes > x_bytes) x_bytes = plan.x_bytes;
    if (plan.lin_bytes > lin_bytes) lin_bytes = plan.lin_bytes;
    if (plan.unit_capacity > unit_capacity) unit_capacity = plan.unit_capacity;
    if (plan.warps > warps) warps = plan.warps;
    if (plan.warp_segments > warp_segments) warp_segments = plan.warp_segments;
    if (plan.column_blocks > column_blocks) column_blocks = plan.column_blocks;
    ring = ring || plan.ring != 0;
  }
  // (ring streaming exists for one column block only: a problem of up to eight rows that streams
  //  cannot share a launch with one of more than eight rows)
  if (fits)
    *fits = skinny_shared_fits(x_bytes, unit_capacity, warps, warp_segments, column_blocks, lin_bytes) &&
            !(ring && column_blocks != 1);
  return bytes;
}

// Problems whose plans do not fit one launch together run as two launches, first half and second
// half, each planned for the whole device (and so on); the scratch is the larger need.
size_t grouped_scratch_split(const sageb200_problem *problems, int count, const DeviceState &device) {
  bool fits = true;
  const size_t bytes = grouped_scratch_bytes(problems, count, device, 0, &fits);
  if (fits || count <= 1) return bytes;
  const size_t first = grouped_scratch_split(problems, count / 2, device);
  const size_t second = grouped_scratch_split(problems + count / 2, count - count / 2, device);
  return first > second ? first : second;
}

// Activation rows of a launch of several rows, for every problem in ONE launch: the row is
// taken from the problem's x (kind 0) or computed from the fused producer's inputs (kind 1
// residual add + RMSNorm - job 0 also writes the new residual - or kind 2 SwiGLU), staged in
// shared memory and written out in the problem's quantised channel order.  grid = (rows, jobs).
struct StageJob {
  const __half *x;
  const int32_t *perm;  // null: identity
  __half *xq;
  int rows, k;
  // routed experts (null: none): the permutation is that of expert expert_ids[expert_slot] inside
  // a stack of expert_count experts starting at global expert expert_first; a slot whose expert
  // lives elsewhere (or is negative: an empty block) is skipped
  const int *expert_ids;
  int expert_slot, expert_first, expert_count;
};
struct StageParams {
  StageJob job[kMaxGrouped];
  int kind;
  float eps;
  const __half *a, *b, *weight;
  __half *residual_out;
};

__global__ void __launch_bounds__(256) stage_rows_kernel(const __grid_constant__ StageParams params) {
  extern __shared__ __half row_shared[];
  __shared__ float sums[8];
  // (the decode kernel behind this launch sets up and prefetches its weights meanwhile; this
  //  launch itself was scheduled while its producer still ran)
  pdl_launch_dependents();
  StageJob job = params.job[blockIdx.y];
  const int row = blockIdx.x;
  const int k = job.k;
  // The permutation and the norm weights are never written by a kernel, and a decode step streams
  // far more than the L2 holds, so they tend to come from HBM: each thread requests its first two
  // 8-channel vectors of both before the wait for the producer, not at the point of use.
  constexpr int kHeld = 2;
  int4 held_lo[kHeld], held_hi[kHeld];
  uint4 held_weight[kHeld];
  const bool hold_perm = job.perm != nullptr && job.expert_ids == nullptr && row < job.rows &&
                         (reinterpret_cast<uintptr_t>(job.perm) & 15) == 0;
  const bool hold_weight = params.kind == 1 && row < job.rows && (reinterpret_cast<uintptr_t>(params.weight) & 15) == 0;
#pragma unroll
  for (int u = 0; u < kHeld; ++u) {
    const int v = threadIdx.x + 256 * u;
    held_lo[u] = held_hi[u] = make_int4(0, 0, 0, 0);
    held_weight[u] = make_uint4(0, 0, 0, 0);
    if (v < (k >> 3)) {
      if (hold_perm) {
        held_lo[u] = __ldg(reinterpret_cast<const int4 *>(job.perm) + 2 * v);
        held_hi[u] = __ldg(reinterpret_cast<const int4 *>(job.perm) + 2 * v + 1);
      }
      if (hold_weight) held_weight[u] = __ldg(reinterpret_cast<const uint4 *>(params.weight) + v);
    }
  }
  pdl_wait();
  if (row >= job.rows) return;
  if (job.expert_ids) {
    const int expert = __ldg(job.expert_ids + job.expert_slot) - job.expert_first;
    if (expert < 0 || expert >= job.expert_count) return;
    if (job.perm) job.perm += static_cast<long long>(expert) * k;
  }
  const size_t offset = static_cast<size_t>(row) * k;
  // eight values per thread and load where the inputs are 16-byte aligned (k is a multiple of 128)
  auto wide = [&](const __half *p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p + offset) & 15) == 0; };
  const int vectors = k >> 3;
  if (params.kind == 0) {
    if (wide(job.x)) {
      for (int v = threadIdx.x; v < vectors; v += 256)
        reinterpret_cast<uint4 *>(row_shared)[v] = reinterpret_cast<const uint4 *>(job.x + offset)[v];
    } else {
      for (int i = threadIdx.x; i < k; i += 256) row_shared[i] = job.x[offset + i];
    }
  } else if (params.kind == 2) {
    if (wide(params.a) && wide(params.b)) {
      for (int v = threadIdx.x; v < vectors; v += 256) {
        const uint4 g4 = reinterpret_cast<const uint4 *>(params.a + offset)[v];
        const uint4 u4 = reinterpret_cast<const uint4 *>(params.b + offset)[v];
        const __half2 *g2 = reinterpret_cast<const __half2 *>(&g4), *u2 = reinterpret_cast<const __half2 *>(&u4);
        uint4 out;
        __half2 *o2 = reinterpret_cast<__half2 *>(&out);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 g = __half22float2(g2[q]);
          o2[q] = __hmul2(__halves2half2(__float2half_rn(silu_fast(g.x)), __float2half_rn(silu_fast(g.y))), u2[q]);
        }
        reinterpret_cast<uint4 *>(row_shared)[v] = out;
      }
    } else {
      for (int i = threadIdx.x; i < k; i += 256) {
        const float g = __half2float(params.a[offset + i]);
        row_shared[i] = __hmul(__float2half_rn(silu_fast(g)), params.b[offset + i]);
      }
    }
  } else {
    float square = 0.0f;
    if (wide(params.a) && wide(params.b) && wide(params.residual_out)) {
      for (int v = threadIdx.x; v < vectors; v += 256) {
        uint4 sum4 = reinterpret_cast<const uint4 *>(params.a + offset)[v];
        __half2 *s2 = reinterpret_cast<__half2 *>(&sum4);
        if (params.b) {
          const uint4 b4 = reinterpret_cast<const uint4 *>(params.b + offset)[v];
          const __half2 *b2 = reinterpret_cast<const __half2 *>(&b4);
#pragma unroll
          for (int q = 0; q < 4; ++q) s2[q] = __hadd2(s2[q], b2[q]);
        }
        reinterpret_cast<uint4 *>(row_shared)[v] = sum4;
        if (blockIdx.y == 0) reinterpret_cast<uint4 *>(params.residual_out + offset)[v] = sum4;
      }
      __syncthreads();
      // the squares in the scalar loop's order (element i in thread i % 256), out of shared memory:
      // the norm is then bit-identical whichever way the row was loaded
      for (int i = threadIdx.x; i < k; i += 256) {
        const float f = __half2float(row_shared[i]);
        square = fmaf(f, f, square);
      }
    } else {
      for (int i = threadIdx.x; i < k; i += 256) {
        const __half v = params.b ? __hadd(params.a[offset + i], params.b[offset + i]) : params.a[offset + i];
        row_shared[i] = v;
        if (blockIdx.y == 0) params.residual_out[offset + i] = v;
        const float f = __half2float(v);
        square = fmaf(f, f, square);
      }
    }
    for (int o = 16; o; o >>= 1) square += __shfl_xor_sync(0xffffffffu, square, o);
    if ((threadIdx.x & 31) == 0) sums[threadIdx.x >> 5] = square;
    __syncthreads();
    float total = 0.0f;
    for (int w = 0; w < 8; ++w) total += sums[w];
    const float scale = rsqrtf(total / k + params.eps);
    if (hold_weight) {  // eight values at a time, the same arithmetic per value
      auto scale_vector = [&](int v, const uint4 &weight4) {
        uint4 value = reinterpret_cast<const uint4 *>(row_shared)[v];
        __half *h = reinterpret_cast<__half *>(&value);
        const __half *w = reinterpret_cast<const __half *>(&weight4);
#pragma unroll
        for (int c = 0; c < 8; ++c) h[c] = __hmul(w[c], __float2half_rn(__half2float(h[c]) * scale));
        reinterpret_cast<uint4 *>(row_shared)[v] = value;
      };
#pragma unroll
      for (int u = 0; u < kHeld; ++u)
        if (threadIdx.x + 256 * u < vectors) scale_vector(threadIdx.x + 256 * u, held_weight[u]);
      for (int v = threadIdx.x + 256 * kHeld; v < vectors; v += 256)
        scale_vector(v, __ldg(reinterpret_cast<const uint4 *>(params.weight) + v));
    } else {
      for (int i = threadIdx.x; i < k; i += 256)
        row_shared[i] = __hmul(params.weight[i], __float2half_rn(__half2float(row_shared[i]) * scale));
    }
  }
  __syncthreads();
  const bool aligned = job.perm == nullptr || (reinterpret_cast<uintptr_t>(job.perm) & 15) == 0;
  auto write_vector = [&](int v, bool held, const int4 &held_low, const int4 &held_high) {
    __align__(16) __half out[8];
    if (job.perm == nullptr) {
      *reinterpret_cast<uint4 *>(out) = reinterpret_cast<const uint4 *>(row_shared)[v];
    } else {
      int source[8];
      if (aligned) {
        const int4 lo = held ? held_low : __ldg(reinterpret_cast<const int4 *>(job.perm) + 2 * v);
        const int4 hi = held ? held_high : __ldg(reinterpret_cast<const int4 *>(job.perm) + 2 * v + 1);
        source[0] = lo.x; source[1] = lo.y; source[2] = lo.z; source[3] = lo.w;
        source[4] = hi.x; source[5] = hi.y; source[6] = hi.z; source[7] = hi.w;
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c) source[c] = __ldg(job.perm + 8 * v + c);
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) out[c] = row_shared[source[c]];
    }
    reinterpret_cast<uint4 *>(job.xq + offset)[v] = *reinterpret_cast<const uint4 *>(out);
  };
#pragma unroll
  for (int u = 0; u < kHeld; ++u)
    if (threadIdx.x + 256 * u < (k >> 3)) write_vector(threadIdx.x + 256 * u, hold_perm, held_lo[u], held_hi[u]);
  for (int v = threadIdx.x + 256 * kHeld; v < (k >> 3); v += 256) write_vector(v, false, held_lo[0], held_hi[0]);
}

cudaError_t configure_stage_rows() {
  return cudaFuncSetAttribute(stage_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(kStageSharedLimit));
}

// rows <= 16, one or more problems, one launch (plus one small gather launch for each
// problem that has several rows and a permutation).
// Expert indirection of one problem of a launch (see SkinnyProblem).
struct ExpertRef {
  const int *ids;
  int slot, first, count;
  long long codes_stride, cell_stride, book_stride;
};

int run_skinny(const sageb200_problem *problems, int count, void *workspace,
               size_t workspace_bytes, cudaStream_t stream, const DeviceState &device,
               const sageb200_activation *activation = nullptr, const ExpertRef *experts = nullptr) {
  if (!activation && count > 1) {
    // plans that do not fit one launch together (the launch reserves the largest share, tables and
    // activation rows of any problem): two launches, as grouped_scratch_split sizes them
    bool fits = true;
    grouped_scratch_bytes(problems, count, device, 0, &fits);
    if (!fits) {
      const int half = count / 2;
      const int status = run_skinny(problems, half, workspace, workspace_bytes, stream, device, nullptr, experts);
      if (status) return status;
      return run_skinny(problems + half, count - half, workspace, workspace_bytes, stream, device, nullptr,
                        experts ? experts + half : nullptr);
    }
  }
  SkinnyParams params;
  std::memset(&params, 0, sizeof(params));
  params.status = device.status;
  // a fused producer of several rows runs in the staging launch, of one row inside the decode kernel
  const bool fused_rows = activation && activation->kind != 0 && count > 0 && problems[0].rows > 1;
  StageParams staging;
  std::memset(&staging, 0, sizeof(staging));
  int jobs = 0, stage_rows = 0, stage_k = 0;
  if (fused_rows) {
    staging.kind = activation->kind;
    staging.eps = activation->eps;
    staging.a = static_cast<const __half *>(activation->a);
    staging.b = static_cast<const __half *>(activation->b);
    staging.weight = static_cast<const __half *>(activation->weight);
    staging.residual_out = static_cast<__half *>(activation->residual_out);
  }
  if (activation && activation->kind != 0 && !fused_rows) {  // one row: inside the decode kernel
    params.act_kind = activation->kind;
    params.act_eps = activation->eps;
    params.act_a = activation->a;
    params.act_b = activation->b;
    params.act_weight = activation->weight;
    params.act_residual_out = activation->residual_out;
  }
  // launch i of a traced run writes block min(i, 63) of 512 CTA records
  params.trace = g_trace ? g_trace + static_cast<size_t>(g_trace_launch < 63 ? g_trace_launch : 63) * 512 * 16 : nullptr;
  if (g_trace) ++g_trace_launch;
  unsigned char *scratch = static_cast<unsigned char *>(workspace);
  size_t offset = kCounterRegionBytes;
  int counters_used = 0;
  int ctas = 0;
  int live = 0;
  int warps = 0, column_blocks = 1;
  int budgets[kMaxGrouped];
  cta_budgets(problems, count, device, budgets);
  for (int i = 0; i < count; ++i) {
    const sageb200_problem &in = problems[i];
    if (in.rows == 0) continue;
    const SkinnyPlan plan =
        plan_skinny(in.rows, in.n, in.k, in.entries, device.sm_count, g_tuning, budgets[i], params.act_kind);
    const size_t partial = plan_bytes(plan);
    const size_t gathered = gather_bytes(in.rows, in.k, in.perm != nullptr || fused_rows);
    if (partial || gathered) {
      if (!workspace || offset + partial + gathered > workspace_bytes) return SAGEB200_ERR_WORKSPACE;
      if (reinterpret_cast<uintptr_t>(workspace) & 255) return SAGEB200_ERR_ALIGNMENT;
    }
    if (plan.needs_scratch && counters_used + plan.tiles > kCounterCapacity) return SAGEB200_ERR_RANGE;
    SkinnyProblem &out = params.problem[live];
    out.x = static_cast<const __half *>(in.x);
    out.perm = in.perm;
    if (gathered) {
      // several activation rows: staged (and gathered) once, by one launch for all problems,
      // instead of once per CTA
      __half *xq = reinterpret_cast<__half *>(scratch + offset + partial);
      if (static_cast<size_t>(in.k) * 2 <= kStageSharedLimit) {
        staging.job[jobs] = StageJob{out.x, in.perm, xq, in.rows, in.k, nullptr, 0, 0, 0};
        if (experts) {
          staging.job[jobs].expert_ids = experts[i].ids;
          staging.job[jobs].expert_slot = experts[i].slot;
          staging.job[jobs].expert_first = experts[i].first;
          staging.job[jobs].expert_count = experts[i].count;
        }
        ++jobs;
        if (in.rows > stage_rows) stage_rows = in.rows;
        if (in.k > stage_k) stage_k = in.k;
      } else {  // a row too long for the staging kernel's shared memory (never with a fused producer)
        if (fused_rows || experts) return SAGEB200_ERR_RANGE;
        if (launch_gather(out.x, in.perm, xq, in.rows, in.k, stream, device.sm_count) != cudaSuccess) {
          cudaGetLastError();
          return SAGEB200_ERR_CUDA;
        }
        g_launches.fetch_add(1, std::memory_order_relaxed);
      }
      out.x = xq;
      out.perm = nullptr;
    }
    out.codes = static_cast<const uint32_t *>(in.codes);
    out.radii = static_cast<const uint32_t *>(in.radii);
    out.grid = static_cast<const uint32_t *>(in.grid);
    out.book = static_cast<const uint32_t *>(in.book);
    out.y = static_cast<__half *>(in.y);
    out.partial = plan.needs_scratch ? reinterpret_cast<float *>(scratch + offset) : nullptr;
    out.counters = plan.needs_scratch ? static_cast<unsigned *>(workspace) + counters_used : nullptr;
    out.rows = in.rows;
    out.n = in.n;
    out.k = in.k;
    out.groups = in.k / 128;
    out.tiles = plan.tiles;
    out.entries = in.entries;
    out.dbits = direction_bits_of(in.entries);
    out.slices = plan.slices;
    out.ctas_per_slice = plan.ctas_per_slice;
    out.slots_per_tile = plan.slots_per_tile;
    out.whole_tiles = plan.whole_tiles;
    out.ring = plan.ring;
    {
      const long long share = plan.whole_tiles ? plan.tiles : static_cast<long long>(plan.tiles) * (in.k / 128);
      out.share_q = static_cast<int>(share / plan.ctas_per_slice);
      out.share_r = static_cast<int>(share % plan.ctas_per_slice);
    }
    out.cta_begin = ctas;
    if (experts) {
      out.expert_ids = experts[i].ids;
      out.expert_slot = experts[i].slot;
      out.expert_first = experts[i].first;
      out.expert_count = experts[i].count;
      out.codes_stride = experts[i].codes_stride;
      out.cell_stride = experts[i].cell_stride;
      out.book_stride = experts[i].book_stride;
    }
    ctas += plan.ctas;
    offset += partial + gathered;
    if (plan.needs_scratch) counters_used += plan.tiles;
    if (static_cast<int>(plan.x_bytes) > params.x_bytes) params.x_bytes = static_cast<int>(plan.x_bytes);
    if (plan.unit_capacity > params.unit_capacity) params.unit_capacity = plan.unit_capacity;
    if (plan.warp_segments > params.warp_segments) params.warp_segments = plan.warp_segments;
    if (static_cast<int>(plan.lin_bytes) > params.lin_bytes) params.lin_bytes = static_cast<int>(plan.lin_bytes);
    if (plan.warps > warps) warps = plan.warps;
    if (plan.column_blocks > column_blocks) column_blocks = plan.column_blocks;
    ++live;
  }
  if (live == 0) return SAGEB200_OK;
  if (jobs > 0) {
    const size_t shared = static_cast<size_t>(stage_k) * sizeof(__half);  // (limit raised per device at set-up)
    launch_dependent<1>(stage_rows_kernel, dim3(stage_rows, jobs), dim3(256), shared, stream, staging);
    if (cudaGetLastError() != cudaSuccess) return SAGEB200_ERR_CUDA;
    g_launches.fetch_add(1, std::memory_order_relaxed);
  }
  params.count = live;
  // floor(2^32 / warps) + 1; unused (and not representable) for a single warp
  params.warps_reciprocal = warps > 1 ? static_cast<unsigned>((1ull << 32) / static_cast<unsigned>(warps)) + 1u : 0u;
  if (launch_skinny(params, warps, column_blocks, ctas, stream) != cudaSuccess) {
    cudaGetLastError();
    return SAGEB200_ERR_CUDA;
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return SAGEB200_OK;
}

int validate_problem(const sageb200_problem &p) {
  int status = check_shape(p.rows, p.n, p.k, p.entries);
  if (status) return status;
  status = check_buffers(p.codes, p.radii, p.grid, p.book);
  if (status) return status;
  if (p.rows > 0 && (!p.x || !p.y)) return SAGEB200_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(p.x) & 1) || (reinterpret_cast<uintptr_t>(p.y) & 1) ||
      (reinterpret_cast<uintptr_t>(p.perm) & 3))
    return SAGEB200_ERR_ALIGNMENT;
  return SAGEB200_OK;
}

}  // namespace

long long *trace_buffer() { return g_trace; }

void count_launches(int launches) { g_launches.fetch_add(static_cast<unsigned long long>(launches), std::memory_order_relaxed); }

int acquire_device(int **status_word, int *sm_count) {
  DeviceState *state = nullptr;
  const int status = device_state(&state);
  if (state) {
    if (status_word) *status_word = state->status;
    if (sm_count) *sm_count = state->sm_count;
  }
  return status;
}

}  // namespace sageb200

using namespace sageb200;

extern "C" {

int sageb200_version(void) { return kVersion; }

const char *sageb200_status_string(int status) {
  switch (status) {
    case SAGEB200_OK: return "ok";
    case SAGEB200_ERR_INVALID_ARGUMENT:
      return "invalid argument: SAGE requires positive N, K divisible by 128, a codebook of "
             "64/128/256 entries and non-null buffers";
    case SAGEB200_ERR_ALIGNMENT:
      return "alignment: SAGE codebook requires 4-byte aligned storage (packed codes, radius "
             "codes, radius grid and dense weight output 16, workspace 256)";
    case SAGEB200_ERR_RANGE: return "SAGE launch dimensions exceed supported range";
    case SAGEB200_ERR_WORKSPACE: return "workspace missing or smaller than sageb200_workspace_bytes";
    case SAGEB200_ERR_CUDA: return "a CUDA call or kernel launch failed";
    case SAGEB200_ERR_NO_DEVICE: return "no current CUDA device of compute capability 10.x";
    case SAGEB200_ERR_TIMEOUT: return "a bounded device-side wait ran out";
    case SAGEB200_ERR_STATIC_SCRATCH:
      return "this shape needs more scratch than the library's built-in static buffer holds "
             "(SAGEB200_STATIC_SCRATCH_BYTES) or more than 16 rows; use sageb200_linear with "
             "caller-provided scratch";
    default: return "unknown status";
  }
}

int sageb200_gemv_fuses_permutation(int n, int k) {
  (void)n;
  (void)k;
  return 1;
}

int sageb200_gemm_splits(int rows, int n, int k, int sm_count) {
  if (n <= 0 || k <= 0 || (k % 128) || rows <= 0) return 1;
  const int planned_rows = rows > 16 ? 16 : rows;
  return plan_skinny(planned_rows, n, k, 256, sm_count > 0 ? sm_count : 148, g_tuning).slices;
}

int sageb200_debug_plan(int rows, int n, int k, int sm_count, int act_kind, int *fields) {
  if (!fields || n <= 0 || k <= 0 || (k % 128) || rows <= 0 || rows > 16 || act_kind < 0 || act_kind > 2)
    return SAGEB200_ERR_INVALID_ARGUMENT;
  const SkinnyPlan plan = plan_skinny(rows, n, k, 256, sm_count > 0 ? sm_count : 148, g_tuning, 0, rows == 1 ? act_kind : 0);
  fields[0] = plan.ctas;
  fields[1] = plan.slices;
  fields[2] = plan.whole_tiles;
  fields[3] = plan.ring;
  fields[4] = plan.unit_capacity;
  fields[5] = plan.warps;
  fields[6] = static_cast<int>(plan.shared_bytes);
  fields[7] = plan.needs_scratch ? 1 : 0;
  return SAGEB200_OK;
}

size_t sageb200_workspace_bytes(int rows, int n, int k) {
  if (n <= 0 || k <= 0 || (k % 128) || rows <= 0) return 0;
  if (rows >= kGemmMinRows)  // arrival counters of split tiles + gathered activations + FP32 split tiles
    return kCounterRegionBytes + align256(static_cast<size_t>(rows) * k * 2) +
           align256(plan_gemm_tc(rows, n, k, planning_sm_count()).partial_bytes);
  const int sms = planning_sm_count();
  size_t bytes = 0;
  // rows > 16 run as 16-row passes plus a tail pass; reserve for the larger of the two
  const int passes[2] = {rows > 16 ? 16 : rows, rows > 16 ? rows % 16 : 0};
  for (int pass : passes) {
    if (pass == 0) continue;
    const size_t need = plan_bytes(plan_skinny(pass, n, k, 256, sms, g_tuning)) + gather_bytes(pass, k, true);
    if (need > bytes) bytes = need;
  }
  return bytes ? kCounterRegionBytes + bytes : 0;
}

namespace {
// (`limit`: the public entry points take SAGEB200_MAX_GROUPED problems, the expert entry points fill
//  launches up to the kernel's own capacity)
size_t grouped_workspace_bytes(const sageb200_problem *problems_host, int count, int limit);
}  // namespace

size_t sageb200_grouped_workspace_bytes(const sageb200_problem *problems_host, int count) {
  return grouped_workspace_bytes(problems_host, count, SAGEB200_MAX_GROUPED);
}

namespace {
size_t grouped_workspace_bytes(const sageb200_problem *problems_host, int count, int limit) {
  if (!problems_host || count <= 0 || count > limit) return 0;
  for (int i = 0; i < count; ++i)
    if (check_shape(problems_host[i].rows, problems_host[i].n, problems_host[i].k, problems_host[i].entries) ||
        problems_host[i].rows > 16)
      return 0;
  DeviceState fallback;
  fallback.sm_count = 148;
  DeviceState *device = nullptr;
  if (device_state(&device) != SAGEB200_OK) device = &fallback;
  const size_t bytes = grouped_scratch_split(problems_host, count, *device);
  return bytes ? kCounterRegionBytes + bytes : 0;
}
}  // namespace

int sageb200_linear_grouped(const sageb200_problem *problems_host, int count, void *workspace,
                            size_t workspace_bytes, void *stream) {
  if (!problems_host || count < 0 || count > SAGEB200_MAX_GROUPED)
    return SAGEB200_ERR_INVALID_ARGUMENT;
  for (int i = 0; i < count; ++i) {
    const int status = validate_problem(problems_host[i]);
    if (status) return status;
    if (problems_host[i].rows > 16) return SAGEB200_ERR_RANGE;
  }
  if (count == 0) return SAGEB200_OK;
  DeviceState *device = nullptr;
  const int status = device_state(&device);
  if (status) return status;
  return run_skinny(problems_host, count, workspace, workspace_bytes,
                    static_cast<cudaStream_t>(stream), *device);
}

int sageb200_linear(const void *x, const void *codes, const void *radii, const void *grid,
                    const void *book, const int32_t *perm, void *y, void *workspace,
                    size_t workspace_bytes, int rows, int n, int k, int entries, void *stream) {
  sageb200_problem problem{x, codes, radii, grid, book, perm, y, rows, n, k, entries};
  int status = validate_problem(problem);
  if (status) return status;
  if (rows == 0) return SAGEB200_OK;
  DeviceState *device = nullptr;
  status = device_state(&device);
  if (status) return status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (rows >= kGemmMinRows) {
    // Prefill: tcgen05 GEMM over activations in quantised channel order.  The gather (or
    // a re-alignment copy) lands in the workspace so the TMA loads see contiguous rows.
    const __half *xq = static_cast<const __half *>(x);
    const size_t gathered_bytes = align256(static_cast<size_t>(rows) * k * 2);
    if (workspace && (reinterpret_cast<uintptr_t>(workspace) & 255)) return SAGEB200_ERR_ALIGNMENT;
    if (perm || (reinterpret_cast<uintptr_t>(x) & 15)) {
      const size_t need = kCounterRegionBytes + gathered_bytes;
      if (!workspace || workspace_bytes < need) return SAGEB200_ERR_WORKSPACE;
      __half *gathered =
          reinterpret_cast<__half *>(static_cast<unsigned char *>(workspace) + kCounterRegionBytes);
      if (launch_gather(xq, perm, gathered, rows, k, s, device->sm_count) != cudaSuccess) {
        cudaGetLastError();
        return SAGEB200_ERR_CUDA;
      }
      g_launches.fetch_add(1, std::memory_order_relaxed);
      xq = gathered;
    }
    // K is split over several CTAs per output tile when the grid would otherwise leave most SMs
    // idle; that needs the FP32 scratch behind the gathered activations (a caller whose workspace
    // predates it, or who passes none for unpermuted input, gets the unsplit plan)
    GemmPlan plan = plan_gemm_tc(rows, n, k, device->sm_count);
    float *partial = nullptr;
    unsigned *counters = nullptr;
    if (plan.k_splits > 1) {
      const size_t need = kCounterRegionBytes + gathered_bytes + align256(plan.partial_bytes);
      if (workspace && workspace_bytes >= need) {
        counters = static_cast<unsigned *>(workspace);
        partial = reinterpret_cast<float *>(static_cast<unsigned char *>(workspace) + kCounterRegionBytes + gathered_bytes);
      } else {
        plan = plan_gemm_tc(rows, n, k, device->sm_count, false);
      }
    }
    if (launch_gemm_tc(xq, static_cast<const uint32_t *>(codes), static_cast<const uint32_t *>(radii),
                       static_cast<const uint32_t *>(grid), static_cast<const uint32_t *>(book),
                       static_cast<__half *>(y), device->status, rows, n, k, entries, plan, s, partial,
                       counters) != cudaSuccess) {
      cudaGetLastError();
      return SAGEB200_ERR_CUDA;
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return SAGEB200_OK;
  }
  // Up to 16 rows go through in one pass; 17..32 rows run as 16-row passes over the
  // packed weights (each pass reuses the scratch, in stream order).
  for (int begin = 0; begin < rows; begin += 16) {
    sageb200_problem chunk = problem;
    chunk.rows = rows - begin < 16 ? rows - begin : 16;
    chunk.x = static_cast<const __half *>(x) + static_cast<size_t>(begin) * k;
    chunk.y = static_cast<__half *>(y) + static_cast<size_t>(begin) * n;
    status = run_skinny(&chunk, 1, workspace, workspace_bytes, s, *device);
    if (status) return status;
  }
  return SAGEB200_OK;
}

int sageb200_dequant(const void *codes, const void *radii, const void *grid, const void *book,
                     const int32_t *perm, void *w, int n, int k, int entries, void *stream) {
  int status = check_shape(0, n, k, entries);
  if (status) return status;
  status = check_buffers(codes, radii, grid, book);
  if (status) return status;
  if (!w) return SAGEB200_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(perm) & 3))
    return SAGEB200_ERR_ALIGNMENT;
  DeviceState *device = nullptr;
  status = device_state(&device);
  if (status) return status;
  if (launch_dequant(static_cast<const uint32_t *>(codes), static_cast<const uint32_t *>(radii),
                     static_cast<const uint32_t *>(grid), static_cast<const uint32_t *>(book), perm,
                     static_cast<__half *>(w), n, k, entries, static_cast<cudaStream_t>(stream),
                     device->sm_count) != cudaSuccess) {
    cudaGetLastError();
    return SAGEB200_ERR_CUDA;
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return SAGEB200_OK;
}

int sageb200_pack_spherical(const void *signs, const void *indices, const void *radius, void *codes,
                            void *high, void *grid_or_scales, void *mins, int n, int k, int entries,
                            int tiled, void *stream) {
  if (n <= 0 || k <= 0 || (k % 128) != 0 || direction_bits_of(entries) < 0 || (!tiled && entries != 64))
    return SAGEB200_ERR_INVALID_ARGUMENT;
  if (!signs || !indices || !radius || !codes || !high || !grid_or_scales || (!tiled && !mins))
    return SAGEB200_ERR_INVALID_ARGUMENT;
  if (static_cast<long long>((n + 15) / 16) * (k / 128) * 16 > INT_MAX) return SAGEB200_ERR_RANGE;
  if ((reinterpret_cast<uintptr_t>(signs) & 15) || (reinterpret_cast<uintptr_t>(indices) & 3) ||
      (reinterpret_cast<uintptr_t>(radius) & 15) || (reinterpret_cast<uintptr_t>(codes) & 15) ||
      (reinterpret_cast<uintptr_t>(high) & 3) || (reinterpret_cast<uintptr_t>(grid_or_scales) & 3) ||
      (reinterpret_cast<uintptr_t>(mins) & 1))
    return SAGEB200_ERR_ALIGNMENT;
  DeviceState *device = nullptr;
  const int status = device_state(&device);
  if (status) return status;
  if (launch_pack(static_cast<const int8_t *>(signs), static_cast<const int32_t *>(indices),
                  static_cast<const float *>(radius), static_cast<uint32_t *>(codes),
                  static_cast<uint32_t *>(high), static_cast<__half *>(grid_or_scales),
                  static_cast<__half *>(mins), n, k, direction_bits_of(entries), tiled != 0,
                  static_cast<cudaStream_t>(stream), device->sm_count) != cudaSuccess) {
    cudaGetLastError();
    return SAGEB200_ERR_CUDA;
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return SAGEB200_OK;
}

size_t sageb200_host_staging_bytes(int rows, int n, int k) {
  if (n <= 0 || k <= 0 || rows <= 0) return 0;
  return align256(static_cast<size_t>(rows) * k * 2) + align256(static_cast<size_t>(rows) * n * 2) +
         align256(sageb200_workspace_bytes(rows, n, k));
}

int sageb200_linear_host(const void *x_host, const void *codes, const void *radii,
                         const void *grid, const void *book, const int32_t *perm, void *y_host,
                         void *staging, size_t staging_bytes, int rows, int n, int k, int entries,
                         void *stream) {
  int status = check_shape(rows, n, k, entries);
  if (status) return status;
  if (rows == 0) return SAGEB200_OK;
  if (!x_host || !y_host || !staging) return SAGEB200_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(staging) & 255) return SAGEB200_ERR_ALIGNMENT;
  if (staging_bytes < sageb200_host_staging_bytes(rows, n, k)) return SAGEB200_ERR_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t x_bytes = static_cast<size_t>(rows) * k * 2;
  const size_t y_bytes = static_cast<size_t>(rows) * n * 2;
  unsigned char *x_dev = static_cast<unsigned char *>(staging);
  unsigned char *y_dev = x_dev + align256(x_bytes);
  unsigned char *work = y_dev + align256(y_bytes);
  const size_t work_bytes = staging_bytes - align256(x_bytes) - align256(y_bytes);
  if (cudaMemcpyAsync(x_dev, x_host, x_bytes, cudaMemcpyHostToDevice, s) != cudaSuccess) {
    cudaGetLastError();
    return SAGEB200_ERR_CUDA;
  }
  status = sageb200_linear(x_dev, codes, radii, grid, book, perm, y_dev, work, work_bytes, rows, n,
                           k, entries, stream);
  if (status) return status;
  if (cudaMemcpyAsync(y_host, y_dev, y_bytes, cudaMemcpyDeviceToHost, s) != cudaSuccess ||
      cudaStreamSynchronize(s) != cudaSuccess) {
    cudaGetLastError();
    return SAGEB200_ERR_CUDA;
  }
  return SAGEB200_OK;
}

int sageb200_clear_status(void) {
  DeviceState *device = nullptr;
  const int status = device_state(&device);
  if (status != SAGEB200_OK && status != SAGEB200_ERR_TIMEOUT) return status;
  // the caller has dealt with the time-out (the stream that reported it must be idle)
  *device->status_host = 0;
  return SAGEB200_OK;
}

int sageb200_debug_gemm_plan(int rows, int n, int k, int sm_count, int allow_split, int *fields) {
  if (!fields || rows < 33 || rows > 65535 || n <= 0 || k <= 0 || (k % 128)) return SAGEB200_ERR_INVALID_ARGUMENT;
  const GemmPlan plan = plan_gemm_tc(rows, n, k, sm_count > 0 ? sm_count : 148, allow_split != 0);
  fields[0] = plan.tokens_per_cta;
  fields[1] = plan.token_blocks;
  fields[2] = plan.row_blocks;
  fields[3] = plan.accumulators;
  fields[4] = plan.pair;
  fields[5] = plan.k_splits;
  fields[6] = plan.groups_per_split;
  fields[7] = plan.stages;
  fields[8] = static_cast<int>(plan.shared_bytes);
  fields[9] = static_cast<int>(plan.partial_bytes >> 10);  // KiB
  return SAGEB200_OK;
}

int sageb200_debug_gemm_pairs(int enabled) {
  g_gemm_pairs = enabled ? 1 : 0;
  return SAGEB200_OK;
}

int sageb200_set_pdl(int enabled) {
  g_sageb200_pdl = enabled & 7;
  return SAGEB200_OK;
}

int sageb200_debug_trace(void *device_buffer) {
  g_trace = static_cast<long long *>(device_buffer);
  g_trace_launch = 0;
  return SAGEB200_OK;
}

int sageb200_set_tuning(int warps, int slices, int ctas_per_sm, int mode) {
  if (warps < 0 || warps > 16 || slices < 0 || slices > 8 || ctas_per_sm < 0 || ctas_per_sm > 8 ||
      mode < 0 || mode > 3)
    return SAGEB200_ERR_INVALID_ARGUMENT;
  g_tuning = Tuning{warps, slices, ctas_per_sm, mode};
  return SAGEB200_OK;
}

unsigned long long sageb200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

unsigned long long sageb200_glue_launch_count(void) {
  return __atomic_load_n(&sageb200::g_sageb200_glue_launches, __ATOMIC_RELAXED);
}

size_t sageb200_fused_workspace_bytes(const sageb200_problem *problems_host, int count) {
  size_t grouped = sageb200_grouped_workspace_bytes(problems_host, count);
  if (!problems_host || count <= 0) return 0;
  if (count <= SAGEB200_MAX_GROUPED) {  // the plan depends on the fused producer: cover both kinds
    DeviceState fallback;
    fallback.sm_count = 148;
    DeviceState *device = nullptr;
    if (device_state(&device) != SAGEB200_OK) device = &fallback;
    for (int kind = 1; kind <= 2; ++kind) {
      const size_t bytes = grouped_scratch_bytes(problems_host, count, *device, kind);
      if (bytes && kCounterRegionBytes + bytes > grouped) grouped = kCounterRegionBytes + bytes;
    }
  }
  const int rows = problems_host[0].rows, k = problems_host[0].k;
  const size_t staged = rows > 1 ? align256(static_cast<size_t>(rows) * k * 2) : 0;
  if (!staged) return grouped;
  return (grouped ? grouped : kCounterRegionBytes) + staged;
}

int sageb200_linear_grouped_fused(const sageb200_problem *problems_host, int count,
                                  const sageb200_activation *activation, void *workspace,
                                  size_t workspace_bytes, void *stream) {
  if (!activation || activation->kind == 0)
    return sageb200_linear_grouped(problems_host, count, workspace, workspace_bytes, stream);
  if (!problems_host || count <= 0 || count > SAGEB200_MAX_GROUPED) return SAGEB200_ERR_INVALID_ARGUMENT;
  if ((activation->kind != 1 && activation->kind != 2) || !activation->a ||
      (activation->kind == 1 && (!activation->weight || !activation->residual_out)) ||
      (activation->kind == 2 && !activation->b))
    return SAGEB200_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(activation->a) & 15) || (reinterpret_cast<uintptr_t>(activation->b) & 15) ||
      (reinterpret_cast<uintptr_t>(activation->weight) & 15) ||
      (reinterpret_cast<uintptr_t>(activation->residual_out) & 15))
    return SAGEB200_ERR_ALIGNMENT;
  sageb200_problem local[SAGEB200_MAX_GROUPED];
  const int rows = problems_host[0].rows, k = problems_host[0].k;
  for (int i = 0; i < count; ++i) {
    local[i] = problems_host[i];
    local[i].x = activation->a;  // placeholder for validation; the kernels compute the row
    if (local[i].rows != rows || local[i].k != k) return SAGEB200_ERR_INVALID_ARGUMENT;
    const int status = validate_problem(local[i]);
    if (status) return status;
    if (rows > 16) return SAGEB200_ERR_RANGE;
  }
  if (rows == 0) return SAGEB200_OK;
  DeviceState *device = nullptr;
  const int status = device_state(&device);
  if (status) return status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (rows > 1) {  // the staging launch computes the producer's rows; it needs the workspace
    const size_t need = sageb200_fused_workspace_bytes(problems_host, count);
    if (!workspace || workspace_bytes < need) return SAGEB200_ERR_WORKSPACE;
    if (static_cast<size_t>(k) * 2 > kStageSharedLimit) return SAGEB200_ERR_RANGE;
  }
  return run_skinny(local, count, workspace, workspace_bytes, s, *device, activation);
}

size_t sageb200_experts_workspace_bytes(const sageb200_expert_stack *stacks_host, int stack_count,
                                        int slots) {
  if (!stacks_host || stack_count <= 0 || slots <= 0) return 0;
  sageb200_problem problems[kMaxGrouped];
  int count = 0;
  for (int s = 0; s < slots && count < kMaxGrouped; ++s)
    for (int t = 0; t < stack_count && count < kMaxGrouped; ++t) {
      problems[count] = sageb200_problem{nullptr, nullptr, nullptr, nullptr, nullptr, stacks_host[t].perm,
                                         nullptr, 1, stacks_host[t].n, stacks_host[t].k,
                                         stacks_host[t].entries};
      ++count;
    }
  return grouped_workspace_bytes(problems, count, kMaxGrouped);
}

int sageb200_experts(const void *x, long long x_slot_stride, const sageb200_expert_stack *stacks_host,
                     void *const *ys_host, int stack_count, const int32_t *expert_ids, int slots,
                     void *workspace, size_t workspace_bytes, void *stream) {
  if (!x || !stacks_host || !ys_host || !expert_ids || stack_count <= 0 || stack_count > SAGEB200_MAX_GROUPED ||
      slots < 0 || x_slot_stride < 0)
    return SAGEB200_ERR_INVALID_ARGUMENT;
  if (slots == 0) return SAGEB200_OK;
  DeviceState *device = nullptr;
  int status = device_state(&device);
  if (status) return status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int slots_per_launch = kMaxGrouped / stack_count;
  for (int begin = 0; begin < slots; begin += slots_per_launch) {
    sageb200_problem problems[kMaxGrouped];
    ExpertRef refs[kMaxGrouped];
    int count = 0;
    for (int slot = begin; slot < slots && slot < begin + slots_per_launch; ++slot)
      for (int t = 0; t < stack_count; ++t) {
        const sageb200_expert_stack &stack = stacks_host[t];
        if (stack.experts <= 0 || !ys_host[t]) return SAGEB200_ERR_INVALID_ARGUMENT;
        sageb200_problem &p = problems[count];
        p = sageb200_problem{static_cast<const __half *>(x) + slot * x_slot_stride, stack.codes, stack.radii,
                             stack.grid, stack.book, stack.perm,
                             static_cast<__half *>(ys_host[t]) + static_cast<size_t>(slot) * stack.n, 1,
                             stack.n, stack.k, stack.entries};
        status = validate_problem(p);
        if (status) return status;
        const long long tiles = (stack.n + 15) / 16, groups = stack.k / 128;
        refs[count] = ExpertRef{expert_ids, slot, stack.first_expert, stack.experts,
                                tiles * groups * 128, tiles * groups * 16, 4ll * stack.entries};
        ++count;
      }
    status = run_skinny(problems, count, workspace, workspace_bytes, s, *device, nullptr, refs);
    if (status) return status;
  }
  return SAGEB200_OK;
}

size_t sageb200_expert_blocks_workspace_bytes(const sageb200_expert_stack *stacks_host, int stack_count, int rows) {
  if (!stacks_host || stack_count <= 0 || stack_count > SAGEB200_MAX_GROUPED || rows <= 0 || rows > 16) return 0;
  sageb200_problem problems[kMaxGrouped];
  const int per_launch = kMaxGrouped / stack_count;
  int count = 0;
  for (int b = 0; b < per_launch; ++b)
    for (int t = 0; t < stack_count; ++t)
      problems[count++] = sageb200_problem{nullptr, nullptr, nullptr, nullptr, nullptr, stacks_host[t].perm, nullptr,
                                           rows, stacks_host[t].n, stacks_host[t].k, stacks_host[t].entries};
  return grouped_workspace_bytes(problems, count, kMaxGrouped);
}

int sageb200_expert_blocks(const void *x, const sageb200_expert_stack *stacks_host, void *const *ys_host,
                           int stack_count, const int32_t *block_expert_ids, int blocks, int rows, void *workspace,
                           size_t workspace_bytes, void *stream) {
  if (!x || !stacks_host || !ys_host || !block_expert_ids || stack_count <= 0 || stack_count > SAGEB200_MAX_GROUPED ||
      blocks < 0 || rows < 1 || rows > 16)
    return SAGEB200_ERR_INVALID_ARGUMENT;
  if (blocks == 0) return SAGEB200_OK;
  DeviceState *device = nullptr;
  int status = device_state(&device);
  if (status) return status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int per_launch = kMaxGrouped / stack_count;
  for (int begin = 0; begin < blocks; begin += per_launch) {
    sageb200_problem problems[kMaxGrouped];
    ExpertRef refs[kMaxGrouped];
    int count = 0;
    for (int block = begin; block < blocks && block < begin + per_launch; ++block)
      for (int t = 0; t < stack_count; ++t) {
        const sageb200_expert_stack &stack = stacks_host[t];
        if (stack.experts <= 0 || !ys_host[t]) return SAGEB200_ERR_INVALID_ARGUMENT;
        sageb200_problem &p = problems[count];
        p = sageb200_problem{static_cast<const __half *>(x) + static_cast<size_t>(block) * rows * stack.k, stack.codes,
                             stack.radii, stack.grid, stack.book, stack.perm,
                             static_cast<__half *>(ys_host[t]) + static_cast<size_t>(block) * rows * stack.n, rows,
                             stack.n, stack.k, stack.entries};
        status = validate_problem(p);
        if (status) return status;
        const long long tiles = (stack.n + 15) / 16, groups = stack.k / 128;
        refs[count] = ExpertRef{block_expert_ids, block, stack.first_expert, stack.experts,
                                tiles * groups * 128, tiles * groups * 16, 4ll * stack.entries};
        ++count;
      }
    status = run_skinny(problems, count, workspace, workspace_bytes, s, *device, nullptr, refs);
    if (status) return status;
  }
  return SAGEB200_OK;
}

/* ---------------------------------------------------------------------------------------
 * sageb200_linear_static: the decode matmul for callers that cannot hand over scratch.
 *
 * Some hosts of this library may not allocate device memory at all once serving has begun:
 * an engine whose whole memory budget was carved up at start-up, a plugin that is only ever
 * given a stream and tensor pointers by the runtime that loaded it, a request handler that
 * must not hit the device-wide synchronisation and possible out-of-memory failure of an
 * allocator call in the middle of a token.  sageb200_linear asks such callers for a
 * workspace they have no way to produce.  This entry point takes none: the partial sums,
 * arrival counters and gathered activations of the decode kernel live in the file-scope
 * device array below, which is part of the loaded library image on every GPU that uses
 * the library and stays there until the process exits.
 *
 * The array's name is only a handle on the host side; the device address is looked up
 * once per device with cudaGetSymbolAddress (with that device current) and that address
 * is what the kernels receive.
 * ------------------------------------------------------------------------------------- */
static __device__ __align__(256) unsigned char g_static_scratch[SAGEB200_STATIC_SCRATCH_BYTES];

namespace {
struct StaticScratch {
  std::atomic<int> ready{0};
  void *address = nullptr;
};
StaticScratch g_static_scratch_state[kMaxDevices];

// Device address of g_static_scratch on the current device; looked up on first use.
int static_scratch_address(void **out) {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
    cudaGetLastError();
    return SAGEB200_ERR_NO_DEVICE;
  }
  StaticScratch &state = g_static_scratch_state[device];
  if (!state.ready.load(std::memory_order_acquire)) {
    void *address = nullptr;
    if (cudaGetSymbolAddress(&address, g_static_scratch) != cudaSuccess || address == nullptr) {
      cudaGetLastError();
      return SAGEB200_ERR_CUDA;
    }
    state.address = address;
    state.ready.store(1, std::memory_order_release);
  }
  *out = state.address;
  return SAGEB200_OK;
}
}  // namespace

int sageb200_linear_static(const void *x, const void *codes, const void *radii, const void *grid,
                           const void *book, const int32_t *perm, void *y, int rows, int n, int k,
                           int entries, void *stream) {
  sageb200_problem problem{x, codes, radii, grid, book, perm, y, rows, n, k, entries};
  int status = validate_problem(problem);
  if (status) return status;
  if (rows == 0) return SAGEB200_OK;
  if (rows > 16) return SAGEB200_ERR_STATIC_SCRATCH;
  DeviceState *device = nullptr;
  status = device_state(&device);
  if (status) return status;
  if (sageb200_workspace_bytes(rows, n, k) > static_cast<size_t>(SAGEB200_STATIC_SCRATCH_BYTES))
    return SAGEB200_ERR_STATIC_SCRATCH;
  void *scratch = nullptr;
  status = static_scratch_address(&scratch);
  if (status) return status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left.  Only the arrival counters have to
  // start at zero; partial sums and gathered activations are fully rewritten before use.
  if (cudaMemsetAsync(scratch, 0, kCounterRegionBytes, s) != cudaSuccess) {
    cudaGetLastError();
    return SAGEB200_ERR_CUDA;
  }
  return run_skinny(&problem, 1, scratch, SAGEB200_STATIC_SCRATCH_BYTES, s, *device);
}

}  // extern "C"
