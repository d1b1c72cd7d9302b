// Routing front end and the sort-and-pad ("moe_align") step.
//
//  * route_topk: softmax over the expert logits, top-k selection, weights
//    renormalised over the selected experts.  One warp per token; the selection
//    is k rounds of a warp-shuffle arg-max (largest logit first, lowest expert
//    index wins ties).  The reference has no router (data.py:178-235 draws the
//    ids directly); this is the front end a caller with logits needs.
//
//  * align: stable counting sort of the flat assignment index n = token*k+kpos
//    by local expert slot, every expert segment padded to 128 rows.  It
//    reproduces the slot order of the reference's schedule builder on one rank
//    (tk_scheme.py:98-126, equal to the argsort key of tk_scheme.py:338-342)
//    and replaces the moe_align_block_size step inside fused_experts
//    (baseline.py:67).  Work is cut into contiguous "units" of assignments, one
//    warp each: per-unit warp-shuffle histograms (match.any), an exclusive scan
//    over units and experts, then a scatter that replays the same match.any
//    ranks, so the order inside an expert is ascending n whatever the grid.

#include "layer.cuh"

namespace mb200 {

namespace {

// ---------------------------------------------------------------- route_topk
constexpr int kRouteMaxPerLane = 32;  // experts <= 1024

__global__ void route_topk_kernel(const float* __restrict__ logits, int tokens, int experts,
                                  int topk, int* __restrict__ ids, float* __restrict__ weights) {
  const int warps_per_block = blockDim.x >> 5;
  const int token = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (token >= tokens) return;
  const float* row = logits + size_t(token) * experts;

  // lane l holds experts l, l+32, ... (coalesced loads)
  float v[kRouteMaxPerLane];
  const int per_lane = (experts + 31) >> 5;
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kRouteMaxPerLane; ++i) {
    if (i < per_lane) {
      int e = i * 32 + lane;
      v[i] = e < experts ? row[e] : -INFINITY;
      mx = fmaxf(mx, v[i]);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));

  float sel_sum = 0.f;
  float my_w = 0.f;   // lane j keeps the j-th selected expert's exp(logit - max)
  int my_id = 0;
  for (int j = 0; j < topk; ++j) {
    // local arg-max (lowest index first on ties: i ascending, strict >)
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kRouteMaxPerLane; ++i) {
      if (i < per_lane) {
        int e = i * 32 + lane;
        if (e < experts && (v[i] > best || (v[i] == best && e < best_e))) { best = v[i]; best_e = e; }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ob = __shfl_xor_sync(0xffffffffu, best, o);
      int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    // retire the winner
    if ((best_e & 31) == lane) {
#pragma unroll
      for (int i = 0; i < kRouteMaxPerLane; ++i)
        if (i == (best_e >> 5)) v[i] = -INFINITY;
    }
    float p = expf(best - mx);
    sel_sum += p;
    if (lane == (j & 31)) { my_w = p; my_id = best_e; }
    if ((j & 31) == 31 || j == topk - 1) {
      // flush up to 32 selections; the renormalisation needs the final sum, so
      // weights are written unnormalised here and scaled below when topk > 32
      int base = j & ~31;
      if (base + lane <= j) {
        ids[size_t(token) * topk + base + lane] = my_id;
        weights[size_t(token) * topk + base + lane] = my_w;
      }
    }
  }
  __syncwarp();
  const float inv = 1.0f / sel_sum;
  for (int j = lane; j < topk; j += 32) weights[size_t(token) * topk + j] *= inv;
}

// ---------------------------------------------------------------- align
constexpr int kAlignWarps = 8;
constexpr int kAlignThreads = kAlignWarps * 32;
constexpr int kMaxUnits = 1024;
constexpr int kFusedMaxAssignments = 8192;  // beyond this the three-kernel form is faster (about 35 us flat)
constexpr int kFusedWarps = 32;

__host__ __device__ inline int64_t unit_chunk(int64_t assignments, int units_cap) {
  int64_t chunk = (assignments + units_cap - 1) / units_cap;
  chunk = (chunk + 31) / 32 * 32;
  // a warp walks its unit 32 assignments at a time, one dependent load per step: short units
  // (more warps in flight) keep the walk from being a chain of load latencies
  return chunk < 256 ? 256 : chunk;
}

__device__ __forceinline__ int slot_of(const int* topk_ids, const int* expert_map, int64_t n,
                                       int64_t assignments, int local_experts) {
  if (n >= assignments) return -1;
  int e = __ldg(topk_ids + n);
  if (expert_map) e = (e >= 0) ? __ldg(expert_map + e) : -1;
  return (e >= 0 && e < local_experts) ? e : -1;
}

// Walk one unit in order, 32 assignments at a time.  `running[e]` counts the
// unit's assignments to expert e seen so far.  Emit(n, slot, rank) gets the rank
// of assignment n among the unit's assignments to the same expert.
template <class Emit>
__device__ __forceinline__ void walk_unit(const int* topk_ids, const int* expert_map,
                                          int64_t begin, int64_t end, int64_t assignments,
                                          int local_experts, int* running, Emit emit) {
  const int lane = threadIdx.x & 31;
  for (int64_t base = begin; base < end; base += 32) {
    const int64_t n = base + lane;
    const int slot = (n < end) ? slot_of(topk_ids, expert_map, n, assignments, local_experts) : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, slot);
    if (slot >= 0) {
      const int before = __popc(peers & ((1u << lane) - 1u));
      const int seen = running[slot];
      emit(n, slot, seen + before);
    } else if (n < assignments && n < end) {
      emit(n, -1, 0);
    }
    __syncwarp();
    if (slot >= 0 && (peers & ((1u << lane) - 1u)) == 0) running[slot] += __popc(peers);
    __syncwarp();
  }
}

__global__ void align_count_kernel(const int* __restrict__ topk_ids, const int* __restrict__ expert_map,
                                   int64_t assignments, int local_experts, int64_t chunk, int units,
                                   int* __restrict__ unit_hist) {
  extern __shared__ int hist_smem[];
  const int warp = threadIdx.x >> 5;
  const int unit = blockIdx.x * kAlignWarps + warp;
  int* running = hist_smem + warp * local_experts;
  for (int e = threadIdx.x & 31; e < local_experts; e += 32) running[e] = 0;
  __syncwarp();
  if (unit >= units) return;
  const int64_t begin = int64_t(unit) * chunk;
  const int64_t end = begin + chunk < assignments ? begin + chunk : assignments;
  walk_unit(topk_ids, expert_map, begin, end, assignments, local_experts, running,
            [](int64_t, int, int) {});
  for (int e = threadIdx.x & 31; e < local_experts; e += 32)
    unit_hist[size_t(unit) * local_experts + e] = running[e];
}

// One block.  unit_hist[u][e] becomes the exclusive prefix over units; counts and
// the cumulative M-tile table are written.  The block's threads form up to 32 groups
// of E threads (thread = one expert, consecutive threads = consecutive experts, so
// every load is a coalesced row segment); each group scans a contiguous range of
// units in two passes: range sums into `part` ([groups][E] ints of shared memory,
// at most blockDim.x), then the prefix starting from the sums of the groups before it.
constexpr int kScanMaxGroups = 32;

__device__ void scan_units_and_experts(int* unit_hist, int units, int local_experts, int* counts,
                                       int* mtile_prefix, int* smem_tiles /*[E+1]*/, int* part, int pad) {
  const int E = local_experts;
  int groups = E < int(blockDim.x) ? int(blockDim.x) / E : 1;
  if (groups > kScanMaxGroups) groups = kScanMaxGroups;
  const int per_group = (units + groups - 1) / groups;
  for (int e0 = 0; e0 < E; e0 += blockDim.x) {  // one trip unless E exceeds the block
    const int g = groups > 1 ? int(threadIdx.x) / E : 0;
    const int e = e0 + (groups > 1 ? int(threadIdx.x) % E : int(threadIdx.x));
    const bool active = e < E && g < groups;
    const int u_lo = g * per_group < units ? g * per_group : units;
    const int u_hi = u_lo + per_group < units ? u_lo + per_group : units;
    int run = 0;
    if (groups > 1) {
      if (active) {
        int sum = 0;
        for (int u0 = u_lo; u0 < u_hi; u0 += 8) {
          int v[8];  // loads first, so eight of them are in flight together
#pragma unroll
          for (int i = 0; i < 8; ++i)
            v[i] = (u0 + i < u_hi) ? unit_hist[size_t(u0 + i) * E + e] : 0;
#pragma unroll
          for (int i = 0; i < 8; ++i) sum += v[i];
        }
        part[g * E + e] = sum;
      }
      __syncthreads();
      if (active)
        for (int w = 0; w < g; ++w) run += part[w * E + e];
    }
    if (active) {
      for (int u0 = u_lo; u0 < u_hi; u0 += 8) {
        int v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          v[i] = (u0 + i < u_hi) ? unit_hist[size_t(u0 + i) * E + e] : 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (u0 + i < u_hi) unit_hist[size_t(u0 + i) * E + e] = run;
          run += v[i];
        }
      }
      if (g == groups - 1) {  // the last group's running sum is the expert's total
        counts[e] = run;
        smem_tiles[e] = (run + pad - 1) / pad;
      }
    }
    if (groups > 1) __syncthreads();  // `part` is reused by the next trip
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    // warp scan: each lane owns a contiguous run of experts
    const int lane = threadIdx.x;
    const int per = (local_experts + 31) / 32;
    const int lo = lane * per;
    const int hi = lo + per < local_experts ? lo + per : local_experts;
    int sum = 0;
    for (int e = lo; e < hi; ++e) sum += smem_tiles[e];
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    int run = incl - sum;
    for (int e = lo; e < hi; ++e) {
      int t = smem_tiles[e];
      mtile_prefix[e] = run;
      run += t;
    }
    if (lane == 31) mtile_prefix[local_experts] = incl;
  }
}

__global__ void align_scan_kernel(int* unit_hist, int units, int local_experts, int* counts,
                                  int* mtile_prefix, int pad) {
  extern __shared__ int tiles_smem[];  // [E+1] tiles per expert, then [blockDim.x] partial sums
  scan_units_and_experts(unit_hist, units, local_experts, counts, mtile_prefix, tiles_smem,
                         tiles_smem + (local_experts + 1), pad);
}

// Mark the padding rows of expert e with -1; `lane`/`width` are the caller's
// position in the group of threads that shares the expert.
__device__ __forceinline__ void fill_padding(const int* counts, const int* mtile_prefix, int e,
                                             int* sorted_ids, int64_t row_capacity, int lane, int width,
                                             int pad) {
  const int64_t begin = int64_t(mtile_prefix[e]) * pad + counts[e];
  int64_t end = int64_t(mtile_prefix[e + 1]) * pad;
  if (end > row_capacity) end = row_capacity;
  for (int64_t p = begin + lane; p < end; p += width) sorted_ids[p] = -1;
}

__global__ void align_scatter_kernel(const int* __restrict__ topk_ids, const int* __restrict__ expert_map,
                                     int64_t assignments, int local_experts, int64_t chunk, int units,
                                     const int* __restrict__ unit_base, const int* __restrict__ counts,
                                     const int* __restrict__ mtile_prefix, int* __restrict__ sorted_ids,
                                     int* __restrict__ inverse, int64_t row_capacity, int pad) {
  extern __shared__ int hist_smem[];
  // one warp per expert, experts strided over every warp of the grid
  for (int e = blockIdx.x * kAlignWarps + (threadIdx.x >> 5); e < local_experts; e += gridDim.x * kAlignWarps)
    fill_padding(counts, mtile_prefix, e, sorted_ids, row_capacity, threadIdx.x & 31, 32, pad);

  const int warp = threadIdx.x >> 5;
  const int unit = blockIdx.x * kAlignWarps + warp;
  int* running = hist_smem + warp * local_experts;
  for (int e = threadIdx.x & 31; e < local_experts; e += 32) running[e] = 0;
  __syncwarp();
  if (unit >= units) return;
  const int64_t begin = int64_t(unit) * chunk;
  const int64_t end = begin + chunk < assignments ? begin + chunk : assignments;
  const int* base = unit_base + size_t(unit) * local_experts;
  walk_unit(topk_ids, expert_map, begin, end, assignments, local_experts, running,
            [&](int64_t n, int slot, int rank) {
              if (slot < 0) { inverse[n] = -1; return; }
              const int64_t row = int64_t(mtile_prefix[slot]) * pad + base[slot] + rank;
              if (row < row_capacity) sorted_ids[row] = int(n);
              inverse[n] = int(row);
            });
}

// Whole step in one block of 32 warps (small problems: one launch instead of three).
__global__ void __launch_bounds__(kFusedWarps * 32)
align_fused_kernel(const int* __restrict__ topk_ids, const int* __restrict__ expert_map,
                   int64_t assignments, int local_experts, int* __restrict__ counts,
                   int* __restrict__ mtile_prefix, int* __restrict__ sorted_ids,
                   int* __restrict__ inverse, int64_t row_capacity, int* __restrict__ unit_hist, int pad) {
  extern __shared__ int smem[];
  int* tiles_smem = smem;                              // [E+1]
  int* running_all = smem + (local_experts + 1);       // [32][E]
  const int warp = threadIdx.x >> 5;
  int64_t chunk = (assignments + kFusedWarps - 1) / kFusedWarps;
  chunk = (chunk + 31) / 32 * 32;
  const int64_t begin = warp * chunk < assignments ? warp * chunk : assignments;
  const int64_t end = begin + chunk < assignments ? begin + chunk : assignments;
  int* running = running_all + warp * local_experts;

  for (int e = threadIdx.x & 31; e < local_experts; e += 32) running[e] = 0;
  __syncwarp();
  walk_unit(topk_ids, expert_map, begin, end, assignments, local_experts, running,
            [](int64_t, int, int) {});
  for (int e = threadIdx.x & 31; e < local_experts; e += 32)
    unit_hist[size_t(warp) * local_experts + e] = running[e];
  __syncthreads();
  // the per-warp counters are free between the two walks and serve as the scan's partial sums
  scan_units_and_experts(unit_hist, kFusedWarps, local_experts, counts, mtile_prefix, tiles_smem,
                         running_all, pad);
  __syncthreads();
  for (int e = warp; e < local_experts; e += kFusedWarps)
    fill_padding(counts, mtile_prefix, e, sorted_ids, row_capacity, threadIdx.x & 31, 32, pad);
  for (int e = threadIdx.x & 31; e < local_experts; e += 32) running[e] = 0;
  __syncwarp();
  const int* base = unit_hist + size_t(warp) * local_experts;
  walk_unit(topk_ids, expert_map, begin, end, assignments, local_experts, running,
            [&](int64_t n, int slot, int rank) {
              if (slot < 0) { inverse[n] = -1; return; }
              const int64_t row = int64_t(mtile_prefix[slot]) * pad + base[slot] + rank;
              if (row < row_capacity) sorted_ids[row] = int(n);
              inverse[n] = int(row);
            });
}

}  // namespace

int launch_route_topk(const float* logits, int tokens, int experts, int topk, int* ids,
                      float* weights, cudaStream_t stream) {
  MB200_REQUIRE(experts >= 1 && experts <= 32 * kRouteMaxPerLane, kUnsupportedShape,
                "route_topk: %d experts, supported 1..%d", experts, 32 * kRouteMaxPerLane);
  MB200_REQUIRE(topk >= 1 && topk <= experts, kInvalidArgument, "route_topk: topk=%d with %d experts",
                topk, experts);
  if (tokens == 0) return kOk;
  const int warps = 4;
  route_topk_kernel<<<(tokens + warps - 1) / warps, warps * 32, 0, stream>>>(logits, tokens, experts,
                                                                              topk, ids, weights);
  MB200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

int64_t align_scratch_ints(int64_t assignments, int experts) {
  int64_t units = kMaxUnits;
  (void)assignments;
  return units * experts;
}

int launch_align(const int* topk_ids, int64_t assignments, const int* expert_map, int local_experts,
                 Schedule sched, int64_t row_capacity, int* scratch, cudaStream_t stream) {
  MB200_REQUIRE(local_experts >= 1 && local_experts <= kMaxExperts, kUnsupportedShape,
                "align: %d local experts, supported 1..%d", local_experts, kMaxExperts);
  MB200_REQUIRE(assignments >= 0 && assignments < (int64_t(1) << 31) - 4096, kUnsupportedShape,
                "align: %lld assignments do not fit 32-bit row indices", (long long)assignments);
  const int pad = sched.pad_rows;
  MB200_REQUIRE(pad >= 1 && pad <= 1024, kInvalidArgument, "align: pad_rows=%d (1..1024)", pad);
  const size_t fused_smem = size_t(local_experts + 1 + kFusedWarps * local_experts) * sizeof(int);
  if (assignments <= kFusedMaxAssignments && fused_smem <= 48 * 1024) {
    align_fused_kernel<<<1, kFusedWarps * 32, fused_smem, stream>>>(
        topk_ids, expert_map, assignments, local_experts, sched.counts, sched.mtile_prefix,
        sched.sorted_ids, sched.inverse, row_capacity, scratch, pad);
    MB200_CHECK_CUDA(cudaGetLastError());
    return kOk;
  }
  const int64_t chunk = unit_chunk(assignments, kMaxUnits);
  const int units = int((assignments + chunk - 1) / chunk);
  const int blocks = (units + kAlignWarps - 1) / kAlignWarps;
  const size_t hist_smem = size_t(kAlignWarps) * local_experts * sizeof(int);
  if (blocks > 0) {
    align_count_kernel<<<blocks, kAlignThreads, hist_smem, stream>>>(
        topk_ids, expert_map, assignments, local_experts, chunk, units, scratch);
    MB200_CHECK_CUDA(cudaGetLastError());
  }
  align_scan_kernel<<<1, 1024, size_t(local_experts + 1 + 1024) * sizeof(int), stream>>>(
      scratch, units, local_experts, sched.counts, sched.mtile_prefix, pad);
  MB200_CHECK_CUDA(cudaGetLastError());
  const int sblocks = blocks > 0 ? blocks : 1;
  align_scatter_kernel<<<sblocks, kAlignThreads, hist_smem, stream>>>(
      topk_ids, expert_map, assignments, local_experts, chunk, units, scratch, sched.counts,
      sched.mtile_prefix, sched.sorted_ids, sched.inverse, row_capacity, pad);
  MB200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

}  // namespace mb200

// ---------------------------------------------------------------------------
// Sort-and-pad without caller-provided scratch.
//
// Some hosts of this library must not allocate device memory once they are
// running: an inference server that handed (nearly) all HBM to its own pool at
// start-up has nothing left for a later cudaMalloc, and inside a latency-
// critical decode loop cudaMalloc/cudaFree would stall the whole device.  For
// them the unit histograms of the sort live in the fixed array below instead of
// a buffer the caller allocates.  The price: 1 MiB of every GPU that loads the
// library is held until the process exits, the problem size is capped, and all
// calls on a device share the one array.
// ---------------------------------------------------------------------------
#include <mutex>

#include "../../include/moe_bench_b200.h"

namespace mb200 {
namespace {

constexpr int kNoAllocMaxExperts = MB200_NOALLOC_MAX_LOCAL_EXPERTS;          // 256
constexpr int64_t kNoAllocMaxAssignments = MB200_NOALLOC_MAX_ASSIGNMENTS;    // 2^20
// units (<= 1024) x experts (<= 256) histogram entries = 1 MiB
static __device__ __align__(256) int g_noalloc_align_scratch[kMaxUnits * kNoAllocMaxExperts];

constexpr int kNoAllocMaxDevices = 64;
std::mutex g_noalloc_mutex;
int* g_noalloc_scratch_ptr[kNoAllocMaxDevices] = {};

// Device address of the array on the CURRENT device, looked up once per device.
// In host code the array's name is only a handle for the runtime, never an
// address a kernel may use, hence cudaGetSymbolAddress.
int noalloc_scratch(int** out) {
  int dev = -1;
  MB200_CHECK_CUDA(cudaGetDevice(&dev));
  MB200_REQUIRE(dev >= 0 && dev < kNoAllocMaxDevices, kUnsupportedShape,
                "align_noalloc: device index %d, supported 0..%d", dev, kNoAllocMaxDevices - 1);
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_scratch_ptr[dev]) {
    void* p = nullptr;
    MB200_CHECK_CUDA(cudaGetSymbolAddress(&p, g_noalloc_align_scratch));
    g_noalloc_scratch_ptr[dev] = static_cast<int*>(p);
  }
  *out = g_noalloc_scratch_ptr[dev];
  return kOk;
}

}  // namespace
}  // namespace mb200

extern "C" int mb200_align_noalloc(const int32_t* topk_ids, int64_t tokens, int topk,
                                   const int32_t* expert_map, int local_experts, int32_t* counts,
                                   int32_t* mtile_prefix, int32_t* sorted_ids, int32_t* inverse,
                                   int64_t row_capacity, int pad_rows, void* stream) {
  using namespace mb200;
  MB200_REQUIRE(pad_rows >= 1 && pad_rows <= 1024, kInvalidArgument, "align_noalloc: pad_rows=%d", pad_rows);
  MB200_REQUIRE(tokens >= 0 && topk >= 1, kInvalidArgument, "align_noalloc: tokens=%lld topk=%d",
                (long long)tokens, topk);
  MB200_REQUIRE(local_experts >= 1 && local_experts <= kNoAllocMaxExperts, kUnsupportedShape,
                "align_noalloc: %d local experts exceed the built-in scratch (at most %d); "
                "use mb200_align with a caller-provided scratch buffer",
                local_experts, kNoAllocMaxExperts);
  // compared before multiplying: tokens * topk must not wrap around on its way to the limit check
  const int64_t assignments = tokens <= kNoAllocMaxAssignments / topk ? tokens * topk : kNoAllocMaxAssignments + 1;
  MB200_REQUIRE(assignments <= kNoAllocMaxAssignments, kUnsupportedShape,
                "align_noalloc: %lld assignments exceed the built-in scratch (at most %lld); "
                "use mb200_align with a caller-provided scratch buffer",
                (long long)assignments, (long long)kNoAllocMaxAssignments);
  MB200_REQUIRE(counts && mtile_prefix && sorted_ids && (tokens == 0 || (topk_ids && inverse)),
                kInvalidArgument, "align_noalloc: null pointer");
  const int64_t touched = assignments < local_experts ? assignments : local_experts;
  const int64_t need = (assignments + touched * (pad_rows - 1) + pad_rows - 1) / pad_rows * pad_rows;
  MB200_REQUIRE(row_capacity >= need, kWorkspaceTooSmall, "align_noalloc: row capacity %lld < %lld",
                (long long)row_capacity, (long long)need);
  int* scratch = nullptr;
  int rc = noalloc_scratch(&scratch);
  if (rc) return rc;
  // Every histogram entry a launch reads is written earlier by the same launch
  // sequence, so nothing left over from the previous call has to be cleared.
  Schedule s{counts, mtile_prefix, sorted_ids, inverse, pad_rows};
  return launch_align(topk_ids, assignments, expert_map, local_experts, s, row_capacity, scratch,
                      reinterpret_cast<cudaStream_t>(stream));
}
