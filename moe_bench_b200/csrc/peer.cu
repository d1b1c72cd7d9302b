// Cross-GPU kernels of the distributed layer that run outside the GEMMs (one
// process per GPU, peers' buffers mapped into this process: plain 64-bit
// pointers over NVLink).  The bulk of the traffic does not pass through this
// file: the dispatch pulls run in helper warps of the gate/up GEMM kernels and
// the combine pushes in helper warps of the down GEMM kernels
// (grouped_gemm.cu, grouped_gemm_fp8.cu); the tensor-parallel sum-and-push is
// in rows.cu.  Ranks meet at the barrier kernel, whose spin is bounded.
//
//   peer_barrier      every rank writes a monotonic sequence number into its slot
//                     of every peer's flag array (st.release.sys after a system
//                     fence) and polls its own array (ld.acquire.sys), the
//                     protocol of the reference's pcie_barrier_all
//                     (kernels/tileoverlap/common/sm120_common.cuh:47-64), with a
//                     time limit and a status word instead of an endless spin.
//   gather_routing    all ranks' topk ids / weights -> one local array in ring
//                     order (own rank first), replacing the two small
//                     all-gathers of schemes.py:122-127 / tk_scheme.py:682-683.
//   gather_rows_fp8   EP dispatch for fp8 with few rows per expert (the
//                     tokens-on-columns kernels have no helper warps; replaces
//                     the all-gather of schemes.py:121): the expert rank pulls
//                     the token rows routed to its experts straight into its
//                     sorted, padded row buffer - e4m3 rows plus their 1x128
//                     scales (fp8 on the wire).
//   gather_blocks     TP: every rank's staged token block, pulled once.
//   reduce_partials   combine of that same few-rows fp8 path (replaces the
//                     reduce-scatter of schemes.py:142): every expert rank has
//                     pre-reduced the contributions of a token that landed on it
//                     into one row; the token's own rank pulls the <= W rows
//                     that exist and sums them in fp32 in rank order.

#include "layer.cuh"

namespace mb200 {

namespace {

// Default limit of the all-rank barrier; word 2 of the status block (milliseconds, 0 = default)
// overrides it, for hosts whose ranks may reach a barrier further apart (a first call that
// still loads modules, a stalled host thread).
constexpr uint64_t kBarrierLimitNs = 3ull * 1000 * 1000 * 1000;
constexpr int kGatherLoads = 7;  // 16-byte loads a lane of the row gather keeps in flight

__global__ void peer_barrier_kernel(PeerTable flags, int rank, int world, uint32_t seq, int* status) {
  const int peer = threadIdx.x;
  if (peer >= world) return;
  // make this GPU's earlier writes visible system-wide before the flag
  __threadfence_system();
  uint32_t* remote = reinterpret_cast<uint32_t*>(flags.ptr[peer]) + rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(seq) : "memory");
  const uint32_t* mine = reinterpret_cast<const uint32_t*>(flags.ptr[rank]) + peer;
  const int limit_ms = status ? status[2] : 0;
  const uint64_t limit_ns = limit_ms > 0 ? uint64_t(limit_ms) * 1000000ull : kBarrierLimitNs;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (int32_t(v - seq) >= 0) break;  // monotonic, wrap-safe
    if ((++spins & 0xFF) == 0) {
      if (global_timer_ns() - t0 > limit_ns) {
        if (status) atomicCAS(status, 0, kDevWaitTimeout + 50 + peer);
        break;
      }
      __nanosleep(64);
    }
  }
  __threadfence_system();
}

// ids_all[ring][t][j] = ids of rank (rank + ring) % world; same for weights.
__global__ void gather_routing_kernel(PeerTable ids, PeerTable weights, int rank, int world,
                                      int per_rank, int* __restrict__ ids_all,
                                      float* __restrict__ weights_all) {
  const int64_t total = int64_t(world) * per_rank;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * blockDim.x) {
    const int ring = int(i / per_rank);
    const int off = int(i - int64_t(ring) * per_rank);
    const int src = (rank + ring) % world;
    ids_all[i] = reinterpret_cast<const int*>(ids.ptr[src])[off];
    weights_all[i] = reinterpret_cast<const float*>(weights.ptr[src])[off];
  }
}

// Tensor parallel: every rank's staged block (tokens, or their scales) pulled once
// into one local array in ring order.  `vec_per_rank` counts 16-byte vectors.
__global__ void gather_blocks_peer_kernel(PeerTable src, int rank, int world, int64_t vec_per_rank,
                                          uint4* __restrict__ dst) {
  const int64_t total = vec_per_rank * world;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * blockDim.x) {
    const int ring = int(i / vec_per_rank);
    const int64_t off = i - int64_t(ring) * vec_per_rank;
    dst[i] = reinterpret_cast<const uint4*>(src.ptr[(rank + ring) % world])[off];
  }
}

// Sorted rows pulled from the source ranks.  n = (ring*T + t)*k + j.
// e4m3 rows + their scales ([T][K/128] at the source) -> sorted rows + group-major scales.
__global__ void gather_rows_peer_fp8_kernel(PeerTable xq, PeerTable xs, int rank, int world, int tokens,
                                            int topk, const int* __restrict__ sorted_ids,
                                            const int* __restrict__ mtile_prefix, int local_experts,
                                            int groups_per_row, uint4* __restrict__ out_q,
                                            float* __restrict__ out_scales_t, int64_t row_capacity, int pad) {
  int64_t rows = int64_t(__ldg(mtile_prefix + local_experts)) * pad;
  if (rows > row_capacity) rows = row_capacity;
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int vec_per_row = groups_per_row * 8;  // 128 bytes per group = 8 x 16 bytes
  for (int64_t row = int64_t(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); row < rows;
       row += int64_t(gridDim.x) * warps_per_block) {
    const int n = __ldg(sorted_ids + row);
    if (n < 0) continue;
    const int tok_global = n / topk;
    const int ring = tok_global / tokens;
    const int t = tok_global - ring * tokens;
    const int src_rank = (rank + ring) % world;
    const uint4* src = reinterpret_cast<const uint4*>(xq.ptr[src_rank]) + int64_t(t) * vec_per_row;
    const float* src_s = reinterpret_cast<const float*>(xs.ptr[src_rank]) + int64_t(t) * groups_per_row;
    uint4* dst = out_q + row * vec_per_row;
    // kGatherLoads 16-byte loads in flight per lane (a load over NVLink takes microseconds)
    for (int v0 = lane; v0 < vec_per_row; v0 += 32 * kGatherLoads) {
      uint4 buf[kGatherLoads];
#pragma unroll
      for (int u = 0; u < kGatherLoads; ++u)
        if (v0 + u * 32 < vec_per_row) buf[u] = src[v0 + u * 32];
#pragma unroll
      for (int u = 0; u < kGatherLoads; ++u)
        if (v0 + u * 32 < vec_per_row) dst[v0 + u * 32] = buf[u];
    }
    for (int g = lane; g < groups_per_row; g += 32) out_scales_t[int64_t(g) * row_capacity + row] = src_s[g];
  }
}

// out[t] = sum over ranks p (ascending) of partial_p[ring(p)*T + t], ring(p) =
// (rank - p) mod world.  experts_per_rank > 0 (EP): only ranks that own one of
// the token's experts are read; 0 (TP): every rank contributes.
__global__ void reduce_partials_kernel(PeerTable partial, int rank, int world, int tokens, int topk,
                                       const int* __restrict__ topk_ids, int experts_per_rank,
                                       int vec_per_row, uint4* __restrict__ out, int fp16) {
  const int64_t total = int64_t(tokens) * vec_per_row;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * blockDim.x) {
    const int t = int(i / vec_per_row);
    const int v = int(i - int64_t(t) * vec_per_row);
    unsigned owners = 0xffffffffu;
    if (experts_per_rank > 0) {
      owners = 0;
      for (int j = 0; j < topk; ++j) {
        const int e = __ldg(topk_ids + int64_t(t) * topk + j);
        if (e >= 0) owners |= 1u << (e / experts_per_rank);
      }
    }
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    // up to 8 peer loads in flight per thread (an NVLink round trip each), summed in ascending p
    for (int p0 = 0; p0 < world; p0 += 8) {
      uint4 val[8];
      bool have[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int p = p0 + u;
        have[u] = p < world && ((owners >> p) & 1u);
        if (have[u]) {
          const int ring = (rank - p + world) % world;
          val[u] = *(reinterpret_cast<const uint4*>(partial.ptr[p]) +
                     (int64_t(ring) * tokens + t) * vec_per_row + v);
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (have[u]) add_h16x8(val[u], acc, fp16);
    }
    out[i] = pack_h16x8(acc, fp16);
  }
}

int grid_for_rows(int64_t items, int threads, int waves) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess && device_sm_count(dev) > 0) sms = device_sm_count(dev);
  int64_t blocks = (items + threads - 1) / threads;
  const int64_t cap = int64_t(sms) * waves;
  if (blocks > cap) blocks = cap;
  return blocks < 1 ? 1 : int(blocks);
}

}  // namespace

int launch_peer_barrier(const PeerTable& flags, int rank, int world, uint32_t seq, int* status,
                        cudaStream_t stream) {
  MB200_REQUIRE(world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world, kInvalidArgument,
                "peer_barrier: rank %d of %d (at most %d ranks)", rank, world, kMaxPeers);
  peer_barrier_kernel<<<1, 32, 0, stream>>>(flags, rank, world, seq, status);
  MB200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

int launch_gather_routing(const PeerTable& ids, const PeerTable& weights, int rank, int world, int per_rank,
                          int* ids_all, float* weights_all, cudaStream_t stream) {
  const int threads = 256;
  gather_routing_kernel<<<grid_for_rows(int64_t(world) * per_rank, threads, 4), threads, 0, stream>>>(
      ids, weights, rank, world, per_rank, ids_all, weights_all);
  MB200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

int launch_gather_blocks_peer(const PeerTable& src, int rank, int world, int64_t bytes_per_rank, void* dst,
                              cudaStream_t stream) {
  MB200_REQUIRE(bytes_per_rank % 16 == 0, kUnsupportedShape, "gather_blocks: %lld bytes per rank is not a multiple of 16",
                (long long)bytes_per_rank);
  if (bytes_per_rank == 0) return kOk;
  const int threads = 256;
  gather_blocks_peer_kernel<<<grid_for_rows(bytes_per_rank / 16 * world, threads, 16), threads, 0, stream>>>(
      src, rank, world, bytes_per_rank / 16, reinterpret_cast<uint4*>(dst));
  MB200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

int launch_gather_rows_peer_fp8(const PeerTable& x, const PeerTable& xs, int rank, int world, int tokens, int topk,
                                const Schedule& sched, int local_experts, int hidden, void* out_rows,
                                float* out_scales_t, int64_t row_capacity, cudaStream_t stream) {
  const int threads = 256;
  const int blocks = grid_for_rows(row_capacity * 32, threads, 16);
  MB200_REQUIRE(hidden % 128 == 0, kUnsupportedShape, "dispatch: hidden=%d must be a multiple of 128", hidden);
  gather_rows_peer_fp8_kernel<<<blocks, threads, 0, stream>>>(
      x, xs, rank, world, tokens, topk, sched.sorted_ids, sched.mtile_prefix, local_experts, hidden / 128,
      reinterpret_cast<uint4*>(out_rows), out_scales_t, row_capacity, sched.pad_rows);
  MB200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

int launch_reduce_partials(const PeerTable& partial, int rank, int world, int tokens, int topk,
                           const int* topk_ids, int experts_per_rank, int hidden, __nv_bfloat16* out,
                           cudaStream_t stream, int fp16) {
  MB200_REQUIRE(hidden % 8 == 0, kUnsupportedShape, "reduce: hidden=%d must be a multiple of 8", hidden);
  const int threads = 256;
  reduce_partials_kernel<<<grid_for_rows(int64_t(tokens) * (hidden / 8), threads, 16), threads, 0, stream>>>(
      partial, rank, world, tokens, topk, topk_ids, experts_per_rank, hidden / 8, reinterpret_cast<uint4*>(out), fp16);
  MB200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

}  // namespace mb200
