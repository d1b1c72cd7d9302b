// Distributed layer forward: expert parallel (EP) and tensor parallel (TP) over
// the GPUs of one NVLink box, one process per GPU.  Declared in
// include/moe_bench_b200.h; replaces the AllGather -> fused_experts ->
// ReduceScatter dataflow of the reference's serial scheme (schemes.py:117-143).
//
// Every rank owns a "symmetric" buffer of identical layout that all peers have
// mapped (flags | routing | token payload | partial planes | received rows).
// One expert-parallel forward:
//   1. stage: own routing and tokens into the symmetric buffer (fp8: quantised to
//      e4m3 + 1x128 scales first, so fp8 travels on the wire);
//   2. barrier;
//   3. routing of all ranks -> ring-ordered local copy; sort-and-pad against this
//      rank's experts;
//   4. gate/up GEMM whose helper warps pull the needed rows from their owners,
//      granule by granule, while the tiles compute (the dispatch); down GEMM whose
//      helper warps push every finished weighted row of another rank's token into
//      that rank's receive buffer (the combine);
//   5. barrier; the token's own rank sums its k received rows.
// Tensor parallel gathers the peers' token blocks once, runs the GEMMs on its slice
// of the intermediate dimension, sums a token's k rows and pushes the sum into the
// owner's plane, barrier, the owner sums its W planes.  fp8 with few rows per expert
// (tokens-on-columns kernels, no helper warps) keeps separate gather, pre-reduce
// and pull-reduce kernels with a third barrier.

#include "../../include/moe_bench_b200.h"
#include <cstring>

#include "layer.cuh"

namespace mb200 {
namespace {

int64_t up1k(int64_t v) { return (v + 1023) / 1024 * 1024; }

struct SymLayout {
  int64_t flags, ids, weights, payload, payload_scales, partial, yrecv, total;
};

SymLayout make_sym_layout(int precision, int64_t tokens, int hidden, int topk, int world) {
  SymLayout l;
  int64_t off = 0;
  auto take = [&](int64_t bytes) { int64_t o = off; off = up1k(off + bytes); return o; };
  l.flags = take(1024);
  l.ids = take(tokens * topk * 4);
  l.weights = take(tokens * topk * 4);
  l.payload = take(tokens * hidden * (precision == MB200_PRECISION_FP8 ? 1 : 2));
  l.payload_scales = take(precision == MB200_PRECISION_FP8 ? tokens * (hidden / 128) * 4 : 0);
  l.partial = take(int64_t(world) * tokens * hidden * 2);
  // expert parallel with the fused combine push: one weighted row per assignment of this
  // rank's tokens, written by whichever rank owns the expert
  l.yrecv = take(tokens * topk * hidden * 2);
  l.total = off;
  return l;
}

PeerTable offset_table(void* const* bases, int world, int64_t off) {
  PeerTable t{};
  for (int i = 0; i < world; ++i) t.ptr[i] = static_cast<char*>(bases[i]) + off;
  return t;
}

}  // namespace
}  // namespace mb200

using namespace mb200;

extern "C" {

int64_t mb200_dist_symmetric_bytes(int precision, int64_t tokens, int hidden, int topk, int world) {
  if (tokens < 0 || hidden <= 0 || topk < 1 || world < 1 || world > kMaxPeers) return -1;
  return make_sym_layout(precision, tokens, hidden, topk, world).total;
}

int64_t mb200_dist_workspace_bytes(int precision, int64_t tokens, int hidden, int intermediate,
                                   int local_experts, int topk, int world) {
  if (world < 1 || world > kMaxPeers) return -1;
  if (check_shape(tokens * world, hidden, intermediate, local_experts, topk)) return -1;
  if (precision == MB200_PRECISION_FP8 && check_shape_fp8(hidden, intermediate)) return -1;
  const Layout l = make_layout(precision, tokens * world, hidden, intermediate, local_experts, topk,
                               pad_rows_of(precision));
  // + ring-ordered routing of all ranks + (tensor parallel) every rank's staged tokens and scales
  const int64_t eb = precision == MB200_PRECISION_FP8 ? 1 : 2;
  return l.total + 2 * up1k(tokens * world * topk * 4) + up1k(tokens * world * hidden * eb) +
         up1k(tokens * world * (hidden / 128) * 4);
}

int mb200_peer_barrier(void* const* symmetric_ptrs, int rank, int world, uint32_t seq, int32_t* status,
                       void* stream) {
  MB200_REQUIRE(symmetric_ptrs && world >= 1 && world <= kMaxPeers, kInvalidArgument, "peer_barrier: bad argument");
  return launch_peer_barrier(offset_table(symmetric_ptrs, world, 0), rank, world, seq, status,
                             reinterpret_cast<cudaStream_t>(stream));
}

int mb200_dist_forward(int precision, int expert_parallel, const void* hidden_states, const void* w1,
                       const void* w2, const float* w1_scale, const float* w2_scale,
                       const int32_t* topk_ids, const float* topk_weights, const int32_t* expert_map,
                       void* out, int64_t tokens, int hidden, int intermediate, int local_experts,
                       int global_experts, int topk, int rank, int world, void* const* symmetric_ptrs,
                       int64_t symmetric_bytes, uint32_t seq_base, void* workspace, int64_t workspace_bytes,
                       int device, void* stream) {
  MB200_REQUIRE(precision == MB200_PRECISION_BF16 || precision == MB200_PRECISION_FP8 ||
                    precision == MB200_PRECISION_FP16,
                kInvalidArgument, "dist_forward: unknown precision %d", precision);
  const int fp16 = precision == MB200_PRECISION_FP16;
  MB200_REQUIRE(world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world, kInvalidArgument,
                "dist_forward: rank %d of %d (at most %d ranks)", rank, world, kMaxPeers);
  const bool fp8 = precision == MB200_PRECISION_FP8;
  const int64_t all_tokens = tokens * world;
  int rc = check_shape(all_tokens, hidden, intermediate, local_experts, topk);
  if (rc) return rc;
  if (fp8 && (rc = check_shape_fp8(hidden, intermediate))) return rc;
  MB200_REQUIRE(tokens > 0, kInvalidArgument, "dist_forward: every rank needs at least one token");
  MB200_REQUIRE(hidden_states && w1 && w2 && topk_ids && topk_weights && out && workspace && symmetric_ptrs,
                kInvalidArgument, "dist_forward: null pointer");
  MB200_REQUIRE(!fp8 || (w1_scale && w2_scale), kInvalidArgument, "dist_forward: fp8 needs weight scales");
  if (expert_parallel) {
    MB200_REQUIRE(expert_map != nullptr, kInvalidArgument, "dist_forward: expert parallel needs expert_map");
    MB200_REQUIRE(global_experts == local_experts * world, kInvalidArgument,
                  "dist_forward: %d global experts != %d local x %d ranks", global_experts, local_experts, world);
  }
  const SymLayout sl = make_sym_layout(precision, tokens, hidden, topk, world);
  MB200_REQUIRE(symmetric_bytes >= sl.total, kWorkspaceTooSmall, "dist_forward: symmetric buffer %lld < %lld bytes",
                (long long)symmetric_bytes, (long long)sl.total);
  // fp8 with few rows per expert: 16-row padding and the tokens-on-columns kernels
  const int64_t expected_local = expert_parallel ? all_tokens * topk / world : all_tokens * topk;
  const int pad = fp8 ? fp8_pad_rows(expected_local, local_experts) : kPadBf16;
  const Layout l = make_layout(precision, all_tokens, hidden, intermediate, local_experts, topk, pad);
  const int64_t l_max_total =
      make_layout(precision, all_tokens, hidden, intermediate, local_experts, topk, pad_rows_of(precision)).total;
  const int64_t routing_bytes = up1k(all_tokens * topk * 4);
  const int64_t need_ws = l_max_total + 2 * routing_bytes + up1k(all_tokens * hidden * (fp8 ? 1 : 2)) +
                          up1k(all_tokens * (hidden / 128) * 4);
  MB200_REQUIRE(workspace_bytes >= need_ws, kWorkspaceTooSmall, "dist_forward: workspace %lld < %lld bytes",
                (long long)workspace_bytes, (long long)need_ws);
  MB200_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 1023) == 0, kInvalidArgument,
                "dist_forward: workspace must be 1024-byte aligned");
  for (int i = 0; i < world; ++i)
    MB200_REQUIRE(symmetric_ptrs[i] && (reinterpret_cast<uintptr_t>(symmetric_ptrs[i]) & 1023) == 0, kInvalidArgument,
                  "dist_forward: symmetric buffer of rank %d missing or not 1024-byte aligned", i);

  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  char* ws = reinterpret_cast<char*>(workspace);
  char* sym = static_cast<char*>(symmetric_ptrs[rank]);
  int* status = reinterpret_cast<int*>(ws + l.status);
  Schedule sched{reinterpret_cast<int*>(ws + l.counts), reinterpret_cast<int*>(ws + l.prefix),
                 reinterpret_cast<int*>(ws + l.sorted), reinterpret_cast<int*>(ws + l.inverse),
                 pad};
  int* ids_all = reinterpret_cast<int*>(ws + l.total);
  float* weights_all = reinterpret_cast<float*>(ws + l.total + routing_bytes);
  const int64_t cap = row_capacity(all_tokens, topk, local_experts, pad);
  const PeerTable flags = offset_table(symmetric_ptrs, world, sl.flags);

  // 1. stage own routing and tokens
  mark_stage(0, s);
  MB200_CHECK_CUDA(cudaMemcpyAsync(sym + sl.ids, topk_ids, tokens * topk * 4, cudaMemcpyDeviceToDevice, s));
  MB200_CHECK_CUDA(cudaMemcpyAsync(sym + sl.weights, topk_weights, tokens * topk * 4, cudaMemcpyDeviceToDevice, s));
  if (fp8) {
    if ((rc = launch_group_quant_fp8(reinterpret_cast<const __nv_bfloat16*>(hidden_states), tokens, hidden,
                                     reinterpret_cast<uint8_t*>(sym + sl.payload),
                                     reinterpret_cast<float*>(sym + sl.payload_scales), hidden / 128, 0, s,
                                     fp8_scale_ue8m0())))
      return rc;
  } else {
    MB200_CHECK_CUDA(cudaMemcpyAsync(sym + sl.payload, hidden_states, tokens * int64_t(hidden) * 2,
                                     cudaMemcpyDeviceToDevice, s));
  }
  // 2. every rank's staging is visible
  if ((rc = launch_peer_barrier(flags, rank, world, seq_base + 1, status, s))) return rc;
  // 3. routing, schedule, dispatch
  if ((rc = launch_gather_routing(offset_table(symmetric_ptrs, world, sl.ids),
                                  offset_table(symmetric_ptrs, world, sl.weights), rank, world,
                                  int(tokens * topk), ids_all, weights_all, s))) return rc;
  if ((rc = launch_align(ids_all, all_tokens * topk, expert_parallel ? expert_map : nullptr, local_experts, sched,
                         cap, reinterpret_cast<int*>(ws + l.scratch), s))) return rc;
  mark_stage(1, s);
  // Which fused forms apply: the 16-bit kernels and the fp8 128-row-tile kernel have dispatch and
  // push warps; the fp8 tokens-on-columns kernel (few rows per expert) keeps separate stages.
  const bool fp8_rows = fp8 && pad == kTileM;
  const bool fused_kernels = !fp8 || fp8_rows;
  const bool push_combine = expert_parallel && fused_kernels;
  int* granule_done = reinterpret_cast<int*>(ws + l.granules);
  int* block_done = reinterpret_cast<int*>(ws + l.blocks);
  if (fused_kernels) MB200_CHECK_CUDA(cudaMemsetAsync(granule_done, 0, size_t(l.counter_span), s));
  FusedDispatch disp{};       // 16-bit: the dispatch pulls run inside the gate/up GEMM kernel
  FusedDispatchFp8 disp8{};   // fp8, 128-row tiles: likewise (e4m3 rows + scales)
  const PeerTable payload = offset_table(symmetric_ptrs, world, sl.payload);
  const PeerTable payload_scales = offset_table(symmetric_ptrs, world, sl.payload_scales);
  if (expert_parallel) {
    // a token has about one expert per rank: pull each needed row straight into its sorted slot
    if (fp8_rows) {
      disp8.xq = payload;
      disp8.xs = payload_scales;
      disp8.rank = rank;
      disp8.world = world;
      disp8.tokens_per_rank = int(tokens);
    } else if (fp8) {
      if ((rc = launch_gather_rows_peer_fp8(payload, payload_scales, rank, world, int(tokens), topk, sched,
                                            local_experts, hidden, ws + l.xg, reinterpret_cast<float*>(ws + l.xs),
                                            cap, s))) return rc;
    } else {
      disp.src = payload;
      disp.rank = rank;
      disp.world = world;
      disp.tokens_per_rank = int(tokens);
    }
  } else {
    // tensor parallel: every rank needs every token for all k assignments, so each peer's
    // token block crosses NVLink once (into the tail of the workspace) and the k-fold
    // replication into sorted rows reads local memory
    const int64_t eb = fp8 ? 1 : 2;
    char* x_all = ws + l.total + 2 * routing_bytes;
    char* xs_all = x_all + up1k(all_tokens * hidden * eb);
    if ((rc = launch_gather_blocks_peer(payload, rank, world, tokens * hidden * eb, x_all, s))) return rc;
    if (fp8 && (rc = launch_gather_blocks_peer(payload_scales, rank, world, tokens * (hidden / 128) * 4, xs_all, s)))
      return rc;
    if (fp8) {
      // one "rank" holding all W*T tokens in ring order
      PeerTable local_x{}, local_s{};
      local_x.ptr[0] = x_all;
      local_s.ptr[0] = xs_all;
      if (fp8_rows) {
        disp8.xq = local_x;
        disp8.xs = local_s;
        disp8.rank = 0;
        disp8.world = 1;
        disp8.tokens_per_rank = int(all_tokens);
      } else if ((rc = launch_gather_rows_peer_fp8(local_x, local_s, 0, 1, int(all_tokens), topk, sched, local_experts,
                                                   hidden, ws + l.xg, reinterpret_cast<float*>(ws + l.xs), cap, s))) {
        return rc;
      }
    } else {
      disp.src.ptr[0] = x_all;
      disp.rank = 0;
      disp.world = 1;
      disp.tokens_per_rank = int(all_tokens);
    }
  }
  if (!fp8) {
    disp.topk = topk;
    disp.vec_per_row = hidden / 8;
    disp.rows_out = reinterpret_cast<uint4*>(ws + l.xg);
    disp.granule_done = granule_done;
    disp.granule_target = kDispatchWarpsPerCta;
    disp.enabled = kDispatchFused;
  } else if (fp8_rows) {
    disp8.topk = topk;
    disp8.groups_per_row = hidden / 128;
    disp8.rows_out = reinterpret_cast<uint4*>(ws + l.xg);
    disp8.scales_t_out = reinterpret_cast<float*>(ws + l.xs);
    disp8.granule_done = granule_done;
    disp8.enabled = 1;
  }
  mark_stage(2, s);
  // 4. grouped GEMMs.  Expert parallel, fused kernels: the down GEMM's push warps send every
  // finished row to the rank that owns its token; otherwise the contributions of a token that
  // landed on this rank are pre-reduced into one row of `partial`.
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(ws + l.y);
  FusedPush push{};
  if (push_combine) {
    push.dst = offset_table(symmetric_ptrs, world, sl.yrecv);
    push.rank = rank;
    push.world = world;
    push.tokens_per_rank = int(tokens);
    push.topk = topk;
    push.vec_per_row = hidden / 8;
    push.own_rows = int(tokens) * topk;
    push.rows_in = reinterpret_cast<const uint4*>(y);
    push.block_done = block_done;
    push.enabled = 1;
  }
  if (fp8) {
    if ((rc = run_gemm_stage_fp8(kGateUpSwiglu, ws + l.xg, reinterpret_cast<float*>(ws + l.xs), cap, w1, w1_scale,
                                 local_experts, hidden, intermediate, sched.counts, sched.mtile_prefix,
                                 sched.sorted_ids, nullptr, ws + l.act, reinterpret_cast<float*>(ws + l.acts), status,
                                 device, s, reinterpret_cast<unsigned long long*>(status + 8), pad,
                                 fp8_rows ? &disp8 : nullptr))) return rc;
    mark_stage(3, s);
    if ((rc = run_gemm_stage_fp8(kDownWeighted, ws + l.act, reinterpret_cast<float*>(ws + l.acts), cap, w2, w2_scale,
                                 local_experts, hidden, intermediate, sched.counts, sched.mtile_prefix,
                                 sched.sorted_ids, weights_all, y, nullptr, status, device, s,
                                 reinterpret_cast<unsigned long long*>(status + 12), pad, nullptr,
                                 push_combine ? &push : nullptr))) return rc;
  } else {
    if ((rc = run_gemm_stage(kGateUpSwiglu, ws + l.xg, cap, w1, local_experts, hidden, intermediate, sched.counts,
                             sched.mtile_prefix, sched.sorted_ids, nullptr, ws + l.act, status, device, s,
                             reinterpret_cast<unsigned long long*>(status + 8), &disp, fp16))) return rc;
    mark_stage(3, s);
    if ((rc = run_gemm_stage(kDownWeighted, ws + l.act, cap, w2, local_experts, hidden, intermediate, sched.counts,
                             sched.mtile_prefix, sched.sorted_ids, weights_all, y, status, device, s,
                             reinterpret_cast<unsigned long long*>(status + 12), nullptr, fp16,
                             push_combine ? &push : nullptr))) return rc;
  }
  mark_stage(4, s);
  if (push_combine) {
    // 5. every rank's pushes have landed; sum the k rows of each own token.  Two barriers per
    // forward are enough: peers push again only after the next forward's first barrier, which
    // this rank reaches after this combine, and tokens are restaged only after every peer has
    // passed this barrier, i.e. has finished pulling them.
    if ((rc = launch_peer_barrier(flags, rank, world, seq_base + 2, status, s))) return rc;
    rc = launch_combine_bf16(reinterpret_cast<const __nv_bfloat16*>(sym + sl.yrecv), nullptr, int(tokens), topk,
                             hidden, reinterpret_cast<__nv_bfloat16*>(out), s, fp16);
  } else if (!expert_parallel) {
    // Tensor parallel: every rank holds a partial result for EVERY token.  The sum over a token's
    // k rows goes straight into the owner's `partial` plane of this rank (16-byte stores over
    // NVLink while the k-fold rows stream from HBM); after the barrier the owner sums its W
    // local planes.  Two barriers per forward, for the reasons given above.
    if ((rc = launch_combine_push(y, int(all_tokens), int(tokens), topk, hidden,
                                  offset_table(symmetric_ptrs, world, sl.partial), rank, world, s, fp16))) return rc;
    if ((rc = launch_peer_barrier(flags, rank, world, seq_base + 2, status, s))) return rc;
    rc = launch_sum_planes(reinterpret_cast<const __nv_bfloat16*>(sym + sl.partial), int(tokens), world, hidden,
                           reinterpret_cast<__nv_bfloat16*>(out), s, fp16);
  } else {
    if ((rc = launch_combine_bf16(y, sched.inverse, int(all_tokens), topk, hidden,
                                  reinterpret_cast<__nv_bfloat16*>(sym + sl.partial), s, fp16))) return rc;
    // 5. combine across ranks
    if ((rc = launch_peer_barrier(flags, rank, world, seq_base + 2, status, s))) return rc;
    if ((rc = launch_reduce_partials(offset_table(symmetric_ptrs, world, sl.partial), rank, world, int(tokens), topk,
                                     topk_ids, local_experts, hidden,
                                     reinterpret_cast<__nv_bfloat16*>(out), s, fp16))) return rc;
    // peers may still be reading this rank's buffers: nobody restages before all are done
    rc = launch_peer_barrier(flags, rank, world, seq_base + 3, status, s);
  }
  mark_stage(5, s);
  return rc;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Set-up helpers: a buffer peers can map through CUDA IPC.  Used by the host
// side when torch's symmetric-memory allocator is not available.  These are the
// only entry points of the library that allocate; they are for setup()/close(),
// never for the timed path.
// ---------------------------------------------------------------------------
extern "C" {

int mb200_ipc_alloc(int64_t bytes, void** ptr_out, void* handle_out64) {
  MB200_REQUIRE(bytes > 0 && ptr_out && handle_out64, kInvalidArgument, "ipc_alloc: bad argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  void* p = nullptr;
  MB200_CHECK_CUDA(cudaMalloc(&p, size_t(bytes)));
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    set_last_error("cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
    return kCudaError;
  }
  MB200_CHECK_CUDA(cudaMemset(p, 0, size_t(bytes)));
  memcpy(handle_out64, &h, sizeof(h));
  *ptr_out = p;
  return kOk;
}

int mb200_ipc_open(const void* handle64, void** ptr_out) {
  MB200_REQUIRE(handle64 && ptr_out, kInvalidArgument, "ipc_open: bad argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  MB200_CHECK_CUDA(cudaIpcOpenMemHandle(ptr_out, h, cudaIpcMemLazyEnablePeerAccess));
  return kOk;
}

int mb200_ipc_close(void* ptr) {
  MB200_CHECK_CUDA(cudaIpcCloseMemHandle(ptr));
  return kOk;
}

int mb200_ipc_free(void* ptr) {
  MB200_CHECK_CUDA(cudaFree(ptr));
  return kOk;
}

}  // extern "C"
