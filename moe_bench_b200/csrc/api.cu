// extern "C" entry points (declared in include/moe_bench_b200.h), tensor-map
// creation and the workspace layout of the forward.

#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "../../include/moe_bench_b200.h"
#include <cstdlib>

#include "layer.cuh"

namespace mb200 {

namespace {
thread_local char g_last_error[512] = "";
constexpr int kStageEvents = 6;
thread_local cudaEvent_t g_stage_events[kStageEvents] = {};
thread_local int g_stage_event_count = 0;
thread_local int g_comm_only = 0;
thread_local int g_fp8_ue8m0 = 0;

}

int fp8_scale_ue8m0() { return g_fp8_ue8m0; }

void mark_stage(int i, cudaStream_t s) {
  if (i < g_stage_event_count && g_stage_events[i]) cudaEventRecord(g_stage_events[i], s);
}

int device_sm_count(int device) {
  static std::atomic<int> cached[kMaxDevices];
  if (device >= 0 && device < kMaxDevices) {
    const int v = cached[device].load(std::memory_order_relaxed);
    if (v > 0) return v;
  }
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  if (device >= 0 && device < kMaxDevices) cached[device].store(sms, std::memory_order_relaxed);
  return sms;
}

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

// ---------------------------------------------------------------------------
// Tensor maps.  cuTensorMapEncodeTiled is resolved through the runtime so the
// library carries no link-time dependency on the driver library.
// ---------------------------------------------------------------------------
namespace {
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  // initialised once, thread-safe (C++11 static initialisation)
  static const EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      return reinterpret_cast<EncodeTiledFn>(p);
    return EncodeTiledFn(nullptr);
  }();
  return fn;
}
}  // namespace

int make_tensor_map_2d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t rows,
                       uint64_t cols, uint32_t box_rows, int fp16) {
  EncodeTiledFn fn = encode_tiled_fn();
  MB200_REQUIRE(fn != nullptr, kDriverEntryMissing, "cuTensorMapEncodeTiled is not available");
  MB200_REQUIRE(elem_bytes == 1 || elem_bytes == 2, kInvalidArgument, "tensor map: element size %d", elem_bytes);
  MB200_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, kInvalidArgument,
                "tensor map: base address must be 16-byte aligned");
  MB200_REQUIRE((cols * elem_bytes) % 16 == 0, kUnsupportedShape,
                "tensor map: row pitch %llu bytes must be a multiple of 16",
                (unsigned long long)(cols * elem_bytes));
  MB200_REQUIRE(box_rows >= 1 && box_rows <= 256, kInvalidArgument, "tensor map: box of %u rows", box_rows);
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * elem_bytes};
  const cuuint32_t box[2] = {uint32_t(128 / elem_bytes), box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dtype = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                    : fp16          ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                    : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUresult r = fn(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  MB200_REQUIRE(r == CUDA_SUCCESS, kCudaError, "cuTensorMapEncodeTiled failed with code %d", int(r));
  return kOk;
}

// ---------------------------------------------------------------------------
// Workspace layout
// ---------------------------------------------------------------------------
int64_t row_capacity(int64_t tokens, int topk, int local_experts, int pad_rows) {
  const int64_t a = tokens * topk;
  const int64_t touched = a < local_experts ? a : local_experts;
  const int64_t rows = a + touched * (pad_rows - 1);
  return (rows + pad_rows - 1) / pad_rows * pad_rows;
}

namespace {
int64_t align_up(int64_t v) { return (v + 1023) / 1024 * 1024; }
cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }
}  // namespace

Layout make_layout(int precision, int64_t tokens, int hidden, int intermediate, int local_experts, int topk,
                   int pad_rows) {
  const int64_t eb = precision == MB200_PRECISION_FP8 ? 1 : 2;  // bytes per activation element
  const int64_t a = tokens * topk;
  const int64_t cap = row_capacity(tokens, topk, local_experts, pad_rows);
  Layout l;
  int64_t off = 0;
  auto take = [&](int64_t bytes) { int64_t o = off; off = align_up(off + bytes); return o; };
  l.status = take(256);
  l.counts = take(int64_t(local_experts) * 4);
  l.prefix = take(int64_t(local_experts + 1) * 4);
  l.sorted = take(cap * 4);
  l.inverse = take((a > 0 ? a : 1) * 4);
  l.scratch = take(align_scratch_ints(a, local_experts) * 4);
  l.xg = take(cap * hidden * eb);
  l.act = take(cap * intermediate * eb);
  l.y = take((a > 0 ? a : 1) * int64_t(hidden) * 2);
  l.xs = l.acts = 0;
  // arrival counters per 16-row granule (fused dispatch) and completion counters per token
  // block (fused combine push), adjacent so that one memset clears both
  l.granule_bytes = (cap / kPadBf16 + 1) * 4;
  l.granules = take(l.granule_bytes);
  l.block_bytes = (cap / kPadBf16 + 1) * 4;
  l.blocks = take(l.block_bytes);
  l.counter_span = l.blocks + l.block_bytes - l.granules;
  l.xq_tok = l.xs_tok = 0;
  if (precision == MB200_PRECISION_FP8) {
    l.xs = take(int64_t(hidden / 128) * cap * 4);
    l.acts = take(int64_t(intermediate / 128) * cap * 4);
    // every token quantised once; the sorted rows are gathered from here
    l.xq_tok = take(tokens * hidden);
    l.xs_tok = take(tokens * int64_t(hidden / 128) * 4);
  }
  l.total = off;
  return l;
}

int check_shape(int64_t tokens, int hidden, int intermediate, int local_experts, int topk) {
  MB200_REQUIRE(tokens >= 0 && topk >= 1 && local_experts >= 1, kInvalidArgument,
                "shape: tokens=%lld topk=%d local_experts=%d", (long long)tokens, topk, local_experts);
  MB200_REQUIRE(local_experts <= kMaxExperts, kUnsupportedShape, "local_experts=%d > %d", local_experts, kMaxExperts);
  MB200_REQUIRE(hidden > 0 && hidden % 64 == 0, kUnsupportedShape, "hidden=%d must be a positive multiple of 64", hidden);
  MB200_REQUIRE(intermediate > 0 && intermediate % 64 == 0, kUnsupportedShape,
                "intermediate=%d must be a positive multiple of 64", intermediate);
  MB200_REQUIRE(tokens * topk < (int64_t(1) << 31) - 4096 * 128, kUnsupportedShape,
                "tokens*topk=%lld does not fit 32-bit row indices", (long long)(tokens * topk));
  return kOk;
}

int run_gemm_stage(int mode, const void* a, int64_t cap, const void* w, int local_experts, int hidden,
                   int intermediate, const int* counts, const int* prefix, const int* sorted,
                   const float* row_scale, void* out, int* status, int device, cudaStream_t stream,
                   unsigned long long* clock_probe, const FusedDispatch* dispatch, int fp16, const FusedPush* push) {
  CUtensorMap map_w;
  TokenMaps maps_t;
  GemmArgs g{};
  g.clock_probe = clock_probe;
  g.fp16 = fp16;
  g.counts = counts;
  g.mtile_prefix = prefix;
  g.sorted_ids = sorted;
  g.num_experts = local_experts;
  g.row_scale = row_scale;
  g.out = out;
  g.status = status;
  int rc;
  const int token_cols = mode == kGateUpSwiglu ? hidden : intermediate;
  for (int i = 0; i < kTokenBoxes; ++i)
    if ((rc = make_tensor_map_2d(&maps_t.m[i], a, 2, uint64_t(cap), uint64_t(token_cols), 16u << i, fp16))) return rc;
  if (mode == kGateUpSwiglu) {
    if ((rc = make_tensor_map_2d(&map_w, w, 2, uint64_t(local_experts) * 2 * intermediate, uint64_t(hidden), 128, fp16))) return rc;
    g.n_tiles = (intermediate + 127) / 128;
    g.k_iters = (hidden + 63) / 64;
    g.b_rows_per_expert = 2 * intermediate;
    g.b_half_offset = intermediate;
    g.out_cols = intermediate;
  } else {
    if ((rc = make_tensor_map_2d(&map_w, w, 2, uint64_t(local_experts) * hidden, uint64_t(intermediate), 256, fp16))) return rc;
    g.n_tiles = (hidden + 255) / 256;
    g.k_iters = (intermediate + 63) / 64;
    g.b_rows_per_expert = hidden;
    g.b_half_offset = 0;
    g.out_cols = hidden;
  }
  if (g_comm_only) g.k_iters = 0;  // decomposition: data movement only (see mb200_set_comm_only)
  FusedDispatch none{};
  FusedPush no_push{};
  return launch_grouped_gemm_bf16(GemmMode(mode), map_w, maps_t, g, dispatch ? *dispatch : none,
                                  push ? *push : no_push, device, stream);
}

int check_shape_fp8(int hidden, int intermediate) {
  MB200_REQUIRE(hidden % 128 == 0 && intermediate % 128 == 0, kUnsupportedShape,
                "fp8: hidden=%d and intermediate=%d must be multiples of the 128x128 scale block", hidden,
                intermediate);
  return kOk;
}

int run_gemm_stage_fp8(int mode, const void* a, const float* a_scale_t, int64_t cap, const void* w,
                       const float* w_scale, int local_experts, int hidden, int intermediate,
                       const int* counts, const int* prefix, const int* sorted, const float* row_scale,
                       void* out, float* out_scale_t, int* status, int device, cudaStream_t stream,
                       unsigned long long* clock_probe, int pad_rows, const FusedDispatchFp8* dispatch,
                       const FusedPush* push) {
  CUtensorMap map_a, map_b;
  GemmFp8Args g{};
  g.clock_probe = clock_probe;
  g.ue8m0 = g_fp8_ue8m0;
  const bool cols = pad_rows == kPadBf16;  // schedule padded to 16 rows: tokens-on-columns kernel
  TokenMaps maps_t;
  if (cols) {
    const int token_cols = mode == kGateUpSwiglu ? hidden : intermediate;
    for (int i = 0; i < kTokenBoxes; ++i) {
      int rc0 = make_tensor_map_2d(&maps_t.m[i], a, 1, uint64_t(cap), uint64_t(token_cols), 16u << i);
      if (rc0) return rc0;
    }
  }
  g.counts = counts;
  g.mtile_prefix = prefix;
  g.sorted_ids = sorted;
  g.num_experts = local_experts;
  g.row_capacity = cap;
  g.a_scale_t = a_scale_t;
  g.w_scale = w_scale;
  g.row_scale = row_scale;
  g.out = out;
  g.out_scale_t = out_scale_t;
  g.status = status;
  int rc;
  if (mode == kGateUpSwiglu) {
    if ((rc = make_tensor_map_2d(&map_a, a, 1, uint64_t(cap), uint64_t(hidden), kTileM))) return rc;
    if ((rc = make_tensor_map_2d(&map_b, w, 1, uint64_t(local_experts) * 2 * intermediate, uint64_t(hidden), 128))) return rc;
    g.n_tiles = intermediate / 128;
    g.k_blocks = hidden / 128;
    g.b_rows_per_expert = 2 * intermediate;
    g.b_half_offset = intermediate;
    g.out_cols = intermediate;
    g.scale_rows_per_expert = 2 * intermediate / 128;
    g.scale_half_offset = intermediate / 128;
  } else {
    if ((rc = make_tensor_map_2d(&map_a, a, 1, uint64_t(cap), uint64_t(intermediate), kTileM))) return rc;
    if ((rc = make_tensor_map_2d(&map_b, w, 1, uint64_t(local_experts) * hidden, uint64_t(intermediate), 256))) return rc;
    g.n_tiles = (hidden + 255) / 256;
    g.k_blocks = intermediate / 128;
    g.b_rows_per_expert = hidden;
    g.b_half_offset = 0;
    g.out_cols = hidden;
    g.scale_rows_per_expert = hidden / 128;
    g.scale_half_offset = 0;
  }
  MB200_REQUIRE(!cols || (!dispatch && !push), kInvalidArgument,
                "fp8: fused dispatch / push exist only in the 128-row-tile kernel");
  if (g_comm_only) g.k_blocks = 0;  // decomposition: data movement only (see mb200_set_comm_only)
  if (cols) return launch_grouped_gemm_fp8_cols(GemmMode(mode), map_b, maps_t, g, device, stream);
  const FusedDispatchFp8 no_disp{};
  const FusedPush no_push{};
  return launch_grouped_gemm_fp8(GemmMode(mode), map_a, map_b, g, dispatch ? *dispatch : no_disp,
                                 push ? *push : no_push, device, stream);
}

}  // namespace mb200

using namespace mb200;

extern "C" {

int mb200_abi_version(void) { return MB200_ABI_VERSION; }

const char* mb200_last_error(void) { return g_last_error; }

int mb200_route_topk(const float* logits, int tokens, int experts, int topk, int32_t* topk_ids,
                     float* topk_weights, void* stream) {
  MB200_REQUIRE(tokens >= 0, kInvalidArgument, "route_topk: tokens=%d", tokens);
  MB200_REQUIRE(tokens == 0 || (logits && topk_ids && topk_weights), kInvalidArgument, "route_topk: null pointer");
  return launch_route_topk(logits, tokens, experts, topk, topk_ids, topk_weights, as_stream(stream));
}

int64_t mb200_row_capacity(int64_t tokens, int topk, int local_experts, int pad_rows) {
  if (pad_rows < 1) return -1;
  return row_capacity(tokens, topk, local_experts, pad_rows);
}

int64_t mb200_align_scratch_bytes(int64_t tokens, int topk, int local_experts) {
  return align_scratch_ints(tokens * topk, local_experts) * 4;
}

int mb200_align(const int32_t* topk_ids, int64_t tokens, int topk, const int32_t* expert_map,
                int local_experts, int32_t* counts, int32_t* mtile_prefix, int32_t* sorted_ids,
                int32_t* inverse, int64_t row_cap, int pad_rows, void* scratch, void* stream) {
  MB200_REQUIRE(tokens >= 0 && topk >= 1, kInvalidArgument, "align: tokens=%lld topk=%d", (long long)tokens, topk);
  MB200_REQUIRE(pad_rows >= 1 && pad_rows <= 1024, kInvalidArgument, "align: pad_rows=%d (1..1024)", pad_rows);
  MB200_REQUIRE(counts && mtile_prefix && sorted_ids && scratch && (tokens == 0 || (topk_ids && inverse)),
                kInvalidArgument, "align: null pointer");
  MB200_REQUIRE(row_cap >= row_capacity(tokens, topk, local_experts, pad_rows), kWorkspaceTooSmall,
                "align: row capacity %lld < %lld", (long long)row_cap,
                (long long)row_capacity(tokens, topk, local_experts, pad_rows));
  Schedule s{counts, mtile_prefix, sorted_ids, inverse, pad_rows};
  return launch_align(topk_ids, tokens * topk, expert_map, local_experts, s, row_cap,
                      reinterpret_cast<int*>(scratch), as_stream(stream));
}

int mb200_group_quant_fp8(const void* x, int64_t rows, int hidden, void* q, float* scales, void* stream) {
  MB200_REQUIRE(rows >= 0 && (rows == 0 || (x && q && scales)), kInvalidArgument, "group_quant: bad argument");
  return launch_group_quant_fp8(reinterpret_cast<const __nv_bfloat16*>(x), rows, hidden,
                                reinterpret_cast<uint8_t*>(q), scales, hidden / 128, 0, as_stream(stream), g_fp8_ue8m0);
}

int mb200_grouped_gemm_bf16(int mode, const void* a, int64_t row_cap, const void* w, int local_experts,
                            int hidden, int intermediate, const int32_t* counts,
                            const int32_t* mtile_prefix, const int32_t* sorted_ids,
                            const float* row_scale, void* out, int32_t* status, int device, void* stream) {
  MB200_REQUIRE(mode == 0 || mode == 1, kInvalidArgument, "grouped_gemm: mode=%d", mode);
  MB200_REQUIRE(a && w && counts && mtile_prefix && sorted_ids && out && (mode == 0 || row_scale),
                kInvalidArgument, "grouped_gemm: null pointer");
  MB200_REQUIRE(row_cap > 0 && row_cap % kPadBf16 == 0, kInvalidArgument,
                "grouped_gemm: row capacity %lld must be a positive multiple of %d", (long long)row_cap, kPadBf16);
  int rc = check_shape(0, hidden, intermediate, local_experts, 1);
  if (rc) return rc;
  return run_gemm_stage(mode, a, row_cap, w, local_experts, hidden, intermediate, counts, mtile_prefix,
                        sorted_ids, row_scale, out, status, device, as_stream(stream), nullptr, nullptr, 0);
}

int mb200_grouped_gemm_bf16_gated(const void* a, int64_t row_cap, const void* w, int local_experts, int hidden,
                                  int intermediate, const int32_t* counts, const int32_t* mtile_prefix,
                                  const int32_t* sorted_ids, const int32_t* granule_done, int granule_target,
                                  void* out, int32_t* status, int device, void* stream) {
  MB200_REQUIRE(a && w && counts && mtile_prefix && sorted_ids && out && granule_done && status, kInvalidArgument,
                "grouped_gemm_gated: null pointer");
  MB200_REQUIRE(granule_target >= 1, kInvalidArgument, "grouped_gemm_gated: granule_target=%d", granule_target);
  MB200_REQUIRE(row_cap > 0 && row_cap % kPadBf16 == 0, kInvalidArgument,
                "grouped_gemm_gated: row capacity %lld must be a positive multiple of %d", (long long)row_cap, kPadBf16);
  int rc = check_shape(0, hidden, intermediate, local_experts, 1);
  if (rc) return rc;
  FusedDispatch gate{};
  gate.granule_done = const_cast<int*>(granule_done);
  gate.granule_target = granule_target;
  gate.enabled = kDispatchExternal;
  return run_gemm_stage(kGateUpSwiglu, a, row_cap, w, local_experts, hidden, intermediate, counts, mtile_prefix,
                        sorted_ids, nullptr, out, status, device, as_stream(stream), nullptr, &gate, 0);
}

int64_t mb200_workspace_bytes(int precision, int64_t tokens, int hidden, int intermediate,
                              int local_experts, int topk) {
  if (check_shape(tokens, hidden, intermediate, local_experts, topk)) return -1;
  if (precision != MB200_PRECISION_BF16 && precision != MB200_PRECISION_FP8 && precision != MB200_PRECISION_FP16) {
    set_last_error("workspace_bytes: unknown precision %d", precision);
    return -1;
  }
  if (precision == MB200_PRECISION_FP8 && check_shape_fp8(hidden, intermediate)) return -1;
  // fp8: the 128-row padding needs the larger buffers; the forward may use the 16-row one
  return make_layout(precision, tokens, hidden, intermediate, local_experts, topk, pad_rows_of(precision)).total;
}

int mb200_forward_layout(int precision, int64_t tokens, int hidden, int intermediate, int local_experts, int topk,
                         int64_t expected_rows, int64_t* out10) {
  MB200_REQUIRE(out10 != nullptr, kInvalidArgument, "forward_layout: null pointer");
  MB200_REQUIRE(precision == MB200_PRECISION_BF16 || precision == MB200_PRECISION_FP8 ||
                    precision == MB200_PRECISION_FP16,
                kInvalidArgument, "forward_layout: unknown precision %d", precision);
  int rc = check_shape(tokens, hidden, intermediate, local_experts, topk);
  if (rc) return rc;
  const bool fp8 = precision == MB200_PRECISION_FP8;
  if (fp8 && (rc = check_shape_fp8(hidden, intermediate))) return rc;
  const int pad = fp8 ? fp8_pad_rows(expected_rows, local_experts) : kPadBf16;
  const Layout l = make_layout(precision, tokens, hidden, intermediate, local_experts, topk, pad);
  const int64_t v[10] = {pad, row_capacity(tokens, topk, local_experts, pad), l.counts, l.prefix, l.sorted,
                         l.inverse, l.xg, l.xs, l.act, l.y};
  for (int i = 0; i < 10; ++i) out10[i] = v[i];
  return kOk;
}

static int moe_forward_16bit(int fp16, const void* hidden_states, const void* w1, const void* w2,
                             const int32_t* topk_ids, const float* topk_weights,
                             const int32_t* expert_map, void* out, int64_t tokens, int hidden,
                             int intermediate, int local_experts, int topk, void* workspace,
                             int64_t workspace_bytes, int device, void* stream) {
  int rc = check_shape(tokens, hidden, intermediate, local_experts, topk);
  if (rc) return rc;
  if (tokens == 0) return kOk;
  MB200_REQUIRE(hidden_states && w1 && w2 && topk_ids && topk_weights && out && workspace, kInvalidArgument,
                "moe_forward (16-bit): null pointer");
  const Layout l = make_layout(MB200_PRECISION_BF16, tokens, hidden, intermediate, local_experts, topk, kPadBf16);
  MB200_REQUIRE(workspace_bytes >= l.total, kWorkspaceTooSmall, "moe_forward (16-bit): workspace %lld < %lld bytes",
                (long long)workspace_bytes, (long long)l.total);
  MB200_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 1023) == 0, kInvalidArgument,
                "moe_forward (16-bit): workspace must be 1024-byte aligned");
  cudaStream_t s = as_stream(stream);
  char* ws = reinterpret_cast<char*>(workspace);
  int* status = reinterpret_cast<int*>(ws + l.status);
  Schedule sched{reinterpret_cast<int*>(ws + l.counts), reinterpret_cast<int*>(ws + l.prefix),
                 reinterpret_cast<int*>(ws + l.sorted), reinterpret_cast<int*>(ws + l.inverse), kPadBf16};
  const int64_t cap = row_capacity(tokens, topk, local_experts, kPadBf16);
  __nv_bfloat16* xg = reinterpret_cast<__nv_bfloat16*>(ws + l.xg);
  __nv_bfloat16* act = reinterpret_cast<__nv_bfloat16*>(ws + l.act);
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(ws + l.y);

  mark_stage(0, s);
  if ((rc = launch_align(topk_ids, tokens * topk, expert_map, local_experts, sched, cap,
                         reinterpret_cast<int*>(ws + l.scratch), s))) return rc;
  mark_stage(1, s);
  // the row gather runs inside the gate/up GEMM kernel (dispatch warps); only its counters are reset here
  FusedDispatch disp{};
  disp.src.ptr[0] = const_cast<void*>(hidden_states);
  disp.rank = 0;
  disp.world = 1;
  disp.tokens_per_rank = int(tokens);
  disp.topk = topk;
  disp.vec_per_row = hidden / 8;
  disp.rows_out = reinterpret_cast<uint4*>(xg);
  disp.granule_done = reinterpret_cast<int*>(ws + l.granules);
  disp.granule_target = kDispatchWarpsPerCta;
  disp.enabled = kDispatchFused;
  MB200_CHECK_CUDA(cudaMemsetAsync(disp.granule_done, 0, size_t(l.granule_bytes), s));
  mark_stage(2, s);
  if ((rc = run_gemm_stage(kGateUpSwiglu, xg, cap, w1, local_experts, hidden, intermediate, sched.counts,
                           sched.mtile_prefix, sched.sorted_ids, nullptr, act, status, device, s,
                             reinterpret_cast<unsigned long long*>(status + 8), &disp, fp16))) return rc;
  mark_stage(3, s);
  if ((rc = run_gemm_stage(kDownWeighted, act, cap, w2, local_experts, hidden, intermediate, sched.counts,
                           sched.mtile_prefix, sched.sorted_ids, topk_weights, y, status, device, s,
                             reinterpret_cast<unsigned long long*>(status + 12), nullptr, fp16))) return rc;
  mark_stage(4, s);
  rc = launch_combine_bf16(y, sched.inverse, int(tokens), topk, hidden, reinterpret_cast<__nv_bfloat16*>(out), s, fp16);
  mark_stage(5, s);
  return rc;
}

int mb200_moe_forward_bf16(const void* hidden_states, const void* w1, const void* w2,
                           const int32_t* topk_ids, const float* topk_weights,
                           const int32_t* expert_map, void* out, int64_t tokens, int hidden,
                           int intermediate, int local_experts, int topk, void* workspace,
                           int64_t workspace_bytes, int device, void* stream) {
  return moe_forward_16bit(0, hidden_states, w1, w2, topk_ids, topk_weights, expert_map, out, tokens, hidden,
                           intermediate, local_experts, topk, workspace, workspace_bytes, device, stream);
}

int mb200_moe_forward_fp16(const void* hidden_states, const void* w1, const void* w2,
                           const int32_t* topk_ids, const float* topk_weights,
                           const int32_t* expert_map, void* out, int64_t tokens, int hidden,
                           int intermediate, int local_experts, int topk, void* workspace,
                           int64_t workspace_bytes, int device, void* stream) {
  return moe_forward_16bit(1, hidden_states, w1, w2, topk_ids, topk_weights, expert_map, out, tokens, hidden,
                           intermediate, local_experts, topk, workspace, workspace_bytes, device, stream);
}

int mb200_grouped_gemm_fp8(int mode, const void* a, const float* a_scale_t, int64_t row_cap, const void* w,
                           const float* w_scale, int local_experts, int hidden, int intermediate,
                           const int32_t* counts, const int32_t* mtile_prefix, const int32_t* sorted_ids,
                           const float* row_scale, void* out, float* out_scale_t, int32_t* status,
                           int device, void* stream) {
  MB200_REQUIRE(mode == 0 || mode == 1, kInvalidArgument, "grouped_gemm_fp8: mode=%d", mode);
  MB200_REQUIRE(a && a_scale_t && w && w_scale && counts && mtile_prefix && sorted_ids && out &&
                    (mode == 0 ? out_scale_t != nullptr : row_scale != nullptr),
                kInvalidArgument, "grouped_gemm_fp8: null pointer");
  MB200_REQUIRE(row_cap > 0 && row_cap % kTileM == 0, kInvalidArgument,
                "grouped_gemm_fp8: row capacity %lld must be a positive multiple of %d", (long long)row_cap, kTileM);
  int rc = check_shape(0, hidden, intermediate, local_experts, 1);
  if (rc) return rc;
  if ((rc = check_shape_fp8(hidden, intermediate))) return rc;
  return run_gemm_stage_fp8(mode, a, a_scale_t, row_cap, w, w_scale, local_experts, hidden, intermediate, counts,
                            mtile_prefix, sorted_ids, row_scale, out, out_scale_t, status, device,
                            as_stream(stream));
}

int mb200_grouped_gemm_fp8_cols(int mode, const void* a, const float* a_scale_t, int64_t row_cap, const void* w,
                                const float* w_scale, int local_experts, int hidden, int intermediate,
                                const int32_t* counts, const int32_t* mtile_prefix, const int32_t* sorted_ids,
                                const float* row_scale, void* out, float* out_scale_t, int32_t* status,
                                int device, void* stream) {
  MB200_REQUIRE(mode == 0 || mode == 1, kInvalidArgument, "grouped_gemm_fp8_cols: mode=%d", mode);
  MB200_REQUIRE(a && a_scale_t && w && w_scale && counts && mtile_prefix && sorted_ids && out &&
                    (mode == 0 ? out_scale_t != nullptr : row_scale != nullptr),
                kInvalidArgument, "grouped_gemm_fp8_cols: null pointer");
  MB200_REQUIRE(row_cap > 0 && row_cap % kPadBf16 == 0, kInvalidArgument,
                "grouped_gemm_fp8_cols: row capacity %lld must be a positive multiple of %d", (long long)row_cap,
                kPadBf16);
  int rc = check_shape(0, hidden, intermediate, local_experts, 1);
  if (rc) return rc;
  if ((rc = check_shape_fp8(hidden, intermediate))) return rc;
  return run_gemm_stage_fp8(mode, a, a_scale_t, row_cap, w, w_scale, local_experts, hidden, intermediate, counts,
                            mtile_prefix, sorted_ids, row_scale, out, out_scale_t, status, device,
                            as_stream(stream), nullptr, kPadBf16);
}

int mb200_moe_forward_fp8(const void* hidden_states, const void* w1, const void* w2, const float* w1_scale,
                          const float* w2_scale, const int32_t* topk_ids, const float* topk_weights,
                          const int32_t* expert_map, void* out, int64_t tokens, int hidden, int intermediate,
                          int local_experts, int topk, void* workspace, int64_t workspace_bytes, int device,
                          void* stream) {
  int rc = check_shape(tokens, hidden, intermediate, local_experts, topk);
  if (rc) return rc;
  if ((rc = check_shape_fp8(hidden, intermediate))) return rc;
  if (tokens == 0) return kOk;
  MB200_REQUIRE(hidden_states && w1 && w2 && w1_scale && w2_scale && topk_ids && topk_weights && out && workspace,
                kInvalidArgument, "moe_forward_fp8: null pointer");
  // few rows per expert: 16-row padding and the tokens-on-columns kernels; else 128-row tiles
  const int pad = fp8_pad_rows(tokens * topk, local_experts);
  const Layout l = make_layout(MB200_PRECISION_FP8, tokens, hidden, intermediate, local_experts, topk, pad);
  const int64_t need = make_layout(MB200_PRECISION_FP8, tokens, hidden, intermediate, local_experts, topk, kTileM).total;
  MB200_REQUIRE(workspace_bytes >= need, kWorkspaceTooSmall, "moe_forward_fp8: workspace %lld < %lld bytes",
                (long long)workspace_bytes, (long long)need);
  MB200_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 1023) == 0, kInvalidArgument,
                "moe_forward_fp8: workspace must be 1024-byte aligned");
  cudaStream_t s = as_stream(stream);
  char* ws = reinterpret_cast<char*>(workspace);
  int* status = reinterpret_cast<int*>(ws + l.status);
  Schedule sched{reinterpret_cast<int*>(ws + l.counts), reinterpret_cast<int*>(ws + l.prefix),
                 reinterpret_cast<int*>(ws + l.sorted), reinterpret_cast<int*>(ws + l.inverse), pad};
  const int64_t cap = row_capacity(tokens, topk, local_experts, pad);
  uint8_t* xq = reinterpret_cast<uint8_t*>(ws + l.xg);
  float* xs_t = reinterpret_cast<float*>(ws + l.xs);
  uint8_t* actq = reinterpret_cast<uint8_t*>(ws + l.act);
  float* acts_t = reinterpret_cast<float*>(ws + l.acts);
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(ws + l.y);

  mark_stage(0, s);
  if ((rc = launch_align(topk_ids, tokens * topk, expert_map, local_experts, sched, cap,
                         reinterpret_cast<int*>(ws + l.scratch), s))) return rc;
  mark_stage(1, s);
  // every token is quantised once (reference.py:143-145 quantises the k-fold replicated rows:
  // the same bytes k times), then its e4m3 row and scales are gathered into the sorted slots
  uint8_t* xq_tok = reinterpret_cast<uint8_t*>(ws + l.xq_tok);
  float* xs_tok = reinterpret_cast<float*>(ws + l.xs_tok);
  if ((rc = launch_group_quant_fp8(reinterpret_cast<const __nv_bfloat16*>(hidden_states), tokens, hidden, xq_tok,
                                   xs_tok, hidden / 128, 0, s, g_fp8_ue8m0))) return rc;
  PeerTable self_q{}, self_s{};
  self_q.ptr[0] = xq_tok;
  self_s.ptr[0] = xs_tok;
  FusedDispatchFp8 disp{};
  if (pad == kTileM) {
    // 128-row-tile kernel: the gather runs inside the gate/up GEMM kernel (helper warps); only its
    // counters are reset here
    disp.xq = self_q;
    disp.xs = self_s;
    disp.rank = 0;
    disp.world = 1;
    disp.tokens_per_rank = int(tokens);
    disp.topk = topk;
    disp.groups_per_row = hidden / 128;
    disp.rows_out = reinterpret_cast<uint4*>(xq);
    disp.scales_t_out = xs_t;
    disp.granule_done = reinterpret_cast<int*>(ws + l.granules);
    disp.enabled = 1;
    MB200_CHECK_CUDA(cudaMemsetAsync(disp.granule_done, 0, size_t(l.granule_bytes), s));
  } else if ((rc = launch_gather_rows_peer_fp8(self_q, self_s, 0, 1, int(tokens), topk, sched, local_experts, hidden,
                                               xq, xs_t, cap, s))) {
    return rc;
  }
  mark_stage(2, s);
  if ((rc = run_gemm_stage_fp8(kGateUpSwiglu, xq, xs_t, cap, w1, w1_scale, local_experts, hidden, intermediate,
                               sched.counts, sched.mtile_prefix, sched.sorted_ids, nullptr, actq, acts_t, status,
                               device, s, reinterpret_cast<unsigned long long*>(status + 8), pad,
                               disp.enabled ? &disp : nullptr))) return rc;
  mark_stage(3, s);
  if ((rc = run_gemm_stage_fp8(kDownWeighted, actq, acts_t, cap, w2, w2_scale, local_experts, hidden, intermediate,
                               sched.counts, sched.mtile_prefix, sched.sorted_ids, topk_weights, y, nullptr, status,
                               device, s, reinterpret_cast<unsigned long long*>(status + 12), pad))) return rc;
  mark_stage(4, s);
  rc = launch_combine_bf16(y, sched.inverse, int(tokens), topk, hidden, reinterpret_cast<__nv_bfloat16*>(out), s);
  mark_stage(5, s);
  return rc;
}

int mb200_set_stage_events(void* const* events, int count) {
  MB200_REQUIRE(count >= 0 && count <= kStageEvents && (count == 0 || events), kInvalidArgument,
                "set_stage_events: count=%d (0..%d)", count, kStageEvents);
  for (int i = 0; i < kStageEvents; ++i)
    g_stage_events[i] = i < count ? reinterpret_cast<cudaEvent_t>(events[i]) : nullptr;
  g_stage_event_count = count;
  return kOk;
}

int mb200_set_fp8_scale_format(int format) {
  MB200_REQUIRE(format == MB200_FP8_SCALES_FP32 || format == MB200_FP8_SCALES_UE8M0, kInvalidArgument,
                "set_fp8_scale_format: unknown format %d", format);
  g_fp8_ue8m0 = format == MB200_FP8_SCALES_UE8M0;
  return kOk;
}

int mb200_set_comm_only(int enabled) {
  g_comm_only = enabled ? 1 : 0;
  return kOk;
}

int mb200_read_status(const void* workspace, int32_t* status_out, void* stream) {
  MB200_REQUIRE(workspace && status_out, kInvalidArgument, "read_status: null pointer");
  MB200_CHECK_CUDA(cudaStreamSynchronize(as_stream(stream)));
  MB200_CHECK_CUDA(cudaMemcpy(status_out, workspace, sizeof(int32_t), cudaMemcpyDeviceToHost));
  return kOk;
}

}  // extern "C"
