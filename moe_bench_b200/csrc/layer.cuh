// Internal interfaces between the translation units of the library: the
// schedule produced by the sort-and-pad step, kernel launchers, and the
// workspace layout used by the forward entry points.
#pragma once

#include "common.cuh"

namespace mb200 {

constexpr int kTileM = 128;        // fp8 path: rows per M tile; expert segments are padded to it
constexpr int kPadBf16 = 16;       // bf16 path: expert segments are padded to 16 rows
constexpr int kMaxExperts = 1024;  // local experts per rank supported by the kernels

constexpr int kMaxDevices = 64;    // device ordinals the per-device caches cover
// SM count of a device, cached (thread-safe); 0 if it cannot be read.
int device_sm_count(int device);

constexpr int kMaxPeers = 16;
struct PeerTable {
  void* ptr[kMaxPeers];  // one pointer per rank, valid in this process
};

// Output of the sort-and-pad step, all in device memory.
struct Schedule {
  int* counts;        // [E]    real rows per local expert
  int* mtile_prefix;  // [E+1]  cumulative row blocks; padded row offset = pad_rows * prefix
  int* sorted_ids;    // [P]    flat assignment index (token*k + kpos) per row, -1 = padding
  int* inverse;       // [A]    row of each assignment, -1 = expert not on this rank
  int pad_rows;       //        granule every expert segment is padded to
};

// ---- route_align.cu ---------------------------------------------------------------
int launch_route_topk(const float* logits, int tokens, int experts, int topk, int* ids,
                      float* weights, cudaStream_t stream);
// scratch: int[align_scratch_ints(A, E)]
int64_t align_scratch_ints(int64_t assignments, int experts);
int launch_align(const int* topk_ids, int64_t assignments, const int* expert_map,
                 int local_experts, Schedule sched, int64_t row_capacity, int* scratch,
                 cudaStream_t stream);

// ---- rows.cu ------------------------------------------------------------------------
// y and out are 16-bit (bf16, or fp16 when fp16 != 0); fp32 sum.
int launch_combine_bf16(const __nv_bfloat16* y, const int* inverse, int tokens, int topk,
                        int hidden, __nv_bfloat16* out, cudaStream_t stream, int fp16 = 0);
// Tensor parallel combine: sum over k and store the row into the owner's `partial` plane of this
// rank; then the owner's sum over its W local planes.
int launch_combine_push(const __nv_bfloat16* y, int all_tokens, int tokens_per_rank, int topk, int hidden,
                        const PeerTable& partial, int rank, int world, cudaStream_t stream, int fp16 = 0);
int launch_sum_planes(const __nv_bfloat16* partial, int tokens, int world, int hidden, __nv_bfloat16* out,
                      cudaStream_t stream, int fp16 = 0);
// Per-row, per-128-group e4m3 quantisation.  scales_t is [K/128][scale_ld] (group-major).
int launch_group_quant_fp8(const __nv_bfloat16* x, int64_t rows, int hidden, uint8_t* q,
                           float* scales, int64_t scale_ld, int transposed, cudaStream_t stream, int ue8m0 = 0);
// Activation scale format the calling thread selected (mb200_set_fp8_scale_format): 0 = fp32
// amax/448, 1 = rounded up to a power of two.
int fp8_scale_ue8m0();

// ---- grouped_gemm.cu -----------------------------------------------------------------
struct GemmArgs {
  const int* counts;
  const int* mtile_prefix;  // cumulative 16-row blocks
  const int* sorted_ids;
  int num_experts;
  int n_tiles;            // feature blocks per expert (128 gate+up pairs, or 256 output rows)
  int k_iters;            // 128-byte K slices per tile
  int b_rows_per_expert;  // rows of the 2-D weight view per expert
  int b_half_offset;      // gate/up: row offset of the up half inside one expert
  int out_cols;           // row length of the output
  void* out;
  const float* row_scale;  // per-assignment combine weight (second GEMM)
  int* status;
  unsigned long long* clock_probe;  // optional [2]: SM cycles and nanoseconds CTA 0 spent in the kernel
  int fp16;                // operands and outputs are fp16 instead of bf16
};
enum GemmMode : int { kGateUpSwiglu = 0, kDownWeighted = 1 };
// Dispatch fused into the gate/up GEMM: extra warps of every CTA fill the sorted
// row buffer 16-row granule by granule (from this GPU's tokens, or from the
// source ranks' staged tokens over NVLink) while the tensor pipeline consumes
// granules that have already arrived.
struct FusedDispatch {
  PeerTable src;          // [rank] -> tokens [tokens_per_rank][hidden] bf16 of that rank
  int rank, world;        // flat assignment n = ((ring*T + t)*topk + j), ring = (src - rank) mod world
  int tokens_per_rank;
  int topk;
  int vec_per_row;        // hidden / 8 (16-byte vectors per row)
  uint4* rows_out;        // sorted row buffer the GEMM's token operand is loaded from
  int* granule_done;      // [row_capacity / 16] arrival counters, zeroed before the launch
  int granule_target;     // a granule is complete when its counter reaches this value
  int enabled;            // kDispatchOff, kDispatchFused or kDispatchExternal
};
// kDispatchFused: this kernel's dispatch warps fill the rows (counter target = their number).
// kDispatchExternal: someone else fills the rows and raises the counters (another kernel, or a
// peer GPU's push); the kernel only waits for them.
enum DispatchMode : int { kDispatchOff = 0, kDispatchFused = 1, kDispatchExternal = 2 };
constexpr int kDispatchWarpsPerCta = 4;
// Combine by push, fused into the down GEMM (expert parallel): the weighted rows of every
// finished token block are forwarded by extra warps of the kernel to the GPU that owns the
// token, straight into its receive buffer at the slot of the assignment (token*topk + kpos),
// while later tiles compute.  Rows of this rank's own tokens are stored there by the epilogue
// itself.  The owner then sums the k rows of each token (all of them arrive: every assignment
// has exactly one expert rank).  Replaces the reduce-scatter of schemes.py:142; the shape of
// the reference's push combine (kernels/tk/tk_moe.cu:1251-1519) without its pre-reduction.
struct FusedPush {
  PeerTable dst;          // [rank] -> receive buffer [tokens_per_rank*topk][hidden] 16-bit of that rank
  int rank, world;        // flat assignment n = ((ring*T + t)*topk + j), owner = (rank + ring) mod world
  int tokens_per_rank;
  int topk;
  int vec_per_row;        // hidden / 8 (16-byte vectors per row)
  int own_rows;           // tokens_per_rank * topk: n < own_rows are this rank's own tokens
  const uint4* rows_in;   // the down GEMM's local output [all assignments][hidden] the pushes read
  int* block_done;        // [token blocks] epilogue-warp arrivals per token block, zeroed before the launch
  int enabled;
};

// Token-operand tensor maps with boxes of 16, 32, 64, 128 and 256 rows; the
// kernel picks one from the largest expert segment it finds in the schedule.
constexpr int kTokenBoxes = 5;
struct TokenMaps {
  CUtensorMap m[kTokenBoxes];
};
int launch_grouped_gemm_bf16(GemmMode mode, const CUtensorMap& map_w, const TokenMaps& maps_t,
                             const GemmArgs& args, const FusedDispatch& dispatch, const FusedPush& push,
                             int device, cudaStream_t stream);

// grouped_gemm_fp8.cu: e4m3 operands, fp32 block scales applied in the epilogue
struct GemmFp8Args {
  const int* counts;
  const int* mtile_prefix;
  const int* sorted_ids;
  int num_experts;
  int n_tiles;
  int k_blocks;               // K / 128
  int b_rows_per_expert;
  int b_half_offset;
  int out_cols;
  int64_t row_capacity;       // leading dimension of the transposed scale arrays
  const float* a_scale_t;     // [k_blocks][row_capacity] activation scales
  const float* w_scale;       // [E][scale_rows_per_expert][k_blocks] weight block scales
  int scale_rows_per_expert;
  int scale_half_offset;      // gate/up: scale row of the up half
  void* out;                  // gate/up: e4m3 [rows][N]; down: bf16 [assignments][hidden]
  float* out_scale_t;         // gate/up: [N/128][row_capacity]
  const float* row_scale;     // down: combine weights
  int* status;
  unsigned long long* clock_probe;  // optional [2]: SM cycles and nanoseconds CTA 0 spent in the kernel
  int ue8m0;                  // gate/up: re-quantise the activations with power-of-two scales
};
// Dispatch fused into the fp8 gate/up GEMM (128-row-tile kernel): two helper warps of every CTA
// fill the sorted row buffer with the tokens' e4m3 rows and their 1x128 scales, 16-row granule by
// granule, from this GPU's quantised tokens or with P2P loads from the source ranks.
struct FusedDispatchFp8 {
  PeerTable xq;           // [rank] -> quantised tokens [tokens_per_rank][hidden] e4m3
  PeerTable xs;           // [rank] -> their scales [tokens_per_rank][hidden/128] fp32
  int rank, world;        // flat assignment n = ((ring*T + t)*topk + j), source = (rank + ring) mod world
  int tokens_per_rank;
  int topk;
  int groups_per_row;     // hidden / 128
  uint4* rows_out;        // sorted rows [row_capacity][hidden] e4m3
  float* scales_t_out;    // [hidden/128][row_capacity]
  int* granule_done;      // [row_capacity / 16] arrival counters, zeroed before the launch
  int enabled;
};
constexpr int kFp8HelperWarps = 2;  // dispatch / push warps of the fp8 128-row-tile kernel
int launch_grouped_gemm_fp8(GemmMode mode, const CUtensorMap& map_a, const CUtensorMap& map_b,
                            const GemmFp8Args& args, const FusedDispatchFp8& dispatch, const FusedPush& push,
                            int device, cudaStream_t stream);
// grouped_gemm_fp8_cols.cu: same arithmetic, tokens on the accumulator columns (schedule padded to 16)
int launch_grouped_gemm_fp8_cols(GemmMode mode, const CUtensorMap& map_w, const TokenMaps& maps_t,
                                 const GemmFp8Args& args, int device, cudaStream_t stream);
// Rows per expert up to which the fp8 forward uses the tokens-on-columns kernel.
constexpr int kFp8ColsMaxAvgRows = 24;  // measured: at 64 rows per expert the 128-row-tile kernel is faster
inline int fp8_pad_rows(int64_t assignments, int experts) {
  return assignments <= int64_t(kFp8ColsMaxAvgRows) * experts ? kPadBf16 : kTileM;
}

// ---- peer.cu: cross-GPU stages over peer-mapped memory -------------------------------------
int launch_peer_barrier(const PeerTable& flags, int rank, int world, uint32_t seq, int* status,
                        cudaStream_t stream);
int launch_gather_routing(const PeerTable& ids, const PeerTable& weights, int rank, int world,
                          int per_rank, int* ids_all, float* weights_all, cudaStream_t stream);
int launch_gather_blocks_peer(const PeerTable& src, int rank, int world, int64_t bytes_per_rank, void* dst,
                              cudaStream_t stream);
int launch_gather_rows_peer_fp8(const PeerTable& x, const PeerTable& xs, int rank, int world, int tokens, int topk,
                                const Schedule& sched, int local_experts, int hidden, void* out_rows,
                                float* out_scales_t, int64_t row_capacity, cudaStream_t stream);
int launch_reduce_partials(const PeerTable& partial, int rank, int world, int tokens, int topk,
                           const int* topk_ids, int experts_per_rank, int hidden, __nv_bfloat16* out,
                           cudaStream_t stream, int fp16 = 0);

// ---- api.cu helpers shared with dist.cu -----------------------------------------------------
struct Layout {
  int64_t status, counts, prefix, sorted, inverse, scratch, xg, act, y, total;
  int64_t xs, acts;  // fp8 only: transposed activation scales [K/128][cap], [N/128][cap]
  int64_t xq_tok, xs_tok;  // fp8 only: the tokens quantised once, [T][K] e4m3 and [T][K/128] scales
  int64_t granules;  // arrival counter per 16-row granule of the sorted row buffer (fused dispatch)
  int64_t granule_bytes;
  int64_t blocks;    // completion counter per token block (fused combine push)
  int64_t block_bytes;
  int64_t counter_span;  // bytes from `granules` to the end of `blocks`
};
Layout make_layout(int precision, int64_t tokens, int hidden, int intermediate, int local_experts, int topk,
                   int pad_rows);
int64_t row_capacity(int64_t tokens, int topk, int local_experts, int pad_rows);
inline int pad_rows_of(int precision) { return precision == 1 /* fp8 */ ? kTileM : kPadBf16; }
inline int elem_bytes_of(int precision) { return precision == 1 /* fp8 */ ? 1 : 2; }
int check_shape(int64_t tokens, int hidden, int intermediate, int local_experts, int topk);
int check_shape_fp8(int hidden, int intermediate);
int run_gemm_stage(int mode, const void* a, int64_t cap, const void* w, int local_experts, int hidden,
                   int intermediate, const int* counts, const int* prefix, const int* sorted,
                   const float* row_scale, void* out, int* status, int device, cudaStream_t stream,
                   unsigned long long* clock_probe = nullptr, const FusedDispatch* dispatch = nullptr,
                   int fp16 = 0, const FusedPush* push = nullptr);
int run_gemm_stage_fp8(int mode, const void* a, const float* a_scale_t, int64_t cap, const void* w,
                       const float* w_scale, int local_experts, int hidden, int intermediate,
                       const int* counts, const int* prefix, const int* sorted, const float* row_scale,
                       void* out, float* out_scale_t, int* status, int device, cudaStream_t stream,
                       unsigned long long* clock_probe = nullptr, int pad_rows = kTileM,
                       const FusedDispatchFp8* dispatch = nullptr, const FusedPush* push = nullptr);
void mark_stage(int i, cudaStream_t s);

// ---- tensormap.cu ----------------------------------------------------------------------
// Row-major 2-D tensor [rows][cols] of elem_bytes elements, boxes of
// box_rows x (128 bytes of columns), 128-byte swizzle.
int make_tensor_map_2d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t rows,
                       uint64_t cols, uint32_t box_rows, int fp16 = 0);

}  // namespace mb200
