/*
 * moe_bench_b200 -- C ABI of the B200 (sm_100a) MoE layer forward.
 *
 * The library is the native side of a moe_bench `MoEImplementation`
 * (reference baseline.py:24-44) / `DistributedScheme` (reference
 * schemes.py:40-61): the plugin's `run()` passes the tensors of a `MoEProblem`
 * (reference data.py:24-61) as raw device pointers.  moe_bench itself has no
 * native boundary for this path (its baseline calls vLLM's Python
 * `fused_experts`, baseline.py:67-76; its experimental kernels are a pybind11
 * module, kernels/tk/tk_moe.cu:1521-1540), so each entry point below cites the
 * reference code whose work it performs.
 *
 * Conventions
 *  - every pointer is a device pointer on the current CUDA device unless said
 *    otherwise; `stream` is a cudaStream_t passed as void*;
 *  - functions return 0 on success, a positive code on error
 *    (1 invalid argument, 2 CUDA error, 3 driver entry point missing,
 *    4 workspace too small, 5 unsupported shape); `mb200_last_error()` gives
 *    the message of the calling thread's last failure;
 *  - entry points only enqueue work on `stream`: no allocation, no
 *    synchronisation, no host reads of device memory (except
 *    `mb200_read_status`), so they may be called under stream capture;
 *  - kernels never spin without a limit: a wait that expires stores
 *    100 + <wait site> in the workspace status word and the kernel returns.
 */
#ifndef MOE_BENCH_B200_H_
#define MOE_BENCH_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MB200_ABI_VERSION 5
#define MB200_PRECISION_BF16 0
#define MB200_PRECISION_FP8 1
#define MB200_PRECISION_FP16 2 /* the bf16 data flow with IEEE half operands and outputs */
#define MB200_PAD_ROWS_BF16 16 /* bf16 forward: expert segments are padded to 16 rows */
#define MB200_PAD_ROWS_FP8 128 /* fp8 forward: expert segments are padded to 128 rows */

int mb200_abi_version(void);
const char* mb200_last_error(void);

/* Router front end: softmax over `experts` logits, top-k (largest first, lowest
 * index wins ties), weights renormalised over the selection.
 * logits [tokens, experts] fp32 -> topk_ids [tokens, topk] int32,
 * topk_weights [tokens, topk] fp32.  The reference has no router: it draws ids
 * and weights directly (data.py:178-235). */
int mb200_route_topk(const float* logits, int tokens, int experts, int topk, int32_t* topk_ids,
                     float* topk_weights, void* stream);

/* Rows the sorted/padded assignment list can need: tokens*topk plus up to
 * pad_rows-1 padding rows per expert that can be hit, rounded up to pad_rows. */
int64_t mb200_row_capacity(int64_t tokens, int topk, int local_experts, int pad_rows);
int64_t mb200_align_scratch_bytes(int64_t tokens, int topk, int local_experts);

/* Sort-and-pad of token->expert assignments (the moe_align_block_size step of
 * fused_experts, baseline.py:67; slot order of tk_scheme.py:98-126).
 * topk_ids [tokens, topk] int32 global ids; expert_map [global experts] int32
 * (global id -> local slot or -1) or NULL when every expert is local.
 * Every expert's segment is padded to a multiple of pad_rows rows
 * (MB200_PAD_ROWS_BF16 / MB200_PAD_ROWS_FP8 for the two GEMM families).
 * counts [E], mtile_prefix [E+1] (cumulative pad_rows-row blocks; padded row offset
 * of expert e is pad_rows*mtile_prefix[e]), sorted_ids [row_capacity] (flat assignment
 * index token*topk+kpos per row, -1 for padding), inverse [tokens*topk] (row of
 * each assignment, -1 if its expert is not local). */
int mb200_align(const int32_t* topk_ids, int64_t tokens, int topk, const int32_t* expert_map,
                int local_experts, int32_t* counts, int32_t* mtile_prefix, int32_t* sorted_ids,
                int32_t* inverse, int64_t row_capacity, int pad_rows, void* scratch, void* stream);

/* mb200_align for callers that cannot allocate device memory.  It has no
 * counterpart in the reference.
 *
 * Who needs it: a serving process that gave all of HBM to its own memory pool
 * at start-up cannot get a scratch buffer from cudaMalloc later, and a decode
 * loop with a latency budget cannot afford the device-wide stall a
 * cudaMalloc/cudaFree causes.  Here the sort's scratch (per-unit expert
 * histograms) is a fixed 1 MiB array inside the library, so the caller passes
 * only inputs and outputs and the call allocates nothing (no cudaMalloc,
 * cudaFree or allocating library routine).
 *
 * Limits and rules:
 *  - local_experts <= MB200_NOALLOC_MAX_LOCAL_EXPERTS and tokens*topk <=
 *    MB200_NOALLOC_MAX_ASSIGNMENTS; larger problems are refused with status 5
 *    and a message naming mb200_align as the alternative;
 *  - every GPU that loads the library holds the 1 MiB array until the process
 *    exits, whether or not this entry point is used;
 *  - the first call on a device looks up the array's device address
 *    (cudaGetSymbolAddress, with that device current); make that first call
 *    before starting any stream capture;
 *  - all calls on one device share the array, which keeps whatever the last call
 *    left in it (nothing needs clearing: each call overwrites what it reads).
 *    Calls that can overlap on the GPU (different streams, or concurrent host
 *    threads) race on it; serialise them, or use mb200_align with one scratch
 *    buffer per stream.
 * Arguments and outputs are those of mb200_align. */
#define MB200_NOALLOC_MAX_LOCAL_EXPERTS 256
#define MB200_NOALLOC_MAX_ASSIGNMENTS 1048576
int mb200_align_noalloc(const int32_t* topk_ids, int64_t tokens, int topk,
                        const int32_t* expert_map, int local_experts, int32_t* counts,
                        int32_t* mtile_prefix, int32_t* sorted_ids, int32_t* inverse,
                        int64_t row_capacity, int pad_rows, void* stream);

/* Dynamic activation quantisation, one fp32 scale per row per 128 elements
 * (reference.py:143-145 -> vLLM per_token_group_quant_fp8).
 * x [rows, hidden] bf16 -> q [rows, hidden] e4m3, scales [rows, hidden/128]. */
int mb200_group_quant_fp8(const void* x, int64_t rows, int hidden, void* q, float* scales,
                          void* stream);

/* One grouped GEMM stage on an existing schedule padded to MB200_PAD_ROWS_BF16
 * (stage-level checks; the forward entry points run both).  mode 0: act[row, 0:N] =
 * SiLU(a.w1[e,0:N]) * (a.w1[e,N:2N]) for a [row_capacity, hidden] bf16 holding
 * the sorted rows, w1 [E, 2N, hidden], act [row_capacity, N] (reference.py:113-114).
 * mode 1: y[n, 0:hidden] = row_scale[n] * (a.w2[e]) for a [row_capacity, N],
 * w2 [E, hidden, N], y [tokens*topk, hidden] indexed by the flat assignment n
 * (reference.py:115,180-181).  status: the head of a status block in device
 * memory, two int32 zeroed by the caller: [0] receives the first failure code of
 * a kernel (0 = none), [1] is the limit of one in-kernel wait in milliseconds
 * (0 = the default of 4 s). */
int mb200_grouped_gemm_bf16(int mode, const void* a, int64_t row_capacity, const void* w,
                            int local_experts, int hidden, int intermediate, const int32_t* counts,
                            const int32_t* mtile_prefix, const int32_t* sorted_ids,
                            const float* row_scale, void* out, int32_t* status, int device,
                            void* stream);

/* The gate/up stage (mode 0 above) for rows that SOMEONE ELSE delivers while the
 * kernel runs: another kernel on another stream, or a peer GPU that pushes rows
 * into `a` (the reference's push dispatch signals row blocks the same way,
 * kernels/tk/tk_moe.cu:647-821).  granule_done[row_capacity/16] counts arrivals
 * per 16-row granule of `a`; the kernel loads a token block only after every
 * granule it spans has reached granule_target (acquire), and gives up with
 * status 106 when one does not within the wait limit of the status block -
 * the launch then ends normally and the context stays usable. */
int mb200_grouped_gemm_bf16_gated(const void* a, int64_t row_capacity, const void* w, int local_experts,
                                  int hidden, int intermediate, const int32_t* counts,
                                  const int32_t* mtile_prefix, const int32_t* sorted_ids,
                                  const int32_t* granule_done, int granule_target, void* out,
                                  int32_t* status, int device, void* stream);

/* Bytes of caller-provided workspace for one forward of the given shape. */
int64_t mb200_workspace_bytes(int precision, int64_t tokens, int hidden, int intermediate,
                              int local_experts, int topk);

/* Where the forward entry points keep their intermediate tables inside the
 * workspace, for checks that read them back (the reference validates its
 * dispatch by comparing the gathered rows with x[src] byte for byte,
 * tools/validate_push3.py:90-95).  `tokens` is the number of token rows the
 * call sorts (mb200_dist_forward: tokens * world); expected_rows = the
 * assignments expected on this rank (tokens*topk, or that divided by world for
 * expert parallel), which picks the fp8 kernel family and its padding.
 * out10 = { pad_rows, row_capacity, then byte offsets of: counts[E],
 * mtile_prefix[E+1], sorted_ids[row_capacity], inverse[tokens*topk], the sorted
 * row buffer [row_capacity][hidden] (16-bit or e4m3), its scales
 * [hidden/128][row_capacity] (fp8, else 0), act [row_capacity][intermediate],
 * y [tokens*topk][hidden] }. */
int mb200_forward_layout(int precision, int64_t tokens, int hidden, int intermediate, int local_experts,
                         int topk, int64_t expected_rows, int64_t* out10);

/* The layer forward, bf16 (reference.py:98-116 + 170-182; baseline.py:62-76):
 * out[t, :] = sum_j topk_weights[t, j] * ( SiLU(x_t.w1g[e]) * (x_t.w1u[e]) ) . w2[e],
 * e = expert_map[topk_ids[t, j]], skipping experts that are not local.
 * hidden_states [tokens, hidden] bf16; w1 [E_local, 2*intermediate, hidden]
 * (gate rows, then up rows); w2 [E_local, hidden, intermediate]; out
 * [tokens, hidden] bf16.  The workspace may be reused by the next call on the
 * same stream; calls that overlap on the device need separate workspaces.
 * The first 256 bytes of the workspace are the status block: the caller zeroes
 * them once before the first call (and again after a reported failure).  Word 0
 * keeps the FIRST failure code of any kernel (100 + site: a bounded in-kernel
 * wait ran out; 150 + peer: a cross-GPU barrier did); while it is non-zero the
 * outputs are not to be trusted - read it with mb200_read_status at a point
 * where the host synchronises anyway.  Word 1 is the limit of one in-kernel
 * wait in milliseconds (0 = 4 s); word 2 is the limit of one cross-GPU barrier
 * in milliseconds (0 = 3 s) - raise it where ranks may reach a barrier further
 * apart than that (a first call that still loads modules, a stalled host). */
int mb200_moe_forward_bf16(const void* hidden_states, const void* w1, const void* w2,
                           const int32_t* topk_ids, const float* topk_weights,
                           const int32_t* expert_map, void* out, int64_t tokens, int hidden,
                           int intermediate, int local_experts, int topk, void* workspace,
                           int64_t workspace_bytes, int device, void* stream);

/* The same forward with fp16 tensors (Precision.FP16, config.py:54 and 212-213;
 * the reference checks it at atol 1e-2, reference.py:41).  Every 16-bit tensor
 * (hidden_states, w1, w2, out) is IEEE half; accumulation stays fp32 and the
 * intermediate activation and the per-assignment rows are rounded to half where
 * the bf16 forward rounds to bf16.  Workspace: mb200_workspace_bytes with
 * MB200_PRECISION_FP16 (the same size as bf16). */
int mb200_moe_forward_fp16(const void* hidden_states, const void* w1, const void* w2,
                           const int32_t* topk_ids, const float* topk_weights,
                           const int32_t* expert_map, void* out, int64_t tokens, int hidden,
                           int intermediate, int local_experts, int topk, void* workspace,
                           int64_t workspace_bytes, int device, void* stream);

/* fp8 counterpart of mb200_grouped_gemm_bf16 (reference.py:65-95 block matmul), on
 * a schedule padded to MB200_PAD_ROWS_FP8.
 * a: e4m3 [row_capacity, K] sorted rows; a_scale_t: fp32 [K/128][row_capacity]
 * (group-major); w: e4m3 weights; w_scale: fp32 [E, rows/128, K/128].
 * mode 0 writes out = e4m3 [row_capacity, N] (SiLU(gate)*up rounded to bf16, then
 * re-quantised per row per 128, reference.py:156-163) and out_scale_t
 * [N/128][row_capacity]; mode 1 writes out = bf16 [tokens*topk, hidden] scaled by
 * row_scale. */
int mb200_grouped_gemm_fp8(int mode, const void* a, const float* a_scale_t, int64_t row_capacity,
                           const void* w, const float* w_scale, int local_experts, int hidden,
                           int intermediate, const int32_t* counts, const int32_t* mtile_prefix,
                           const int32_t* sorted_ids, const float* row_scale, void* out,
                           float* out_scale_t, int32_t* status, int device, void* stream);

/* The same two stages on a schedule padded to MB200_PAD_ROWS_BF16 (16 rows), with
 * the tokens on the MMA N dimension: what the fp8 forward uses when experts get
 * few rows each (at most 24 on average), where 128-row token tiles would be
 * mostly padding.  Arguments as mb200_grouped_gemm_fp8. */
int mb200_grouped_gemm_fp8_cols(int mode, const void* a, const float* a_scale_t, int64_t row_capacity,
                                const void* w, const float* w_scale, int local_experts, int hidden,
                                int intermediate, const int32_t* counts, const int32_t* mtile_prefix,
                                const int32_t* sorted_ids, const float* row_scale, void* out,
                                float* out_scale_t, int32_t* status, int device, void* stream);

/* The layer forward with fp8 block-quantised weights (reference.py:119-167 +
 * 170-182; baseline.py:62-76 with quant_config).  w1/w2 are e4m3 with fp32
 * scales w1_scale [E_local, 2*intermediate/128, hidden/128] and w2_scale
 * [E_local, hidden/128, intermediate/128]; hidden_states and out are bf16.
 * Activations are quantised per token per 128 elements on the fly. */
int mb200_moe_forward_fp8(const void* hidden_states, const void* w1, const void* w2,
                          const float* w1_scale, const float* w2_scale, const int32_t* topk_ids,
                          const float* topk_weights, const int32_t* expert_map, void* out,
                          int64_t tokens, int hidden, int intermediate, int local_experts, int topk,
                          void* workspace, int64_t workspace_bytes, int device, void* stream);

/* ---- distributed layer: one process per GPU, peers' buffers mapped by the caller ----
 *
 * Replaces the serial scheme's AllGather -> fused_experts -> ReduceScatter
 * (schemes.py:117-143) for both parallel modes of config.py:18-35:
 *   expert_parallel = 1  rank r owns experts [r*E_local, (r+1)*E_local) (data.py:238-253)
 *   expert_parallel = 0  tensor parallel: all experts, intermediate/world columns
 * Every rank passes its own token shard (hidden_states [tokens, hidden], routing
 * over GLOBAL expert ids) and receives its own rows of the combined output.
 * precision: MB200_PRECISION_BF16, _FP8 (bf16 tokens and output, e4m3 weights
 * with scales) or _FP16 (half tokens, weights and output; scales unused).
 *
 * symmetric_ptrs[world]: base pointers, valid in THIS process, of one buffer per
 * rank with mb200_dist_symmetric_bytes() bytes, 1024-byte aligned, zero-filled
 * once after allocation; entry [rank] is this rank's own buffer.  Token rows are
 * LOADED from the peers' buffers (dispatch); what the library STORES into a
 * peer's buffer are 4-byte barrier flags and, expert parallel, the weighted
 * output rows of that peer's tokens (combine by push into its receive area).
 * One forward = stage own tokens and routing | barrier | routing of all ranks,
 * sort-and-pad | gate/up GEMM whose helper warps pull the rows it needs over
 * NVLink | down GEMM whose helper warps push finished rows to the tokens' owners
 * | barrier | sum of the k rows of every own token.  (Tensor parallel: peers'
 * token blocks are gathered before the GEMM and each rank pushes the sum over a
 * token's k rows to the owner, who sums W planes; two barriers.  fp8 with at
 * most 24 rows per expert: rows gathered before the GEMM, pre-reduced partial
 * rows pulled after a barrier; three barriers.)
 * seq_base: a counter that is equal on all ranks and grows by
 * MB200_DIST_SEQ_STRIDE per call (barrier sequence numbers are never reset).
 * All ranks must make the same calls in the same order.  A barrier that does not
 * complete within 3 s stores 150+peer in the workspace status word and the call's
 * kernels carry on, so the context stays usable; the output is then undefined. */
#define MB200_DIST_SEQ_STRIDE 4
int64_t mb200_dist_symmetric_bytes(int precision, int64_t tokens, int hidden, int topk, int world);
int64_t mb200_dist_workspace_bytes(int precision, int64_t tokens, int hidden, int intermediate,
                                   int local_experts, int topk, int world);
int mb200_dist_forward(int precision, int expert_parallel, const void* hidden_states, const void* w1,
                       const void* w2, const float* w1_scale, const float* w2_scale,
                       const int32_t* topk_ids, const float* topk_weights, const int32_t* expert_map,
                       void* out, int64_t tokens, int hidden, int intermediate, int local_experts,
                       int global_experts, int topk, int rank, int world, void* const* symmetric_ptrs,
                       int64_t symmetric_bytes, uint32_t seq_base, void* workspace, int64_t workspace_bytes,
                       int device, void* stream);
/* The all-rank barrier used inside mb200_dist_forward, exposed for set-up and
 * tear-down (protocol of sm120_common.cuh:47-64, with a time limit).  status:
 * null, or the head of a status block in device memory, four int32 zeroed by
 * the caller: [0] receives 150 + peer when that peer did not arrive in time,
 * [2] is the limit in milliseconds (0 = 3 s); [1] and [3] are not used here. */
int mb200_peer_barrier(void* const* symmetric_ptrs, int rank, int world, uint32_t seq, int32_t* status,
                       void* stream);

/* Set-up only: a zero-filled device buffer that other processes on the same box
 * can map through CUDA IPC (for hosts without another way to share GPU memory;
 * the reference's TK path uses a VMM/IPC broker, experience/11:13-21).  alloc
 * returns the pointer and a 64-byte handle to send to the peers; open maps a
 * peer's handle; close/free undo them.  These four are the only allocating
 * entry points and are never called from the forward path. */
int mb200_ipc_alloc(int64_t bytes, void** ptr_out, void* handle_out64);
int mb200_ipc_open(const void* handle64, void** ptr_out);
int mb200_ipc_close(void* ptr);
int mb200_ipc_free(void* ptr);

/* Per-stage timing hook for benchmarks.  After mb200_set_stage_events(ev, 6) the
 * forward entry points called from this thread record ev[0] before the first
 * stage and ev[1..5] after the sort-and-pad, row gather, gate/up GEMM, down GEMM
 * and combine stages (cudaEvent_t handles created by the caller).  Call with
 * (NULL, 0) to switch it off.  moe_bench times whole calls only
 * (bench.py:52-101); this exists so one kernel's duration can be read inside a
 * timed region. */
int mb200_set_stage_events(void* const* events, int count);

/* The forward entry points also leave, in the first 256 bytes of the workspace
 * (after the status word at byte 0), two pairs of uint64 at byte 32 and byte 48:
 * {SM cycles, nanoseconds} that CTA 0 of the gate/up and of the down GEMM spent
 * in the kernel during the last call; cycles/ns is the SM clock in GHz the kernel
 * really ran at (a power-capped part runs tensor kernels far below the clock
 * that the management library reports between kernels). */

/* Format of the fp8 ACTIVATION scales (one per token per 128 elements) that the
 * calling thread's later calls compute, in the input quantiser and in the gate/up
 * GEMM's re-quantiser.  The reference obtains them from vLLM's
 * per_token_group_quant_fp8 (reference.py:143-145,157-163), whose result depends
 * on the platform: plain fp32 amax/448, or - when vLLM runs with DeepGEMM's E8M0
 * scales, its default on Hopper and Blackwell GPUs (vllm/utils/deep_gemm.py,
 * is_deep_gemm_e8m0_used) - that value rounded up to a power of two.  To verify
 * against the reference on a given box the library has to quantise the way the
 * reference does there; moe_bench_b200.plugin asks vLLM when it is importable.
 * Weight scales are inputs and are used as given.  Default: MB200_FP8_SCALES_FP32. */
#define MB200_FP8_SCALES_FP32 0
#define MB200_FP8_SCALES_UE8M0 1
int mb200_set_fp8_scale_format(int format);

/* Decomposition aid (the reference times dispatch and combine without the GEMMs in
 * tools/time_dispatch.py and tools/analyze_overlap.py:88-100).  While enabled for
 * the calling thread, the forward entry points launch the same kernels but with
 * zero K steps: routing exchange, barriers, dispatch of rows, stores and combine
 * traffic all happen, the arithmetic does not, and the outputs mean nothing. */
int mb200_set_comm_only(int enabled);

/* Copies the workspace status word to the host after synchronising `stream`
 * (0 = no kernel gave up a wait).  Not capturable. */
int mb200_read_status(const void* workspace, int32_t* status_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOE_BENCH_B200_H_ */
