// Grouped per-expert GEMMs on e4m3 operands with fp32 software block scales.
//
// Scales follow the reference's w8a8 block scheme (reference.py:65-95,119-167):
// one fp32 scale per 128x128 weight block and one per activation row per 128
// elements of K.  The weight scales are plain fp32 numbers (amax/448), not powers
// of two (the activation scales are either, see fp8_group_scale), so the hardware
// block-scaled MMA cannot apply them.  Instead every 128-deep K block is multiplied
// on the tensor cores into its own tensor-memory buffer (tcgen05.mma kind::f8f6f4,
// 4 x K32) and the epilogue warps promote it:
//     acc += partial * (a_scale[row, kb] * w_scale[nblock, kb])
// in fp32 registers, in ascending K-block order like the reference.  Two
// 256-column partial buffers let the promotion of block kb overlap the MMAs of
// block kb+1.
//
// Roles per CTA (384 threads, register file re-split with setmaxnreg): warp 0 TMA
// producer (4-stage ring, one stage = one K block: 128 rows x 128 B of A + 256 rows
// x 128 B of weights, plus the K block's 128 activation scales as a 512-byte bulk
// copy on the same barrier), warp 1 tensor-memory owner and MMA issuer, warps 2-3
// helpers (gate/up: the dispatch - they pull e4m3 rows and scales of the tile's
// tokens from their source ranks, or gather them locally, granule by granule; down,
// expert parallel: they push finished rows to the ranks that own the tokens),
// warps 4-11 epilogue.  Epilogue warp w reads tensor-memory lanes 32*(w%4).. (one
// accumulator row per thread) and one column half: 128 fp32 accumulators per thread,
// held as 64 packed pairs and updated with fma.rn.f32x2.
//   gate/up:  columns = 64 gate + the matching 64 up outputs; at the end of the
//             tile SiLU(gate)*up is rounded to bf16 and re-quantised per row over
//             the tile's 128 outputs (= one quantisation group, amax exchanged
//             between the two column halves through shared memory), so the
//             second GEMM's A operand reaches HBM only as e4m3 + scales
//             (reference.py:156-163).  Rows past the expert's last one are zeroed
//             first (their garbage would send the divisions down the slow path).
//   down:     columns = 128 outputs = one weight scale block; scaled by the
//             combine weight, transposed through a per-warp block of shared memory
//             and stored as bf16, 64 contiguous bytes per row, at the row's flat
//             assignment.

#include <atomic>

#include "layer.cuh"

namespace mb200 {

namespace {

constexpr int kStages = 4;
constexpr int kABytes = kTileM * 128;
constexpr int kBBytes = 256 * 128;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kAccCols = 256;
constexpr int kTmemCols = 512;
constexpr int kEpilogueWarps = 8;
constexpr int kFirstEpilogueWarp = 4;  // warps 0-3: one warpgroup of helpers (TMA, MMA, two spare)
constexpr int kThreads = (kFirstEpilogueWarp + kEpilogueWarps) * 32;
// Registers per thread after the warpgroups re-split the register file (setmaxnreg): the
// epilogue threads hold 128 accumulators + two 32-register load buffers, the helpers need few.
// 128 * helper + 256 * epilogue <= 65536.  The split is per kernel: these are the ones the
// compiler fits without spilling (64 + 216 for both at present).
template <int kMode> struct RegSplit { static constexpr int kHelper = 64, kEpilogue = 216; };
template <> struct RegSplit<kDownWeighted> { static constexpr int kHelper = 64, kEpilogue = 216; };
constexpr int kMaxKBlocks = 128;  // K up to 16384
constexpr int kScaleSlots = kStages + 2 + 1;
constexpr int kXposePitch = 80;
constexpr int kHelperLoads = 7;  // 16-byte loads a lane of the dispatch / push warps keeps in flight

struct SmemTail {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t part_full[2];
  uint64_t part_empty[2];
  uint64_t epi_bar;
  uint32_t tmem_base;
  int abort_flag;
  float wscale[2][2][kMaxKBlocks];  // [tile parity][column half / gate,up][k block]
  float amax[2][kTileM];            // [column half][row]
  // activation scales of the K blocks in flight, one 128-row slice per K block, filled by the
  // TMA warp together with the stage (a load the epilogue threads issued themselves would wait
  // microseconds behind the weight stream).  A slot is reused only after the epilogue has
  // folded its K block in: the loader is at most kStages blocks ahead of the tensor core and
  // that at most 2 partial buffers ahead of the epilogue.
  alignas(16) float ascale[kScaleSlots][kTileM];
  // down GEMM: per-warp block the output rows are transposed through, 32 rows x 64 bytes (+16 pad)
  alignas(16) uint8_t xpose[kEpilogueWarps][32 * kXposePitch];
  int prefix[kMaxExperts + 1];
};

constexpr size_t kSmemBytes = 1024 + size_t(kStages) * kStageBytes + sizeof(SmemTail);
static_assert(kSmemBytes <= 227 * 1024, "shared memory of the fp8 kernel");

struct TileCoord {
  int expert, n_tile, row0, valid_rows;
};

__device__ __forceinline__ TileCoord decode_tile(int tile, const int* prefix, const int* counts,
                                                 int num_experts, int n_tiles) {
  int lo = 0, hi = num_experts;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (prefix[mid] * n_tiles <= tile) lo = mid; else hi = mid - 1;
  }
  TileCoord c;
  c.expert = lo;
  int local = tile - prefix[lo] * n_tiles;
  int m_tiles = prefix[lo + 1] - prefix[lo];
  c.n_tile = local / m_tiles;
  int m_local = local - c.n_tile * m_tiles;
  c.row0 = (prefix[lo] + m_local) * kTileM;
  int left = __ldg(counts + lo) - m_local * kTileM;
  c.valid_rows = left < kTileM ? left : kTileM;
  return c;
}

// Barrier among the epilogue warps, built on an mbarrier so that, like every
// other wait in the kernel, it gives up after the wait limit instead of hanging.
__device__ __forceinline__ bool epilogue_barrier(uint64_t* bar, uint32_t& phase, WaitCtx& ctx, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(smem_u32(bar));
  const bool ok = mbar_wait(smem_u32(bar), phase, ctx, 5);
  phase ^= 1;
  return ok;
}

__device__ __forceinline__ float bf16_round(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

__device__ __forceinline__ float silu_mul(float g, float u) {
  // fast reciprocal: ~2 ulp, far inside the bf16 rounding that follows
  return __fdividef(g, 1.0f + __expf(-g)) * u;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

template <int kMode>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_fp8_kernel(const __grid_constant__ CUtensorMap map_a,
                        const __grid_constant__ CUtensorMap map_b, const GemmFp8Args args,
                        const FusedDispatchFp8 disp, const FusedPush push) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t tiles_addr = raw_addr + pad;
  SmemTail* tail = reinterpret_cast<SmemTail*>(smem + size_t(kStages) * kStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    prefetch_tmap(&map_a);
    prefetch_tmap(&map_b);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&tail->full[s]), 1);
      mbar_init(smem_u32(&tail->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&tail->part_full[b]), 1);
      mbar_init(smem_u32(&tail->part_empty[b]), kEpilogueWarps);
    }
    mbar_init(smem_u32(&tail->epi_bar), kEpilogueWarps);
    tail->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tail->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  for (int i = threadIdx.x; i <= args.num_experts; i += kThreads) tail->prefix[i] = args.mtile_prefix[i];
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const unsigned long long probe_c0 = clock64(), probe_t0 = global_timer_ns();
  const uint32_t tmem_base = tail->tmem_base;
  const int total_tiles = tail->prefix[args.num_experts] * args.n_tiles;
  const int k_blocks = args.k_blocks;
  WaitCtx ctx{&tail->abort_flag, args.status, wait_limit_ns(args.status)};

  // Each role's code sits inside the branch that re-sizes its warpgroup's registers, so the
  // compiler knows which budget applies where.
  if (warp < kFirstEpilogueWarp) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(RegSplit<kMode>::kHelper));
  if (warp == 0) {
    // ---------------- TMA producer ----------------
    int stage = 0;
    uint32_t phase = 0;
    uint32_t slot = 0;  // scale slot of the K block being loaded
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      TileCoord tc = decode_tile(tile, tail->prefix, args.counts, args.num_experts, args.n_tiles);
      const int b_row = tc.expert * args.b_rows_per_expert;
      if (kMode == kGateUpSwiglu && disp.enabled) {
        // the eight 16-row granules of this token tile must have been dispatched
        const int g0 = tc.row0 / 16;
        uint32_t spins = 0;
        WaitClock clock;
        while (true) {
          int v = kFp8HelperWarps;
          if (lane < kTileM / 16)
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(disp.granule_done + g0 + lane) : "memory");
          if (__all_sync(0xffffffffu, v >= kFp8HelperWarps)) break;
          if ((++spins & 0x3F) == 0) {
            const bool aborted = __any_sync(0xffffffffu, *ctx.abort_flag != 0);
            const bool late = __any_sync(0xffffffffu, clock.expired(ctx));
            if (aborted || late) {
              if (!aborted && lane == 0) wait_give_up(ctx, 6);
              ok = false;
              break;
            }
            __nanosleep(128);
          }
        }
        if (!ok) break;
        // rows and scales were written with ordinary stores by other SMs; the TMA engine reads them
        asm volatile("fence.proxy.async;" ::: "memory");
      }
      for (int kb = 0; kb < k_blocks; ++kb) {
        ok = mbar_wait(smem_u32(&tail->empty[stage]), phase ^ 1, ctx, 1);
        if (!ok) break;
        if (lane == 0) {
          const uint32_t bar = smem_u32(&tail->full[stage]);
          const uint32_t a_dst = tiles_addr + stage * kStageBytes;
          const uint32_t b_dst = a_dst + kABytes;
          const int kcol = kb * 128;
          mbar_expect_tx(bar, kStageBytes + kTileM * 4);
          tma_load_1d(smem_u32(tail->ascale[slot]), args.a_scale_t + size_t(kb) * args.row_capacity + tc.row0,
                      kTileM * 4, bar);
          tma_load_2d(a_dst, &map_a, kcol, tc.row0, bar);
          if (kMode == kGateUpSwiglu) {
            tma_load_2d(b_dst, &map_b, kcol, b_row + tc.n_tile * 128, bar);
            tma_load_2d(b_dst + kBBytes / 2, &map_b, kcol,
                        b_row + args.b_half_offset + tc.n_tile * 128, bar);
          } else {
            tma_load_2d(b_dst, &map_b, kcol, b_row + tc.n_tile * 256, bar);
          }
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1; }
        if (++slot == kScaleSlots) slot = 0;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: one K block per partial buffer ----------------
    constexpr uint32_t idesc = make_idesc(0, 0, kTileM, kAccCols);  // e4m3 x e4m3 -> fp32
    int stage = 0;
    uint32_t phase = 0;
    uint32_t pit = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      for (int kb = 0; kb < k_blocks; ++kb, ++pit) {
        const uint32_t pbuf = pit & 1;
        ok = mbar_wait(smem_u32(&tail->full[stage]), phase, ctx, 3);
        if (!ok) break;
        ok = mbar_wait(smem_u32(&tail->part_empty[pbuf]), ((pit >> 1) & 1) ^ 1, ctx, 2);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_addr = tiles_addr + stage * kStageBytes;
          const uint64_t a_desc = make_kmajor_sw128_desc(a_addr);
          const uint64_t b_desc = make_kmajor_sw128_desc(a_addr + kABytes);
          const uint32_t d_tmem = tmem_base + pbuf * kAccCols;
#pragma unroll
          for (int k = 0; k < 4; ++k)  // 32 e4m3 = 32 bytes of K per instruction
            umma_fp8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, k != 0);
          tc_commit(smem_u32(&tail->empty[stage]));
          tc_commit(smem_u32(&tail->part_full[pbuf]));
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (kMode == kGateUpSwiglu) {
    // ---------------- warps 2-3, gate/up: fused dispatch ----------------
    // Fill the sorted row buffer 16-row granule by granule (granules strided over the CTAs in
    // row order): the token's e4m3 row and its 1x128 scales, from this GPU's quantised tokens
    // or, expert-parallel, with P2P loads from the source rank over NVLink.  These warps
    // never wait; the TMA warp starts a tile once its eight granules have arrived.
    if (disp.enabled) {
      const int dw = warp - 2;
      const int granules = tail->prefix[args.num_experts] * (kTileM / 16);
      const int vec_per_row = disp.groups_per_row * 8;
      for (int g = blockIdx.x; g < granules; g += gridDim.x) {
        for (int i = dw; i < 16; i += kFp8HelperWarps) {
          const int row = g * 16 + i;
          const int n = __ldg(args.sorted_ids + row);
          if (n >= 0) {
            const int tok_global = n / disp.topk;
            const int ring = tok_global / disp.tokens_per_rank;
            const int t = tok_global - ring * disp.tokens_per_rank;
            const int src_rank = (disp.rank + ring) % disp.world;
            const uint4* src = reinterpret_cast<const uint4*>(disp.xq.ptr[src_rank]) + size_t(t) * vec_per_row;
            const float* src_s = reinterpret_cast<const float*>(disp.xs.ptr[src_rank]) + size_t(t) * disp.groups_per_row;
            uint4* dst = disp.rows_out + size_t(row) * vec_per_row;
            float sc[2];
#pragma unroll
            for (int u = 0; u < 2; ++u)
              if (lane + 32 * u < disp.groups_per_row) sc[u] = src_s[lane + 32 * u];
            for (int v0 = lane; v0 < vec_per_row; v0 += 32 * kHelperLoads) {
              uint4 buf[kHelperLoads];
#pragma unroll
              for (int u = 0; u < kHelperLoads; ++u)
                if (v0 + u * 32 < vec_per_row) buf[u] = src[v0 + u * 32];
#pragma unroll
              for (int u = 0; u < kHelperLoads; ++u)
                if (v0 + u * 32 < vec_per_row) dst[v0 + u * 32] = buf[u];
            }
#pragma unroll
            for (int u = 0; u < 2; ++u)
              if (lane + 32 * u < disp.groups_per_row)
                disp.scales_t_out[size_t(lane + 32 * u) * args.row_capacity + row] = sc[u];
            for (int gi = lane + 64; gi < disp.groups_per_row; gi += 32)  // hidden > 8192
              disp.scales_t_out[size_t(gi) * args.row_capacity + row] = src_s[gi];
          }
        }
        __threadfence();  // this warp's rows before its arrival count
        __syncwarp();
        if (lane == 0) atomicAdd(disp.granule_done + g, 1);
      }
    }
  } else {
    // ---------------- warps 2-3, down GEMM: fused combine push (expert parallel) ----------------
    // A 16-row granule is forwarded to the GPUs that own its tokens once all feature blocks of
    // its 128-row tile have been stored (counted per tile by the epilogue warps of whichever
    // CTAs computed them).  The GEMM warps never wait for these warps.
    if (push.enabled) {
      const int pw = warp - 2;
      const int granules = tail->prefix[args.num_experts] * (kTileM / 16);
      const int target = args.n_tiles * kEpilogueWarps;
      bool ok = true;
      for (int g = blockIdx.x; ok && g < granules; g += gridDim.x) {
        const int tb = g / (kTileM / 16);
        uint32_t spins = 0;
        WaitClock clock;
        while (true) {
          int v;
          asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(push.block_done + tb) : "memory");
          if (v >= target) break;
          if ((++spins & 0x3F) == 0) {
            const bool aborted = __any_sync(0xffffffffu, *ctx.abort_flag != 0);
            const bool late = __any_sync(0xffffffffu, clock.expired(ctx));
            if (aborted || late) {
              if (!aborted && lane == 0) wait_give_up(ctx, 7);
              ok = false;
              break;
            }
          }
          __nanosleep(256);
        }
        if (!ok) break;
        for (int i = pw; i < 16; i += kFp8HelperWarps) {
          const int n = __ldg(args.sorted_ids + g * 16 + i);
          if (n >= push.own_rows) {  // a token of another rank (own tokens were stored in place; -1 = padding)
            const int ring = (n / push.topk) / push.tokens_per_rank;
            const int slot = n - ring * push.own_rows;
            const uint4* src = push.rows_in + size_t(n) * push.vec_per_row;
            uint4* dst = reinterpret_cast<uint4*>(push.dst.ptr[(push.rank + ring) % push.world]) +
                         size_t(slot) * push.vec_per_row;
            for (int v0 = lane; v0 < push.vec_per_row; v0 += 32 * kHelperLoads) {
              uint4 buf[kHelperLoads];
#pragma unroll
              for (int u = 0; u < kHelperLoads; ++u)
                if (v0 + u * 32 < push.vec_per_row) buf[u] = __ldcg(src + v0 + u * 32);
#pragma unroll
              for (int u = 0; u < kHelperLoads; ++u)
                if (v0 + u * 32 < push.vec_per_row) dst[v0 + u * 32] = buf[u];
            }
          }
        }
      }
      __threadfence_system();  // the stores to the peers are performed before the kernel ends
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(RegSplit<kMode>::kEpilogue));
    // ---------------- epilogue: promote partials, then finish the tile ----------------
    const int ew = warp - kFirstEpilogueWarp;
    const int quarter = warp & 3;
    const int half = ew >> 2;
    const int r = quarter * 32 + lane;
    const int etid = threadIdx.x - kFirstEpilogueWarp * 32;
    uint32_t pit = 0;
    uint32_t it = 0;
    uint32_t epi_phase = 0;
    uint32_t slot = 0;  // scale slot of the K block being folded in
    bool ok = true;
    // Weight scales of a tile, [half][kb]: thread i of the 256 fetches element i.  The fetch for
    // tile t+1 is issued while tile t is computed, so its latency never shows.
    auto fetch_wscale = [&](int tile) -> float {
      if (tile >= total_tiles || etid >= 2 * k_blocks) return 0.f;
      const TileCoord nt = decode_tile(tile, tail->prefix, args.counts, args.num_experts, args.n_tiles);
      const int h = etid / k_blocks, kb = etid - h * k_blocks;
      const int sblock = (kMode == kGateUpSwiglu) ? (h * args.scale_half_offset + nt.n_tile) : (2 * nt.n_tile + h);
      if (sblock >= args.scale_rows_per_expert) return 0.f;
      return __ldg(args.w_scale + (size_t(nt.expert) * args.scale_rows_per_expert + sblock) * k_blocks + kb);
    };
    float ws_next = fetch_wscale(blockIdx.x);
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
      TileCoord tc = decode_tile(tile, tail->prefix, args.counts, args.num_experts, args.n_tiles);
      const int par = it & 1;
      if (etid < 2 * k_blocks) (&tail->wscale[par][0][0])[(etid / k_blocks) * kMaxKBlocks + etid % k_blocks] = ws_next;
      ok = epilogue_barrier(&tail->epi_bar, epi_phase, ctx, lane);
      if (!ok) break;
      ws_next = fetch_wscale(tile + int(gridDim.x));

      const int row = tc.row0 + r;
      const bool row_ok = r < tc.valid_rows;
      // down GEMM: destination and combine weight of this thread's row, wanted at the end of the tile
      int assignment = -1;
      float row_w = 0.f;
      if (kMode == kDownWeighted && row_ok) {
        assignment = __ldg(args.sorted_ids + row);
        if (assignment >= 0) row_w = __ldg(args.row_scale + assignment);
      }
      // 128 fp32 accumulators per thread, kept as register pairs for fma.rn.f32x2:
      //   gate/up: pairs 0..31 = this thread's 64 gate columns, 32..63 = the matching up columns
      //   down:    pairs 0..63 = 128 consecutive output columns
      uint64_t acc[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) acc[i] = 0ull;
      // tensor-memory column of this thread's four 32-column chunks
      const uint32_t col0 = kMode == kGateUpSwiglu ? uint32_t(half * 64) : uint32_t(half * 128);
      const uint32_t col2 = kMode == kGateUpSwiglu ? uint32_t(128 + half * 64) : uint32_t(half * 128 + 64);

      for (int kb = 0; kb < k_blocks; ++kb, ++pit) {
        const uint32_t pbuf = pit & 1;
        ok = mbar_wait(smem_u32(&tail->part_full[pbuf]), (pit >> 1) & 1, ctx, 4);
        if (!ok) break;
        tc_fence_after();
        const float a_s = tail->ascale[slot][r];  // arrived with the stage this partial was computed from
        if (++slot == kScaleSlots) slot = 0;
        const uint32_t taddr = tmem_base + pbuf * kAccCols + (uint32_t(quarter * 32) << 16);
        // scale of the first two chunks and of the last two (gate / up weight blocks differ)
        const float s_lo = a_s * tail->wscale[par][kMode == kGateUpSwiglu ? 0 : half][kb];
        const float s_hi = kMode == kGateUpSwiglu ? a_s * tail->wscale[par][1][kb] : s_lo;
        const uint64_t s01 = pack_f32x2(__float_as_uint(s_lo), __float_as_uint(s_lo));
        const uint64_t s23 = pack_f32x2(__float_as_uint(s_hi), __float_as_uint(s_hi));
        // Promotion acc += partial * scale, software-pipelined: the tensor-memory load of
        // chunk c+1 is in flight while chunk c is folded in.
        uint32_t pa[32], pb[32];
        tmem_ld32(taddr + col0, pa);
        tmem_ld_wait32(pa);
        tmem_ld32(taddr + col0 + 32, pb);
#pragma unroll
        for (int j = 0; j < 16; ++j) fma_f32x2(acc[j], pack_f32x2(pa[2 * j], pa[2 * j + 1]), s01);
        tmem_ld_wait32(pb);
        tmem_ld32(taddr + col2, pa);
#pragma unroll
        for (int j = 0; j < 16; ++j) fma_f32x2(acc[16 + j], pack_f32x2(pb[2 * j], pb[2 * j + 1]), s01);
        tmem_ld_wait32(pa);
        tmem_ld32(taddr + col2 + 32, pb);
#pragma unroll
        for (int j = 0; j < 16; ++j) fma_f32x2(acc[32 + j], pack_f32x2(pa[2 * j], pa[2 * j + 1]), s23);
        tmem_ld_wait32(pb);
        // the whole partial is in registers: hand the buffer back before the last 32 columns are folded in
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&tail->part_empty[pbuf]));
#pragma unroll
        for (int j = 0; j < 16; ++j) fma_f32x2(acc[48 + j], pack_f32x2(pb[2 * j], pb[2 * j + 1]), s23);
      }
      if (!ok) break;

      if (kMode == kGateUpSwiglu) {
        // SiLU(gate)*up, rounded to bf16 as the reference does before re-quantising
        // Rows beyond the expert's last one hold whatever the tile's padding rows contained
        // (possibly NaN or Inf, which would send every division of the warp down its slow
        // path): they are zeroed first; nothing of them is stored.
        float v[64];
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float g0, g1, u0, u1;
          unpack_f32x2(row_ok ? acc[j] : 0ull, g0, g1);
          unpack_f32x2(row_ok ? acc[32 + j] : 0ull, u0, u1);
          v[2 * j] = bf16_round(silu_mul(g0, u0));
          v[2 * j + 1] = bf16_round(silu_mul(g1, u1));
          amax = fmaxf(amax, fmaxf(fabsf(v[2 * j]), fabsf(v[2 * j + 1])));
        }
        tail->amax[half][r] = amax;
        ok = epilogue_barrier(&tail->epi_bar, epi_phase, ctx, lane);
        if (!ok) break;
        amax = fmaxf(fmaxf(amax, tail->amax[half ^ 1][r]), 1e-10f);
        const float scale = fp8_group_scale(amax, args.ue8m0);
        const int out_col0 = tc.n_tile * 128 + half * 64;
        if (row_ok && out_col0 < args.out_cols) {
          uint8_t* dst = reinterpret_cast<uint8_t*>(args.out) + size_t(row) * args.out_cols + out_col0;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int j = q * 16 + i * 4;
              w[i] = pack_e4m3x4(fminf(fmaxf(__fdiv_rn(v[j], scale), -448.f), 448.f),
                                 fminf(fmaxf(__fdiv_rn(v[j + 1], scale), -448.f), 448.f),
                                 fminf(fmaxf(__fdiv_rn(v[j + 2], scale), -448.f), 448.f),
                                 fminf(fmaxf(__fdiv_rn(v[j + 3], scale), -448.f), 448.f));
            }
            if (out_col0 + q * 16 < args.out_cols)
              reinterpret_cast<uint4*>(dst)[q] = make_uint4(w[0], w[1], w[2], w[3]);
          }
          if (half == 0) args.out_scale_t[size_t(tc.n_tile) * args.row_capacity + row] = scale;
        }
      } else {
        const float w = row_w;
        const int out_col0 = tc.n_tile * 256 + half * 128;
        // A thread holds 128 columns of ONE row; stored from here a warp instruction would touch
        // 32 different rows with 16 bytes each.  Four passes of 32 columns go through a per-warp
        // block of shared memory instead, and leave as 64 contiguous bytes per row, 8 rows per
        // instruction (full sectors, a quarter of the memory transactions).
        // expert parallel: rows of this rank's own tokens go straight into its receive buffer
        void* base = (push.enabled && assignment < push.own_rows) ? push.dst.ptr[push.rank] : args.out;
        const unsigned long long my_dst =
            assignment >= 0 ? reinterpret_cast<unsigned long long>(reinterpret_cast<__nv_bfloat16*>(base) +
                                                                   size_t(assignment) * args.out_cols + out_col0)
                            : 0ull;
        uint8_t* xp = tail->xpose[ew];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) unpack_f32x2(acc[(p * 4 + q) * 4 + i], f[2 * i], f[2 * i + 1]);
            *reinterpret_cast<uint4*>(xp + lane * kXposePitch + q * 16) =
                make_uint4(pack_bf16x2(w * f[0], w * f[1]), pack_bf16x2(w * f[2], w * f[3]),
                           pack_bf16x2(w * f[4], w * f[5]), pack_bf16x2(w * f[6], w * f[7]));
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int src_row = (lane >> 2) + 8 * i, piece = lane & 3;
            const uint4 val = *reinterpret_cast<const uint4*>(xp + src_row * kXposePitch + piece * 16);
            const unsigned long long dst = __shfl_sync(0xffffffffu, my_dst, src_row);
            const int col = p * 32 + piece * 8;
            if (dst != 0ull && out_col0 + col < args.out_cols)
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dst) + col) = val;
          }
          __syncwarp();
        }
        if (push.enabled) {
          // this warp's share of the 128-row tile is stored: count it for the push warps
          __threadfence();
          __syncwarp();
          if (lane == 0) atomicAdd(push.block_done + tc.row0 / kTileM, 1);
        }
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && blockIdx.x == 0 && args.clock_probe) {
    // lets a benchmark read the SM clock the kernel really ran at (cycles / ns)
    args.clock_probe[0] = clock64() - probe_c0;
    args.clock_probe[1] = global_timer_ns() - probe_t0;
  }
  if (warp == 1) {
    tc_fence_after();
    if (tail->abort_flag) {
      for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

int launch_grouped_gemm_fp8(GemmMode mode, const CUtensorMap& map_a, const CUtensorMap& map_b,
                            const GemmFp8Args& args, const FusedDispatchFp8& dispatch, const FusedPush& push,
                            int device, cudaStream_t stream) {
  MB200_REQUIRE(args.num_experts >= 1 && args.num_experts <= kMaxExperts, kUnsupportedShape,
                "grouped_gemm_fp8: %d local experts, supported 1..%d", args.num_experts, kMaxExperts);
  MB200_REQUIRE(args.k_blocks >= 0 && args.k_blocks <= kMaxKBlocks, kUnsupportedShape,
                "grouped_gemm_fp8: %d K blocks of 128, supported 0..%d", args.k_blocks, kMaxKBlocks);
  MB200_REQUIRE(args.out_cols % 16 == 0, kUnsupportedShape,
                "grouped_gemm_fp8: output row length %d must be a multiple of 16", args.out_cols);
  MB200_REQUIRE((reinterpret_cast<uintptr_t>(args.a_scale_t) & 15) == 0 && args.row_capacity % kTileM == 0,
                kInvalidArgument, "grouped_gemm_fp8: activation scales must be 16-byte aligned with a leading "
                "dimension that is a multiple of %d", kTileM);
  MB200_REQUIRE((!dispatch.enabled || mode == kGateUpSwiglu) && (!push.enabled || mode == kDownWeighted),
                kInvalidArgument, "grouped_gemm_fp8: fused dispatch belongs to the gate/up stage, fused push to the down stage");
  const int sms = device_sm_count(device);
  MB200_REQUIRE(sms > 0, kCudaError, "grouped_gemm_fp8: cannot read the SM count of device %d", device);
  auto kernel = mode == kGateUpSwiglu ? grouped_gemm_fp8_kernel<kGateUpSwiglu>
                                      : grouped_gemm_fp8_kernel<kDownWeighted>;
  // once per device and kernel; a second thread that sets it again does no harm
  static std::atomic<bool> configured[kMaxDevices][2];
  if (device < 0 || device >= kMaxDevices || !configured[device][mode].load(std::memory_order_acquire)) {
    MB200_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          int(kSmemBytes)));
    if (device >= 0 && device < kMaxDevices) configured[device][mode].store(true, std::memory_order_release);
  }
  if (dispatch.enabled || push.enabled) {
    // the tile loader waits for rows that other CTAs' dispatch warps deliver, the push warps for
    // tiles that other CTAs compute: all CTAs must be resident (a cooperative launch guarantees it)
    void* params[] = {const_cast<CUtensorMap*>(&map_a), const_cast<CUtensorMap*>(&map_b),
                      const_cast<GemmFp8Args*>(&args), const_cast<FusedDispatchFp8*>(&dispatch),
                      const_cast<FusedPush*>(&push)};
    MB200_CHECK_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kernel), dim3(sms), dim3(kThreads),
                                                 params, kSmemBytes, stream));
  } else {
    kernel<<<sms, kThreads, kSmemBytes, stream>>>(map_a, map_b, args, dispatch, push);
    MB200_CHECK_CUDA(cudaGetLastError());
  }
  return kOk;
}

}  // namespace mb200
