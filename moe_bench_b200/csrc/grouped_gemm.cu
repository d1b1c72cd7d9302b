// Grouped per-expert 16-bit (bf16 or fp16) GEMMs of the MoE layer on the sm_100a tensor cores.
//
// Orientation: the WEIGHT rows sit on the accumulator rows (tensor-memory lanes,
// MMA M = 128) and the TOKENS on the accumulator columns (MMA N, any multiple of
// 16 up to 256).  Expert segments are therefore padded to 16 rows only, a tile
// takes as many tokens as the expert has (up to 256), and a 64-deep K step moves
// 32 KB of weights + at most 32 KB of tokens into shared memory for two
// 128 x ntok x 64 products - half the bytes per MMA cycle of a 128-token tile.
// A 128 x N x 16 tcgen05.mma takes N/2 cycles, but a K step of a tile costs about
// 1000 cycles whatever its N between 16 and 224 (the rate at which one SM takes
// 128-byte rows from L2, about 64 B per clock, paces it, not the tensor pipe), so
// the fewest, fullest tiles win: segments longer than 256 rows are split into
// equal parts.
//
//   gate/up:  acc0 = w1[e, f0:f0+128, :] . X^T, acc1 = w1[e, N+f0 : N+f0+128, :] . X^T
//             act[token, f0+i] = SiLU(acc0[i, token]) * acc1[i, token]      (bf16)
//   down:     acc0/acc1 = w2[e, h0(+128) : +128, :] . act^T
//             y[assignment(token), h0 + 128a + i] = weight(token) * acc_a[i, token]
// (reference.py:107-115,180-181; replaces the Triton fused_experts of
// baseline.py:62-76 and the ThunderKittens grouped GEMM of
// kernels/tileoverlap/common/sm120_common.cuh:149-274).
//
// One persistent CTA per SM, 512 threads: warp 0 issues TMA loads into a ring of
// 128-byte-swizzled stages (32 KiB of weights + exactly the tile's token rows, one
// TMA box per set bit of ntok/16), warp 1 owns tensor memory and issues tcgen05.mma,
// warps 2-9 drain the accumulators: tcgen05.ld of two 16-token chunks per round
// trip, accumulator released after the warp's last load, each chunk rounded,
// transposed through a 1 KiB per-warp block of shared memory and stored as 16-byte
// vectors (8 features of one token per thread).  Warps 10-13 are the fused dispatch
// of the gate/up GEMM: they copy token rows (local, or P2P loads from the source
// ranks over NVLink) into the sorted row buffer one 16-row granule at a time,
// granules strided over the CTAs in row order, and count each granule's arrival;
// the TMA warp starts a tile only when all granules of its token block have
// arrived (acquire on the counters, then a proxy fence).  Dispatch warps never
// wait, so a cooperative launch (all CTAs resident) makes the scheme deadlock-free.
// In the down GEMM, which has no dispatch, warps 10-13 drain accumulators too; expert
// parallel, its warps 14-15 push finished rows to the GPUs that own the tokens.
// The token box (16/32/64/128/256 rows), the stage size, the number of stages and
// whether the accumulators are double-buffered (token box <= 128) are derived on
// the device from the largest expert segment in the schedule, so one launch suits
// a 1-token and an 8192-token batch.  Every wait is bounded.

#include <atomic>

#include "layer.cuh"

namespace mb200 {

namespace {

constexpr int kPad = kPadBf16;                // rows an expert segment is padded to
constexpr int kWeightBytes = 256 * 128;       // 32 KiB: 2 x 128 weight rows x 128 bytes of K
constexpr int kMaxStages = 8;
constexpr int kTmemCols = 512;
constexpr int kEpilogueWarps = 8;
constexpr int kFirstEpilogueWarp = 2;
constexpr int kDispatchWarps = kDispatchWarpsPerCta;  // warps 10-13: fused dispatch (gate/up GEMM only)
constexpr int kDispatchLoads = 14;  // 16-byte loads each dispatch lane keeps in flight
constexpr int kFirstDispatchWarp = kFirstEpilogueWarp + kEpilogueWarps;
constexpr int kPushWarps = 2;       // warps 14-15: fused combine push (down GEMM, expert parallel)
constexpr int kFirstPushWarp = kFirstDispatchWarp + kDispatchWarps;
constexpr int kThreads = (kFirstPushWarp + kPushWarps) * 32;
constexpr int kMaxTokens = 256;

struct SmemTail {
  // epilogue transposition scratch: per warp one [16 tokens][32 features] 16-bit block.
  // (Every KiB here comes out of the stage ring: at 256-token tiles three 64 KiB stages
  // must fit, and a build with two stages measured 44 % slower.)
  alignas(16) uint16_t transpose[kEpilogueWarps + kDispatchWarps][16 * 32];
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t epi_bar;
  uint32_t tmem_base;
  int abort_flag;
  int max_blocks16;                 // largest expert segment, in 16-row blocks
  int tile_assign[2][kMaxTokens];   // down GEMM: flat assignment of each token column
  float tile_weight[2][kMaxTokens];
  int prefix[kMaxExperts + 1];      // cumulative 16-row blocks per expert
  int tb_prefix[kMaxExperts + 1];   // cumulative token blocks per expert
};

// dynamic shared memory: 1 KiB alignment slack + stage ring + tail
constexpr size_t kSmemLimit = 227 * 1024;
constexpr size_t kRingBytes = (kSmemLimit - 1024 - sizeof(SmemTail)) / 1024 * 1024;
constexpr size_t kSmemBytes = 1024 + kRingBytes + sizeof(SmemTail);
static_assert(kRingBytes >= 3 * (kWeightBytes + kMaxTokens * 128), "256-token tiles need three stages");

struct Geometry {
  int box_index;    // which token tensor map
  int tb_rows;      // token rows per tile (and per TMA box)
  int stage_bytes;
  int stages;
  int acc_bufs;     // 2 when both accumulators of a tile fit in 256 columns
};

__device__ __forceinline__ Geometry make_geometry(int max_blocks16) {
  Geometry g;
  int rows = max_blocks16 * kPad;
  g.box_index = rows <= 16 ? 0 : rows <= 32 ? 1 : rows <= 64 ? 2 : rows <= 128 ? 3 : 4;
  g.tb_rows = 16 << g.box_index;
  g.stage_bytes = kWeightBytes + g.tb_rows * 128;
  int s = int(kRingBytes) / g.stage_bytes;
  g.stages = s > kMaxStages ? kMaxStages : s;
  g.acc_bufs = g.tb_rows <= 128 ? 2 : 1;
  return g;
}

struct TileCoord {
  int expert;
  int fblock;   // feature block
  int row0;     // first sorted row of the token block
  int ntok;     // token columns computed (multiple of 16)
  int valid;    // real tokens among them
  int tb;       // index of the token block among all token blocks of the schedule
};

// Tiles are numbered expert-major; inside an expert the token blocks of one
// feature block are adjacent, so CTAs running side by side stream the same
// weight rows and all but the first read hit L2.
__device__ __forceinline__ TileCoord decode_tile(int tile, const SmemTail* t, const int* counts,
                                                 int num_experts, int n_fblocks, int tb_rows) {
  int lo = 0, hi = num_experts;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (t->tb_prefix[mid] * n_fblocks <= tile) lo = mid; else hi = mid - 1;
  }
  TileCoord c;
  c.expert = lo;
  const int local = tile - t->tb_prefix[lo] * n_fblocks;
  const int nb = t->tb_prefix[lo + 1] - t->tb_prefix[lo];
  c.fblock = local / nb;
  const int j = local - c.fblock * nb;
  const int blocks16 = t->prefix[lo + 1] - t->prefix[lo];
  const int per = (blocks16 + nb - 1) / nb;  // balanced split of the segment
  const int start16 = j * per;
  int len16 = blocks16 - start16;
  if (len16 > per) len16 = per;
  c.row0 = (t->prefix[lo] + start16) * kPad;
  c.tb = t->tb_prefix[lo] + j;
  c.ntok = len16 * kPad;
  int left = __ldg(counts + lo) - start16 * kPad;
  c.valid = left < 0 ? 0 : (left < c.ntok ? left : c.ntok);
  (void)tb_rows;
  return c;
}

__device__ __forceinline__ bool epilogue_barrier(uint64_t* bar, uint32_t& phase, WaitCtx& ctx, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(smem_u32(bar));
  const bool ok = mbar_wait(smem_u32(bar), phase, ctx, 5);
  phase ^= 1;
  return ok;
}

__device__ __forceinline__ float silu_mul(float g, float u) {
  // fast reciprocal: ~2 ulp, far inside the 16-bit rounding of the result
  return __fdividef(g, 1.0f + __expf(-g)) * u;
}

// kPush (down GEMM, expert parallel): warps 14-15 forward finished rows to the GPUs that own
// the tokens (they idle otherwise).
template <int kMode, bool kPush>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_w,
                         const __grid_constant__ TokenMaps maps_t, const GemmArgs args,
                         const FusedDispatch disp, const FusedPush push) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t ring_addr = raw_addr + pad;
  SmemTail* tail = reinterpret_cast<SmemTail*>(smem + kRingBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int E = args.num_experts;
  // the down GEMM has no dispatch: its warps 10-13 drain accumulators too
  constexpr int kEpiWarps = kMode == kDownWeighted ? kEpilogueWarps + kDispatchWarps : kEpilogueWarps;
  constexpr int kChunkStride = kEpiWarps / 4;  // warps per tensor-memory lane quarter
  const int worker = int(blockIdx.x);
  const int workers = int(gridDim.x);

  if (threadIdx.x == 0) {
    prefetch_tmap(&map_w);
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(smem_u32(&tail->full[s]), 1);
      mbar_init(smem_u32(&tail->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&tail->acc_full[b]), 1);
      mbar_init(smem_u32(&tail->acc_empty[b]), kEpiWarps);
    }
    mbar_init(smem_u32(&tail->epi_bar), kEpiWarps);
    tail->abort_flag = 0;
    tail->max_blocks16 = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tail->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  for (int i = threadIdx.x; i <= E; i += kThreads) tail->prefix[i] = args.mtile_prefix[i];
  __syncthreads();
  // largest expert segment -> token box, stage geometry
  {
    int mx = 0;
    for (int e = threadIdx.x; e < E; e += kThreads) {
      int b = tail->prefix[e + 1] - tail->prefix[e];
      mx = b > mx ? b : mx;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      int other = __shfl_xor_sync(0xffffffffu, mx, o);
      mx = other > mx ? other : mx;
    }
    if (lane == 0 && mx > 0) atomicMax(&tail->max_blocks16, mx);
  }
  __syncthreads();
  const Geometry geo = make_geometry(tail->max_blocks16);
  // token blocks per expert, exclusive scan by warp 0 (each lane owns a run of experts)
  if (warp == 0) {
    const int blocks_per_tile = geo.tb_rows / kPad;
    const int per = (E + 31) / 32;
    const int lo = lane * per;
    const int hi = lo + per < E ? lo + per : E;
    int sum = 0;
    for (int e = lo; e < hi; ++e)
      sum += (tail->prefix[e + 1] - tail->prefix[e] + blocks_per_tile - 1) / blocks_per_tile;
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    int run = incl - sum;
    for (int e = lo; e < hi; ++e) {
      tail->tb_prefix[e] = run;
      run += (tail->prefix[e + 1] - tail->prefix[e] + blocks_per_tile - 1) / blocks_per_tile;
    }
    if (lane == 31) tail->tb_prefix[E] = incl;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const unsigned long long probe_c0 = clock64(), probe_t0 = global_timer_ns();
  const uint32_t tmem_base = tail->tmem_base;
  const int n_fgroups = args.n_tiles;
  const int total_tiles = tail->tb_prefix[E] * n_fgroups;
  const uint32_t acc1_off = geo.acc_bufs == 2 ? 128u : 256u;  // column of the second accumulator
  WaitCtx ctx{&tail->abort_flag, args.status, wait_limit_ns(args.status)};

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane < kTokenBoxes) prefetch_tmap(&maps_t.m[lane]);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = worker; ok && tile < total_tiles; tile += workers) {
      const TileCoord tc = decode_tile(tile, tail, args.counts, E, n_fgroups, geo.tb_rows);
      const int fblock = tc.fblock;
      const int w_row = tc.expert * args.b_rows_per_expert;
      if (kMode == kGateUpSwiglu && disp.enabled) {
        // all 16-row granules of this token block must have been dispatched
        const int g0 = tc.row0 / kPad, ng = tc.ntok / kPad;  // ng <= 16
        uint32_t spins = 0;
        WaitClock clock;
        while (true) {
          int v = disp.granule_target;
          if (lane < ng)
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(disp.granule_done + g0 + lane) : "memory");
          if (__all_sync(0xffffffffu, v >= disp.granule_target)) break;
          if ((++spins & 0x3F) == 0) {
            // warp-uniform decisions: the lanes read the flag and the timer at slightly different moments
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
        // rows were written with ordinary stores by other SMs; the TMA engine reads them
        asm volatile("fence.proxy.async;" ::: "memory");
      }
      for (int kb = 0; kb < args.k_iters; ++kb) {
        ok = mbar_wait(smem_u32(&tail->empty[stage]), phase ^ 1, ctx, 1);
        if (!ok) break;
        if (lane == 0) {
          const uint32_t bar = smem_u32(&tail->full[stage]);
          const uint32_t w_dst = ring_addr + stage * geo.stage_bytes;
          const uint32_t t_dst = w_dst + kWeightBytes;
          const int kcol = kb * 64;
          mbar_expect_tx(bar, uint32_t(kWeightBytes + tc.ntok * 128));
          if (kMode == kGateUpSwiglu) {
            tma_load_2d(w_dst, &map_w, kcol, w_row + fblock * 128, bar);
            tma_load_2d(w_dst + kWeightBytes / 2, &map_w, kcol,
                        w_row + args.b_half_offset + fblock * 128, bar);
          } else {
            tma_load_2d(w_dst, &map_w, kcol, w_row + fblock * 256, bar);
          }
          // exactly ntok token rows: one box per set bit of ntok/16 (largest first), so a
          // 144-token tile moves 18 KB of tokens, not the 32 KB of the launch's largest box
          const int nb16 = tc.ntok >> 4;
          int r = 0;
#pragma unroll
          for (int b = kTokenBoxes - 1; b >= 0; --b) {
            if (nb16 & (1 << b)) {
              tma_load_2d(t_dst + uint32_t(r) * 128u, &maps_t.m[b], kcol, tc.row0 + r, bar);
              r += 16 << b;
            }
          }
        }
        __syncwarp();
        if (++stage == geo.stages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    int stage = 0;
    uint32_t phase = 0;
    uint32_t it = 0;
    bool ok = true;
    for (int tile = worker; ok && tile < total_tiles; tile += workers, ++it) {
      const TileCoord tc = decode_tile(tile, tail, args.counts, E, n_fgroups, geo.tb_rows);
      const uint32_t buf = geo.acc_bufs == 2 ? (it & 1) : 0;
      const uint32_t use = geo.acc_bufs == 2 ? (it >> 1) : it;
      ok = mbar_wait(smem_u32(&tail->acc_empty[buf]), (use & 1) ^ 1, ctx, 2);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d0 = tmem_base + buf * 256;
      const uint32_t d1 = d0 + acc1_off;
      const uint32_t fmt = args.fp16 ? 0u : 1u;  // kind::f16 operand format: 0 = f16, 1 = bf16
      const uint32_t idesc = make_idesc(fmt, fmt, 128, uint32_t(tc.ntok));
      for (int kb = 0; kb < args.k_iters; ++kb) {
        ok = mbar_wait(smem_u32(&tail->full[stage]), phase, ctx, 3);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t w_addr = ring_addr + stage * geo.stage_bytes;
          const uint64_t w0_desc = make_kmajor_sw128_desc(w_addr);
          const uint64_t w1_desc = make_kmajor_sw128_desc(w_addr + kWeightBytes / 2);
          const uint64_t t_desc = make_kmajor_sw128_desc(w_addr + kWeightBytes);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // 16 bf16 = 32 bytes of K per instruction: +2 in the 16-byte address field
            const uint32_t accumulate = (kb | k) != 0;
            umma_bf16(d0, w0_desc + 2 * k, t_desc + 2 * k, idesc, accumulate);
            umma_bf16(d1, w1_desc + 2 * k, t_desc + 2 * k, idesc, accumulate);
          }
          // the stage is free once these MMAs have read it
          tc_commit(smem_u32(&tail->empty[stage]));
        }
        __syncwarp();
        if (++stage == geo.stages) { stage = 0; phase ^= 1; }
      }
      if (ok && lane == 0) tc_commit(smem_u32(&tail->acc_full[buf]));
      __syncwarp();
    }
  } else if (warp >= kFirstPushWarp && !(kMode == kDownWeighted && kPush)) {
    // warps 14-15 have no work in this kernel variant
  } else if (kMode == kGateUpSwiglu && warp >= kFirstDispatchWarp) {
    // ---------------- fused dispatch (gate/up GEMM): fill the sorted row buffer ----------------
    if (kMode == kGateUpSwiglu && disp.enabled == kDispatchFused) {
      const int dw = warp - kFirstDispatchWarp;
      const int granules = tail->prefix[E];
      for (int g = blockIdx.x; g < granules; g += gridDim.x) {
        // each of the 4 dispatch warps takes 4 of the granule's 16 rows
        for (int i = dw; i < kPad; i += kDispatchWarps) {
          const int row = g * kPad + i;
          const int n = __ldg(args.sorted_ids + row);
          if (n >= 0) {
            const int tok_global = n / disp.topk;
            const int ring = tok_global / disp.tokens_per_rank;
            const int t = tok_global - ring * disp.tokens_per_rank;
            const uint4* src = reinterpret_cast<const uint4*>(disp.src.ptr[(disp.rank + ring) % disp.world]) +
                               size_t(t) * disp.vec_per_row;
            uint4* dst = disp.rows_out + size_t(row) * disp.vec_per_row;
            // kDispatchLoads 16-byte loads in flight per lane: a load over NVLink takes microseconds and
            // only 4 warps per SM do this work
            for (int v0 = lane; v0 < disp.vec_per_row; v0 += 32 * kDispatchLoads) {
              uint4 buf[kDispatchLoads];
#pragma unroll
              for (int u = 0; u < kDispatchLoads; ++u)
                if (v0 + u * 32 < disp.vec_per_row) buf[u] = src[v0 + u * 32];
#pragma unroll
              for (int u = 0; u < kDispatchLoads; ++u)
                if (v0 + u * 32 < disp.vec_per_row) dst[v0 + u * 32] = buf[u];
            }
          }
        }
        __threadfence();  // this warp's rows before its arrival count
        __syncwarp();
        if (lane == 0) atomicAdd(disp.granule_done + g, 1);
      }
    }
  } else if (kMode == kDownWeighted && kPush && warp >= kFirstPushWarp) {
    // ---------------- fused combine push (down GEMM, expert parallel) ----------------
    // Work unit = one 16-row granule of the sorted rows, granules strided over the CTAs in row
    // order (= the order in which the tiles finish).  A granule is forwarded once every feature
    // block of its token block has been stored by the epilogue warps of whichever CTAs computed
    // them.  The GEMM warps never wait for these warps, so with all CTAs resident (cooperative
    // launch) the wait cannot deadlock; it is bounded like every other wait.
    const int pw = warp - kFirstPushWarp;
    const int granules = tail->prefix[E];
    const int target = args.n_tiles * kEpiWarps;
    bool ok = true;
    for (int g = blockIdx.x; ok && g < granules; g += gridDim.x) {
      int lo = 0, hi = E - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (tail->prefix[mid] <= g) lo = mid; else hi = mid - 1;
      }
      const int blocks16 = tail->prefix[lo + 1] - tail->prefix[lo];
      const int nb = tail->tb_prefix[lo + 1] - tail->tb_prefix[lo];
      const int per = (blocks16 + nb - 1) / nb;
      const int tb = tail->tb_prefix[lo] + (g - tail->prefix[lo]) / per;
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
      for (int i = pw; i < kPad; i += kPushWarps) {
        const int n = __ldg(args.sorted_ids + g * kPad + i);
        if (n >= push.own_rows) {  // a token of another rank (own tokens were stored in place; -1 = padding)
          const int tok_global = n / push.topk;
          const int ring = tok_global / push.tokens_per_rank;
          const int slot = n - ring * push.own_rows;
          const uint4* src = push.rows_in + size_t(n) * push.vec_per_row;
          uint4* dst = reinterpret_cast<uint4*>(push.dst.ptr[(push.rank + ring) % push.world]) +
                       size_t(slot) * push.vec_per_row;
          for (int v0 = lane; v0 < push.vec_per_row; v0 += 32 * kDispatchLoads) {
            uint4 buf[kDispatchLoads];
#pragma unroll
            for (int u = 0; u < kDispatchLoads; ++u)
              if (v0 + u * 32 < push.vec_per_row) buf[u] = __ldcg(src + v0 + u * 32);
#pragma unroll
            for (int u = 0; u < kDispatchLoads; ++u)
              if (v0 + u * 32 < push.vec_per_row) dst[v0 + u * 32] = buf[u];
          }
        }
      }
    }
    // this warp's stores to the peers are performed before the kernel ends (the cross-GPU
    // barrier that follows on the stream then covers them)
    __threadfence_system();
  } else {
    // ---------------- epilogue: 8 (gate/up) or 12 (down) warps, one accumulator row (feature) per thread ----------------
    const int ew = warp - kFirstEpilogueWarp;
    const int quarter = warp & 3;     // tensor-memory lanes 32*quarter .. +31
    const int cgroup = ew >> 2;       // which 16-column chunks this warp takes (c mod kChunkStride)
    const int etid = threadIdx.x - kFirstEpilogueWarp * 32;
    uint32_t it = 0;
    uint32_t epi_phase = 0;
    bool ok = true;
    for (int tile = worker; ok && tile < total_tiles; tile += workers, ++it) {
      const TileCoord tc = decode_tile(tile, tail, args.counts, E, n_fgroups, geo.tb_rows);
      const int fblock = tc.fblock;
      const uint32_t buf = geo.acc_bufs == 2 ? (it & 1) : 0;
      const uint32_t use = geo.acc_bufs == 2 ? (it >> 1) : it;
      const int par = it & 1;
      if (kMode == kDownWeighted) {
        // per-token destination row and combine weight, shared by all feature rows
        for (int j = etid; j < tc.ntok; j += kEpiWarps * 32) {
          int a = -1;
          float w = 0.f;
          if (j < tc.valid) {
            a = __ldg(args.sorted_ids + tc.row0 + j);
            if (a >= 0) w = __ldg(args.row_scale + a);
          }
          tail->tile_assign[par][j] = a;
          tail->tile_weight[par][j] = w;
        }
        ok = epilogue_barrier(&tail->epi_bar, epi_phase, ctx, lane);
        if (!ok) break;
      }
      ok = mbar_wait(smem_u32(&tail->acc_full[buf]), use & 1, ctx, 4);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t0 = tmem_base + buf * 256 + (uint32_t(quarter * 32) << 16);
      const uint32_t t1 = t0 + acc1_off;
      uint16_t* out = reinterpret_cast<uint16_t*>(args.out);
      uint16_t* out_own = kPush ? reinterpret_cast<uint16_t*>(push.dst.ptr[push.rank]) : out;
      const int chunks = tc.ntok >> 4;

      // A thread holds one feature (accumulator row) of 16 tokens; memory wants the
      // features of a token side by side.  Each 16-token chunk is rounded, transposed
      // through a 1 KiB per-warp block of shared memory and leaves as 16-byte stores
      // (8 features of one token per thread), two per thread and output block.
      uint16_t* sc0 = tail->transpose[ew];
      bool released = false;
      auto release = [&]() {
        // every value of this warp's share is in registers: the accumulator may be overwritten
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&tail->acc_empty[buf]));
        released = true;
      };
      if (kMode == kGateUpSwiglu) {
        const int feat_base = fblock * 128 + quarter * 32;
        auto emit = [&](int c, const uint32_t (&g)[16], const uint32_t (&u)[16]) {
          if (c * 16 >= tc.valid) return;  // padding rows only
#pragma unroll
          for (int j = 0; j < 16; ++j)
            sc0[j * 32 + lane] = to_h16(silu_mul(__uint_as_float(g[j]), __uint_as_float(u[j])), args.fp16);
          __syncwarp();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int piece = lane + 32 * h;  // token piece>>2 of the chunk, features 8*(piece&3) .. +7
            const int token = c * 16 + (piece >> 2);
            const int feat = feat_base + (piece & 3) * 8;
            if (token < tc.valid && feat < args.out_cols)
              *reinterpret_cast<uint4*>(out + size_t(tc.row0 + token) * args.out_cols + feat) =
                  *reinterpret_cast<const uint4*>(sc0 + piece * 8);
          }
          __syncwarp();
        };
        // two chunks per tensor-memory round trip
        for (int c = cgroup; c < chunks; c += 2 * kChunkStride) {
          uint32_t ga[16], ua[16], gb[16], ub[16];
          const int c2 = c + kChunkStride;
          const bool two = c2 < chunks;
          tmem_ld16(t0 + c * 16, ga);
          tmem_ld16(t1 + c * 16, ua);
          if (two) {
            tmem_ld16(t0 + c2 * 16, gb);
            tmem_ld16(t1 + c2 * 16, ub);
          }
          tmem_ld_wait();
          if (c + 2 * kChunkStride >= chunks) release();
          emit(c, ga, ua);
          if (two) emit(c2, gb, ub);
        }
      } else {
        const int feat_base = fblock * 256 + quarter * 32;
        auto emit = [&](int c, const uint32_t (&v0)[16], const uint32_t (&v1)[16]) {
          if (c * 16 >= tc.valid) return;
          // the two 128-row halves of the tile go through the block one after the other
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const uint32_t (&v)[16] = half == 0 ? v0 : v1;
#pragma unroll
            for (int j = 0; j < 16; ++j)
              sc0[j * 32 + lane] = to_h16(tail->tile_weight[par][c * 16 + j] * __uint_as_float(v[j]), args.fp16);
            __syncwarp();
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int piece = lane + 32 * h;
              const int a = tail->tile_assign[par][c * 16 + (piece >> 2)];
              const int feat = feat_base + half * 128 + (piece & 3) * 8;
              if (a >= 0 && feat < args.out_cols) {
                // expert parallel: rows of this rank's own tokens go straight into its receive buffer
                uint16_t* base = (kPush && a < push.own_rows) ? out_own : out;
                *reinterpret_cast<uint4*>(base + size_t(a) * args.out_cols + feat) =
                    *reinterpret_cast<const uint4*>(sc0 + piece * 8);
              }
            }
            __syncwarp();
          }
        };
        for (int c = cgroup; c < chunks; c += 2 * kChunkStride) {
          uint32_t a0[16], a1[16], b0[16], b1[16];
          const int c2 = c + kChunkStride;
          const bool two = c2 < chunks;
          tmem_ld16(t0 + c * 16, a0);
          tmem_ld16(t1 + c * 16, a1);
          if (two) {
            tmem_ld16(t0 + c2 * 16, b0);
            tmem_ld16(t1 + c2 * 16, b1);
          }
          tmem_ld_wait();
          if (c + 2 * kChunkStride >= chunks) release();
          emit(c, a0, a1);
          if (two) emit(c2, b0, b1);
        }
      }
      if (!released) release();
      if (kPush) {
        // this warp's share of the token block is stored: count it for the push warps
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(push.block_done + tc.tb, 1);
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
      // A wait was abandoned: give loads still in flight time to land before
      // the shared memory is handed to the next CTA.
      for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

using KernelFn = void (*)(const CUtensorMap, const TokenMaps, const GemmArgs, const FusedDispatch, const FusedPush);

}  // namespace

int launch_grouped_gemm_bf16(GemmMode mode, const CUtensorMap& map_w, const TokenMaps& maps_t,
                             const GemmArgs& args, const FusedDispatch& dispatch, const FusedPush& push,
                             int device, cudaStream_t stream) {
  MB200_REQUIRE(args.num_experts >= 1 && args.num_experts <= kMaxExperts, kUnsupportedShape,
                "grouped_gemm: %d local experts, supported 1..%d", args.num_experts, kMaxExperts);
  MB200_REQUIRE(!dispatch.enabled || mode == kGateUpSwiglu, kInvalidArgument,
                "grouped_gemm: fused dispatch belongs to the gate/up stage");
  MB200_REQUIRE((reinterpret_cast<uintptr_t>(args.out) & 15) == 0 && args.out_cols % 8 == 0, kInvalidArgument,
                "grouped_gemm: output must be 16-byte aligned with a row length that is a multiple of 8");
  MB200_REQUIRE(!push.enabled || mode == kDownWeighted, kInvalidArgument,
                "grouped_gemm: the fused combine push belongs to the down stage");
  const int variant = mode == kGateUpSwiglu ? 0 : (push.enabled ? 2 : 1);
  KernelFn kernel = variant == 0   ? grouped_gemm_bf16_kernel<kGateUpSwiglu, false>
                    : variant == 1 ? grouped_gemm_bf16_kernel<kDownWeighted, false>
                                   : grouped_gemm_bf16_kernel<kDownWeighted, true>;
  // once per device and kernel; a second thread that sets it again does no harm
  static std::atomic<bool> configured[kMaxDevices][3];
  if (device < 0 || device >= kMaxDevices || !configured[device][variant].load(std::memory_order_acquire)) {
    MB200_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemBytes)));
    if (device >= 0 && device < kMaxDevices) configured[device][variant].store(true, std::memory_order_release);
  }
  const int sms = device_sm_count(device);
  MB200_REQUIRE(sms > 0, kCudaError, "grouped_gemm: cannot read the SM count of device %d", device);
  if (dispatch.enabled == kDispatchFused || push.enabled) {
    // the tile loader waits for rows that other CTAs' dispatch warps deliver, the push warps
    // for tiles that other CTAs compute: all CTAs must be resident, which a cooperative
    // launch guarantees (or refuses)
    void* params[] = {const_cast<CUtensorMap*>(&map_w), const_cast<TokenMaps*>(&maps_t),
                      const_cast<GemmArgs*>(&args), const_cast<FusedDispatch*>(&dispatch),
                      const_cast<FusedPush*>(&push)};
    MB200_CHECK_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kernel), dim3(sms), dim3(kThreads),
                                                 params, kSmemBytes, stream));
  } else {
    kernel<<<sms, kThreads, kSmemBytes, stream>>>(map_w, maps_t, args, dispatch, push);
    MB200_CHECK_CUDA(cudaGetLastError());
  }
  return kOk;
}

}  // namespace mb200
