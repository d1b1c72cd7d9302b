// Grouped per-expert GEMMs on e4m3 operands, tokens on the accumulator COLUMNS.
//
// Companion of grouped_gemm_fp8.cu (tokens on the accumulator rows, 128-row
// tiles) for batches with few rows per expert: there a 128-row token tile is
// mostly padding and a third of the shared-memory fill is wasted.  Here, as in
// the bf16 kernel, the weight rows sit on the tensor-memory lanes (MMA M = 128,
// two accumulators = 128 gate + 128 up rows, or 256 output rows) and the tokens
// on the MMA N dimension (16..128, expert segments padded to 16 rows), so a K
// block moves 32 KB of weights + at most 16 KB of tokens.
//
// Block scales as in reference.py:65-95: every 128-deep K block is accumulated
// into its own pair of partial accumulators and the epilogue warps promote it in
// fp32 registers.  A pair takes 2 x (token box) columns of tensor memory, so the
// 512 columns hold 2 pairs for a 128-token box and 16 pairs for a 16-token box:
// the latency of one hand-over (MMA commit -> tcgen05.ld -> buffer release) is
// spread over that many K blocks, which is what keeps the weight stream at HBM
// speed when an expert has a handful of rows,
//     acc[i, j] += partial[i, j] * (a_scale[token j, kb] * w_scale[block of i, kb]),
// in ascending K-block order.  The activation scale varies along the columns,
// so each thread multiplies its columns' scales (read through L1, prefetched one
// K block ahead) with the tile's weight scale.  gate/up: SiLU(gate)*up is
// rounded to bf16 and re-quantised per token over the tile's 128 features (one
// quantisation group): the amax runs across the 128 lanes (warp shuffles + a
// shared-memory exchange between the four lane quarters), reference.py:156-163.
//
// Roles per CTA (320 threads): warp 0 TMA producer, warp 1 tensor-memory owner
// and MMA issuer (kind::f8f6f4, K = 32 per instruction), warps 2-9 epilogue:
// warp w reads lanes 32*(w%4).. (one feature row per thread) and the 16-column
// chunks of parity (w-2)/4, at most 64 columns x 2 accumulators per thread.

#include <atomic>

#include "layer.cuh"

namespace mb200 {

namespace {

constexpr int kPad = kPadBf16;            // 16-row granule of the schedule
constexpr int kWeightBytes = 256 * 128;   // 32 KiB per K block
constexpr int kMaxStages = 8;
constexpr int kTmemCols = 512;
constexpr int kEpilogueWarps = 8;
constexpr int kFirstEpilogueWarp = 2;
constexpr int kThreads = (kFirstEpilogueWarp + kEpilogueWarps) * 32;
constexpr int kMaxTokens = 128;           // columns per accumulator (two partial pairs fit tensor memory)
constexpr int kMaxKBlocks = 128;
constexpr int kMaxPartials = 16;          // partial accumulator pairs in flight (16-token box)
constexpr int kScaleFloats = 1024;        // activation scales of the K blocks in flight (see SmemTail::ascale)

struct SmemTail {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t part_full[kMaxPartials];
  uint64_t part_empty[kMaxPartials];
  uint64_t epi_bar;
  uint32_t tmem_base;
  int abort_flag;
  int max_blocks16;
  float wscale[2][2][kMaxKBlocks];      // [tile parity][accumulator][k block]
  // Activation scales of the K blocks in flight: slots of tb_rows floats, filled by the TMA warp
  // together with the stage (a load issued by the epilogue threads themselves would wait
  // microseconds behind the weight stream).  A slot is reused after stages + partials + 1 K
  // blocks at the earliest, and kScaleFloats / tb_rows slots are always more than that.
  alignas(16) float ascale[kScaleFloats];
  float col_amax[2][4][kMaxTokens];     // [tile parity][lane quarter][token column]
  int tile_assign[2][kMaxTokens];
  float tile_weight[2][kMaxTokens];
  int prefix[kMaxExperts + 1];
  int tb_prefix[kMaxExperts + 1];
};

constexpr size_t kSmemLimit = 227 * 1024;
constexpr size_t kRingBytes = (kSmemLimit - 1024 - sizeof(SmemTail)) / 1024 * 1024;
constexpr size_t kSmemBytes = 1024 + kRingBytes + sizeof(SmemTail);

struct Geometry {
  int box_index, tb_rows, stage_bytes, stages;
  int partials;  // partial accumulator pairs that fit the 512 tensor-memory columns
  int scale_slots;
};

__device__ __forceinline__ Geometry make_geometry(int max_blocks16) {
  Geometry g;
  const int rows = max_blocks16 * kPad;
  g.box_index = rows <= 16 ? 0 : rows <= 32 ? 1 : rows <= 64 ? 2 : 3;  // larger segments are split into 128-token blocks
  g.tb_rows = 16 << g.box_index;
  g.stage_bytes = kWeightBytes + g.tb_rows * 128;
  const int s = int(kRingBytes) / g.stage_bytes;
  g.stages = s > kMaxStages ? kMaxStages : s;
  g.partials = kTmemCols / (2 * g.tb_rows);
  g.scale_slots = kScaleFloats / g.tb_rows;  // 8 / 16 / 32 / 64 slots >= stages + partials + 1 for every box
  return g;
}

struct TileCoord {
  int expert, fblock, row0, ntok, valid;
};

__device__ __forceinline__ TileCoord decode_tile(int tile, const SmemTail* t, const int* counts,
                                                 int num_experts, int n_fblocks) {
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
  const int per = (blocks16 + nb - 1) / nb;
  const int start16 = j * per;
  int len16 = blocks16 - start16;
  if (len16 > per) len16 = per;
  c.row0 = (t->prefix[lo] + start16) * kPad;
  c.ntok = len16 * kPad;
  const int left = __ldg(counts + lo) - start16 * kPad;
  c.valid = left < 0 ? 0 : (left < c.ntok ? left : c.ntok);
  return c;
}

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

__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return uint8_t(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

template <int kMode>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_fp8_cols_kernel(const __grid_constant__ CUtensorMap map_w,
                             const __grid_constant__ TokenMaps maps_t, const GemmFp8Args args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t ring_addr = raw_addr + pad;
  SmemTail* tail = reinterpret_cast<SmemTail*>(smem + kRingBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int E = args.num_experts;
  const int k_blocks = args.k_blocks;

  if (threadIdx.x == 0) {
    prefetch_tmap(&map_w);
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(smem_u32(&tail->full[s]), 1);
      mbar_init(smem_u32(&tail->empty[s]), 1);
    }
    for (int b = 0; b < kMaxPartials; ++b) {
      mbar_init(smem_u32(&tail->part_full[b]), 1);
      mbar_init(smem_u32(&tail->part_empty[b]), kEpilogueWarps);
    }
    mbar_init(smem_u32(&tail->epi_bar), kEpilogueWarps);
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
  {
    int mx = 0;
    for (int e = threadIdx.x; e < E; e += kThreads) {
      const int b = tail->prefix[e + 1] - tail->prefix[e];
      mx = b > mx ? b : mx;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const int other = __shfl_xor_sync(0xffffffffu, mx, o);
      mx = other > mx ? other : mx;
    }
    if (lane == 0 && mx > 0) atomicMax(&tail->max_blocks16, mx);
  }
  __syncthreads();
  const Geometry geo = make_geometry(tail->max_blocks16);
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
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
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
  const int total_tiles = tail->tb_prefix[E] * args.n_tiles;
  WaitCtx ctx{&tail->abort_flag, args.status, wait_limit_ns(args.status)};

  if (warp == 0) {
    // ---------------- TMA producer: one stage = one 128-deep K block ----------------
    const CUtensorMap* map_t = &maps_t.m[geo.box_index];
    if (lane == 0) prefetch_tmap(map_t);
    int stage = 0;
    uint32_t phase = 0;
    int slot = 0;  // scale slot of the K block being loaded
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      const TileCoord tc = decode_tile(tile, tail, args.counts, E, args.n_tiles);
      const int w_row = tc.expert * args.b_rows_per_expert;
      for (int kb = 0; kb < k_blocks; ++kb) {
        ok = mbar_wait(smem_u32(&tail->empty[stage]), phase ^ 1, ctx, 1);
        if (!ok) break;
        if (lane == 0) {
          const uint32_t bar = smem_u32(&tail->full[stage]);
          const uint32_t w_dst = ring_addr + stage * geo.stage_bytes;
          const uint32_t t_dst = w_dst + kWeightBytes;
          const int kcol = kb * 128;
          mbar_expect_tx(bar, uint32_t(geo.stage_bytes + tc.ntok * 4));
          tma_load_1d(smem_u32(tail->ascale + slot * geo.tb_rows),
                      args.a_scale_t + size_t(kb) * args.row_capacity + tc.row0, uint32_t(tc.ntok * 4), bar);
          if (kMode == kGateUpSwiglu) {
            tma_load_2d(w_dst, &map_w, kcol, w_row + tc.fblock * 128, bar);
            tma_load_2d(w_dst + kWeightBytes / 2, &map_w, kcol,
                        w_row + args.b_half_offset + tc.fblock * 128, bar);
          } else {
            tma_load_2d(w_dst, &map_w, kcol, w_row + tc.fblock * 256, bar);
          }
          tma_load_2d(t_dst, map_t, kcol, tc.row0, bar);
        }
        __syncwarp();
        if (++stage == geo.stages) { stage = 0; phase ^= 1; }
        if (++slot == geo.scale_slots) slot = 0;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: one K block per partial pair ----------------
    int stage = 0;
    uint32_t phase = 0;
    uint32_t pbuf = 0, puse = 0;  // partial pair and how often the ring has wrapped
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      const TileCoord tc = decode_tile(tile, tail, args.counts, E, args.n_tiles);
      const uint32_t idesc = make_idesc(0, 0, 128, uint32_t(tc.ntok));  // e4m3 x e4m3 -> fp32
      for (int kb = 0; kb < k_blocks; ++kb) {
        ok = mbar_wait(smem_u32(&tail->full[stage]), phase, ctx, 3);
        if (!ok) break;
        ok = mbar_wait(smem_u32(&tail->part_empty[pbuf]), (puse & 1) ^ 1, ctx, 2);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t w_addr = ring_addr + stage * geo.stage_bytes;
          const uint64_t w0_desc = make_kmajor_sw128_desc(w_addr);
          const uint64_t w1_desc = make_kmajor_sw128_desc(w_addr + kWeightBytes / 2);
          const uint64_t t_desc = make_kmajor_sw128_desc(w_addr + kWeightBytes);
          const uint32_t d0 = tmem_base + pbuf * 2 * geo.tb_rows;
          const uint32_t d1 = d0 + geo.tb_rows;
#pragma unroll
          for (int k = 0; k < 4; ++k) {  // 32 e4m3 = 32 bytes of K per instruction
            umma_fp8(d0, w0_desc + 2 * k, t_desc + 2 * k, idesc, k != 0);
            umma_fp8(d1, w1_desc + 2 * k, t_desc + 2 * k, idesc, k != 0);
          }
          tc_commit(smem_u32(&tail->empty[stage]));
          tc_commit(smem_u32(&tail->part_full[pbuf]));
        }
        __syncwarp();
        if (++stage == geo.stages) { stage = 0; phase ^= 1; }
        if (++pbuf == uint32_t(geo.partials)) { pbuf = 0; ++puse; }
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int ew = warp - kFirstEpilogueWarp;
    const int quarter = warp & 3;
    const int cgroup = ew >> 2;  // takes the 16-column chunks with (chunk & 1) == cgroup
    const int r = quarter * 32 + lane;
    const int etid = threadIdx.x - kFirstEpilogueWarp * 32;
    uint32_t pbuf = 0, puse = 0, it = 0, epi_phase = 0;
    int slot = 0;  // scale slot of the K block being folded in
    bool ok = true;
    // Per-tile tables: weight scales of the two accumulators (thread i fetches element i of
    // [accumulator][kb]); down GEMM: destination row and combine weight of token column i.
    // They are fetched for tile t+1 while tile t is computed, so their latency never shows.
    struct TileTables { float ws; int assign; float weight; };
    auto fetch_tables = [&](int tile) -> TileTables {
      TileTables t{0.f, -1, 0.f};
      if (tile >= total_tiles) return t;
      const TileCoord nt = decode_tile(tile, tail, args.counts, E, args.n_tiles);
      if (etid < 2 * k_blocks) {
        const int h = etid / k_blocks, kb = etid - h * k_blocks;
        const int sblock = (kMode == kGateUpSwiglu) ? (h * args.scale_half_offset + nt.fblock) : (2 * nt.fblock + h);
        if (sblock < args.scale_rows_per_expert)
          t.ws = __ldg(args.w_scale + (size_t(nt.expert) * args.scale_rows_per_expert + sblock) * k_blocks + kb);
      }
      if (kMode == kDownWeighted && etid < nt.valid) {
        t.assign = __ldg(args.sorted_ids + nt.row0 + etid);
        if (t.assign >= 0) t.weight = __ldg(args.row_scale + t.assign);
      }
      return t;
    };
    TileTables next = fetch_tables(blockIdx.x);
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
      const TileCoord tc = decode_tile(tile, tail, args.counts, E, args.n_tiles);
      const int par = it & 1;
      if (etid < 2 * k_blocks) (&tail->wscale[par][0][0])[(etid / k_blocks) * kMaxKBlocks + etid % k_blocks] = next.ws;
      if (kMode == kDownWeighted && etid < kMaxTokens) {
        tail->tile_assign[par][etid] = next.assign;
        tail->tile_weight[par][etid] = next.weight;
      }
      ok = epilogue_barrier(&tail->epi_bar, epi_phase, ctx, lane);
      if (!ok) break;
      next = fetch_tables(tile + int(gridDim.x));

      const int chunks = tc.ntok >> 4;                 // 16-column chunks in this tile (<= 8)
      const int my_chunks = (chunks - cgroup + 1) >> 1;  // chunks cgroup, cgroup+2, ... (<= 4)
      float acc0[64], acc1[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) { acc0[i] = 0.f; acc1[i] = 0.f; }

      for (int kb = 0; ok && kb < k_blocks; ++kb) {
        ok = mbar_wait(smem_u32(&tail->part_full[pbuf]), puse & 1, ctx, 4);
        if (!ok) break;
        tc_fence_after();
        const float w0 = tail->wscale[par][0][kb], w1 = tail->wscale[par][1][kb];
        // this K block's activation scales arrived in shared memory with its stage
        const float4* a_s4 = reinterpret_cast<const float4*>(tail->ascale + slot * geo.tb_rows);
        if (++slot == geo.scale_slots) slot = 0;
        const uint32_t t0 = tmem_base + pbuf * 2 * geo.tb_rows + (uint32_t(quarter * 32) << 16);
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          if (m < my_chunks) {
            const int c = cgroup + 2 * m;
            uint32_t p0[16], p1[16];
            tmem_ld16(t0 + c * 16, p0);
            tmem_ld16(t0 + geo.tb_rows + c * 16, p1);
            float as[16];
#pragma unroll
            for (int q = 0; q < 4; ++q) {  // the same 16 bytes for every lane: a broadcast read
              const float4 v = a_s4[c * 4 + q];
              as[4 * q] = v.x; as[4 * q + 1] = v.y; as[4 * q + 2] = v.z; as[4 * q + 3] = v.w;
            }
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              acc0[m * 16 + j] = fmaf(__uint_as_float(p0[j]), as[j] * w0, acc0[m * 16 + j]);
              acc1[m * 16 + j] = fmaf(__uint_as_float(p1[j]), as[j] * w1, acc1[m * 16 + j]);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&tail->part_empty[pbuf]));
        if (++pbuf == uint32_t(geo.partials)) { pbuf = 0; ++puse; }
      }
      if (!ok) break;

      if (kMode == kGateUpSwiglu) {
        // act[token, feature]: SiLU(gate)*up -> bf16 -> per-token amax over the tile's 128 features
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          if (m < my_chunks) {
            const int c = cgroup + 2 * m;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              // columns beyond the expert's last token hold whatever the padding rows contained
              // (possibly NaN or Inf, which would send the division down its slow path): zeroed
              const bool col_ok = c * 16 + j < tc.valid;
              const float g = col_ok ? acc0[m * 16 + j] : 0.f;
              const float v = bf16_round(__fdividef(g, 1.0f + __expf(-g)) * (col_ok ? acc1[m * 16 + j] : 0.f));
              acc0[m * 16 + j] = v;
              float a = fabsf(v);
#pragma unroll
              for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
              if (lane == 0) tail->col_amax[par][quarter][c * 16 + j] = a;
            }
          }
        }
        ok = epilogue_barrier(&tail->epi_bar, epi_phase, ctx, lane);
        if (!ok) break;
        const int feature = tc.fblock * 128 + r;
        uint8_t* out = reinterpret_cast<uint8_t*>(args.out);
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          if (m < my_chunks) {
            const int c = cgroup + 2 * m;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int col = c * 16 + j;
              float amax = fmaxf(fmaxf(tail->col_amax[par][0][col], tail->col_amax[par][1][col]),
                                 fmaxf(tail->col_amax[par][2][col], tail->col_amax[par][3][col]));
              amax = fmaxf(amax, 1e-10f);
              const float scale = fp8_group_scale(amax, args.ue8m0);
              if (col < tc.valid) {
                const float q = fminf(fmaxf(__fdiv_rn(acc0[m * 16 + j], scale), -448.f), 448.f);
                if (feature < args.out_cols) out[size_t(tc.row0 + col) * args.out_cols + feature] = to_e4m3(q);
                if (r == 0) args.out_scale_t[size_t(tc.fblock) * args.row_capacity + tc.row0 + col] = scale;
              }
            }
          }
        }
      } else {
        const int feature = tc.fblock * 256 + r;
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(args.out);
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          if (m < my_chunks) {
            const int c = cgroup + 2 * m;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int a = tail->tile_assign[par][c * 16 + j];
              if (a >= 0) {
                const float w = tail->tile_weight[par][c * 16 + j];
                __nv_bfloat16* dst = out + size_t(a) * args.out_cols + feature;
                if (feature < args.out_cols) dst[0] = __float2bfloat16_rn(w * acc0[m * 16 + j]);
                if (feature + 128 < args.out_cols) dst[128] = __float2bfloat16_rn(w * acc1[m * 16 + j]);
              }
            }
          }
        }
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && blockIdx.x == 0 && args.clock_probe) {
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

int launch_grouped_gemm_fp8_cols(GemmMode mode, const CUtensorMap& map_w, const TokenMaps& maps_t,
                                 const GemmFp8Args& args, int device, cudaStream_t stream) {
  MB200_REQUIRE(args.num_experts >= 1 && args.num_experts <= kMaxExperts, kUnsupportedShape,
                "grouped_gemm_fp8: %d local experts, supported 1..%d", args.num_experts, kMaxExperts);
  MB200_REQUIRE(args.k_blocks >= 0 && args.k_blocks <= kMaxKBlocks, kUnsupportedShape,
                "grouped_gemm_fp8: %d K blocks of 128, supported 0..%d", args.k_blocks, kMaxKBlocks);
  const int sms = device_sm_count(device);
  MB200_REQUIRE(sms > 0, kCudaError, "grouped_gemm_fp8: cannot read the SM count of device %d", device);
  auto kernel = mode == kGateUpSwiglu ? grouped_gemm_fp8_cols_kernel<kGateUpSwiglu>
                                      : grouped_gemm_fp8_cols_kernel<kDownWeighted>;
  // once per device and kernel; a second thread that sets it again does no harm
  static std::atomic<bool> configured[kMaxDevices][2];
  if (device < 0 || device >= kMaxDevices || !configured[device][mode].load(std::memory_order_acquire)) {
    MB200_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          int(kSmemBytes)));
    if (device >= 0 && device < kMaxDevices) configured[device][mode].store(true, std::memory_order_release);
  }
  kernel<<<sms, kThreads, kSmemBytes, stream>>>(map_w, maps_t, args);
  MB200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

}  // namespace mb200
