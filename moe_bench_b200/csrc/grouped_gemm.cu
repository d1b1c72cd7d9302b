// Grouped per-expert GEMMs of the MoE layer on the sm_100a tensor cores.
//
// One persistent, warp-specialised kernel, two epilogues:
//   gate/up:  act[row, n]  = SiLU(A[row,:] . w1[e, n, :]) * (A[row,:] . w1[e, N+n, :])
//   down:     y[assignment, h] = weight[assignment] * (act[row,:] . w2[e, h, :])
// Rows are the sorted, 128-padded assignment rows of the schedule; a tile is 128
// rows x 256 accumulator columns (gate/up: 128 gate + the matching 128 up
// columns, so SiLU(gate)*up is formed in registers and only [rows, N] is
// written).
//
// Roles per CTA (192 threads): warp 0 issues TMA loads into a 4-stage ring of
// 128-byte-swizzled tiles, warp 1 owns tensor memory and issues tcgen05.mma
// (128x256x16 per instruction, fp32 accumulators in tensor memory, two
// accumulator buffers of 256 columns), warps 2-5 drain accumulators with
// tcgen05.ld and write the output.  Every wait is bounded.
//
// What it replaces in the reference: the per-expert masked matmuls of
// reference.py:107-115 and the ThunderKittens grouped GEMM
// kernels/tileoverlap/common/sm120_common.cuh:149-274.

#include "layer.cuh"

namespace mb200 {

namespace {

constexpr int kStages = 4;
constexpr int kABytes = kTileM * 128;     // 16 KiB: 128 rows x 128 bytes of K
constexpr int kBBytes = 256 * 128;        // 32 KiB: 256 weight rows x 128 bytes of K
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kAccCols = 256;
constexpr int kTmemCols = 512;
constexpr int kThreads = 192;
constexpr int kEpilogueThreads = 128;

struct SmemTail {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int prefix[kMaxExperts + 1];
};

constexpr size_t kSmemBytes = 1024 + size_t(kStages) * kStageBytes + sizeof(SmemTail);

struct TileCoord {
  int expert;
  int n_tile;
  int row0;        // first padded row of the tile
  int valid_rows;  // real rows in the tile
};

// Tiles are numbered expert-major; inside an expert the M tiles of one weight
// tile are adjacent, so CTAs running side by side stream the same weights and
// the second read hits L2.
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

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float silu_mul(float g, float u) {
  return g / (1.0f + __expf(-g)) * u;
}

template <int kMode>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a,
                         const __grid_constant__ CUtensorMap map_b, const GemmArgs args) {
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
      mbar_init(smem_u32(&tail->acc_full[b]), 1);
      mbar_init(smem_u32(&tail->acc_empty[b]), kEpilogueThreads);
    }
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

  const uint32_t tmem_base = tail->tmem_base;
  const int total_tiles = tail->prefix[args.num_experts] * args.n_tiles;
  WaitCtx ctx{&tail->abort_flag, args.status, global_timer_ns()};

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      TileCoord tc = decode_tile(tile, tail->prefix, args.counts, args.num_experts, args.n_tiles);
      const int b_row = tc.expert * args.b_rows_per_expert;
      for (int kb = 0; kb < args.k_iters; ++kb) {
        ok = mbar_wait(smem_u32(&tail->empty[stage]), phase ^ 1, ctx, 1);
        if (!ok) break;
        if (lane == 0) {
          const uint32_t bar = smem_u32(&tail->full[stage]);
          const uint32_t a_dst = tiles_addr + stage * kStageBytes;
          const uint32_t b_dst = a_dst + kABytes;
          const int kcol = kb * 64;
          mbar_expect_tx(bar, kStageBytes);
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
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    constexpr uint32_t idesc = make_idesc(1, 1, kTileM, kAccCols);
    int stage = 0;
    uint32_t phase = 0;
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
      const uint32_t buf = it & 1;
      ok = mbar_wait(smem_u32(&tail->acc_empty[buf]), ((it >> 1) & 1) ^ 1, ctx, 2);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + buf * kAccCols;
      for (int kb = 0; kb < args.k_iters; ++kb) {
        ok = mbar_wait(smem_u32(&tail->full[stage]), phase, ctx, 3);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_addr = tiles_addr + stage * kStageBytes;
          const uint64_t a_desc = make_kmajor_sw128_desc(a_addr);
          const uint64_t b_desc = make_kmajor_sw128_desc(a_addr + kABytes);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // 16 bf16 = 32 bytes of K per instruction: +2 in the 16-byte address field
            umma_bf16(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
          }
          tc_commit(smem_u32(&tail->empty[stage]));
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
      if (ok && lane == 0) tc_commit(smem_u32(&tail->acc_full[buf]));
      __syncwarp();
    }
  } else {
    // ---------------- epilogue (4 warps, one accumulator row per thread) ----------------
    const int quarter = warp & 3;  // tensor-memory lanes this warp may read: 32*quarter ..
    const int r = quarter * 32 + lane;
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
      TileCoord tc = decode_tile(tile, tail->prefix, args.counts, args.num_experts, args.n_tiles);
      const uint32_t buf = it & 1;
      if (!mbar_wait(smem_u32(&tail->acc_full[buf]), (it >> 1) & 1, ctx, 4)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + buf * kAccCols + (uint32_t(quarter * 32) << 16);
      const bool row_ok = r < tc.valid_rows;

      if (kMode == kGateUpSwiglu) {
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(args.out);
        const int col0 = tc.n_tile * 128;
        __nv_bfloat16* dst = out + size_t(tc.row0 + r) * args.out_cols + col0;
#pragma unroll 2
        for (int c = 0; c < 8; ++c) {
          uint32_t g[16], u[16];
          tmem_ld16(taddr + c * 16, g);
          tmem_ld16(taddr + 128 + c * 16, u);
          tmem_ld_wait();
          if (row_ok && col0 + c * 16 < args.out_cols) {
            uint32_t p[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              p[j] = pack_bf16x2(silu_mul(__uint_as_float(g[2 * j]), __uint_as_float(u[2 * j])),
                                 silu_mul(__uint_as_float(g[2 * j + 1]), __uint_as_float(u[2 * j + 1])));
            }
            uint4* d4 = reinterpret_cast<uint4*>(dst + c * 16);
            d4[0] = make_uint4(p[0], p[1], p[2], p[3]);
            d4[1] = make_uint4(p[4], p[5], p[6], p[7]);
          }
        }
      } else {
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(args.out);
        int assignment = -1;
        float w = 0.f;
        if (row_ok) {
          assignment = __ldg(args.sorted_ids + tc.row0 + r);
          if (assignment >= 0) w = __ldg(args.row_scale + assignment);
        }
        const int col0 = tc.n_tile * 256;
        __nv_bfloat16* dst = out + size_t(assignment < 0 ? 0 : assignment) * args.out_cols + col0;
#pragma unroll 2
        for (int c = 0; c < 16; ++c) {
          uint32_t v[16];
          tmem_ld16(taddr + c * 16, v);
          tmem_ld_wait();
          if (assignment >= 0 && col0 + c * 16 < args.out_cols) {
            uint32_t p[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              p[j] = pack_bf16x2(w * __uint_as_float(v[2 * j]), w * __uint_as_float(v[2 * j + 1]));
            }
            uint4* d4 = reinterpret_cast<uint4*>(dst + c * 16);
            d4[0] = make_uint4(p[0], p[1], p[2], p[3]);
            d4[1] = make_uint4(p[4], p[5], p[6], p[7]);
          }
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&tail->acc_empty[buf]));
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
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

}  // namespace

int launch_grouped_gemm_bf16(GemmMode mode, const CUtensorMap& map_a, const CUtensorMap& map_b,
                             const GemmArgs& args, int device, cudaStream_t stream) {
  MB200_REQUIRE(args.num_experts >= 1 && args.num_experts <= kMaxExperts, kUnsupportedShape,
                "grouped_gemm: %d local experts, supported 1..%d", args.num_experts, kMaxExperts);
  MB200_REQUIRE(args.out_cols % 16 == 0, kUnsupportedShape,
                "grouped_gemm: output row length %d must be a multiple of 16", args.out_cols);
  static bool configured[64][2] = {};
  int sms = 0;
  MB200_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  auto kernel = mode == kGateUpSwiglu ? grouped_gemm_bf16_kernel<kGateUpSwiglu>
                                      : grouped_gemm_bf16_kernel<kDownWeighted>;
  if (device >= 0 && device < 64 && !configured[device][mode]) {
    MB200_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          int(kSmemBytes)));
    configured[device][mode] = true;
  }
  kernel<<<sms, kThreads, kSmemBytes, stream>>>(map_a, map_b, args);
  MB200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

}  // namespace mb200
