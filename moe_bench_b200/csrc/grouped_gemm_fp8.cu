// Grouped per-expert GEMMs on e4m3 operands with fp32 software block scales.
//
// Scales follow the reference's w8a8 block scheme (reference.py:65-95,119-167):
// one fp32 scale per 128x128 weight block and one per activation row per 128
// elements of K.  They are plain fp32 numbers (amax/448), not powers of two, so
// the hardware block-scaled MMA cannot apply them.  Instead every 128-deep K
// block is multiplied on the tensor cores into its own tensor-memory buffer
// (tcgen05.mma kind::f8f6f4, 4 x K32) and the epilogue warps promote it:
//     acc += partial * (a_scale[row, kb] * w_scale[nblock, kb])
// in fp32 registers, in ascending K-block order like the reference.  Two
// 256-column partial buffers let the promotion of block kb overlap the MMAs of
// block kb+1.
//
// Roles per CTA (320 threads): warp 0 TMA producer (4-stage ring, one stage =
// one K block: 128 rows x 128 B of A + 256 rows x 128 B of weights), warp 1
// tensor-memory owner and MMA issuer, warps 2-9 epilogue.  Epilogue warp w reads
// tensor-memory lanes 32*(w%4).. (one accumulator row per thread) and the column
// half w/4: 128 fp32 accumulators per thread.
//   gate/up:  columns = 64 gate + the matching 64 up outputs; at the end of the
//             tile SiLU(gate)*up is rounded to bf16 and re-quantised per row over
//             the tile's 128 outputs (= one quantisation group, amax exchanged
//             between the two column halves through shared memory), so the
//             second GEMM's A operand reaches HBM only as e4m3 + scales
//             (reference.py:156-163).
//   down:     columns = 128 outputs = one weight scale block; scaled by the
//             combine weight and stored as bf16 at the row's flat assignment.

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
// compiler fits without spilling (gate/up: 64 + 216, down: 80 + 208).
template <int kMode> struct RegSplit { static constexpr int kHelper = 64, kEpilogue = 216; };
template <> struct RegSplit<kDownWeighted> { static constexpr int kHelper = 80, kEpilogue = 208; };
constexpr int kMaxKBlocks = 128;  // K up to 16384

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
  int prefix[kMaxExperts + 1];
};

constexpr size_t kSmemBytes = 1024 + size_t(kStages) * kStageBytes + sizeof(SmemTail);

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
                        const __grid_constant__ CUtensorMap map_b, const GemmFp8Args args) {
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
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      TileCoord tc = decode_tile(tile, tail->prefix, args.counts, args.num_experts, args.n_tiles);
      const int b_row = tc.expert * args.b_rows_per_expert;
      for (int kb = 0; kb < k_blocks; ++kb) {
        ok = mbar_wait(smem_u32(&tail->empty[stage]), phase ^ 1, ctx, 1);
        if (!ok) break;
        if (lane == 0) {
          const uint32_t bar = smem_u32(&tail->full[stage]);
          const uint32_t a_dst = tiles_addr + stage * kStageBytes;
          const uint32_t b_dst = a_dst + kABytes;
          const int kcol = kb * 128;
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
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
      TileCoord tc = decode_tile(tile, tail->prefix, args.counts, args.num_experts, args.n_tiles);
      const int par = it & 1;
      // weight scales of this tile: [half][kb]
      for (int i = etid; i < 2 * k_blocks; i += kEpilogueWarps * 32) {
        const int h = i / k_blocks, kb = i - h * k_blocks;
        const int sblock = (kMode == kGateUpSwiglu) ? (h * args.scale_half_offset + tc.n_tile)
                                                    : (2 * tc.n_tile + h);
        float v = 0.f;
        if (sblock < args.scale_rows_per_expert)
          v = __ldg(args.w_scale + (size_t(tc.expert) * args.scale_rows_per_expert + sblock) * k_blocks + kb);
        tail->wscale[par][h][kb] = v;
      }
      ok = epilogue_barrier(&tail->epi_bar, epi_phase, ctx, lane);
      if (!ok) break;

      const int row = tc.row0 + r;
      const bool row_ok = r < tc.valid_rows;
      const float* a_scale = args.a_scale_t + row;  // [kb][row_capacity]
      // 128 fp32 accumulators per thread, kept as register pairs for fma.rn.f32x2:
      //   gate/up: pairs 0..31 = this thread's 64 gate columns, 32..63 = the matching up columns
      //   down:    pairs 0..63 = 128 consecutive output columns
      uint64_t acc[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) acc[i] = 0ull;
      float a_s_next = __ldg(a_scale);
      // tensor-memory column of this thread's four 32-column chunks
      const uint32_t col0 = kMode == kGateUpSwiglu ? uint32_t(half * 64) : uint32_t(half * 128);
      const uint32_t col2 = kMode == kGateUpSwiglu ? uint32_t(128 + half * 64) : uint32_t(half * 128 + 64);

      for (int kb = 0; kb < k_blocks; ++kb, ++pit) {
        const uint32_t pbuf = pit & 1;
        ok = mbar_wait(smem_u32(&tail->part_full[pbuf]), (pit >> 1) & 1, ctx, 4);
        if (!ok) break;
        tc_fence_after();
        const float a_s = a_s_next;
        if (kb + 1 < k_blocks) a_s_next = __ldg(a_scale + size_t(kb + 1) * args.row_capacity);
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
        float v[64];
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float g0, g1, u0, u1;
          unpack_f32x2(acc[j], g0, g1);
          unpack_f32x2(acc[32 + j], u0, u1);
          v[2 * j] = bf16_round(g0 / (1.0f + __expf(-g0)) * u0);
          v[2 * j + 1] = bf16_round(g1 / (1.0f + __expf(-g1)) * u1);
          amax = fmaxf(amax, fmaxf(fabsf(v[2 * j]), fabsf(v[2 * j + 1])));
        }
        tail->amax[half][r] = amax;
        ok = epilogue_barrier(&tail->epi_bar, epi_phase, ctx, lane);
        if (!ok) break;
        amax = fmaxf(fmaxf(amax, tail->amax[half ^ 1][r]), 1e-10f);
        const float scale = __fdiv_rn(amax, 448.0f);
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
        int assignment = -1;
        float w = 0.f;
        if (row_ok) {
          assignment = __ldg(args.sorted_ids + row);
          if (assignment >= 0) w = __ldg(args.row_scale + assignment);
        }
        const int out_col0 = tc.n_tile * 256 + half * 128;
        if (assignment >= 0) {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(args.out) + size_t(assignment) * args.out_cols + out_col0;
#pragma unroll
          for (int q = 0; q < 16; ++q) {
            if (out_col0 + q * 8 < args.out_cols) {
              float f[8];
#pragma unroll
              for (int i = 0; i < 4; ++i) unpack_f32x2(acc[q * 4 + i], f[2 * i], f[2 * i + 1]);
              reinterpret_cast<uint4*>(dst)[q] =
                  make_uint4(pack_bf16x2(w * f[0], w * f[1]), pack_bf16x2(w * f[2], w * f[3]),
                             pack_bf16x2(w * f[4], w * f[5]), pack_bf16x2(w * f[6], w * f[7]));
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
                            const GemmFp8Args& args, int device, cudaStream_t stream) {
  MB200_REQUIRE(args.num_experts >= 1 && args.num_experts <= kMaxExperts, kUnsupportedShape,
                "grouped_gemm_fp8: %d local experts, supported 1..%d", args.num_experts, kMaxExperts);
  MB200_REQUIRE(args.k_blocks >= 1 && args.k_blocks <= kMaxKBlocks, kUnsupportedShape,
                "grouped_gemm_fp8: %d K blocks of 128, supported 1..%d", args.k_blocks, kMaxKBlocks);
  MB200_REQUIRE(args.out_cols % 16 == 0, kUnsupportedShape,
                "grouped_gemm_fp8: output row length %d must be a multiple of 16", args.out_cols);
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
  kernel<<<sms, kThreads, kSmemBytes, stream>>>(map_a, map_b, args);
  MB200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

}  // namespace mb200
