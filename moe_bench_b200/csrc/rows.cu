// Row-wise, bandwidth-bound stages around the grouped GEMMs:
//   combine:       (inverse == nullptr: every assignment is present)
//                  out[t, :] = sum over the k local assignments of token t of
//                  the already weighted rows y[t*k + j, :], fp32 sum, bf16 store
//                  (reference.py:180-182).
//   combine_push:  tensor parallel: the same sum, stored straight into the plane of
//                  the token's owner that belongs to this rank (16-byte P2P stores);
//   sum_planes:    the owner's sum over its W planes (the output reduce of
//                  schemes.py:72-75,142).
//   group_quant:   per row, per 128-wide group dynamic e4m3 quantisation of
//                  activations (reference.py:143-145,157-163).
// All of them move 16 bytes per thread per access and size their grids as a
// multiple of the SM count.

#include "layer.cuh"

namespace mb200 {

namespace {

__global__ void combine_bf16_kernel(const uint4* __restrict__ y, const int* __restrict__ inverse,
                                    int tokens, int topk, int vec_per_row, uint4* __restrict__ out, int fp16) {
  const int64_t total = int64_t(tokens) * vec_per_row;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * blockDim.x) {
    const int64_t t = i / vec_per_row;
    const int v = int(i - t * vec_per_row);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    // up to 8 row loads in flight per thread, summed in ascending j
    for (int j0 = 0; j0 < topk; j0 += 8) {
      uint4 val[8];
      bool have[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int64_t n = t * topk + j0 + u;
        // an expert on another rank contributes zero
        have[u] = j0 + u < topk && (inverse == nullptr || __ldg(inverse + n) >= 0);
        if (have[u]) val[u] = __ldg(y + n * vec_per_row + v);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (have[u]) add_h16x8(val[u], acc, fp16);
    }
    out[i] = pack_h16x8(acc, fp16);
  }
}

// Tensor parallel: the same sum over a token's k rows, but the result goes straight to the rank
// that owns the token, into the plane of its `partial` buffer that belongs to this rank
// (row i of y's token space is token t = i mod T of rank (rank + i / T) mod W), as 16-byte
// stores over NVLink.  Replaces "sum locally, barrier, owner pulls": the owner then sums W
// local planes.
__global__ void combine_push_kernel(const uint4* __restrict__ y, int all_tokens, int tokens_per_rank, int topk,
                                    int vec_per_row, PeerTable partial, int rank, int world, int fp16) {
  const int64_t total = int64_t(all_tokens) * vec_per_row;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * blockDim.x) {
    const int64_t row = i / vec_per_row;
    const int v = int(i - row * vec_per_row);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j0 = 0; j0 < topk; j0 += 8) {
      uint4 val[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (j0 + u < topk) val[u] = __ldg(y + (row * topk + j0 + u) * vec_per_row + v);
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (j0 + u < topk) add_h16x8(val[u], acc, fp16);
    }
    const int ring = int(row / tokens_per_rank);
    const int t = int(row - int64_t(ring) * tokens_per_rank);
    uint4* dst = reinterpret_cast<uint4*>(partial.ptr[(rank + ring) % world]) +
                 (int64_t(rank) * tokens_per_rank + t) * vec_per_row + v;
    *dst = pack_h16x8(acc, fp16);
  }
  __threadfence_system();  // the stores to the peers are performed before the kernel ends
}

// out[t] = sum over the W planes of this rank's own `partial` buffer, ascending plane.
__global__ void sum_planes_kernel(const uint4* __restrict__ partial, int tokens, int world, int vec_per_row,
                                  uint4* __restrict__ out, int fp16) {
  const int64_t total = int64_t(tokens) * vec_per_row;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int p0 = 0; p0 < world; p0 += 8) {
      uint4 val[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (p0 + u < world) val[u] = __ldg(partial + int64_t(p0 + u) * total + i);
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (p0 + u < world) add_h16x8(val[u], acc, fp16);
    }
    out[i] = pack_h16x8(acc, fp16);
  }
}

// Quantise the 16 elements a thread holds of a 128-wide group shared by 8
// consecutive lanes; returns the group's scale (identical in the 8 lanes).
__device__ __forceinline__ float quantize_slice16(const uint4& a, const uint4& b, uint32_t (&w)[4], int ue8m0) {
  float f[16];
  const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 fa = __bfloat1622float2(ha[i]), fb = __bfloat1622float2(hb[i]);
    f[2 * i] = fa.x; f[2 * i + 1] = fa.y; f[8 + 2 * i] = fb.x; f[8 + 2 * i + 1] = fb.y;
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(f[i]));
  const unsigned group_mask = 0xFFu << (threadIdx.x & 24);  // the 8 lanes sharing this group
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(group_mask, amax, o));
  amax = fmaxf(amax, 1e-10f);
  const float scale = fp8_group_scale(amax, ue8m0);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float qv = fminf(fmaxf(__fdiv_rn(f[4 * i + j], scale), -448.f), 448.f);
      packed |= uint32_t(__nv_cvt_float_to_fp8(qv, __NV_SATFINITE, __NV_E4M3)) << (8 * j);
    }
    w[i] = packed;
  }
  return scale;
}

// One 128-wide group per 8 lanes (16 bf16 each).
__global__ void group_quant_fp8_kernel(const uint4* __restrict__ x, int64_t rows, int groups_per_row,
                                       uint2* __restrict__ q, float* __restrict__ scales,
                                       int64_t scale_ld, int transposed, int ue8m0) {
  const int64_t total_groups = rows * groups_per_row;
  const int sub = threadIdx.x & 7;
  for (int64_t g = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 3; g < total_groups;
       g += (int64_t(gridDim.x) * blockDim.x) >> 3) {
    const uint4* src = x + g * 16 + sub * 2;  // 16 elements = two 16-byte loads
    uint32_t w[4];
    const float scale = quantize_slice16(__ldg(src), __ldg(src + 1), w, ue8m0);
    uint2* dst = q + g * 16 + sub * 2;
    dst[0] = make_uint2(w[0], w[1]);
    dst[1] = make_uint2(w[2], w[3]);
    if (sub == 0) {
      const int64_t row = g / groups_per_row;
      const int64_t grp = g - row * groups_per_row;
      if (transposed) scales[grp * scale_ld + row] = scale;
      else scales[row * scale_ld + grp] = scale;
    }
  }
}

int grid_for(int64_t work_items, int threads, int device_sms, int waves) {
  int64_t blocks = (work_items + threads - 1) / threads;
  int64_t cap = int64_t(device_sms) * waves;
  if (blocks > cap) blocks = cap;
  return blocks < 1 ? 1 : int(blocks);
}

int sm_count() {
  int dev = 0;
  const int sms = cudaGetDevice(&dev) == cudaSuccess ? device_sm_count(dev) : 0;
  return sms > 0 ? sms : 148;
}

}  // namespace

int launch_combine_bf16(const __nv_bfloat16* y, const int* inverse, int tokens, int topk, int hidden,
                        __nv_bfloat16* out, cudaStream_t stream, int fp16) {
  MB200_REQUIRE(hidden % 8 == 0, kUnsupportedShape, "combine: hidden=%d must be a multiple of 8", hidden);
  if (tokens == 0) return kOk;
  const int threads = 256;
  const int blocks = grid_for(int64_t(tokens) * (hidden / 8), threads, sm_count(), 16);
  combine_bf16_kernel<<<blocks, threads, 0, stream>>>(reinterpret_cast<const uint4*>(y), inverse, tokens,
                                                     topk, hidden / 8, reinterpret_cast<uint4*>(out), fp16);
  MB200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

int launch_combine_push(const __nv_bfloat16* y, int all_tokens, int tokens_per_rank, int topk, int hidden,
                        const PeerTable& partial, int rank, int world, cudaStream_t stream, int fp16) {
  MB200_REQUIRE(hidden % 8 == 0, kUnsupportedShape, "combine: hidden=%d must be a multiple of 8", hidden);
  const int threads = 256;
  const int blocks = grid_for(int64_t(all_tokens) * (hidden / 8), threads, sm_count(), 16);
  combine_push_kernel<<<blocks, threads, 0, stream>>>(reinterpret_cast<const uint4*>(y), all_tokens, tokens_per_rank,
                                                     topk, hidden / 8, partial, rank, world, fp16);
  MB200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

int launch_sum_planes(const __nv_bfloat16* partial, int tokens, int world, int hidden, __nv_bfloat16* out,
                      cudaStream_t stream, int fp16) {
  const int threads = 256;
  const int blocks = grid_for(int64_t(tokens) * (hidden / 8), threads, sm_count(), 16);
  sum_planes_kernel<<<blocks, threads, 0, stream>>>(reinterpret_cast<const uint4*>(partial), tokens, world, hidden / 8,
                                                   reinterpret_cast<uint4*>(out), fp16);
  MB200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

int launch_group_quant_fp8(const __nv_bfloat16* x, int64_t rows, int hidden, uint8_t* q, float* scales,
                           int64_t scale_ld, int transposed, cudaStream_t stream, int ue8m0) {
  MB200_REQUIRE(hidden % 128 == 0, kUnsupportedShape, "group_quant: hidden=%d must be a multiple of 128", hidden);
  if (rows == 0) return kOk;
  const int threads = 256;
  const int blocks = grid_for(rows * (hidden / 128) * 8, threads, sm_count(), 16);
  group_quant_fp8_kernel<<<blocks, threads, 0, stream>>>(reinterpret_cast<const uint4*>(x), rows,
                                                        hidden / 128, reinterpret_cast<uint2*>(q), scales,
                                                        scale_ld, transposed, ue8m0);
  MB200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

}  // namespace mb200
