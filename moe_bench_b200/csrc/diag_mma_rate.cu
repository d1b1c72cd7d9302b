// Diagnostic, not part of the library: issue rate of tcgen05.mma alone.
//
// One CTA (or one per SM) keeps two 128 x 64 bf16 A tiles and one N x 64 B tile
// resident in shared memory (zero-filled; values do not change the timing) and a
// single thread issues 2000 x 8 MMAs of shape 128 x N x 16 into two accumulators,
// the instruction mix of one K step of the grouped GEMM, with no TMA traffic.
// Prints SM cycles per MMA for N = 16 .. 256.  Measured on B200: exactly N/2
// cycles from N = 128 up (4096 FMA/clk/SM), 44-64 cycles below.  The wait on the
// commit barrier is bounded like every wait of the library.
//
//   python -m moe_bench_b200.build --diagnostics && ./moe_bench_b200/diag_mma_rate
#include <cstdio>
#include "common.cuh"
using namespace mb200;

__global__ void __launch_bounds__(128, 1) mma_n_kernel(int n, int iters, long long* out) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw & 1023u)) & 1023u;
  const uint32_t base = raw + pad;
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  for (int i = threadIdx.x; i < (64 * 1024) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem_raw + pad)[i] = 0;
  if (threadIdx.x == 0) { mbar_init(smem_u32(&bar), 1); abort_flag = 0; asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
  if (threadIdx.x < 32) { tmem_alloc(smem_u32(&tmem_base_s), 512); tmem_relinquish(); }
  asm volatile("fence.proxy.async;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  if (threadIdx.x == 0) {
    WaitCtx ctx{&abort_flag, nullptr, global_timer_ns()};
    const uint32_t idesc = make_idesc(1, 1, 128, uint32_t(n));
    const uint64_t a0 = make_kmajor_sw128_desc(base);
    const uint64_t a1 = make_kmajor_sw128_desc(base + 16384);
    const uint64_t b = make_kmajor_sw128_desc(base + 32768);
    long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        umma_bf16(tmem, a0 + 2 * k, b + 2 * k, idesc, 1);
        umma_bf16(tmem + 256, a1 + 2 * k, b + 2 * k, idesc, 1);
      }
    }
    tc_commit(smem_u32(&bar));
    mbar_wait(smem_u32(&bar), 0, ctx, 1);
    long long t1 = clock64();
    if (blockIdx.x == 0) out[0] = t1 - t0;
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

int main() {
  long long* d; cudaMalloc(&d, 8);
  cudaFuncSetAttribute(mma_n_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 66 * 1024);
  int sms = 0; cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
  const int iters = 2000;
  for (int rep = 0; rep < 2; ++rep)
    for (int n : {16, 32, 64, 96, 112, 128, 136, 144, 160, 176, 192, 208, 224, 240, 256}) {
      for (int grid : {1, sms}) {
        mma_n_kernel<<<grid, 128, 66 * 1024>>>(n, iters, d);
        cudaError_t e = cudaDeviceSynchronize();
        long long c = 0; cudaMemcpy(&c, d, 8, cudaMemcpyDeviceToHost);
        if (rep == 1) printf("N=%3d grid=%3d  cycles per 128xNx16 MMA: %.1f  (N/2 = %.1f)  %s\n", n, grid, double(c) / (iters * 8), n / 2.0, cudaGetErrorString(e));
      }
    }
  return 0;
}
