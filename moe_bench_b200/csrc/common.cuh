// Shared device helpers for the sm_100a MoE layer kernels: error reporting,
// mbarrier / TMA / tcgen05 PTX wrappers and bounded waits.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mb200 {

// ---- status codes (also returned through the C ABI) ------------------------
enum Status : int {
  kOk = 0,
  kInvalidArgument = 1,
  kCudaError = 2,
  kDriverEntryMissing = 3,
  kWorkspaceTooSmall = 4,
  kUnsupportedShape = 5,
  // device-side codes, written to the status word in the workspace
  kDevWaitTimeout = 100,
};

void set_last_error(const char* fmt, ...);

#define MB200_CHECK_CUDA(expr)                                                        \
  do {                                                                                \
    cudaError_t _e = (expr);                                                          \
    if (_e != cudaSuccess) {                                                          \
      ::mb200::set_last_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                              __FILE__, __LINE__);                                    \
      return ::mb200::kCudaError;                                                     \
    }                                                                                 \
  } while (0)

#define MB200_REQUIRE(cond, code, ...)        \
  do {                                        \
    if (!(cond)) {                            \
      ::mb200::set_last_error(__VA_ARGS__);   \
      return (code);                          \
    }                                         \
  } while (0)

// ---- small device utilities -------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---- 16-bit activations: bf16 or fp16, chosen at run time (a warp-uniform flag) ----
__device__ __forceinline__ uint16_t to_h16(float v, int fp16) {
  if (fp16) return __half_as_ushort(__float2half_rn(v));
  return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}
__device__ __forceinline__ void add_h16x8(const uint4& v, float (&acc)[8], int fp16) {
  if (fp16) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      acc[2 * i] += f.x;
      acc[2 * i + 1] += f.y;
    }
  } else {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      acc[2 * i] += f.x;
      acc[2 * i + 1] += f.y;
    }
  }
}
__device__ __forceinline__ uint4 pack_h16x8(const float (&acc)[8], int fp16) {
  uint4 o;
  uint32_t* w = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int k = 0; k < 4; ++k)
    w[k] = uint32_t(to_h16(acc[2 * k], fp16)) | (uint32_t(to_h16(acc[2 * k + 1], fp16)) << 16);
  return o;
}

// ---- fp8 activation scale ------------------------------------------------------
// Scale of one 1x128 activation group from its absolute maximum (already clamped to
// 1e-10): amax / 448 (the reference's quantiser, reference.py:143-145 -> vLLM
// per_token_group_quant_fp8), or, when vLLM runs with DeepGEMM's E8M0 scales (its
// default on Hopper / Blackwell), that value rounded UP to a power of two:
// exp2(ceil(log2(.))), the formula of vLLM's quantiser.
__device__ __forceinline__ float fp8_group_scale(float amax, int ue8m0) {
  float scale = __fdiv_rn(amax, 448.0f);
  if (ue8m0) scale = exp2f(ceilf(log2f(fmaxf(fabsf(scale), 1e-10f))));
  return scale;
}

// ---- mbarrier -----------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Every in-kernel wait is bounded.  The limit applies to ONE wait (the clock starts
// when that wait first finds nothing to do), so it bounds lack of progress, not the
// length of the launch.  A wait that gives up writes kDevWaitTimeout + site to the
// status word (first failure wins), raises the CTA's abort flag and the kernel
// leaves through its normal teardown, so the context stays usable.
// Default limit; word 1 of the status block (milliseconds, 0 = default) overrides it.
constexpr uint64_t kDefaultWaitLimitNs = 4ull * 1000 * 1000 * 1000;

struct WaitCtx {
  volatile int* abort_flag;  // shared memory, one per CTA
  int* status;               // global status block (may be null): [0] status, [1] wait limit in ms
  uint64_t limit_ns;
};

__device__ __forceinline__ uint64_t wait_limit_ns(const int* status) {
  const int ms = status ? __ldg(status + 1) : 0;
  return ms > 0 ? uint64_t(ms) * 1000000ull : kDefaultWaitLimitNs;
}

// Bookkeeping of one bounded wait: call expired() every few hundred polls.
struct WaitClock {
  uint64_t begin = 0;
  __device__ __forceinline__ bool expired(const WaitCtx& ctx) {
    const uint64_t now = global_timer_ns();
    if (begin == 0) { begin = now; return false; }
    return now - begin > ctx.limit_ns;
  }
};

__device__ __forceinline__ void wait_give_up(WaitCtx& ctx, int where) {
  *ctx.abort_flag = 1;
  if (ctx.status) atomicCAS(ctx.status, 0, kDevWaitTimeout + where);
}

// Warp-collective: all 32 lanes call it together and get the same answer (a lane
// that saw the phase complete while another lane ran out of time would otherwise
// leave the warp split).  Returns false when the wait was abandoned.
__device__ __forceinline__ bool mbar_wait_lane(uint32_t bar, uint32_t parity, WaitCtx& ctx, int where);
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, WaitCtx& ctx, int where) {
  const bool ok = mbar_wait_lane(bar, parity, ctx, where);
  return __all_sync(0xffffffffu, ok);
}
__device__ __forceinline__ bool mbar_wait_lane(uint32_t bar, uint32_t parity, WaitCtx& ctx, int where) {
  uint32_t spins = 0;
  WaitClock clock;
  while (true) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((++spins & 0x3FF) == 0) {
      if (*ctx.abort_flag) return false;
      if (clock.expired(ctx)) {
        wait_give_up(ctx, where);
        return false;
      }
    }
  }
}

// ---- TMA ------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// 2-D tiled load global -> shared (this CTA), completion on an mbarrier.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int c0, int c1,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

// Untiled bulk copy global -> shared (this CTA), completion on an mbarrier.  Both
// addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
      : "memory");
}

// ---- tcgen05 / tensor memory ----------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive on an mbarrier once every tcgen05.mma issued so far by this thread has
// finished (it implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile whose rows are
// 128 bytes wide and were written with the 128-byte swizzle (TMA
// SWIZZLE_128B): 8-row groups are 1024 bytes apart (SBO), the leading byte
// offset is not used by swizzled K-major layouts (1), descriptor version 1,
// layout type 2 = SWIZZLE_128B.  The tile base must be 1024-byte aligned;
// stepping along K inside the 128-byte row adds the byte offset to the start
// address field.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor, dense, fp32 accumulate, both operands K-major.
//   fmt: kind::f16 -> 0 = f16, 1 = bf16;  kind::f8f6f4 -> 0 = e4m3, 1 = e5m2
__host__ __device__ constexpr uint32_t make_idesc(uint32_t fmt_a, uint32_t fmt_b, uint32_t m,
                                                   uint32_t n) {
  return (1u << 4) | (fmt_a << 7) | (fmt_b << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_fp8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32 lanes x 16 consecutive fp32 columns of tensor memory -> 16 registers per
// thread (thread i of the warp reads lane base+i).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32"
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 32 lanes x 32 consecutive fp32 columns -> 32 registers per thread.  The load is
// asynchronous: the registers hold the data only after tmem_ld_wait32 on the same array.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32"
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
// Waits for every tensor-memory load this thread has issued.  The array is named as an
// in/out operand so that the compiler cannot move a use of it above the wait while an
// independent load into ANOTHER array stays in flight across it.
__device__ __forceinline__ void tmem_ld_wait32(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                 "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]),
                 "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]),
                 "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}

// Two fp32 lanes per instruction (fma.rn.f32x2): acc = p * s + acc on register pairs.
// Each lane is an IEEE fused multiply-add, bit-identical to fmaf.
__device__ __forceinline__ uint64_t pack_f32x2(uint32_t lo, uint32_t hi) {
  uint64_t v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "r"(lo), "r"(hi));
  return v;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
  uint32_t a, b;
  asm("mov.b64 {%0, %1}, %2;" : "=r"(a), "=r"(b) : "l"(v));
  lo = __uint_as_float(a);
  hi = __uint_as_float(b);
}
__device__ __forceinline__ void fma_f32x2(uint64_t& acc, uint64_t p, uint64_t s) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(p), "l"(s));
}

}  // namespace mb200
