// Shared device/host helpers for the W4A16 projection kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>

#include "../../include/cudalm_b200.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "this library is written for sm_100a (B200) only"
#endif

namespace cb200 {

// ---------------------------------------------------------------------------
// Host-side bookkeeping
// ---------------------------------------------------------------------------
extern thread_local int g_last_cuda_error;
extern std::atomic<long long> g_launch_count;
// Device-side status word of the current device (bounded waits report here).
int* device_status_word();
int num_sms();

#define CB200_CUDA_TRY(call)                                  \
  do {                                                        \
    cudaError_t cb200_e__ = (call);                           \
    if (cb200_e__ != cudaSuccess) {                           \
      ::cb200::g_last_cuda_error = static_cast<int>(cb200_e__); \
      return CUDALM_B200_ERR_CUDA;                            \
    }                                                         \
  } while (0)

inline int check_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    g_last_cuda_error = static_cast<int>(e);
    return CUDALM_B200_ERR_CUDA;
  }
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return CUDALM_B200_OK;
}

inline bool aligned_to(const void* p, std::uintptr_t a) {
  return (reinterpret_cast<std::uintptr_t>(p) & (a - 1)) == 0;
}

// Largest dynamic shared memory a CTA may opt into on B200 (227 KB).
constexpr int kMaxSmemBytes = 232448;

// ---------------------------------------------------------------------------
// Device helpers
// ---------------------------------------------------------------------------
#ifdef __CUDACC__

__device__ __forceinline__ std::uint32_t smem_u32(const void* p) {
  return static_cast<std::uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier (shared::cta) ------------------------------------------------
__device__ __forceinline__ void mbar_init(std::uint64_t* bar, std::uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(count)
               : "memory");
}
// Makes freshly initialised barriers visible to the async (bulk-copy) proxy.
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(std::uint64_t* bar,
                                                      std::uint32_t tx_bytes) {
  asm volatile(
      "mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
      "r"(tx_bytes)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive(std::uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(std::uint64_t* bar,
                                              std::uint32_t parity) {
  std::uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// ---- bulk async copy global -> shared (TMA engine, untiled form) -----------
// dst and src 16-byte aligned, bytes a multiple of 16.  Completion is
// signalled on `bar` as `bytes` of transaction count.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src,
                                         std::uint32_t bytes, std::uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ std::uint64_t policy_evict_first() {
  std::uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// ---- shared-memory loads ---------------------------------------------------
// Plain (non-volatile) loads: the compiler is free to hoist them above earlier
// tensor-core instructions, which is what hides their latency.  They stay
// behind the mbarrier wait because that asm clobbers memory.
__device__ __forceinline__ uint4 lds128(const std::uint8_t* p) {
  return *reinterpret_cast<const uint4*>(p);
}
__device__ __forceinline__ uint2 lds64(const std::uint8_t* p) {
  return *reinterpret_cast<const uint2*>(p);
}
__device__ __forceinline__ std::uint16_t lds16(const std::uint8_t* p) {
  return *reinterpret_cast<const std::uint16_t*>(p);
}

// ---- int4 -> bf16 dequantisation --------------------------------------------
// Building blocks: for a 4-bit two's-complement value n, (n ^ 8) is q + 8 in
// [0, 15]; OR-ing it under the bf16 pattern 0x4300 (128.0, whose ulp is 1) gives
// the bf16 number 136 + q; subtracting 136.0 (0x4308) is exact.  One LOP3 computes
// (w & 0x000F000F) ^ 0x43084308 for two nibbles of a word.
__device__ __forceinline__ std::uint32_t lop3_and_xor(std::uint32_t a,
                                                      std::uint32_t b,
                                                      std::uint32_t c) {
  std::uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ std::uint32_t sub_bf16x2(std::uint32_t a, std::uint32_t b) {
  std::uint32_t d;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// ---- legacy-path tensor-core MMA (m16n8k16, bf16 x bf16 -> fp32) -------------
__device__ __forceinline__ void mma_m16n8k16_bf16(float (&c)[4], std::uint32_t a0,
                                                  std::uint32_t a1, std::uint32_t a2,
                                                  std::uint32_t a3, std::uint32_t b0,
                                                  std::uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float bf16_bits_to_float(std::uint16_t b) {
  return __uint_as_float(static_cast<std::uint32_t>(b) << 16);
}
__device__ __forceinline__ std::uint16_t float_to_bf16_bits(float f) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}

#endif  // __CUDACC__

#ifdef __CUDACC__
// Epilogues of the MLP, in CUDALM's rounding order.
__device__ __forceinline__ std::uint16_t silu_bits(std::uint16_t gate_bits) {
  const float g = bf16_bits_to_float(gate_bits);
  return float_to_bf16_bits(__fdiv_rn(g, 1.0f + expf(-g)));
}
__device__ __forceinline__ std::uint16_t silu_mul_bits(float g, std::uint16_t up_bits) {
  const float s = bf16_bits_to_float(float_to_bf16_bits(__fdiv_rn(g, 1.0f + expf(-g))));
  return float_to_bf16_bits(s * bf16_bits_to_float(up_bits));
}
__device__ __forceinline__ std::uint16_t add_bits(std::uint16_t a, std::uint16_t b) {
  return float_to_bf16_bits(bf16_bits_to_float(a) + bf16_bits_to_float(b));
}

#endif

}  // namespace cb200
