// GPU quantize + pack: bf16 W [N, K] -> int4 [N, K/2] + fp16 scales [N, K/128],
// bit-exact with CUDALM's offline quantizer (tools/common/w4a16_quant.py:25-60).
//
// Sixteen lanes own one group of 128 values: each lane loads 16 bytes (8 bf16),
// the group's max |w| is reduced with four shuffles, and each lane writes the
// four packed bytes of its eight values.  The arithmetic is the quantizer's,
// operation for operation: scale32 = amax / 7 (IEEE fp32 divide), q =
// round-half-even(w / scale32) (IEEE fp32 divide, not a reciprocal multiply),
// clamp to [-7, 7]; a group whose fp32 scale is zero stores q = 0; the stored
// scale is fp16_rn(scale32), which may be zero although q is not.
#include "common.cuh"

namespace cb200 {

// rint(fl(w / s)) for |w| <= 7 s.  The common case avoids the IEEE divide: the
// approximate quotient w * (1/s) is within a few ulps of the true one, so
// unless it lies within 2^-10 of a rounding boundary (k + 0.5) both round to
// the same integer; only then is the exact divide evaluated.
__device__ __forceinline__ float quant_round(float w, float s, float inv_s) {
  const float approx = w * inv_s;
  const float r = rintf(approx);
  const float frac = fabsf(approx - r);
  // also taken when the reciprocal overflowed (denormal scale): frac is NaN
  if (!(frac <= 0.499f)) return rintf(__fdiv_rn(w, s));
  return r;
}

// Inserts the low four bits of `v` into `word` at bit position `pos`.
__device__ __forceinline__ std::uint32_t insert_nibble(std::uint32_t word, std::uint32_t v, int pos) {
  std::uint32_t r;
  asm("bfi.b32 %0, %1, %2, %3, 4;" : "=r"(r) : "r"(v), "r"(word), "r"(pos));
  return r;
}

// One group's share of a lane: eight values in, one packed word out.
__device__ __forceinline__ std::uint32_t quantize_eight(const uint4& v, unsigned mask, float* scale_out) {
  const std::uint32_t words[4] = {v.x, v.y, v.z, v.w};
  float w[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    w[2 * i] = __uint_as_float(words[i] << 16);
    w[2 * i + 1] = __uint_as_float(words[i] & 0xFFFF0000u);
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(w[i]));
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(mask, amax, off));
  const float scale32 = __fdiv_rn(amax, 7.0f);
  *scale_out = scale32;
  if (scale32 == 0.f) return 0u;  // the whole group (all 16 lanes see the same scale)
  const float inv = __frcp_rn(scale32);
  std::uint32_t out = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    // No clamp: |w| <= amax and scale32 = fl(amax / 7) >= (amax / 7)(1 - 2^-24) (for a
    // subnormal scale: within 2^-14 of it, the smallest bf16 being 2^-133), so the quotient
    // stays below 7.5 and rounds into [-7, 7] by itself, as the quantizer's clip then
    // never acts on finite inputs.
    const float q = quant_round(w[i], scale32, inv);
    // q is an integer in [-7, 7]: adding 1.5 * 2^23 leaves it, in two's
    // complement, in the low mantissa bits
    out = insert_nibble(out, __float_as_uint(q + 12582912.0f), 4 * i);
  }
  return out;
}

__global__ void __launch_bounds__(256)
quantize_w4a16_kernel(const uint4* __restrict__ W, std::uint32_t* __restrict__ packed,
                      std::uint16_t* __restrict__ scales, long long n_groups) {
  const int lane16 = threadIdx.x & 15;
  const long long half_warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 4;
  long long grp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4;
  // The 16 lanes of a half-warp share `grp`; the two halves of a warp may leave
  // the loop at different times, so the shuffles name only their own half.
  const unsigned mask = (threadIdx.x & 16) ? 0xFFFF0000u : 0x0000FFFFu;
  // four groups per trip so that four loads are in flight per lane
  for (; grp + 3 * half_warps < n_groups; grp += 4 * half_warps) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = __ldg(W + (grp + u * half_warps) * 16 + lane16);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float scale32;
      const std::uint32_t out = quantize_eight(v[u], mask, &scale32);
      const long long g = grp + u * half_warps;
      packed[g * 16 + lane16] = out;
      if (lane16 == 0) scales[g] = __half_as_ushort(__float2half_rn(scale32));
    }
  }
  for (; grp < n_groups; grp += half_warps) {
    const uint4 v = __ldg(W + grp * 16 + lane16);
    float scale32;
    const std::uint32_t out = quantize_eight(v, mask, &scale32);
    packed[grp * 16 + lane16] = out;
    if (lane16 == 0) scales[grp] = __half_as_ushort(__float2half_rn(scale32));
  }
}

}  // namespace cb200

extern "C" int cudalm_b200_quantize_w4a16(const uint16_t* w_bf16, int N, int K, uint8_t* packed,
                                          uint16_t* scales, void* stream) {
  using namespace cb200;
  if (!w_bf16 || !packed || !scales) return CUDALM_B200_ERR_NULL;
  if (N < 1 || K <= 0 || (K % 128) != 0) return CUDALM_B200_ERR_BAD_SHAPE;
  if (!aligned_to(w_bf16, 16) || !aligned_to(packed, 4)) return CUDALM_B200_ERR_MISALIGNED;
  const long long n_groups = static_cast<long long>(N) * (K / 128);
  const int threads = 256;
  // a half-warp takes four groups per trip: size the grid so that it has them
  long long blocks = (((n_groups + 3) / 4) * 16 + threads - 1) / threads;
  const long long cap = static_cast<long long>(num_sms()) * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  quantize_w4a16_kernel<<<static_cast<int>(blocks), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(w_bf16), reinterpret_cast<std::uint32_t*>(packed), scales,
      n_groups);
  return check_launch();
}
