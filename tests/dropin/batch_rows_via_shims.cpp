// A C++ caller that uses CUDALM's own names and signatures -- cudalm::int4_gemv_bf16
// and cudalm::kernels::batch_int4_gemv_bf16, as include/cudalm_b200_shims.hpp provides
// them over the C ABI -- and checks what CUDALM's batch-kernel test checks for the
// W4A16 GEMV (CUDALM tests/cuda/test_qwen35_batch_kernels.cpp:88-134): row b of a
// batched call is bit-identical to the single call on row b's own input.  Here that
// holds for every batch width the batched call shares a kernel with the single call
// (up to 8 rows), on that test's shape and on the production shapes.
//
// Exit status 0 when every row of every case is bit-identical.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

#include "cudalm_b200_shims.hpp"

namespace {

struct Lcg {  // deterministic values in [-1, 1)
  std::uint32_t s;
  explicit Lcg(std::uint32_t seed) : s(seed ? seed : 1u) {}
  float next() {
    s = s * 1664525u + 1013904223u;
    return static_cast<float>(s >> 8) * (2.0f / static_cast<float>(1u << 24)) - 1.0f;
  }
};

#define CUDA_OK(call)                                                              \
  do {                                                                             \
    cudaError_t e__ = (call);                                                      \
    if (e__ != cudaSuccess) {                                                      \
      std::fprintf(stderr, "%s: %s\n", #call, cudaGetErrorString(e__));            \
      return 2;                                                                    \
    }                                                                              \
  } while (0)

int check_shape(int N, int K, int B, cudaStream_t st) {
  Lcg rng(101u + static_cast<std::uint32_t>(N) * 7u + static_cast<std::uint32_t>(K) + static_cast<std::uint32_t>(B));
  std::vector<std::uint8_t> W(static_cast<std::size_t>(N) * K / 2);
  std::vector<__half> S(static_cast<std::size_t>(N) * (K / 128));
  std::vector<__nv_bfloat16> x(static_cast<std::size_t>(B) * K);
  for (auto& w : W) w = static_cast<std::uint8_t>(rng.next() * 127.0f + 127.0f);
  for (auto& s : S) s = __float2half(0.01f * rng.next() + 0.011f);
  for (auto& v : x) v = __float2bfloat16_rn(rng.next());

  std::uint8_t* dW = nullptr;
  __half* dS = nullptr;
  __nv_bfloat16 *dx = nullptr, *dy = nullptr, *dy1 = nullptr;
  CUDA_OK(cudaMalloc(&dW, W.size()));
  CUDA_OK(cudaMalloc(&dS, S.size() * sizeof(__half)));
  CUDA_OK(cudaMalloc(&dx, x.size() * sizeof(__nv_bfloat16)));
  CUDA_OK(cudaMalloc(&dy, static_cast<std::size_t>(B) * N * sizeof(__nv_bfloat16)));
  CUDA_OK(cudaMalloc(&dy1, static_cast<std::size_t>(N) * sizeof(__nv_bfloat16)));
  CUDA_OK(cudaMemcpyAsync(dW, W.data(), W.size(), cudaMemcpyHostToDevice, st));
  CUDA_OK(cudaMemcpyAsync(dS, S.data(), S.size() * sizeof(__half), cudaMemcpyHostToDevice, st));
  CUDA_OK(cudaMemcpyAsync(dx, x.data(), x.size() * sizeof(__nv_bfloat16), cudaMemcpyHostToDevice, st));

  cudalm::kernels::batch_int4_gemv_bf16(dW, dS, dx, dy, N, K, B, st);
  std::vector<std::uint16_t> batch(static_cast<std::size_t>(B) * N), one(static_cast<std::size_t>(N));
  CUDA_OK(cudaMemcpyAsync(batch.data(), dy, batch.size() * 2, cudaMemcpyDeviceToHost, st));
  int bad = 0;
  for (int b = 0; b < B; ++b) {
    cudalm::int4_gemv_bf16(dW, dS, dx + static_cast<std::size_t>(b) * K, dy1, N, K, st);
    CUDA_OK(cudaMemcpyAsync(one.data(), dy1, one.size() * 2, cudaMemcpyDeviceToHost, st));
    CUDA_OK(cudaStreamSynchronize(st));
    const bool same = std::memcmp(one.data(), batch.data() + static_cast<std::size_t>(b) * N, one.size() * 2) == 0;
    bool nonzero = false;
    for (std::uint16_t v : one) nonzero |= (v & 0x7FFFu) != 0;
    if (!same || !nonzero) {
      std::fprintf(stderr, "  N=%d K=%d B=%d row %d: %s\n", N, K, B, b, same ? "all zero" : "differs from the single call");
      ++bad;
    }
  }
  cudaFree(dW);
  cudaFree(dS);
  cudaFree(dx);
  cudaFree(dy);
  cudaFree(dy1);
  return bad;
}

}  // namespace

int main() {
  CUDA_OK(cudaSetDevice(0));
  cudaStream_t st = nullptr;
  CUDA_OK(cudaStreamCreate(&st));
  const int shapes[][3] = {{512, 512, 3},   {16, 1024, 2},  {512, 1024, 3},  {1024, 2048, 2}, {1024, 3584, 3},
                           {2048, 1024, 8}, {3584, 1024, 5}, {4096, 1024, 2}, {6144, 1024, 3}, {37, 256, 8}};
  int bad = 0;
  for (const auto& s : shapes) bad += check_shape(s[0], s[1], s[2], st);
  CUDA_OK(cudaStreamDestroy(st));
  if (bad) {
    std::fprintf(stderr, "batch_rows_via_shims: FAIL (%d rows)\n", bad);
    return 1;
  }
  std::printf("batch_rows_via_shims: PASS (every batched row is bit-identical to the single call)\n");
  return 0;
}
