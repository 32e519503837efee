// Bridge to the CUDALM reference's own code.  TEST INFRASTRUCTURE ONLY.
//
// This translation unit pulls the reference's CPU test functions in by
// including the reference source files where they lie (the REF include root is
// given on the compiler command line by oracle/Makefile) and re-exports them
// with C linkage, so Python can call the reference itself:
//
//   * ref_gemv_bf16          tests/cuda/test_int4_gemv_bf16.cpp:54-69
//   * argmax_bf16            include/cudalm/greedy.h:28-39
//   * effective_probabilities (top-k keep set) include/cudalm/sampling.h:131-206
//   * int4::pack_byte / unpack_lo / unpack_hi  include/cudalm/weight_loader.h:102-119
//   * compare_bf16_stages    include/cudalm/stage_compare.h:117-137
//
// and, for a second opinion on a GPU box, the reference's CUDA entry points
// (int4_gemv_bf16, batch_int4_gemv_bf16, bf16_gemv) compiled from the
// reference's .cu files for sm_100a.  Nothing from the reference is copied
// into this repository; the resulting library lives in oracle/_ref/ and is not
// committed.  The shipped library never links or loads it.
#include <cstdint>
#include <cstring>
#include <vector>

// The reference test file defines main(); rename it so the file can be
// included for its helper functions (they sit in an anonymous namespace and
// are therefore reachable only from this translation unit).
#define main cudalm_ref_test_int4_gemv_bf16_main
#include "tests/cuda/test_int4_gemv_bf16.cpp"
#undef main

#include "cudalm/greedy.h"
#include "cudalm/kernels/batch_decode.h"
#include "cudalm/kernels/bf16_gemv.h"
#include "cudalm/sampling.h"
#include "cudalm/weight_loader.h"

extern "C" {

// The reference CPU GEMV, unchanged.  Pointers are host memory holding raw
// fp16 / bf16 bits.
void ref_cpu_gemv_bf16(const std::uint8_t* W, const std::uint16_t* S,
                       const std::uint16_t* x, int N, int K, std::uint16_t* y) {
  std::vector<__nv_bfloat16> out;
  ref_gemv_bf16(W, reinterpret_cast<const __half*>(S),
                reinterpret_cast<const __nv_bfloat16*>(x), N, K, &out);
  std::memcpy(y, out.data(), sizeof(std::uint16_t) * static_cast<std::size_t>(N));
}

int ref_cpu_argmax_bf16(const std::uint16_t* logits, int n) {
  return cudalm::argmax_bf16(reinterpret_cast<const __nv_bfloat16*>(logits), n);
}

// keep[i] = 1 when token i survives the reference's top-k filter at
// temperature 1 and top_p 1.  (The reference exposes the kept set through the
// probabilities it returns; a kept token has probability > 0 unless it is
// more than ~100 below the maximum, so callers use moderate logit ranges.)
void ref_cpu_topk_keep(const std::uint16_t* logits, int vocab, int k,
                       std::uint8_t* keep) {
  cudalm::SamplingConfig cfg;
  cfg.temperature = 1.0f;
  cfg.top_k = k;
  cfg.top_p = 1.0f;
  const std::vector<float> p = cudalm::effective_probabilities(
      reinterpret_cast<const __nv_bfloat16*>(logits), vocab, cfg);
  for (int i = 0; i < vocab; ++i) keep[i] = p[static_cast<std::size_t>(i)] > 0.0f;
}

// The reference's sample_token (include/cudalm/sampling.h:200-234) on full
// logits; *state is the SplitMix64 state before the call and after it.
int ref_cpu_sample_token(const std::uint16_t* logits, int vocab, float temperature, int top_k,
                         float top_p, std::uint64_t* state) {
  cudalm::SamplingConfig cfg;
  cfg.temperature = temperature;
  cfg.top_k = top_k;
  cfg.top_p = top_p;
  cudalm::SplitMix64 rng(*state);
  const int tok = cudalm::sample_token(reinterpret_cast<const __nv_bfloat16*>(logits), vocab, cfg, &rng);
  *state = rng.state;
  return tok;
}

int ref_cpu_unpack_lo(int b) {
  return cudalm::int4::unpack_lo(static_cast<std::uint8_t>(b));
}
int ref_cpu_unpack_hi(int b) {
  return cudalm::int4::unpack_hi(static_cast<std::uint8_t>(b));
}
int ref_cpu_pack_byte(int lo, int hi) { return cudalm::int4::pack_byte(lo, hi); }

// The reference's bf16 stage comparator (atol = rtol = 1e-2 by default).
int ref_cpu_compare_bf16_ok(const std::uint16_t* ref, const std::uint16_t* act,
                            std::size_t n) {
  return cudalm::compare_bf16_stages(ref, act, n).ok ? 1 : 0;
}

// ---- reference CUDA entry points (device pointers; GPU box only) ---------
void ref_gpu_int4_gemv_bf16(const void* W, const void* S, const void* x, void* y,
                            int N, int K, void* stream) {
  cudalm::int4_gemv_bf16(static_cast<const std::uint8_t*>(W),
                         static_cast<const __half*>(S),
                         static_cast<const __nv_bfloat16*>(x),
                         static_cast<__nv_bfloat16*>(y), N, K,
                         static_cast<cudaStream_t>(stream));
}
void ref_gpu_batch_int4_gemv_bf16(const void* W, const void* S, const void* x,
                                  void* y, int N, int K, int B, void* stream) {
  cudalm::kernels::batch_int4_gemv_bf16(
      static_cast<const std::uint8_t*>(W), static_cast<const __half*>(S),
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), N, K,
      B, static_cast<cudaStream_t>(stream));
}
void ref_gpu_bf16_gemv(const void* W, const void* x, void* y, int N, int K,
                       void* stream) {
  cudalm::bf16_gemv(static_cast<const __nv_bfloat16*>(W),
                    static_cast<const __nv_bfloat16*>(x),
                    static_cast<__nv_bfloat16*>(y), N, K,
                    static_cast<cudaStream_t>(stream));
}

}  // extern "C"
