// C++ shims with CUDALM's own names and signatures over the C ABI, so that
// CUDALM's call sites (src/runtime/qwen35_deltanet.cpp:166-252,327-412,
// src/runtime/qwen35_full_attention.cpp:211-340,466-558,
// src/runtime/qwen35_model.cpp:177-181,290-292,500-502) compile unchanged.
//
// CUDALM's kernels abort on a contract violation or a CUDA error
// (include/cudalm/cuda_check.h:38-63); the C ABI returns a status instead, and
// these shims restore the print-and-abort so caller semantics are kept.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include "cudalm_b200.h"

namespace cudalm {

namespace b200_detail {
inline void check(int status, const char* what) {
  if (status != CUDALM_B200_OK) {
    std::fprintf(stderr, "[cudalm] %s failed: %s (status %d, cudaError %d)\n", what,
                 cudalm_b200_status_string(status), status, cudalm_b200_last_cuda_error());
    std::abort();
  }
}
inline const std::uint16_t* u16(const void* p) { return static_cast<const std::uint16_t*>(p); }
inline std::uint16_t* u16(void* p) { return static_cast<std::uint16_t*>(p); }
}  // namespace b200_detail

// include/cudalm/kernels/int4_gemv_bf16.h:46-48
inline void int4_gemv_bf16(const std::uint8_t* weight, const __half* scales,
                           const __nv_bfloat16* x, __nv_bfloat16* y, int N, int K,
                           cudaStream_t stream) {
  b200_detail::check(cudalm_b200_int4_gemv_bf16(weight, b200_detail::u16(scales),
                                                b200_detail::u16(x), b200_detail::u16(y), N, K,
                                                stream),
                     "int4_gemv_bf16");
}

namespace kernels {

// include/cudalm/kernels/batch_decode.h:61-63
inline void batch_int4_gemv_bf16(const std::uint8_t* weight, const __half* scale,
                                 const __nv_bfloat16* x, __nv_bfloat16* y, int N, int K, int B,
                                 cudaStream_t stream) {
  b200_detail::check(cudalm_b200_batch_int4_gemv_bf16(weight, b200_detail::u16(scale),
                                                      b200_detail::u16(x), b200_detail::u16(y), N,
                                                      K, B, stream),
                     "batch_int4_gemv_bf16");
}

// The MLP's gate and up projections over one input in a single launch; replaces
// the pair of calls at src/runtime/qwen35_deltanet.cpp:236-243 and
// src/runtime/qwen35_full_attention.cpp:317-326 (B = 1) and their batched forms.
inline void gate_up_int4_gemv_bf16(const std::uint8_t* gate_weight, const __half* gate_scale,
                                   const std::uint8_t* up_weight, const __half* up_scale,
                                   const __nv_bfloat16* x, __nv_bfloat16* gate_y,
                                   __nv_bfloat16* up_y, int N, int K, int B,
                                   cudaStream_t stream) {
  b200_detail::check(
      cudalm_b200_gate_up_bf16(gate_weight, b200_detail::u16(gate_scale), up_weight,
                               b200_detail::u16(up_scale), b200_detail::u16(x),
                               b200_detail::u16(gate_y), b200_detail::u16(up_y), N, K, B, stream),
      "gate_up_int4_gemv_bf16");
}

// The MLP's gate and up projections with silu(gate) * up applied in the same
// launch; replaces the two projections and qwen35_silu_mul
// (include/cudalm/kernels/qwen35_kernels.h:137-155) at
// src/runtime/qwen35_deltanet.cpp:236-247 and its batched form.
inline void gate_up_silu_int4_gemv_bf16(const std::uint8_t* gate_weight, const __half* gate_scale,
                                        const std::uint8_t* up_weight, const __half* up_scale,
                                        const __nv_bfloat16* x, __nv_bfloat16* act, int N, int K,
                                        int B, cudaStream_t stream) {
  b200_detail::check(
      cudalm_b200_gate_up_silu_bf16(gate_weight, b200_detail::u16(gate_scale), up_weight,
                                    b200_detail::u16(up_scale), b200_detail::u16(x),
                                    b200_detail::u16(act), N, K, B, stream),
      "gate_up_silu_int4_gemv_bf16");
}

// A projection followed by the residual add (qwen35_add,
// include/cudalm/kernels/qwen35_kernels.h:137-145) in one launch; `y` may be
// `residual`.  Replaces src/runtime/qwen35_deltanet.cpp:248-252 and the o_proj /
// out_proj call sites followed by an add.
inline void int4_gemv_residual_bf16(const std::uint8_t* weight, const __half* scale,
                                    const __nv_bfloat16* x, const __nv_bfloat16* residual,
                                    __nv_bfloat16* y, int N, int K, int B, cudaStream_t stream) {
  b200_detail::check(
      cudalm_b200_linear_residual_bf16(weight, b200_detail::u16(scale), b200_detail::u16(x),
                                       b200_detail::u16(residual), b200_detail::u16(y), N, K, B,
                                       stream),
      "int4_gemv_residual_bf16");
}

// lm_head stored as W4A16 with the token pick on the device; replaces
// batch_bf16_gemv (include/cudalm/kernels/batch_decode.h:77-79) followed by the
// host pick (src/runtime/scheduler.cpp:91-108).  `logits` may be null.
inline void lm_head_int4_topk_bf16(const std::uint8_t* weight, const __half* scale,
                                   const __nv_bfloat16* x, int N, int K, int B, int top_k,
                                   __nv_bfloat16* logits, std::int32_t* argmax,
                                   std::int32_t* topk_idx, __nv_bfloat16* topk_val,
                                   void* workspace, std::size_t workspace_bytes,
                                   cudaStream_t stream) {
  b200_detail::check(
      cudalm_b200_lm_head_topk(weight, b200_detail::u16(scale), b200_detail::u16(x), N, K, B,
                               top_k, 0, b200_detail::u16(logits), argmax, topk_idx,
                               b200_detail::u16(topk_val), workspace, workspace_bytes, stream),
      "lm_head_int4_topk_bf16");
}

// sample_token (include/cudalm/sampling.h:200-234) for B rows on the device, over
// the candidate lists lm_head_int4_topk_bf16 returned; rng_state holds one
// SplitMix64 state per row (device memory) and advances by one draw per row.
inline void sample_tokens_topk(const std::int32_t* topk_idx, const __nv_bfloat16* topk_val,
                               int list_len, int B, float temperature, int top_k, float top_p,
                               std::uint64_t* rng_state, std::int32_t* tokens,
                               cudaStream_t stream) {
  b200_detail::check(cudalm_b200_sample_topk(topk_idx, b200_detail::u16(topk_val), list_len, B,
                                             temperature, top_k, top_p, rng_state, tokens, stream),
                     "sample_tokens_topk");
}

}  // namespace kernels
}  // namespace cudalm
