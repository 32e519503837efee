// Token sampling on the device over the candidate lists the vocabulary
// projection returns: CUDALM's sample_token (include/cudalm/sampling.h:131-234)
// for configurations with 1 <= top_k <= list length, where every token outside
// the first top_k candidates has probability zero.  One thread per row; a row is
// at most 64 candidates, so the work is tiny, and what matters is that only a
// token id crosses PCIe instead of 497 KB of logits per row
// (src/runtime/scheduler.cpp:59-108).
//
// The arithmetic follows the reference operation for operation: logit / T, exp
// and all sums in double; top-p accumulates in candidate order (value
// descending, tie -> lower id); the normalising sum and the cumulative walk run
// in ascending token id; probabilities are rounded to float before the walk;
// one SplitMix64 draw per sampled row, none on the greedy path.
#include "common.cuh"

namespace cb200 {
namespace {

constexpr int kMaxSampleK = 64;

__global__ void __launch_bounds__(64)
sample_topk_kernel(const std::int32_t* __restrict__ topk_idx, const std::uint16_t* __restrict__ topk_val,
                   int list_len, int M, float temperature, int top_k, float top_p,
                   unsigned long long* __restrict__ rng_state, std::int32_t* __restrict__ token_out) {
  // the lists may come from a kernel launched just before
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int m = blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= M) return;
  const std::int32_t* idx = topk_idx + static_cast<std::size_t>(m) * list_len;
  const std::uint16_t* val = topk_val + static_cast<std::size_t>(m) * list_len;
  if (!(temperature > 0.0f)) {  // greedy: the argmax, no draw
    token_out[m] = idx[0];
    return;
  }
  const int k = top_k;
  double f[kMaxSampleK];
  int ids[kMaxSampleK], order[kMaxSampleK];
  for (int i = 0; i < k; ++i) {
    f[i] = static_cast<double>(bf16_bits_to_float(val[i])) / static_cast<double>(temperature);
    ids[i] = idx[i];
  }
  const double max_f = f[0];
  int kept = k;
  if (top_p < 1.0f) {
    double total = 0.0;
    for (int i = 0; i < k; ++i) total += exp(f[i] - max_f);
    double cum = 0.0;
    int cut = k - 1;
    for (int j = 0; j < k; ++j) {
      cum += exp(f[j] - max_f);
      if (cum >= static_cast<double>(top_p) * total || j + 1 == k) {
        cut = j;
        break;
      }
    }
    kept = cut + 1;
  }
  // ascending token id over the kept candidates
  for (int i = 0; i < kept; ++i) order[i] = i;
  for (int i = 1; i < kept; ++i) {
    const int o = order[i];
    int j = i - 1;
    while (j >= 0 && ids[order[j]] > ids[o]) {
      order[j + 1] = order[j];
      --j;
    }
    order[j + 1] = o;
  }
  double norm = 0.0;
  for (int i = 0; i < kept; ++i) norm += exp(f[order[i]] - max_f);
  // SplitMix64 (include/cudalm/sampling.h:99-116)
  unsigned long long z = (rng_state[m] += 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z = z ^ (z >> 31);
  const double u = static_cast<double>(z >> 11) * 0x1.0p-53;
  double cum = 0.0;
  int last_kept = -1, token = -1;
  for (int i = 0; i < kept && token < 0; ++i) {
    const float p = static_cast<float>(exp(f[order[i]] - max_f) / norm);
    if (p > 0.0f) {
      cum += static_cast<double>(p);
      last_kept = ids[order[i]];
      if (u < cum) token = last_kept;
    }
  }
  token_out[m] = token >= 0 ? token : (last_kept >= 0 ? last_kept : idx[0]);
}

}  // namespace
}  // namespace cb200

extern "C" int cudalm_b200_sample_topk(const int32_t* topk_idx, const uint16_t* topk_val,
                                       int list_len, int M, float temperature, int top_k,
                                       float top_p, uint64_t* rng_state, int32_t* token_out,
                                       void* stream) {
  using namespace cb200;
  if (!topk_idx || !topk_val || !token_out) return CUDALM_B200_ERR_NULL;
  if (list_len < 1 || M < 1) return CUDALM_B200_ERR_BAD_SHAPE;
  // the reference's validation (include/cudalm/sampling.h:73-91): values it rejects
  if (temperature != temperature || temperature - temperature != 0.0f) return CUDALM_B200_ERR_BAD_SHAPE;
  if (top_k < 0 || !(top_p > 0.0f) || top_p > 1.0f) return CUDALM_B200_ERR_BAD_SHAPE;
  const bool greedy = !(temperature > 0.0f);
  if (!greedy) {
    if (!rng_state) return CUDALM_B200_ERR_NULL;
    // top_k = 0 (or beyond the list) lets tokens outside the list keep a
    // non-zero probability: that needs the whole row of logits
    if (top_k < 1 || top_k > list_len) return CUDALM_B200_ERR_UNSUPPORTED;
    if (top_k > kMaxSampleK) return CUDALM_B200_ERR_TOO_LARGE;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>((M + 63) / 64));
  cfg.blockDim = dim3(64);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t le =
      cudaLaunchKernelEx(&cfg, sample_topk_kernel, topk_idx, topk_val, list_len, M, temperature, top_k,
                         top_p, reinterpret_cast<unsigned long long*>(rng_state), token_out);
  if (le != cudaSuccess) {
    g_last_cuda_error = static_cast<int>(le);
    (void)cudaGetLastError();
    return CUDALM_B200_ERR_CUDA;
  }
  return check_launch();
}
