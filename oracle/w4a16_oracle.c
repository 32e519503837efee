/*
 * CPU oracle for the W4A16 projection path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the CPU algorithms that the CUDALM reference
 * uses to define correct results for its int4-weight x bf16-activation linear
 * projection.  It is the checker the GPU kernels are compared against.  It is
 * never linked into, imported by, or called from the shipped library: only the
 * test suite, the smoke check and the benchmark's CPU-baseline leg may use it.
 *
 * Parity pin: every function here is checked (tests/test_oracle_pins.py)
 * against golden vectors produced by the reference's own code -- the Python
 * quantizer imported from the reference tree, and the reference's C++ test
 * functions compiled from the reference sources (oracle/ref_shim.cpp).
 *
 * Data layouts (reference include/cudalm/kernels/int4_gemv_bf16.h:29-48):
 *   weight  uint8 [N, K/2] row-major; low nibble = k=2b, high nibble = k=2b+1,
 *           4-bit two's complement
 *   scales  fp16  [N, K/128] row-major (raw IEEE binary16 bits here)
 *   x       bf16  [K] or [B, K]        (raw bfloat16 bits here)
 *   y       bf16  [N] or [B, N]
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off, no fast-math: the
 * results must be the IEEE fp32 results the reference's code produces).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

/* ------------------------------------------------------------------------ */
/* Scalar type conversions (IEEE, round-to-nearest-even)                     */
/* ------------------------------------------------------------------------ */

static inline float bits_to_f32(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint32_t f32_to_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}

/* bfloat16 is the upper half of an fp32. */
float orc_bf16_to_f32(uint16_t h) { return bits_to_f32((uint32_t)h << 16); }

/* fp32 -> bf16, round to nearest even (what __float2bfloat16_rn does). */
uint16_t orc_f32_to_bf16(float f) {
  uint32_t u = f32_to_bits(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fffu; /* NaN */
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

/* binary16 -> fp32 (exact). */
float orc_f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  if (exp == 0) {
    if (man == 0) return bits_to_f32(sign);
    /* subnormal: value = man * 2^-24 */
    float v = (float)man * 5.9604644775390625e-8f;
    return (sign ? -v : v);
  }
  if (exp == 31) return bits_to_f32(sign | 0x7f800000u | (man << 13));
  return bits_to_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

/* fp32 -> binary16, round to nearest even (what torch .to(float16) and
 * __float2half_rn do). */
uint16_t orc_f32_to_f16(float f) {
  uint32_t u = f32_to_bits(f);
  uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
  uint32_t a = u & 0x7fffffffu;
  if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u); /* NaN */
  if (a >= 0x477ff000u) {
    /* >= 65520 rounds to inf (65504 + half ulp); includes inf */
    return (uint16_t)(sign | 0x7c00u);
  }
  if (a < 0x33000001u) {
    /* <= 2^-25 rounds to zero (exactly 2^-25 ties to even = 0) */
    return sign;
  }
  int32_t e = (int32_t)(a >> 23) - 127;
  uint32_t m = (a & 0x7fffffu) | 0x800000u; /* 24-bit significand */
  uint32_t shift;
  uint32_t hexp;
  if (e < -14) {
    /* subnormal result: value = m * 2^(e-23); target unit 2^-24 */
    shift = (uint32_t)(13 + (-14 - e));
    hexp = 0;
  } else {
    shift = 13;
    hexp = (uint32_t)(e + 15);
  }
  uint32_t q = m >> shift;
  uint32_t rem = m & ((1u << shift) - 1u);
  uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) q++;
  uint32_t out;
  if (hexp == 0) {
    out = q; /* may carry into exponent 1: correct encoding */
  } else {
    out = ((hexp - 1) << 10) + q; /* q includes the implicit 1 (bit 10) */
  }
  return (uint16_t)(sign | out);
}

/* ------------------------------------------------------------------------ */
/* int4 nibble helpers (reference include/cudalm/weight_loader.h:102-119)    */
/* ------------------------------------------------------------------------ */

int orc_unpack_lo(uint8_t b) { return (int)(int8_t)((b & 0x0Fu) << 4) >> 4; }
int orc_unpack_hi(uint8_t b) { return (int)(int8_t)b >> 4; }
uint8_t orc_pack_byte(int lo, int hi) {
  return (uint8_t)(((hi & 0xF) << 4) | (lo & 0xF));
}

/* ------------------------------------------------------------------------ */
/* Minimal parallel-for over [0, n) in fixed chunks (pthreads).  Each index  */
/* is computed by exactly one thread with the single-thread arithmetic, so   */
/* results do not depend on the thread count.                                */
/* ------------------------------------------------------------------------ */
typedef void (*orc_range_fn)(void* ctx, long i0, long i1);
typedef struct {
  orc_range_fn fn;
  void* ctx;
  long n, chunk;
  long next; /* guarded by mu */
  pthread_mutex_t mu;
} orc_pf;

static void* orc_pf_worker(void* p) {
  orc_pf* pf = (orc_pf*)p;
  for (;;) {
    pthread_mutex_lock(&pf->mu);
    long i0 = pf->next;
    pf->next += pf->chunk;
    pthread_mutex_unlock(&pf->mu);
    if (i0 >= pf->n) break;
    long i1 = i0 + pf->chunk < pf->n ? i0 + pf->chunk : pf->n;
    pf->fn(pf->ctx, i0, i1);
  }
  return NULL;
}

static void orc_parallel_for(long n, long chunk, int threads, orc_range_fn fn,
                             void* ctx) {
  orc_pf pf = {fn, ctx, n, chunk, 0, PTHREAD_MUTEX_INITIALIZER};
  if (threads <= 1) {
    fn(ctx, 0, n);
    return;
  }
  if (threads > 256) threads = 256;
  pthread_t tid[256];
  int started = 0;
  for (int t = 0; t < threads - 1; ++t)
    if (pthread_create(&tid[started], NULL, orc_pf_worker, &pf) == 0) ++started;
  orc_pf_worker(&pf);
  for (int t = 0; t < started; ++t) pthread_join(tid[t], NULL);
}

int orc_max_threads(void) {
  long n = sysconf(_SC_NPROCESSORS_ONLN);
  return n < 1 ? 1 : (int)n;
}

/* ------------------------------------------------------------------------ */
/* W4A16 GEMV (reference tests/cuda/test_int4_gemv_bf16.cpp:54-69)           */
/*                                                                          */
/* Term order is the reference's: for each byte b ascending,                 */
/*   acc += lo * s * x[2b];  acc += hi * s * x[2b+1]                         */
/* with every product evaluated left to right in fp32, s = scales[b >> 6],   */
/* and ONE bf16 round-to-nearest-even at the store.                          */
/* ------------------------------------------------------------------------ */

static void gemv_rows(const uint8_t* W, const uint16_t* S, const float* xf,
                      int n0, int n1, int K, uint16_t* y, float* acc_out) {
  const int half_k = K / 2;
  const int groups = K / 128;
  for (int n = n0; n < n1; ++n) {
    const uint8_t* wrow = W + (size_t)n * half_k;
    const uint16_t* srow = S + (size_t)n * groups;
    float acc = 0.f;
    for (int b = 0; b < half_k; ++b) {
      const float s = orc_f16_to_f32(srow[b >> 6]);
      const float lo = (float)orc_unpack_lo(wrow[b]);
      const float hi = (float)orc_unpack_hi(wrow[b]);
      acc += lo * s * xf[2 * b];
      acc += hi * s * xf[2 * b + 1];
    }
    y[n] = orc_f32_to_bf16(acc);
    if (acc_out) acc_out[n] = acc;
  }
}

/* Single thread, exactly as written in the reference. acc_out (optional,
 * may be NULL) receives the fp32 value before the bf16 round. */
int orc_gemv_bf16(const uint8_t* W, const uint16_t* S, const uint16_t* x,
                  int N, int K, uint16_t* y, float* acc_out) {
  if (N < 1 || K <= 0 || K % 128 != 0) return 1;
  float* xf = (float*)malloc(sizeof(float) * (size_t)K);
  if (!xf) return 2;
  for (int k = 0; k < K; ++k) xf[k] = orc_bf16_to_f32(x[k]);
  gemv_rows(W, S, xf, 0, N, K, y, acc_out);
  free(xf);
  return 0;
}

/* Batched form: row b of x against the same weights; y is [B, N]
 * (reference src/kernels/batch_decode.cu:95-190: x offset b*K, y offset b*N).
 * Rows of W are split over `threads` host threads; each output keeps the
 * single-thread term order, so results are bit-identical for any `threads`. */
typedef struct {
  const uint8_t* W;
  const uint16_t* S;
  const float* xf;
  uint16_t* y;
  int N, K, B;
  long chunks_per_b;
} orc_gemv_ctx;

static void orc_gemv_range(void* p, long c0, long c1) {
  const orc_gemv_ctx* c = (const orc_gemv_ctx*)p;
  for (long i = c0; i < c1; ++i) {
    const long b = i / c->chunks_per_b;
    const long ch = i % c->chunks_per_b;
    const int n0 = (int)(ch * 64);
    const int n1 = n0 + 64 < c->N ? n0 + 64 : c->N;
    gemv_rows(c->W, c->S, c->xf + (size_t)b * c->K, n0, n1, c->K,
              c->y + (size_t)b * c->N, NULL);
  }
}

int orc_batch_gemv_bf16(const uint8_t* W, const uint16_t* S, const uint16_t* x,
                        int N, int K, int B, uint16_t* y, int threads) {
  if (N < 1 || K <= 0 || K % 128 != 0 || B < 1) return 1;
  float* xf = (float*)malloc(sizeof(float) * (size_t)K * (size_t)B);
  if (!xf) return 2;
  for (size_t i = 0; i < (size_t)K * (size_t)B; ++i)
    xf[i] = orc_bf16_to_f32(x[i]);
  orc_gemv_ctx c = {W, S, xf, y, N, K, B, (N + 63) / 64};
  orc_parallel_for(c.chunks_per_b * B, 1, threads, orc_gemv_range, &c);
  free(xf);
  return 0;
}

/* ------------------------------------------------------------------------ */
/* Quantize + pack (reference tools/common/w4a16_quant.py:25-60)             */
/*                                                                          */
/*   Wg      = float(W) viewed [N, K/128, 128]                               */
/*   amax    = max |Wg| per group                 (fp32)                     */
/*   scale32 = amax / 7                           (fp32 divide)              */
/*   zero    = scale32 == 0                                                  */
/*   q       = round_half_even(Wg / (zero ? 1 : scale32))   (fp32 divide)    */
/*   q       = clamp(q, -7, 7); zero group -> q = 0                          */
/*   byte    = ((hi & 15) << 4) | (lo & 15)                                  */
/*   scale16 = fp16_rn(scale32)                                              */
/* Input is bf16 (raw bits), finite.                                         */
/* ------------------------------------------------------------------------ */
typedef struct {
  const uint16_t* W;
  uint8_t* packed;
  uint16_t* scale16;
  int N, K;
} orc_quant_ctx;

static void orc_quant_range(void* p, long n0, long n1) {
  const orc_quant_ctx* c = (const orc_quant_ctx*)p;
  const int K = c->K;
  const int groups = K / 128;
  for (long n = n0; n < n1; ++n) {
    for (int g = 0; g < groups; ++g) {
      const uint16_t* w = c->W + (size_t)n * K + (size_t)g * 128;
      float amax = 0.f;
      for (int i = 0; i < 128; ++i) {
        float a = fabsf(orc_bf16_to_f32(w[i]));
        if (a > amax) amax = a;
      }
      volatile float scale32 = amax / 7.0f;
      const int zero = (scale32 == 0.f);
      const float safe = zero ? 1.0f : scale32;
      int q[128];
      for (int i = 0; i < 128; ++i) {
        volatile float r = orc_bf16_to_f32(w[i]) / safe;
        float rq = nearbyintf(r); /* default rounding mode: half to even */
        if (rq > 7.f) rq = 7.f;
        if (rq < -7.f) rq = -7.f;
        q[i] = zero ? 0 : (int)rq;
      }
      uint8_t* out = c->packed + (size_t)n * (K / 2) + (size_t)g * 64;
      for (int i = 0; i < 64; ++i) out[i] = orc_pack_byte(q[2 * i], q[2 * i + 1]);
      c->scale16[(size_t)n * groups + g] = orc_f32_to_f16(scale32);
    }
  }
}

int orc_quantize_w4a16(const uint16_t* W, int N, int K, uint8_t* packed,
                       uint16_t* scale16, int threads) {
  if (N < 1 || K <= 0 || K % 128 != 0) return 1;
  orc_quant_ctx c = {W, packed, scale16, N, K};
  orc_parallel_for(N, 64, threads, orc_quant_range, &c);
  return 0;
}

/* ------------------------------------------------------------------------ */
/* Token pick                                                               */
/* ------------------------------------------------------------------------ */

/* Greedy argmax over bf16 logits (reference include/cudalm/greedy.h:28-39):
 * compares float values with strict '>', so an exact tie keeps the lowest
 * index (and -0 ties with +0). */
int orc_argmax_bf16(const uint16_t* logits, int n) {
  int best = 0;
  float best_val = orc_bf16_to_f32(logits[0]);
  for (int i = 1; i < n; ++i) {
    const float v = orc_bf16_to_f32(logits[i]);
    if (v > best_val) {
      best = i;
      best_val = v;
    }
  }
  return best;
}

/* Top-k order of the reference sampler (include/cudalm/sampling.h:152-166):
 * value descending, tie -> lower id; keep the first k; k > n clamps to n.
 * The reference compares logit/T in double for T > 0, which preserves the
 * order of the bf16 values, so the float compare here selects the same ids
 * in the same order.  Returns the number of entries written (min(k, n)).
 * idx_out/val_out (bf16 bits) are in selection order; element 0 is the
 * argmax. Simple O(n*k) insertion; the oracle favours clarity over speed. */
int orc_topk_bf16(const uint16_t* logits, int n, int k, int32_t* idx_out,
                  uint16_t* val_out) {
  if (n < 1 || k < 1) return 0;
  if (k > n) k = n;
  int filled = 0;
  for (int i = 0; i < n; ++i) {
    const float v = orc_bf16_to_f32(logits[i]);
    /* position after every kept entry that is >= v (ids ascend, so an equal
     * value already kept has a lower id and stays ahead) */
    if (filled == k && !(v > orc_bf16_to_f32(val_out[k - 1]))) continue;
    int pos = filled < k ? filled : k - 1;
    while (pos > 0 && v > orc_bf16_to_f32(val_out[pos - 1])) {
      if (pos < k) {
        idx_out[pos] = idx_out[pos - 1];
        val_out[pos] = val_out[pos - 1];
      }
      --pos;
    }
    idx_out[pos] = i;
    val_out[pos] = logits[i];
    if (filled < k) ++filled;
  }
  return filled;
}

/* ------------------------------------------------------------------------ */
/* MLP elementwise steps either side of the projections                      */
/* (reference src/kernels/qwen35_kernels.cu:442-476)                         */
/* ------------------------------------------------------------------------ */

/* y = bf16( float(bf16( g / (1 + exp(-g)) )) * float(u) ) */
/* sample_token (CUDALM include/cudalm/sampling.h:131-234) restated on a
 * candidate list: the first `list_len` tokens of the row in the reference's
 * order (logit descending, tie -> lower id), as the vocabulary projection
 * returns them.  Needs 1 <= top_k <= list_len: then the top-k survivors are the
 * first top_k entries, the row maximum is entry 0, and nothing outside the list
 * can have a non-zero probability.  temperature <= 0 is the greedy path: entry
 * 0, no draw.  Arithmetic as in the reference: logit / T, exp and the sums in
 * double; top-p accumulates in list order; the normalising sum and the
 * cumulative walk run in ascending token id; probabilities are rounded to
 * float before the walk.  *state is the SplitMix64 state (:99-116).
 * Returns the token id, or -1 when the arguments are outside that domain. */
int orc_sample_from_topk(const int32_t* idx, const uint16_t* val, int list_len, float temperature,
                         int top_k, float top_p, uint64_t* state) {
  if (list_len < 1) return -1;
  if (!(temperature > 0.0f)) return idx[0];
  if (top_k < 1 || top_k > list_len || top_k > 64) return -1;
  double f[64];
  int ids[64], order[64];
  const int k = top_k;
  for (int i = 0; i < k; ++i) {
    f[i] = (double)orc_bf16_to_f32(val[i]) / (double)temperature;
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
      if (cum >= (double)top_p * total || j + 1 == k) {
        cut = j;
        break;
      }
    }
    kept = cut + 1;
  }
  /* ascending token id over the kept entries */
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
  uint64_t z = (*state += 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z = z ^ (z >> 31);
  const double u = (double)(z >> 11) * 0x1.0p-53;
  double cum = 0.0;
  int last_kept = -1;
  for (int i = 0; i < kept; ++i) {
    const float p = (float)(exp(f[order[i]] - max_f) / norm);
    if (p > 0.0f) {
      cum += (double)p;
      last_kept = ids[order[i]];
      if (u < cum) return last_kept;
    }
  }
  return last_kept >= 0 ? last_kept : idx[0];
}

void orc_silu_mul_bf16(const uint16_t* gate, const uint16_t* up, uint16_t* y,
                       size_t n) {
  for (size_t i = 0; i < n; ++i) {
    const float g = orc_bf16_to_f32(gate[i]);
    const uint16_t s = orc_f32_to_bf16(g / (1.0f + expf(-g)));
    y[i] = orc_f32_to_bf16(orc_bf16_to_f32(s) * orc_bf16_to_f32(up[i]));
  }
}

/* y = bf16( float(a) + float(b) ) */
void orc_add_bf16(const uint16_t* a, const uint16_t* b, uint16_t* y, size_t n) {
  for (size_t i = 0; i < n; ++i)
    y[i] = orc_f32_to_bf16(orc_bf16_to_f32(a[i]) + orc_bf16_to_f32(b[i]));
}
