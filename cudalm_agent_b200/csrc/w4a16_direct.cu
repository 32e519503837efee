// Lean W4A16 kernel for single calls of a few megabytes with up to 8 activation
// rows: the form in which a decode step calls cudalm::int4_gemv_bf16 (one
// projection per launch, each depending on the one before).
//
// Such a call moves 0.3 - 3 MB, i.e. well under a microsecond of HBM time, so
// what the caller sees is the kernel's fixed cost.  This kernel has none of the
// streaming kernel's set-up: no dynamic shared memory, no mbarriers, no tensor
// maps, no activation staging and a single CTA-wide barrier.  Every warp loads
// its bytes straight from global memory into registers with 128-bit loads:
//
//   * a CTA of 8 warps works on m-tiles of 16 weight rows; the K dimension of an
//     m-tile is split over the warps (a warp takes `gps` consecutive quantisation
//     groups), so a 1024-wide projection has one 16-row m-tile per CTA and one
//     group per warp: every byte of a 6144 x 1024 matrix is requested within the
//     first few hundred cycles of the launch;
//   * lane (r8, t) = (lane / 4, lane % 4) loads, per group, the 16 bytes
//     [64 g + 16 t, +16) of rows r8 and r8 + 8, and the 32 activations
//     k = 128 g + 32 t ... of activation row r8 (through L1: the vector is shared
//     by every warp of the SM);
//   * the 4-bit values become exact bf16 integers (one LOP3 and one packed
//     subtraction per two values) and go through mma.sync m16n8k16 with the 16
//     weight rows as the A operand and the activation rows as the 8 columns, eight
//     MMAs per group, then acc += scale * group_sum in fp32.  Products are exact,
//     sums are fp32, activations are used as they are (any finite or non-finite
//     value), and a group of zero nibbles contributes an exact zero;
//   * the warps' partial sums meet in 4 KB of shared memory and are added in the
//     fixed order of the K splits, so results do not depend on timing.
//
// The MLP epilogues of the streaming kernel are available here too: a pair
// (out = silu(gate x) * (up x): every warp works on its K split of both matrices,
// so the sums are those of two separate calls) and a residual (out = residual + W x).
//
// Weights are requested before griddepcontrol.wait (they are constants of the
// model); activations, residual and outputs are touched only after it.
#include <atomic>
#include <cstring>

#include "common.cuh"

namespace cb200 {

constexpr int kDirectWarps = 8;
constexpr int kDirectThreads = kDirectWarps * 32;
constexpr int kDirectBatch = 4;     // groups whose weights a lane holds in registers at once
constexpr int kDirectMaxRows = 8;   // activation rows (the 8 columns of the MMA)

enum : int { kDirectPlain = 0, kDirectPair = 1, kDirectResidual = 2 };

struct DirectDesc {
  const std::uint8_t* W;
  const std::uint8_t* W2;     // pair: the up matrix
  const std::uint16_t* S;
  const std::uint16_t* S2;
  const std::uint16_t* x;
  const std::uint16_t* res;   // residual [M][N]
  std::uint16_t* y;
  int N, K, M;
  int cta_begin;       // first CTA of this projection in the launch
  int gps;             // quantisation groups per K split
  int nsplit;          // K splits per matrix
  int tiles_per_cta;   // m-tiles per CTA
  int mode;
};

struct DirectParams {
  DirectDesc d[CUDALM_B200_MAX_INLINE_LINEARS];
  int n_desc;
};

// Largest number of weight bytes (all projections of a call together) that takes
// this kernel; larger calls stream through the persistent kernel.
std::atomic<long long> g_direct_max_bytes{8ll << 20};

namespace {

__device__ __forceinline__ uint4 ldg_weights(const std::uint8_t* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// ordered after griddepcontrol.wait (both are volatile)
__device__ __forceinline__ uint4 ldg_activations(const std::uint16_t* p) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Eight nibbles of a word -> four exact bf16 pairs {q(i), q(i + 4)}, i = 0..3.
__device__ __forceinline__ void dequant_pairs(std::uint32_t w, std::uint32_t (&out)[4]) {
  constexpr std::uint32_t kMagic = 0x43084308u;  // {136, 136}: 128 + (nibble ^ 8) - 136 = q
#pragma unroll
  for (int i = 0; i < 4; ++i)
    out[i] = sub_bf16x2(lop3_and_xor(w >> (4 * i), 0x000F000Fu, kMagic), kMagic);
}

// One quantisation group of rows (r8, r8 + 8): sum[0..3] = the group's four sums
// of the lane's fragment (rows r8 / r8 + 8, activation rows 2t / 2t + 1).
__device__ __forceinline__ void direct_group(const uint4& qa, const uint4& qb, const uint4 (&X)[4],
                                             float (&sum)[4]) {
  const std::uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w};
  const std::uint32_t wb[4] = {qb.x, qb.y, qb.z, qb.w};
  float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    std::uint32_t A[4], B[4];
    dequant_pairs(wa[w], A);
    dequant_pairs(wb[w], B);
    // activations k = 8 w + {0..7} of this lane's 32: pairs (i, i + 4) to match the weights
    const std::uint32_t b00 = __byte_perm(X[w].x, X[w].z, 0x5410);  // {x0, x4}
    const std::uint32_t b01 = __byte_perm(X[w].x, X[w].z, 0x7632);  // {x1, x5}
    const std::uint32_t b10 = __byte_perm(X[w].y, X[w].w, 0x5410);  // {x2, x6}
    const std::uint32_t b11 = __byte_perm(X[w].y, X[w].w, 0x7632);  // {x3, x7}
    mma_m16n8k16_bf16(c0, A[0], B[0], A[1], B[1], b00, b01);
    mma_m16n8k16_bf16(c1, A[2], B[2], A[3], B[3], b10, b11);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) sum[i] = c0[i] + c1[i];
}

__global__ void __launch_bounds__(kDirectThreads, 3)
w4a16_direct_kernel(const __grid_constant__ DirectParams p) {
  __shared__ float4 red[2][kDirectWarps][32];
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  int di = 0;
#pragma unroll
  for (int i = 1; i < CUDALM_B200_MAX_INLINE_LINEARS; ++i)
    if (i < p.n_desc && static_cast<int>(blockIdx.x) >= p.d[i].cta_begin) di = i;
  const DirectDesc& d = p.d[di];
  const int N = d.N, K = d.K, M = d.M, mode = d.mode;
  const int G = K >> 7;
  const int nsplit = d.nsplit;  // warps per m-tile
  const bool pair = mode == kDirectPair;
  const int tile_in_cta = warp / nsplit;
  const int split = warp - tile_in_cta * nsplit;
  const int tile0 = (static_cast<int>(blockIdx.x) - d.cta_begin) * d.tiles_per_cta;
  const int row0 = (tile0 + tile_in_cta) * 16;
  const bool active = tile_in_cta < d.tiles_per_cta && row0 < N;

  float acc[4] = {0.f, 0.f, 0.f, 0.f};   // the projection, or the gate matrix of a pair
  float acc2[4] = {0.f, 0.f, 0.f, 0.f};  // the up matrix of a pair
  bool waited = false;
  if (active) {
    const int r8 = lane >> 2, t = lane & 3;
    // rows past N are clamped for the loads; their sums are never stored
    const int ra = min(row0 + r8, N - 1), rb = min(row0 + r8 + 8, N - 1);
    const std::size_t wa_off = static_cast<std::size_t>(ra) * (K >> 1) + t * 16;
    const std::size_t wb_off = static_cast<std::size_t>(rb) * (K >> 1) + t * 16;
    const std::size_t sa_off = static_cast<std::size_t>(ra) * G;
    const std::size_t sb_off = static_cast<std::size_t>(rb) * G;
    const bool x_real = r8 < M;  // MMA columns past M are fed zeros
    const std::uint16_t* xr = d.x + static_cast<std::size_t>(x_real ? r8 : 0) * K + t * 32;
    const int gbeg = split * d.gps;
    const int gend = min(G, gbeg + d.gps);
    // A lane holds kDirectBatch (group, matrix) slots at a time: four groups of the one
    // matrix, or two groups of each matrix of a pair (slots 0, 1: gate; 2, 3: up).
    const int step = pair ? kDirectBatch / 2 : kDirectBatch;
    for (int g0 = gbeg; g0 < gend; g0 += step) {
      uint4 qa[kDirectBatch], qb[kDirectBatch];
      std::uint16_t sca[kDirectBatch], scb[kDirectBatch];
#pragma unroll
      for (int j = 0; j < kDirectBatch; ++j) {
        const bool second = pair && j >= kDirectBatch / 2;
        const int g = g0 + (pair ? (j & (kDirectBatch / 2 - 1)) : j);
        if (g < gend) {
          const std::uint8_t* Wm = second ? d.W2 : d.W;
          const std::uint16_t* Sm = second ? d.S2 : d.S;
          qa[j] = ldg_weights(Wm + wa_off + g * 64);
          qb[j] = ldg_weights(Wm + wb_off + g * 64);
          sca[j] = __ldg(Sm + sa_off + g);
          scb[j] = __ldg(Sm + sb_off + g);
        }
      }
      if (!waited) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        waited = true;
      }
#pragma unroll
      for (int j = 0; j < kDirectBatch; ++j) {
        const bool second = pair && j >= kDirectBatch / 2;
        const int g = g0 + (pair ? (j & (kDirectBatch / 2 - 1)) : j);
        if (g < gend) {
          uint4 X[4];
#pragma unroll
          for (int w = 0; w < 4; ++w)
            X[w] = x_real ? ldg_activations(xr + g * 128 + w * 8) : make_uint4(0u, 0u, 0u, 0u);
          float sum[4];
          direct_group(qa[j], qb[j], X, sum);
          const float s_lo = __half2float(__ushort_as_half(sca[j]));
          const float s_hi = __half2float(__ushort_as_half(scb[j]));
          if (second) {
            acc2[0] = fmaf(s_lo, sum[0], acc2[0]);
            acc2[1] = fmaf(s_lo, sum[1], acc2[1]);
            acc2[2] = fmaf(s_hi, sum[2], acc2[2]);
            acc2[3] = fmaf(s_hi, sum[3], acc2[3]);
          } else {
            acc[0] = fmaf(s_lo, sum[0], acc[0]);
            acc[1] = fmaf(s_lo, sum[1], acc[1]);
            acc[2] = fmaf(s_hi, sum[2], acc[2]);
            acc[3] = fmaf(s_hi, sum[3], acc[3]);
          }
        }
      }
    }
  }
  if (!waited) asm volatile("griddepcontrol.wait;" ::: "memory");

  red[0][warp][lane] = make_float4(acc[0], acc[1], acc[2], acc[3]);
  if (pair) red[1][warp][lane] = make_float4(acc2[0], acc2[1], acc2[2], acc2[3]);
  __syncthreads();

  // Outputs of the CTA's m-tiles: (row r, activation row c) of a tile sits in lane
  // (r % 8) * 4 + c / 2, element (r / 8) * 2 + c % 2 of each of the tile's warps.
  const int n_out = d.tiles_per_cta * 128;
  for (int idx = tid; idx < n_out; idx += kDirectThreads) {
    const int tile = idx >> 7, c = (idx >> 4) & 7, r = idx & 15;
    const int row = (tile0 + tile) * 16 + r;
    if (c >= M || row >= N) continue;
    const int src_lane = (r & 7) * 4 + (c >> 1);
    const int elem = (r >> 3) * 2 + (c & 1);
    const int w0 = tile * nsplit;
    float v = 0.f;
    for (int s = 0; s < nsplit; ++s) v += reinterpret_cast<const float*>(&red[0][w0 + s][src_lane])[elem];
    std::uint16_t o = float_to_bf16_bits(v);
    const std::size_t at = static_cast<std::size_t>(c) * N + row;
    if (pair) {
      float u = 0.f;
      for (int s = 0; s < nsplit; ++s) u += reinterpret_cast<const float*>(&red[1][w0 + s][src_lane])[elem];
      // CUDALM's rounding order (src/kernels/qwen35_kernels.cu:459-476)
      o = silu_mul_bits(bf16_bits_to_float(o), float_to_bf16_bits(u));
    } else if (mode == kDirectResidual) {
      o = add_bits(d.res[at], o);  // src/kernels/qwen35_kernels.cu:442-456
    }
    d.y[at] = o;
  }
}

}  // namespace

// True when the lean kernel takes this projection.
bool direct_eligible(const cudalm_b200_linear& l, const std::uint8_t* weight2) {
  if (l.M < 1 || l.M > kDirectMaxRows || l.N < 1 || l.K <= 0 || (l.K % 128) != 0) return false;
  if (!aligned_to(l.weight, 16) || !aligned_to(l.x, 16)) return false;
  if (weight2 && !aligned_to(weight2, 16)) return false;
  return true;
}

long long direct_weight_bytes(const cudalm_b200_linear& l, bool pair) {
  return static_cast<long long>(l.N) * (l.K / 2) * (pair ? 2 : 1);
}

// One launch over up to CUDALM_B200_MAX_INLINE_LINEARS projections.  `weight2` /
// `scales2` / `residual` (arrays of `count`, or null) select the pair and residual
// epilogues per projection.
int run_direct(const cudalm_b200_linear* ls, int count, const std::uint8_t* const* weight2,
               const std::uint16_t* const* scales2, const std::uint16_t* const* residual,
               cudaStream_t stream) {
  if (count < 1 || count > CUDALM_B200_MAX_INLINE_LINEARS) return CUDALM_B200_ERR_BAD_SHAPE;
  DirectParams p;
  std::memset(&p, 0, sizeof(p));
  long long ctas = 0;
  for (int i = 0; i < count; ++i) {
    const cudalm_b200_linear& l = ls[i];
    DirectDesc& d = p.d[i];
    d.W = l.weight;
    d.S = l.scales;
    d.x = l.x;
    d.y = l.y;
    d.N = l.N;
    d.K = l.K;
    d.M = l.M;
    d.mode = kDirectPlain;
    if (weight2 && weight2[i]) {
      d.W2 = weight2[i];
      d.S2 = scales2[i];
      d.mode = kDirectPair;
    } else if (residual && residual[i]) {
      d.res = residual[i];
      d.mode = kDirectResidual;
    }
    const int G = l.K >> 7;
    // K is cut the same way with and without a second matrix, so that the fused pair
    // sums in exactly the order of two separate calls
    d.gps = (G + kDirectWarps - 1) / kDirectWarps;
    d.nsplit = (G + d.gps - 1) / d.gps;
    d.tiles_per_cta = kDirectWarps / d.nsplit;
    const int mtiles = (l.N + 15) / 16;
    d.cta_begin = static_cast<int>(ctas);
    ctas += (mtiles + d.tiles_per_cta - 1) / d.tiles_per_cta;
    if (ctas > 0x7fffffff) return CUDALM_B200_ERR_TOO_LARGE;
  }
  p.n_desc = count;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(ctas));
  cfg.blockDim = dim3(kDirectThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t le = cudaLaunchKernelEx(&cfg, w4a16_direct_kernel, p);
  if (le != cudaSuccess) {
    g_last_cuda_error = static_cast<int>(le);
    (void)cudaGetLastError();
    return CUDALM_B200_ERR_CUDA;
  }
  return check_launch();
}

int direct_kernel_regs() {
  cudaFuncAttributes attr;
  if (cudaFuncGetAttributes(&attr, reinterpret_cast<const void*>(&w4a16_direct_kernel)) != cudaSuccess) {
    (void)cudaGetLastError();
    return -1;
  }
  return attr.numRegs;
}

}  // namespace cb200
