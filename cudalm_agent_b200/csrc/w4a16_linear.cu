// W4A16 linear projections: M = 1 GEMV, batched rows, several projections per
// launch, fused gate+up.  Host entry points of the C ABI plus the streaming
// kernel they launch.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <algorithm>
#include <vector>

#include "w4a16_stream.cuh"

namespace cb200 {

// tensor-memory path for batched rows (w4a16_tc.cu)
bool tc_eligible(const cudalm_b200_linear& l);
int run_tc(const cudalm_b200_linear* ls, int count, cudaStream_t stream);
int run_tc_with_pick(const cudalm_b200_linear& l, const PickTail& pick, cudaStream_t stream, int* grid_out);
int run_tc_extra(const cudalm_b200_linear& l, const std::uint8_t* weight2,
                 const std::uint16_t* scales2, const std::uint16_t* residual, cudaStream_t stream);
struct TcGroup;
int tc_group_create(const cudalm_b200_linear* ls, int count, TcGroup** out);
int tc_group_run(const TcGroup* g, cudaStream_t stream);
void tc_group_destroy(TcGroup* g);
// Smallest M that takes the tensor-memory kernel (runtime knob; see
// cudalm_b200_set_tensor_path_min_rows).
std::atomic<int> g_tc_min_rows{17};
// lean kernel for single calls of a few megabytes (w4a16_direct.cu)
bool direct_eligible(const cudalm_b200_linear& l, const std::uint8_t* weight2);
long long direct_weight_bytes(const cudalm_b200_linear& l, bool pair);
int run_direct(const cudalm_b200_linear* ls, int count, const std::uint8_t* const* weight2,
               const std::uint16_t* const* scales2, const std::uint16_t* const* residual,
               cudaStream_t stream);
int direct_kernel_regs();
extern std::atomic<long long> g_direct_max_bytes;

// ---------------------------------------------------------------------------
// Fallback for inputs the streaming kernel does not take: a weight base that is
// not 16-byte aligned (CUDALM src/kernels/int4_gemv_bf16.cu:174-213 keeps such
// calls legal) or K above the staged limit.  One warp per output row, byte
// loads, fp32 accumulation in a fixed order.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float fallback_row_dot(const std::uint8_t* wrow, const std::uint16_t* srow,
                                                  const std::uint16_t* xm, int K, int lane) {
  float acc = 0.f;
  for (int g = 0; g < (K >> 7); ++g) {
    const float s = __half2float(__ushort_as_half(srow[g]));
    float part = 0.f;
    for (int b = lane; b < 64; b += 32) {
      const std::uint8_t byte = wrow[g * 64 + b];
      const int lo = static_cast<int>(static_cast<std::int8_t>((byte & 0x0Fu) << 4)) >> 4;
      const int hi = static_cast<int>(static_cast<std::int8_t>(byte)) >> 4;
      const int k = g * 128 + 2 * b;
      part = fmaf(static_cast<float>(lo), bf16_bits_to_float(xm[k]), part);
      part = fmaf(static_cast<float>(hi), bf16_bits_to_float(xm[k + 1]), part);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
    acc = fmaf(s, part, acc);
  }
  return acc;
}

// W2/S2 non-null: y = silu(W x) * (W2 x); res non-null: y = res + W x (CUDALM's
// rounding order, see silu_mul_bits / add_bits).
__global__ void __launch_bounds__(256)
w4a16_fallback_kernel(const std::uint8_t* __restrict__ W, const std::uint16_t* __restrict__ S,
                      const std::uint16_t* __restrict__ x, std::uint16_t* __restrict__ y, int N,
                      int K, int M, const std::uint8_t* __restrict__ W2 = nullptr,
                      const std::uint16_t* __restrict__ S2 = nullptr,
                      const std::uint16_t* __restrict__ res = nullptr) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= N) return;
  for (int m = 0; m < M; ++m) {
    const std::uint16_t* xm = x + static_cast<std::size_t>(m) * K;
    std::uint16_t o = float_to_bf16_bits(fallback_row_dot(W + row * (K >> 1), S + row * (K >> 7), xm, K, lane));
    if (W2) {
      const std::uint16_t u = float_to_bf16_bits(
          fallback_row_dot(W2 + row * (K >> 1), S2 + row * (K >> 7), xm, K, lane));
      o = silu_mul_bits(bf16_bits_to_float(o), u);
    } else if (res) {
      o = add_bits(res[static_cast<std::size_t>(m) * N + row], o);
    }
    if (lane == 0) y[static_cast<std::size_t>(m) * N + row] = o;
  }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
namespace {

#ifndef CB200_CG
#define CB200_CG 8  // measured on B200: 8 groups (8 KB) per chunk beats 4 and 2
#endif
constexpr int kCG = CB200_CG;        // groups per chunk (CG * 128 values of k)
constexpr int kRS = kCG * 64;        // stage row stride
constexpr int kMaxStreamK = 4096;    // largest K the staged path takes

inline int round_up(int v, int a) { return (v + a - 1) / a * a; }

struct Plan {
  int nt;       // MMA column tiles: activations rows per pass = 8 * nt
  int nwarps;   // consumer warps: 12 or 8
  int depth;
  int stage_bytes;
  int x_bytes;
  int x_buffers;
  int smem_bytes;
};

// Chooses the kernel shape for the largest K and M of a launch.  Returns false
// when even 8 rows of activations do not fit beside the rings.
bool make_plan(int kmax, int mmax, Plan* out, bool several = false) {
  const int stage = kMTileRows * kRS + round_up(kmax / 4, 128);
  int nt = 1;
  while (nt * 8 < mmax && nt < 8) nt *= 2;
  // at least 4 KB: the region doubles as reduction scratch at the kernel's end
  // activations, + the all-zero row, + the per-group offset sums [K/128][8*nt]
  // ... + the out-of-range flag word in the buffer's last bytes
  int x_bytes = round_up((mmax + 1) * (2 * kmax + kXRowPad) + (kmax / 128) * nt * 8 * 4, 128) + kXFlagBytes;
  if (x_bytes < 4096) x_bytes = 4096;
#ifdef CB200_WARPS
  for (int nwarps : {CB200_WARPS}) {
#else
  for (int nwarps : {12, 8}) {
#endif
    if (nt == 8 && nwarps != 8) continue;  // 32 accumulators per lane need the larger register budget
    // a launch of several projections with few rows keeps two activation
    // buffers, so that a change of projection needs no CTA-wide barrier
    int x_buffers = (several && static_cast<long long>(mmax) * kmax <= kAsyncFillMaxValues) ? 2 : 1;
    const int staging = kAsyncFillMaxValues * 2;  // raw activations on their way in
    if (kMaxSmemBytes - kHeaderBytes - 2 * x_bytes - staging < 2 * nwarps * stage) x_buffers = 1;
    const int fixed = kHeaderBytes + x_buffers * x_bytes + (x_buffers == 2 ? staging : 0);
    const int avail = kMaxSmemBytes - fixed;
    if (avail < 2 * nwarps * stage) continue;
    int depth = avail / (nwarps * stage);
    if (depth > kMaxDepth) depth = kMaxDepth;
    *out = Plan{nt, nwarps, depth, stage, x_bytes, x_buffers, fixed + nwarps * depth * stage};
    return true;
  }
  return false;
}

// Largest number of activation rows one pass can take for this K.
int max_rows_per_pass(int k) {
  int best = 0;
  for (int m : {8, 16, 32, 64}) {
    Plan pl;
    if (make_plan(k, m, &pl)) best = m;
  }
  return best;
}

#ifndef CB200_PRODUCERS
#define CB200_PRODUCERS 1  // producer warps for the 8-consumer form
#endif

template <int NT, int NWARPS, bool CTA_MAX, bool EXTRA = false>
int launch_instance(const StreamParams& p, const Plan& pl, int grid, cudaStream_t stream) {
  // producer warps need registers: only the 8-consumer form has room for them
  constexpr int kProd = (CB200_PRODUCERS && NWARPS == 8) ? NWARPS / 4 : 0;
  auto kern = w4a16_stream_kernel<NT, kCG, NWARPS, CTA_MAX, kProd, EXTRA>;
  // the attribute is per device; set it on every device this process uses
  static std::mutex mu;
  static std::vector<int> done_devices;
  int dev = 0;
  CB200_CUDA_TRY(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lk(mu);
    bool done = false;
    for (int d : done_devices) done |= (d == dev);
    if (!done) {
      const cudaError_t attr_err = cudaFuncSetAttribute(
          kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmemBytes);
      if (attr_err != cudaSuccess) {
        g_last_cuda_error = static_cast<int>(attr_err);
        return CUDALM_B200_ERR_CUDA;
      }
      done_devices.push_back(dev);
    }
  }
  // Programmatic dependent launch: the next kernel in the stream may start its
  // CTAs while this one drains.  Only kernels that execute
  // griddepcontrol.launch_dependents let their successor start early, and the
  // streaming kernel touches nothing an earlier kernel may have written
  // (activations, outputs) before its griddepcontrol.wait.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3((NWARPS + kProd) * 32);
  cfg.dynamicSmemBytes = static_cast<size_t>(pl.smem_bytes);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t le = cudaLaunchKernelEx(&cfg, kern, p);
  if (le != cudaSuccess) {
    g_last_cuda_error = static_cast<int>(le);
    (void)cudaGetLastError();
    return CUDALM_B200_ERR_CUDA;
  }
  return check_launch();
}

int launch_stream(StreamParams& p, int kmax, int mmax, cudaStream_t stream,
                  int* grid_out = nullptr, int forced_grid = 0, bool extra = false) {
  Plan pl;
  if (!make_plan(kmax, mmax, &pl, p.n_desc > 1)) return CUDALM_B200_ERR_UNSUPPORTED;
  p.depth = pl.depth;
  p.stage_bytes = pl.stage_bytes;
  p.x_bytes = pl.x_bytes;
  p.x_buffers = pl.x_buffers;
  p.status = device_status_word();
  if (p.status == nullptr) return CUDALM_B200_ERR_CUDA;
  int grid = num_sms();
  if (grid > p.total_mt) grid = p.total_mt;
  if (grid < 1) grid = 1;
  if (forced_grid > 0) grid = forced_grid;  // a group's per-CTA ranges were cut for this grid
  const bool want_max = p.pick.slots != nullptr;
  if (want_max && grid > kTailMaxCtas) grid = kTailMaxCtas;  // one slot per CTA in the pick's table
  if (grid_out) *grid_out = grid;
  if (extra) {
    // launches with an MLP epilogue: at most 16 rows, no per-CTA maxima
    if (pl.nt == 1 && pl.nwarps == 12) return launch_instance<1, 12, false, true>(p, pl, grid, stream);
    if (pl.nt == 2 && pl.nwarps == 12) return launch_instance<2, 12, false, true>(p, pl, grid, stream);
    if (pl.nt == 1 && pl.nwarps == 8) return launch_instance<1, 8, false, true>(p, pl, grid, stream);
    if (pl.nt == 2 && pl.nwarps == 8) return launch_instance<2, 8, false, true>(p, pl, grid, stream);
    return CUDALM_B200_ERR_UNSUPPORTED;
  }
#define CB200_CASE(NT_, NW_)                                                        \
  if (pl.nt == NT_ && pl.nwarps == NW_)                                             \
    return want_max ? launch_instance<NT_, NW_, true>(p, pl, grid, stream)          \
                    : launch_instance<NT_, NW_, false>(p, pl, grid, stream);
  CB200_CASE(1, 12) CB200_CASE(2, 12) CB200_CASE(4, 12)
  CB200_CASE(1, 8) CB200_CASE(2, 8) CB200_CASE(4, 8) CB200_CASE(8, 8)
#undef CB200_CASE
  return CUDALM_B200_ERR_UNSUPPORTED;
}

int validate(const cudalm_b200_linear& l) {
  if (!l.weight || !l.scales || !l.x || !l.y) return CUDALM_B200_ERR_NULL;
  if (l.N < 1 || l.K <= 0 || (l.K % 128) != 0 || l.M < 1) return CUDALM_B200_ERR_BAD_SHAPE;
  return CUDALM_B200_OK;
}

bool stream_eligible(const cudalm_b200_linear& l) {
  return aligned_to(l.weight, 16) && l.K <= kMaxStreamK;
}

inline int chunks_per_mtile(int K) { return ((K >> 7) + kCG - 1) / kCG; }
inline int mtiles(int N) { return (N + kMTileRows - 1) / kMTileRows; }

// cuTensorMapEncodeTiled, fetched from the driver at first use (the library
// links no driver stub, so it still loads on a machine without a GPU).
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static std::once_flag once;
  static EncodeTiledFn fn = nullptr;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) ==
            cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    else
      (void)cudaGetLastError();
  });
  return fn;
}

// Describes the packed weight matrix to the TMA unit as uint32 [N][K/8] with a
// box of 16 rows x kCG*16 words (= kCG groups of 128 nibbles per row).
// A tensor map depends only on (address, N, K), so encodings are kept in a small
// direct-mapped cache: the decode loop calls the same projections every step.
struct MapCacheEntry {
  const std::uint8_t* weight = nullptr;
  int N = 0, K = 0;
  CUtensorMap map;
};
constexpr int kMapCacheSize = 512;

int encode_weight_map_uncached(const std::uint8_t* weight, int N, int K, CUtensorMap* out);

int encode_weight_map(const std::uint8_t* weight, int N, int K, CUtensorMap* out) {
  static std::mutex mu;
  static MapCacheEntry cache[kMapCacheSize];
  const std::uintptr_t h = reinterpret_cast<std::uintptr_t>(weight);
  const int slot = static_cast<int>(((h >> 8) ^ (h >> 17) ^ static_cast<std::uintptr_t>(N) * 31u) %
                                    kMapCacheSize);
  {
    std::lock_guard<std::mutex> lk(mu);
    const MapCacheEntry& e = cache[slot];
    if (e.weight == weight && e.N == N && e.K == K) {
      *out = e.map;
      return CUDALM_B200_OK;
    }
  }
  if (int rc = encode_weight_map_uncached(weight, N, K, out)) return rc;
  std::lock_guard<std::mutex> lk(mu);
  cache[slot].weight = weight;
  cache[slot].N = N;
  cache[slot].K = K;
  cache[slot].map = *out;
  return CUDALM_B200_OK;
}

int encode_weight_map_uncached(const std::uint8_t* weight, int N, int K, CUtensorMap* out) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return CUDALM_B200_ERR_CUDA;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K / 8), static_cast<cuuint64_t>(N)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K / 2)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kCG * 16), static_cast<cuuint32_t>(kMTileRows)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2,
                        const_cast<std::uint8_t*>(weight), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = static_cast<int>(r);
    return CUDALM_B200_ERR_CUDA;
  }
  return CUDALM_B200_OK;
}

// What the fused MLP entries add to a projection: a second matrix over the same
// input (out = silu(W x) * (W2 x)) or a residual (out = residual + W x).
struct LinearExtra {
  const std::uint8_t* weight2 = nullptr;
  const std::uint16_t* scales2 = nullptr;
  const std::uint16_t* residual = nullptr;
};

int to_dev(const cudalm_b200_linear& l, int mt_begin, int cost_begin, LinearDev* d,
           const LinearExtra* ex = nullptr) {
  if (int rc = encode_weight_map(l.weight, l.N, l.K, &d->tmap)) return rc;
  d->W = l.weight;
  d->W2 = nullptr;
  d->S2 = nullptr;
  d->res = nullptr;
  int extra_flags = 0;
  if (ex && ex->weight2) {
    if (int rc = encode_weight_map(ex->weight2, l.N, l.K, &d->tmap2)) return rc;
    d->W2 = ex->weight2;
    d->S2 = ex->scales2;
    extra_flags |= kFlagPair | (aligned_to(ex->scales2, 16) ? kFlagScales2Bulk : 0);
  } else if (ex && ex->residual) {
    d->res = ex->residual;
    extra_flags |= kFlagResidual;
  }
  d->S = l.scales;
  d->x = l.x;
  d->y = l.y;
  d->N = l.N;
  d->K = l.K;
  d->M = l.M;
  d->mt_begin = mt_begin;
  d->flags = (aligned_to(l.scales, 16) ? kFlagScalesBulk : 0) | extra_flags;
  d->cost_begin = cost_begin;
  return CUDALM_B200_OK;
}

int run_fallback(const cudalm_b200_linear& l, cudaStream_t stream) {
  const int rows_per_block = 8;
  const int grid = (l.N + rows_per_block - 1) / rows_per_block;
  w4a16_fallback_kernel<<<grid, rows_per_block * 32, 0, stream>>>(l.weight, l.scales, l.x, l.y,
                                                                  l.N, l.K, l.M);
  return check_launch();
}

// One projection with any M: passes of as many rows as fit in shared memory.
int run_single(cudalm_b200_linear l, cudaStream_t stream) {
  if (int rc = validate(l)) return rc;
  if (direct_eligible(l, nullptr) &&
      direct_weight_bytes(l, false) <= g_direct_max_bytes.load(std::memory_order_relaxed))
    return run_direct(&l, 1, nullptr, nullptr, nullptr, stream);
  if (l.M >= g_tc_min_rows.load(std::memory_order_relaxed)) {
    // passes of up to 64 rows on the tensor-memory kernel
    cudalm_b200_linear probe = l;
    probe.M = l.M < 64 ? l.M : 64;
    if (tc_eligible(probe)) {
      for (int m0 = 0; m0 < l.M; m0 += 64) {
        cudalm_b200_linear part = l;
        part.M = (l.M - m0 < 64) ? (l.M - m0) : 64;
        part.x = l.x + static_cast<std::size_t>(m0) * l.K;
        part.y = l.y + static_cast<std::size_t>(m0) * l.N;
        if (int rc = run_tc(&part, 1, stream)) return rc;
      }
      return CUDALM_B200_OK;
    }
  }
  if (!stream_eligible(l)) return run_fallback(l, stream);
  const int per_pass = max_rows_per_pass(l.K);
  if (per_pass == 0) return run_fallback(l, stream);
  const int M = l.M;
  for (int m0 = 0; m0 < M; m0 += per_pass) {
    cudalm_b200_linear part = l;
    part.M = (M - m0 < per_pass) ? (M - m0) : per_pass;
    part.x = l.x + static_cast<std::size_t>(m0) * l.K;
    part.y = l.y + static_cast<std::size_t>(m0) * l.N;
    StreamParams p;
    std::memset(&p, 0, sizeof(p));
    p.table = nullptr;
    if (int rc = to_dev(part, 0, 0, &p.inl[0])) return rc;
    p.n_desc = 1;
    p.total_mt = mtiles(l.N);
    p.total_cost = p.total_mt * chunks_per_mtile(l.K);
    if (int rc = launch_stream(p, l.K, part.M, stream)) return rc;
  }
  return CUDALM_B200_OK;
}

// A projection with an MLP epilogue: passes of up to 16 rows on the streaming
// kernel (the pair keeps its first outputs in registers), or the slow kernel.
int run_extra(cudalm_b200_linear l, const LinearExtra& ex, cudaStream_t stream) {
  if (int rc = validate(l)) return rc;
  const bool pair = ex.weight2 != nullptr;
  if (pair && !ex.scales2) return CUDALM_B200_ERR_NULL;
  if (direct_eligible(l, ex.weight2) &&
      direct_weight_bytes(l, pair) <= g_direct_max_bytes.load(std::memory_order_relaxed)) {
    const std::uint8_t* w2[1] = {ex.weight2};
    const std::uint16_t* s2[1] = {ex.scales2};
    const std::uint16_t* rs[1] = {ex.residual};
    return run_direct(&l, 1, w2, s2, rs, stream);
  }
  if (l.M >= g_tc_min_rows.load(std::memory_order_relaxed)) {
    // passes of up to 64 rows on the tensor-memory kernel, when it takes the call
    bool done = true;
    for (int m0 = 0; m0 < l.M && done; m0 += 64) {
      cudalm_b200_linear part = l;
      part.M = (l.M - m0 < 64) ? (l.M - m0) : 64;
      part.x = l.x + static_cast<std::size_t>(m0) * l.K;
      part.y = l.y + static_cast<std::size_t>(m0) * l.N;
      const int rc = tc_eligible(part)
                         ? run_tc_extra(part, ex.weight2, ex.scales2,
                                        ex.residual ? ex.residual + static_cast<std::size_t>(m0) * l.N : nullptr,
                                        stream)
                         : CUDALM_B200_ERR_UNSUPPORTED;
      if (rc == CUDALM_B200_ERR_UNSUPPORTED && m0 == 0) done = false;  // streaming passes instead
      else if (rc != CUDALM_B200_OK) return rc;
    }
    if (done) return CUDALM_B200_OK;
  }
  int per_pass = stream_eligible(l) && (!pair || aligned_to(ex.weight2, 16)) ? max_rows_per_pass(l.K) : 0;
  if (per_pass > 16) per_pass = 16;
  if (per_pass == 0) {
    const int rows_per_block = 8;
    const int grid = (l.N + rows_per_block - 1) / rows_per_block;
    w4a16_fallback_kernel<<<grid, rows_per_block * 32, 0, stream>>>(
        l.weight, l.scales, l.x, l.y, l.N, l.K, l.M, ex.weight2, ex.scales2, ex.residual);
    return check_launch();
  }
  const int M = l.M;
  for (int m0 = 0; m0 < M; m0 += per_pass) {
    cudalm_b200_linear part = l;
    part.M = (M - m0 < per_pass) ? (M - m0) : per_pass;
    part.x = l.x + static_cast<std::size_t>(m0) * l.K;
    part.y = l.y + static_cast<std::size_t>(m0) * l.N;
    LinearExtra pex = ex;
    if (ex.residual) pex.residual = ex.residual + static_cast<std::size_t>(m0) * l.N;
    StreamParams p;
    std::memset(&p, 0, sizeof(p));
    if (int rc = to_dev(part, 0, 0, &p.inl[0], &pex)) return rc;
    p.n_desc = 1;
    p.total_mt = mtiles(l.N);
    p.total_cost = p.total_mt * chunks_per_mtile(l.K) * (pair ? 2 : 1);
    if (int rc = launch_stream(p, l.K, part.M, stream, nullptr, 0, true)) return rc;
  }
  return CUDALM_B200_OK;
}

}  // namespace

// Used by the vocabulary projection: one staged launch of a single projection (M rows
// in one pass) whose CTAs also leave their largest outputs per activation row in the
// pick's table.  Returns ERR_UNSUPPORTED when the projection cannot take the staged path
// in one pass.
int run_linear_with_pick(const cudalm_b200_linear& l, const PickTail& pick, cudaStream_t stream,
                         int* grid_out) {
  if (int rc = validate(l)) return rc;
  if (l.M >= g_tc_min_rows.load(std::memory_order_relaxed) && tc_eligible(l))
    return run_tc_with_pick(l, pick, stream, grid_out);
  if (!stream_eligible(l)) return CUDALM_B200_ERR_UNSUPPORTED;
  if (max_rows_per_pass(l.K) < l.M) return CUDALM_B200_ERR_UNSUPPORTED;
  StreamParams p;
  std::memset(&p, 0, sizeof(p));
  if (int rc = to_dev(l, 0, 0, &p.inl[0])) return rc;
  p.n_desc = 1;
  p.total_mt = mtiles(l.N);
  p.total_cost = p.total_mt * chunks_per_mtile(l.K);
  p.pick = pick;
  return launch_stream(p, l.K, l.M, stream, grid_out);
}

// True when run_linear_with_pick would take the projection (the same tests, no launch).
bool linear_with_pick_eligible(const cudalm_b200_linear& l) {
  if (validate(l) != CUDALM_B200_OK) return false;
  if (l.M >= g_tc_min_rows.load(std::memory_order_relaxed) && tc_eligible(l)) return true;
  return stream_eligible(l) && max_rows_per_pass(l.K) >= l.M;
}
bool linear_with_pick_on_tensor_path(const cudalm_b200_linear& l) {
  return l.M >= g_tc_min_rows.load(std::memory_order_relaxed) && tc_eligible(l);
}

int stream_rows_per_pass(int K) {
  return (K > 0 && K % 128 == 0 && K <= kMaxStreamK) ? max_rows_per_pass(K) : 0;
}

int run_linear_any(const cudalm_b200_linear& l, cudaStream_t stream) { return run_single(l, stream); }

}  // namespace cb200

// ---------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------
using namespace cb200;

struct cudalm_b200_group {
  cb200::TcGroup* tc = nullptr;  // set when the group runs on the tensor-memory kernel
  // set when no single launch takes the whole group: the projections run one by one
  std::vector<cudalm_b200_linear> singles;
  LinearDev* table_dev = nullptr;
  int2* ranges_dev = nullptr;  // per-CTA {first m-tile, projection}, grid + 1 entries
  int grid = 0;
  int count = 0;
  int total_mt = 0;
  int total_cost = 0;
  int kmax = 0;
  int mmax = 0;
  long long bytes = 0;
  int device = 0;
};

extern "C" {

int cudalm_b200_int4_gemv_bf16(const uint8_t* weight, const uint16_t* scales, const uint16_t* x,
                               uint16_t* y, int N, int K, void* stream) {
  cudalm_b200_linear l{weight, scales, x, y, N, K, 1, 0};
  return run_single(l, static_cast<cudaStream_t>(stream));
}

int cudalm_b200_batch_int4_gemv_bf16(const uint8_t* weight, const uint16_t* scales,
                                     const uint16_t* x, uint16_t* y, int N, int K, int B,
                                     void* stream) {
  cudalm_b200_linear l{weight, scales, x, y, N, K, B, 0};
  return run_single(l, static_cast<cudaStream_t>(stream));
}

int cudalm_b200_linear_multi(const cudalm_b200_linear* linears, int count, void* stream) {
  if (!linears) return CUDALM_B200_ERR_NULL;
  if (count < 1 || count > CUDALM_B200_MAX_INLINE_LINEARS) return CUDALM_B200_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  bool all_stream = true;
  int kmax = 0, mmax = 0;
  for (int i = 0; i < count; ++i) {
    if (int rc = validate(linears[i])) return rc;
    if (linears[i].reserved != 0) return CUDALM_B200_ERR_BAD_SHAPE;
    all_stream &= stream_eligible(linears[i]);
    kmax = linears[i].K > kmax ? linears[i].K : kmax;
    mmax = linears[i].M > mmax ? linears[i].M : mmax;
  }
  {
    bool all_direct = true;
    long long wbytes = 0;
    for (int i = 0; i < count; ++i) {
      all_direct &= direct_eligible(linears[i], nullptr);
      wbytes += direct_weight_bytes(linears[i], false);
    }
    if (all_direct && wbytes <= g_direct_max_bytes.load(std::memory_order_relaxed))
      return run_direct(linears, count, nullptr, nullptr, nullptr, st);
  }
  if (mmax >= g_tc_min_rows.load(std::memory_order_relaxed)) {
    bool all_tc = true;
    for (int i = 0; i < count; ++i) all_tc &= tc_eligible(linears[i]);
    if (all_tc) return run_tc(linears, count, st);
  }
  Plan pl;
  if (!all_stream || mmax > CUDALM_B200_MAX_GROUP_M || !make_plan(kmax, mmax, &pl)) {
    // not all of them fit one staged launch: run them one by one
    for (int i = 0; i < count; ++i)
      if (int rc = run_single(linears[i], st)) return rc;
    return CUDALM_B200_OK;
  }
  StreamParams p;
  std::memset(&p, 0, sizeof(p));
  int mt = 0, cost = 0;
  for (int i = 0; i < count; ++i) {
    if (int rc = to_dev(linears[i], mt, cost, &p.inl[i])) return rc;
    mt += mtiles(linears[i].N);
    cost += mtiles(linears[i].N) * chunks_per_mtile(linears[i].K);
  }
  p.n_desc = count;
  p.total_mt = mt;
  p.total_cost = cost;
  return launch_stream(p, kmax, mmax, st);
}

int cudalm_b200_gate_up_bf16(const uint8_t* gate_weight, const uint16_t* gate_scales,
                             const uint8_t* up_weight, const uint16_t* up_scales,
                             const uint16_t* x, uint16_t* gate_y, uint16_t* up_y, int N, int K,
                             int M, void* stream) {
  if (M < 1) return CUDALM_B200_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // rows of x beyond what one launch holds go in further passes
  int per_pass = (K > 0 && K % 128 == 0 && K <= kMaxStreamK) ? max_rows_per_pass(K) : 0;
  if (per_pass == 0) per_pass = M;
  // batched rows go to the tensor-memory kernel in passes of 64 (linear_multi falls
  // back to the streaming kernel, in its own passes, when that kernel does not take them)
  if (M >= g_tc_min_rows.load(std::memory_order_relaxed)) per_pass = 64;
  for (int m0 = 0; m0 < M; m0 += per_pass) {
    const int mm = (M - m0 < per_pass) ? (M - m0) : per_pass;
    cudalm_b200_linear two[2] = {
        {gate_weight, gate_scales, x ? x + static_cast<size_t>(m0) * K : x,
         gate_y ? gate_y + static_cast<size_t>(m0) * N : gate_y, N, K, mm, 0},
        {up_weight, up_scales, x ? x + static_cast<size_t>(m0) * K : x,
         up_y ? up_y + static_cast<size_t>(m0) * N : up_y, N, K, mm, 0}};
    if (int rc = cudalm_b200_linear_multi(two, 2, st)) return rc;
  }
  return CUDALM_B200_OK;
}

int cudalm_b200_gate_up_silu_bf16(const uint8_t* gate_weight, const uint16_t* gate_scales,
                                  const uint8_t* up_weight, const uint16_t* up_scales,
                                  const uint16_t* x, uint16_t* out, int N, int K, int M,
                                  void* stream) {
  if (!up_weight || !up_scales) return CUDALM_B200_ERR_NULL;
  cudalm_b200_linear l{gate_weight, gate_scales, x, out, N, K, M, 0};
  LinearExtra ex;
  ex.weight2 = up_weight;
  ex.scales2 = up_scales;
  return run_extra(l, ex, static_cast<cudaStream_t>(stream));
}

int cudalm_b200_linear_residual_bf16(const uint8_t* weight, const uint16_t* scales,
                                     const uint16_t* x, const uint16_t* residual, uint16_t* y,
                                     int N, int K, int M, void* stream) {
  if (!residual) return CUDALM_B200_ERR_NULL;
  cudalm_b200_linear l{weight, scales, x, y, N, K, M, 0};
  LinearExtra ex;
  ex.residual = residual;
  return run_extra(l, ex, static_cast<cudaStream_t>(stream));
}

int cudalm_b200_group_create(const cudalm_b200_linear* linears, int count,
                             cudalm_b200_group** group_out) {
  if (!linears || !group_out) return CUDALM_B200_ERR_NULL;
  if (count < 1) return CUDALM_B200_ERR_BAD_SHAPE;
  {
    // batched groups go to the tensor-memory kernel when every projection fits it
    int m_all = 0;
    long long tc_bytes = 0;
    for (int i = 0; i < count; ++i) {
      const cudalm_b200_linear& l = linears[i];
      if (int rc = validate(l)) return rc;
      m_all = l.M > m_all ? l.M : m_all;
      tc_bytes += static_cast<long long>(l.N) * (l.K / 2) + static_cast<long long>(l.N) * (l.K / 128) * 2 +
                  static_cast<long long>(l.M) * l.K * 2 + static_cast<long long>(l.M) * l.N * 2;
    }
    // ... and so do groups of fewer rows that do not fit the streaming kernel's
    // shared memory (long K with 9..16 rows)
    int k_all = 0;
    for (int i = 0; i < count; ++i) k_all = linears[i].K > k_all ? linears[i].K : k_all;
    Plan probe;
    const bool stream_fits = m_all <= CUDALM_B200_MAX_GROUP_M && k_all <= kMaxStreamK &&
                             make_plan(k_all, m_all, &probe);
    if (m_all >= g_tc_min_rows.load(std::memory_order_relaxed) || !stream_fits) {
      TcGroup* tg = nullptr;
      const int rc = tc_group_create(linears, count, &tg);
      if (rc == CUDALM_B200_OK) {
        cudalm_b200_group* g = new cudalm_b200_group();
        g->tc = tg;
        g->count = count;
        g->bytes = tc_bytes;
        *group_out = g;
        return CUDALM_B200_OK;
      }
      if (rc != CUDALM_B200_ERR_UNSUPPORTED) return rc;
    }
  }
  std::vector<LinearDev> tbl(static_cast<size_t>(count));
  int mt = 0, kmax = 0, mmax = 0;
  long long bytes = 0, cost = 0;
  bool one_by_one = false;
  for (int i = 0; i < count; ++i) {
    const cudalm_b200_linear& l = linears[i];
    if (int rc = validate(l)) return rc;
    if (l.reserved != 0) return CUDALM_B200_ERR_BAD_SHAPE;
    if (!aligned_to(l.weight, 16) || l.K > kMaxStreamK || l.M > CUDALM_B200_MAX_GROUP_M) {
      one_by_one = true;
      break;
    }
    if (int rc = to_dev(l, mt, static_cast<int>(cost), &tbl[static_cast<size_t>(i)])) return rc;
    mt += mtiles(l.N);
    cost += static_cast<long long>(mtiles(l.N)) * chunks_per_mtile(l.K);
    if (cost > 0x3fffffff) return CUDALM_B200_ERR_TOO_LARGE;
    kmax = l.K > kmax ? l.K : kmax;
    mmax = l.M > mmax ? l.M : mmax;
    bytes += static_cast<long long>(l.N) * (l.K / 2) + static_cast<long long>(l.N) * (l.K / 128) * 2 +
             static_cast<long long>(l.M) * l.K * 2 + static_cast<long long>(l.M) * l.N * 2;
  }
  Plan pl;
  if (!one_by_one && !make_plan(kmax, mmax, &pl, count > 1)) one_by_one = true;
  if (one_by_one) {
    // a projection that only the slow kernel takes, or rows that do not fit one
    // staged launch: same results, one launch (or several passes) per projection
    cudalm_b200_group* g = new cudalm_b200_group();
    g->count = count;
    g->singles.assign(linears, linears + count);
    for (int i = 0; i < count; ++i) {
      const cudalm_b200_linear& l = linears[i];
      g->bytes += static_cast<long long>(l.N) * (l.K / 2) + static_cast<long long>(l.N) * (l.K / 128) * 2 +
                  static_cast<long long>(l.M) * l.K * 2 + static_cast<long long>(l.M) * l.N * 2;
    }
    *group_out = g;
    return CUDALM_B200_OK;
  }
  cudalm_b200_group* g = new cudalm_b200_group();
  g->count = count;
  g->total_mt = mt;
  g->total_cost = static_cast<int>(cost);
  g->kmax = kmax;
  g->mmax = mmax;
  g->bytes = bytes;
  // Per-CTA ranges.  Inside a CTA warp w takes the range's m-tiles w, w + NW,
  // w + 2 NW, ... whole, so a CTA is as slow as its most loaded warp: 54 m-tiles
  // of a long K over 8 warps cost as much as 56.  The ranges are therefore cut
  // by that model: an m-tile weighs its quantisation groups plus what its
  // chunks and its epilogue cost (measured: issuing a chunk's copies ~1.85
  // groups' worth of time, an epilogue ~0.7), a change of projection a few
  // groups more, and a range's cost is the largest per-warp sum.  The smallest
  // bound T under which greedy ranges cover the launch with one CTA per SM is
  // found by bisection.
#ifndef CB200_SWITCH_WEIGHT
#define CB200_SWITCH_WEIGHT 800
#endif
  constexpr long long kSwitchWeight = CB200_SWITCH_WEIGHT;  // hundredths of a group
  g->grid = num_sms() < mt ? num_sms() : mt;
  std::vector<int2> ranges(static_cast<size_t>(g->grid) + 1);
  {
    const int nw = pl.nwarps;
    std::vector<int> weight(static_cast<size_t>(count));
    for (int i = 0; i < count; ++i)
      weight[static_cast<size_t>(i)] = 100 * (linears[i].K >> 7) + 185 * chunks_per_mtile(linears[i].K) + 73;
    // greedy cut under bound T; returns the number of CTAs used (grid + 1 when T is too small)
    auto cut = [&](long long T, std::vector<int2>* out) {
      int d = 0, pos = 0, used = 0;  // pos: next m-tile to place, d: its projection
      std::vector<long long> load(static_cast<size_t>(nw));
      while (pos < mt) {
        if (used == g->grid) return g->grid + 1;
        if (out) (*out)[static_cast<size_t>(used)] = make_int2(pos, d);
        std::fill(load.begin(), load.end(), 0);
        long long extra = 0;  // changes of projection, paid by every warp
        long long worst = 0;  // most loaded warp
        int taken = 0;
        int dd = d;
        while (pos < mt) {
          while (pos >= tbl[static_cast<size_t>(dd)].mt_begin + mtiles(tbl[static_cast<size_t>(dd)].N)) ++dd;
          const long long sw = (taken > 0 && dd != d) ? kSwitchWeight : 0;
          long long& slot = load[static_cast<size_t>(taken % nw)];
          const long long cand = slot + weight[static_cast<size_t>(dd)];
          const long long worst_then = cand > worst ? cand : worst;
          if (taken > 0 && worst_then + extra + sw > T) break;
          worst = worst_then;
          slot = cand;
          extra += sw;
          d = dd;
          ++taken;
          ++pos;
        }
        // the next range starts in the projection that holds `pos`
        while (pos < mt && pos >= tbl[static_cast<size_t>(d)].mt_begin + mtiles(tbl[static_cast<size_t>(d)].N)) ++d;
        ++used;
      }
      if (out)
        for (int b = used; b <= g->grid; ++b) (*out)[static_cast<size_t>(b)] = make_int2(mt, count);
      return used;
    };
    long long lo = 0, hi = 0;
    for (int i = 0; i < count; ++i)
      hi += static_cast<long long>(mtiles(linears[i].N)) * weight[static_cast<size_t>(i)] + kSwitchWeight;
    while (lo + 1 < hi) {  // invariant: hi is feasible, lo is not
      const long long mid = lo + (hi - lo) / 2;
      if (cut(mid, nullptr) <= g->grid) hi = mid; else lo = mid;
    }
    (void)cut(hi, &ranges);
  }
  cudaError_t e = cudaGetDevice(&g->device);
  if (e == cudaSuccess) e = cudaMalloc(&g->table_dev, sizeof(LinearDev) * tbl.size());
  if (e == cudaSuccess)
    e = cudaMemcpy(g->table_dev, tbl.data(), sizeof(LinearDev) * tbl.size(), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMalloc(&g->ranges_dev, sizeof(int2) * ranges.size());
  if (e == cudaSuccess)
    e = cudaMemcpy(g->ranges_dev, ranges.data(), sizeof(int2) * ranges.size(), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    g_last_cuda_error = static_cast<int>(e);
    if (g->table_dev) cudaFree(g->table_dev);
    if (g->ranges_dev) cudaFree(g->ranges_dev);
    delete g;
    return CUDALM_B200_ERR_CUDA;
  }
  *group_out = g;
  return CUDALM_B200_OK;
}

int cudalm_b200_group_run(const cudalm_b200_group* group, void* stream) {
  if (!group) return CUDALM_B200_ERR_NULL;
  if (group->tc) return tc_group_run(group->tc, static_cast<cudaStream_t>(stream));
  if (!group->singles.empty()) {
    for (const cudalm_b200_linear& l : group->singles)
      if (int rc = run_linear_any(l, static_cast<cudaStream_t>(stream))) return rc;
    return CUDALM_B200_OK;
  }
  StreamParams p;
  std::memset(&p, 0, sizeof(p));
  p.table = group->table_dev;
  p.n_desc = group->count;
  p.total_mt = group->total_mt;
  p.total_cost = group->total_cost;
  p.cta_ranges = group->ranges_dev;
  return launch_stream(p, group->kmax, group->mmax, static_cast<cudaStream_t>(stream), nullptr,
                       group->grid);
}

int cudalm_b200_group_destroy(cudalm_b200_group* group) {
  if (!group) return CUDALM_B200_OK;
  if (group->tc) {
    tc_group_destroy(group->tc);
    delete group;
    return CUDALM_B200_OK;
  }
  if (!group->singles.empty()) {
    delete group;
    return CUDALM_B200_OK;
  }
  cudaError_t e = cudaFree(group->table_dev);
  const cudaError_t e2 = cudaFree(group->ranges_dev);
  if (e == cudaSuccess) e = e2;
  delete group;
  if (e != cudaSuccess) {
    g_last_cuda_error = static_cast<int>(e);
    return CUDALM_B200_ERR_CUDA;
  }
  return CUDALM_B200_OK;
}

int cudalm_b200_set_tensor_path_min_rows(int min_rows) {
  if (min_rows < 1) min_rows = 1;
  return g_tc_min_rows.exchange(min_rows);
}

int64_t cudalm_b200_set_direct_path_max_bytes(int64_t max_bytes) {
  if (max_bytes < 0) max_bytes = 0;
  return g_direct_max_bytes.exchange(max_bytes);
}

int64_t cudalm_b200_group_bytes(const cudalm_b200_group* group) {
  return group ? group->bytes : 0;
}

int cudalm_b200_kernel_regs(const char* kernel_name) {
  if (!kernel_name) return -1;
  const void* fn = nullptr;
#define CB200_NAME(NT_, NW_)                                                     \
  if (std::strcmp(kernel_name, "w4a16_stream_nt" #NT_ "_w" #NW_) == 0)           \
    fn = reinterpret_cast<const void*>(                                           \
        &w4a16_stream_kernel<NT_, kCG, NW_, false, (CB200_PRODUCERS && NW_ == 8) ? 2 : 0, false>);
  CB200_NAME(1, 12) CB200_NAME(2, 12) CB200_NAME(4, 12)
  CB200_NAME(1, 8) CB200_NAME(2, 8) CB200_NAME(4, 8) CB200_NAME(8, 8)
#undef CB200_NAME
  if (std::strcmp(kernel_name, "w4a16_fallback") == 0)
    fn = reinterpret_cast<const void*>(&w4a16_fallback_kernel);
  if (std::strcmp(kernel_name, "w4a16_direct") == 0) return direct_kernel_regs();
  if (!fn) return -1;
  cudaFuncAttributes attr;
  if (cudaFuncGetAttributes(&attr, fn) != cudaSuccess) {
    (void)cudaGetLastError();
    return -1;
  }
  return attr.numRegs;
}

}  // extern "C"
