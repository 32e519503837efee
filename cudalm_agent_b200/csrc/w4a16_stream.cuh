// Building blocks of the streaming W4A16 kernels.
//
// Work unit: an "m-tile" = 16 consecutive output rows of one projection, cut
// along K into chunks of CG quantisation groups (CG*128 values of k).  Each
// warp owns whole m-tiles and feeds itself: it keeps a private ring of `depth`
// shared-memory stages and fills a stage with ONE tiled TMA copy
// (cp.async.bulk.tensor.2d: a box of 16 rows x CG*64 bytes out of the pitched
// weight matrix; rows past N and bytes past K/2 arrive as zeros) plus one bulk
// copy of the m-tile's scales, both completing on the stage's mbarrier.  The
// warp refills a stage as soon as it has consumed it.  Issuing a TMA copy costs
// the issuing warp tens of cycles, which is why a stage is one box and not one
// copy per row.
//
// Inside a CTA's range of m-tiles warp w takes m-tiles w, w + NWARPS, ...  The
// activation vector is the only thing the warps share.  When two activation
// buffers fit (few rows), a change of projection needs no CTA-wide barrier:
// the next projection's activations are copied into a staging area while the
// warps still work from the current buffer, and each warp converts its share
// into the free buffer when it next looks.  Otherwise the CTA synchronises at
// the change and refills the single buffer together.
//
// Stage layout: 16 row segments of CG*64 bytes, then the m-tile's scale block
// fp16 [16][K/128].
//
// Arithmetic: the 4-bit values become exact bf16 integers (times a power of
// two) in registers and go through mma.sync m16n8k16 (weights = the 16-row
// operand, up to 8 activation rows = the 8 columns), one quantisation group at
// a time into a group accumulator; the group's fp32 sum is then folded in as
// acc += scale * sum.  Products are exact (4-bit x 8-bit significands) and all
// sums are fp32.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "lm_head_pick.cuh"

namespace cb200 {

constexpr int kMTileRows = 16;
constexpr int kMaxDepth = 4;
constexpr int kMaxWarps = 16;
// shared-memory header: "full" mbarriers [kMaxWarps][kMaxDepth], CtaControl, and in
// its last 512 bytes the "empty" mbarriers [kMaxWarps][kMaxDepth] of the producer form
constexpr int kHeaderBytes = 2176;
// projections of a CTA's range whose descriptors are kept in shared memory
constexpr int kDescCache = 8;
// largest M*K one warp refills on its own (the barrier-free change of projection)
constexpr int kAsyncFillMaxValues = 8192;

enum : int {
  kFlagScalesBulk = 1,   // the scales' base is 16-byte aligned: bulk copies
  kFlagPair = 2,         // gate and up matrices over one input: out = silu(gate) * up
  kFlagScales2Bulk = 4,  // the same for the second matrix of a pair
  kFlagResidual = 8,     // out = residual + projection
};

// Device-side projection descriptor.
struct alignas(64) LinearDev {
  CUtensorMap tmap;   // weight matrix as uint32 [N][K/8], box 16 rows x CG*16 words
  CUtensorMap tmap2;  // second matrix of a pair (kFlagPair)
  const std::uint8_t* W;     // the same matrices for plain loads (activations out of range)
  const std::uint8_t* W2;
  const std::uint16_t* S;
  const std::uint16_t* S2;   // scales of the second matrix
  const std::uint16_t* res;  // residual [M][N] (kFlagResidual)
  const std::uint16_t* x;
  std::uint16_t* y;
  int N, K, M;
  int mt_begin;    // index of this projection's first m-tile in the launch
  int flags;
  int cost_begin;  // chunks (m-tiles x chunks per m-tile) before this projection
};

struct StreamParams {
  LinearDev inl[CUDALM_B200_MAX_INLINE_LINEARS];
  const LinearDev* table;  // device table, or nullptr to use `inl`
  int n_desc;
  int total_mt;
  int total_cost;   // chunks in the whole launch
  int depth;        // stages per warp ring, 2..kMaxDepth
  int stage_bytes;  // 16 * CG*64 + scale block of the largest K
  int x_bytes;      // one activation buffer
  int x_buffers;    // 1, or 2 for the barrier-free change of projection
  int* status;      // device status word
  // CTA_MAX only (the vocabulary projection, one projection per launch): the table the
  // CTAs leave their maxima in for the token pick (lm_head_pick.cuh)
  PickTail pick;
  // Optional, for launches with a device table: per CTA {first m-tile, its
  // projection}, gridDim.x + 1 entries, so that a CTA finds its range with two
  // loads instead of a chain of dependent table look-ups.
  const int2* cta_ranges;
};

#ifdef __CUDACC__

__device__ __forceinline__ const LinearDev* desc_table(const StreamParams& p) {
  return p.table ? p.table : p.inl;
}

__device__ __forceinline__ int desc_mtiles(int N) { return (N + kMTileRows - 1) / kMTileRows; }

// Descriptor that holds m-tile `mt` (binary search over mt_begin).
__device__ __forceinline__ int find_desc(const StreamParams& p, int mt) {
  const LinearDev* tbl = desc_table(p);
  int lo = 0, hi = p.n_desc - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (tbl[mid].mt_begin <= mt) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// First m-tile of the CTA range that starts at chunk position `cost`: CTAs get
// equal shares of chunks (bytes), not of m-tiles, because an m-tile of a
// projection with a long K is several times larger than one with a short K.
template <int CG>
__device__ __forceinline__ int mtile_at_cost(const StreamParams& p, long long cost) {
  if (cost >= p.total_cost) return p.total_mt;
  const LinearDev* tbl = desc_table(p);
  int lo = 0, hi = p.n_desc - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (tbl[mid].cost_begin <= cost) lo = mid; else hi = mid - 1;
  }
  const int nch = (((tbl[lo].K >> 7) + CG - 1) / CG) * ((tbl[lo].flags & kFlagPair) ? 2 : 1);
  const int within = static_cast<int>(cost) - tbl[lo].cost_begin;
  return tbl[lo].mt_begin + (within + nch - 1) / nch;
}

// Per-CTA bookkeeping in shared memory.
// What the kernel needs of a projection, without the tensor map itself.
struct DescLite {
  const CUtensorMap* tmap;
  const CUtensorMap* tmap2;
  const std::uint8_t* W;
  const std::uint8_t* W2;
  const std::uint16_t* S;
  const std::uint16_t* S2;
  const std::uint16_t* res;
  const std::uint16_t* x;
  std::uint16_t* y;
  int N, K, M, mt_begin, flags, pad;
};

struct CtaControl {
  unsigned long long xbar;  // mbarrier of the activation staging copy
  int pad;
  int fill_claim;           // first projection whose activation refill nobody has taken
  int fill_done;            // every projection before this one has its activations in place
  int fill_parts;           // warps that have converted their share of the refill under way
  int abort;                // a bounded wait ran out somewhere in the CTA
  // CTA_MAX: per activation row, key + 1 of the largest output this CTA has produced
  std::uint32_t row_key[kMaxPassRows];
  int issued[kMaxWarps];    // producer form: stages issued so far for each consumer warp
  int cur_desc[kMaxWarps];  // projection each warp is consuming (INT_MAX when done)
  // The CTA's first projections.  Under load a dependent load from global
  // memory waits microseconds behind the weight stream, so nothing in the
  // steady state reads the descriptor table there.
  DescLite desc[kDescCache];
};

struct DescSource {
  const StreamParams* p;
  const DescLite* cache;
  int d_first;
};

static_assert(2 * kMaxWarps * kMaxDepth * 8 + sizeof(CtaControl) <= kHeaderBytes, "header too small");

__device__ __forceinline__ int ld_volatile_s32(const int* p) {
  return *reinterpret_cast<const volatile int*>(p);
}
__device__ __forceinline__ void st_volatile_s32(int* p, int v) {
  *reinterpret_cast<volatile int*>(p) = v;
}

__device__ __forceinline__ DescLite get_desc(const DescSource& ds, int d) {
  if (d - ds.d_first < kDescCache) return ds.cache[d - ds.d_first];
  const LinearDev* L = desc_table(*ds.p) + d;
  return DescLite{&L->tmap, &L->tmap2, L->W, L->W2, L->S, L->S2, L->res, L->x, L->y,
                  L->N,     L->K,      L->M,  L->mt_begin, L->flags, 0};
}

// Position of a warp in the launch: an m-tile, the chunk inside it and the
// projection it belongs to.
template <int CG>
struct Cursor {
  int d, mt, chunk;
  int mt_begin, mt_end, N, G, flags;
  int nch;        // chunks of one matrix per m-tile
  int nch_total;  // chunks per m-tile: twice nch for a pair (first matrix, then second)
  const CUtensorMap* tmap;
  const CUtensorMap* tmap2;
  const std::uint16_t* S;
  const std::uint16_t* S2;
  bool valid;

  __device__ __forceinline__ void bind(const DescSource& ds, int dd) {
    const DescLite L = get_desc(ds, dd);
    d = dd;
    mt_begin = L.mt_begin;
    N = L.N;
    mt_end = mt_begin + desc_mtiles(N);
    G = L.K >> 7;
    flags = L.flags;
    tmap = L.tmap;
    tmap2 = L.tmap2;
    S = L.S;
    S2 = L.S2;
    nch = (G + CG - 1) / CG;
    nch_total = (flags & kFlagPair) ? 2 * nch : nch;
  }
  // The current chunk's matrix (a pair: first all chunks of the gate matrix,
  // then all chunks of the up matrix) and its index inside that matrix.
  __device__ __forceinline__ bool second() const { return chunk >= nch; }
  __device__ __forceinline__ int chunk_in() const { return chunk >= nch ? chunk - nch : chunk; }
  __device__ __forceinline__ const CUtensorMap* cur_map() const { return chunk >= nch ? tmap2 : tmap; }
  __device__ __forceinline__ const std::uint16_t* cur_scales() const { return chunk >= nch ? S2 : S; }
  __device__ __forceinline__ bool cur_scales_aligned() const {
    return (flags & (chunk >= nch ? kFlagScales2Bulk : kFlagScalesBulk)) != 0;
  }
  // Moves to m-tile m, which is at or after the current one; m >= mt_hi ends
  // the walk.
  __device__ __forceinline__ void seek(const DescSource& ds, int m, int mt_hi) {
    mt = m;
    chunk = 0;
    valid = m < mt_hi;
    if (valid)
      while (mt >= mt_end) bind(ds, d + 1);
  }
};

// Tiled TMA copy: a box of the 2-D tensor described by `tmap`, starting at
// (x = word column, y = row), into `smem_dst`; completes on `bar`.  x must be a
// multiple of 4 words (16 bytes); it always is, being a multiple of CG*16.
__device__ __forceinline__ void tma_box_2d(void* smem_dst, const CUtensorMap* tmap, int x, int y,
                                           std::uint64_t* bar, std::uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

// Starts the copies that fill `stage` with the cursor's item.
template <int CG, bool EXTRA>
__device__ __forceinline__ void issue_item(const Cursor<CG>& c, std::uint8_t* stage,
                                           std::uint64_t* bar, int lane,
                                           std::uint64_t policy) {
  constexpr int RS = CG * 64;
  constexpr std::uint32_t kBoxBytes = kMTileRows * RS;
  const int row0 = (c.mt - c.mt_begin) * kMTileRows;
  const int rows = min(kMTileRows, c.N - row0);
  const std::uint32_t sbytes = static_cast<std::uint32_t>(rows * c.G) * 2u;
  const std::uint16_t* ssrc = (EXTRA ? c.cur_scales() : c.S) + static_cast<std::size_t>(row0) * c.G;
  const bool sbulk = (EXTRA ? c.cur_scales_aligned() : (c.flags & kFlagScalesBulk) != 0) &&
                     ((sbytes & 15u) == 0u);
  std::uint8_t* sdst = stage + kBoxBytes;
  if (!sbulk) {
    // ragged scale block (or an unaligned scale base): plain loads
    for (int i = lane; i < rows * c.G; i += 32)
      reinterpret_cast<std::uint16_t*>(sdst)[i] = __ldg(ssrc + i);
  }
  // order this warp's earlier reads of the stage before the async writes
#ifndef CB200_NO_ISSUE_FENCE
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
#endif
  __syncwarp();
  if (lane == 0) {
    mbar_arrive_expect_tx(bar, kBoxBytes + (sbulk ? sbytes : 0u));
    tma_box_2d(stage, EXTRA ? c.cur_map() : c.tmap, (EXTRA ? c.chunk_in() : c.chunk) * (CG * 16), row0,
               bar, policy);
    if (sbulk) bulk_g2s(sdst, ssrc, sbytes, bar);
  }
}

// The same from a single thread that is not the stage's reader (producer form): the
// reader released the stage through an mbarrier, which orders its reads before these
// copies.  A ragged or unaligned scale block is left to the reader (stage_scales_bulk).
template <int CG, bool EXTRA>
__device__ __forceinline__ bool stage_scales_bulk(const Cursor<CG>& c) {
  const int row0 = (c.mt - c.mt_begin) * kMTileRows;
  const int rows = min(kMTileRows, c.N - row0);
  return (EXTRA ? c.cur_scales_aligned() : (c.flags & kFlagScalesBulk) != 0) &&
         (((rows * c.G * 2) & 15) == 0);
}
template <int CG, bool EXTRA>
__device__ __forceinline__ void issue_item_single(const Cursor<CG>& c, std::uint8_t* stage,
                                                  std::uint64_t* bar, std::uint64_t policy) {
  constexpr int RS = CG * 64;
  constexpr std::uint32_t kBoxBytes = kMTileRows * RS;
  const int row0 = (c.mt - c.mt_begin) * kMTileRows;
  const int rows = min(kMTileRows, c.N - row0);
  const std::uint32_t sbytes = static_cast<std::uint32_t>(rows * c.G) * 2u;
  const bool sbulk = stage_scales_bulk<CG, EXTRA>(c);
  mbar_arrive_expect_tx(bar, kBoxBytes + (sbulk ? sbytes : 0u));
  tma_box_2d(stage, EXTRA ? c.cur_map() : c.tmap, (EXTRA ? c.chunk_in() : c.chunk) * (CG * 16), row0,
             bar, policy);
  if (sbulk)
    bulk_g2s(stage + kBoxBytes, (EXTRA ? c.cur_scales() : c.S) + static_cast<std::size_t>(row0) * c.G,
             sbytes, bar);
}

// Bounded wait on a stage; false when it ran out (about two seconds).
__device__ __forceinline__ bool wait_stage(std::uint64_t* bar, std::uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
  for (;;) {
    // back off between polls so that a waiting warp leaves the issue slots to
    // the warps that have data
    for (int i = 0; i < 256; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
      __nanosleep(40);
    }
    unsigned long long t1;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
    if (t1 - t0 > 2000000000ull) return false;
  }
}

// Power-of-two factors of the tiny-number dequantisation (see dequant_word):
// weights carry 2^-133 (even nibbles) or 2^-129 (odd nibbles), activations are
// stored times 2^64 or 2^60, so a group sum comes out times 2^-69.
#define CB200_X_SCALE_EVEN 0x1p64f
#define CB200_X_SCALE_ODD 0x1p60f
#define CB200_OUT_SCALE 0x1p69f
constexpr int kXRowPad = 64;  // bytes between the end of one activation row and the next

// Activation layout in shared memory for the MMA fragments: row n at stride
// rsx = 2K + 64 bytes (kXRowPad: rows alternate between the two halves of the banks);
// inside a row the values are permuted so that the eight values a lane needs for the
// two MMAs of one weight word are 16 contiguous bytes, one load:
//   k = 128 g + 32 t + 8 w + i   (t = lane & 3, w = word of the lane's 16 weight
//   bytes, i = nibble in the word) goes to slot (((g*4 + w)*4 + t)*2 + h)*4 + e with
//   h = (i & 3) >> 1 (the MMA j = 2w + h), e = 2*(i & 1) + (i >> 2).
// Values are stored times 2^64 (even i) or 2^60 (odd i); both are exact in bf16
// for |x| < 2^63.  Row M (one past the real rows) is all zeros: MMA columns
// beyond M read it, so the fragment loads need no predicate.
__device__ __forceinline__ void store_x_value(std::uint8_t* xs, int rsx, int n, int k,
                                              std::uint16_t bits) {
  const int g = k >> 7, r = k & 127, t = r >> 5, q = r & 31, w = q >> 3, i = q & 7;
  const int h = (i & 3) >> 1;
  const int e = 2 * (i & 1) + (i >> 2);
  const float f = bf16_bits_to_float(bits) * ((i & 1) ? CB200_X_SCALE_ODD : CB200_X_SCALE_EVEN);
  *reinterpret_cast<std::uint16_t*>(xs + n * rsx + ((((((g * 4 + w) * 4 + t) * 2 + h) * 4) + e) * 2)) =
      float_to_bf16_bits(f);
}

// Range of activations the tiny-number arithmetic represents: x * 2^64 must stay
// finite (|x| < 2^63; 2^62 is used), and a quantisation group whose largest magnitude is
// below 2^-50 would lose its products to fp32 underflow.  A projection whose
// activations fall outside (infinities and NaNs included) is flagged when its
// activations are staged, and its m-tiles are then recomputed from global memory in
// the CPU reference's own order (slow_mtile), so that every input a bf16 can hold gives
// the reference's result.  The flag word sits in the last 16 bytes of an activation
// buffer and holds (projection index + 1) of a flagged projection.
constexpr std::uint32_t kXBigBits = (127u + 62u) << 7;
constexpr std::uint32_t kXTinyBits = (127u - 50u) << 7;
constexpr int kXFlagBytes = 128;  // reserved at the end of every activation buffer
__device__ __forceinline__ std::uint32_t abs_bits4(uint2 v) {
  const std::uint32_t a = v.x & 0x7FFF7FFFu, b = v.y & 0x7FFF7FFFu;
  return max(max(a & 0xFFFFu, a >> 16), max(b & 0xFFFFu, b >> 16));
}
// `absmax` = this lane's largest |bits| over a span that the warp covers together
// (at most one quantisation group of one activation row); all 32 lanes call.
__device__ __forceinline__ bool span_out_of_range(std::uint32_t absmax) {
  const std::uint32_t m = __reduce_max_sync(0xffffffffu, absmax);
  return m >= kXBigBits || (m != 0u && m < kXTinyBits);
}
__device__ __forceinline__ int* x_flag_word(std::uint8_t* xs, int x_bytes) {
  return reinterpret_cast<int*>(xs + x_bytes - 16);
}

// The m-tile's outputs of this lane's fragment, from global memory, term by term in the
// order of the CPU reference (CUDALM tests/cuda/test_int4_gemv_bf16.cpp:54-69): for
// each byte, acc += (lo * s) * x[2b], then acc += (hi * s) * x[2b + 1].
template <int NT>
__device__ __noinline__ void slow_mtile(const std::uint8_t* W, const std::uint16_t* S,
                                        const std::uint16_t* x, int N, int K, int M, int row0,
                                        int lane, float (&out)[NT][4]) {
  const int r8 = lane >> 2, t = lane & 3;
  for (int nt = 0; nt < NT; ++nt) {
    for (int e = 0; e < 4; ++e) {
      const int row = row0 + r8 + (e >> 1) * 8;
      const int col = nt * 8 + 2 * t + (e & 1);
      float a = 0.f;
      if (row < N && col < M) {
        const std::uint8_t* wr = W + static_cast<std::size_t>(row) * (K >> 1);
        const std::uint16_t* sr = S + static_cast<std::size_t>(row) * (K >> 7);
        const std::uint16_t* xr = x + static_cast<std::size_t>(col) * K;
        for (int b = 0; b < (K >> 1); ++b) {
          const std::uint8_t byte = wr[b];
          const float sc = __half2float(__ushort_as_half(sr[b >> 6]));
          const int lo = static_cast<int>(static_cast<std::int8_t>((byte & 0x0Fu) << 4)) >> 4;
          const int hi = static_cast<int>(static_cast<std::int8_t>(byte)) >> 4;
          a = __fadd_rn(a, __fmul_rn(__fmul_rn(static_cast<float>(lo), sc), bf16_bits_to_float(xr[2 * b])));
          a = __fadd_rn(a, __fmul_rn(__fmul_rn(static_cast<float>(hi), sc), bf16_bits_to_float(xr[2 * b + 1])));
        }
      }
      out[nt][e] = a;
    }
  }
}

template <int U, bool kFromShared = false>
__device__ __forceinline__ void fill_x_fragments(std::uint8_t* xs, const std::uint16_t* x,
                                                 int M, int K, int rsx, int tid,
                                                 int nthreads, int* flag, int tag) {
  const int total = M * K;
  bool bad = false;
  if ((reinterpret_cast<std::uintptr_t>(x) & 7u) == 0) {
    // four values per 8-byte load, U loads in flight per thread; a warp's 32 loads of
    // one step are 128 consecutive values, i.e. one group of one row
    const int quads = total >> 2;
    for (int q0 = tid; q0 < quads; q0 += U * nthreads) {
      uint2 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int qi = q0 + u * nthreads;
        v[u] = qi >= quads    ? make_uint2(0u, 0u)
               : kFromShared ? reinterpret_cast<const uint2*>(x)[qi]
                             : __ldg(reinterpret_cast<const uint2*>(x) + qi);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int qi = q0 + u * nthreads;
        bad |= span_out_of_range(abs_bits4(v[u]));
        if (qi < quads) {
          const int idx = qi << 2;
          const int n = idx / K;
          const int k = idx - n * K;
          store_x_value(xs, rsx, n, k, static_cast<std::uint16_t>(v[u].x & 0xFFFFu));
          store_x_value(xs, rsx, n, k + 1, static_cast<std::uint16_t>(v[u].x >> 16));
          store_x_value(xs, rsx, n, k + 2, static_cast<std::uint16_t>(v[u].y & 0xFFFFu));
          store_x_value(xs, rsx, n, k + 3, static_cast<std::uint16_t>(v[u].y >> 16));
        }
      }
    }
  } else {
    for (int idx = tid; idx < total; idx += nthreads) {
      const int n = idx / K;
      const std::uint16_t bits = kFromShared ? x[idx] : __ldg(x + idx);
      bad |= span_out_of_range(bits & 0x7FFFu);
      store_x_value(xs, rsx, n, idx - n * K, bits);
    }
  }
  if (bad && (tid & 31) == 0) st_volatile_s32(flag, tag);
  for (int idx = tid; idx < K / 2; idx += nthreads)
    *reinterpret_cast<std::uint32_t*>(xs + M * rsx + idx * 4) = 0u;
}

// int4 -> bf16 through bf16's tiny numbers.  A bf16 whose high byte is zero is
// the integer in its low byte times 2^-133 (the subnormals run on linearly into
// the first normal binade), so (w & 0x000F000F) and (w & 0x00F000F0) are
// already bf16 pairs holding n * 2^-133 and 16 n * 2^-133: four of a word's
// eight nibbles need no shift.  XOR 8, folded into the same LOP3, turns the
// two's-complement nibble n into the offset-binary u = q + 8 in [0, 15].  For a
// word holding n0..n7 (n_i at bits 4i): out[i] = { u(n_i), u(n_{i+4}) } (low
// half, high half) times 2^-133 (even i) or 2^-129 (odd i).
//
// The offset is removed per quantisation group, not per value:
//   sum_k q_k x_k = sum_k u_k x_k - 8 sum_k x_k,
// where the second sum is the same for every weight row.  It is computed once
// per projection and activation row (build_bias) by the very same MMA sequence
// fed with the constant u = 8, so that an all-zero group cancels to an exact
// zero, and subtracted from each group sum before the scale is applied.
constexpr std::uint32_t kBiasEven = 0x00080008u;  // { 8, 8 } * 2^-133
constexpr std::uint32_t kBiasOdd = 0x00800080u;   // { 8, 8 } * 2^-129
__device__ __forceinline__ void dequant_word(std::uint32_t w, std::uint32_t (&out)[4]) {
  const std::uint32_t w8 = w >> 8;
  out[0] = lop3_and_xor(w, 0x000F000Fu, kBiasEven);
  out[1] = lop3_and_xor(w, 0x00F000F0u, kBiasOdd);
  out[2] = lop3_and_xor(w8, 0x000F000Fu, kBiasEven);
  out[3] = lop3_and_xor(w8, 0x00F000F0u, kBiasOdd);
}

// The eight MMAs of a group are spread over kC independent accumulation chains;
// the group sum is the chains' sum in a fixed order, the same in build_bias and
// consume_chunk.  Measured on the M=1 set: 2 chains 49.0 us, 4 chains 52.0 us,
// 8 chains 54.9 us per launch (the extra adds and registers cost more than the
// shorter dependency chains bring).
#ifndef CB200_CHAINS
#define CB200_CHAINS 2
#endif
__host__ __device__ constexpr int chains_per_group(int nt) { return nt <= 2 ? CB200_CHAINS : 2; }
__device__ __forceinline__ constexpr int chain_of(int kc, int w, int h) {
  return kc == 2 ? h : (kc == 4 ? (w & 1) * 2 + h : 2 * w + h);
}
template <int kC>
__device__ __forceinline__ float chain_sum(const float (*part)[4], int e) {
  if (kC == 2) return part[0][e] + part[1][e];
  if (kC == 4) return (part[0][e] + part[1][e]) + (part[2][e] + part[3][e]);
  return ((part[0][e] + part[1][e]) + (part[2][e] + part[3][e])) +
         ((part[4][e] + part[5][e]) + (part[6][e] + part[7][e]));
}

// Offset sums: bias[g][n] = (sum over group g of 8 * x[n][k]) * 2^-69, for the
// 8*NT MMA columns n, written by the lanes that own row 0 of the fragment.
// The instruction sequence mirrors one_group() in consume_chunk exactly.
template <int NT>
__device__ __forceinline__ void build_bias(const std::uint8_t* xs, float* bias, int G, int rsx,
                                           int M, int warp, int lane, int nwarps) {
  const int r8 = lane >> 2, t = lane & 3;
  const std::uint8_t* xrow[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int n = nt * 8 + r8;
    xrow[nt] = xs + (n < M ? n : M) * rsx + t * 16;
  }
  for (int g = warp; g < G; g += nwarps) {
    constexpr int kC = chains_per_group(NT);
    float part[NT][kC][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < kC; ++c)
        part[nt][c][0] = part[nt][c][1] = part[nt][c][2] = part[nt][c][3] = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint4 b = lds128(xrow[nt] + g * 256 + w * 64);
        mma_m16n8k16_bf16(part[nt][chain_of(kC, w, 0)], kBiasEven, kBiasEven, kBiasOdd, kBiasOdd, b.x, b.y);
        mma_m16n8k16_bf16(part[nt][chain_of(kC, w, 1)], kBiasEven, kBiasEven, kBiasOdd, kBiasOdd, b.z, b.w);
      }
    }
    if (r8 == 0) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        bias[g * (NT * 8) + nt * 8 + 2 * t] = chain_sum<kC>(part[nt], 0);
        bias[g * (NT * 8) + nt * 8 + 2 * t + 1] = chain_sum<kC>(part[nt], 1);
      }
    }
  }
}

// One chunk of one m-tile: acc[nt][0..3] += sum over the chunk's groups (times
// 2^-69).  Fragment ownership (lane = 4*r8 + t): rows r8 and r8+8 of the
// m-tile, activation rows (columns of the MMA) nt*8 + 2t and nt*8 + 2t + 1.
template <int NT, int CG>
__device__ __forceinline__ void consume_chunk(const std::uint8_t* stage, const std::uint8_t* xs,
                                              const float* bias, int G, int g0, int cg, int rsx,
                                              int M, int lane, float (&acc)[NT][4]) {
  constexpr int RS = CG * 64;
  const int r8 = lane >> 2, t = lane & 3;
  const std::uint8_t* wa = stage + r8 * RS + t * 16;
  const std::uint8_t* wb = wa + 8 * RS;
  const std::uint8_t* sa = stage + kMTileRows * RS + (r8 * G + g0) * 2;
  const std::uint8_t* sb = sa + 8 * G * 2;
  const std::uint8_t* xrow[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int n = nt * 8 + r8;
    xrow[nt] = xs + (n < M ? n : M) * rsx + g0 * 256 + t * 16;
  }
  const float* brow = bias + g0 * (NT * 8) + 2 * t;
  auto one_group = [&](int g) {
    const uint4 qa = lds128(wa + g * 64);
    const uint4 qb = lds128(wb + g * 64);
    // (one 8-byte load for four groups' scales was measured slower: the sixteen values
    // that then live across the unrolled groups cost more than the loads they save)
    const float s_lo = __half2float(__ushort_as_half(lds16(sa + 2 * g)));
    const float s_hi = __half2float(__ushort_as_half(lds16(sb + 2 * g)));
    const std::uint32_t wordA[4] = {qa.x, qa.y, qa.z, qa.w};
    const std::uint32_t wordB[4] = {qb.x, qb.y, qb.z, qb.w};
    // several accumulation chains per column tile cut the MMA dependency depth
    constexpr int kC = chains_per_group(NT);
    float part[NT][kC][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < kC; ++c)
        part[nt][c][0] = part[nt][c][1] = part[nt][c][2] = part[nt][c][3] = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      std::uint32_t A[4], B[4];
      dequant_word(wordA[w], A);
      dequant_word(wordB[w], B);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint4 b = lds128(xrow[nt] + g * 256 + w * 64);
        mma_m16n8k16_bf16(part[nt][chain_of(kC, w, 0)], A[0], B[0], A[1], B[1], b.x, b.y);
        mma_m16n8k16_bf16(part[nt][chain_of(kC, w, 1)], A[2], B[2], A[3], B[3], b.z, b.w);
      }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const float2 b8 = *reinterpret_cast<const float2*>(brow + g * (NT * 8) + nt * 8);
      acc[nt][0] = fmaf(s_lo, chain_sum<kC>(part[nt], 0) - b8.x, acc[nt][0]);
      acc[nt][1] = fmaf(s_lo, chain_sum<kC>(part[nt], 1) - b8.y, acc[nt][1]);
      acc[nt][2] = fmaf(s_hi, chain_sum<kC>(part[nt], 2) - b8.x, acc[nt][2]);
      acc[nt][3] = fmaf(s_hi, chain_sum<kC>(part[nt], 3) - b8.y, acc[nt][3]);
    }
  };
  if (cg == CG) {
    // full chunk: unrolled so that the next group's loads overlap this group's math
    constexpr int kUnroll = (NT <= 2) ? CG : 1;
#pragma unroll kUnroll
    for (int g = 0; g < CG; ++g) one_group(g);
  } else {
    // a partial chunk (K = 3584: the last four of 28 groups): four groups at a time, so
    // that their loads and MMAs overlap as in a full chunk
    int g = 0;
    if (NT <= 2) {
      for (; g + 4 <= cg; g += 4) {
        one_group(g);
        one_group(g + 1);
        one_group(g + 2);
        one_group(g + 3);
      }
    }
    for (; g < cg; ++g) one_group(g);
  }
}

// ---------------------------------------------------------------------------
// Streaming kernel.  CTA_MAX (the vocabulary projection) additionally keeps, per
// activation row, the largest bf16-rounded output the CTA has produced and leaves it in
// the table that the token pick derives its bounds from (lm_head_pick.cuh).
// ---------------------------------------------------------------------------

// Shared-memory address of activation buffer b.  The offset goes through an
// opaque move so that loads from the buffer cannot be scheduled ahead of the
// wait that precedes this call.
__device__ __forceinline__ std::uint8_t* x_buffer(std::uint8_t* xs0, int x_bytes, int b) {
  int off = b * x_bytes;
  asm volatile("" : "+r"(off)::"memory");
  return xs0 + off;
}

// Barrier-free change of projection (two activation buffers; projection e
// lives in buffer e & 1).  Refills happen one at a time and in order:
// fill_claim and fill_done only grow, fill_claim == fill_done + 1 while a refill
// is under way.  Any warp may start the refill of e once e - 1 is in place and
// every warp is past e - 2, the buffer's previous tenant: it issues one bulk
// copy of the raw activations into the staging area.  After the copy has
// landed every warp, whenever it next looks (once per chunk), converts its
// share of the quantisation groups into the fragment layout and computes their
// offset sums; the last one publishes fill_done = e + 1.  No warp waits for
// another unless it actually needs the activations.
__device__ __forceinline__ void try_start_fill(const DescSource& ds, CtaControl* ctl,
                                               std::uint8_t* staging, int e, int d_first,
                                               int nwarps, int lane) {
  if (lane == 0 && ld_volatile_s32(&ctl->fill_claim) == e && ld_volatile_s32(&ctl->fill_done) == e) {
    bool free_now = true;
    if (e - 2 >= d_first)
      for (int w = 0; w < nwarps; ++w) free_now &= ld_volatile_s32(&ctl->cur_desc[w]) > e - 2;
    if (free_now && atomicCAS(&ctl->fill_claim, e, e + 1) == e) {
      const DescLite L = get_desc(ds, e);
      const std::uint32_t bytes = static_cast<std::uint32_t>(L.M) * L.K * 2u;
      std::uint64_t* bar = reinterpret_cast<std::uint64_t*>(&ctl->xbar);
      if ((reinterpret_cast<std::uintptr_t>(L.x) & 15u) == 0) {
        // earlier generic reads of the staging area come before the async write
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive_expect_tx(bar, bytes);
        bulk_g2s(staging, L.x, bytes, bar);
      } else {
        mbar_arrive_expect_tx(bar, 0);  // keeps the barrier's phase in step; shares are loaded directly
      }
    }
  }
  __syncwarp();
}

struct XFill {
  int part_done;  // latest projection this warp has converted its share of
};

// One look at the refill machinery.  Returns true when this warp did some work.
template <int NT>
__device__ __forceinline__ bool service_fill(const DescSource& ds, CtaControl* ctl,
                                             std::uint8_t* xs0, std::uint8_t* staging, XFill& xf,
                                             int d_own, int d_first, int d_last, int nwarps,
                                             int warp, int lane) {
  int dn = 0, c = 0;
  if (lane == 0) {
    dn = ld_volatile_s32(&ctl->fill_done);
    c = ld_volatile_s32(&ctl->fill_claim);
  }
  dn = __shfl_sync(0xffffffffu, dn, 0);
  c = __shfl_sync(0xffffffffu, c, 0);
  const int e = dn;
  if (c > dn) {
    // a refill of e is under way (had it completed between the two reads, this
    // warp's share would already be done)
    if (xf.part_done >= e) return false;
    std::uint64_t* bar = reinterpret_cast<std::uint64_t*>(&ctl->xbar);
    if (!mbar_try_wait(bar, static_cast<std::uint32_t>(e - d_first - 1) & 1u)) return false;
    const DescLite L = get_desc(ds, e);
    const int LK = L.K, LM = L.M, G = LK >> 7;
    const int rsx = 2 * LK + kXRowPad;
    std::uint8_t* xb = x_buffer(xs0, ds.p->x_bytes, e & 1);
    const bool staged = (reinterpret_cast<std::uintptr_t>(L.x) & 15u) == 0;
    bool bad = false;
    for (int g = warp; g < G; g += nwarps) {
      for (int n = 0; n < LM; ++n) {
        const int k = g * 128 + lane * 4;
        uint2 v;
        if (staged) {
          v = *reinterpret_cast<const uint2*>(staging + (static_cast<std::size_t>(n) * LK + k) * 2);
        } else {
          const std::uint16_t* src = L.x + static_cast<std::size_t>(n) * LK + k;
          v.x = static_cast<std::uint32_t>(__ldg(src)) | (static_cast<std::uint32_t>(__ldg(src + 1)) << 16);
          v.y = static_cast<std::uint32_t>(__ldg(src + 2)) | (static_cast<std::uint32_t>(__ldg(src + 3)) << 16);
        }
        bad |= span_out_of_range(abs_bits4(v));
        store_x_value(xb, rsx, n, k, static_cast<std::uint16_t>(v.x & 0xFFFFu));
        store_x_value(xb, rsx, n, k + 1, static_cast<std::uint16_t>(v.x >> 16));
        store_x_value(xb, rsx, n, k + 2, static_cast<std::uint16_t>(v.y & 0xFFFFu));
        store_x_value(xb, rsx, n, k + 3, static_cast<std::uint16_t>(v.y >> 16));
      }
      // the all-zero row's part of this group
      *reinterpret_cast<uint2*>(xb + LM * rsx + g * 256 + lane * 8) = make_uint2(0u, 0u);
    }
    if (bad && lane == 0) st_volatile_s32(x_flag_word(xb, ds.p->x_bytes), e + 1);
    __syncwarp();
    build_bias<NT>(xb, reinterpret_cast<float*>(xb + (LM + 1) * rsx), G, rsx, LM, warp, lane, nwarps);
    __threadfence_block();
    __syncwarp();
    xf.part_done = e;
    if (lane == 0 && atomicAdd(&ctl->fill_parts, 1) == nwarps - 1) {
      st_volatile_s32(&ctl->fill_parts, 0);
      __threadfence_block();
      st_volatile_s32(&ctl->fill_done, e + 1);
    }
    return true;
  }
  // nothing under way: start the next refill if it is due.  While this warp
  // itself still reads the buffer's previous tenant there is no point in
  // looking at the other warps.
  if (e <= d_last && d_own > e - 2) try_start_fill(ds, ctl, staging, e, d_first, nwarps, lane);
  return false;
}

// Works on refills until every projection up to d is in place.  False when a
// bounded wait ran out.
template <int NT>
__device__ __forceinline__ bool wait_x_ready(const DescSource& ds, CtaControl* ctl,
                                             std::uint8_t* xs0, std::uint8_t* staging, XFill& xf,
                                             int d, int d_own, int d_first, int d_last,
                                             int nwarps, int warp, int lane) {
  unsigned long long t0 = 0;
  for (int spin = 0;; ++spin) {
    int done = 0;
    if (lane == 0) done = ld_volatile_s32(&ctl->fill_done);
    done = __shfl_sync(0xffffffffu, done, 0);
    if (done > d) {
      __threadfence_block();
      return true;
    }
    if (service_fill<NT>(ds, ctl, xs0, staging, xf, d_own, d_first, d_last, nwarps, warp, lane))
      continue;
    __nanosleep(64);
    if ((spin & 1023) == 1023) {
      unsigned long long t1;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
      if (t0 == 0) t0 = t1;
      else if (t1 - t0 > 2000000000ull) return false;
    }
  }
}

// NPROD = 0: every warp feeds itself.  NPROD > 0 (= NWARPS / 4): the NWARPS
// consumer warps only compute; NPROD further warps issue the copies, one thread
// each for four consumers, as soon as a consumer hands a stage back through its
// "empty" mbarrier (issuing a chunk's copies costs a warp several hundred cycles).
// EXTRA: the launch may hold a pair (silu(gate) * up) or a projection with a
// residual; plain launches are compiled without any of that.
template <int NT, int CG, int NWARPS, bool CTA_MAX, int NPROD, bool EXTRA>
__global__ void __launch_bounds__((NWARPS + NPROD) * 32, 1)
w4a16_stream_kernel(const __grid_constant__ StreamParams p) {
  extern __shared__ __align__(128) std::uint8_t smem[];
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int depth = p.depth;
  const bool async_switch = p.x_buffers == 2;
  // barrier over the consumer warps only
  auto consumer_sync = [&]() {
    if (NPROD == 0) __syncthreads();
    else asm volatile("bar.sync 1, %0;" ::"r"(NWARPS * 32) : "memory");
  };

  // shared memory: [barriers, control][activation buffers][NWARPS rings of `depth` stages]
  std::uint64_t* all_full = reinterpret_cast<std::uint64_t*>(smem);
  std::uint64_t* all_empty = reinterpret_cast<std::uint64_t*>(smem + kHeaderBytes - kMaxWarps * kMaxDepth * 8);
  std::uint64_t* bars = all_full + (warp < NWARPS ? warp : 0) * kMaxDepth;
  std::uint64_t* ebars = all_empty + (warp < NWARPS ? warp : 0) * kMaxDepth;
  CtaControl* ctl = reinterpret_cast<CtaControl*>(smem + kMaxWarps * kMaxDepth * 8);
  std::uint8_t* xs0 = smem + kHeaderBytes;
  // the staging area of the barrier-free change of projection follows the two buffers
  std::uint8_t* staging = xs0 + 2 * static_cast<std::size_t>(p.x_bytes);
  std::uint8_t* rings = xs0 + static_cast<std::size_t>(p.x_buffers) * p.x_bytes +
                        (async_switch ? kAsyncFillMaxValues * 2 : 0);
  std::uint8_t* ring = rings + static_cast<std::size_t>(warp < NWARPS ? warp : 0) * depth * p.stage_bytes;

  // this CTA's contiguous range of m-tiles: an equal share of the launch's work
  int mt_lo, mt_hi, d_first;
  if (p.cta_ranges) {
    const int2 r0 = p.cta_ranges[blockIdx.x], r1 = p.cta_ranges[blockIdx.x + 1];
    mt_lo = r0.x;
    d_first = r0.y;
    mt_hi = r1.x;
  } else {
    mt_lo = mtile_at_cost<CG>(p, static_cast<long long>(blockIdx.x) * p.total_cost / gridDim.x);
    mt_hi = mtile_at_cost<CG>(p, static_cast<long long>(blockIdx.x + 1) * p.total_cost / gridDim.x);
    d_first = mt_lo < mt_hi ? find_desc(p, mt_lo) : p.n_desc;
  }
  if (mt_lo >= mt_hi) d_first = p.n_desc;

  if (lane == 0 && warp < NWARPS) {
    for (int s = 0; s < depth; ++s) {
      mbar_init(&bars[s], 1);
      if (NPROD > 0) mbar_init(&ebars[s], 1);
    }
    mbar_init_fence();
  }
  if (tid < NWARPS) ctl->issued[tid] = 0;
  if (tid == 0) {
    *x_flag_word(xs0, p.x_bytes) = 0;
    if (async_switch) *x_flag_word(xs0 + p.x_bytes, p.x_bytes) = 0;
    ctl->fill_claim = ctl->fill_done = d_first;
    ctl->fill_parts = 0;
    ctl->abort = 0;
    mbar_init(reinterpret_cast<std::uint64_t*>(&ctl->xbar), 1);
    mbar_init_fence();
  }
  if (tid < NWARPS) ctl->cur_desc[tid] = d_first;
  if (CTA_MAX && tid < kMaxPassRows) ctl->row_key[tid] = 0u;
  if (tid < kDescCache) {
    // descriptors are written when a launch is set up, never by a kernel, so
    // they may be read before the wait on the previous grid
    const int d = d_first + tid;
    DescLite v{nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
               0,       0,       0,       0x7fffffff, 0, 0};
    if (d < p.n_desc) {
      const LinearDev* L = desc_table(p) + d;
      v = DescLite{&L->tmap, &L->tmap2, L->W, L->W2, L->S, L->S2, L->res, L->x, L->y,
                   L->N,     L->K,      L->M,  L->mt_begin, L->flags, 0};
    }
    ctl->desc[tid] = v;
  }
  __syncthreads();
  const DescSource ds{&p, ctl->desc, d_first};

  const std::uint64_t policy = policy_evict_first();

  if (NPROD > 0 && warp >= NWARPS) {
    // ---------------- producer: one thread feeds four consumer warps ----------------
    // It touches only weights and scales, constants of the model, so it does not
    // wait for the previous grid either.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (lane != 0 || d_first >= p.n_desc) return;
    const int w0 = (warp - NWARPS) * 4;
    Cursor<CG> pc[4];
    int taken[4], pslot[4], nissued[4];
    std::uint32_t pphase[4];
    int live = 0;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      pc[c].valid = false;
      pc[c].bind(ds, d_first);
      taken[c] = 1;
      pslot[c] = 0;
      pphase[c] = 1;  // a fresh barrier reads as "phase 1 complete": the first round does not wait
      nissued[c] = 0;
      const int m = mt_lo + w0 + c;
      pc[c].seek(ds, m < mt_hi ? m : mt_hi, mt_hi);
      live += pc[c].valid ? 1 : 0;
    }
    unsigned long long t0 = 0;
    int idle = 0;
    while (live > 0) {
      bool progressed = false;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        if (!pc[c].valid) continue;
        std::uint64_t* eb = all_empty + (w0 + c) * kMaxDepth + pslot[c];
        if (!mbar_try_wait(eb, pphase[c])) continue;
        std::uint8_t* st = rings + (static_cast<std::size_t>(w0 + c) * depth + pslot[c]) * p.stage_bytes;
        issue_item_single<CG, EXTRA>(pc[c], st, all_full + (w0 + c) * kMaxDepth + pslot[c], policy);
        st_volatile_s32(&ctl->issued[w0 + c], ++nissued[c]);
        if (++pslot[c] == depth) {
          pslot[c] = 0;
          pphase[c] ^= 1u;
        }
        if (++pc[c].chunk >= (EXTRA ? pc[c].nch_total : pc[c].nch)) {
          const int m = mt_lo + w0 + c + taken[c] * NWARPS;
          ++taken[c];
          pc[c].seek(ds, m < mt_hi ? m : mt_hi, mt_hi);
          if (!pc[c].valid) --live;
        }
        progressed = true;
      }
      if (progressed) {
        idle = 0;
        t0 = 0;
        continue;
      }
      // nothing to do: a bounded, abort-aware pause
      if (++idle >= 64) {
        idle = 0;
        if (ld_volatile_s32(&ctl->abort)) return;
        unsigned long long t1;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
        if (t0 == 0) t0 = t1;
        else if (t1 - t0 > 4000000000ull) {
          atomicExch(p.status, CUDALM_B200_ERR_TIMEOUT);
          return;
        }
        __nanosleep(32);
      }
    }
    return;
  }

  // Two cursors over this warp's m-tiles (mt_lo + warp, + NWARPS, ...): `fc`
  // runs ahead issuing copies, `cc` consumes.  (Handing m-tiles out dynamically
  // from a shared counter was measured slower: the atomic per m-tile costs more
  // than the better balance brings.)
  Cursor<CG> fc, cc;
  fc.valid = false;
  if (d_first < p.n_desc) fc.bind(ds, d_first);
  cc = fc;
  int fc_taken = 0, cc_taken = 0;
  auto fc_next_mtile = [&]() {
    const int m = mt_lo + warp + fc_taken * NWARPS;
    ++fc_taken;
    fc.seek(ds, m < mt_hi ? m : mt_hi, mt_hi);
  };
  auto cc_next_mtile = [&]() {
    const int m = mt_lo + warp + cc_taken * NWARPS;
    ++cc_taken;
    cc.seek(ds, m < mt_hi ? m : mt_hi, mt_hi);
  };
  auto fc_advance = [&]() {
    if (++fc.chunk < (EXTRA ? fc.nch_total : fc.nch)) return;
    fc_next_mtile();
  };

  // Weights and scales are constants of the model: their first copies go out
  // before this grid waits for its predecessor in the stream, so they overlap
  // the predecessor's tail.  Activations and outputs are touched only after.
  int in_flight = 0;  // self-feeding form: stages issued and not yet consumed
  int consumed = 0;   // producer form: stages consumed so far
  if (d_first < p.n_desc) {
    if (NPROD == 0) {
      fc_next_mtile();
      for (int s = 0; s < depth && fc.valid; ++s) {
        issue_item<CG, EXTRA>(fc, ring + s * p.stage_bytes, &bars[s], lane, policy);
        fc_advance();
        ++in_flight;
      }
    }
    cc_next_mtile();
  }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  int slot = 0;              // stage the next item arrives in
  std::uint32_t parity = 0;  // phase of that stage's barrier

  float vmax[NT][2];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) vmax[nt][0] = vmax[nt][1] = -INFINITY;

  bool dead = false;     // a wait ran out: stop computing, keep attending barriers
  XFill xf{d_first};
  // last projection of this CTA's range
  int d_last = d_first;
  while (d_last + 1 < p.n_desc && get_desc(ds, d_last + 1).mt_begin < mt_hi) ++d_last;
  for (int d = d_first; d < p.n_desc; ++d) {
    const DescLite L = get_desc(ds, d);
    if (L.mt_begin >= mt_hi) break;
    const int LN = L.N, LK = L.K, LM = L.M;
    const int rsx = 2 * LK + kXRowPad;
    const int G = LK >> 7;
    std::uint16_t* y = L.y;
    std::uint8_t* xs;
    if (!async_switch || d == d_first) {
      // the whole CTA refills the buffer together
      consumer_sync();  // every warp is done with the previous activations
      xs = x_buffer(xs0, p.x_bytes, async_switch ? (d & 1) : 0);
      fill_x_fragments<4>(xs, L.x, LM, LK, rsx, tid, NWARPS * 32, x_flag_word(xs, p.x_bytes), d + 1);
      consumer_sync();
      build_bias<NT>(xs, reinterpret_cast<float*>(xs + (LM + 1) * rsx), G, rsx, LM, warp, lane,
                     NWARPS);
      if (async_switch && tid == 0) {
        ctl->fill_claim = d + 1;
        ctl->fill_done = d + 1;
      }
      consumer_sync();
    } else {
      // this warp is past every earlier projection, whether it has work here or not
      __threadfence_block();  // this warp's reads of the earlier activations come first
      __syncwarp();
      if (lane == 0) st_volatile_s32(&ctl->cur_desc[warp], d);
      if (!(cc.valid && cc.d == d)) continue;
      if (!dead &&
          !wait_x_ready<NT>(ds, ctl, xs0, staging, xf, d, d, d_first, d_last, NWARPS, warp, lane)) {
        dead = true;
        if (lane == 0) {
          atomicExch(p.status, CUDALM_B200_ERR_TIMEOUT);
          st_volatile_s32(&ctl->abort, 1);
        }
      }
      xs = x_buffer(xs0, p.x_bytes, d & 1);
    }
    const float* bias = reinterpret_cast<const float*>(xs + (LM + 1) * rsx);
    // activations outside the range of the tiny-number arithmetic: see slow_mtile
    const bool odd = ld_volatile_s32(x_flag_word(xs, p.x_bytes)) == d + 1;

    while (cc.valid && cc.d == d) {
      float acc[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
      const int row0 = (cc.mt - cc.mt_begin) * kMTileRows;
      const int nch = cc.nch, nch_total = EXTRA ? cc.nch_total : cc.nch;
      // a pair's first (gate) outputs, rounded to bf16, while the second matrix streams
      constexpr int kGateTiles = (EXTRA && NT <= 2) ? NT : 1;
      float gate[kGateTiles][4];
      for (int chunk = 0; chunk < nch_total; ++chunk) {
        if (EXTRA) cc.chunk = chunk;
        const int ch = (EXTRA && chunk >= nch) ? chunk - nch : chunk;
        if (EXTRA && NT <= 2 && chunk == nch) {
#pragma unroll
          for (int nt = 0; nt < kGateTiles; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              gate[nt][i] = bf16_bits_to_float(float_to_bf16_bits(acc[nt][i] * CB200_OUT_SCALE));
              acc[nt][i] = 0.f;
            }
        }
        std::uint8_t* stage = ring + slot * p.stage_bytes;
        if (!dead && !wait_stage(&bars[slot], parity)) {
          dead = true;
          if (lane == 0) {
            atomicExch(p.status, CUDALM_B200_ERR_TIMEOUT);
            st_volatile_s32(&ctl->abort, 1);
          }
        }
        if (!dead) {
          const int g0 = ch * CG;
          if (NPROD > 0 && !stage_scales_bulk<CG, EXTRA>(cc)) {
            // a ragged or unaligned scale block, which the producer leaves to the reader
            const int srow0 = (cc.mt - cc.mt_begin) * kMTileRows;
            const int n_sc = min(kMTileRows, cc.N - srow0) * cc.G;
            const std::uint16_t* ssrc = (EXTRA ? cc.cur_scales() : cc.S) + static_cast<std::size_t>(srow0) * cc.G;
            std::uint16_t* sdst = reinterpret_cast<std::uint16_t*>(stage + kMTileRows * CG * 64);
            for (int i = lane; i < n_sc; i += 32) sdst[i] = __ldg(ssrc + i);
            __syncwarp();
          }
          consume_chunk<NT, CG>(stage, xs, bias, G, g0, min(CG, G - g0), rsx, LM, lane, acc);
          __syncwarp();
          if (NPROD > 0) {
            ++consumed;
            if (lane == 0) mbar_arrive(&ebars[slot]);  // hands the stage back to the producer
          } else {
            --in_flight;
            if (fc.valid) {
              issue_item<CG, EXTRA>(fc, stage, &bars[slot], lane, policy);
              fc_advance();
              ++in_flight;
            }
          }
          if (async_switch) {
            (void)service_fill<NT>(ds, ctl, xs0, staging, xf, d, d_first, d_last, NWARPS, warp, lane);
          }
        }
        if (++slot == depth) {
          slot = 0;
          parity ^= 1u;
        }
      }
      cc_next_mtile();
      float out_scale = CB200_OUT_SCALE;
      if (odd && !dead) {
        out_scale = 1.0f;
        if (EXTRA && NT <= 2 && (L.flags & kFlagPair)) {
          float g[NT][4];
          slow_mtile<NT>(L.W, L.S, L.x, LN, LK, LM, row0, lane, g);
#pragma unroll
          for (int nt = 0; nt < kGateTiles; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) gate[nt][i] = bf16_bits_to_float(float_to_bf16_bits(g[nt][i]));
          slow_mtile<NT>(L.W2, L.S2, L.x, LN, LK, LM, row0, lane, acc);
        } else {
          slow_mtile<NT>(L.W, L.S, L.x, LN, LK, LM, row0, lane, acc);
        }
      }
      if (!dead) {
        const int r8 = lane >> 2, t = lane & 3;
        const int row_lo = row0 + r8, row_hi = row_lo + 8;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int col = nt * 8 + 2 * t;
          std::uint16_t o0 = float_to_bf16_bits(acc[nt][0] * out_scale);
          std::uint16_t o1 = float_to_bf16_bits(acc[nt][1] * out_scale);
          std::uint16_t o2 = float_to_bf16_bits(acc[nt][2] * out_scale);
          std::uint16_t o3 = float_to_bf16_bits(acc[nt][3] * out_scale);
          if (EXTRA && NT <= 2 && (L.flags & kFlagPair)) {
            // CUDALM's rounding order (src/kernels/qwen35_kernels.cu:459-476):
            // s = bf16(g / (1 + exp(-g))), then bf16(float(s) * float(u))
            const int gi = nt < kGateTiles ? nt : 0;
            o0 = silu_mul_bits(gate[gi][0], o0);
            o1 = silu_mul_bits(gate[gi][1], o1);
            o2 = silu_mul_bits(gate[gi][2], o2);
            o3 = silu_mul_bits(gate[gi][3], o3);
          } else if (EXTRA && (L.flags & kFlagResidual)) {
            // bf16(float(residual) + float(projection)) (src/kernels/qwen35_kernels.cu:442-456)
            const std::uint16_t* res = L.res;
            if (col < LM) {
              if (row_lo < LN) o0 = add_bits(res[static_cast<std::size_t>(col) * LN + row_lo], o0);
              if (row_hi < LN) o2 = add_bits(res[static_cast<std::size_t>(col) * LN + row_hi], o2);
            }
            if (col + 1 < LM) {
              if (row_lo < LN) o1 = add_bits(res[static_cast<std::size_t>(col + 1) * LN + row_lo], o1);
              if (row_hi < LN) o3 = add_bits(res[static_cast<std::size_t>(col + 1) * LN + row_hi], o3);
            }
          }
          if (col < LM) {
            if (row_lo < LN) y[static_cast<std::size_t>(col) * LN + row_lo] = o0;
            if (row_hi < LN) y[static_cast<std::size_t>(col) * LN + row_hi] = o2;
          }
          if (col + 1 < LM) {
            if (row_lo < LN) y[static_cast<std::size_t>(col + 1) * LN + row_lo] = o1;
            if (row_hi < LN) y[static_cast<std::size_t>(col + 1) * LN + row_hi] = o3;
          }
          if (CTA_MAX) {
            if (row_lo < LN) {
              vmax[nt][0] = fmaxf(vmax[nt][0], bf16_bits_to_float(o0));
              vmax[nt][1] = fmaxf(vmax[nt][1], bf16_bits_to_float(o1));
            }
            if (row_hi < LN) {
              vmax[nt][0] = fmaxf(vmax[nt][0], bf16_bits_to_float(o2));
              vmax[nt][1] = fmaxf(vmax[nt][1], bf16_bits_to_float(o3));
            }
          }
        }
      }
    }
  }
  // done: this warp holds neither activation buffer any more
  __threadfence_block();
  __syncwarp();
  if (lane == 0) st_volatile_s32(&ctl->cur_desc[warp], 0x7fffffff);
  // the other warps may still need this warp's share of later refills
  if (async_switch && d_first < p.n_desc && !dead &&
      !wait_x_ready<NT>(ds, ctl, xs0, staging, xf, d_last, 0x7fffffff, d_first, d_last, NWARPS, warp,
                        lane)) {
    dead = true;
    if (lane == 0) {
      atomicExch(p.status, CUDALM_B200_ERR_TIMEOUT);
      st_volatile_s32(&ctl->abort, 1);
    }
  }
  if (dead) {
    // Give copies still in flight a bounded chance to land before the CTA's
    // shared memory is released.
    if (NPROD > 0) {
      __nanosleep(2000);  // the producer stops at the abort flag
      in_flight = ld_volatile_s32(&ctl->issued[warp]) - consumed;
    }
    for (int i = 0; i < in_flight; ++i) {
      (void)wait_stage(&bars[slot], parity);
      if (++slot == depth) {
        slot = 0;
        parity ^= 1u;
      }
    }
  }

  if (CTA_MAX) {
    // This CTA's largest outputs per activation row into its slots of the table that the
    // follow-up launch derives the rows' bounds from: reduce over the eight row-lanes
    // that share a column pair, then over the warps (shared-memory maxima of keys).
    const int M = desc_table(p)->M;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float v = vmax[nt][c];
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
        const int col = nt * 8 + 2 * lane + c;
        if (lane < 4 && col < M && col < kMaxPassRows)
          atomicMax(&ctl->row_key[col], order_key(float_to_bf16_bits(v)) + 1u);
      }
    }
    consumer_sync();
    if (tid < 32) tail_publish(p.pick, ctl->row_key, tid);
  }
}

#endif  // __CUDACC__

}  // namespace cb200
