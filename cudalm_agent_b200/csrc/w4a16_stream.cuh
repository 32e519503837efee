// Building blocks of the streaming W4A16 kernels.
//
// Work unit: an "m-tile" = 16 consecutive output rows of one projection, cut
// along K into chunks of CG quantisation groups (CG*128 values of k).  Each
// warp owns whole m-tiles and feeds itself: it keeps a private ring of `depth`
// shared-memory stages, fills a stage with bulk async copies (one per weight
// row segment plus one for the m-tile's scales) that complete on the stage's
// mbarrier, and refills the stage as soon as it has consumed it.  Nothing but
// the activation vector is shared between warps, so the only CTA-wide
// synchronisation is at a change of projection.
//
// Stage layout: 16 row segments at a stride of RS = CG*64 + 64 bytes (the extra
// 64 bytes put rows 2p and 2p+1 in different halves of a 128-byte bank line, so
// the fragment loads below are conflict free), then the m-tile's scale block
// fp16 [16][K/128].
//
// Arithmetic: the 4-bit values become exact bf16 integers in registers and go
// through mma.sync m16n8k16 (weights = the 16-row operand, up to 8 activation
// rows = the 8 columns), one quantisation group at a time into a group
// accumulator; the group's fp32 sum is then folded in as acc += scale * sum.
// Products are exact (4-bit x 8-bit significands) and all sums are fp32.
#pragma once

#include "common.cuh"

#ifndef CB200_LOADER
#define CB200_LOADER 0  // 0: one bulk copy per weight row segment (product); 1, 2: experiments
#endif

namespace cb200 {

constexpr int kMTileRows = 16;
constexpr int kMaxDepth = 4;

enum : int { kFlagScalesBulk = 1 };

// Device-side projection descriptor.
struct LinearDev {
  const std::uint8_t* W;
  const std::uint16_t* S;
  const std::uint16_t* x;
  std::uint16_t* y;
  int N, K, M;
  int mt_begin;    // index of this projection's first m-tile in the launch
  int flags;
  int cost_begin;  // chunks (m-tiles x chunks per m-tile) before this projection
};

struct StreamParams {
  const LinearDev* table;  // device table, or nullptr to use `inl`
  LinearDev inl[CUDALM_B200_MAX_INLINE_LINEARS];
  int n_desc;
  int total_mt;
  int total_cost;   // chunks in the whole launch
  int depth;        // stages per warp ring, 2..kMaxDepth
  int stage_bytes;  // 16*RS + scale block of the largest K
  int x_bytes;      // activation region
  int* status;      // device status word
  float* cta_max;   // [gridDim.x][M] when the kernel is built with CTA_MAX
};

#ifdef __CUDACC__

__device__ __forceinline__ LinearDev load_desc(const StreamParams& p, int d) {
  const LinearDev* tbl = p.table ? p.table : p.inl;
  return tbl[d];
}

__device__ __forceinline__ int desc_mtiles(int N) { return (N + kMTileRows - 1) / kMTileRows; }

// Descriptor that holds m-tile `mt` (binary search over mt_begin).
__device__ __forceinline__ int find_desc(const StreamParams& p, int mt) {
  const LinearDev* tbl = p.table ? p.table : p.inl;
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
  const LinearDev* tbl = p.table ? p.table : p.inl;
  int lo = 0, hi = p.n_desc - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (tbl[mid].cost_begin <= cost) lo = mid; else hi = mid - 1;
  }
  const int nch = ((tbl[lo].K >> 7) + CG - 1) / CG;
  const int within = static_cast<int>(cost) - tbl[lo].cost_begin;
  return tbl[lo].mt_begin + (within + nch - 1) / nch;
}

// Position of a warp in its own list of (m-tile, chunk) items.
template <int CG>
struct Cursor {
  int d, mt, chunk;
  int mt_begin, mt_end, nch, N, K, flags;
  const std::uint8_t* W;
  const std::uint16_t* S;
  bool valid;

  __device__ __forceinline__ void bind(const StreamParams& p, int dd) {
    const LinearDev L = load_desc(p, dd);
    d = dd;
    mt_begin = L.mt_begin;
    mt_end = L.mt_begin + desc_mtiles(L.N);
    N = L.N;
    K = L.K;
    flags = L.flags;
    W = L.W;
    S = L.S;
    nch = ((L.K >> 7) + CG - 1) / CG;
  }
  __device__ __forceinline__ void start(const StreamParams& p, int mt0, int mt_hi) {
    mt = mt0;
    chunk = 0;
    valid = mt0 < mt_hi;
    if (valid) bind(p, find_desc(p, mt0));
  }
  // Next item of this warp: next chunk, else the warp's next m-tile (`stride`
  // m-tiles further on), moving to a later projection when needed.
  __device__ __forceinline__ void advance(const StreamParams& p, int stride, int mt_hi) {
    if (++chunk < nch) return;
    chunk = 0;
    mt += stride;
    if (mt >= mt_hi) {
      valid = false;
      return;
    }
    while (mt >= mt_end) bind(p, d + 1);
  }
};

// Starts the copies that fill `stage` with the cursor's item.
template <int CG>
__device__ __forceinline__ void issue_item(const Cursor<CG>& c, std::uint8_t* stage,
                                           std::uint64_t* bar, int lane,
                                           std::uint64_t policy) {
  constexpr int RS = CG * 64 + 64;
  const int row0 = (c.mt - c.mt_begin) * kMTileRows;
  const int rows = min(kMTileRows, c.N - row0);
  const int G = c.K >> 7;
  const int g0 = c.chunk * CG;
  const int cg = min(CG, G - g0);
  const std::uint32_t seg = static_cast<std::uint32_t>(cg) * 64u;
  const std::uint32_t sbytes = static_cast<std::uint32_t>(rows * G) * 2u;
  const std::uint16_t* ssrc = c.S + static_cast<std::size_t>(row0) * G;
  const bool sbulk = (c.flags & kFlagScalesBulk) && ((sbytes & 15u) == 0u);
  std::uint8_t* sdst = stage + kMTileRows * RS;
  if (!sbulk) {
    // ragged scale block (or an unaligned scale base): plain loads
    for (int i = lane; i < rows * G; i += 32)
      reinterpret_cast<std::uint16_t*>(sdst)[i] = __ldg(ssrc + i);
  }
#if CB200_LOADER == 2
  // experiment: per-thread 16-byte async copies (LDGSTS), one commit group per stage
  {
    (void)bar; (void)policy;
    if (sbulk) {
      for (int i = lane; i < rows * G; i += 32)
        reinterpret_cast<std::uint16_t*>(sdst)[i] = __ldg(ssrc + i);
    }
    const int per_row = static_cast<int>(seg) >> 4;
    const int pieces = rows * per_row;
    for (int pidx = lane; pidx < pieces; pidx += 32) {
      const int r = pidx / per_row, cidx = pidx - r * per_row;
      const std::uint8_t* src = c.W + static_cast<std::size_t>(row0 + r) * (c.K >> 1) + g0 * 64 + cidx * 16;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(stage + r * RS + cidx * 16)), "l"(src) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    return;
  }
#endif
  // order this warp's earlier reads of the stage before the async writes
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();
#if CB200_LOADER == 1
  // experiment: one contiguous copy when the chunk spans whole rows
  if (seg == static_cast<std::uint32_t>(c.K >> 1)) {
    if (lane == 0) {
      mbar_arrive_expect_tx(bar, static_cast<std::uint32_t>(rows) * seg + (sbulk ? sbytes : 0u));
      bulk_g2s_hint(stage, c.W + static_cast<std::size_t>(row0) * (c.K >> 1), rows * seg, bar, policy);
      if (sbulk) bulk_g2s(sdst, ssrc, sbytes, bar);
    }
    return;
  }
#endif
  if (lane == 0)
    mbar_arrive_expect_tx(bar, static_cast<std::uint32_t>(rows) * seg + (sbulk ? sbytes : 0u));
  __syncwarp();
  if (lane < rows) {
#ifdef CB200_NO_L2_HINT
    bulk_g2s(stage + lane * RS,
             c.W + static_cast<std::size_t>(row0 + lane) * (c.K >> 1) + g0 * 64, seg, bar);
#else
    bulk_g2s_hint(stage + lane * RS,
                  c.W + static_cast<std::size_t>(row0 + lane) * (c.K >> 1) + g0 * 64, seg,
                  bar, policy);
#endif
  } else if (lane == kMTileRows && sbulk) {
    bulk_g2s(sdst, ssrc, sbytes, bar);
  }
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

// Activation layout in shared memory for the MMA fragments: row n at stride
// rsx = 2K + 32 bytes; inside a row the values are permuted so that the four
// values a lane needs for one MMA are 8 contiguous bytes:
//   k = 128 g + 32 t + 8 w + i   (t = lane & 3, w = word of the lane's 16 weight
//   bytes, i = nibble in the word) goes to slot ((g*8 + j)*4 + t)*4 + e with
//   j = 2w + ((i & 3) >> 1), e = 2*(i & 1) + (i >> 2).
// Row M (one past the real rows) is all zeros: MMA columns beyond M read it, so
// the fragment loads need no predicate.
//
// kDequant == 1 stores the activations scaled by 2^100 (even nibbles) or 2^96
// (odd nibbles), both exact in bf16, to match dequant_word_tiny below.
template <int DQ>
__device__ __forceinline__ void fill_x_fragments(std::uint8_t* xs, const std::uint16_t* x,
                                                 int M, int K, int rsx, int tid,
                                                 int nthreads) {
  const int total = M * K;
  for (int idx = tid; idx < total; idx += nthreads) {
    const int n = idx / K;
    const int k = idx - n * K;
    std::uint16_t v = __ldg(x + idx);
    const int g = k >> 7, r = k & 127, t = r >> 5, q = r & 31, w = q >> 3, i = q & 7;
    const int j = 2 * w + ((i & 3) >> 1);
    const int e = 2 * (i & 1) + (i >> 2);
    if (DQ == 1) {
      const float f = bf16_bits_to_float(v) * ((i & 1) ? 0x1p96f : 0x1p100f);
      v = float_to_bf16_bits(f);
    }
    *reinterpret_cast<std::uint16_t*>(xs + n * rsx + ((((g * 8 + j) * 4 + t) * 4 + e) * 2)) = v;
  }
  for (int idx = tid; idx < K / 2; idx += nthreads)
    *reinterpret_cast<std::uint32_t*>(xs + M * rsx + idx * 4) = 0u;
}

// Dequantisation through bf16's tiny numbers.  A bf16 whose high byte is zero
// is the integer in its low byte times 2^-133 (the subnormals run on linearly
// into the first normal binade), so (w & 0x000F000F) and (w & 0x00F000F0) are
// already bf16 pairs holding n * 2^-133 and 16 n * 2^-133: four of the eight
// nibbles need no shift.  XOR 8 (folded into the same LOP3) and an exact
// subtraction of 8 (or 128) units give q * 2^-133 and 16 q * 2^-133.  The
// activations are pre-scaled by 2^100 and 2^96 to compensate, and the group sum
// comes out scaled by 2^-33, which the scale multiplication undoes.
__device__ __forceinline__ void dequant_word_tiny(std::uint32_t w, std::uint32_t (&out)[4]) {
  const std::uint32_t w8 = w >> 8;
  out[0] = sub_bf16x2(lop3_and_xor(w, 0x000F000Fu, 0x00080008u), 0x00080008u);
  out[1] = sub_bf16x2(lop3_and_xor(w, 0x00F000F0u, 0x00800080u), 0x00800080u);
  out[2] = sub_bf16x2(lop3_and_xor(w8, 0x000F000Fu, 0x00080008u), 0x00080008u);
  out[3] = sub_bf16x2(lop3_and_xor(w8, 0x00F000F0u, 0x00800080u), 0x00800080u);
}

// One chunk of one m-tile: acc[nt][0..3] += sum over the chunk's groups.
// Fragment ownership (lane = 4*r8 + t): rows r8 and r8+8 of the m-tile,
// activation rows (columns of the MMA) nt*8 + 2t and nt*8 + 2t + 1.
template <int NT, int CG, int DQ>
__device__ __forceinline__ void consume_chunk(std::uint32_t stage, std::uint32_t xs, int G,
                                              int g0, int cg, int rsx, int M, int lane,
                                              float (&acc)[NT][4]) {
  constexpr int RS = CG * 64 + 64;
  const int r8 = lane >> 2, t = lane & 3;
  const std::uint32_t wa = stage + r8 * RS + t * 16;
  const std::uint32_t wb = wa + 8 * RS;
  const std::uint32_t sa = stage + kMTileRows * RS + (r8 * G + g0) * 2;
  const std::uint32_t sb = sa + 8 * G * 2;
  std::uint32_t xrow[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int n = nt * 8 + r8;
    xrow[nt] = xs + (n < M ? n : M) * rsx + g0 * 256 + t * 8;
  }
#ifdef CB200_SKIP_COMPUTE  // measurement aid: touch the stage, do no arithmetic
  {
    const uint4 qa = lds128(wa);
    acc[0][0] += __uint_as_float(qa.x & 1u);
    return;
  }
#endif
  auto one_group = [&](int g) {
    const uint4 qa = lds128(wa + g * 64);
    const uint4 qb = lds128(wb + g * 64);
    float s_lo = __half2float(__ushort_as_half(lds16(sa + 2 * g)));
    float s_hi = __half2float(__ushort_as_half(lds16(sb + 2 * g)));
    if (DQ == 1) {
      s_lo *= 0x1p33f;
      s_hi *= 0x1p33f;
    }
    const std::uint32_t wordA[4] = {qa.x, qa.y, qa.z, qa.w};
    const std::uint32_t wordB[4] = {qb.x, qb.y, qb.z, qb.w};
    // two accumulation chains per column tile halve the MMA dependency depth
    float part[NT][2][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < 2; ++c)
        part[nt][c][0] = part[nt][c][1] = part[nt][c][2] = part[nt][c][3] = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      std::uint32_t A[4], B[4];
      if (DQ == 1) {
        dequant_word_tiny(wordA[w], A);
        dequant_word_tiny(wordB[w], B);
      } else {
        dequant_word_bf16x2(wordA[w], A);
        dequant_word_bf16x2(wordB[w], B);
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int j = 2 * w + h;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint2 b = lds64(xrow[nt] + g * 256 + j * 32);
          mma_m16n8k16_bf16(part[nt][h], A[2 * h], B[2 * h], A[2 * h + 1], B[2 * h + 1], b.x, b.y);
        }
      }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      acc[nt][0] = fmaf(s_lo, part[nt][0][0] + part[nt][1][0], acc[nt][0]);
      acc[nt][1] = fmaf(s_lo, part[nt][0][1] + part[nt][1][1], acc[nt][1]);
      acc[nt][2] = fmaf(s_hi, part[nt][0][2] + part[nt][1][2], acc[nt][2]);
      acc[nt][3] = fmaf(s_hi, part[nt][0][3] + part[nt][1][3], acc[nt][3]);
    }
  };
  if (cg == CG) {
    // full chunk: unrolled so that the next group's loads overlap this group's math
    constexpr int kUnroll = (NT <= 2) ? CG : 1;
#pragma unroll kUnroll
    for (int g = 0; g < CG; ++g) one_group(g);
  } else {
    for (int g = 0; g < cg; ++g) one_group(g);
  }
}

// ---------------------------------------------------------------------------
// Streaming kernel.  CTA_MAX additionally records, per CTA and activation row,
// the largest bf16-rounded output the CTA produced (used by the vocabulary
// projection to bound its top-k search): p.cta_max[blockIdx.x * M + m].
// ---------------------------------------------------------------------------
template <int NT, int CG, int NWARPS, bool CTA_MAX, int DQ>
__global__ void __launch_bounds__(NWARPS * 32, 1)
w4a16_stream_kernel(const __grid_constant__ StreamParams p) {
  extern __shared__ __align__(128) std::uint8_t smem[];
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int depth = p.depth;

  // shared memory: [barriers][activations][NWARPS rings of `depth` stages]
  std::uint64_t* bars = reinterpret_cast<std::uint64_t*>(smem) + warp * kMaxDepth;
  std::uint8_t* xs = smem + NWARPS * kMaxDepth * 8;
  std::uint8_t* ring = xs + p.x_bytes + static_cast<std::size_t>(warp) * depth * p.stage_bytes;

  // this CTA's contiguous range of m-tiles: an equal share of the launch's chunks
  const int mt_lo = mtile_at_cost<CG>(p, static_cast<long long>(blockIdx.x) * p.total_cost / gridDim.x);
  const int mt_hi = mtile_at_cost<CG>(p, static_cast<long long>(blockIdx.x + 1) * p.total_cost / gridDim.x);

  if (lane == 0) {
    for (int s = 0; s < depth; ++s) mbar_init(&bars[s], 1);
    mbar_init_fence();
  }
  __syncwarp();

  const std::uint64_t policy = policy_evict_first();

  // Two cursors over this warp's items: `fc` runs ahead issuing copies, `cc`
  // consumes.  The warp takes m-tiles mt_lo + warp, + NWARPS, ...
  Cursor<CG> fc, cc;
  fc.start(p, mt_lo + warp, mt_hi);
  cc = fc;
  int issued = 0, consumed = 0;
  for (int s = 0; s < depth && fc.valid; ++s) {
    issue_item<CG>(fc, ring + s * p.stage_bytes, &bars[s], lane, policy);
    fc.advance(p, NWARPS, mt_hi);
    ++issued;
  }

  float vmax[NT][2];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) vmax[nt][0] = vmax[nt][1] = -INFINITY;

  bool dead = false;  // a wait ran out: stop computing, keep attending barriers
  const int d_first = mt_lo < mt_hi ? find_desc(p, mt_lo) : p.n_desc;
  for (int d = d_first; d < p.n_desc; ++d) {
    const LinearDev L = load_desc(p, d);
    if (L.mt_begin >= mt_hi) break;
    const int rsx = 2 * L.K + 32;
    __syncthreads();  // every warp is done with the previous activations
    fill_x_fragments<DQ>(xs, L.x, L.M, L.K, rsx, tid, NWARPS * 32);
    __syncthreads();
    const std::uint32_t xs_addr = smem_u32(xs);
    const int G = L.K >> 7;

    while (cc.valid && cc.d == d) {
      float acc[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
      const int row0 = (cc.mt - cc.mt_begin) * kMTileRows;
      const int nch = cc.nch;
      for (int ch = 0; ch < nch; ++ch) {
        const int slot = consumed % depth;
        const std::uint32_t parity = static_cast<std::uint32_t>(consumed / depth) & 1u;
        std::uint8_t* stage = ring + slot * p.stage_bytes;
#if CB200_LOADER == 2
        (void)parity;
        if (issued - consumed >= 3) asm volatile("cp.async.wait_group 2;" ::: "memory");
        else if (issued - consumed == 2) asm volatile("cp.async.wait_group 1;" ::: "memory");
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();
#else
        if (!dead && !wait_stage(&bars[slot], parity)) {
          dead = true;
          if (lane == 0) atomicExch(p.status, CUDALM_B200_ERR_TIMEOUT);
        }
#endif
        if (!dead) {
          const int g0 = ch * CG;
          consume_chunk<NT, CG, DQ>(smem_u32(stage), xs_addr, G, g0, min(CG, G - g0), rsx, L.M,
                                lane, acc);
          __syncwarp();
          if (fc.valid) {
            issue_item<CG>(fc, stage, &bars[slot], lane, policy);
            fc.advance(p, NWARPS, mt_hi);
            ++issued;
          }
        }
        ++consumed;
        cc.advance(p, NWARPS, mt_hi);
      }
      if (!dead) {
        const int r8 = lane >> 2, t = lane & 3;
        const int row_lo = row0 + r8, row_hi = row_lo + 8;
        std::uint16_t* y = L.y;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int col = nt * 8 + 2 * t;
          const std::uint16_t o0 = float_to_bf16_bits(acc[nt][0]);
          const std::uint16_t o1 = float_to_bf16_bits(acc[nt][1]);
          const std::uint16_t o2 = float_to_bf16_bits(acc[nt][2]);
          const std::uint16_t o3 = float_to_bf16_bits(acc[nt][3]);
          if (col < L.M) {
            if (row_lo < L.N) y[static_cast<std::size_t>(col) * L.N + row_lo] = o0;
            if (row_hi < L.N) y[static_cast<std::size_t>(col) * L.N + row_hi] = o2;
          }
          if (col + 1 < L.M) {
            if (row_lo < L.N) y[static_cast<std::size_t>(col + 1) * L.N + row_lo] = o1;
            if (row_hi < L.N) y[static_cast<std::size_t>(col + 1) * L.N + row_hi] = o3;
          }
          if (CTA_MAX) {
            if (row_lo < L.N) {
              vmax[nt][0] = fmaxf(vmax[nt][0], bf16_bits_to_float(o0));
              vmax[nt][1] = fmaxf(vmax[nt][1], bf16_bits_to_float(o1));
            }
            if (row_hi < L.N) {
              vmax[nt][0] = fmaxf(vmax[nt][0], bf16_bits_to_float(o2));
              vmax[nt][1] = fmaxf(vmax[nt][1], bf16_bits_to_float(o3));
            }
          }
        }
      }
    }
  }

  if (dead) {
    // Give copies still in flight a bounded chance to land before the CTA's
    // shared memory is released.
    for (int i = consumed; i < issued; ++i)
      (void)wait_stage(&bars[i % depth], static_cast<std::uint32_t>(i / depth) & 1u);
  }

  if (CTA_MAX) {
    // reduce over the eight row-lanes that share a column pair, then over warps
    const int M = load_desc(p, 0).M;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float v = vmax[nt][c];
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
        vmax[nt][c] = v;
      }
    }
    __syncthreads();  // the activation region is free again; reuse it as scratch
    float* red = reinterpret_cast<float*>(xs);  // [NWARPS][NT*8]
    if (lane < 4) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        red[warp * (NT * 8) + nt * 8 + 2 * lane] = vmax[nt][0];
        red[warp * (NT * 8) + nt * 8 + 2 * lane + 1] = vmax[nt][1];
      }
    }
    __syncthreads();
    if (tid < M && tid < NT * 8) {
      float v = -INFINITY;
      for (int w = 0; w < NWARPS; ++w) v = fmaxf(v, red[w * (NT * 8) + tid]);
      p.cta_max[static_cast<std::size_t>(blockIdx.x) * M + tid] = v;
    }
  }
}

#endif  // __CUDACC__

}  // namespace cb200
