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
  int mt_begin;  // index of this projection's first m-tile in the launch
  int flags;
  int pad;
};

struct StreamParams {
  const LinearDev* table;  // device table, or nullptr to use `inl`
  LinearDev inl[CUDALM_B200_MAX_INLINE_LINEARS];
  int n_desc;
  int total_mt;
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
  // order this warp's earlier reads of the stage before the async writes
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();
  if (lane == 0)
    mbar_arrive_expect_tx(bar, static_cast<std::uint32_t>(rows) * seg + (sbulk ? sbytes : 0u));
  __syncwarp();
  if (lane < rows) {
    bulk_g2s_hint(stage + lane * RS,
                  c.W + static_cast<std::size_t>(row0 + lane) * (c.K >> 1) + g0 * 64, seg,
                  bar, policy);
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
    if (mbar_wait_bounded(bar, parity, 256)) return true;
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
__device__ __forceinline__ void fill_x_fragments(std::uint8_t* xs, const std::uint16_t* x,
                                                 int M, int K, int rsx, int tid,
                                                 int nthreads) {
  const int total = M * K;
  for (int idx = tid; idx < total; idx += nthreads) {
    const int n = idx / K;
    const int k = idx - n * K;
    const std::uint16_t v = __ldg(x + idx);
    const int g = k >> 7, r = k & 127, t = r >> 5, q = r & 31, w = q >> 3, i = q & 7;
    const int j = 2 * w + ((i & 3) >> 1);
    const int e = 2 * (i & 1) + (i >> 2);
    *reinterpret_cast<std::uint16_t*>(xs + n * rsx + ((((g * 8 + j) * 4 + t) * 4 + e) * 2)) = v;
  }
}

// One chunk of one m-tile: acc[nt][0..3] += sum over the chunk's groups.
// Fragment ownership (lane = 4*r8 + t): rows r8 and r8+8 of the m-tile,
// activation rows (columns of the MMA) nt*8 + 2t and nt*8 + 2t + 1.
template <int NT, int CG>
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
  bool xok[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int n = nt * 8 + r8;
    xok[nt] = n < M;
    xrow[nt] = xs + (xok[nt] ? n : 0) * rsx + g0 * 256 + t * 8;
  }
  for (int g = 0; g < cg; ++g) {
    const uint4 qa = lds128(wa + g * 64);
    const uint4 qb = lds128(wb + g * 64);
    const float s_lo = __half2float(__ushort_as_half(lds16(sa + 2 * g)));
    const float s_hi = __half2float(__ushort_as_half(lds16(sb + 2 * g)));
    const std::uint32_t wordA[4] = {qa.x, qa.y, qa.z, qa.w};
    const std::uint32_t wordB[4] = {qb.x, qb.y, qb.z, qb.w};
    float part[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      part[nt][0] = part[nt][1] = part[nt][2] = part[nt][3] = 0.f;
    }
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      std::uint32_t A[4], B[4];
      dequant_word_bf16x2(wordA[w], A);
      dequant_word_bf16x2(wordB[w], B);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int j = 2 * w + h;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          uint2 b = make_uint2(0u, 0u);
          if (xok[nt]) b = lds64(xrow[nt] + g * 256 + j * 32);
          mma_m16n8k16_bf16(part[nt], A[2 * h], B[2 * h], A[2 * h + 1], B[2 * h + 1], b.x, b.y);
        }
      }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      acc[nt][0] = fmaf(s_lo, part[nt][0], acc[nt][0]);
      acc[nt][1] = fmaf(s_lo, part[nt][1], acc[nt][1]);
      acc[nt][2] = fmaf(s_hi, part[nt][2], acc[nt][2]);
      acc[nt][3] = fmaf(s_hi, part[nt][3], acc[nt][3]);
    }
  }
}


// ---------------------------------------------------------------------------
// Streaming kernel.  CTA_MAX additionally records, per CTA and activation row,
// the largest bf16-rounded output the CTA produced (used by the vocabulary
// projection to bound its top-k search): p.cta_max[blockIdx.x * M + m].
// ---------------------------------------------------------------------------
template <int NT, int CG, int NWARPS, bool CTA_MAX>
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

  // this CTA's contiguous range of m-tiles (the host keeps gridDim.x <= total_mt)
  const int mt_lo = static_cast<int>(static_cast<long long>(blockIdx.x) * p.total_mt / gridDim.x);
  const int mt_hi = static_cast<int>(static_cast<long long>(blockIdx.x + 1) * p.total_mt / gridDim.x);

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
    fill_x_fragments(xs, L.x, L.M, L.K, rsx, tid, NWARPS * 32);
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
        if (!dead && !wait_stage(&bars[slot], parity)) {
          dead = true;
          if (lane == 0) atomicExch(p.status, CUDALM_B200_ERR_TIMEOUT);
        }
        if (!dead) {
          const int g0 = ch * CG;
          consume_chunk<NT, CG>(smem_u32(stage), xs_addr, G, g0, min(CG, G - g0), rsx, L.M,
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
