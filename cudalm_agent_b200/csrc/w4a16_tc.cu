// Batched rows (M >= 16) on the fifth-generation tensor cores.
//
// One CTA per SM works on items of 256 weight rows (two 128-row MMA tiles) of one
// projection; the M activation rows (padded to NTOK = 16, 32 or 64) are the N
// dimension of the MMA.  Per quantisation group of 128 k:
//
//   * the TMA unit has staged the packed weights of the item, 128 bytes (two
//     groups) per row and stage, with the 128-byte swizzle so that a thread
//     reading its own row meets no bank conflict;
//   * each of 256 "row" threads turns its row's 64 bytes into 64 registers of
//     exact bf16 pairs and writes them to tensor memory (tcgen05.st) as the A
//     operand of eight K=16 MMAs: lane = row, 8 columns per MMA;
//   * one thread issues the eight tcgen05.mma (A from tensor memory, B = the
//     activations in shared memory in the canonical K-major core-matrix layout)
//     into a per-group accumulator in tensor memory and commits to mbarriers;
//   * the row threads read the accumulator back (tcgen05.ld) and fold it into
//     registers: acc[n] += scale[row, group] * sum[n].
//
// A and D are double buffered in tensor memory (2 tiles x (2 x 64 + 2 x NTOK)
// columns <= 512), so the dequantisation of group g+1 overlaps the MMAs of group
// g and the read-back of group g-1.  Products are exact and sums are fp32, as in
// the streaming kernel; only the summation order differs.
//
// The k order inside a K=16 MMA is a private permutation shared by A and B: word
// w of a row (k = 8w .. 8w+7) yields four registers {n_i, n_{i+4}}, i = 0..3, which
// become columns 4(w & 1) + i of MMA w >> 1; the activations are stored to match
// (fill_b_operand), times 2^64 / 2^60 to offset the 2^-133 / 2^-129 of the tiny-number
// dequantisation (see w4a16_stream.cuh).
//
// Every wait is bounded; a wait that runs out raises a CTA-wide abort flag, the
// kernel stores ERR_TIMEOUT in the status word, frees its tensor memory and returns.
#include <cuda.h>

#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace cb200 {

constexpr int kTcRowsPerTile = 128;
constexpr int kTcTiles = 2;                      // MMA tiles per item
constexpr int kTcItemRows = kTcRowsPerTile * kTcTiles;
constexpr int kTcMaxStages = 4;  // as many as fit beside the activations, at least 2
constexpr int kTcStageBytes = kTcItemRows * 128;  // two groups of every row of the item
// Warp roles.  Dequantisation and read-back are separate warps so that the
// threads that feed the tensor core never wait for its results.
//   warps 0..7   dequantise: tile = warp >> 2, rows 32 (warp & 3) .. +31 of the tile
//   warps 8..15  read the accumulators back and fold them in: same row mapping
//   warp 16      TMA producer
//   warps 17,18  MMA issuers, one per tile
constexpr int kTcDequantWarps = 8;
constexpr int kTcFoldWarp0 = 8;
constexpr int kTcProducerWarp = 16;
constexpr int kTcMmaWarp = 17;
constexpr int kTcThreads = 608;
constexpr int kTcMaxBBytes = 128 * 1024;          // activations resident in shared memory
constexpr unsigned long long kTcWaitNs = 400000000ull;

struct alignas(64) TcDesc {
  CUtensorMap tmap;  // weights as uint32 [N][K/8], box 128 rows x 32 words, 128-byte swizzle
  const std::uint16_t* S;
  const std::uint16_t* x;
  std::uint16_t* y;
  int N, K, M;
  int item_begin;   // first item (256-row block) of this projection in the launch
  int cost_begin;   // stage loads before this projection
  int pad;
};

struct TcParams {
  TcDesc inl[CUDALM_B200_MAX_INLINE_LINEARS];
  const TcDesc* table;
  int n_stages;
  int n_desc;
  int total_items;
  int total_cost;
  int* status;
};

// ---------------------------------------------------------------------------
// tcgen05 wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(std::uint32_t* smem_slot, std::uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_slot)),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(std::uint32_t taddr, std::uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(std::uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(std::uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; accumulate = 0 overwrites D.
__device__ __forceinline__ void tc_mma_ts(std::uint32_t d_tmem, std::uint32_t a_tmem,
                                          std::uint64_t b_desc, std::uint32_t idesc,
                                          std::uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      :
      : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// 16 consecutive 32-bit columns of this thread's lane
__device__ __forceinline__ void tmem_st16(std::uint32_t taddr, const std::uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(std::uint32_t taddr, float* f) {
  std::uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) f[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tmem_ld8(std::uint32_t taddr, float* f) {
  std::uint32_t r[8];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of one K=16 slice of the B operand: K-major,
// no swizzle, core matrices of 8 rows x 16 bytes; 128 bytes between the two
// core matrices along K (leading byte offset), 256 bytes between 8-row groups
// (stride byte offset); descriptor version 1.
__device__ __forceinline__ std::uint64_t tc_b_desc(std::uint32_t smem_addr) {
  std::uint64_t d = 0;
  d |= static_cast<std::uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<std::uint64_t>(128u >> 4) << 16;
  d |= static_cast<std::uint64_t>(256u >> 4) << 32;
  d |= static_cast<std::uint64_t>(1u) << 46;
  return d;
}

// Instruction descriptor: D fp32, A and B bf16, both K-major, M = 128, N = ntok.
__host__ __device__ constexpr std::uint32_t tc_idesc(int ntok) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<std::uint32_t>(ntok >> 3) << 17) |
         (static_cast<std::uint32_t>(kTcRowsPerTile >> 4) << 24);
}

// Bounded, abort-aware wait.  Returns false when the wait ran out or another
// thread of the CTA already gave up.
__device__ __forceinline__ bool tc_wait(std::uint64_t* bar, std::uint32_t parity,
                                        volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
  for (;;) {
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (*abort_flag) return false;
    unsigned long long t1;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
    if (t1 - t0 > kTcWaitNs) {
      *abort_flag = 1;
      return false;
    }
  }
}

// Activations -> B operand.  For MMA slice kt (16 values of k) and activation row
// n the 16 slots are laid out as core matrices: byte offset
//   kt * ntok * 32 + (n / 8) * 256 + (slot / 8) * 128 + (n % 8) * 16 + (slot % 8) * 2.
// Value k = 16 kt + 8 w + i (w = word parity, i = nibble in the word) goes to slot
// 8 w + 2 (i & 3) + (i >> 2), times 2^64 (even i) or 2^60 (odd i).
template <int NTOK>
__device__ __forceinline__ void fill_b_operand(std::uint8_t* bsm, const std::uint16_t* x, int M,
                                               int K, int tid, int nthreads) {
  // one block of eight consecutive k (one weight word) = one 16-byte core-matrix row:
  // slots 0..7 of the block hold k offsets 0,4,1,5,2,6,3,7
  const int blocks_per_row = K >> 3;
  const int total = NTOK * blocks_per_row;
  const bool vec = (reinterpret_cast<std::uintptr_t>(x) & 15u) == 0;
  for (int b = tid; b < total; b += nthreads) {
    const int n = b / blocks_per_row;
    const int kb = b - n * blocks_per_row;  // k = 8 kb .. 8 kb + 7
    std::uint16_t v[8];
    if (n < M) {
      const std::uint16_t* src = x + static_cast<std::size_t>(n) * K + kb * 8;
      if (vec) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(src));
        const std::uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          v[2 * i] = static_cast<std::uint16_t>(w[i] & 0xFFFFu);
          v[2 * i + 1] = static_cast<std::uint16_t>(w[i] >> 16);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __ldg(src + i);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0;
    }
    std::uint32_t out[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float sc = (i & 1) ? 0x1p60f : 0x1p64f;
      const std::uint32_t lo = float_to_bf16_bits(bf16_bits_to_float(v[i]) * sc);
      const std::uint32_t hi = float_to_bf16_bits(bf16_bits_to_float(v[i + 4]) * sc);
      out[i] = lo | (hi << 16);
    }
    const int kt = kb >> 1, w = kb & 1;
    *reinterpret_cast<uint4*>(bsm + static_cast<std::size_t>(kt) * NTOK * 32 + (n >> 3) * 256 + w * 128 +
                              (n & 7) * 16) = make_uint4(out[0], out[1], out[2], out[3]);
  }
}

// int4 word -> four exact bf16 pairs {q(n_i), q(n_{i+4})} * 2^-133 (even i) or
// 2^-129 (odd i); see dequant_word in w4a16_stream.cuh for the encoding.  Here the
// offset 8 is subtracted per value (an exact bf16 subtraction) because the
// accumulators live in tensor memory, where a per-group correction would cost more.
__device__ __forceinline__ void dequant_word_exact(std::uint32_t w, std::uint32_t* out) {
  const std::uint32_t w8 = w >> 8;
  out[0] = sub_bf16x2(lop3_and_xor(w, 0x000F000Fu, 0x00080008u), 0x00080008u);
  out[1] = sub_bf16x2(lop3_and_xor(w, 0x00F000F0u, 0x00800080u), 0x00800080u);
  out[2] = sub_bf16x2(lop3_and_xor(w8, 0x000F000Fu, 0x00080008u), 0x00080008u);
  out[3] = sub_bf16x2(lop3_and_xor(w8, 0x00F000F0u, 0x00800080u), 0x00800080u);
}

// Shared-memory map of the kernel.
struct TcSmem {
  std::uint64_t full[kTcMaxStages];
  std::uint64_t empty[kTcMaxStages];
  std::uint64_t a_full[kTcTiles][2];
  std::uint64_t a_free[kTcTiles][2];
  std::uint64_t d_full[kTcTiles][2];
  std::uint64_t d_free[kTcTiles][2];
  std::uint32_t tmem_base;
  int abort_flag;
};
constexpr int kTcHeaderBytes = 1024;
static_assert(sizeof(TcSmem) <= kTcHeaderBytes, "barrier block too large");

// ---------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------
template <int NTOK>
__global__ void __launch_bounds__(kTcThreads, 1) w4a16_tc_kernel(const __grid_constant__ TcParams p) {
  extern __shared__ __align__(1024) std::uint8_t smem_raw[];
  // the swizzled TMA destinations need 1024-byte alignment; the launch adds the slack
  std::uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  TcSmem* sm = reinterpret_cast<TcSmem*>(smem);
  std::uint8_t* stages = smem + kTcHeaderBytes;                       // 1024-byte aligned
  const int kTcStages = p.n_stages;
  std::uint8_t* bsm = stages + kTcStages * kTcStageBytes;             // B operand
  volatile int* abort_flag = &sm->abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const TcDesc* tbl = p.table ? p.table : p.inl;
  constexpr int kColsPerTile = 128 + 2 * NTOK;
  constexpr std::uint32_t kIdesc = tc_idesc(NTOK);

  if (tid == 0) {
    for (int s = 0; s < kTcStages; ++s) {
      mbar_init(&sm->full[s], 1);
      mbar_init(&sm->empty[s], kTcDequantWarps * 32);
    }
    for (int t = 0; t < kTcTiles; ++t)
      for (int b = 0; b < 2; ++b) {
        mbar_init(&sm->a_full[t][b], kTcRowsPerTile);
        mbar_init(&sm->a_free[t][b], 1);
        mbar_init(&sm->d_full[t][b], 1);
        mbar_init(&sm->d_free[t][b], kTcRowsPerTile);
      }
    sm->abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&sm->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const std::uint32_t tmem_base = sm->tmem_base;

  // This CTA's contiguous range of items: an equal share of the stage loads.
  int it_lo, it_hi, d_first;
  {
    auto item_at = [&](long long cost) -> int {
      if (cost >= p.total_cost) return p.total_items;
      int lo = 0, hi = p.n_desc - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (tbl[mid].cost_begin <= cost) lo = mid; else hi = mid - 1;
      }
      const int per_item = ((tbl[lo].K >> 7) + 1) >> 1;
      return tbl[lo].item_begin + static_cast<int>((cost - tbl[lo].cost_begin + per_item - 1) / per_item);
    };
    it_lo = item_at(static_cast<long long>(blockIdx.x) * p.total_cost / gridDim.x);
    it_hi = item_at(static_cast<long long>(blockIdx.x + 1) * p.total_cost / gridDim.x);
    d_first = 0;
    while (d_first + 1 < p.n_desc && tbl[d_first + 1].item_begin <= it_lo) ++d_first;
    if (it_lo >= it_hi) d_first = p.n_desc;
  }

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  std::uint32_t sit = 0;  // stage loads so far (same count in every role)
  std::uint32_t git = 0;  // groups so far (same count in every role)

  for (int d = d_first; d < p.n_desc; ++d) {
    const TcDesc* L = tbl + d;
    if (L->item_begin >= it_hi) break;
    const int LN = L->N, LK = L->K, LM = L->M;
    const int G = LK >> 7;
    const int items_here = (LN + kTcItemRows - 1) / kTcItemRows;
    const int i0 = max(it_lo, L->item_begin), i1 = min(it_hi, L->item_begin + items_here);

    // (also) all MMAs that read the previous activations have completed
    if (__syncthreads_or(sm->abort_flag)) break;
    fill_b_operand<NTOK>(bsm, L->x, LM, LK, tid, kTcThreads);
    // make the generic-proxy writes visible to the tensor core's (async proxy) reads
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();

    if (warp == kTcProducerWarp) {
      // ---------------- TMA producer ----------------
      if (lane == 0) {
        const std::uint64_t policy = policy_evict_first();
        for (int item = i0; item < i1 && !*abort_flag; ++item) {
          const int row0 = (item - L->item_begin) * kTcItemRows;
          for (int c = 0; c < (G + 1) / 2; ++c, ++sit) {
            const int s = sit % kTcStages;
            const std::uint32_t use = sit / kTcStages;
            if (use >= 1 && !tc_wait(&sm->empty[s], (use - 1) & 1u, abort_flag)) break;
            std::uint8_t* st = stages + s * kTcStageBytes;
            mbar_arrive_expect_tx(&sm->full[s], kTcStageBytes);
            for (int t = 0; t < kTcTiles; ++t) {
              asm volatile(
                  "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
                  ".L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(
                      smem_u32(st + t * kTcRowsPerTile * 128)),
                  "l"(&L->tmap), "r"(c * 32), "r"(row0 + t * kTcRowsPerTile),
                  "r"(smem_u32(&sm->full[s])), "l"(policy)
                  : "memory");
            }
          }
        }
      } else {
        for (int item = i0; item < i1; ++item) sit += (G + 1) / 2;
      }
      sit = __shfl_sync(0xffffffffu, sit, 0);
    } else if (warp >= kTcMmaWarp) {
      // ---------------- MMA issuer ----------------
      if (lane == 0) {
        const std::uint32_t b_base = smem_u32(bsm);
        for (int item = i0; item < i1 && !*abort_flag; ++item) {
          for (int g = 0; g < G; ++g, ++git) {
            const int buf = git & 1;
            const std::uint32_t use = git >> 1;
            bool ok = true;
            {
              const int t = warp - kTcMmaWarp;
              ok = tc_wait(&sm->a_full[t][buf], use & 1u, abort_flag);
              if (ok && use >= 1) ok = tc_wait(&sm->d_free[t][buf], (use - 1) & 1u, abort_flag);
              if (!ok) break;
              tc_fence_after();
              const std::uint32_t tile_base = tmem_base + t * kColsPerTile;
              const std::uint32_t a_addr = tile_base + buf * 64;
              const std::uint32_t d_addr = tile_base + 128 + buf * NTOK;
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const std::uint64_t bd = tc_b_desc(b_base + static_cast<std::uint32_t>(g * 8 + j) * (NTOK * 32));
                tc_mma_ts(d_addr, a_addr + j * 8, bd, kIdesc, j > 0 ? 1u : 0u);
              }
              tc_commit(&sm->a_free[t][buf]);
              tc_commit(&sm->d_full[t][buf]);
            }
            if (!ok) break;
          }
        }
      } else {
        for (int item = i0; item < i1; ++item) git += G;
      }
      git = __shfl_sync(0xffffffffu, git, 0);
      for (int item = i0; item < i1; ++item) sit += (G + 1) / 2;
    } else if (warp < kTcDequantWarps) {
      // ---------------- dequantise and feed the A operand ----------------
      const int tile = warp >> 2;
      const int lrow = (warp & 3) * 32 + lane;                      // row inside the tile
      const std::uint32_t lane_base = static_cast<std::uint32_t>((warp & 3) * 32) << 16;
      const std::uint32_t tile_base = tmem_base + tile * kColsPerTile + lane_base;
      bool alive = true;
      for (int item = i0; item < i1 && alive; ++item) {
        for (int g = 0; g < G && alive; ++g, ++git) {
          const int half = g & 1;
          const int s = sit % kTcStages;
          if (half == 0) {
            bool ok = tc_wait(&sm->full[s], (sit / kTcStages) & 1u, abort_flag);
            alive = __all_sync(0xffffffffu, ok);
            if (!alive) break;
          }
          const std::uint8_t* rowp = stages + s * kTcStageBytes + tile * kTcRowsPerTile * 128 + lrow * 128;
          std::uint32_t regs[64];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint4 v = lds128(rowp + (((4 * half + q) ^ (lrow & 7)) << 4));
            dequant_word_exact(v.x, regs + 16 * q);
            dequant_word_exact(v.y, regs + 16 * q + 4);
            dequant_word_exact(v.z, regs + 16 * q + 8);
            dequant_word_exact(v.w, regs + 16 * q + 12);
          }
          if (half == 1 || g == G - 1) {
            mbar_arrive(&sm->empty[s]);  // this thread has taken its bytes out of the stage
            ++sit;
          }
          const int buf = git & 1;
          const std::uint32_t use = git >> 1;
          if (use >= 1) {
            bool ok = tc_wait(&sm->a_free[tile][buf], (use - 1) & 1u, abort_flag);
            alive = __all_sync(0xffffffffu, ok);
            if (!alive) break;
          }
          tc_fence_after();
          const std::uint32_t a_addr = tile_base + buf * 64;
#pragma unroll
          for (int q = 0; q < 4; ++q) tmem_st16(a_addr + 16 * q, regs + 16 * q);
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          tc_fence_before();
          mbar_arrive(&sm->a_full[tile][buf]);
        }
      }
    } else if (warp < kTcProducerWarp) {
      // ---------------- read the accumulators back: acc += scale * sum ----------------
      const int fw = warp - kTcFoldWarp0;
      const int tile = fw >> 2;
      const int lrow = (fw & 3) * 32 + lane;
      const std::uint32_t lane_base = static_cast<std::uint32_t>((fw & 3) * 32) << 16;
      const std::uint32_t tile_base = tmem_base + tile * kColsPerTile + lane_base;
      bool alive = true;
      for (int item = i0; item < i1 && alive; ++item) {
        const int row = (item - L->item_begin) * kTcItemRows + tile * kTcRowsPerTile + lrow;
        const bool row_ok = row < LN;
        const std::uint16_t* srow = L->S + static_cast<std::size_t>(row_ok ? row : 0) * G;
        float acc[NTOK];
#pragma unroll
        for (int n = 0; n < NTOK; ++n) acc[n] = 0.f;
        for (int g = 0; g < G && alive; ++g, ++git) {
          const float sc = row_ok ? __half2float(__ushort_as_half(__ldg(srow + g))) : 0.f;
          const int buf = git & 1;
          bool ok = tc_wait(&sm->d_full[tile][buf], (git >> 1) & 1u, abort_flag);
          alive = __all_sync(0xffffffffu, ok);
          if (!alive) break;
          tc_fence_after();
          const std::uint32_t d_addr = tile_base + 128 + buf * NTOK;
#pragma unroll
          for (int c = 0; c < NTOK / 16; ++c) {
            float f[16];
            tmem_ld16(d_addr + c * 16, f);
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[c * 16 + i] = fmaf(sc, f[i], acc[c * 16 + i]);
          }
          tc_fence_before();
          mbar_arrive(&sm->d_free[tile][buf]);
        }
        if (alive && row_ok) {
          std::uint16_t* y = L->y;
#pragma unroll
          for (int n = 0; n < NTOK; ++n)
            if (n < LM) y[static_cast<std::size_t>(n) * LN + row] = float_to_bf16_bits(acc[n] * 0x1p69f);
        }
      }
    }
  }

  __syncthreads();
  if (*abort_flag && tid == 0) atomicExch(p.status, CUDALM_B200_ERR_TIMEOUT);
  tc_fence_after();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn tc_encode_fn() {
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

// weights as uint32 [N][K/8]; box = 32 words (two groups) x 128 rows, 128-byte swizzle
int tc_encode(const std::uint8_t* weight, int N, int K, CUtensorMap* out) {
  EncodeTiledFn fn = tc_encode_fn();
  if (!fn) return CUDALM_B200_ERR_CUDA;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K / 8), static_cast<cuuint64_t>(N)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K / 2)};
  const cuuint32_t box[2] = {32, static_cast<cuuint32_t>(kTcRowsPerTile)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<std::uint8_t*>(weight),
                        dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = static_cast<int>(r);
    return CUDALM_B200_ERR_CUDA;
  }
  return CUDALM_B200_OK;
}

int tc_ntok(int M) { return M <= 16 ? 16 : (M <= 32 ? 32 : 64); }

template <int NTOK>
int tc_launch(const TcParams& p_in, int kmax, cudaStream_t stream) {
  auto kern = w4a16_tc_kernel<NTOK>;
  int n_stages = (kMaxSmemBytes - 1024 - kTcHeaderBytes - NTOK * kmax * 2) / kTcStageBytes;
  if (n_stages > kTcMaxStages) n_stages = kTcMaxStages;
  if (n_stages < 2) return CUDALM_B200_ERR_UNSUPPORTED;
  TcParams p = p_in;
  p.n_stages = n_stages;
  const int smem = 1024 + kTcHeaderBytes + n_stages * kTcStageBytes + NTOK * kmax * 2;
  static std::mutex mu;
  static std::vector<int> done;
  int dev = 0;
  CB200_CUDA_TRY(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lk(mu);
    bool seen = false;
    for (int d : done) seen |= (d == dev);
    if (!seen) {
      CB200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          kMaxSmemBytes));
      done.push_back(dev);
    }
  }
  int grid = num_sms();
  if (grid > p.total_items) grid = p.total_items;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(kTcThreads);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem);
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

}  // namespace

// True when the tensor-memory kernel takes this projection in one pass.
bool tc_eligible(const cudalm_b200_linear& l) {
  if (l.M < 1 || l.M > 64 || l.K <= 0 || (l.K % 128) != 0) return false;
  if (!aligned_to(l.weight, 16)) return false;
  return static_cast<long long>(tc_ntok(l.M)) * l.K * 2 <= kTcMaxBBytes;
}

// Fills `out[count]` and the launch totals; UNSUPPORTED when a projection (or the
// widest M with the longest K) does not fit the kernel's shared-memory budget.
int tc_describe(const cudalm_b200_linear* ls, int count, TcDesc* out, int* items_out,
                int* cost_out, int* kmax_out, int* ntok_out) {
  int items = 0, cost = 0, kmax = 0, ntok = 0;
  for (int i = 0; i < count; ++i) {
    const cudalm_b200_linear& l = ls[i];
    if (!tc_eligible(l)) return CUDALM_B200_ERR_UNSUPPORTED;
    ntok = tc_ntok(l.M) > ntok ? tc_ntok(l.M) : ntok;
    TcDesc& d = out[i];
    if (int rc = tc_encode(l.weight, l.N, l.K, &d.tmap)) return rc;
    d.S = l.scales;
    d.x = l.x;
    d.y = l.y;
    d.N = l.N;
    d.K = l.K;
    d.M = l.M;
    d.item_begin = items;
    d.cost_begin = cost;
    const int n_items = (l.N + kTcItemRows - 1) / kTcItemRows;
    items += n_items;
    cost += n_items * (((l.K >> 7) + 1) >> 1);
    kmax = l.K > kmax ? l.K : kmax;
  }
  if (static_cast<long long>(ntok) * kmax * 2 > kTcMaxBBytes) return CUDALM_B200_ERR_UNSUPPORTED;
  *items_out = items;
  *cost_out = cost;
  *kmax_out = kmax;
  *ntok_out = ntok;
  return CUDALM_B200_OK;
}

int tc_run_params(TcParams& p, int kmax, int ntok, cudaStream_t stream) {
  p.status = device_status_word();
  if (!p.status) return CUDALM_B200_ERR_CUDA;
  if (ntok == 16) return tc_launch<16>(p, kmax, stream);
  if (ntok == 32) return tc_launch<32>(p, kmax, stream);
  return tc_launch<64>(p, kmax, stream);
}

// Up to CUDALM_B200_MAX_INLINE_LINEARS projections in one launch.
int run_tc(const cudalm_b200_linear* ls, int count, cudaStream_t stream) {
  if (count < 1 || count > CUDALM_B200_MAX_INLINE_LINEARS) return CUDALM_B200_ERR_BAD_SHAPE;
  TcParams p;
  std::memset(&p, 0, sizeof(p));
  int kmax = 0, ntok = 0;
  if (int rc = tc_describe(ls, count, p.inl, &p.total_items, &p.total_cost, &kmax, &ntok)) return rc;
  p.n_desc = count;
  return tc_run_params(p, kmax, ntok, stream);
}

// Any number of projections: the descriptor table lives on the device.
struct TcGroup {
  TcDesc* table_dev = nullptr;
  int count = 0, items = 0, cost = 0, kmax = 0, ntok = 0;
};

int tc_group_create(const cudalm_b200_linear* ls, int count, TcGroup** out) {
  std::vector<TcDesc> tbl(static_cast<size_t>(count));
  TcGroup* g = new TcGroup();
  g->count = count;
  if (int rc = tc_describe(ls, count, tbl.data(), &g->items, &g->cost, &g->kmax, &g->ntok)) {
    delete g;
    return rc;
  }
  cudaError_t e = cudaMalloc(&g->table_dev, sizeof(TcDesc) * tbl.size());
  if (e == cudaSuccess)
    e = cudaMemcpy(g->table_dev, tbl.data(), sizeof(TcDesc) * tbl.size(), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    g_last_cuda_error = static_cast<int>(e);
    if (g->table_dev) cudaFree(g->table_dev);
    delete g;
    return CUDALM_B200_ERR_CUDA;
  }
  *out = g;
  return CUDALM_B200_OK;
}

int tc_group_run(const TcGroup* g, cudaStream_t stream) {
  TcParams p;
  std::memset(&p, 0, sizeof(p));
  p.table = g->table_dev;
  p.n_desc = g->count;
  p.total_items = g->items;
  p.total_cost = g->cost;
  return tc_run_params(p, g->kmax, g->ntok, stream);
}

void tc_group_destroy(TcGroup* g) {
  if (!g) return;
  cudaFree(g->table_dev);
  delete g;
}

}  // namespace cb200
