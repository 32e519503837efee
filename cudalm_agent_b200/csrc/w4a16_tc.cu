// Batched rows (M >= 17 by default) on the fifth-generation tensor cores.
//
// One CTA per SM works on items of 256 weight rows (two 128-row MMA tiles) of one
// projection; the M activation rows (padded to NTOK = 16, 32 or 64) are the N
// dimension of the MMA.  A stage of shared memory holds two quantisation groups
// (256 values of k) of an item: the packed weights, 128 bytes per row, and the
// matching slice of the activations, both brought in by the TMA unit with the
// 128-byte swizzle (weights: a thread reading its own row meets no bank
// conflict; activations: the canonical K-major operand layout of the MMA).
// Per group of 128 k:
//
//   * each of 256 "row" threads turns its row's 64 bytes into 64 registers of
//     exact bf16 pairs (k, k + 1) and writes them to tensor memory (tcgen05.st)
//     as the A operand of eight K=16 MMAs: lane = row, 8 columns per MMA;
//   * one thread per tile and buffer issues the eight tcgen05.mma (A from tensor
//     memory, B = the activations in the stage) into a per-group accumulator in
//     tensor memory and commits to an mbarrier;
//   * the row threads of the read-back warps fetch the accumulator
//     (tcgen05.ld) and fold it into registers: acc[n] += scale[row, group] * sum[n].
//
// A and D are double buffered in tensor memory (2 tiles x (2 x 64 + 2 x NTOK)
// columns <= 512), so the dequantisation of group g+1 overlaps the MMAs of group
// g and the read-back of group g-1.  Products are exact and sums are fp32, as in
// the streaming kernel; only the summation order differs.  Finished rows go
// through a shared-memory tile and one TMA store per tile, which also clips the
// rows past N and the columns past M.
//
// Nothing is resident per projection, so a CTA moves from one projection to the
// next without any CTA-wide step, and K is not limited by shared memory.
//
// Every wait is bounded; a wait that runs out raises a CTA-wide abort flag, the
// kernel stores ERR_TIMEOUT in the status word, frees its tensor memory and returns.
#include <cuda.h>

#include <cstring>
#include <mutex>
#include <utility>
#include <vector>

#include "common.cuh"
#include "lm_head_pick.cuh"

namespace cb200 {

constexpr int kTcRowsPerTile = 128;
constexpr int kTcTiles = 2;                      // MMA tiles per item
constexpr int kTcItemRows = kTcRowsPerTile * kTcTiles;
constexpr int kTcMaxStages = 4;  // as many as fit, at least 2
constexpr int kTcWeightBytes = kTcItemRows * 128;  // two groups of every row of the item
// a stage: the weights, then four activation boxes of 64 k x NTOK rows (128 bytes per row)
__host__ __device__ constexpr int tc_stage_bytes(int ntok) { return kTcWeightBytes + ntok * 512; }
// output tile of one MMA tile on its way to global memory: [NTOK][128 rows] bf16
__host__ __device__ constexpr int tc_out_bytes(int ntok) { return ntok * kTcRowsPerTile * 2; }
// Warp roles.  Dequantisation and read-back are separate warps so that the
// threads that feed the tensor core never wait for its results.
// Consecutive groups alternate between two A and two D buffers per tile.  Issuing eight
// small MMAs and a commit keeps a single thread busy for longer than the tensor pipe needs
// for them (it competes for issue slots with the arithmetic warps), so every (tile,
// buffer) pair has an issuer of its own: four threads share the issue work, and one
// issuer's waits and commits run while the others' MMAs occupy the pipe.
//   warps 0..7   dequantise: tile = warp >> 2, rows 32 (warp & 3) .. +31 of the tile
//                (a warp reaches only its own quarter of tensor memory)
//   warps 8..15  read the accumulators back and fold them in: same row mapping
//   warp 16      TMA producer
//   warps 17..20 MMA issuers: buffer = (warp - 17) >> 1, tile = (warp - 17) & 1
//   warp 21      output stores: lane 0 for tile 0, lane 1 for tile 1 (so that no
//                read-back thread waits on a store)
//   warps 22,23  idle (register reallocation works on groups of four warps)
constexpr int kTcDequantWarps = 8;
constexpr int kTcFoldWarp0 = 8;
constexpr int kTcProducerWarp = 16;
constexpr int kTcMmaWarp = 17;
constexpr int kTcStoreWarp = 21;  // lanes 0 and 1 issue the TMA stores of tiles 0 and 1
constexpr int kTcThreads = 768;   // 24 warps, 80 registers each at launch
constexpr unsigned long long kTcWaitNs = 400000000ull;

struct alignas(64) TcDesc {
  CUtensorMap tmap;    // weights as uint32 [N][K/8], box 128 rows x 32 words, 128-byte swizzle
  CUtensorMap xmap;    // activations as bf16 [M][K], box NTOK rows x 64 values, 128-byte swizzle
  CUtensorMap ymap;    // outputs as bf16 [M][N], box NTOK rows x 128 values
  CUtensorMap tmap2;   // mode kTcPair: the second (up) matrix, same shape as the first (gate)
  CUtensorMap rmap;    // mode kTcResidual: the residual as bf16 [M][N], box as ymap
  const std::uint16_t* S;
  const std::uint16_t* S2;   // scales of the second matrix
  const std::uint16_t* res;  // mode kTcResidual: residual [M][N]
  std::uint16_t* y;
  int N, K, M;
  int item_begin;   // first unit of this projection in the launch (a unit: one K-slice of one item)
  int cost_begin;   // stage loads before this projection
  // Split K: an item's stages are cut into `split` slices of `slice_stages` stages (the
  // last one may be shorter), each a unit of its own, so that projections with few items
  // still occupy every SM.  The units leave their fp32 sums in `partial`
  // ([item][slice][tile][NTOK][row]); a small follow-up kernel adds the slices up in
  // slice order, applies the residual and stores the outputs (tc_split_combine_kernel).
  int split;
  int slice_stages;
  float* partial;
  int direct_store;  // outputs cannot take the TMA store (base or row pitch off 16 bytes)
  // kTcPlain; kTcPair: out = silu(gate x) * (up x): an item is 128 rows, tile 0 works
  // on the gate matrix and tile 1 on the same rows of the up matrix;
  // kTcResidual: out = res + W x
  int mode;
};
enum : int { kTcPlain = 0, kTcPair = 1, kTcResidual = 2 };
// units of a projection: its items times its K-slices
__host__ __device__ inline int tc_desc_items(const TcDesc& d) {
  return (d.mode == kTcPair ? (d.N + kTcRowsPerTile - 1) / kTcRowsPerTile
                            : (d.N + kTcItemRows - 1) / kTcItemRows) * d.split;
}
// Unit `uu` of projection d: its item, its slice, the first group and the number of groups.
struct TcUnit {
  int j, slice, g_lo, groups;
};
__device__ __forceinline__ TcUnit tc_unit(const TcDesc& d, int uu) {
  TcUnit u;
  u.j = uu / d.split;
  u.slice = uu - u.j * d.split;
  const int G = d.K >> 7;
  u.g_lo = 2 * u.slice * d.slice_stages;
  int g_hi = u.g_lo + 2 * d.slice_stages;
  if (g_hi > G) g_hi = G;
  u.groups = g_hi - u.g_lo;
  return u;
}

struct TcParams {
  TcDesc inl[CUDALM_B200_MAX_INLINE_LINEARS];
  const TcDesc* table;
  int n_stages;
  int n_desc;
  int total_items;
  int total_cost;
  int* status;
  // Launches with a device table: per CTA {first unit, its projection}, gridDim.x + 1
  // entries, cut on the host, so that a CTA finds its range with two loads; a search of
  // the table from the kernel is a chain of dependent global loads (tens of them for the
  // last CTAs of a launch of 48 projections: 12 us before the CTA could start).
  const int2* cta_ranges;
  // Optional (vocabulary projection, one projection per launch; pick.slots non-null):
  // the CTAs keep per activation row the largest bf16-rounded output they have produced
  // and leave it in the table the token pick derives its bounds from (lm_head_pick.cuh).
  PickTail pick;
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
// The eight K=16 MMAs of one quantisation group in one go: D = A[:, 0:16) * B0 and
// then D += A[:, 16j:16j+16) * Bj.  A advances 8 columns per MMA; the B descriptor's
// start-address field (units of 16 bytes) advances 32 bytes per MMA inside an
// activation box and `box_step16` between the group's two boxes.  Issuing a
// tcgen05.mma costs the issuing thread on the order of a hundred cycles, so
// nothing else is computed between them.
__device__ __forceinline__ void tc_mma_group(std::uint32_t d_tmem, std::uint32_t a_tmem,
                                             std::uint32_t desc_lo, std::uint32_t desc_hi,
                                             std::uint32_t box_step16, std::uint32_t idesc) {
  asm volatile(
      "{\n\t"
      ".reg .pred pf, pt;\n\t"
      ".reg .b32 lo, aa;\n\t"
      ".reg .b64 bd;\n\t"
      "setp.ne.b32 pf, 0, 0;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "mov.b64 bd, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], bd, %5, pf;\n\t"
      "add.u32 lo, %2, 2;\n\t mov.b64 bd, {lo, %3};\n\t add.u32 aa, %1, 8;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [aa], bd, %5, pt;\n\t"
      "add.u32 lo, %2, 4;\n\t mov.b64 bd, {lo, %3};\n\t add.u32 aa, %1, 16;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [aa], bd, %5, pt;\n\t"
      "add.u32 lo, %2, 6;\n\t mov.b64 bd, {lo, %3};\n\t add.u32 aa, %1, 24;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [aa], bd, %5, pt;\n\t"
      "add.u32 lo, %2, %4;\n\t mov.b64 bd, {lo, %3};\n\t add.u32 aa, %1, 32;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [aa], bd, %5, pt;\n\t"
      "add.u32 lo, lo, 2;\n\t mov.b64 bd, {lo, %3};\n\t add.u32 aa, %1, 40;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [aa], bd, %5, pt;\n\t"
      "add.u32 lo, lo, 2;\n\t mov.b64 bd, {lo, %3};\n\t add.u32 aa, %1, 48;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [aa], bd, %5, pt;\n\t"
      "add.u32 lo, lo, 2;\n\t mov.b64 bd, {lo, %3};\n\t add.u32 aa, %1, 56;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [aa], bd, %5, pt;\n\t"
      "}"
      :
      : "r"(d_tmem), "r"(a_tmem), "r"(desc_lo), "r"(desc_hi), "r"(box_step16), "r"(idesc)
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
__device__ __forceinline__ void tmem_ld16_nowait(std::uint32_t taddr, std::uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32_nowait(std::uint32_t taddr, std::uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld64_nowait(std::uint32_t taddr, std::uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// NCOL consecutive accumulator columns of this thread's lane, one instruction, one wait
template <int NCOL>
__device__ __forceinline__ void tmem_ld_cols(std::uint32_t taddr, std::uint32_t* r) {
  if (NCOL == 64) tmem_ld64_nowait(taddr, r);
  else if (NCOL == 32) tmem_ld32_nowait(taddr, r);
  else tmem_ld16_nowait(taddr, r);
  tmem_ld_wait();
}

// Shared-memory matrix descriptor of one K=16 slice of the B operand inside an
// activation box: K-major, 128-byte swizzle (rows of 128 bytes, eight rows per
// 1024-byte swizzle atom, so 1024 bytes between 8-row groups); the slice is
// selected by adding its byte offset (32 bytes per K=16) to the start address.
// Descriptor version 1.
__device__ __forceinline__ std::uint64_t tc_b_desc(std::uint32_t smem_addr) {
  std::uint64_t d = 0;
  d |= static_cast<std::uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<std::uint64_t>(1u) << 16;            // leading byte offset: unused with a swizzle
  d |= static_cast<std::uint64_t>(1024u >> 4) << 32;    // stride byte offset
  d |= static_cast<std::uint64_t>(1u) << 46;            // version
  d |= static_cast<std::uint64_t>(2u) << 61;            // 128-byte swizzle
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

// int4 word (k = 8w .. 8w+7, nibble i at bits 4i) -> four exact bf16 pairs
// {q(k), q(k + 1)}, k = 8w, 8w+2, 8w+4, 8w+6, in the natural order of k so that
// the activations need no rearrangement.  Byte b of the word holds nibbles 2b
// (low) and 2b+1 (high); in w >> 4 the same byte position holds nibble 2b+1 in
// its low four bits.  PRMT puts byte b of w into the low half of a register and
// byte b of w >> 4 into the high half; one LOP3 keeps the two low nibbles, flips
// their sign bits (two's complement n -> offset binary u = q + 8) and ORs in the
// bf16 pattern of 128, whose seven mantissa bits then hold u: {128 + u0,
// 128 + u1}, exact; subtracting {136, 136} leaves {q0, q1}, exact.
__device__ __forceinline__ void dequant_word_natural(std::uint32_t w, std::uint32_t* out) {
  const std::uint32_t w4 = w >> 4;
  constexpr std::uint32_t kMagic = 0x43084308u;  // {136, 136} = {128 + 8, 128 + 8}
  out[0] = sub_bf16x2(lop3_and_xor(__byte_perm(w, w4, 0x4400u), 0x000F000Fu, kMagic), kMagic);
  out[1] = sub_bf16x2(lop3_and_xor(__byte_perm(w, w4, 0x5511u), 0x000F000Fu, kMagic), kMagic);
  out[2] = sub_bf16x2(lop3_and_xor(__byte_perm(w, w4, 0x6622u), 0x000F000Fu, kMagic), kMagic);
  out[3] = sub_bf16x2(lop3_and_xor(__byte_perm(w, w4, 0x7733u), 0x000F000Fu, kMagic), kMagic);
}

// Shared-memory map of the kernel.
struct TcSmem {
  std::uint64_t full[kTcMaxStages];
  std::uint64_t empty[kTcMaxStages];
  // [tile][buffer]: the A buffer holds the group (128 dequantising threads) and its D
  // buffer has been read back (128 read-back threads, which arrive once at the start)
  std::uint64_t a_full[kTcTiles][2];
  // the group's MMAs have completed: its A buffer is free again, its D buffer is full
  std::uint64_t mma_done[kTcTiles][2];
  std::uint64_t g_full;   // pair: tile 0's gate outputs are in its buffer
  std::uint64_t g_free;   // pair: tile 1 has taken them
  std::uint64_t res_full[kTcTiles];  // residual: the tile's residual values are in its buffer
  std::uint64_t out_free[kTcTiles];  // the tile's output buffer has been read by its last store
  std::uint64_t out_full[kTcTiles];  // every row thread has written the tile's output buffer
  std::uint32_t tmem_base;
  int abort_flag;
  std::uint32_t row_max[64];  // per activation row: order-preserving key of the CTA's maximum
};
constexpr int kTcHeaderBytes = 1024;

// Order-preserving map of bf16 bits to a 16-bit key (and back to the float value), so
// that an integer max gives the float max.
__device__ __forceinline__ std::uint32_t bf16_key(std::uint32_t bits) {
  const std::uint32_t b = bits & 0xFFFFu;
  return (b & 0x8000u) ? (~b & 0xFFFFu) : (b | 0x8000u);
}
constexpr std::uint32_t kKeyMinusInf = 0x007Fu;  // bf16_key(0xFF80)
// two floats rounded to nearest even into one word of bf16 values (lo in the low half)
__device__ __forceinline__ std::uint32_t pack_bf16x2(float lo, float hi) {
  std::uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ std::uint32_t max_bf16x2(std::uint32_t a, std::uint32_t b) {
  std::uint32_t r;
  asm("max.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ float key_float(std::uint32_t k) {
  const std::uint32_t bits = (k & 0x8000u) ? (k & 0x7FFFu) : (~k & 0xFFFFu);
  return __uint_as_float(bits << 16);
}
static_assert(sizeof(TcSmem) <= kTcHeaderBytes, "barrier block too large");

// Walks the items of a CTA's range, keeping track of the projection they belong to.
struct TcWalk {
  const TcDesc* tbl;
  int d;           // projection of the current item
  int item_end;    // first item after projection d
  int n_desc;
  __device__ __forceinline__ void start(const TcDesc* t, int nd, int d_first) {
    tbl = t;
    n_desc = nd;
    d = d_first;
    item_end = d < nd ? t[d].item_begin + tc_desc_items(t[d]) : 0;
  }
  // true when the item lies in a later projection than the previous one did
  __device__ __forceinline__ bool seek(int item) {
    bool moved = false;
    while (item >= item_end) {
      ++d;
      item_end = tbl[d].item_begin + tc_desc_items(tbl[d]);
      moved = true;
    }
    return moved;
  }
};

// ---------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------
// EXTRA: the launch holds a pair (silu(gate) * up) or a projection with a residual;
// plain launches are compiled without that code (it is large: 64 unrolled epilogues).
template <int NTOK, bool EXTRA>
__global__ void __launch_bounds__(kTcThreads, 1) w4a16_tc_kernel(const __grid_constant__ TcParams p) {
  extern __shared__ __align__(1024) std::uint8_t smem_raw[];
  // the swizzled TMA destinations need 1024-byte alignment; the launch adds the slack
  std::uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  TcSmem* sm = reinterpret_cast<TcSmem*>(smem);
  std::uint8_t* stages = smem + kTcHeaderBytes;  // 1024-byte aligned
  const int kTcStages = p.n_stages;
  constexpr int kStageBytes = tc_stage_bytes(NTOK);
  constexpr int kBoxBytes = NTOK * 128;  // one activation box: NTOK rows x 64 values
  std::uint8_t* outsm = stages + kTcStages * kStageBytes;  // [tile][NTOK][128] bf16
  volatile int* abort_flag = &sm->abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const TcDesc* tbl = p.table ? p.table : p.inl;
  constexpr int kColsPerTile = 128 + 2 * NTOK;
  constexpr std::uint32_t kIdesc = tc_idesc(NTOK);

  if (tid == 0) {
    for (int s = 0; s < kTcStages; ++s) {
      mbar_init(&sm->full[s], 1);
      // every dequantising thread has taken its bytes out, and the MMAs that read the
      // activations are done (one arrival per read-back warp and group, two groups)
      mbar_init(&sm->empty[s], kTcDequantWarps * 32 + 16);
    }
    for (int t = 0; t < kTcTiles; ++t) {
      for (int b = 0; b < 2; ++b) {
        mbar_init(&sm->a_full[t][b], 2 * kTcRowsPerTile);
        mbar_init(&sm->mma_done[t][b], 1);
      }
      if (t == 0) {
        mbar_init(&sm->g_full, kTcRowsPerTile);
        mbar_init(&sm->g_free, kTcRowsPerTile);
      }
      mbar_init(&sm->res_full[t], 1);
      mbar_init(&sm->out_free[t], 1);
      mbar_init(&sm->out_full[t], kTcRowsPerTile);
    }
    sm->abort_flag = 0;
    mbar_init_fence();
  }
  if (tid < 64) sm->row_max[tid] = kKeyMinusInf;
  if (warp == 0) tmem_alloc(&sm->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const std::uint32_t tmem_base = sm->tmem_base;

  // This CTA's contiguous range of items: an equal share of the stage loads.
  int it_lo, it_hi, d_first;
  if (p.cta_ranges != nullptr) {
    const int2 a = __ldg(p.cta_ranges + blockIdx.x), b = __ldg(p.cta_ranges + blockIdx.x + 1);
    it_lo = a.x;
    it_hi = b.x;
    d_first = it_lo >= it_hi ? p.n_desc : a.y;
  } else {
    auto item_at = [&](long long cost) -> int {
      if (cost >= p.total_cost) return p.total_items;
      int lo = 0, hi = p.n_desc - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (tbl[mid].cost_begin <= cost) lo = mid; else hi = mid - 1;
      }
      const int per_item = tbl[lo].slice_stages;
      return tbl[lo].item_begin + static_cast<int>((cost - tbl[lo].cost_begin + per_item - 1) / per_item);
    };
    it_lo = item_at(static_cast<long long>(blockIdx.x) * p.total_cost / gridDim.x);
    it_hi = item_at(static_cast<long long>(blockIdx.x + 1) * p.total_cost / gridDim.x);
    d_first = 0;
    while (d_first + 1 < p.n_desc && tbl[d_first + 1].item_begin <= it_lo) ++d_first;
    if (it_lo >= it_hi) d_first = p.n_desc;
  }

  // Programmatic dependent launch: everything but the copy thread waits here for the
  // preceding kernel; the copy thread first starts the weight copies of its first stages
  // (weights are nobody's output) and waits before the first activation copy.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (warp != kTcProducerWarp) asm volatile("griddepcontrol.wait;" ::: "memory");

  std::uint32_t git = 0;  // groups so far (same count in every role)
  TcWalk wk;
  wk.start(tbl, p.n_desc, d_first);

  // Registers follow the roles (warp groups of four warps; every warp of a group executes
  // the same reallocation before the group's roles part): the read-back warps keep a row
  // of accumulators and half a fetched group sum in registers, the dequantising warps
  // work in chunks of 16 registers, the copy, issue and store warps need next to none.
  // 256 x 56 + 256 x 144 + 256 x 40 is the 768 x 80 the CTA was launched with.
  if (warp >= kTcProducerWarp) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;" ::: "memory");
    if (warp == kTcProducerWarp) {
      // ---------------- TMA producer ----------------
      if (lane == 0) {
        const std::uint64_t policy = policy_evict_first();
        bool ok = true;
        const TcDesc* L = nullptr;
        int item_begin = 0;
        bool pair = false;
        int ps = 0;                  // stage to fill next
        std::uint32_t ps_phase = 0;  // phase its `full` barrier completes next
        bool ps_round = false;       // every stage has been used at least once
        // activation copies held back until the preceding kernel has completed
        const CUtensorMap* pend_map[kTcMaxStages];
        int pend_c[kTcMaxStages];
        int n_pend = 0;
        bool waited = false;
        auto activations = [&](int s, const CUtensorMap* xmap, int c) {
          std::uint8_t* st = stages + s * kStageBytes;
          // four boxes of 64 k each; k past K and rows past M arrive as zeros
          for (int q = 0; q < 4; ++q) {
            asm volatile(
                "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
                " [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(st + kTcWeightBytes + q * kBoxBytes)),
                "l"(xmap), "r"(c * 256 + q * 64), "r"(0), "r"(smem_u32(&sm->full[s]))
                : "memory");
          }
        };
        auto release_pending = [&]() {
          asm volatile("griddepcontrol.wait;" ::: "memory");
          for (int i = 0; i < n_pend; ++i) activations(i, pend_map[i], pend_c[i]);
          waited = true;
        };
        for (int item = it_lo; item < it_hi && ok && !*abort_flag; ++item) {
          if (wk.seek(item) || L == nullptr) {
            L = tbl + wk.d;
            item_begin = L->item_begin;
            pair = L->mode == kTcPair;
          }
          const TcUnit u = tc_unit(*L, item - item_begin);
          const int j = u.j;
          // plain: tiles are consecutive 128-row blocks of one matrix; pair: the same
          // 128 rows of the gate (tile 0) and up (tile 1) matrices
          const int row0 = pair ? j * kTcRowsPerTile : j * kTcItemRows;
          const int tile_step = pair ? 0 : kTcRowsPerTile;
          for (int c = u.g_lo >> 1; c < (u.g_lo + u.groups + 1) >> 1; ++c) {
            // second and later uses of a stage wait until its previous content is done with
            if (ps_round && !tc_wait(&sm->empty[ps], ps_phase ^ 1u, abort_flag)) {
              ok = false;
              break;
            }
            const int s = ps;
            std::uint8_t* st = stages + s * kStageBytes;
            mbar_arrive_expect_tx(&sm->full[s], kStageBytes);
            for (int t = 0; t < kTcTiles; ++t) {
              asm volatile(
                  "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
                  ".L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(
                      smem_u32(st + t * kTcRowsPerTile * 128)),
                  "l"((pair && t == 1) ? &L->tmap2 : &L->tmap), "r"(c * 32), "r"(row0 + t * tile_step),
                  "r"(smem_u32(&sm->full[s])), "l"(policy)
                  : "memory");
            }
            if (waited) {
              activations(s, &L->xmap, c);
            } else {
              // (the first pass over the ring: stage s is the s-th one filled)
              pend_map[n_pend] = &L->xmap;
              pend_c[n_pend] = c;
              if (++n_pend == kTcStages) release_pending();
            }
            if (++ps == kTcStages) {
              ps = 0;
              ps_phase ^= 1u;
              ps_round = true;
            }
          }
        }
        if (!waited) release_pending();
      }
    } else if (warp >= kTcMmaWarp && warp < kTcStoreWarp) {
      // ---------------- MMA issuer, one per buffer and tile ----------------
      if (lane == 0) {
        const std::uint32_t buf = static_cast<std::uint32_t>(warp - kTcMmaWarp) >> 1;  // A and D buffer
        const int t = (warp - kTcMmaWarp) & 1;
        const std::uint32_t desc_hi = static_cast<std::uint32_t>(tc_b_desc(0) >> 32);
        const std::uint32_t desc_lo0 = static_cast<std::uint32_t>(tc_b_desc(0));
        const std::uint32_t stage0 = smem_u32(stages) + kTcWeightBytes;
        const std::uint32_t d_tmem = tmem_base + t * kColsPerTile + 128 + buf * NTOK;
        const std::uint32_t a_tmem = tmem_base + t * kColsPerTile + buf * 64;
        std::uint64_t* const a_full = &sm->a_full[t][buf];
        std::uint64_t* const mma_done = &sm->mma_done[t][buf];
        bool ok = true;
        int s = 0;  // stage of the current group
        for (int item = it_lo; item < it_hi && ok && !*abort_flag; ++item) {
          (void)wk.seek(item);
          const int G = tc_unit(tbl[wk.d], item - tbl[wk.d].item_begin).groups;
          for (int g = 0; g < G; ++g, ++git) {
            if ((git & 1u) == buf) {
              const std::uint32_t b_addr = stage0 + s * kStageBytes + (g & 1) * 2 * kBoxBytes;
              // the A buffer holds the group and the D buffer has been read back; the
              // stage's activations have landed (the row threads saw its barrier
              // complete before they arrived here)
              ok = tc_wait(a_full, (git >> 1) & 1u, abort_flag);
              if (!ok) break;
              tc_fence_after();
              tc_mma_group(d_tmem, a_tmem, desc_lo0 | ((b_addr & 0x3FFFFu) >> 4), desc_hi,
                           kBoxBytes >> 4, kIdesc);
              tc_commit(mma_done);
            }
            if (((g & 1) || g == G - 1) && ++s == kTcStages) s = 0;
          }
        }
      }
    } else if (warp == kTcStoreWarp) {
      // ---------------- output stores, one lane per tile ----------------
      if (lane < kTcTiles) {
        const int tile = lane;
        const TcDesc* L = nullptr;
        int LN = 0, item_begin = 0;
        bool direct = false, pair = false;
        std::uint32_t n_stores = 0;  // items of this tile that went through the output buffer
        bool ok = true;
        for (int item = it_lo; item < it_hi && ok && !*abort_flag; ++item) {
          if (wk.seek(item) || L == nullptr) {
            L = tbl + wk.d;
            LN = L->N;
            item_begin = L->item_begin;
            // (also the outputs of a projection whose K is split: whichever unit ends last
            // stores them)
            direct = L->direct_store != 0 || L->split > 1;
            pair = L->mode == kTcPair;
          }
          if (direct) continue;  // the read-back threads store these rows themselves
          const int j = item - item_begin;
          if (pair && tile == 0) continue;  // a pair's outputs all leave through tile 1's buffer
          const int row0 = pair ? j * kTcRowsPerTile : j * kTcItemRows + tile * kTcRowsPerTile;
          if (EXTRA && L->mode == kTcResidual) {
            // the buffer is free here (the previous store has read it): fetch the tile's
            // residual values into it while the item is being computed
            std::uint8_t* buf = outsm + tile * tc_out_bytes(NTOK);
            if (row0 < LN) {
              mbar_arrive_expect_tx(&sm->res_full[tile], tc_out_bytes(NTOK));
              asm volatile(
                  "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
                  " [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(buf)),
                  "l"(&L->rmap), "r"(row0), "r"(0), "r"(smem_u32(&sm->res_full[tile]))
                  : "memory");
            } else {
              mbar_arrive_expect_tx(&sm->res_full[tile], 0);
            }
          }
          if (!tc_wait(&sm->out_full[tile], n_stores & 1u, abort_flag)) {
            ok = false;
            break;
          }
          if (row0 < LN) {
            asm volatile(
                "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(
                    &L->ymap),
                "r"(row0), "r"(0), "r"(smem_u32(outsm + tile * tc_out_bytes(NTOK)))
                : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          }
          mbar_arrive(&sm->out_free[tile]);
          ++n_stores;
        }
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      }
    }
  } else if (warp < kTcDequantWarps) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;" ::: "memory");
    // ---------------- dequantise and feed the A operand ----------------
    const int tile = warp >> 2;
    const int lrow = (warp & 3) * 32 + lane;  // row inside the tile
    const std::uint32_t lane_base = static_cast<std::uint32_t>((warp & 3) * 32) << 16;
    const std::uint32_t tile_base = tmem_base + tile * kColsPerTile + lane_base;
    bool alive = true;
    int s = 0;                  // stage of the current group
    std::uint32_t s_phase = 0;  // phase of its `full` barrier
    for (int item = it_lo; item < it_hi && alive; ++item) {
      (void)wk.seek(item);
      const int G = tc_unit(tbl[wk.d], item - tbl[wk.d].item_begin).groups;
      for (int g = 0; g < G && alive; ++g, ++git) {
        const int half = g & 1;
        if (half == 0) {
          const bool ok = tc_wait(&sm->full[s], s_phase, abort_flag);
          alive = __all_sync(0xffffffffu, ok);
          if (!alive) break;
        }
        const std::uint8_t* rowp = stages + s * kStageBytes + tile * kTcRowsPerTile * 128 + lrow * 128;
        // The A buffer of this group is free once the MMAs of two groups ago are done,
        // which in a kernel bound by this very loop is long past: wait first, then
        // dequantise and store 16 registers at a time.
        const int buf = git & 1;
        const std::uint32_t use = git >> 1;
        if (use >= 1) {
          const bool ok = tc_wait(&sm->mma_done[tile][buf], (use - 1) & 1u, abort_flag);
          alive = __all_sync(0xffffffffu, ok);
          if (!alive) break;
        }
        tc_fence_after();
        const std::uint32_t a_addr = tile_base + buf * 64;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          std::uint32_t regs[16];
          const uint4 v = lds128(rowp + (((4 * half + q) ^ (lrow & 7)) << 4));
          dequant_word_natural(v.x, regs);
          dequant_word_natural(v.y, regs + 4);
          dequant_word_natural(v.z, regs + 8);
          dequant_word_natural(v.w, regs + 12);
          tmem_st16(a_addr + 16 * q, regs);
        }
        if (half == 1 || g == G - 1) {
          mbar_arrive(&sm->empty[s]);  // this thread has taken its bytes out of the stage
          if (++s == kTcStages) {
            s = 0;
            s_phase ^= 1u;
          }
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        mbar_arrive(&sm->a_full[tile][buf]);
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 144;" ::: "memory");
    // ---------------- read the accumulators back: acc += scale * sum ----------------
    const int fw = warp - kTcFoldWarp0;
    const int tile = fw >> 2;
    // both of the tile's accumulator buffers start out free
    mbar_arrive(&sm->a_full[tile][0]);
    mbar_arrive(&sm->a_full[tile][1]);
    const int lrow = (fw & 3) * 32 + lane;
    const std::uint32_t lane_base = static_cast<std::uint32_t>((fw & 3) * 32) << 16;
    const std::uint32_t tile_base = tmem_base + tile * kColsPerTile + lane_base;
    std::uint8_t* outp = outsm + tile * tc_out_bytes(NTOK) + lrow * 2;
    std::uint32_t eit = 0;      // items of this tile that went through its output buffer
    std::uint32_t n_pairs = 0;  // pair items finished
    std::uint32_t n_res = 0;    // residual items finished
    bool alive = true;
    int fs = 0;  // stage of the current group
    const TcDesc* L = nullptr;
    std::uint16_t* y = nullptr;
    int LN = 0, LM = 0, GK = 0, item_begin = 0, mode = kTcPlain, split = 1;
    bool direct = false;
    for (int item = it_lo; item < it_hi && alive; ++item) {
      if (wk.seek(item) || L == nullptr) {
        L = tbl + wk.d;
        y = L->y;
        LN = L->N;
        LM = L->M;
        GK = L->K >> 7;
        item_begin = L->item_begin;
        split = L->split;
        direct = L->direct_store != 0 || split > 1;
        mode = L->mode;
      }
      const TcUnit u = tc_unit(*L, item - item_begin);
      const int j = u.j;
      const int G = u.groups;
      const bool pair = EXTRA && mode == kTcPair;
      const bool second = pair && tile == 1;         // this tile works on the up matrix
      const bool first_of_pair = pair && tile == 0;  // this tile works on the gate matrix
      const std::uint16_t* S = second ? L->S2 : L->S;
      const int row0 = pair ? j * kTcRowsPerTile : j * kTcItemRows + tile * kTcRowsPerTile;
      const int row = row0 + lrow;
      const bool row_ok = row < LN;
      const std::uint16_t* srow = S + static_cast<std::size_t>(row_ok ? row : 0) * GK + u.g_lo;
      float acc[NTOK];
#pragma unroll
      for (int n = 0; n < NTOK; ++n) acc[n] = 0.f;
      // the scale of the next group is fetched while this one's accumulator is awaited
      std::uint16_t sc_bits = __ldg(srow);
      for (int g = 0; g < G && alive; ++g, ++git) {
        const float sc = row_ok ? __half2float(__ushort_as_half(sc_bits)) : 0.f;
        if (g + 1 < G) sc_bits = __ldg(srow + g + 1);
        const int buf = git & 1;
        const bool ok = tc_wait(&sm->mma_done[tile][buf], (git >> 1) & 1u, abort_flag);
        alive = __all_sync(0xffffffffu, ok);
        if (!alive) break;
        tc_fence_after();
        // the group's MMAs were the last readers of its activations in the stage; a stage
        // that holds one group only gets both of its arrivals from that group
        if (lane == 0) {
          mbar_arrive(&sm->empty[fs]);
          if (g == G - 1 && (g & 1) == 0) mbar_arrive(&sm->empty[fs]);
        }
        if (((g & 1) || g == G - 1) && ++fs == kTcStages) fs = 0;
        const std::uint32_t d_addr = tile_base + 128 + buf * NTOK;
        // at most 32 columns per load (two loads for 64 rows of activations: the register
        // budget does not hold a whole 64-column group sum beside the 64 accumulators)
        constexpr int kCols = NTOK < 32 ? NTOK : 32;
#pragma unroll
        for (int c = 0; c < NTOK / kCols; ++c) {
          std::uint32_t d[kCols];
          tmem_ld_cols<kCols>(d_addr + c * kCols, d);
          if (c == NTOK / kCols - 1) {
            // the accumulator is in registers: hand the buffer back before the arithmetic
            tc_fence_before();
            mbar_arrive(&sm->a_full[tile][buf]);
          }
#pragma unroll
          for (int i = 0; i < kCols; ++i) acc[c * kCols + i] = fmaf(sc, __uint_as_float(d[i]), acc[c * kCols + i]);
        }
      }
      if (!alive) break;
      if (p.pick.slots != nullptr) {
        // Maxima over the warp's 32 weight rows for every activation row at once: the
        // outputs are rounded to bf16 two to a word, and a butterfly of packed bf16
        // maxima that halves the words a lane holds at each step leaves every word
        // reduced over the warp on one lane, which merges it into the CTA's table.
        constexpr int V = NTOK / 2;
        std::uint32_t kv[V];
#pragma unroll
        for (int i = 0; i < V; ++i)
          kv[i] = row_ok ? pack_bf16x2(acc[2 * i], acc[2 * i + 1]) : 0xFF80FF80u;  // -inf, -inf
        int word = 0;  // which word this lane ends up holding
#pragma unroll
        for (int s = 0; s < 5; ++s) {
          const int off = 16 >> s;
          const int cnt = (V >> s) > 1 ? (V >> s) : 1;
          if (cnt > 1) {
            const int half = cnt / 2;
            const bool upper = (lane & off) != 0;
#pragma unroll
            for (int i = 0; i < half; ++i) {
              const std::uint32_t keep = upper ? kv[i + half] : kv[i];
              const std::uint32_t send = upper ? kv[i] : kv[i + half];
              kv[i] = max_bf16x2(keep, __shfl_xor_sync(0xffffffffu, send, off));
            }
            if (upper) word += half;
          } else {
            kv[0] = max_bf16x2(kv[0], __shfl_xor_sync(0xffffffffu, kv[0], off));
          }
        }
        // V = 32: every lane holds a word of its own and merges both halves; fewer
        // words: 32 / V lanes hold the same word and the first two take a half each
        constexpr int kCopies = 32 / V;
        const int copy = lane & (kCopies - 1);
        if (kCopies == 1) {
          if (2 * word < LM) atomicMax(&sm->row_max[2 * word], bf16_key(kv[0] & 0xFFFFu));
          if (2 * word + 1 < LM) atomicMax(&sm->row_max[2 * word + 1], bf16_key(kv[0] >> 16));
        } else if (copy < 2) {
          const int n = 2 * word + copy;
          if (n < LM) atomicMax(&sm->row_max[n], bf16_key(copy ? (kv[0] >> 16) : (kv[0] & 0xFFFFu)));
        }
      }
      if (split > 1) {
        // this unit's sums go to the item's scratch ([activation row][weight row]: a warp's
        // store is 128 contiguous bytes); the follow-up kernel adds the slices up
        float* part = L->partial +
                      ((static_cast<std::size_t>(j) * split + u.slice) * kTcTiles + tile) * kTcRowsPerTile * NTOK + lrow;
#pragma unroll
        for (int n = 0; n < NTOK; ++n) __stcg(part + n * kTcRowsPerTile, acc[n]);
        continue;
      }
      if (direct) {
        // outputs the TMA unit cannot address: plain stores, one row per thread
        if (row_ok) {
#pragma unroll
          for (int n = 0; n < NTOK; ++n)
            if (n < LM) y[static_cast<std::size_t>(n) * LN + row] = float_to_bf16_bits(acc[n]);
        }
        continue;
      }
      // the tile's rows leave through shared memory and one TMA store, issued by the
      // tile's store warp; the buffer is free again once the previous store has read it
      if (first_of_pair) {
        // the gate outputs go to tile 0's buffer, where tile 1's thread of the same
        // row picks them up; the buffer is free once tile 1 has taken the previous ones
        if (n_pairs >= 1) {
          const bool ok = tc_wait(&sm->g_free, (n_pairs - 1) & 1u, abort_flag);
          alive = __all_sync(0xffffffffu, ok);
          if (!alive) break;
        }
#pragma unroll
        for (int n = 0; n < NTOK; ++n)
          *reinterpret_cast<std::uint16_t*>(outp + n * (kTcRowsPerTile * 2)) = float_to_bf16_bits(acc[n]);
        // silu of the rounded gate value, itself rounded, as CUDALM's epilogue forms it;
        // a rolled loop over the thread's own slots keeps the kernel's code small, and
        // tile 1's threads are left with one multiplication per value
#pragma unroll 2
        for (int n = 0; n < NTOK; ++n) {
          std::uint16_t* slot = reinterpret_cast<std::uint16_t*>(outp + n * (kTcRowsPerTile * 2));
          *slot = silu_bits(*slot);
        }
        mbar_arrive(&sm->g_full);
        ++n_pairs;
        continue;
      }
      if (eit >= 1) {
        const bool ok = tc_wait(&sm->out_free[tile], (eit - 1) & 1u, abort_flag);
        alive = __all_sync(0xffffffffu, ok);
        if (!alive) break;
      }
      const std::uint8_t* gate_slots = outsm + lrow * 2;  // tile 0's buffer, this thread's row
      if (second) {
        const bool ok = tc_wait(&sm->g_full, n_pairs & 1u, abort_flag);
        alive = __all_sync(0xffffffffu, ok);
        if (!alive) break;
      }
      if (EXTRA && mode == kTcResidual) {
        // the store lane has brought the tile's residual values into the buffer
        const bool ok = tc_wait(&sm->res_full[tile], n_res & 1u, abort_flag);
        ++n_res;
        alive = __all_sync(0xffffffffu, ok);
        if (!alive) break;
#pragma unroll
        for (int n = 0; n < NTOK; ++n) {
          std::uint16_t* slot = reinterpret_cast<std::uint16_t*>(outp + n * (kTcRowsPerTile * 2));
          *slot = add_bits(*slot, float_to_bf16_bits(acc[n]));
        }
      } else {
#pragma unroll
        for (int n = 0; n < NTOK; ++n)
          *reinterpret_cast<std::uint16_t*>(outp + n * (kTcRowsPerTile * 2)) = float_to_bf16_bits(acc[n]);
      }
      if (EXTRA && second) {
#pragma unroll 8
        for (int n = 0; n < NTOK; ++n) {
          std::uint16_t* slot = reinterpret_cast<std::uint16_t*>(outp + n * (kTcRowsPerTile * 2));
          const std::uint16_t s_bits =
              *reinterpret_cast<const std::uint16_t*>(gate_slots + n * (kTcRowsPerTile * 2));
          *slot = float_to_bf16_bits(bf16_bits_to_float(s_bits) * bf16_bits_to_float(*slot));
        }
      }
      if (second) {
        mbar_arrive(&sm->g_free);
        ++n_pairs;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(&sm->out_full[tile]);
      ++eit;
    }
  }

  __syncthreads();
  if (p.pick.slots != nullptr) {
    // final maxima of this CTA in its slots (every copy of the table); the follow-up launch
    // derives the rows' bounds from them and scans the logits
    const int LM = tbl[0].M;
    for (int i = tid; i < kSlotReplicas * LM; i += kTcThreads) {
      const int r = i / LM, n = i - r * LM;
      if (n < kMaxPassRows)
        p.pick.slots[(static_cast<std::size_t>(r) * LM + n) * gridDim.x + blockIdx.x] = sm->row_max[n] + 1u;
    }
  }
  if (*abort_flag && tid == 0) atomicExch(p.status, CUDALM_B200_ERR_TIMEOUT);
  tc_fence_after();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
}

// Outputs of the projections whose K was split: blockIdx.z is the projection, blockIdx.x
// its 128-row tile, one thread per weight row, blockIdx.y strides over the activation
// rows.  The slices are added in slice order, so the result does not depend on how the
// units were spread over the CTAs.
__global__ void __launch_bounds__(kTcRowsPerTile)
tc_split_combine_kernel(const __grid_constant__ TcParams p, int ntok) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const TcDesc& L = (p.table ? p.table : p.inl)[blockIdx.z];
  if (L.split <= 1) return;
  const int t = blockIdx.x;
  const int lrow = threadIdx.x;
  const int row = t * kTcRowsPerTile + lrow;
  if (row >= L.N) return;
  const bool pair = L.mode == kTcPair;  // an item is one tile of rows: tile 0 gate, tile 1 up
  const int j = pair ? t : t / kTcTiles, tile = pair ? 0 : t - j * kTcTiles;
  const std::size_t slice_floats = static_cast<std::size_t>(kTcTiles) * kTcRowsPerTile * ntok;
  const float* p0 = L.partial + (static_cast<std::size_t>(j) * L.split * kTcTiles + tile) * kTcRowsPerTile * ntok + lrow;
  for (int n = blockIdx.y; n < L.M; n += gridDim.y) {
    float a = 0.f;
    for (int sl = 0; sl < L.split; ++sl) a += __ldcg(p0 + sl * slice_floats + n * kTcRowsPerTile);
    const std::size_t at = static_cast<std::size_t>(n) * L.N + row;
    std::uint16_t bits = float_to_bf16_bits(a);
    if (pair) {
      // CUDALM's rounding order: bf16 after each projection, after silu, after the product
      float b = 0.f;
      const float* p1 = p0 + static_cast<std::size_t>(kTcRowsPerTile) * ntok;
      for (int sl = 0; sl < L.split; ++sl) b += __ldcg(p1 + sl * slice_floats + n * kTcRowsPerTile);
      bits = float_to_bf16_bits(bf16_bits_to_float(silu_bits(bits)) * bf16_bits_to_float(float_to_bf16_bits(b)));
    } else if (L.mode == kTcResidual) {
      bits = add_bits(L.res[at], bits);
    }
    L.y[at] = bits;
  }
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

// A 2-D tensor map: `inner` x `outer` elements with a row pitch of inner * esize
// bytes, box `box_inner` x `box_outer`.  The decode loop passes the same
// pointers step after step, so encodings are kept in a small direct-mapped cache.
struct TcMapKey {
  const void* base = nullptr;
  int inner = 0, outer = 0, box_inner = 0, box_outer = 0, kind = 0;
};
struct TcMapEntry {
  TcMapKey key;
  CUtensorMap map;
};
constexpr int kTcMapCache = 1024;

int tc_encode(const void* base, int inner, int outer, int box_inner, int box_outer, int kind,
              CUtensorMap* out) {
  // kind 0: packed weights as uint32, 128-byte swizzle; 1: activations as bf16, 128-byte
  // swizzle; 2: outputs as bf16, no swizzle
  static std::mutex mu;
  static TcMapEntry cache[kTcMapCache];
  const std::uintptr_t h = reinterpret_cast<std::uintptr_t>(base);
  const int slot = static_cast<int>(((h >> 4) ^ (h >> 15) ^ static_cast<std::uintptr_t>(inner) * 31u ^
                                     static_cast<std::uintptr_t>(outer) * 131u ^
                                     static_cast<std::uintptr_t>(kind) * 7919u ^
                                     static_cast<std::uintptr_t>(box_outer) * 17u) % kTcMapCache);
  {
    std::lock_guard<std::mutex> lk(mu);
    const TcMapEntry& e = cache[slot];
    if (e.key.base == base && e.key.inner == inner && e.key.outer == outer &&
        e.key.box_inner == box_inner && e.key.box_outer == box_outer && e.key.kind == kind) {
      *out = e.map;
      return CUDALM_B200_OK;
    }
  }
  EncodeTiledFn fn = tc_encode_fn();
  if (!fn) return CUDALM_B200_ERR_CUDA;
  const int esize = kind == 0 ? 4 : 2;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(inner) * esize};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_outer)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r =
      fn(out, kind == 0 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 2,
         const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
         kind == 2 ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = static_cast<int>(r);
    return CUDALM_B200_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lk(mu);
  cache[slot].key = TcMapKey{base, inner, outer, box_inner, box_outer, kind};
  cache[slot].map = *out;
  return CUDALM_B200_OK;
}

int tc_ntok(int M) { return M <= 16 ? 16 : (M <= 32 ? 32 : 64); }

template <int NTOK, bool EXTRA = false>
int tc_launch(const TcParams& p_in, cudaStream_t stream, int* grid_out = nullptr, int max_grid = 0) {
  auto kern = w4a16_tc_kernel<NTOK, EXTRA>;
  constexpr int kFixed = 1024 + kTcHeaderBytes + kTcTiles * tc_out_bytes(NTOK);
  int n_stages = (kMaxSmemBytes - kFixed) / tc_stage_bytes(NTOK);
  if (n_stages > kTcMaxStages) n_stages = kTcMaxStages;
  if (n_stages < 2) return CUDALM_B200_ERR_UNSUPPORTED;
  TcParams p = p_in;
  p.n_stages = n_stages;
  const int smem = kFixed + n_stages * tc_stage_bytes(NTOK);
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
  if (max_grid > 0 && grid > max_grid) grid = max_grid;
  if (grid_out) *grid_out = grid;
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

// True when the tensor-memory kernel takes this projection: the TMA unit needs
// 16-byte aligned bases for the weights and activations (their row pitches are
// multiples of 64 bytes already).  Outputs that it cannot address (base or row
// pitch off 16 bytes) are stored with plain stores instead.
bool tc_eligible(const cudalm_b200_linear& l) {
  if (l.M < 1 || l.M > 64 || l.K <= 0 || (l.K % 128) != 0 || l.N < 1) return false;
  return aligned_to(l.weight, 16) && aligned_to(l.x, 16);
}

// Scratch of the projections whose K is split (TcDesc::partial, ::tickets).
struct TcScratchPlan {
  size_t bytes = 0;  // the partial sums of every split projection
  int tiles = 0;     // most 128-row tiles of any split projection: the combine kernel's grid.x
};

// Fills `out[count]` and the launch totals; UNSUPPORTED when a projection does
// not meet the kernel's alignment rules.  `pair`: the one projection is a gate/up pair
// (the caller adds the second matrix).  With `scratch` non-null, a launch with few
// 128-row tiles (at most one per SM: the length of one item's chain of groups, not the
// bytes, then sets the time) has the K of its projections from K = 2048 on split into
// slices of two stages (four groups), and `scratch` receives the size of the memory the
// caller has to provide through tc_bind_scratch; with `scratch` null nothing is split.
// Launches with more tiles are not split: measured on 96 items of 28 groups, the extra
// traffic and the per-unit costs outweigh the shorter chains (29 -> 37 us).
int tc_describe(const cudalm_b200_linear* ls, int count, TcDesc* out, int* items_out,
                int* cost_out, int* ntok_out, TcScratchPlan* scratch = nullptr, bool pair = false) {
  int items = 0, cost = 0, ntok = 0;
  long long tiles = 0;
  for (int i = 0; i < count; ++i) {
    if (!tc_eligible(ls[i])) return CUDALM_B200_ERR_UNSUPPORTED;
    ntok = tc_ntok(ls[i].M) > ntok ? tc_ntok(ls[i].M) : ntok;
    tiles += pair ? 2ll * ((ls[i].N + kTcRowsPerTile - 1) / kTcRowsPerTile)
                  : static_cast<long long>(kTcTiles) * ((ls[i].N + kTcItemRows - 1) / kTcItemRows);
  }
  const bool few_tiles = scratch != nullptr && tiles <= num_sms();
  size_t partial_floats = 0;
  int split_tiles = 0;
  for (int i = 0; i < count; ++i) {
    const cudalm_b200_linear& l = ls[i];
    TcDesc& d = out[i];
    if (int rc = tc_encode(l.weight, l.K / 8, l.N, 32, kTcRowsPerTile, 0, &d.tmap)) return rc;
    if (int rc = tc_encode(l.x, l.K, l.M, 64, ntok, 1, &d.xmap)) return rc;
    d.direct_store = (!aligned_to(l.y, 16) || (l.N % 8) != 0) ? 1 : 0;
    if (!d.direct_store)
      if (int rc = tc_encode(l.y, l.N, l.M, kTcRowsPerTile, ntok, 2, &d.ymap)) return rc;
    d.S = l.scales;
    d.S2 = nullptr;
    d.res = nullptr;
    d.mode = pair ? kTcPair : kTcPlain;
    d.y = l.y;
    d.N = l.N;
    d.K = l.K;
    d.M = l.M;
    d.item_begin = items;
    d.cost_begin = cost;
    const int n_items = pair ? (l.N + kTcRowsPerTile - 1) / kTcRowsPerTile : (l.N + kTcItemRows - 1) / kTcItemRows;
    const int stages = ((l.K >> 7) + 1) >> 1;
    const int split = (few_tiles && stages >= 8) ? stages / 2 : 1;
    d.slice_stages = (stages + split - 1) / split;
    d.split = (stages + d.slice_stages - 1) / d.slice_stages;  // no empty slice
    d.partial = nullptr;
    if (d.split > 1) {
      const int out_tiles = pair ? n_items : n_items * kTcTiles;
      if (out_tiles > split_tiles) split_tiles = out_tiles;
      partial_floats += static_cast<size_t>(n_items) * d.split * kTcItemRows * ntok;
    }
    items += n_items * d.split;
    cost += n_items * d.split * d.slice_stages;
  }
  if (scratch) {
    scratch->bytes = partial_floats * sizeof(float);
    scratch->tiles = split_tiles;
  }
  *items_out = items;
  *cost_out = cost;
  *ntok_out = ntok;
  return CUDALM_B200_OK;
}

// Points the split projections of `tbl` into `mem` (TcScratchPlan::bytes, 256-byte aligned).
void tc_bind_scratch(TcDesc* tbl, int count, int ntok, void* mem) {
  float* partial = static_cast<float*>(mem);
  for (int i = 0; i < count; ++i) {
    TcDesc& d = tbl[i];
    if (d.split <= 1) continue;
    const int n_items = tc_desc_items(d) / d.split;
    d.partial = partial;
    partial += static_cast<size_t>(n_items) * d.split * kTcItemRows * ntok;
  }
}

// The follow-up launch of a launch with split projections.
int tc_launch_combine(const TcParams& p, int ntok, int tiles, cudaStream_t stream) {
  if (tiles <= 0) return CUDALM_B200_OK;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(tiles), 16u, static_cast<unsigned>(p.n_desc));
  cfg.blockDim = dim3(kTcRowsPerTile);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t le = cudaLaunchKernelEx(&cfg, tc_split_combine_kernel, p, ntok);
  if (le != cudaSuccess) {
    g_last_cuda_error = static_cast<int>(le);
    (void)cudaGetLastError();
    return CUDALM_B200_ERR_CUDA;
  }
  return check_launch();
}

// The library's own memory pool of a device for the stream-ordered scratch below (its
// release threshold is unlimited, so that a decode loop's allocations are served from
// memory the pool already holds; the device's default pool is left alone).
cudaMemPool_t tc_scratch_pool() {
  static std::mutex mu;
  static std::vector<std::pair<int, cudaMemPool_t>> pools;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> lk(mu);
  for (const auto& e : pools)
    if (e.first == dev) return e.second;
  cudaMemPoolProps props = {};
  props.allocType = cudaMemAllocationTypePinned;
  props.handleTypes = cudaMemHandleTypeNone;
  props.location.type = cudaMemLocationTypeDevice;
  props.location.id = dev;
  cudaMemPool_t pool = nullptr;
  if (cudaMemPoolCreate(&pool, &props) != cudaSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  unsigned long long keep = ~0ull;
  (void)cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
  pools.emplace_back(dev, pool);
  return pool;
}

// Stream-ordered scratch for one launch: allocated before it, freed after it.
struct TcCallScratch {
  void* mem = nullptr;
  cudaStream_t stream = nullptr;
  int acquire(const TcScratchPlan& plan, cudaStream_t st) {
    stream = st;
    if (plan.bytes == 0) return CUDALM_B200_OK;
    cudaMemPool_t pool = tc_scratch_pool();
    if (pool) {
      CB200_CUDA_TRY(cudaMallocFromPoolAsync(&mem, plan.bytes, pool, st));
    } else {
      CB200_CUDA_TRY(cudaMallocAsync(&mem, plan.bytes, st));
    }
    return CUDALM_B200_OK;
  }
  ~TcCallScratch() {
    if (mem) (void)cudaFreeAsync(mem, stream);
  }
};

int tc_run_params(TcParams& p, int ntok, cudaStream_t stream, int* grid_out = nullptr, int max_grid = 0) {
  p.status = device_status_word();
  if (!p.status) return CUDALM_B200_ERR_CUDA;
  if (ntok == 16) return tc_launch<16>(p, stream, grid_out, max_grid);
  if (ntok == 32) return tc_launch<32>(p, stream, grid_out, max_grid);
  return tc_launch<64>(p, stream, grid_out, max_grid);
}

// One projection with an MLP epilogue: weight2/scales2 non-null -> out = silu(W x) * (W2 x),
// residual non-null -> out = residual + W x.  UNSUPPORTED unless the outputs can take
// the TMA store and the second matrix is 16-byte aligned.
int run_tc_extra(const cudalm_b200_linear& l, const std::uint8_t* weight2,
                 const std::uint16_t* scales2, const std::uint16_t* residual, cudaStream_t stream) {
  TcParams p;
  std::memset(&p, 0, sizeof(p));
  int ntok = 0;
  TcScratchPlan plan;
  if (weight2 && (!aligned_to(weight2, 16) || !scales2)) return CUDALM_B200_ERR_UNSUPPORTED;
  if (int rc = tc_describe(&l, 1, p.inl, &p.total_items, &p.total_cost, &ntok, &plan, weight2 != nullptr))
    return rc;
  TcDesc& d = p.inl[0];
  if (d.direct_store) return CUDALM_B200_ERR_UNSUPPORTED;
  TcCallScratch scratch;
  if (int rc = scratch.acquire(plan, stream)) return rc;
  if (scratch.mem) tc_bind_scratch(p.inl, 1, ntok, scratch.mem);
  if (weight2) {
    if (int rc = tc_encode(weight2, l.K / 8, l.N, 32, kTcRowsPerTile, 0, &d.tmap2)) return rc;
    d.S2 = scales2;
  } else if (residual) {
    if (!aligned_to(residual, 16)) return CUDALM_B200_ERR_UNSUPPORTED;
    if (int rc = tc_encode(residual, l.N, l.M, kTcRowsPerTile, ntok, 2, &d.rmap)) return rc;
    d.res = residual;
    d.mode = kTcResidual;
  }
  p.n_desc = 1;
  p.status = device_status_word();
  if (!p.status) return CUDALM_B200_ERR_CUDA;
  const int rc = ntok == 16   ? tc_launch<16, true>(p, stream)
                 : ntok == 32 ? tc_launch<32, true>(p, stream)
                              : tc_launch<64, true>(p, stream);
  if (rc != CUDALM_B200_OK) return rc;
  return tc_launch_combine(p, ntok, plan.tiles, stream);
}

// The vocabulary projection: one projection whose CTAs also collect the candidates of
// the token pick.  The grid is bounded by the pick's slot table before anything is enqueued.
int run_tc_with_pick(const cudalm_b200_linear& l, const PickTail& pick, cudaStream_t stream, int* grid_out) {
  TcParams p;
  std::memset(&p, 0, sizeof(p));
  int ntok = 0;
  if (int rc = tc_describe(&l, 1, p.inl, &p.total_items, &p.total_cost, &ntok)) return rc;
  p.n_desc = 1;
  p.pick = pick;
  return tc_run_params(p, ntok, stream, grid_out, kTailMaxCtas);
}

// Up to CUDALM_B200_MAX_INLINE_LINEARS projections in one launch.
int run_tc(const cudalm_b200_linear* ls, int count, cudaStream_t stream) {
  if (count < 1 || count > CUDALM_B200_MAX_INLINE_LINEARS) return CUDALM_B200_ERR_BAD_SHAPE;
  TcParams p;
  std::memset(&p, 0, sizeof(p));
  int ntok = 0;
  TcScratchPlan plan;
  if (int rc = tc_describe(ls, count, p.inl, &p.total_items, &p.total_cost, &ntok, &plan)) return rc;
  TcCallScratch scratch;
  if (int rc = scratch.acquire(plan, stream)) return rc;
  if (scratch.mem) tc_bind_scratch(p.inl, count, ntok, scratch.mem);
  p.n_desc = count;
  if (int rc = tc_run_params(p, ntok, stream)) return rc;
  return tc_launch_combine(p, ntok, plan.tiles, stream);
}

// Any number of projections: the descriptor table lives on the device.
struct TcGroup {
  TcDesc* table_dev = nullptr;
  int2* ranges_dev = nullptr;  // per-CTA ranges for `grid` CTAs
  int grid = 0;
  void* scratch = nullptr;  // of the projections whose K is split; the group's for its lifetime
  int count = 0, items = 0, cost = 0, ntok = 0, split_tiles = 0;
};

int tc_group_create(const cudalm_b200_linear* ls, int count, TcGroup** out) {
  std::vector<TcDesc> tbl(static_cast<size_t>(count));
  TcGroup* g = new TcGroup();
  g->count = count;
  TcScratchPlan plan;
  if (int rc = tc_describe(ls, count, tbl.data(), &g->items, &g->cost, &g->ntok, &plan)) {
    delete g;
    return rc;
  }
  cudaError_t e = cudaSuccess;
  if (plan.bytes) {
    e = cudaMalloc(&g->scratch, plan.bytes);
    if (e == cudaSuccess) tc_bind_scratch(tbl.data(), count, g->ntok, g->scratch);
    g->split_tiles = plan.tiles;
  }
  if (e == cudaSuccess) e = cudaMalloc(&g->table_dev, sizeof(TcDesc) * tbl.size());
  if (e == cudaSuccess)
    e = cudaMemcpy(g->table_dev, tbl.data(), sizeof(TcDesc) * tbl.size(), cudaMemcpyHostToDevice);
  // the CTAs' ranges: equal shares of the stage loads, as the kernel cuts them itself
  // for launches without a device table
  g->grid = num_sms() < g->items ? num_sms() : g->items;
  std::vector<int2> ranges(static_cast<size_t>(g->grid) + 1);
  {
    auto unit_at = [&](long long cost) -> int {
      if (cost >= g->cost) return g->items;
      int lo = 0, hi = count - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (tbl[static_cast<size_t>(mid)].cost_begin <= cost) lo = mid; else hi = mid - 1;
      }
      const TcDesc& d = tbl[static_cast<size_t>(lo)];
      return d.item_begin + static_cast<int>((cost - d.cost_begin + d.slice_stages - 1) / d.slice_stages);
    };
    int d = 0;
    for (int b = 0; b <= g->grid; ++b) {
      const int u = unit_at(static_cast<long long>(b) * g->cost / g->grid);
      while (d + 1 < count && tbl[static_cast<size_t>(d) + 1].item_begin <= u) ++d;
      ranges[static_cast<size_t>(b)] = make_int2(u, d);
    }
  }
  if (e == cudaSuccess) e = cudaMalloc(&g->ranges_dev, sizeof(int2) * ranges.size());
  if (e == cudaSuccess)
    e = cudaMemcpy(g->ranges_dev, ranges.data(), sizeof(int2) * ranges.size(), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    g_last_cuda_error = static_cast<int>(e);
    if (g->table_dev) cudaFree(g->table_dev);
    if (g->ranges_dev) cudaFree(g->ranges_dev);
    if (g->scratch) cudaFree(g->scratch);
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
  p.cta_ranges = g->ranges_dev;
  if (int rc = tc_run_params(p, g->ntok, stream, nullptr, g->grid)) return rc;
  return tc_launch_combine(p, g->ntok, g->split_tiles, stream);
}

void tc_group_destroy(TcGroup* g) {
  if (!g) return;
  cudaFree(g->table_dev);
  if (g->ranges_dev) cudaFree(g->ranges_dev);
  if (g->scratch) cudaFree(g->scratch);
  delete g;
}

}  // namespace cb200

