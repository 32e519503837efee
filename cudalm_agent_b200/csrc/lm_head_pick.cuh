// Device side of the token pick that follows the vocabulary projection: candidate
// collection, ranking, and the exchange of candidates between vocabulary-parallel
// ranks.  Included by the projection kernels (whose last CTA finishes the pick) and
// by lm_head.cu (stand-alone pick, merge and exchange kernels).
//
// Ordering rule (CUDALM include/cudalm/greedy.h:28-39 and
// include/cudalm/sampling.h:152-166): candidates are ordered by their bf16 logit,
// descending, compared as floats (so -0 ties with +0); ties go to the lower token
// id.  Element 0 of the top-k list is therefore the argmax.
//
// Candidates are 64-bit composites: bits 63..48 = the bf16 logit mapped to an
// unsigned key that grows with the value, bits 47..16 = ~id, bits 15..0 = the
// logit's original bits, so that one unsigned compare implements the ordering
// rule and the value can be reported unchanged.
//
// How a call finds its candidates:
//   * every CTA of the projection keeps, per activation row, the largest logit it has
//     produced and leaves it (as key + 1; 0 means "nothing") in a table of one slot per
//     CTA at its end;
//   * the follow-up launch, several CTAs per activation row, takes the k-th largest slot
//     of the row as a bound: it is a lower bound on the k-th largest logit of the whole
//     vocabulary, because every slot is the largest logit of a different set of rows.
//     Each CTA scans its slice of the row's logits (still in L2) and appends those at or
//     above the bound to the row's candidate list (typically 50-150 entries out of
//     248,320); the CTA that finishes a row's scan last ranks the candidates, exchanges
//     them with the other ranks when the vocabulary is split, and leaves the row's
//     counter, ticket and slots cleared for the next call.
// A row whose candidate list overflows (e.g. all logits equal) is redone by an exact
// search over the full row.
//
// (Finishing the pick inside the projection kernel -- candidates from each CTA's own
// rows, ranked by one CTA of the same launch -- was built and measured: 39-40 us per call
// at M = 1 against 38-39 us with the follow-up launch, because every step of that tail is
// a dependent round trip to L2 of about a microsecond on the critical path of the last
// CTA, while the follow-up launch spreads the same steps over many CTAs.)
#pragma once

#include "common.cuh"

namespace cb200 {

constexpr int kMaxTopK = 64;
constexpr int kCandCap = 2048;     // candidate slots per row
constexpr int kMaxPassRows = 32;   // activation rows per pass
constexpr int kMaxCtas = 2048;     // words per activation row in the table of per-CTA maxima
constexpr int kTailMaxCtas = 256;  // largest grid whose CTAs pick in the projection kernel
// The table of maxima is kept in several copies, each on lines of its own: every CTA
// reads the whole table at about the same time, and requests for one line of L2 are
// served one after the other (about 45 ns each), so one copy would cost every call
// 148 x 45 ns.  A CTA writes all copies and reads copy blockIdx % kSlotReplicas.  Inside
// a copy the slots of one activation row are contiguous, so that the warp that works out
// a row's bound touches a handful of lines.
constexpr int kSlotReplicas = kMaxCtas / kTailMaxCtas;
constexpr int kSelectThreads = 256;
constexpr int kMaxPeers = 8;

struct SelectArgs {
  // candidate source A: composites collected by the scan, cand[m][0 .. counts[m]) (a
  // count above kCandCap: overflow); the count is cleared once read
  const std::uint64_t* cand;
  int* counts;
  // candidate source B: lists[l][m][k] of ids and values (ids < 0 are padding)
  const std::int32_t* list_idx;
  const std::uint16_t* list_val;
  int n_lists;
  int list_k;
  long long idx_stride;  // elements from one list's ids to the next list's
  long long val_stride;  // likewise for the values
  // full logits of this shard, for the exact search after an overflow
  const std::uint16_t* logits;
  int N;
  int id_offset;
  int rows;
  int k;
  std::int32_t* argmax_out;
  std::int32_t* topk_idx;
  std::uint16_t* topk_val;
};

// Candidate exchange between vocabulary-parallel ranks.  A rank's buffer holds, in
// 64-bit words, lists [2][world][slot_words] and then its per-row epochs (32-bit).
// Every word carries its own validity: {id (32 bits), epoch tag (16), bf16 value
// (16)}, written by one 8-byte store, so neither a fence nor a separate flag crosses
// NVLink: a receiver polls the words themselves.  Lists are double buffered by the
// parity of the row's epoch: a rank can be at most one call ahead of a peer that is
// still merging, since the call after needs that peer's next words.
struct ExchangeArgs {
  unsigned long long* bufs[kMaxPeers];  // every rank's buffer as mapped here; bufs[rank] is local
  const std::int32_t* local_packed;     // this rank's picks: ids [rows_cap][k], then bf16 values
  int rank, world, slot_words, rows_cap, M, k;
  long long wait_ns;                    // limit of the wait for the peers' words
  std::int32_t* argmax_out;
  std::int32_t* topk_idx;
  std::uint16_t* topk_val;
  int* status;
};

// What a projection kernel needs to leave its maxima for the pick.
struct PickTail {
  std::uint32_t* slots;   // [kSlotReplicas][M][grid]: key + 1 of each CTA's largest logit per row
  int M;
};

#ifdef __CUDACC__

// bf16 bits -> unsigned key that increases with the float value; -0 maps to +0.
__device__ __forceinline__ std::uint32_t order_key(std::uint16_t bits) {
  std::uint32_t b = bits;
  if (b == 0x8000u) b = 0u;
  return (b & 0x8000u) ? (~b & 0xFFFFu) : (b | 0x8000u);
}
__device__ __forceinline__ std::uint64_t make_composite(std::uint16_t bits, std::uint32_t id) {
  return (static_cast<std::uint64_t>(order_key(bits)) << 48) |
         (static_cast<std::uint64_t>(static_cast<std::uint32_t>(~id)) << 16) | bits;
}
__device__ __forceinline__ std::uint32_t composite_id(std::uint64_t c) {
  return ~static_cast<std::uint32_t>(c >> 16);
}
__device__ __forceinline__ std::uint16_t composite_bits(std::uint64_t c) {
  return static_cast<std::uint16_t>(c & 0xFFFFu);
}

// Barrier over the kSelectThreads threads that rank and exchange (the first 256 of
// a projection CTA, or a whole CTA of the stand-alone kernels).
__device__ __forceinline__ void pick_sync() {
  asm volatile("bar.sync 2, %0;" ::"n"(kSelectThreads) : "memory");
}

__device__ __forceinline__ long long global_ns() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

struct SelectSmem {
  std::uint64_t buf[kCandCap];
  int scratch[kSelectThreads / 32];
  int take;
  int ok;
};

// Bitonic sort, descending, of n (a power of two) composites in shared memory.
__device__ inline void bitonic_sort_desc(std::uint64_t* a, int n, int tid) {
  for (int size = 2; size <= n; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      pick_sync();
      for (int i = tid; i < (n >> 1); i += kSelectThreads) {
        const int lo = 2 * i - (i & (stride - 1));
        const int hi = lo + stride;
        const bool desc = (lo & size) == 0;
        const std::uint64_t x = a[lo], y = a[hi];
        if ((x < y) == desc) {
          a[lo] = y;
          a[hi] = x;
        }
      }
    }
  }
  pick_sync();
}

// Sum of one int per thread over the kSelectThreads threads (result to every thread).
__device__ inline int block_sum(int v, int* scratch, int tid) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  pick_sync();
  if ((tid & 31) == 0) scratch[tid >> 5] = v;
  pick_sync();
  int total = 0;
  for (int w = 0; w < (kSelectThreads >> 5); ++w) total += scratch[w];
  return total;
}

// Ranks the n composites in sm.buf and writes row m's pick.
__device__ inline void rank_and_write(const SelectArgs& a, int m, int n, int tid, SelectSmem& sm) {
  std::uint64_t* buf = sm.buf;
  pick_sync();
  if (n <= kSelectThreads) {
    // the usual case, a few dozen candidates: every thread ranks its own candidate by
    // counting (equal composites, which only padding produces, rank in slot order)
    const std::uint64_t mine = tid < n ? buf[tid] : 0ull;
    int rank = 0;
    if (tid < n)
      for (int j = 0; j < n; ++j) {
        const std::uint64_t other = buf[j];
        rank += (other > mine) || (other == mine && j < tid);
      }
    pick_sync();
    if (tid < n) buf[rank] = mine;
    pick_sync();
  } else {
    // pad to a power of two with zeros, which sort last
    int P = 64;
    while (P < n) P <<= 1;
    for (int i = n + tid; i < P; i += kSelectThreads) buf[i] = 0ull;
    bitonic_sort_desc(buf, P, tid);
  }
  const int kk = a.k;
  for (int j = tid; j < kk; j += kSelectThreads) {
    const std::uint64_t c = buf[j];
    const bool real = (j < n) && c != 0ull;
    a.topk_idx[static_cast<size_t>(m) * kk + j] = real ? static_cast<std::int32_t>(composite_id(c)) : -1;
    a.topk_val[static_cast<size_t>(m) * kk + j] =
        real ? composite_bits(c) : static_cast<std::uint16_t>(0xFF80u);
    if (j == 0 && a.argmax_out) a.argmax_out[m] = real ? static_cast<std::int32_t>(composite_id(c)) : -1;
  }
}

// The pick of row m by kSelectThreads threads.
__device__ inline void select_row(const SelectArgs& a, int m, int tid, SelectSmem& sm) {
  std::uint64_t* buf = sm.buf;
  int* scratch = sm.scratch;
  int n = 0;
  bool overflow = false;
  if (a.cand) {
    // written by other CTAs of this launch: read from L2
    n = __ldcg(a.counts + m);
    overflow = n > kCandCap;
    if (!overflow)
      for (int i = tid; i < n; i += kSelectThreads)
        buf[i] = __ldcg(a.cand + static_cast<size_t>(m) * kCandCap + i);
    pick_sync();
    if (tid == 0) a.counts[m] = 0;  // every thread has read the count: clear it for the next call
  } else {
    n = a.n_lists * a.list_k;  // host guarantees n <= kCandCap
    for (int i = tid; i < n; i += kSelectThreads) {
      const int l = i / a.list_k, j = i - l * a.list_k;
      const size_t within = static_cast<size_t>(m) * a.list_k + j;
      const std::int32_t id = __ldcg(a.list_idx + static_cast<size_t>(l) * a.idx_stride + within);
      const std::uint16_t v = __ldcg(a.list_val + static_cast<size_t>(l) * a.val_stride + within);
      buf[i] = id < 0 ? 0ull : make_composite(v, static_cast<std::uint32_t>(id));
    }
  }

  if (overflow) {
    // Exact search over the whole row.  (1) bisection on the 16-bit value key
    // for the k-th largest value; (2) everything above it is taken; (3) of the
    // entries equal to it, the lowest ids are taken by an ordered scan.
    const std::uint16_t* row = a.logits + static_cast<size_t>(m) * a.N;
    const int kk = a.k < a.N ? a.k : a.N;
    std::uint32_t T = 0;
    for (int bit = 15; bit >= 0; --bit) {
      const std::uint32_t trial = T | (1u << bit);
      int c = 0;
      for (int i = tid; i < a.N; i += kSelectThreads) c += order_key(__ldcg(row + i)) >= trial;
      if (block_sum(c, scratch, tid) >= kk) T = trial;
    }
    int c = 0;
    for (int i = tid; i < a.N; i += kSelectThreads) c += order_key(__ldcg(row + i)) > T;
    const int n_gt = block_sum(c, scratch, tid);
    if (tid == 0) sm.take = 0;
    pick_sync();
    // entries above T: any order (sorted below)
    for (int i = tid; i < a.N; i += kSelectThreads) {
      const std::uint16_t bits = __ldcg(row + i);
      if (order_key(bits) > T) {
        const int pos = atomicAdd(&sm.take, 1);
        buf[pos] = make_composite(bits, static_cast<std::uint32_t>(a.id_offset + i));
      }
    }
    pick_sync();
    // entries equal to T, in id order, until kk are taken
    int need = kk - n_gt;
    for (int base = 0; base < a.N && need > 0; base += kSelectThreads) {
      const int i = base + tid;
      const std::uint16_t bits = i < a.N ? __ldcg(row + i) : static_cast<std::uint16_t>(0);
      const bool eq = i < a.N && order_key(bits) == T;
      // rank of this thread among the block's matches
      const unsigned ballot = __ballot_sync(0xffffffffu, eq);
      pick_sync();
      if ((tid & 31) == 0) scratch[tid >> 5] = __popc(ballot);
      pick_sync();
      int before = 0, total = 0;
      for (int w = 0; w < kSelectThreads / 32; ++w) {
        if (w < (tid >> 5)) before += scratch[w];
        total += scratch[w];
      }
      const int rank = before + __popc(ballot & ((1u << (tid & 31)) - 1u));
      if (eq && rank < need)
        buf[n_gt + (kk - n_gt - need) + rank] = make_composite(bits, static_cast<std::uint32_t>(a.id_offset + i));
      need -= total < need ? total : need;
    }
    n = kk;
    pick_sync();
  }
  rank_and_write(a, m, n, tid, sm);
}

// ---- exchange between ranks ---------------------------------------------------------
__device__ __forceinline__ void st_word_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_word_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ std::uint32_t* exchange_epochs(const ExchangeArgs& e) {
  return reinterpret_cast<std::uint32_t*>(e.bufs[e.rank] + 2ull * e.world * e.slot_words);
}

// Row m's local pick (in e.local_packed) into slot [rank] of every rank's buffer.
__device__ inline void exchange_send_row(const ExchangeArgs& e, int m, int tid) {
  const std::uint32_t epoch = exchange_epochs(e)[m] + 1u;  // advanced at the end of the receive
  const unsigned long long tag = static_cast<unsigned long long>(epoch & 0xFFFFu) << 48;
  const int k = e.k;
  const std::int32_t* src_idx = e.local_packed + static_cast<size_t>(m) * k;
  const std::uint16_t* src_val =
      reinterpret_cast<const std::uint16_t*>(e.local_packed + static_cast<size_t>(e.rows_cap) * k) +
      static_cast<size_t>(m) * k;
  const size_t at = (static_cast<size_t>(epoch & 1u) * e.world + e.rank) * e.slot_words + static_cast<size_t>(m) * k;
  for (int i = tid; i < e.world * k; i += kSelectThreads) {
    const int p = i / k, j = i - p * k;
    const unsigned long long w = static_cast<unsigned long long>(static_cast<std::uint32_t>(src_idx[j])) |
                                 (static_cast<unsigned long long>(src_val[j]) << 32) | tag;
    st_word_sys(e.bufs[p] + at + j, w);
  }
}

// Waits for every rank's words of row m (time limit e.wait_ns) and merges them into the
// final pick.  When a rank's words do not arrive the status word reads TIMEOUT and the
// row's outputs are ids -1 with values -inf, so that the miss shows in the data.
__device__ inline void exchange_recv_row(const ExchangeArgs& e, int m, int tid, SelectSmem& sm) {
  std::uint32_t* epochs = exchange_epochs(e);
  const std::uint32_t epoch = epochs[m] + 1u;
  const unsigned long long tag = epoch & 0xFFFFu;
  const int k = e.k, n = e.world * k;
  const unsigned long long* mine = e.bufs[e.rank] + static_cast<size_t>(epoch & 1u) * e.world * e.slot_words;
  if (tid == 0) sm.ok = 1;
  pick_sync();
  bool ok = true;
  const long long t0 = global_ns();
  for (int i = tid; i < n; i += kSelectThreads) {
    const int src = i / k, j = i - src * k;
    const unsigned long long* w = mine + static_cast<size_t>(src) * e.slot_words + static_cast<size_t>(m) * k + j;
    unsigned long long v = ld_word_sys(w);
    while (ok && (v >> 48) != tag) {
      if (global_ns() - t0 > e.wait_ns) {
        ok = false;
        break;
      }
      __nanosleep(40);
      v = ld_word_sys(w);
    }
    const std::int32_t id = static_cast<std::int32_t>(static_cast<std::uint32_t>(v));
    sm.buf[i] = (!ok || id < 0) ? 0ull : make_composite(static_cast<std::uint16_t>((v >> 32) & 0xFFFFu),
                                                         static_cast<std::uint32_t>(id));
  }
  if (!ok) {
    sm.ok = 0;
    atomicExch(e.status, CUDALM_B200_ERR_TIMEOUT);
  }
  pick_sync();
  if (tid == 0) epochs[m] = epoch;  // every thread has read the previous value
  SelectArgs a;
  a.k = k;
  a.argmax_out = e.argmax_out;
  a.topk_idx = e.topk_idx;
  a.topk_val = e.topk_val;
  if (!sm.ok) {
    for (int j = tid; j < k; j += kSelectThreads) {
      a.topk_idx[static_cast<size_t>(m) * k + j] = -1;
      a.topk_val[static_cast<size_t>(m) * k + j] = static_cast<std::uint16_t>(0xFF80u);
      if (j == 0 && a.argmax_out) a.argmax_out[m] = -1;
    }
    pick_sync();
    return;
  }
  rank_and_write(a, m, n, tid, sm);
}

// ---- the table of per-CTA maxima ---------------------------------------------------------
// Publishes a CTA's maxima (shared-memory keys + 1) in its slots of every copy of the
// table; called by a whole warp.
__device__ __forceinline__ void tail_publish(const PickTail& t, const std::uint32_t* row_key, int lane) {
  const int grid = static_cast<int>(gridDim.x);
  for (int i = lane; i < kSlotReplicas * t.M; i += 32) {
    const int r = i / t.M, m = i - r * t.M;
    t.slots[(static_cast<size_t>(r) * t.M + m) * grid + blockIdx.x] = row_key[m];
  }
}

// The k-th largest of the `grid` slots of one activation row (`row_slots`, a row of one
// copy of the table), by one warp.  Slot values are keys + 1; the result is 0 when fewer
// than k slots hold a value, which lets everything pass.
__device__ inline std::uint32_t row_bound(const std::uint32_t* row_slots, int grid, int k, int lane) {
  constexpr int kPerLane = kTailMaxCtas / 32;
  std::uint32_t key[kPerLane];
#pragma unroll
  for (int j = 0; j < kPerLane; ++j) {
    const int c = lane + 32 * j;
    key[j] = c < grid ? __ldcg(row_slots + c) : 0u;
  }
  std::uint32_t T = 0;
  for (int bit = 16; bit >= 0; --bit) {
    const std::uint32_t trial = T | (1u << bit);
    int c = 0;
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) c += key[j] >= trial;
    c = __reduce_add_sync(0xffffffffu, c);
    if (c >= k) T = trial;
  }
  return T;
}

#endif  // __CUDACC__

}  // namespace cb200
