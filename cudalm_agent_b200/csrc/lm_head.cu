// Vocabulary projection with an on-device token pick: W4A16 GEMV over the
// vocabulary rows, then argmax and top-k per activation row.
//
// Ordering rule (CUDALM include/cudalm/greedy.h:28-39 and
// include/cudalm/sampling.h:152-166): candidates are ordered by their bf16
// logit value, descending, compared as floats (so -0 ties with +0); ties go to
// the lower token id.  Element 0 of the top-k list is therefore the argmax.
//
// Three launches per call, all on the caller's stream:
//   1. the streaming projection kernel writes the bf16 logits and, per CTA and
//      activation row, the largest logit that CTA produced;
//   2. collect: the k-th largest of those per-CTA maxima is a lower bound on the
//      k-th largest logit (each maximum is a distinct logit), so only logits
//      at or above it can be in the top-k; they are appended to a per-row
//      candidate list (typically 50-150 entries out of the whole vocabulary);
//   3. select: one CTA per row sorts its candidates by (value desc, id asc) and
//      writes the first k.  A row whose candidate list overflowed (e.g. all
//      logits equal) is redone by an exact search over the full row.
//
// Candidates are 64-bit composites: bits 63..48 = the bf16 logit mapped to an
// unsigned key that grows with the value, bits 47..16 = ~id, bits 15..0 = the
// logit's original bits, so that one unsigned compare implements the ordering
// rule and the value can be reported unchanged.
#include <cstring>

#include "common.cuh"

namespace cb200 {

int run_linear_with_cta_max(const cudalm_b200_linear& l, float* cta_max, int* grid_out,
                            cudaStream_t stream, int* clear_words, int clear_count);
int stream_rows_per_pass(int K);
int run_linear_any(const cudalm_b200_linear& l, cudaStream_t stream);

namespace {

constexpr int kMaxTopK = 64;
constexpr int kCandCap = 2048;     // candidate slots per row
constexpr int kMaxPassRows = 32;   // activation rows per pass
constexpr int kMaxCtas = 1024;     // per-CTA maxima slots
constexpr int kSelectThreads = 256;

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

struct Workspace {
  int* counts;              // [kMaxPassRows] candidates per row, then [kMaxPassRows] scan tickets per row
  float* cta_max;           // [kMaxCtas][rows]
  std::uint64_t* cand;      // [rows][kCandCap]
  std::uint16_t* logits;    // [rows][N] when the caller gave no logits buffer
};

constexpr size_t kCountsBytes = 256;

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

size_t workspace_layout(int N, int rows, bool need_logits, unsigned char* base, Workspace* ws) {
  size_t off = 0;
  if (ws) ws->counts = reinterpret_cast<int*>(base + off);
  off += kCountsBytes;
  if (ws) ws->cta_max = reinterpret_cast<float*>(base + off);
  off += align_up(static_cast<size_t>(kMaxCtas) * rows * sizeof(float), 256);
  if (ws) ws->cand = reinterpret_cast<std::uint64_t*>(base + off);
  off += align_up(static_cast<size_t>(rows) * kCandCap * sizeof(std::uint64_t), 256);
  if (ws) ws->logits = reinterpret_cast<std::uint16_t*>(base + off);
  if (need_logits) off += align_up(static_cast<size_t>(rows) * N * sizeof(std::uint16_t), 256);
  return off;
}

// ---------------------------------------------------------------------------
// The scan of one CTA of grid (slices, rows): the row's bound from the per-CTA
// maxima (smax: kMaxCtas floats of shared memory), then the CTA's slice of the
// row's logits; values at or above the bound become candidates.
// ---------------------------------------------------------------------------
__device__ void scan_slice(const std::uint16_t* __restrict__ logits, int N, int rows,
                           const float* __restrict__ cta_max, int ncta, int k, int id_offset,
                           int* counts, std::uint64_t* cand, float* smax) {
  __shared__ float bound;
  const int m = blockIdx.y;
  const int tid = threadIdx.x;
  for (int i = tid; i < ncta; i += blockDim.x) smax[i] = cta_max[static_cast<size_t>(i) * rows + m];
  if (tid == 0) bound = -INFINITY;
  __syncthreads();
  if (ncta >= k) {
    // the entry with exactly k-1 entries ahead of it (value desc, index asc)
    for (int i = tid; i < ncta; i += blockDim.x) {
      const float v = smax[i];
      int ahead = 0;
      for (int j = 0; j < ncta; ++j) {
        const float u = smax[j];
        ahead += (u > v) || (u == v && j < i);
      }
      if (ahead == k - 1) bound = v;
    }
  }
  __syncthreads();
  const float b = bound;
  const std::uint16_t* row = logits + static_cast<size_t>(m) * N;
  // slices are whole 16-byte vectors of the row, so that a row on a 16-byte
  // boundary is read eight values at a time, several loads in flight per thread
  long long per = (static_cast<long long>(N) + gridDim.x - 1) / gridDim.x;
  per = (per + 7) & ~7ll;
  const long long lo = per * blockIdx.x;
  long long hi = lo + per;
  if (hi > N) hi = N;
  if (lo >= hi) return;  // (uniform over the CTA)
  auto offer = [&](std::uint16_t bits, long long i) {
    if (bf16_bits_to_float(bits) >= b) {
      const int pos = atomicAdd(&counts[m], 1);
      if (pos < kCandCap)
        cand[static_cast<size_t>(m) * kCandCap + pos] =
            make_composite(bits, static_cast<std::uint32_t>(id_offset) + static_cast<std::uint32_t>(i));
    }
  };
  long long done = lo;
  if ((reinterpret_cast<std::uintptr_t>(row) & 15u) == 0) {
    const uint4* vrow = reinterpret_cast<const uint4*>(row + lo);
    const long long nv = (hi - lo) >> 3;
    constexpr int kInFlight = 8;
    for (long long v0 = tid; v0 < nv; v0 += static_cast<long long>(kInFlight) * blockDim.x) {
      uint4 q[kInFlight];
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) {
        const long long v = v0 + static_cast<long long>(u) * blockDim.x;
        q[u] = v < nv ? __ldg(vrow + v) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) {
        const long long v = v0 + static_cast<long long>(u) * blockDim.x;
        if (v >= nv) break;
        const std::uint32_t w[4] = {q[u].x, q[u].y, q[u].z, q[u].w};
        const long long i0 = lo + (v << 3);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          offer(static_cast<std::uint16_t>(w[e] & 0xFFFFu), i0 + 2 * e);
          offer(static_cast<std::uint16_t>(w[e] >> 16), i0 + 2 * e + 1);
        }
      }
    }
    done = lo + (nv << 3);
  }
  for (long long i = done + tid; i < hi; i += blockDim.x) offer(row[i], i);
}

// Bitonic sort, descending, of n (a power of two) composites in shared memory.
__device__ void bitonic_sort_desc(std::uint64_t* a, int n, int tid, int nthreads) {
  for (int size = 2; size <= n; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      __syncthreads();
      for (int i = tid; i < (n >> 1); i += nthreads) {
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
  __syncthreads();
}

// CTA-wide sum of one int per thread (result to every thread).
__device__ int block_sum(int v, int* scratch, int tid, int nthreads) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  __syncthreads();
  if ((tid & 31) == 0) scratch[tid >> 5] = v;
  __syncthreads();
  int total = 0;
  for (int w = 0; w < (nthreads >> 5); ++w) total += scratch[w];
  return total;
}

// ---------------------------------------------------------------------------
// select: one CTA per row.  Also used to merge already-selected lists (the
// vocabulary-parallel case), which arrive as (id, bf16 value) pairs.
// ---------------------------------------------------------------------------
struct SelectArgs {
  // candidate source A: composites collected by lm_head_collect_kernel
  const std::uint64_t* cand;
  const int* counts;
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

struct SelectSmem {
  std::uint64_t buf[kCandCap];
  int scratch[kSelectThreads / 32];
  int take;
};

// The pick of row m by one CTA of kSelectThreads threads.
__device__ void select_row(const SelectArgs& a, int m, int tid, SelectSmem& sm) {
  std::uint64_t* buf = sm.buf;
  int* scratch = sm.scratch;
  int& s_take = sm.take;
  int n = 0;
  bool overflow = false;
  if (a.cand) {
    // written by other CTAs of the same launch when the scan's last CTA picks: read from L2
    n = __ldcg(a.counts + m);
    overflow = n > kCandCap;
    if (!overflow)
      for (int i = tid; i < n; i += kSelectThreads)
        buf[i] = __ldcg(a.cand + static_cast<size_t>(m) * kCandCap + i);
  } else {
    n = a.n_lists * a.list_k;  // host guarantees n <= kCandCap
    for (int i = tid; i < n; i += kSelectThreads) {
      const int l = i / a.list_k, j = i - l * a.list_k;
      const size_t within = static_cast<size_t>(m) * a.list_k + j;
      // read from L2: a peer GPU may have written the lists into this GPU's memory
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
      for (int i = tid; i < a.N; i += kSelectThreads) c += order_key(row[i]) >= trial;
      if (block_sum(c, scratch, tid, kSelectThreads) >= kk) T = trial;
    }
    int c = 0;
    for (int i = tid; i < a.N; i += kSelectThreads) c += order_key(row[i]) > T;
    const int n_gt = block_sum(c, scratch, tid, kSelectThreads);
    if (tid == 0) s_take = 0;
    __syncthreads();
    // entries above T: any order (sorted below)
    for (int i = tid; i < a.N; i += kSelectThreads) {
      if (order_key(row[i]) > T) {
        const int pos = atomicAdd(&s_take, 1);
        buf[pos] = make_composite(row[i], static_cast<std::uint32_t>(a.id_offset + i));
      }
    }
    __syncthreads();
    // entries equal to T, in id order, until kk are taken
    int need = kk - n_gt;
    for (int base = 0; base < a.N && need > 0; base += kSelectThreads) {
      const int i = base + tid;
      const bool eq = i < a.N && order_key(row[i]) == T;
      // rank of this thread among the block's matches
      const unsigned ballot = __ballot_sync(0xffffffffu, eq);
      __syncthreads();
      if ((tid & 31) == 0) scratch[tid >> 5] = __popc(ballot);
      __syncthreads();
      int before = 0, total = 0;
      for (int w = 0; w < kSelectThreads / 32; ++w) {
        if (w < (tid >> 5)) before += scratch[w];
        total += scratch[w];
      }
      const int rank = before + __popc(ballot & ((1u << (tid & 31)) - 1u));
      if (eq && rank < need)
        buf[n_gt + (kk - n_gt - need) + rank] =
            make_composite(row[i], static_cast<std::uint32_t>(a.id_offset + i));
      need -= total < need ? total : need;
    }
    n = kk;
    __syncthreads();
  }

  __syncthreads();
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
    __syncthreads();
    if (tid < n) buf[rank] = mine;
    __syncthreads();
  } else {
    // pad to a power of two with zeros, which sort last
    int P = 64;
    while (P < n) P <<= 1;
    for (int i = n + tid; i < P; i += kSelectThreads) buf[i] = 0ull;
    bitonic_sort_desc(buf, P, tid, kSelectThreads);
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

__global__ void __launch_bounds__(kSelectThreads)
lm_head_select_kernel(const SelectArgs a) {
  __shared__ SelectSmem sm;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  select_row(a, blockIdx.x, threadIdx.x, sm);
}

constexpr int kMaxPeers = 8;
constexpr long long kExchangeWaitNs = 2000000000ll;  // 2 s

struct ExchangeArgs {
  std::uint32_t* bufs[kMaxPeers];  // every rank's buffer as mapped here; bufs[rank] is the local one
  const std::int32_t* local_packed;
  int rank, world, words_per_list, rows_cap, M, k;
  std::int32_t* argmax_out;
  std::int32_t* topk_idx;
  std::uint16_t* topk_val;
  int* status;
};

__device__ __forceinline__ void st_release_sys(std::uint32_t* p, std::uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ std::uint32_t ld_acquire_sys(const std::uint32_t* p) {
  std::uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ long long global_ns() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Row m's exchange and merge by one CTA of kSelectThreads threads.
__device__ void exchange_row(const ExchangeArgs& e, int m, int tid, SelectSmem& sm) {
  __shared__ int s_ok;
  const size_t lists_words = static_cast<size_t>(e.world) * e.words_per_list;
  std::uint32_t* mine = e.bufs[e.rank];
  std::uint32_t* my_flags = mine + 2 * lists_words;
  std::uint32_t* my_epochs = my_flags + static_cast<size_t>(e.world) * kMaxPassRows;
  const std::uint32_t epoch = my_epochs[m] + 1u;  // written only by this row's CTA, one call earlier
  const size_t parity_off = (epoch & 1u) * lists_words;

  // (1) this rank's candidates of row m into slot [rank] of every rank's buffer
  const int k = e.k;
  const size_t val_base = static_cast<size_t>(e.rows_cap) * k;  // in words: values start here
  const std::int32_t* src_idx = e.local_packed + static_cast<size_t>(m) * k;
  const std::uint16_t* src_val =
      reinterpret_cast<const std::uint16_t*>(e.local_packed + val_base) + static_cast<size_t>(m) * k;
  for (int i = tid; i < e.world * 2 * k; i += kSelectThreads) {
    const int p = i / (2 * k), j = i - p * 2 * k;
    std::uint32_t* slot = e.bufs[p] + parity_off + static_cast<size_t>(e.rank) * e.words_per_list;
    if (j < k)
      slot[static_cast<size_t>(m) * k + j] = static_cast<std::uint32_t>(src_idx[j]);
    else
      (reinterpret_cast<std::uint16_t*>(slot + val_base))[static_cast<size_t>(m) * k + (j - k)] = src_val[j - k];
  }
  // (2) the row's epoch on every rank, (3) wait for every rank's.  The CTA's stores are
  // ordered before the flags by the barrier and the publishing threads' own fence
  // (fences are cumulative), so only `world` threads pay a system-wide fence.
  if (tid == 0) s_ok = 1;
  __syncthreads();
  if (tid < e.world) {
    __threadfence_system();
    std::uint32_t* peer_flags = e.bufs[tid] + 2 * lists_words;
    st_release_sys(peer_flags + static_cast<size_t>(e.rank) * kMaxPassRows + m, epoch);
    const std::uint32_t* f = my_flags + static_cast<size_t>(tid) * kMaxPassRows + m;
    const long long t0 = global_ns();
    bool ok = true;
    while (static_cast<std::int32_t>(ld_acquire_sys(f) - epoch) < 0) {
      if (global_ns() - t0 > kExchangeWaitNs) {
        ok = false;
        break;
      }
      __nanosleep(100);
    }
    if (!ok) {
      s_ok = 0;
      atomicExch(e.status, CUDALM_B200_ERR_TIMEOUT);
    }
  }
  __syncthreads();
  if (tid == 0) my_epochs[m] = epoch;
  if (!s_ok) return;  // a rank did not arrive: the status word says so, nothing is merged

  // (4) merge the lists that arrived here
  SelectArgs a;
  a.cand = nullptr;
  a.counts = nullptr;
  const std::uint32_t* lists = mine + parity_off;
  a.list_idx = reinterpret_cast<const std::int32_t*>(lists);
  a.list_val = reinterpret_cast<const std::uint16_t*>(lists + val_base);
  a.n_lists = e.world;
  a.list_k = k;
  a.idx_stride = e.words_per_list;
  a.val_stride = 2ll * e.words_per_list;
  a.logits = nullptr;
  a.N = 0;
  a.id_offset = 0;
  a.rows = e.M;
  a.k = k;
  a.argmax_out = e.argmax_out;
  a.topk_idx = e.topk_idx;
  a.topk_val = e.topk_val;
  select_row(a, m, tid, sm);
}

__global__ void __launch_bounds__(kSelectThreads)
topk_exchange_merge_kernel(const ExchangeArgs e) {
  __shared__ SelectSmem sm;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  exchange_row(e, blockIdx.x, threadIdx.x, sm);
}

// ---------------------------------------------------------------------------
// scan + pick: grid (slices, rows).  Each CTA derives the row's bound from the
// per-CTA maxima and scans its slice of the row's logits for candidates; the
// CTA that finishes a row's scan last (a ticket per row) picks the row's
// tokens, so the call needs no third launch.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kSelectThreads)
lm_head_scan_pick_kernel(const std::uint16_t* __restrict__ logits, int N, int rows,
                         const float* __restrict__ cta_max, int ncta, int k, int id_offset,
                         int* counts, int* tickets, std::uint64_t* cand, const SelectArgs a,
                         const ExchangeArgs e) {
  __shared__ SelectSmem sm;
  __shared__ int s_last;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int m = blockIdx.y;
  const int tid = threadIdx.x;
  scan_slice(logits, N, rows, cta_max, ncta, k, id_offset, counts, cand, reinterpret_cast<float*>(sm.buf));
  // this CTA's candidates and count are visible before its ticket: the barrier orders
  // them before thread 0's fence, which is cumulative
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    s_last = atomicAdd(&tickets[m], 1) == static_cast<int>(gridDim.x) - 1;
    __threadfence();
  }
  __syncthreads();
  if (!s_last) return;
  select_row(a, m, tid, sm);
  if (e.world >= 1) {  // 0: no exchange
    // vocabulary-parallel: the same CTA sends the row's pick to the other ranks and
    // merges theirs (its own global stores are visible to it after the barrier)
    __syncthreads();
    exchange_row(e, m, tid, sm);
  }
}

__global__ void zero_counts_kernel(int* counts, int n) {
  if (threadIdx.x < n) counts[threadIdx.x] = 0;
}

}  // namespace
}  // namespace cb200

using namespace cb200;

namespace cb200 {
namespace {
// Launch that may overlap its predecessor's tail (the kernel waits with
// griddepcontrol.wait before it reads anything).
template <typename... KArgs, typename... Args>
int launch_after(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t le = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (le != cudaSuccess) {
    g_last_cuda_error = static_cast<int>(le);
    (void)cudaGetLastError();
    return CUDALM_B200_ERR_CUDA;
  }
  return check_launch();
}
}  // namespace
}  // namespace cb200

extern "C" {

size_t cudalm_b200_lm_head_workspace_bytes(int N, int K, int M, int top_k, int need_logits) {
  (void)K;
  (void)top_k;
  if (N < 1 || M < 1) return 0;
  const int rows = M < kMaxPassRows ? M : kMaxPassRows;
  return workspace_layout(N, rows, need_logits != 0, nullptr, nullptr);
}

// `ex` non-null: the rows' picks are also exchanged with the other ranks and merged
// by the CTA that made them (one pass only).
static int lm_head_topk_impl(const uint8_t* weight, const uint16_t* scales, const uint16_t* x,
                             int N, int K, int M, int top_k, int id_offset,
                             uint16_t* logits_out, int32_t* argmax_out, int32_t* topk_idx,
                             uint16_t* topk_val, void* workspace, size_t workspace_bytes,
                             void* stream, const ExchangeArgs* ex) {
  if (!weight || !scales || !x || !topk_idx || !topk_val) return CUDALM_B200_ERR_NULL;
  if (N < 1 || K <= 0 || (K % 128) != 0 || M < 1 || id_offset < 0) return CUDALM_B200_ERR_BAD_SHAPE;
  if (top_k < 1 || top_k > kMaxTopK) return CUDALM_B200_ERR_TOO_LARGE;
  if (!workspace) return CUDALM_B200_ERR_WORKSPACE;
  if (!aligned_to(workspace, 256)) return CUDALM_B200_ERR_MISALIGNED;
  if (workspace_bytes < cudalm_b200_lm_head_workspace_bytes(N, K, M, top_k, logits_out == nullptr))
    return CUDALM_B200_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  int per_pass = stream_rows_per_pass(K);
  if (per_pass > kMaxPassRows) per_pass = kMaxPassRows;
  const bool staged = per_pass > 0 && aligned_to(weight, 16);
  if (!staged) per_pass = kMaxPassRows;
  const int rows_cap = M < kMaxPassRows ? M : kMaxPassRows;

  if (ex && M > per_pass) return CUDALM_B200_ERR_UNSUPPORTED;
  ExchangeArgs no_exchange;
  std::memset(&no_exchange, 0, sizeof(no_exchange));

  for (int m0 = 0; m0 < M; m0 += per_pass) {
    const int rows = (M - m0 < per_pass) ? (M - m0) : per_pass;
    Workspace ws;
    workspace_layout(N, rows_cap, logits_out == nullptr, static_cast<unsigned char*>(workspace), &ws);
    // the maxima table is indexed [cta][rows of this pass]
    uint16_t* logits = logits_out ? logits_out + static_cast<size_t>(m0) * N : ws.logits;
    cudalm_b200_linear l{weight, scales, x + static_cast<size_t>(m0) * K, logits, N, K, rows, 0};

    int ncta = 0;
    if (staged) {
      // the projection's first CTA also clears the candidate counters
      if (int rc = run_linear_with_cta_max(l, ws.cta_max, &ncta, st, ws.counts, 2 * kMaxPassRows)) return rc;
      if (ncta > kMaxCtas) return CUDALM_B200_ERR_TOO_LARGE;
    } else {
      // no per-CTA maxima on the slow path: every logit is a candidate, and a
      // row longer than the candidate list takes the exact search
      zero_counts_kernel<<<1, 64, 0, st>>>(ws.counts, 2 * kMaxPassRows);
      if (int rc = check_launch()) return rc;
      if (int rc = run_linear_any(l, st)) return rc;
      ncta = 0;
    }

    // every CTA first ranks the per-CTA maxima to find the row's bound, so the scan is
    // cut into few, long slices: about two CTAs per SM over all rows
    int slices = (N + 4095) / 4096;
    const int cap = (2 * num_sms() + rows - 1) / rows;
    if (slices > cap) slices = cap;
    if (slices < 1) slices = 1;
    SelectArgs a;
    std::memset(&a, 0, sizeof(a));
    a.cand = ws.cand;
    a.counts = ws.counts;
    a.logits = logits;
    a.N = N;
    a.id_offset = id_offset;
    a.rows = rows;
    a.k = top_k;
    a.argmax_out = argmax_out ? argmax_out + m0 : nullptr;
    a.topk_idx = topk_idx + static_cast<size_t>(m0) * top_k;
    a.topk_val = topk_val + static_cast<size_t>(m0) * top_k;
    if (int rc = launch_after(lm_head_scan_pick_kernel, dim3(slices, rows), dim3(kSelectThreads), st,
                              static_cast<const std::uint16_t*>(logits), N, rows,
                              static_cast<const float*>(ws.cta_max), ncta, top_k, id_offset, ws.counts,
                              ws.counts + kMaxPassRows, ws.cand, a, ex ? *ex : no_exchange))
      return rc;
  }
  return CUDALM_B200_OK;
}

int cudalm_b200_lm_head_topk(const uint8_t* weight, const uint16_t* scales, const uint16_t* x,
                             int N, int K, int M, int top_k, int id_offset,
                             uint16_t* logits_out, int32_t* argmax_out, int32_t* topk_idx,
                             uint16_t* topk_val, void* workspace, size_t workspace_bytes,
                             void* stream) {
  return lm_head_topk_impl(weight, scales, x, N, K, M, top_k, id_offset, logits_out, argmax_out,
                           topk_idx, topk_val, workspace, workspace_bytes, stream, nullptr);
}

int cudalm_b200_topk_merge(const int32_t* list_idx, const uint16_t* list_val, int n_lists, int M,
                           int k, int32_t* argmax_out, int32_t* topk_idx, uint16_t* topk_val,
                           void* stream) {
  if (!list_idx || !list_val || !topk_idx || !topk_val) return CUDALM_B200_ERR_NULL;
  if (n_lists < 1 || M < 1 || k < 1) return CUDALM_B200_ERR_BAD_SHAPE;
  if (k > kMaxTopK || static_cast<long long>(n_lists) * k > kCandCap) return CUDALM_B200_ERR_TOO_LARGE;
  SelectArgs a;
  std::memset(&a, 0, sizeof(a));
  a.list_idx = list_idx;
  a.list_val = list_val;
  a.n_lists = n_lists;
  a.list_k = k;
  a.idx_stride = static_cast<long long>(M) * k;
  a.val_stride = static_cast<long long>(M) * k;
  a.rows = M;
  a.k = k;
  a.argmax_out = argmax_out;
  a.topk_idx = topk_idx;
  a.topk_val = topk_val;
  lm_head_select_kernel<<<M, kSelectThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return check_launch();
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Allocation-free variant of the vocabulary projection.
//
// Some callers of this library may not allocate device memory at the moment
// they need a token pick: an inference server that has handed all of the GPU's
// memory to its own pools at start-up, a decode step that runs inside a
// latency-critical loop where a cudaMalloc (which synchronises the device) is
// forbidden, or a host language binding that has no allocator for device
// memory at all.  For them the scratch that cudalm_b200_lm_head_topk takes as
// `workspace` lives here instead, in a fixed array inside the library's device
// image.  Every GPU that loads the library holds these bytes until the process
// exits.  The caller still passes every input and output, the logits buffer
// included.
//
// The array's name is a host-side stand-in in host code, not a device address:
// the address is taken once per device with cudaGetSymbolAddress, with that
// device current, and that pointer is what the kernels receive.
// ---------------------------------------------------------------------------
namespace cb200 {
namespace {

constexpr int kStaticMaxRows = 32;  // activation rows per call
// counts + per-CTA maxima + candidate lists for kStaticMaxRows rows (the same
// layout workspace_layout() produces for a caller-provided logits buffer)
constexpr size_t kStaticScratchBytes =
    kCountsBytes + static_cast<size_t>(kMaxCtas) * kStaticMaxRows * sizeof(float) +
    static_cast<size_t>(kStaticMaxRows) * kCandCap * sizeof(std::uint64_t);

static __device__ __align__(256) unsigned char g_lm_head_scratch[kStaticScratchBytes];

// Device address of the scratch array on the current device (looked up once per
// device; the first call on a device performs the lookup).
int static_scratch(void** out) {
  static std::atomic<void*> cached[64];
  int dev = 0;
  CB200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return CUDALM_B200_ERR_UNSUPPORTED;
  void* p = cached[dev].load(std::memory_order_acquire);
  if (!p) {
    const cudaError_t e = cudaGetSymbolAddress(&p, g_lm_head_scratch);
    if (e != cudaSuccess || p == nullptr) {
      g_last_cuda_error = static_cast<int>(e);
      return CUDALM_B200_ERR_CUDA;
    }
    cached[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return CUDALM_B200_OK;
}

}  // namespace
}  // namespace cb200

extern "C" {

size_t cudalm_b200_lm_head_static_scratch_bytes(void) { return cb200::kStaticScratchBytes; }

int cudalm_b200_lm_head_topk_static(const uint8_t* weight, const uint16_t* scales,
                                    const uint16_t* x, int N, int K, int M, int top_k,
                                    int id_offset, uint16_t* logits_out, int32_t* argmax_out,
                                    int32_t* topk_idx, uint16_t* topk_val, void* stream) {
  if (!logits_out) return CUDALM_B200_ERR_NULL;  // the logits are an output here, never scratch
  if (M > cb200::kStaticMaxRows) return CUDALM_B200_ERR_TOO_LARGE;
  if (M >= 1 && N >= 1 &&
      cudalm_b200_lm_head_workspace_bytes(N, K, M, top_k, 0) > cb200::kStaticScratchBytes)
    return CUDALM_B200_ERR_TOO_LARGE;
  void* scratch = nullptr;
  if (int rc = cb200::static_scratch(&scratch)) return rc;
  return cudalm_b200_lm_head_topk(weight, scales, x, N, K, M, top_k, id_offset, logits_out,
                                  argmax_out, topk_idx, topk_val, scratch,
                                  cb200::kStaticScratchBytes, stream);
}

}  // extern "C"

// Merge of candidate lists that arrive packed as one buffer per rank, the form
// in which a single all-gather delivers them: per rank `words_per_list` 32-bit
// words = ids int32 [rows_cap][k] followed by values bf16 [rows_cap][k].
extern "C" int cudalm_b200_topk_merge_packed(const int32_t* gathered, int n_lists,
                                             int words_per_list, int rows_cap, int M, int k,
                                             int32_t* argmax_out, int32_t* topk_idx,
                                             uint16_t* topk_val, void* stream) {
  if (!gathered || !topk_idx || !topk_val) return CUDALM_B200_ERR_NULL;
  if (n_lists < 1 || M < 1 || k < 1 || rows_cap < M) return CUDALM_B200_ERR_BAD_SHAPE;
  const long long need = static_cast<long long>(rows_cap) * k + (static_cast<long long>(rows_cap) * k + 1) / 2;
  if (words_per_list < need) return CUDALM_B200_ERR_BAD_SHAPE;
  if (k > kMaxTopK || static_cast<long long>(n_lists) * k > kCandCap) return CUDALM_B200_ERR_TOO_LARGE;
  SelectArgs a;
  std::memset(&a, 0, sizeof(a));
  a.list_idx = gathered;
  a.list_val = reinterpret_cast<const std::uint16_t*>(gathered + static_cast<size_t>(rows_cap) * k);
  a.n_lists = n_lists;
  a.list_k = k;
  a.idx_stride = words_per_list;
  a.val_stride = 2ll * words_per_list;
  a.rows = M;
  a.k = k;
  a.argmax_out = argmax_out;
  a.topk_idx = topk_idx;
  a.topk_val = topk_val;
  lm_head_select_kernel<<<M, kSelectThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return check_launch();
}

// ---------------------------------------------------------------------------
// Candidate exchange over peer memory, fused with the merge.
//
// Vocabulary-parallel ranks on one node each hold an exchange buffer that the
// others map (CUDA IPC).  One kernel per rank, one CTA per activation row:
// the CTA stores the row's local candidates (k ids, k values) into every rank's
// buffer over NVLink, publishes a per-row epoch flag on every rank, waits (with
// a time limit) until every rank's flag for the row has reached the epoch, and
// merges the lists that have arrived in its own buffer.  Lists are double
// buffered by epoch parity: a rank can be at most one call ahead of a peer
// that is still merging, since the call after needs that peer's next flag.
// Epochs live on the device (one per row), so a captured call replays.
//
// Buffer layout in 32-bit words: lists [2][world][words_per_list], then flags
// [world][kMaxPassRows], then this rank's epochs [kMaxPassRows].
// ---------------------------------------------------------------------------
namespace cb200 {
namespace {

size_t exchange_words(int world, int words_per_list) {
  return 2 * static_cast<size_t>(world) * words_per_list + static_cast<size_t>(world) * kMaxPassRows +
         kMaxPassRows;
}

}  // namespace
}  // namespace cb200

extern "C" {

size_t cudalm_b200_exchange_bytes(int world, int words_per_list) {
  if (world < 1 || world > cb200::kMaxPeers || words_per_list < 1) return 0;
  return cb200::exchange_words(world, words_per_list) * sizeof(std::uint32_t);
}

int cudalm_b200_exchange_create(size_t bytes, void** local, unsigned char* handle64) {
  if (!local || !handle64 || bytes == 0) return CUDALM_B200_ERR_NULL;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are 64 bytes");
  void* p = nullptr;
  CB200_CUDA_TRY(cudaMalloc(&p, bytes));
  cudaError_t err = cudaMemset(p, 0, bytes);
  if (err == cudaSuccess) err = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (err == cudaSuccess) err = cudaIpcGetMemHandle(&h, p);
  if (err != cudaSuccess) {
    cb200::g_last_cuda_error = static_cast<int>(err);
    cudaFree(p);
    return CUDALM_B200_ERR_CUDA;
  }
  std::memcpy(handle64, &h, sizeof(h));
  *local = p;
  return CUDALM_B200_OK;
}

int cudalm_b200_exchange_open(const unsigned char* handle64, void** peer) {
  if (!handle64 || !peer) return CUDALM_B200_ERR_NULL;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, sizeof(h));
  CB200_CUDA_TRY(cudaIpcOpenMemHandle(peer, h, cudaIpcMemLazyEnablePeerAccess));
  return CUDALM_B200_OK;
}

int cudalm_b200_exchange_close(void* peer) {
  if (!peer) return CUDALM_B200_ERR_NULL;
  CB200_CUDA_TRY(cudaIpcCloseMemHandle(peer));
  return CUDALM_B200_OK;
}

int cudalm_b200_exchange_destroy(void* local) {
  if (!local) return CUDALM_B200_ERR_NULL;
  CB200_CUDA_TRY(cudaFree(local));
  return CUDALM_B200_OK;
}

static int fill_exchange_args(const int32_t* local_packed, void* const* bufs, int rank, int world,
                              int words_per_list, int rows_cap, int M, int k, int32_t* argmax_out,
                              int32_t* topk_idx, uint16_t* topk_val, cb200::ExchangeArgs* out) {
  using namespace cb200;
  if (!local_packed || !bufs || !topk_idx || !topk_val) return CUDALM_B200_ERR_NULL;
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || M < 1 || k < 1 || rows_cap < M)
    return CUDALM_B200_ERR_BAD_SHAPE;
  if (M > kMaxPassRows || k > kMaxTopK || static_cast<long long>(world) * k > kCandCap)
    return CUDALM_B200_ERR_TOO_LARGE;
  const long long need = static_cast<long long>(rows_cap) * k + (static_cast<long long>(rows_cap) * k + 1) / 2;
  if (words_per_list < need) return CUDALM_B200_ERR_BAD_SHAPE;
  ExchangeArgs e;
  std::memset(&e, 0, sizeof(e));
  for (int r = 0; r < world; ++r) {
    if (!bufs[r]) return CUDALM_B200_ERR_NULL;
    e.bufs[r] = static_cast<std::uint32_t*>(bufs[r]);
  }
  e.local_packed = local_packed;
  e.rank = rank;
  e.world = world;
  e.words_per_list = words_per_list;
  e.rows_cap = rows_cap;
  e.M = M;
  e.k = k;
  e.argmax_out = argmax_out;
  e.topk_idx = topk_idx;
  e.topk_val = topk_val;
  e.status = device_status_word();
  if (!e.status) return CUDALM_B200_ERR_CUDA;
  *out = e;
  return CUDALM_B200_OK;
}

int cudalm_b200_topk_exchange_merge(const int32_t* local_packed, void* const* bufs, int rank,
                                    int world, int words_per_list, int rows_cap, int M, int k,
                                    int32_t* argmax_out, int32_t* topk_idx, uint16_t* topk_val,
                                    void* stream) {
  cb200::ExchangeArgs e;
  if (int rc = fill_exchange_args(local_packed, bufs, rank, world, words_per_list, rows_cap, M, k,
                                  argmax_out, topk_idx, topk_val, &e))
    return rc;
  return cb200::launch_after(cb200::topk_exchange_merge_kernel, dim3(M), dim3(cb200::kSelectThreads),
                             static_cast<cudaStream_t>(stream), e);
}

int cudalm_b200_lm_head_topk_exchange(const uint8_t* weight, const uint16_t* scales,
                                      const uint16_t* x, int N, int K, int M, int top_k,
                                      int id_offset, uint16_t* logits_out, int32_t* local_packed,
                                      int rows_cap, void* workspace, size_t workspace_bytes,
                                      void* const* bufs, int rank, int world, int words_per_list,
                                      int32_t* argmax_out, int32_t* topk_idx, uint16_t* topk_val,
                                      void* stream) {
  if (!local_packed) return CUDALM_B200_ERR_NULL;
  if (rows_cap < M || rows_cap < 1 || top_k < 1) return CUDALM_B200_ERR_BAD_SHAPE;
  cb200::ExchangeArgs e;
  if (int rc = fill_exchange_args(local_packed, bufs, rank, world, words_per_list, rows_cap, M, top_k,
                                  argmax_out, topk_idx, topk_val, &e))
    return rc;
  // the local pick lands in the packed buffer: ids [rows_cap][k], then values
  int32_t* local_idx = local_packed;
  uint16_t* local_val = reinterpret_cast<uint16_t*>(local_packed + static_cast<size_t>(rows_cap) * top_k);
  return lm_head_topk_impl(weight, scales, x, N, K, M, top_k, id_offset, logits_out, nullptr, local_idx,
                           local_val, workspace, workspace_bytes, stream, &e);
}

}  // extern "C"
