// Vocabulary projection with an on-device token pick: W4A16 GEMV over the
// vocabulary rows, then argmax and top-k per activation row.  The device side of the
// pick (ordering rule, candidate collection, ranking, the exchange between
// vocabulary-parallel ranks) is in lm_head_pick.cuh; this file holds the host entry
// points and the stand-alone kernels.
//
// One call is two launches: the projection, whose CTAs leave their largest outputs in a
// table, and the scan of the logits with several CTAs per activation row, whose last CTA
// per row ranks the candidates and, when the vocabulary is split over ranks, exchanges
// them.  A projection the staged kernels do not take (a weight base off 16 bytes, K above
// the staged limit) goes through the general kernels and the same scan without a table.
#include <atomic>
#include <cstring>

#include "lm_head_pick.cuh"

namespace cb200 {

int run_linear_with_pick(const cudalm_b200_linear& l, const PickTail& pick, cudaStream_t stream,
                         int* grid_out);
bool linear_with_pick_eligible(const cudalm_b200_linear& l);
bool linear_with_pick_on_tensor_path(const cudalm_b200_linear& l);
int stream_rows_per_pass(int K);
int run_linear_any(const cudalm_b200_linear& l, cudaStream_t stream);

// limit of the wait for the other ranks' candidates (cudalm_b200_set_exchange_timeout_ns)
std::atomic<long long> g_exchange_wait_ns{2000000000ll};


namespace {

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
// The scan of one CTA of grid (slices, rows): the row's bound from the table of per-CTA
// maxima the projection left (`slots`: kSlotReplicas copies of [rows][ncta] keys + 1;
// ncta == 0: no table, everything is a candidate), then the CTA's slice of the row's
// logits; values at or above the bound become candidates.
// ---------------------------------------------------------------------------
__device__ void scan_slice(const std::uint16_t* __restrict__ logits, int N, int rows,
                           const std::uint32_t* __restrict__ slots, int ncta, int k, int id_offset,
                           int* counts, std::uint64_t* cand) {
  __shared__ std::uint32_t bound;
  const int m = blockIdx.y;
  const int tid = threadIdx.x;
  if (tid < 32) {
    std::uint32_t T = 0;
    if (ncta > 0) {
      const std::uint32_t* copy = slots + static_cast<size_t>(blockIdx.x % kSlotReplicas) * ncta * rows;
      T = row_bound(copy + static_cast<size_t>(m) * ncta, ncta, k, tid);
    }
    if (tid == 0) bound = T == 0u ? 0u : T - 1u;  // a slot holds key + 1
  }
  __syncthreads();
  const std::uint32_t b = bound;
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
    if (order_key(bits) >= b) {
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

// ---------------------------------------------------------------------------
// Stand-alone kernels
// ---------------------------------------------------------------------------
// One CTA per row: ranks the row's candidates (collected by the projection, or
// gathered lists) and, when `e.world` >= 1, exchanges the pick with the other ranks.
__global__ void __launch_bounds__(kSelectThreads)
lm_head_select_kernel(const SelectArgs a, const ExchangeArgs e) {
  __shared__ SelectSmem sm;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int m = blockIdx.x, tid = threadIdx.x;
  select_row(a, m, tid, sm);
  if (e.world >= 1) {
    pick_sync();
    exchange_send_row(e, m, tid);
    pick_sync();
    exchange_recv_row(e, m, tid, sm);
  }
}

// One CTA per row: sends the row's pick (already in e.local_packed) and merges.
__global__ void __launch_bounds__(kSelectThreads)
topk_exchange_merge_kernel(const ExchangeArgs e) {
  __shared__ SelectSmem sm;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  exchange_send_row(e, blockIdx.x, threadIdx.x);
  pick_sync();
  exchange_recv_row(e, blockIdx.x, threadIdx.x, sm);
}

// scan + pick: grid (slices, rows).  Each CTA scans its slice of the row's logits for
// candidates; the CTA that finishes a row's scan last (a ticket per row) picks the row's
// tokens, exchanges them when the vocabulary is split, and leaves the row's counter,
// ticket and slots cleared for the next call.
__global__ void __launch_bounds__(kSelectThreads)
lm_head_scan_pick_kernel(const std::uint16_t* __restrict__ logits, int N, int rows, std::uint32_t* slots,
                         int ncta, int k, int id_offset, int* counts, int* tickets, std::uint64_t* cand,
                         const SelectArgs a, const ExchangeArgs e) {
  __shared__ SelectSmem sm;
  __shared__ int s_last;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int m = blockIdx.y;
  const int tid = threadIdx.x;
  scan_slice(logits, N, rows, slots, ncta, k, id_offset, counts, cand);
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    s_last = atomicAdd(&tickets[m], 1) == static_cast<int>(gridDim.x) - 1;
    __threadfence();
  }
  __syncthreads();
  if (!s_last) return;
  if (tid == 0) tickets[m] = 0;
  // every CTA of the row is past the table: clear the row's slots in every copy
  for (int i = tid; i < kSlotReplicas * ncta; i += kSelectThreads) {
    const int r = i / ncta, c = i - r * ncta;
    slots[(static_cast<size_t>(r) * rows + m) * ncta + c] = 0u;
  }
  select_row(a, m, tid, sm);
  if (e.world >= 1) {
    pick_sync();
    exchange_send_row(e, m, tid);
    pick_sync();
    exchange_recv_row(e, m, tid, sm);
  }
}

__global__ void zero_counts_kernel(int* counts, int n) {
  for (int i = threadIdx.x; i < n; i += blockDim.x) counts[i] = 0;
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

int cudalm_b200_lm_head_workspace_init(void* workspace, size_t workspace_bytes, void* stream) {
  if (!workspace) return CUDALM_B200_ERR_NULL;
  // counters, tickets and the per-CTA slots: what a call expects to find zero
  size_t n = kCountsBytes + static_cast<size_t>(kMaxCtas) * kMaxPassRows * sizeof(float);
  if (n > workspace_bytes) n = workspace_bytes;
  CB200_CUDA_TRY(cudaMemsetAsync(workspace, 0, n, static_cast<cudaStream_t>(stream)));
  return CUDALM_B200_OK;
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

  // rows per pass: 32 on the tensor-memory kernel, what fits its shared memory on the
  // streaming kernel, 32 on the general path
  const int rows_cap = M < kMaxPassRows ? M : kMaxPassRows;
  int per_pass = kMaxPassRows;
  {
    cudalm_b200_linear probe{weight, scales, x, logits_out, N, K, rows_cap, 0};
    if (!linear_with_pick_on_tensor_path(probe)) {
      const int fit = stream_rows_per_pass(K);
      if (fit > 0 && aligned_to(weight, 16)) per_pass = fit < kMaxPassRows ? fit : kMaxPassRows;
    }
  }
  if (ex && M > per_pass) return CUDALM_B200_ERR_UNSUPPORTED;
  ExchangeArgs no_exchange;
  std::memset(&no_exchange, 0, sizeof(no_exchange));
  const ExchangeArgs& e = ex ? *ex : no_exchange;

  for (int m0 = 0; m0 < M; m0 += per_pass) {
    const int rows = (M - m0 < per_pass) ? (M - m0) : per_pass;
    Workspace ws;
    workspace_layout(N, rows_cap, logits_out == nullptr, static_cast<unsigned char*>(workspace), &ws);
    uint16_t* logits = logits_out ? logits_out + static_cast<size_t>(m0) * N : ws.logits;
    cudalm_b200_linear l{weight, scales, x + static_cast<size_t>(m0) * K, logits, N, K, rows, 0};

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

    if (linear_with_pick_eligible(l)) {
      // the projection leaves the table of per-CTA maxima; many CTAs per row then scan the
      // logits, and the last one of a row ranks
      PickTail t;
      t.slots = reinterpret_cast<std::uint32_t*>(ws.cta_max);
      t.M = rows;
      int grid = 0;
      if (int rc = run_linear_with_pick(l, t, st, &grid)) return rc;
      // (measured: 2048 logits per CTA and four CTAs per SM in all; 32 rows 74.6 -> 70.6 us)
      int slices = (N + 2047) / 2048;
      const int cap = (4 * num_sms() + rows - 1) / rows;
      if (slices > cap) slices = cap;
      if (slices < 1) slices = 1;
      if (int rc = launch_after(lm_head_scan_pick_kernel, dim3(slices, rows), dim3(kSelectThreads), st,
                                static_cast<const std::uint16_t*>(logits), N, rows, t.slots, grid, top_k,
                                id_offset, ws.counts, ws.counts + kMaxPassRows, ws.cand, a, e))
        return rc;
      continue;
    }

    // general path: no per-CTA maxima, so every logit is a candidate and a row longer
    // than the candidate list takes the exact search
    zero_counts_kernel<<<1, 64, 0, st>>>(ws.counts, kMaxPassRows);
    if (int rc = check_launch()) return rc;
    if (int rc = run_linear_any(l, st)) return rc;
    int slices = (N + 2047) / 2048;
    const int cap = (4 * num_sms() + rows - 1) / rows;
    if (slices > cap) slices = cap;
    if (slices < 1) slices = 1;
    if (int rc = launch_after(lm_head_scan_pick_kernel, dim3(slices, rows), dim3(kSelectThreads), st,
                              static_cast<const std::uint16_t*>(logits), N, rows,
                              reinterpret_cast<std::uint32_t*>(ws.cta_max), 0, top_k, id_offset, ws.counts,
                              ws.counts + kMaxPassRows, ws.cand, a, e))
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

static int launch_merge(const SelectArgs& a, int M, void* stream) {
  cb200::ExchangeArgs none;
  std::memset(&none, 0, sizeof(none));
  lm_head_select_kernel<<<M, kSelectThreads, 0, static_cast<cudaStream_t>(stream)>>>(a, none);
  return check_launch();
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
  return launch_merge(a, M, stream);
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
// device current, and that pointer is what the kernels receive.  The array
// starts zeroed (as the pick expects its counters) and every call leaves the
// counters zeroed again.
// ---------------------------------------------------------------------------
namespace cb200 {
namespace {

constexpr int kStaticMaxRows = 32;  // activation rows per call
// counts + per-CTA slots + candidate lists for kStaticMaxRows rows (the same
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
  return launch_merge(a, M, stream);
}

// ---------------------------------------------------------------------------
// Candidate exchange over peer memory, fused with the pick and the merge.
//
// Vocabulary-parallel ranks on one node each hold an exchange buffer that the
// others map (CUDA IPC).  The threads that have ranked a row's local candidates
// store them (k words of {id, epoch tag, value}) into every rank's buffer over
// NVLink with plain 8-byte stores, wait (with a time limit) until every rank's
// words for the row carry the row's epoch, and merge what has arrived in their
// own buffer.  See ExchangeArgs in lm_head_pick.cuh for the layout.  Epochs live
// on the device (one per row), so a captured call replays.
// ---------------------------------------------------------------------------
extern "C" {

size_t cudalm_b200_exchange_bytes(int world, int words_per_list) {
  if (world < 1 || world > cb200::kMaxPeers || words_per_list < 1) return 0;
  return 2 * static_cast<size_t>(world) * words_per_list * sizeof(unsigned long long) +
         cb200::kMaxPassRows * sizeof(std::uint32_t);
}

int64_t cudalm_b200_set_exchange_timeout_ns(int64_t ns) {
  if (ns < 1000) ns = 1000;
  return cb200::g_exchange_wait_ns.exchange(ns);
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
    if (!aligned_to(bufs[r], 8)) return CUDALM_B200_ERR_MISALIGNED;
    e.bufs[r] = static_cast<unsigned long long*>(bufs[r]);
  }
  e.local_packed = local_packed;
  e.rank = rank;
  e.world = world;
  e.slot_words = words_per_list;
  e.rows_cap = rows_cap;
  e.M = M;
  e.k = k;
  e.wait_ns = g_exchange_wait_ns.load(std::memory_order_relaxed);
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
