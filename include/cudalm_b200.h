/*
 * cudalm_b200.h -- C ABI of the B200-native W4A16 projection engine.
 *
 * A drop-in for the CUDALM inference engine's int4-weight x bf16-activation
 * linear path.  Every entry point takes plain pointers and sizes, enqueues work
 * on the caller's CUDA stream and returns a status code; none of them aborts,
 * synchronises, or (unless stated) allocates.  All tensor pointers are
 * caller-owned DEVICE memory.
 *
 * Data layouts (CUDALM include/cudalm/kernels/int4_gemv_bf16.h:29-48):
 *   weight  uint8 [N, K/2] row-major; low nibble = k = 2b, high nibble =
 *           k = 2b+1; nibbles are 4-bit two's complement (0x8 decodes to -8)
 *   scales  IEEE binary16 [N, K/128] row-major, one per 128 consecutive k
 *   x       bfloat16 [K] or [M, K]
 *   y       bfloat16 [N] or [M, N]
 * Math:   y[m,n] = bf16_rn( sum_k float(q[n,k]) * float(scale[n,k/128]) *
 *                           float(x[m,k]) ), fp32 accumulation, one rounding.
 *
 * 16-bit float data is passed as uint16_t* holding the raw bits so that this
 * header needs no CUDA headers.  `stream` is a cudaStream_t passed as void*.
 */
#ifndef CUDALM_B200_H_
#define CUDALM_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define CUDALM_B200_API __attribute__((visibility("default")))
#else
#define CUDALM_B200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes.  CUDALM itself aborts on a contract violation
 * (include/cudalm/cuda_check.h:53-63); this ABI reports it instead and the
 * C++ shim in cudalm_b200_shims.hpp restores the abort for drop-in callers. */
enum {
  CUDALM_B200_OK = 0,
  CUDALM_B200_ERR_BAD_SHAPE = 1,   /* N < 1, K <= 0, K % 128 != 0, M < 1, ... */
  CUDALM_B200_ERR_NULL = 2,        /* a required pointer is null            */
  CUDALM_B200_ERR_MISALIGNED = 3,  /* a pointer misses a stated alignment   */
  CUDALM_B200_ERR_CUDA = 4,        /* a CUDA runtime call failed            */
  CUDALM_B200_ERR_TIMEOUT = 5,     /* a bounded device-side wait ran out    */
  CUDALM_B200_ERR_UNSUPPORTED = 6, /* legal in CUDALM but outside this build */
  CUDALM_B200_ERR_TOO_LARGE = 7,   /* exceeds a stated fixed capacity       */
  CUDALM_B200_ERR_WORKSPACE = 8,   /* workspace missing or too small        */
  CUDALM_B200_ERR_FILE = 9         /* a weight file is missing or malformed  */
};

CUDALM_B200_API const char* cudalm_b200_status_string(int status);
/* cudaError_t of the most recent CUDALM_B200_ERR_CUDA on this host thread. */
CUDALM_B200_API int cudalm_b200_last_cuda_error(void);
/* Library build info: "sm_100a;<git-less build tag>". */
CUDALM_B200_API const char* cudalm_b200_build_info(void);

/* Reads (and clears) the device-side status word of the current device.  The
 * kernels bound every wait; a wait that runs out stores ERR_TIMEOUT there and
 * the kernel returns without touching its outputs further.  This call
 * synchronises the device; it is for tests and diagnostics, not the hot path. */
CUDALM_B200_API int cudalm_b200_device_status(int* status_out);

/* ---- M = 1 GEMV -------------------------------------------------------
 * Replaces cudalm::int4_gemv_bf16
 * (CUDALM include/cudalm/kernels/int4_gemv_bf16.h:46-48,
 *  src/kernels/int4_gemv_bf16.cu:221-243).
 * Preconditions: N >= 1, K > 0, K % 128 == 0.  No alignment is required of
 * any pointer (a weight base that is not 16-byte aligned takes a slower
 * kernel, as in CUDALM). */
CUDALM_B200_API int cudalm_b200_int4_gemv_bf16(const uint8_t* weight, const uint16_t* scales,
                               const uint16_t* x, uint16_t* y, int N, int K,
                               void* stream);

/* ---- batched decode, M = B rows -----------------------------------------
 * Replaces cudalm::kernels::batch_int4_gemv_bf16
 * (CUDALM include/cudalm/kernels/batch_decode.h:61-63,
 *  src/kernels/batch_decode.cu:95-190,647-659): x is [B, K], y is [B, N].
 * Unlike CUDALM's, the weights are read once for all B rows.
 * From 17 rows on (tensor-memory kernel), a call whose projections have few rows
 * and K >= 2048 cuts K into slices that separate CTAs work on and adds them up in a
 * fixed order in a second launch; the fp32 partial sums live in stream-ordered
 * scratch from a memory pool the library owns (allocated and freed on `stream`, so
 * the call stays asynchronous and can be captured in a CUDA graph).  The same holds
 * for cudalm_b200_linear_multi, _gate_up_silu_bf16 and _linear_residual_bf16; a
 * group allocates its scratch once in cudalm_b200_group_create, which is why a
 * group must not run on two streams at the same time. */
CUDALM_B200_API int cudalm_b200_batch_int4_gemv_bf16(const uint8_t* weight,
                                     const uint16_t* scales, const uint16_t* x,
                                     uint16_t* y, int N, int K, int B,
                                     void* stream);

/* ---- several projections in one launch ------------------------------------
 * One descriptor per projection.  Used for the projections of a layer that
 * share an input (CUDALM src/runtime/qwen35_deltanet.cpp:166-181: qkv, z, b, a;
 * src/runtime/qwen35_full_attention.cpp:211-231: q, k, v; the MLP's gate and
 * up, qwen35_deltanet.cpp:236-243) and for streaming a whole model's set.
 * The projections of one call must be independent of one another. */
typedef struct cudalm_b200_linear {
  const uint8_t* weight;  /* [N, K/2]            */
  const uint16_t* scales; /* fp16 [N, K/128]     */
  const uint16_t* x;      /* bf16 [M, K]         */
  uint16_t* y;            /* bf16 [M, N]         */
  int32_t N;
  int32_t K;
  int32_t M;              /* rows of x, 1..CUDALM_B200_MAX_GROUP_M */
  int32_t reserved;       /* must be 0           */
} cudalm_b200_linear;

#define CUDALM_B200_MAX_INLINE_LINEARS 4
#define CUDALM_B200_MAX_GROUP_M 64

/* Up to CUDALM_B200_MAX_INLINE_LINEARS projections, descriptors in HOST
 * memory, passed to the kernel by value: allocates nothing. */
CUDALM_B200_API int cudalm_b200_linear_multi(const cudalm_b200_linear* linears, int count,
                             void* stream);

/* Any number of projections.  create() copies the descriptor table to the
 * device (it allocates, and synchronises once); run() only launches. */
typedef struct cudalm_b200_group cudalm_b200_group;
CUDALM_B200_API int cudalm_b200_group_create(const cudalm_b200_linear* linears, int count,
                             cudalm_b200_group** group_out);
CUDALM_B200_API int cudalm_b200_group_run(const cudalm_b200_group* group, void* stream);
CUDALM_B200_API int cudalm_b200_group_destroy(cudalm_b200_group* group);
/* Algorithmic bytes one run() moves: sum of N*K/2 + N*(K/128)*2 + M*K*2 + M*N*2. */
CUDALM_B200_API int64_t cudalm_b200_group_bytes(const cudalm_b200_group* group);

/* ---- fused gate + up ------------------------------------------------------
 * Replaces the two calls at CUDALM src/runtime/qwen35_deltanet.cpp:236-243 /
 * src/runtime/qwen35_full_attention.cpp:317-326 with one launch over the shared
 * input x [M, K]; gate_y and up_y are [M, N] each and equal the two separate
 * calls row for row. */
CUDALM_B200_API int cudalm_b200_gate_up_bf16(const uint8_t* gate_weight,
                             const uint16_t* gate_scales,
                             const uint8_t* up_weight, const uint16_t* up_scales,
                             const uint16_t* x, uint16_t* gate_y, uint16_t* up_y,
                             int N, int K, int M, void* stream);

/* ---- MLP epilogues fused into the projection ----------------------------------
 * gate_up_silu: out[m][n] = bf16(float(bf16(silu(g))) * float(u)) with g, u the
 * bf16 outputs of the gate and up projections of x [M, K]; replaces the two
 * projections and qwen35_silu_mul (CUDALM include/cudalm/kernels/qwen35_kernels.h:137-155,
 * src/kernels/qwen35_kernels.cu:459-476; call sites src/runtime/qwen35_deltanet.cpp:236-247,
 * src/runtime/qwen35_full_attention.cpp:317-331) with one launch per 16 rows, or per
 * 64 rows when M is at least the tensor path's smallest row count.
 * linear_residual: y[m][n] = bf16(float(residual[m][n]) + float(p)) with p the bf16
 * output of the projection; replaces the down / o_proj / out_proj projection and the
 * qwen35_add that follows it (src/kernels/qwen35_kernels.cu:442-456;
 * src/runtime/qwen35_deltanet.cpp:248-252).  y may alias residual.
 * The intermediate values are rounded exactly where CUDALM rounds them, so the
 * results equal the unfused sequence on this library's own projections bit for bit. */
CUDALM_B200_API int cudalm_b200_gate_up_silu_bf16(const uint8_t* gate_weight,
                             const uint16_t* gate_scales,
                             const uint8_t* up_weight, const uint16_t* up_scales,
                             const uint16_t* x, uint16_t* out,
                             int N, int K, int M, void* stream);
CUDALM_B200_API int cudalm_b200_linear_residual_bf16(const uint8_t* weight,
                             const uint16_t* scales, const uint16_t* x,
                             const uint16_t* residual, uint16_t* y,
                             int N, int K, int M, void* stream);

/* ---- vocabulary projection with on-device token pick --------------------------
 * Replaces the lm_head call cudalm::bf16_gemv / kernels::batch_bf16_gemv
 * (CUDALM include/cudalm/kernels/bf16_gemv.h:39-40,
 *  include/cudalm/kernels/batch_decode.h:77-79; call sites
 *  src/runtime/qwen35_model.cpp:177-181,290-292,500-502) and the host-side pick
 * that follows it (src/runtime/scheduler.cpp:59-108, argmax_bf16 in
 * include/cudalm/greedy.h:28-39, the top-k order of
 * include/cudalm/sampling.h:152-166) for an lm_head stored as W4A16.
 *
 * weight/scales are this caller's rows [N, ...] of the vocabulary matrix;
 * id_offset is the token id of row 0 (non-zero for a vocabulary-parallel shard).
 * Outputs, per activation row m: argmax_out[m] (may be null), topk_idx[m][top_k]
 * and topk_val[m][top_k] (bf16 bits) ordered by value descending, ties by lower
 * id; when N < top_k the tail is filled with id -1.  logits_out (may be null) is
 * the full bf16 logits [M, N], as CUDALM's call produces.  top_k <= 64.
 * workspace: device memory, 256-byte aligned, of at least
 * cudalm_b200_lm_head_workspace_bytes(..., need_logits = logits_out == NULL), zeroed
 * once before its first use (cudalm_b200_lm_head_workspace_init, or a memset of the
 * whole of it): it holds the counters of the pick, which every call leaves at zero
 * for the next one.  Calls that share a workspace must not overlap on the GPU; after
 * a CUDALM_B200_ERR_TIMEOUT in the device status word, zero it again.
 * A call is two launches: the projection, then the scan of the logits (still in L2)
 * whose last CTA per activation row ranks the candidates. */
CUDALM_B200_API size_t cudalm_b200_lm_head_workspace_bytes(int N, int K, int M, int top_k,
                                                           int need_logits);
CUDALM_B200_API int cudalm_b200_lm_head_workspace_init(void* workspace, size_t workspace_bytes,
                                                       void* stream);
CUDALM_B200_API int cudalm_b200_lm_head_topk(
    const uint8_t* weight, const uint16_t* scales, const uint16_t* x, int N, int K,
    int M, int top_k, int id_offset, uint16_t* logits_out, int32_t* argmax_out,
    int32_t* topk_idx, uint16_t* topk_val, void* workspace, size_t workspace_bytes,
    void* stream);

/* ---- vocabulary projection without any allocation ------------------------------
 * (No counterpart in CUDALM: its lm_head call needs no scratch because it
 * leaves the token pick to the host.)
 *
 * Same computation and outputs as cudalm_b200_lm_head_topk, for callers that
 * cannot allocate device memory for the workspace -- a server whose memory pools
 * own the whole GPU, a decode loop in which cudaMalloc is forbidden because it
 * synchronises the device, a binding with no device allocator.  The scratch is
 * a fixed array of cudalm_b200_lm_head_static_scratch_bytes() (about 640 KB)
 * inside the library's device image; every GPU that loads the library holds it
 * until the process exits.  The call itself allocates nothing, and the array needs
 * no initialisation by the caller.
 *
 * Limits: M <= 32 activation rows per call (more: CUDALM_B200_ERR_TOO_LARGE);
 * logits_out is required (CUDALM_B200_ERR_NULL when null).
 * The first call on each device looks up the array's device address; make that
 * first call before any stream capture begins on the device.
 * All calls on a device share the one array, which keeps the previous call's
 * contents (the entry point clears what must start at zero): two calls whose
 * kernels overlap on the GPU -- different streams, no ordering between them --
 * race on it.  Order such calls, or use cudalm_b200_lm_head_topk with one
 * workspace per stream. */
CUDALM_B200_API size_t cudalm_b200_lm_head_static_scratch_bytes(void);
CUDALM_B200_API int cudalm_b200_lm_head_topk_static(
    const uint8_t* weight, const uint16_t* scales, const uint16_t* x, int N, int K,
    int M, int top_k, int id_offset, uint16_t* logits_out, int32_t* argmax_out,
    int32_t* topk_idx, uint16_t* topk_val, void* stream);

/* Merges n_lists candidate lists (one per vocabulary shard, gathered from the
 * ranks) into the final pick: list_idx/list_val are [n_lists, M, k]; ids < 0 are
 * padding.  Same ordering rule; n_lists * k <= 2048. */
CUDALM_B200_API int cudalm_b200_topk_merge(const int32_t* list_idx, const uint16_t* list_val,
                                           int n_lists, int M, int k, int32_t* argmax_out,
                                           int32_t* topk_idx, uint16_t* topk_val,
                                           void* stream);

/* The same merge for lists that arrive packed, one buffer of `words_per_list`
 * 32-bit words per shard: ids int32 [rows_cap][k] followed by values bf16
 * [rows_cap][k] (the layout in which ONE all-gather delivers them). */
CUDALM_B200_API int cudalm_b200_topk_merge_packed(const int32_t* gathered, int n_lists,
                                                  int words_per_list, int rows_cap, int M,
                                                  int k, int32_t* argmax_out,
                                                  int32_t* topk_idx, uint16_t* topk_val,
                                                  void* stream);

/* ---- candidate exchange over peer memory, fused with the merge -------------------
 * For vocabulary-parallel ranks on one node (up to 8): instead of an all-gather
 * followed by cudalm_b200_topk_merge_packed, ONE kernel per rank stores the rank's
 * packed candidates (the layout above, `local_packed`) into every rank's exchange
 * buffer over NVLink -- one 8-byte word per candidate that carries id, value and the
 * call's epoch, so no flag and no fence follow the data -- waits for every rank's
 * words and merges what has arrived.  The wait is limited (2 s by default,
 * cudalm_b200_set_exchange_timeout_ns); when it runs out the status word reads
 * CUDALM_B200_ERR_TIMEOUT (cudalm_b200_device_status) and the affected rows' outputs
 * are ids -1 with values -inf, so a miss shows in the data.  After a TIMEOUT the ranks'
 * epochs may differ: destroy the buffers and create new ones.  There is no counterpart
 * in CUDALM, whose lm_head is single-GPU (src/runtime/qwen35_model.cpp:290-292).
 *
 * Every rank creates a buffer of cudalm_b200_exchange_bytes(world, words_per_list)
 * (zeroed; `handle64` receives its 64-byte CUDA IPC handle), sends the handle to
 * its peers by any host channel, opens the peers' handles, and passes the `world`
 * pointers (its own at [rank]) as the HOST array `bufs`.  All ranks must have opened
 * all buffers before the first call, make the same sequence of calls (same M), and
 * keep the calls of one rank on one stream.  M <= 32 rows per call. */
CUDALM_B200_API size_t cudalm_b200_exchange_bytes(int world, int words_per_list);
/* Limit of the wait for the other ranks' candidates, for calls made from now on
 * (at least 1000 ns).  Returns the previous value. */
CUDALM_B200_API int64_t cudalm_b200_set_exchange_timeout_ns(int64_t ns);
CUDALM_B200_API int cudalm_b200_exchange_create(size_t bytes, void** local, unsigned char* handle64);
CUDALM_B200_API int cudalm_b200_exchange_open(const unsigned char* handle64, void** peer);
CUDALM_B200_API int cudalm_b200_exchange_close(void* peer);
CUDALM_B200_API int cudalm_b200_exchange_destroy(void* local);
CUDALM_B200_API int cudalm_b200_topk_exchange_merge(const int32_t* local_packed, void* const* bufs,
                                                    int rank, int world, int words_per_list,
                                                    int rows_cap, int M, int k,
                                                    int32_t* argmax_out, int32_t* topk_idx,
                                                    uint16_t* topk_val, void* stream);

/* The whole vocabulary-parallel step of one rank in two launches: the projection of
 * this rank's rows, then the scan whose last CTA per row picks the row's local
 * candidates (into `local_packed`: ids int32 [rows_cap][top_k], then values bf16),
 * sends them to the other ranks and merges theirs as cudalm_b200_topk_exchange_merge
 * does; argmax_out / topk_idx / topk_val receive the merged pick.  Arguments as
 * cudalm_b200_lm_head_topk and cudalm_b200_topk_exchange_merge; M must fit one pass
 * (UNSUPPORTED otherwise: call the two entries one after the other). */
CUDALM_B200_API int cudalm_b200_lm_head_topk_exchange(
    const uint8_t* weight, const uint16_t* scales, const uint16_t* x, int N, int K, int M,
    int top_k, int id_offset, uint16_t* logits_out, int32_t* local_packed, int rows_cap,
    void* workspace, size_t workspace_bytes, void* const* bufs, int rank, int world,
    int words_per_list, int32_t* argmax_out, int32_t* topk_idx, uint16_t* topk_val, void* stream);

/* ---- token sampling over the candidate lists -----------------------------------
 * CUDALM's sample_token (include/cudalm/sampling.h:131-234; called per row on the
 * host after a 497 KB copy of the logits, src/runtime/scheduler.cpp:59-108) on the
 * lists cudalm_b200_lm_head_topk / cudalm_b200_topk_merge return: topk_idx,
 * topk_val [M, list_len] ordered by value descending, tie -> lower id.
 * temperature <= 0: the greedy pick (entry 0), no draw, rng_state may be null.
 * Otherwise 1 <= top_k <= list_len is required (UNSUPPORTED else: with top-k
 * disabled every token of the vocabulary keeps a probability, which a list cannot
 * answer), 0 < top_p <= 1, and rng_state [M] (device) holds each row's SplitMix64
 * state, advanced by one draw.  token_out [M] receives global token ids.  Same
 * arithmetic as the reference (double precision, its summation orders). */
CUDALM_B200_API int cudalm_b200_sample_topk(const int32_t* topk_idx, const uint16_t* topk_val,
                             int list_len, int M, float temperature, int top_k,
                             float top_p, uint64_t* rng_state, int32_t* token_out,
                             void* stream);

/* ---- `.cudalm` v2 weight container -----------------------------------------------
 * Reader of the file CUDALM's converter writes and WeightFileV2::load reads
 * (CUDALM include/cudalm/weight_format_v2.h:35-190,
 *  src/runtime/weight_loader_v2.cpp:49-242), with the same validation rules.
 * open() reads and validates the whole file (CUDALM_B200_ERR_FILE with the
 * reason in `err`); the handle owns the bytes until close().  Tensor and metadata
 * strings and host_bytes point into the handle.  upload() enqueues one copy of a
 * tensor's bytes to device memory.  linear() checks that two tensors form a
 * W4A16 projection (int4_packed [N, K/2] + fp16_scale [N, K/128]). */
enum {
  CUDALM_B200_V2_FP16 = 1,
  CUDALM_B200_V2_INT4_PACKED = 2,
  CUDALM_B200_V2_FP16_SCALE = 3,
  CUDALM_B200_V2_FP32 = 4,
  CUDALM_B200_V2_BF16 = 5
};
typedef struct cudalm_b200_v2_file cudalm_b200_v2_file;
typedef struct cudalm_b200_v2_tensor {
  const char* name;
  int32_t dtype;
  int32_t ndim;
  int64_t dims[8];        /* int4_packed: in packed bytes (last dim = K/2) */
  uint64_t offset;        /* from the start of the payload section */
  uint64_t byte_size;
  int32_t align;
  int32_t reserved;
  const void* host_bytes; /* the tensor's bytes inside the handle */
} cudalm_b200_v2_tensor;
CUDALM_B200_API int cudalm_b200_v2_open(const char* path, cudalm_b200_v2_file** out, char* err,
                             size_t err_cap);
CUDALM_B200_API void cudalm_b200_v2_close(cudalm_b200_v2_file* file);
CUDALM_B200_API int cudalm_b200_v2_num_tensors(const cudalm_b200_v2_file* file);
CUDALM_B200_API int cudalm_b200_v2_num_metadata(const cudalm_b200_v2_file* file);
CUDALM_B200_API int cudalm_b200_v2_tensor_at(const cudalm_b200_v2_file* file, int index,
                             cudalm_b200_v2_tensor* out);
CUDALM_B200_API int cudalm_b200_v2_find(const cudalm_b200_v2_file* file, const char* name);
CUDALM_B200_API int cudalm_b200_v2_config_blob(const cudalm_b200_v2_file* file, uint8_t* out88);
CUDALM_B200_API int cudalm_b200_v2_metadata_at(const cudalm_b200_v2_file* file, int index,
                             const char** key, const char** value);
CUDALM_B200_API int cudalm_b200_v2_upload(const cudalm_b200_v2_file* file, int index, void* device_dst,
                             size_t capacity, void* stream);
CUDALM_B200_API int cudalm_b200_v2_linear(const cudalm_b200_v2_file* file, const char* weight_name,
                             const char* scale_name, int* weight_index, int* scale_index,
                             int* N, int* K);

/* ---- model-level loading ----------------------------------------------------------
 * The tensor set of one decoder layer, checked against the file's configuration
 * and uploaded: CUDALM's WeightFileV2::validate_layer / validate_full_model and
 * Qwen35LayerWeights::load (src/runtime/weight_loader_v2.cpp:273-372, 383-408,
 * 416-499; include/cudalm/weight_loader_v2.h:39,83-84).  A layer is a gated-
 * DeltaNet layer or, every full_attention_interval-th one, a full-attention layer
 * (include/cudalm/qwen35_config.h:82-88); both hold the MLP.  validate_* return
 * CUDALM_B200_ERR_FILE with the reference's message in `err` ("missing tensor
 * '...'", "dtype mismatch for '...'", "shape mismatch for '...'").
 *
 * load_layer uploads the layer's 24 tensors into caller-owned device memory
 * (`device_dst`, 256-byte aligned, at least cudalm_b200_v2_layer_device_bytes();
 * every tensor starts on a 256-byte boundary, as CUDALM's DeviceBuffer gives) with
 * one copy per tensor on `stream`, and fills `out`: proj[] holds the layer's W4A16
 * projections with weight, scales, N = dim 0 and K = 2 * dim 1 set and x, y, M left
 * zero for the caller; projections the layer type lacks stay all-zero.  The file
 * handle must stay open until the copies have completed. */
enum {
  CUDALM_B200_PROJ_GATE = 0, CUDALM_B200_PROJ_UP, CUDALM_B200_PROJ_DOWN,
  CUDALM_B200_PROJ_Q, CUDALM_B200_PROJ_K, CUDALM_B200_PROJ_V, CUDALM_B200_PROJ_O,
  CUDALM_B200_PROJ_IN_QKV, CUDALM_B200_PROJ_IN_Z, CUDALM_B200_PROJ_IN_B,
  CUDALM_B200_PROJ_IN_A, CUDALM_B200_PROJ_OUT,
  CUDALM_B200_LAYER_PROJECTIONS
};
enum {
  CUDALM_B200_AUX_INPUT_LAYERNORM = 0, CUDALM_B200_AUX_POST_ATTENTION_LAYERNORM,
  CUDALM_B200_AUX_Q_NORM, CUDALM_B200_AUX_K_NORM, CUDALM_B200_AUX_CONV1D,
  CUDALM_B200_AUX_DT_BIAS, CUDALM_B200_AUX_A_LOG, CUDALM_B200_AUX_LINEAR_NORM,
  CUDALM_B200_LAYER_AUX
};
typedef struct cudalm_b200_v2_layer {
  int32_t layer_idx;
  int32_t full_attention; /* 1: q, k, v, o; 0: in_proj_qkv, z, b, a and out_proj */
  cudalm_b200_linear proj[CUDALM_B200_LAYER_PROJECTIONS];
  const void* aux[CUDALM_B200_LAYER_AUX];     /* the layer's other tensors (device) */
  int32_t aux_dtype[CUDALM_B200_LAYER_AUX];   /* CUDALM_B200_V2_* */
  uint64_t aux_bytes[CUDALM_B200_LAYER_AUX];
} cudalm_b200_v2_layer;
CUDALM_B200_API int cudalm_b200_v2_validate_layer(const cudalm_b200_v2_file* file, int layer_idx,
                             char* err, size_t err_cap);
CUDALM_B200_API int cudalm_b200_v2_validate_full_model(const cudalm_b200_v2_file* file, char* err,
                             size_t err_cap);
CUDALM_B200_API size_t cudalm_b200_v2_layer_device_bytes(const cudalm_b200_v2_file* file, int layer_idx);
CUDALM_B200_API int cudalm_b200_v2_load_layer(const cudalm_b200_v2_file* file, int layer_idx,
                             void* device_dst, size_t capacity, void* stream,
                             cudalm_b200_v2_layer* out, char* err, size_t err_cap);

/* ---- quantize + pack --------------------------------------------------------
 * GPU form of CUDALM's offline quantizer quantize_w4a16
 * (CUDALM tools/common/w4a16_quant.py:25-60): bf16 W [N, K] ->
 * packed int4 [N, K/2] and fp16 scales [N, K/128], bit-exact with it.
 * W must be 16-byte aligned; packed 4-byte aligned. */
CUDALM_B200_API int cudalm_b200_quantize_w4a16(const uint16_t* w_bf16, int N, int K,
                               uint8_t* packed, uint16_t* scales, void* stream);

/* ---- runtime knob -------------------------------------------------------------
 * Batched calls with M >= min_rows rows take the tcgen05 / tensor-memory kernel
 * (when its shared-memory budget allows), smaller ones the streaming kernel.
 * Default 17 (measured crossover on B200: up to 16 rows the streaming kernel with
 * two MMA column tiles is faster).  Returns the previous value.  (CUDALM has no counterpart: its
 * batch kernel is the M = 1 kernel with blockIdx.y = b,
 * src/kernels/batch_decode.cu:95-190.) */
CUDALM_B200_API int cudalm_b200_set_tensor_path_min_rows(int min_rows);
/* Single calls (int4_gemv_bf16, batch_int4_gemv_bf16, linear_multi, gate_up*,
 * linear_residual) with at most 8 activation rows whose weights total at most
 * max_bytes take the lean kernel, which has no set-up cost and answers a call of a
 * few megabytes in about one memory round trip; larger ones stream through the
 * persistent kernel.  0 switches the lean kernel off.  Returns the previous value.
 * (CUDALM's counterpart is its one kernel per call,
 * src/kernels/int4_gemv_bf16.cu:221-243.) */
CUDALM_B200_API int64_t cudalm_b200_set_direct_path_max_bytes(int64_t max_bytes);

/* ---- introspection ---------------------------------------------------------
 * Registers per thread / static+dynamic shared memory of the named kernel
 * (CUDALM exposes the same for its kernels: int4_gemv_bf16_rowtile4_regs(),
 * src/kernels/int4_gemv_bf16.cu:247-253).  Returns -1 when unknown. */
CUDALM_B200_API int cudalm_b200_kernel_regs(const char* kernel_name);
/* Number of kernels this library has launched from the calling process. */
CUDALM_B200_API int64_t cudalm_b200_launch_count(void);

#ifdef __cplusplus
} /* extern "C" */
#endif
#endif /* CUDALM_B200_H_ */
