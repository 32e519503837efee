"""B200-native W4A16 projection engine: a drop-in for CUDALM's int4-weight x
bf16-activation linear path (GEMV, batched rows, fused gate+up, vocabulary
projection with on-device pick, quantize+pack).  See ``include/cudalm_b200.h``
for the C ABI; this package is its host-side mirror of the reference interface.
"""
from .api import (CudalmB200Error, GROUP_SIZE, INT4_MAX, LinearGroup, LmHead, W4A16Linear,
                  batch_int4_gemv_bf16, device_status, gate_up_bf16, gate_up_silu_bf16, int4_gemv_bf16, linear_residual_bf16, sample_topk,
                  launch_count, library_path, linear_multi, lm_head_static_scratch_bytes,
                  lm_head_topk_static, load_library, quantize_w4a16, set_direct_path_max_bytes, set_exchange_timeout_ns,
                  set_tensor_path_min_rows, topk_merge)
from .api import packed_words, topk_merge_packed
from .vocab_parallel import (VocabParallelLmHead, gather_packed, merge_topk_host, shard_rows,
                             unpack_candidates)

__all__ = [
    "CudalmB200Error", "GROUP_SIZE", "INT4_MAX", "LinearGroup", "LmHead", "W4A16Linear",
    "batch_int4_gemv_bf16", "device_status", "gate_up_bf16", "gate_up_silu_bf16", "int4_gemv_bf16", "linear_residual_bf16", "sample_topk", "launch_count",
    "library_path", "linear_multi", "lm_head_static_scratch_bytes", "lm_head_topk_static",
    "load_library", "quantize_w4a16", "topk_merge", "set_tensor_path_min_rows",
    "set_direct_path_max_bytes", "set_exchange_timeout_ns",
    "VocabParallelLmHead", "merge_topk_host", "shard_rows", "gather_packed", "unpack_candidates",
    "packed_words", "topk_merge_packed",
]
