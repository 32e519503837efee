"""Host-side mirror of CUDALM's W4A16 operator interface over the C ABI.

Function names, argument order and error behaviour follow the reference's C++
entry points (``cudalm::int4_gemv_bf16``, ``cudalm::kernels::batch_int4_gemv_bf16``,
``W4A16Linear``, the offline ``quantize_w4a16``), so that tests written against
the reference read the same here.  Arguments are ``torch`` tensors on a CUDA
device; torch is used only to own device memory and to name the current stream.
Every call goes through ``libcudalm_b200.so``; there is no CPU path, and a
missing library or a non-zero status raises.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from . import build as _build

GROUP_SIZE = 128
INT4_MAX = 7
MAX_TOP_K = 64

OK = 0
ERR_BAD_SHAPE = 1
ERR_NULL = 2
ERR_MISALIGNED = 3
ERR_CUDA = 4
ERR_TIMEOUT = 5
ERR_UNSUPPORTED = 6
ERR_TOO_LARGE = 7
ERR_WORKSPACE = 8


class CudalmB200Error(RuntimeError):
    """A C-ABI call returned a non-zero status (CUDALM itself would abort)."""

    def __init__(self, fn: str, status: int, detail: str):
        super().__init__(f"{fn} failed: status {status} ({detail})")
        self.status = status


class _LinearStruct(ctypes.Structure):
    _fields_ = [("weight", ctypes.c_void_p), ("scales", ctypes.c_void_p),
                ("x", ctypes.c_void_p), ("y", ctypes.c_void_p),
                ("N", ctypes.c_int32), ("K", ctypes.c_int32),
                ("M", ctypes.c_int32), ("reserved", ctypes.c_int32)]


_vp = ctypes.c_void_p
_ci = ctypes.c_int

# name -> (restype, argtypes); every symbol include/cudalm_b200.h declares
SIGNATURES = {
    "cudalm_b200_status_string": (ctypes.c_char_p, [_ci]),
    "cudalm_b200_last_cuda_error": (_ci, []),
    "cudalm_b200_build_info": (ctypes.c_char_p, []),
    "cudalm_b200_device_status": (_ci, [ctypes.POINTER(_ci)]),
    "cudalm_b200_int4_gemv_bf16": (_ci, [_vp, _vp, _vp, _vp, _ci, _ci, _vp]),
    "cudalm_b200_batch_int4_gemv_bf16": (_ci, [_vp, _vp, _vp, _vp, _ci, _ci, _ci, _vp]),
    "cudalm_b200_linear_multi": (_ci, [ctypes.POINTER(_LinearStruct), _ci, _vp]),
    "cudalm_b200_group_create": (_ci, [ctypes.POINTER(_LinearStruct), _ci, ctypes.POINTER(_vp)]),
    "cudalm_b200_group_run": (_ci, [_vp, _vp]),
    "cudalm_b200_group_destroy": (_ci, [_vp]),
    "cudalm_b200_group_bytes": (ctypes.c_int64, [_vp]),
    "cudalm_b200_gate_up_bf16": (_ci, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _vp]),
    "cudalm_b200_v2_open": (_ci, [ctypes.c_char_p, _vp, ctypes.c_char_p, ctypes.c_size_t]),
    "cudalm_b200_v2_close": (None, [_vp]),
    "cudalm_b200_v2_num_tensors": (_ci, [_vp]),
    "cudalm_b200_v2_num_metadata": (_ci, [_vp]),
    "cudalm_b200_v2_tensor_at": (_ci, [_vp, _ci, _vp]),
    "cudalm_b200_v2_find": (_ci, [_vp, ctypes.c_char_p]),
    "cudalm_b200_v2_config_blob": (_ci, [_vp, _vp]),
    "cudalm_b200_v2_metadata_at": (_ci, [_vp, _ci, _vp, _vp]),
    "cudalm_b200_v2_upload": (_ci, [_vp, _ci, _vp, ctypes.c_size_t, _vp]),
    "cudalm_b200_v2_linear": (_ci, [_vp, ctypes.c_char_p, ctypes.c_char_p, _vp, _vp, _vp, _vp]),
    "cudalm_b200_v2_validate_layer": (_ci, [_vp, _ci, ctypes.c_char_p, ctypes.c_size_t]),
    "cudalm_b200_v2_validate_full_model": (_ci, [_vp, ctypes.c_char_p, ctypes.c_size_t]),
    "cudalm_b200_v2_layer_device_bytes": (ctypes.c_size_t, [_vp, _ci]),
    "cudalm_b200_v2_load_layer": (_ci, [_vp, _ci, _vp, ctypes.c_size_t, _vp, _vp, ctypes.c_char_p,
                                        ctypes.c_size_t]),
    "cudalm_b200_sample_topk": (_ci, [_vp, _vp, _ci, _ci, ctypes.c_float, _ci, ctypes.c_float, _vp,
                                      _vp, _vp]),
    "cudalm_b200_gate_up_silu_bf16": (_ci, [_vp, _vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _vp]),
    "cudalm_b200_linear_residual_bf16": (_ci, [_vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _vp]),
    "cudalm_b200_lm_head_workspace_bytes": (ctypes.c_size_t, [_ci, _ci, _ci, _ci, _ci]),
    "cudalm_b200_lm_head_workspace_init": (_ci, [_vp, ctypes.c_size_t, _vp]),
    "cudalm_b200_lm_head_topk": (_ci, [_vp, _vp, _vp, _ci, _ci, _ci, _ci, _ci, _vp, _vp, _vp,
                                      _vp, _vp, ctypes.c_size_t, _vp]),
    "cudalm_b200_lm_head_static_scratch_bytes": (ctypes.c_size_t, []),
    "cudalm_b200_lm_head_topk_static": (_ci, [_vp, _vp, _vp, _ci, _ci, _ci, _ci, _ci, _vp, _vp, _vp,
                                             _vp, _vp]),
    "cudalm_b200_topk_merge": (_ci, [_vp, _vp, _ci, _ci, _ci, _vp, _vp, _vp, _vp]),
    "cudalm_b200_topk_merge_packed": (_ci, [_vp, _ci, _ci, _ci, _ci, _ci, _vp, _vp, _vp, _vp]),
    "cudalm_b200_exchange_bytes": (ctypes.c_size_t, [_ci, _ci]),
    "cudalm_b200_set_exchange_timeout_ns": (ctypes.c_int64, [ctypes.c_int64]),
    "cudalm_b200_exchange_create": (_ci, [ctypes.c_size_t, ctypes.POINTER(_vp), _vp]),
    "cudalm_b200_exchange_open": (_ci, [_vp, ctypes.POINTER(_vp)]),
    "cudalm_b200_exchange_close": (_ci, [_vp]),
    "cudalm_b200_exchange_destroy": (_ci, [_vp]),
    "cudalm_b200_topk_exchange_merge": (_ci, [_vp, ctypes.POINTER(_vp), _ci, _ci, _ci, _ci, _ci, _ci,
                                             _vp, _vp, _vp, _vp]),
    "cudalm_b200_lm_head_topk_exchange": (_ci, [_vp, _vp, _vp, _ci, _ci, _ci, _ci, _ci, _vp, _vp, _ci,
                                               _vp, ctypes.c_size_t, ctypes.POINTER(_vp), _ci, _ci,
                                               _ci, _vp, _vp, _vp, _vp]),
    "cudalm_b200_quantize_w4a16": (_ci, [_vp, _ci, _ci, _vp, _vp, _vp]),
    "cudalm_b200_set_tensor_path_min_rows": (_ci, [_ci]),
    "cudalm_b200_set_direct_path_max_bytes": (ctypes.c_int64, [ctypes.c_int64]),
    "cudalm_b200_kernel_regs": (_ci, [ctypes.c_char_p]),
    "cudalm_b200_launch_count": (ctypes.c_int64, []),
}

_lib: Optional[ctypes.CDLL] = None


def library_path() -> str:
    """Path of the native library; ``CUDALM_B200_LIBRARY`` overrides the in-tree build."""
    return os.environ.get("CUDALM_B200_LIBRARY") or _build.LIB_PATH


def load_library() -> ctypes.CDLL:
    """Loads ``libcudalm_b200.so`` (it must have been built; see ``build.py``)."""
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise CudalmB200Error("load_library", ERR_UNSUPPORTED,
                                  f"{path} is missing: run python -m cudalm_agent_b200.build")
        lib = ctypes.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def _check(fn: str, status: int) -> None:
    if status != OK:
        lib = load_library()
        detail = lib.cudalm_b200_status_string(status).decode()
        if status == ERR_CUDA:
            detail += f"; cudaError {lib.cudalm_b200_last_cuda_error()}"
        raise CudalmB200Error(fn, status, detail)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, dtype: torch.dtype, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _need_current_device(*tensors: torch.Tensor) -> None:
    """The library works on the current device (its per-device caches, status word and
    scratch): a tensor of another device would be read through the wrong context."""
    cur = torch.cuda.current_device()
    for t in tensors:
        if t.device.index != cur:
            raise ValueError(f"a tensor is on cuda:{t.device.index}, the current device is cuda:{cur}")


def _need_sizes(weight: torch.Tensor, scales: torch.Tensor, x: torch.Tensor, y: torch.Tensor,
                N: int, K: int, B: int) -> None:
    """The buffers must hold what the kernel reads and writes."""
    if K <= 0 or K % GROUP_SIZE != 0 or N < 1 or B < 1:
        raise ValueError(f"bad shape N={N} K={K} B={B} (K must be a positive multiple of {GROUP_SIZE})")
    if weight.numel() < N * (K // 2) or scales.numel() < N * (K // GROUP_SIZE):
        raise ValueError("weight must hold [N, K/2] bytes and scales [N, K/128] values")
    if x.numel() != B * K:
        raise ValueError(f"x holds {x.numel()} values, expected B * K = {B * K}")
    if y.numel() < B * N:
        raise ValueError(f"y holds {y.numel()} values, needs B * N = {B * N}")


def device_status() -> int:
    """Synchronises and returns (then clears) the device-side status word."""
    out = _ci(0)
    _check("device_status", load_library().cudalm_b200_device_status(ctypes.byref(out)))
    return out.value


def set_tensor_path_min_rows(min_rows: int) -> int:
    """Batched calls with at least this many rows take the tcgen05 kernel
    (default 17); returns the previous value."""
    return int(load_library().cudalm_b200_set_tensor_path_min_rows(int(min_rows)))


def set_direct_path_max_bytes(max_bytes: int) -> int:
    """Single calls with at most 8 rows and at most this many weight bytes take
    the lean kernel (0: never); returns the previous value."""
    return int(load_library().cudalm_b200_set_direct_path_max_bytes(int(max_bytes)))


def set_exchange_timeout_ns(ns: int) -> int:
    """Limit of the device-side wait for the other ranks' candidates (default 2 s);
    returns the previous value."""
    return int(load_library().cudalm_b200_set_exchange_timeout_ns(int(ns)))


def launch_count() -> int:
    return int(load_library().cudalm_b200_launch_count())


@dataclass
class W4A16Linear:
    """One projection: packed int4 weight ``[N, K/2]`` uint8 and fp16 group
    scales ``[N, K/128]`` (CUDALM include/cudalm/weight_loader.h:58-63)."""
    weight: torch.Tensor
    scale: torch.Tensor
    N: int = 0
    K: int = 0

    def __post_init__(self):
        _need(self.weight, torch.uint8, "weight")
        _need(self.scale, torch.float16, "scale")
        n, half_k = self.weight.shape
        # CUDALM src/runtime/weight_loader_v2.cpp:479-482: N = dim0, K = 2*dim1
        self.N, self.K = int(n), int(half_k) * 2
        if tuple(self.scale.shape) != (self.N, self.K // GROUP_SIZE):
            raise ValueError("scale must be [N, K/128]")

    def bytes(self, M: int = 1) -> int:
        return self.N * self.K // 2 + self.N * (self.K // GROUP_SIZE) * 2 + M * self.K * 2 + M * self.N * 2


def int4_gemv_bf16(weight: torch.Tensor, scales: torch.Tensor, x: torch.Tensor,
                   y: Optional[torch.Tensor] = None, N: Optional[int] = None,
                   K: Optional[int] = None) -> torch.Tensor:
    """``y[n] = sum_k q[n,k] * scale[n,k/128] * x[k]`` (CUDALM
    include/cudalm/kernels/int4_gemv_bf16.h:46-48).  x bf16 ``[K]`` -> y bf16 ``[N]``."""
    _need(weight, torch.uint8, "weight")
    _need(scales, torch.float16, "scales")
    _need(x, torch.bfloat16, "x")
    N = int(weight.shape[0]) if N is None else N
    K = int(weight.shape[1]) * 2 if K is None else K
    if y is None:
        y = torch.empty(N, dtype=torch.bfloat16, device=x.device)
    _need(y, torch.bfloat16, "y")
    _need_current_device(weight, scales, x, y)
    _need_sizes(weight, scales, x, y, N, K, 1)
    st = load_library().cudalm_b200_int4_gemv_bf16(_ptr(weight), _ptr(scales), _ptr(x), _ptr(y),
                                                   N, K, _stream())
    _check("int4_gemv_bf16", st)
    return y


def batch_int4_gemv_bf16(weight: torch.Tensor, scales: torch.Tensor, x: torch.Tensor,
                         y: Optional[torch.Tensor] = None, N: Optional[int] = None,
                         K: Optional[int] = None, B: Optional[int] = None) -> torch.Tensor:
    """B rows against the same weights (CUDALM include/cudalm/kernels/batch_decode.h:61-63):
    x bf16 ``[B, K]`` -> y bf16 ``[B, N]``."""
    _need(weight, torch.uint8, "weight")
    _need(scales, torch.float16, "scales")
    _need(x, torch.bfloat16, "x")
    N = int(weight.shape[0]) if N is None else N
    K = int(weight.shape[1]) * 2 if K is None else K
    B = int(x.shape[0]) if B is None else B
    if y is None:
        y = torch.empty((B, N), dtype=torch.bfloat16, device=x.device)
    _need(y, torch.bfloat16, "y")
    _need_current_device(weight, scales, x, y)
    _need_sizes(weight, scales, x, y, N, K, B)
    st = load_library().cudalm_b200_batch_int4_gemv_bf16(_ptr(weight), _ptr(scales), _ptr(x),
                                                         _ptr(y), N, K, B, _stream())
    _check("batch_int4_gemv_bf16", st)
    return y


def _fill(desc: _LinearStruct, lin: W4A16Linear, x: torch.Tensor, y: torch.Tensor) -> None:
    _need(x, torch.bfloat16, "x")
    _need(y, torch.bfloat16, "y")
    M = 1 if x.dim() == 1 else int(x.shape[0])
    if x.numel() != M * lin.K or y.numel() != M * lin.N:
        raise ValueError("x must be [M, K] and y [M, N]")
    desc.weight, desc.scales = _ptr(lin.weight), _ptr(lin.scale)
    desc.x, desc.y = _ptr(x), _ptr(y)
    desc.N, desc.K, desc.M, desc.reserved = lin.N, lin.K, M, 0


def linear_multi(items: Sequence[Tuple[W4A16Linear, torch.Tensor, torch.Tensor]]) -> None:
    """Up to four independent projections ``(linear, x, y)`` in one launch."""
    arr = (_LinearStruct * len(items))()
    for d, (lin, x, y) in zip(arr, items):
        _fill(d, lin, x, y)
    _check("linear_multi", load_library().cudalm_b200_linear_multi(arr, len(items), _stream()))


def gate_up_bf16(gate: W4A16Linear, up: W4A16Linear, x: torch.Tensor,
                 gate_y: Optional[torch.Tensor] = None,
                 up_y: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """The MLP's gate and up projections over the shared input in one launch
    (CUDALM src/runtime/qwen35_deltanet.cpp:236-243 issues them as two calls)."""
    _need(x, torch.bfloat16, "x")
    if gate.N != up.N or gate.K != up.K:
        raise ValueError("gate and up must have the same shape")
    M = 1 if x.dim() == 1 else int(x.shape[0])
    shape = (gate.N,) if x.dim() == 1 else (M, gate.N)
    if gate_y is None:
        gate_y = torch.empty(shape, dtype=torch.bfloat16, device=x.device)
    if up_y is None:
        up_y = torch.empty(shape, dtype=torch.bfloat16, device=x.device)
    st = load_library().cudalm_b200_gate_up_bf16(
        _ptr(gate.weight), _ptr(gate.scale), _ptr(up.weight), _ptr(up.scale), _ptr(x),
        _ptr(gate_y), _ptr(up_y), gate.N, gate.K, M, _stream())
    _check("gate_up_bf16", st)
    return gate_y, up_y


def sample_topk(topk_idx: torch.Tensor, topk_val: torch.Tensor, temperature: float, top_k: int,
                top_p: float, rng_state: Optional[torch.Tensor] = None,
                token_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """CUDALM's sample_token (include/cudalm/sampling.h:200-234) on the device, over
    candidate lists [M, list_len] (value descending, tie -> lower id).  rng_state is an
    int64 tensor [M] holding each row's SplitMix64 state; it is advanced in place."""
    _need(topk_idx, torch.int32, "topk_idx")
    _need(topk_val, torch.bfloat16, "topk_val")
    M, list_len = int(topk_idx.shape[0]), int(topk_idx.shape[1])
    if rng_state is not None:
        _need(rng_state, torch.int64, "rng_state")
    if token_out is None:
        token_out = torch.empty((M,), dtype=torch.int32, device=topk_idx.device)
    st = load_library().cudalm_b200_sample_topk(
        _ptr(topk_idx), _ptr(topk_val), list_len, M, float(temperature), int(top_k), float(top_p),
        _ptr(rng_state) if rng_state is not None else None, _ptr(token_out), _stream())
    _check("sample_topk", st)
    return token_out


def gate_up_silu_bf16(gate: W4A16Linear, up: W4A16Linear, x: torch.Tensor,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(gate(x)) * up(x) in one launch, rounded as CUDALM rounds it
    (src/kernels/qwen35_kernels.cu:459-476 after the two projections)."""
    _need(x, torch.bfloat16, "x")
    if gate.N != up.N or gate.K != up.K:
        raise ValueError("gate and up must have the same shape")
    M = 1 if x.dim() == 1 else int(x.shape[0])
    if out is None:
        out = torch.empty((gate.N,) if x.dim() == 1 else (M, gate.N), dtype=torch.bfloat16,
                          device=x.device)
    st = load_library().cudalm_b200_gate_up_silu_bf16(
        _ptr(gate.weight), _ptr(gate.scale), _ptr(up.weight), _ptr(up.scale), _ptr(x), _ptr(out),
        gate.N, gate.K, M, _stream())
    _check("gate_up_silu_bf16", st)
    return out


def linear_residual_bf16(lin: W4A16Linear, x: torch.Tensor, residual: torch.Tensor,
                         y: Optional[torch.Tensor] = None) -> torch.Tensor:
    """residual + lin(x), rounded as CUDALM rounds it (projection to bf16, then
    src/kernels/qwen35_kernels.cu:442-456)."""
    _need(x, torch.bfloat16, "x")
    _need(residual, torch.bfloat16, "residual")
    M = 1 if x.dim() == 1 else int(x.shape[0])
    if y is None:
        y = torch.empty_like(residual)
    st = load_library().cudalm_b200_linear_residual_bf16(
        _ptr(lin.weight), _ptr(lin.scale), _ptr(x), _ptr(residual), _ptr(y), lin.N, lin.K, M,
        _stream())
    _check("linear_residual_bf16", st)
    return y


class LinearGroup:
    """Any number of independent projections run by one launch.  The
    descriptor table lives on the device; ``run()`` only launches."""

    def __init__(self, items: Sequence[Tuple[W4A16Linear, torch.Tensor, torch.Tensor]]):
        arr = (_LinearStruct * len(items))()
        for d, (lin, x, y) in zip(arr, items):
            _fill(d, lin, x, y)
        self._keep = list(items)  # the tensors must outlive the group
        handle = _vp()
        _check("group_create",
               load_library().cudalm_b200_group_create(arr, len(items), ctypes.byref(handle)))
        self._handle = handle

    @property
    def bytes(self) -> int:
        return int(load_library().cudalm_b200_group_bytes(self._handle))

    def run(self) -> None:
        _check("group_run", load_library().cudalm_b200_group_run(self._handle, _stream()))

    def close(self) -> None:
        if self._handle is not None:
            h, self._handle = self._handle, None
            _check("group_destroy", load_library().cudalm_b200_group_destroy(h))

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def quantize_w4a16(W: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 ``W [N, K]`` -> (packed uint8 ``[N, K/2]``, fp16 scale ``[N, K/128]``),
    bit-exact with CUDALM tools/common/w4a16_quant.py:25-60 (which also returns
    the unpacked q and the fp32 scale; those are not produced here)."""
    if W.dim() != 2:
        raise ValueError(f"expected 2-D W, got {W.dim()}D")
    _need(W, torch.bfloat16, "W")
    N, K = int(W.shape[0]), int(W.shape[1])
    if K % GROUP_SIZE != 0:
        raise ValueError(f"K must be a multiple of {GROUP_SIZE}, got {K}")
    packed = torch.empty((N, K // 2), dtype=torch.uint8, device=W.device)
    scale = torch.empty((N, K // GROUP_SIZE), dtype=torch.float16, device=W.device)
    st = load_library().cudalm_b200_quantize_w4a16(_ptr(W), N, K, _ptr(packed), _ptr(scale), _stream())
    _check("quantize_w4a16", st)
    return packed, scale


def packed_words(rows: int, k: int) -> int:
    """32-bit words of one packed candidate buffer: ids int32 ``[rows][k]`` then
    values bf16 ``[rows][k]``."""
    return rows * k + (rows * k + 1) // 2


def topk_merge_packed(gathered: torch.Tensor, rows_cap: int, M: int, k: int):
    """Merges ``[L, packed_words(rows_cap, k)]`` gathered candidate buffers."""
    _need(gathered, torch.int32, "gathered")
    L, words = int(gathered.shape[0]), int(gathered.shape[1])
    dev = gathered.device
    argmax = torch.empty(M, dtype=torch.int32, device=dev)
    idx = torch.empty((M, k), dtype=torch.int32, device=dev)
    val = torch.empty((M, k), dtype=torch.bfloat16, device=dev)
    st = load_library().cudalm_b200_topk_merge_packed(_ptr(gathered), L, words, rows_cap, M, k,
                                                      _ptr(argmax), _ptr(idx), _ptr(val), _stream())
    _check("topk_merge_packed", st)
    return argmax, idx, val


class LmHead:
    """Vocabulary projection stored as W4A16 with an on-device pick.

    ``rows`` are this rank's vocabulary rows; ``id_offset`` is the token id of
    row 0.  ``forward(x)`` returns ``(argmax [M] int32, topk_idx [M, k] int32,
    topk_val [M, k] bf16)``, ordered by value descending with ties to the lower
    id (CUDALM include/cudalm/greedy.h:28-39, include/cudalm/sampling.h:152-166).
    """

    def __init__(self, rows: W4A16Linear, top_k: int = 50, id_offset: int = 0,
                 max_rows: int = 32, keep_logits: bool = False):
        if not 1 <= top_k <= MAX_TOP_K:
            raise ValueError(f"top_k must be in 1..{MAX_TOP_K}")
        self.rows, self.top_k, self.id_offset = rows, top_k, id_offset
        self.max_rows = max_rows
        dev = rows.weight.device
        self.logits = (torch.empty((max_rows, rows.N), dtype=torch.bfloat16, device=dev)
                       if keep_logits else None)
        nbytes = int(load_library().cudalm_b200_lm_head_workspace_bytes(
            rows.N, rows.K, max_rows, top_k, 0 if keep_logits else 1))
        # 256-byte aligned by the caching allocator (512-byte granularity); zeroed once:
        # the pick's counters start at zero and every call leaves them there
        self.workspace = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
        self.argmax = torch.empty(max_rows, dtype=torch.int32, device=dev)
        # ids and values share one buffer so that a vocabulary-parallel caller can
        # send both with a single all-gather: int32 [R][k] then bf16 [R][k]
        n = max_rows * top_k
        self.packed = torch.empty(packed_words(max_rows, top_k), dtype=torch.int32, device=dev)
        self.topk_idx = self.packed[:n].view(max_rows, top_k)
        self.topk_val = self.packed[n:].view(torch.bfloat16)[:n].view(max_rows, top_k)

    def forward(self, x: torch.Tensor):
        _need(x, torch.bfloat16, "x")
        M = 1 if x.dim() == 1 else int(x.shape[0])
        if M > self.max_rows:
            raise ValueError(f"M={M} exceeds max_rows={self.max_rows}")
        if x.numel() != M * self.rows.K:
            raise ValueError(f"x holds {x.numel()} values, expected M * K = {M * self.rows.K}")
        _need_current_device(x, self.rows.weight)
        st = load_library().cudalm_b200_lm_head_topk(
            _ptr(self.rows.weight), _ptr(self.rows.scale), _ptr(x), self.rows.N, self.rows.K, M,
            self.top_k, self.id_offset, _ptr(self.logits), _ptr(self.argmax),
            _ptr(self.topk_idx), _ptr(self.topk_val), _ptr(self.workspace),
            self.workspace.numel(), _stream())
        _check("lm_head_topk", st)
        return self.argmax[:M], self.topk_idx[:M], self.topk_val[:M]


def lm_head_static_scratch_bytes() -> int:
    """Size of the fixed scratch array ``lm_head_topk_static`` uses (bytes held
    on every GPU that loads the library)."""
    return int(load_library().cudalm_b200_lm_head_static_scratch_bytes())


def lm_head_topk_static(rows: W4A16Linear, x: torch.Tensor, logits_out: torch.Tensor,
                        argmax_out: torch.Tensor, topk_idx: torch.Tensor, topk_val: torch.Tensor,
                        id_offset: int = 0) -> None:
    """The vocabulary projection and pick of ``LmHead.forward`` for callers that
    cannot allocate device memory for a workspace (a server whose pools own the
    whole GPU, a decode loop where ``cudaMalloc`` is forbidden): the scratch is a
    fixed array inside the library, nothing is allocated by the call, and every
    output buffer -- the ``[M, N]`` logits included -- is the caller's.

    At most 32 activation rows per call.  All calls on a device share the one
    scratch array, so calls that could overlap on the GPU (different streams,
    unordered) race; order them.  Make the first call on a device outside any
    stream capture."""
    _need(x, torch.bfloat16, "x")
    _need(logits_out, torch.bfloat16, "logits_out")
    _need(argmax_out, torch.int32, "argmax_out")
    _need(topk_idx, torch.int32, "topk_idx")
    _need(topk_val, torch.bfloat16, "topk_val")
    M = 1 if x.dim() == 1 else int(x.shape[0])
    top_k = int(topk_idx.shape[-1])
    if logits_out.numel() < M * rows.N or topk_idx.numel() < M * top_k or \
            topk_val.numel() < M * top_k or argmax_out.numel() < M:
        raise ValueError("an output buffer is too small")
    st = load_library().cudalm_b200_lm_head_topk_static(
        _ptr(rows.weight), _ptr(rows.scale), _ptr(x), rows.N, rows.K, M, top_k, id_offset,
        _ptr(logits_out), _ptr(argmax_out), _ptr(topk_idx), _ptr(topk_val), _stream())
    _check("lm_head_topk_static", st)


def topk_merge(list_idx: torch.Tensor, list_val: torch.Tensor):
    """Merges ``[L, M, k]`` candidate lists (ids < 0 are padding) into the final
    ``(argmax [M], topk_idx [M, k], topk_val [M, k])``."""
    _need(list_idx, torch.int32, "list_idx")
    _need(list_val, torch.bfloat16, "list_val")
    L, M, k = (int(v) for v in list_idx.shape)
    dev = list_idx.device
    argmax = torch.empty(M, dtype=torch.int32, device=dev)
    idx = torch.empty((M, k), dtype=torch.int32, device=dev)
    val = torch.empty((M, k), dtype=torch.bfloat16, device=dev)
    st = load_library().cudalm_b200_topk_merge(_ptr(list_idx), _ptr(list_val), L, M, k,
                                               _ptr(argmax), _ptr(idx), _ptr(val), _stream())
    _check("topk_merge", st)
    return argmax, idx, val
