"""ctypes front end of the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Loads ``oracle/liboracle.so`` (the plain-C restatement in ``w4a16_oracle.c``)
and, when it has been built, ``oracle/_ref/libcudalm_ref.so`` (the reference's
own functions compiled from the reference sources by ``oracle/Makefile``).

Only the test suite, the smoke check and the benchmark's CPU-baseline leg may
import this module; the shipped package never does.

All 16-bit float data crosses this boundary as raw bits in ``numpy.uint16``
arrays (numpy has no bfloat16): bf16 for activations/outputs/logits, IEEE
binary16 for scales.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libcudalm_ref.so")

_u8p = ctypes.POINTER(ctypes.c_uint8)
_u16p = ctypes.POINTER(ctypes.c_uint16)
_i32p = ctypes.POINTER(ctypes.c_int32)
_f32p = ctypes.POINTER(ctypes.c_float)


def build(force: bool = False) -> None:
    """Compile the oracle (and the reference bridge when the reference tree is
    present) with ``make -C oracle``."""
    if force or not os.path.exists(_LIB_PATH):
        subprocess.run(["make", "-C", _HERE, "all"], check=True,
                       stdout=subprocess.DEVNULL)


_lib = None
_ref = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        L.orc_bf16_to_f32.restype = ctypes.c_float
        L.orc_bf16_to_f32.argtypes = [ctypes.c_uint16]
        L.orc_f32_to_bf16.restype = ctypes.c_uint16
        L.orc_f32_to_bf16.argtypes = [ctypes.c_float]
        L.orc_f16_to_f32.restype = ctypes.c_float
        L.orc_f16_to_f32.argtypes = [ctypes.c_uint16]
        L.orc_f32_to_f16.restype = ctypes.c_uint16
        L.orc_f32_to_f16.argtypes = [ctypes.c_float]
        L.orc_unpack_lo.argtypes = [ctypes.c_uint8]
        L.orc_unpack_hi.argtypes = [ctypes.c_uint8]
        L.orc_pack_byte.restype = ctypes.c_uint8
        L.orc_pack_byte.argtypes = [ctypes.c_int, ctypes.c_int]
        L.orc_gemv_bf16.argtypes = [_u8p, _u16p, _u16p, ctypes.c_int,
                                    ctypes.c_int, _u16p, _f32p]
        L.orc_batch_gemv_bf16.argtypes = [_u8p, _u16p, _u16p, ctypes.c_int,
                                          ctypes.c_int, ctypes.c_int, _u16p,
                                          ctypes.c_int]
        L.orc_quantize_w4a16.argtypes = [_u16p, ctypes.c_int, ctypes.c_int,
                                         _u8p, _u16p, ctypes.c_int]
        L.orc_argmax_bf16.argtypes = [_u16p, ctypes.c_int]
        L.orc_topk_bf16.argtypes = [_u16p, ctypes.c_int, ctypes.c_int, _i32p,
                                    _u16p]
        L.orc_sample_from_topk.argtypes = [_i32p, _u16p, ctypes.c_int, ctypes.c_float, ctypes.c_int,
                                           ctypes.c_float, ctypes.POINTER(ctypes.c_uint64)]
        L.orc_sample_from_topk.restype = ctypes.c_int
        L.orc_silu_mul_bf16.argtypes = [_u16p, _u16p, _u16p, ctypes.c_size_t]
        L.orc_silu_mul_bf16.restype = None
        L.orc_add_bf16.argtypes = [_u16p, _u16p, _u16p, ctypes.c_size_t]
        L.orc_add_bf16.restype = None
        _lib = L
    return _lib


def have_ref() -> bool:
    return os.path.exists(_REF_PATH)


def ref() -> ctypes.CDLL:
    """The reference's own functions (CPU entry points are safe without a
    GPU; the ``ref_gpu_*`` ones need one)."""
    global _ref
    if _ref is None:
        R = ctypes.CDLL(_REF_PATH)
        R.ref_cpu_gemv_bf16.argtypes = [_u8p, _u16p, _u16p, ctypes.c_int,
                                        ctypes.c_int, _u16p]
        R.ref_cpu_gemv_bf16.restype = None
        R.ref_cpu_argmax_bf16.argtypes = [_u16p, ctypes.c_int]
        R.ref_cpu_topk_keep.argtypes = [_u16p, ctypes.c_int, ctypes.c_int, _u8p]
        R.ref_cpu_topk_keep.restype = None
        R.ref_cpu_sample_token.argtypes = [_u16p, ctypes.c_int, ctypes.c_float, ctypes.c_int,
                                           ctypes.c_float, ctypes.POINTER(ctypes.c_uint64)]
        R.ref_cpu_sample_token.restype = ctypes.c_int
        R.ref_cpu_compare_bf16_ok.argtypes = [_u16p, _u16p, ctypes.c_size_t]
        for name in ("ref_gpu_int4_gemv_bf16",):
            getattr(R, name).argtypes = [ctypes.c_void_p] * 4 + [
                ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
            getattr(R, name).restype = None
        R.ref_gpu_batch_int4_gemv_bf16.argtypes = [ctypes.c_void_p] * 4 + [
            ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        R.ref_gpu_batch_int4_gemv_bf16.restype = None
        R.ref_gpu_bf16_gemv.argtypes = [ctypes.c_void_p] * 3 + [
            ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        R.ref_gpu_bf16_gemv.restype = None
        _ref = R
    return _ref


# --------------------------------------------------------------------------
# numpy helpers for 16-bit float bit patterns
# --------------------------------------------------------------------------
def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bits, round to nearest even (finite inputs)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    lsb = (u >> np.uint32(16)) & np.uint32(1)
    r = u + np.uint32(0x7FFF) + lsb
    return (r >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32)
            << np.uint32(16)).view(np.float32)


def _c(a: np.ndarray, dtype) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=dtype)
    return a


def _p(a: np.ndarray, ptype):
    return a.ctypes.data_as(ptype)


# --------------------------------------------------------------------------
# Oracle API
# --------------------------------------------------------------------------
def gemv_bf16(W: np.ndarray, S: np.ndarray, x: np.ndarray,
              return_acc: bool = False):
    """y[n] = bf16(sum_k q[n,k] * s[n,k/128] * x[k]) in the reference's term
    order.  W uint8 [N,K/2]; S uint16 (fp16 bits) [N,K/128]; x uint16 (bf16
    bits) [K].  Returns uint16 bf16 bits [N] (and the fp32 sums if asked)."""
    W = _c(W, np.uint8)
    S = _c(S, np.uint16)
    x = _c(x, np.uint16)
    N, K = W.shape[0], W.shape[1] * 2
    assert S.shape == (N, K // 128) and x.shape == (K,)
    y = np.empty(N, np.uint16)
    acc = np.empty(N, np.float32)
    rc = lib().orc_gemv_bf16(_p(W, _u8p), _p(S, _u16p), _p(x, _u16p), N, K,
                             _p(y, _u16p), _p(acc, _f32p))
    if rc:
        raise ValueError(f"orc_gemv_bf16 rejected N={N} K={K}")
    return (y, acc) if return_acc else y


def batch_gemv_bf16(W, S, x, threads: int = 1) -> np.ndarray:
    """Batched GEMV: x uint16 [B,K] -> y uint16 [B,N]; row b equals
    ``gemv_bf16(W, S, x[b])`` bit for bit whatever ``threads`` is."""
    W = _c(W, np.uint8)
    S = _c(S, np.uint16)
    x = _c(x, np.uint16)
    N, K = W.shape[0], W.shape[1] * 2
    B = x.shape[0]
    assert x.shape == (B, K)
    y = np.empty((B, N), np.uint16)
    rc = lib().orc_batch_gemv_bf16(_p(W, _u8p), _p(S, _u16p), _p(x, _u16p), N,
                                   K, B, _p(y, _u16p), threads)
    if rc:
        raise ValueError(f"orc_batch_gemv_bf16 rejected N={N} K={K} B={B}")
    return y


def quantize_w4a16(Wbf16: np.ndarray, threads: int = 1):
    """bf16 bits [N,K] -> (packed uint8 [N,K/2], scale fp16 bits [N,K/128])."""
    Wb = _c(Wbf16, np.uint16)
    N, K = Wb.shape
    packed = np.empty((N, K // 2), np.uint8)
    scale = np.empty((N, K // 128), np.uint16)
    rc = lib().orc_quantize_w4a16(_p(Wb, _u16p), N, K, _p(packed, _u8p),
                                  _p(scale, _u16p), threads)
    if rc:
        raise ValueError(f"orc_quantize_w4a16 rejected N={N} K={K}")
    return packed, scale


def argmax_bf16(logits: np.ndarray) -> int:
    l = _c(logits, np.uint16)
    return int(lib().orc_argmax_bf16(_p(l, _u16p), l.size))


def topk_bf16(logits: np.ndarray, k: int):
    """Returns (ids int32 [min(k,n)], values bf16 bits) ordered by value
    descending, ties by lower id."""
    l = _c(logits, np.uint16)
    kk = min(k, l.size)
    idx = np.empty(kk, np.int32)
    val = np.empty(kk, np.uint16)
    n = lib().orc_topk_bf16(_p(l, _u16p), l.size, k, _p(idx, _i32p),
                            _p(val, _u16p))
    assert n == kk
    return idx, val


def sample_from_topk(idx: np.ndarray, val: np.ndarray, temperature: float, top_k: int,
                     top_p: float, state: int):
    """The reference's sample_token on a candidate list (value descending, tie ->
    lower id); returns (token, new SplitMix64 state)."""
    i = np.ascontiguousarray(idx, dtype=np.int32)
    v = np.ascontiguousarray(val, dtype=np.uint16)
    st = ctypes.c_uint64(state)
    tok = lib().orc_sample_from_topk(_p(i, _i32p), _p(v, _u16p), i.size, float(temperature),
                                     int(top_k), float(top_p), ctypes.byref(st))
    return int(tok), int(st.value)


def silu_mul_bf16(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    g = _c(gate, np.uint16)
    u = _c(up, np.uint16)
    y = np.empty_like(g)
    lib().orc_silu_mul_bf16(_p(g, _u16p), _p(u, _u16p), _p(y, _u16p), g.size)
    return y


def add_bf16(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    a = _c(a, np.uint16)
    b = _c(b, np.uint16)
    y = np.empty_like(a)
    lib().orc_add_bf16(_p(a, _u16p), _p(b, _u16p), _p(y, _u16p), a.size)
    return y


def unpack_int4(W: np.ndarray) -> np.ndarray:
    """uint8 [N,K/2] -> int8 [N,K] (low nibble first, sign-extended)."""
    W = _c(W, np.uint8)
    lo = (W & 15).astype(np.int8)
    hi = (W >> 4).astype(np.int8)
    lo = np.where(lo > 7, lo - 16, lo).astype(np.int8)
    hi = np.where(hi > 7, hi - 16, hi).astype(np.int8)
    return np.stack([lo, hi], axis=-1).reshape(W.shape[0], -1)


# --------------------------------------------------------------------------
# The reference's own CPU functions (present only when oracle/_ref is built)
# --------------------------------------------------------------------------
def ref_gemv_bf16(W, S, x) -> np.ndarray:
    W = _c(W, np.uint8)
    S = _c(S, np.uint16)
    x = _c(x, np.uint16)
    N, K = W.shape[0], W.shape[1] * 2
    y = np.empty(N, np.uint16)
    ref().ref_cpu_gemv_bf16(_p(W, _u8p), _p(S, _u16p), _p(x, _u16p), N, K,
                            _p(y, _u16p))
    return y


def ref_argmax_bf16(logits) -> int:
    l = _c(logits, np.uint16)
    return int(ref().ref_cpu_argmax_bf16(_p(l, _u16p), l.size))


def ref_topk_keep(logits, k: int) -> np.ndarray:
    l = _c(logits, np.uint16)
    keep = np.zeros(l.size, np.uint8)
    ref().ref_cpu_topk_keep(_p(l, _u16p), l.size, k, _p(keep, _u8p))
    return keep.astype(bool)


def ref_sample_token(logits, temperature: float, top_k: int, top_p: float, state: int):
    """The reference's own sample_token on full logits; returns (token, new state)."""
    l = _c(logits, np.uint16)
    st = ctypes.c_uint64(state)
    tok = ref().ref_cpu_sample_token(_p(l, _u16p), l.size, float(temperature), int(top_k),
                                     float(top_p), ctypes.byref(st))
    return int(tok), int(st.value)


def ref_compare_bf16_ok(ref_bits, act_bits) -> bool:
    r = _c(ref_bits, np.uint16).ravel()
    a = _c(act_bits, np.uint16).ravel()
    return bool(ref().ref_cpu_compare_bf16_ok(_p(r, _u16p), _p(a, _u16p), r.size))
