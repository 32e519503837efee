"""CUDALM's ``.cudalm`` v2 weight container on this side of the projection path.

* ``V2Reader`` wraps the library's reader (``cudalm_b200_v2_*``): the same
  validation as CUDALM's ``WeightFileV2::load``
  (src/runtime/weight_loader_v2.cpp:49-242), tensors looked up by name and
  uploaded to the GPU, W4A16 projections returned as ``W4A16Linear``.
* ``write_v2`` emits the layout CUDALM's Python writer emits
  (tools/common/cudalm_v2.py:311-372: header | config | metadata | table | pad |
  payload, tensors 16-byte aligned inside the payload, padding bytes part of it),
  byte for byte.
* ``quantized_tensors`` turns a bf16 matrix on the GPU into the two records of a
  W4A16 projection with the library's quantizer (the GPU form of
  tools/convert_qwen35.py:181-189).
"""
from __future__ import annotations

import ctypes
import struct
from typing import Dict, Iterable, List, NamedTuple, Optional, Sequence, Tuple

import torch

from . import api

DT_FP16, DT_INT4_PACKED, DT_FP16_SCALE, DT_FP32, DT_BF16 = 1, 2, 3, 4, 5
ELEMENT_BYTES = {DT_FP16: 2, DT_INT4_PACKED: 1, DT_FP16_SCALE: 2, DT_FP32: 4, DT_BF16: 2}
_TORCH_DTYPE = {DT_FP16: torch.float16, DT_INT4_PACKED: torch.uint8, DT_FP16_SCALE: torch.float16,
                DT_FP32: torch.float32, DT_BF16: torch.bfloat16}
HEADER_BYTES = 88
CONFIG_BYTES = 88
PAYLOAD_ALIGN = 16


class V2FormatError(ValueError):
    """A file the reader rejects, or a record the writer cannot emit."""


class TensorInfo(NamedTuple):
    name: str
    dtype: int
    dims: Tuple[int, ...]
    offset: int
    byte_size: int
    align: int


class _TensorStruct(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("dtype", ctypes.c_int32), ("ndim", ctypes.c_int32),
                ("dims", ctypes.c_int64 * 8), ("offset", ctypes.c_uint64),
                ("byte_size", ctypes.c_uint64), ("align", ctypes.c_int32),
                ("reserved", ctypes.c_int32), ("host_bytes", ctypes.c_void_p)]


class V2Reader:
    """An open, validated ``.cudalm`` v2 file."""

    def __init__(self, path: str):
        lib = api.load_library()
        handle = ctypes.c_void_p()
        err = ctypes.create_string_buffer(512)
        st = lib.cudalm_b200_v2_open(path.encode(), ctypes.byref(handle), err, len(err))
        if st != 0:
            raise V2FormatError(f"{path}: {err.value.decode(errors='replace') or 'status %d' % st}")
        self._lib, self._h = lib, handle
        self.tensors: List[TensorInfo] = []
        self._host: Dict[str, Tuple[int, int]] = {}
        t = _TensorStruct()
        for i in range(lib.cudalm_b200_v2_num_tensors(handle)):
            api._check("v2_tensor_at", lib.cudalm_b200_v2_tensor_at(handle, i, ctypes.byref(t)))
            info = TensorInfo(t.name.decode(), t.dtype, tuple(t.dims[:t.ndim]), t.offset, t.byte_size,
                              t.align)
            self.tensors.append(info)
            self._host[info.name] = (t.host_bytes, t.byte_size)
        blob = (ctypes.c_uint8 * CONFIG_BYTES)()
        api._check("v2_config_blob", lib.cudalm_b200_v2_config_blob(handle, blob))
        self.config_blob = bytes(blob)
        self.metadata: Dict[str, str] = {}
        k, v = ctypes.c_char_p(), ctypes.c_char_p()
        for i in range(lib.cudalm_b200_v2_num_metadata(handle)):
            api._check("v2_metadata_at",
                       lib.cudalm_b200_v2_metadata_at(handle, i, ctypes.byref(k), ctypes.byref(v)))
            self.metadata[k.value.decode()] = v.value.decode()

    def close(self) -> None:
        if self._h:
            self._lib.cudalm_b200_v2_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def find(self, name: str) -> Optional[TensorInfo]:
        i = self._lib.cudalm_b200_v2_find(self._h, name.encode())
        return self.tensors[i] if i >= 0 else None

    def host_bytes(self, name: str) -> bytes:
        ptr, size = self._host[name]
        return ctypes.string_at(ptr, size)

    def upload(self, name: str, device: str = "cuda") -> torch.Tensor:
        """The tensor on the GPU, in its stored dtype and dims."""
        i = self._lib.cudalm_b200_v2_find(self._h, name.encode())
        if i < 0:
            raise KeyError(name)
        info = self.tensors[i]
        out = torch.empty(info.dims, dtype=_TORCH_DTYPE[info.dtype], device=device)
        api._check("v2_upload", self._lib.cudalm_b200_v2_upload(
            self._h, i, api._ptr(out), out.numel() * out.element_size(), api._stream()))
        return out

    def linear(self, weight_name: str, scale_name: str) -> "api.W4A16Linear":
        """A W4A16 projection stored as int4_packed [N, K/2] + fp16_scale [N, K/128]."""
        n, k = ctypes.c_int(), ctypes.c_int()
        st = self._lib.cudalm_b200_v2_linear(self._h, weight_name.encode(), scale_name.encode(), None,
                                             None, ctypes.byref(n), ctypes.byref(k))
        if st != 0:
            raise V2FormatError(f"{weight_name} / {scale_name} are not a W4A16 projection")
        return api.W4A16Linear(self.upload(weight_name), self.upload(scale_name))


class Record(NamedTuple):
    """One tensor to write; ``dims`` of an int4_packed tensor are in packed bytes."""
    name: str
    dtype: int
    dims: Tuple[int, ...]
    data: bytes
    align: int = PAYLOAD_ALIGN


def _check_record(r: Record) -> None:
    if r.dtype not in ELEMENT_BYTES:
        raise V2FormatError(f"bad dtype id {r.dtype}")
    raw = r.name.encode("utf-8")
    if not 1 <= len(raw) <= 255 or not all(
            c.isascii() and (c.isalnum() or c in "._-") for c in r.name):
        raise V2FormatError(f"bad tensor name {r.name!r}")
    if not 1 <= len(r.dims) <= 8 or not all(0 < d <= 100000000 for d in r.dims):
        raise V2FormatError(f"bad dims {r.dims} for {r.name!r}")
    numel = 1
    for d in r.dims:
        numel *= d
    if len(r.data) != numel * ELEMENT_BYTES[r.dtype]:
        raise V2FormatError(f"{r.name!r}: {len(r.data)} bytes do not match dtype and dims")
    if r.align not in (1, 2, 4, 8, 16):
        raise V2FormatError(f"bad align {r.align} for {r.name!r}")


def to_bytes(config_blob: bytes, metadata: Dict[str, str], records: Sequence[Record]) -> bytes:
    """The file image.  Section order and padding follow CUDALM's writer."""
    if len(config_blob) != CONFIG_BYTES:
        raise V2FormatError("the config blob is 88 bytes")
    if len(records) > 100000 or len(metadata) > 256:
        raise V2FormatError("too many tensors or metadata entries")
    names = [r.name for r in records]
    if len(set(names)) != len(names):
        raise V2FormatError("duplicate tensor name")
    meta = bytearray()
    for k, v in metadata.items():
        kb, vb = k.encode("utf-8"), v.encode("utf-8")
        if len(kb) > 255 or len(vb) > 4096:
            raise V2FormatError(f"metadata entry too long: {k!r}")
        meta += struct.pack("<B", len(kb)) + kb + struct.pack("<H", len(vb)) + vb
    table, payload = bytearray(), bytearray()
    for r in records:
        _check_record(r)
        dims8 = list(r.dims) + [0] * (8 - len(r.dims))
        nb = r.name.encode("utf-8")
        table += struct.pack("<B", len(nb)) + nb
        table += struct.pack("<BBH", r.dtype, len(r.dims), 0)
        table += struct.pack("<8q", *dims8)
        table += struct.pack("<QQ", len(payload), len(r.data))
        table += struct.pack("<BB", r.align, 0)
        payload += r.data
        payload += b"\x00" * ((-len(payload)) % PAYLOAD_ALIGN)  # the padding is payload
    config_off = HEADER_BYTES
    meta_off = config_off + CONFIG_BYTES
    table_off = meta_off + len(meta)
    payload_off = table_off + len(table)
    payload_off += (-payload_off) % PAYLOAD_ALIGN
    header = struct.pack("<8sIIIHHQQQQQQQQ", b"CUDLMW02", 2, 0, len(records), len(metadata), 0,
                         config_off, CONFIG_BYTES, meta_off, len(meta), table_off, len(table),
                         payload_off, len(payload))
    body = header + config_blob + bytes(meta) + bytes(table)
    return body + b"\x00" * (payload_off - len(body)) + bytes(payload)


def write_v2(path: str, config_blob: bytes, metadata: Dict[str, str],
             records: Sequence[Record]) -> None:
    with open(path, "wb") as f:
        f.write(to_bytes(config_blob, metadata, records))


def tensor_record(name: str, t: torch.Tensor) -> Record:
    """A record holding a tensor as it is (fp16, fp32 or bf16)."""
    dtype = {torch.float16: DT_FP16, torch.float32: DT_FP32, torch.bfloat16: DT_BF16}.get(t.dtype)
    if dtype is None:
        raise V2FormatError(f"{name!r}: dtype {t.dtype} has no v2 encoding")
    raw = t.detach().contiguous().cpu().view(torch.uint8).numpy().tobytes()
    return Record(name, dtype, tuple(int(d) for d in t.shape), raw)


def quantized_tensors(weight_name: str, scale_name: str, w_bf16: torch.Tensor) -> List[Record]:
    """The two records of a W4A16 projection, quantized on the GPU from a bf16
    matrix [N, K] (bit-exact with CUDALM's tools/common/w4a16_quant.py:25-60)."""
    packed, scale = api.quantize_w4a16(w_bf16)
    n, k = int(w_bf16.shape[0]), int(w_bf16.shape[1])
    return [Record(weight_name, DT_INT4_PACKED, (n, k // 2), packed.cpu().numpy().tobytes()),
            Record(scale_name, DT_FP16_SCALE, (n, k // 128),
                   scale.cpu().view(torch.uint8).numpy().tobytes())]
