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
* ``V2Reader.validate_layer`` / ``validate_full_model`` / ``load_layer`` are the
  model-level loader: a layer's tensor set checked against the configuration and
  uploaded, its W4A16 projections returned ready to call
  (src/runtime/weight_loader_v2.cpp:273-372, 383-408, 416-499).
* ``convert_safetensors`` walks a bf16 safetensors checkpoint as CUDALM's converter
  does (tools/convert_qwen35.py:181-264) and writes the v2 file, quantizing on the GPU.
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


class ModelConfig(NamedTuple):
    """The 88-byte configuration blob of a v2 file (field order is part of the
    format: CUDALM include/cudalm/weight_format_v2.h, tools/common/cudalm_v2.py:95-221)."""
    hidden_size: int
    num_hidden_layers: int
    intermediate_size: int
    vocab_size: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    lin_num_k_heads: int
    lin_num_v_heads: int
    lin_key_head_dim: int
    lin_value_head_dim: int
    lin_conv_kernel_dim: int
    full_attention_interval: int
    group_size: int
    max_seq_len: int
    eps: float
    rope_theta: float
    partial_rotary_factor: float
    mrope_section: Tuple[int, int, int] = (11, 11, 10)

    def to_blob(self) -> bytes:
        return struct.pack("<15i3f4i", *self[:15], self.eps, self.rope_theta,
                           self.partial_rotary_factor, *self.mrope_section, 0)

    @classmethod
    def from_blob(cls, blob: bytes) -> "ModelConfig":
        v = struct.unpack("<15i3f4i", blob)
        if v[21] != 0:
            raise V2FormatError("config blob reserved word must be 0")
        return cls(*v[:18], tuple(v[18:21]))

    # derived sizes (CUDALM include/cudalm/qwen35_config.h:55-88)
    @property
    def q_proj_out(self) -> int:
        return self.n_heads * self.head_dim * 2

    @property
    def kv_proj_out(self) -> int:
        return self.n_kv_heads * self.head_dim

    @property
    def o_proj_in(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def linear_value_dim(self) -> int:
        return self.lin_num_v_heads * self.lin_value_head_dim

    @property
    def linear_conv_dim(self) -> int:
        return 2 * self.lin_num_k_heads * self.lin_key_head_dim + self.linear_value_dim

    def is_full_attention(self, i: int) -> bool:
        return 0 <= i < self.num_hidden_layers and (i + 1) % self.full_attention_interval == 0


# names of cudalm_b200_v2_layer.proj[] / .aux[] in index order
PROJECTIONS = ("mlp.gate_proj", "mlp.up_proj", "mlp.down_proj", "self_attn.q_proj", "self_attn.k_proj",
               "self_attn.v_proj", "self_attn.o_proj", "linear_attn.in_proj_qkv",
               "linear_attn.in_proj_z", "linear_attn.in_proj_b", "linear_attn.in_proj_a",
               "linear_attn.out_proj")
AUX_TENSORS = ("input_layernorm.weight", "post_attention_layernorm.weight", "self_attn.q_norm.weight",
               "self_attn.k_norm.weight", "linear_attn.conv1d.weight", "linear_attn.dt_bias",
               "linear_attn.A_log", "linear_attn.norm.weight")


class _LayerStruct(ctypes.Structure):
    _fields_ = [("layer_idx", ctypes.c_int32), ("full_attention", ctypes.c_int32),
                ("proj", api._LinearStruct * len(PROJECTIONS)),
                ("aux", ctypes.c_void_p * len(AUX_TENSORS)),
                ("aux_dtype", ctypes.c_int32 * len(AUX_TENSORS)),
                ("aux_bytes", ctypes.c_uint64 * len(AUX_TENSORS))]


class LayerWeights:
    """One decoder layer on the GPU (CUDALM's Qwen35LayerWeights,
    include/cudalm/weight_loader_v2.h:60-110): ``linears`` maps the layer's projection
    names (``mlp.gate_proj``, ``self_attn.q_proj``, ``linear_attn.in_proj_qkv`` ...) to
    ``W4A16Linear`` and ``aux`` its other tensors by name; all are views of ``buffer``."""

    def __init__(self, layer_idx: int, full_attention: bool, buffer: torch.Tensor,
                 linears: Dict[str, "api.W4A16Linear"], aux: Dict[str, torch.Tensor]):
        self.layer_idx, self.full_attention, self.buffer = layer_idx, full_attention, buffer
        self.linears, self.aux = linears, aux


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

    @property
    def config(self) -> ModelConfig:
        return ModelConfig.from_blob(self.config_blob)

    def validate_layer(self, layer_idx: int) -> None:
        """Raises ``V2FormatError`` with the reference's message unless layer
        ``layer_idx`` holds its full tensor set with the dtypes and shapes the
        configuration implies."""
        err = ctypes.create_string_buffer(512)
        st = self._lib.cudalm_b200_v2_validate_layer(self._h, int(layer_idx), err, len(err))
        if st != 0:
            raise V2FormatError(err.value.decode(errors="replace") or f"status {st}")

    def validate_full_model(self) -> None:
        """Embedding, final norm, every layer and the tied vocabulary projection."""
        err = ctypes.create_string_buffer(512)
        st = self._lib.cudalm_b200_v2_validate_full_model(self._h, err, len(err))
        if st != 0:
            raise V2FormatError(err.value.decode(errors="replace") or f"status {st}")

    def load_layer(self, layer_idx: int, device: str = "cuda") -> LayerWeights:
        """Validates and uploads one layer into a single device buffer."""
        nbytes = int(self._lib.cudalm_b200_v2_layer_device_bytes(self._h, int(layer_idx)))
        if nbytes == 0:
            self.validate_layer(layer_idx)
            raise V2FormatError(f"layer {layer_idx} is empty")
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)  # 512-byte aligned by torch
        out = _LayerStruct()
        err = ctypes.create_string_buffer(512)
        st = self._lib.cudalm_b200_v2_load_layer(self._h, int(layer_idx), api._ptr(buf), nbytes,
                                                 api._stream(), ctypes.byref(out), err, len(err))
        if st != 0:
            raise V2FormatError(err.value.decode(errors="replace") or f"load_layer: status {st}")
        torch.cuda.current_stream().synchronize()  # the copies read the handle's host bytes
        base = buf.data_ptr()

        def view(ptr: int, nb: int, dtype: torch.dtype, shape) -> torch.Tensor:
            return buf[ptr - base:ptr - base + nb].view(dtype).view(shape)

        linears: Dict[str, "api.W4A16Linear"] = {}
        for name, l in zip(PROJECTIONS, out.proj):
            if not l.weight:
                continue
            n, k = int(l.N), int(l.K)
            linears[name] = api.W4A16Linear(view(l.weight, n * k // 2, torch.uint8, (n, k // 2)),
                                            view(l.scales, n * (k // 128) * 2, torch.float16, (n, k // 128)))
        aux: Dict[str, torch.Tensor] = {}
        for name, ptr, dt, nb in zip(AUX_TENSORS, out.aux, out.aux_dtype, out.aux_bytes):
            if ptr:
                info = self.find(f"layers.{layer_idx}.{name}")
                aux[name] = view(ptr, int(nb), _TORCH_DTYPE[int(dt)], info.dims)
        return LayerWeights(int(layer_idx), bool(out.full_attention), buf, linears, aux)

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


def convert_safetensors(st_path: str, out_path: str, config: ModelConfig, metadata: Dict[str, str],
                        layers: Optional[Sequence[int]] = None, full_model: bool = False,
                        prefix: str = "model.language_model.", device: str = "cuda") -> List[Record]:
    """bf16 safetensors checkpoint -> ``.cudalm`` v2, the walk of CUDALM's converter
    (tools/convert_qwen35.py:181-264) with the projections quantized by this library
    on the GPU: per layer the input layernorm, the attention or DeltaNet tensors, the
    post-attention layernorm and the MLP, then the final norm and, for a full model,
    the embedding (to which the vocabulary projection is tied).  Tensor order, names,
    dtypes and bytes are the reference converter's; ``metadata`` is written as given."""
    from safetensors import safe_open

    n_layers = config.num_hidden_layers
    layer_list = list(range(n_layers)) if (full_model or layers is None) else sorted(set(layers))
    for i in layer_list:
        if not 0 <= i < n_layers:
            raise V2FormatError(f"layer {i} out of range")
    records: List[Record] = []

    with safe_open(st_path, framework="pt") as f:
        def get(name: str) -> torch.Tensor:
            return f.get_tensor(prefix + name)

        def plain(name: str, want: torch.dtype) -> None:
            t = get(name)
            if t.dtype != want:
                raise V2FormatError(f"{name}: expected {want} source, got {t.dtype}")
            records.append(tensor_record(name, t))

        def w4(name: str) -> None:
            t = get(name + ".weight")
            if t.dtype != torch.bfloat16 or t.dim() != 2:
                raise V2FormatError(f"{name}: expected a 2-D bf16 source")
            records.extend(quantized_tensors(name + ".weight", name + ".scale", t.to(device)))

        for i in layer_list:
            L = f"layers.{i}."
            plain(L + "input_layernorm.weight", torch.bfloat16)
            if config.is_full_attention(i):
                for p in ("q_proj", "k_proj", "v_proj", "o_proj"):
                    w4(L + "self_attn." + p)
                plain(L + "self_attn.q_norm.weight", torch.bfloat16)
                plain(L + "self_attn.k_norm.weight", torch.bfloat16)
            else:
                for p in ("in_proj_qkv", "in_proj_z", "in_proj_b", "in_proj_a", "out_proj"):
                    w4(L + "linear_attn." + p)
                plain(L + "linear_attn.conv1d.weight", torch.bfloat16)
                plain(L + "linear_attn.dt_bias", torch.bfloat16)
                plain(L + "linear_attn.A_log", torch.float32)
                plain(L + "linear_attn.norm.weight", torch.float32)
            plain(L + "post_attention_layernorm.weight", torch.bfloat16)
            for p in ("gate_proj", "up_proj", "down_proj"):
                w4(L + "mlp." + p)
        plain("norm.weight", torch.bfloat16)
        if full_model:
            plain("embed_tokens.weight", torch.bfloat16)
    write_v2(out_path, config.to_blob(), metadata, records)
    return records
