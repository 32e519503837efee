"""`.cudalm` v2 container: the library's reader and the Python writer against a
file written by the reference's own writer (tests/golden/make_golden.py), and the
rejections the reference's reader makes (CUDALM src/runtime/weight_loader_v2.cpp:49-242,
tests/cpu/test_cudalm_v2_format.cpp)."""
import os
import struct

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="module")
def v2():
    from cudalm_agent_b200 import weights_v2
    return weights_v2


@pytest.fixture(scope="module")
def want():
    return np.load(os.path.join(GOLD, "tiny_v2.npz"))


def gold_bytes():
    with open(os.path.join(GOLD, "tiny_v2.cudalm"), "rb") as f:
        return f.read()


def test_reader_parses_the_reference_writers_file(v2, want):
    with v2.V2Reader(os.path.join(GOLD, "tiny_v2.cudalm")) as r:
        assert r.config_blob == want["config_blob"].tobytes()
        assert list(r.metadata.keys()) == list(want["meta_keys"])
        assert list(r.metadata.values()) == list(want["meta_values"])
        assert [t.name for t in r.tensors] == list(want["names"])
        for i, t in enumerate(r.tensors):
            assert t.dtype == int(want["dtypes"][i]) and t.align == int(want["aligns"][i])
            assert t.dims == tuple(int(d) for d in want[f"dims{i}"])
            assert r.host_bytes(t.name) == want[f"data{i}"].tobytes()
            assert t.offset % 16 == 0
        assert r.find("layers.0.mlp.gate_proj.scale").dims == (16, 2)
        assert r.find("no.such.tensor") is None


def test_writer_reproduces_the_reference_writers_bytes(v2, want):
    recs = [v2.Record(str(want["names"][i]), int(want["dtypes"][i]),
                      tuple(int(d) for d in want[f"dims{i}"]), want[f"data{i}"].tobytes(),
                      int(want["aligns"][i])) for i in range(len(want["names"]))]
    meta = dict(zip((str(k) for k in want["meta_keys"]), (str(v) for v in want["meta_values"])))
    assert v2.to_bytes(want["config_blob"].tobytes(), meta, recs) == gold_bytes()


def _rejected(v2, tmp_path, raw, needle):
    p = tmp_path / "bad.cudalm"
    p.write_bytes(raw)
    with pytest.raises(v2.V2FormatError) as ei:
        v2.V2Reader(str(p))
    assert needle in str(ei.value), str(ei.value)


def test_reader_rejections(v2, tmp_path):
    good = gold_bytes()
    hdr = struct.unpack("<8sIIIHHQQQQQQQQ", good[:88])
    table_off, payload_off = hdr[10], hdr[12]

    def patch(off, data):
        b = bytearray(good)
        b[off:off + len(data)] = data
        return bytes(b)

    _rejected(v2, tmp_path, good[:40], "too small")
    _rejected(v2, tmp_path, patch(0, b"CUDLMW01"), "magic")
    _rejected(v2, tmp_path, patch(8, struct.pack("<I", 3)), "version")
    _rejected(v2, tmp_path, patch(12, struct.pack("<I", 1)), "flags")
    _rejected(v2, tmp_path, patch(32, struct.pack("<Q", 80)), "config_size")
    _rejected(v2, tmp_path, good[:-8], "out of bounds")                       # payload cut short
    _rejected(v2, tmp_path, patch(72, struct.pack("<QQ", payload_off + 8, hdr[13] - 8)), "aligned")
    _rejected(v2, tmp_path, patch(40, struct.pack("<Q", 88 + 40)), "overlap")  # metadata inside config
    _rejected(v2, tmp_path, patch(88 + 84, struct.pack("<I", 7)), "reserved")
    _rejected(v2, tmp_path, patch(88 + 0, struct.pack("<i", 0)), "validation")  # hidden_size 0
    # first table entry: name_len, name, dtype, ndim, pad, dims...
    nlen = good[table_off]
    e = table_off + 1 + nlen
    _rejected(v2, tmp_path, patch(table_off + 1, b"l yers"), "character")
    _rejected(v2, tmp_path, patch(e, b"\x09"), "dtype")
    _rejected(v2, tmp_path, patch(e + 1, b"\x00"), "ndim")
    _rejected(v2, tmp_path, patch(e + 4, struct.pack("<q", 0)), "bad dim")
    _rejected(v2, tmp_path, patch(e + 4 + 16, struct.pack("<q", 5)), "unused dim")
    _rejected(v2, tmp_path, patch(e + 4 + 64 + 8, struct.pack("<Q", 17)), "byte_size")
    _rejected(v2, tmp_path, patch(e + 4 + 64 + 16, b"\x03"), "align")
    _rejected(v2, tmp_path, patch(e + 4 + 64, struct.pack("<Q", 1 << 40)), "payload bounds")
    # a duplicate name: rename the second tensor to the first one's name (same length needed)
    second = e + 4 + 64 + 16 + 2
    n2 = good[second]
    name1 = good[table_off + 1:table_off + 1 + nlen]
    if n2 >= nlen:
        dup = bytes([nlen]) + name1
        # shrinking a name shifts the table: rebuild only when lengths agree
        if n2 == nlen:
            _rejected(v2, tmp_path, patch(second, dup), "duplicate")
    with pytest.raises(v2.V2FormatError):
        v2.V2Reader(str(tmp_path / "missing.cudalm"))


def test_writer_rejects_bad_records(v2, want):
    cfg = want["config_blob"].tobytes()
    with pytest.raises(v2.V2FormatError):
        v2.to_bytes(cfg, {}, [v2.Record("a b", v2.DT_FP32, (1,), b"\x00" * 4)])
    with pytest.raises(v2.V2FormatError):
        v2.to_bytes(cfg, {}, [v2.Record("x", v2.DT_FP32, (2,), b"\x00" * 4)])
    with pytest.raises(v2.V2FormatError):
        v2.to_bytes(cfg, {}, [v2.Record("x", v2.DT_FP32, (1,), b"\x00" * 4)] * 2)
    with pytest.raises(v2.V2FormatError):
        v2.to_bytes(cfg[:80], {}, [])


@pytest.mark.gpu
def test_gpu_conversion_round_trip(v2, want, tmp_path):
    # bf16 matrix -> quantized on the GPU -> written -> read -> uploaded -> projection
    import torch
    import cudalm_agent_b200 as eng
    w = torch.from_numpy(want["w_bf16"].astype(np.int16)).view(torch.bfloat16).cuda()
    recs = v2.quantized_tensors("layers.0.mlp.gate_proj.weight", "layers.0.mlp.gate_proj.scale", w)
    # bit-exact with the reference's quantizer, whose output the golden file holds
    assert recs[0].data == want["data0"].tobytes() and recs[1].data == want["data1"].tobytes()
    extra = v2.tensor_record("layers.0.input_layernorm.weight",
                             torch.arange(24, dtype=torch.float32).to(torch.bfloat16))
    path = str(tmp_path / "conv.cudalm")
    v2.write_v2(path, want["config_blob"].tobytes(), {"arch": "qwen3_5"}, recs + [extra])
    with v2.V2Reader(path) as r:
        lin = r.linear("layers.0.mlp.gate_proj.weight", "layers.0.mlp.gate_proj.scale")
        assert (lin.N, lin.K) == (16, 256)
        assert lin.weight.cpu().numpy().tobytes() == want["data0"].tobytes()
        norm = r.upload("layers.0.input_layernorm.weight")
        assert torch.equal(norm.cpu(), torch.arange(24, dtype=torch.float32).to(torch.bfloat16))
        with pytest.raises(v2.V2FormatError):
            r.linear("layers.0.input_layernorm.weight", "layers.0.mlp.gate_proj.scale")
        x = torch.randn(256, device="cuda").to(torch.bfloat16)
        y = eng.int4_gemv_bf16(lin.weight, lin.scale, x)
        assert y.shape == (16,) and torch.isfinite(y.float()).all()
