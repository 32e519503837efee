"""Model-level loading of a `.cudalm` v2 file and the safetensors conversion, against a
two-layer model converted by the reference's own converter walk, quantizer and writer
(tests/golden/tiny_model_v2.cudalm, made by tests/golden/make_golden.py).

Reference: WeightFileV2::validate_layer / validate_full_model and
Qwen35LayerWeights::load (CUDALM src/runtime/weight_loader_v2.cpp:273-372, 383-408,
416-499); tools/convert_qwen35.py:181-264.
"""
import os

import numpy as np
import pytest

from helpers import CHECKPOINT_PREFIX, TINY_MODEL, TINY_MODEL_META, tiny_model_tensors

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = os.path.join(ROOT, "tests", "golden", "tiny_model_v2.cudalm")


@pytest.fixture(scope="module")
def v2():
    from cudalm_agent_b200 import weights_v2
    return weights_v2


def _records(v2, reader):
    return [v2.Record(t.name, t.dtype, t.dims, reader.host_bytes(t.name), t.align) for t in reader.tensors]


def test_config_and_full_model_validate(v2):
    with v2.V2Reader(GOLD) as r:
        c = r.config
        assert c.to_blob() == r.config_blob == v2.ModelConfig(**TINY_MODEL).to_blob()
        assert (c.hidden_size, c.intermediate_size, c.vocab_size, c.mrope_section) == (128, 128, 256, (3, 3, 2))
        assert not c.is_full_attention(0) and c.is_full_attention(1)
        r.validate_layer(0)
        r.validate_layer(1)
        r.validate_full_model()
        for bad in (-1, 2):
            with pytest.raises(v2.V2FormatError, match="layer_idx out of range"):
                r.validate_layer(bad)


def _rewrite(v2, tmp_path, change, meta=None):
    """The golden file with its record list changed by `change`, reopened."""
    with v2.V2Reader(GOLD) as r:
        recs = change(_records(v2, r))
        blob, md = r.config_blob, dict(r.metadata) if meta is None else meta
    p = tmp_path / "changed.cudalm"
    v2.write_v2(str(p), blob, md, recs)
    return v2.V2Reader(str(p))


def test_layer_faults_are_reported_as_the_reference_reports_them(v2, tmp_path):
    # a missing tensor
    r = _rewrite(v2, tmp_path, lambda rs: [x for x in rs if x.name != "layers.1.self_attn.k_proj.scale"])
    r.validate_layer(0)
    with pytest.raises(v2.V2FormatError, match=r"missing tensor 'layers\.1\.self_attn\.k_proj\.scale'"):
        r.validate_layer(1)
    with pytest.raises(v2.V2FormatError, match=r"layer 1: missing tensor"):
        r.validate_full_model()
    r.close()

    # a wrong dtype: the scale stored as plain fp16
    def as_fp16(rs):
        return [x._replace(dtype=v2.DT_FP16) if x.name == "layers.0.mlp.up_proj.scale" else x for x in rs]
    r = _rewrite(v2, tmp_path, as_fp16)
    with pytest.raises(v2.V2FormatError,
                       match=r"dtype mismatch for 'layers\.0\.mlp\.up_proj\.scale' \(expected fp16_scale\)"):
        r.validate_layer(0)
    r.close()

    # a wrong shape: same bytes, transposed dims
    def transposed(rs):
        return [x._replace(dims=(x.dims[1], x.dims[0])) if x.name == "layers.0.linear_attn.in_proj_z.weight"
                else x for x in rs]
    r = _rewrite(v2, tmp_path, transposed)
    with pytest.raises(v2.V2FormatError,
                       match=r"shape mismatch for 'layers\.0\.linear_attn\.in_proj_z\.weight' \(expected 2-D\)"):
        r.validate_layer(0)
    r.close()

    # the first fault in the reference's order is the one reported: norms before the MLP
    r = _rewrite(v2, tmp_path, lambda rs: [x for x in rs if x.name not in (
        "layers.0.mlp.gate_proj.weight", "layers.0.post_attention_layernorm.weight")])
    with pytest.raises(v2.V2FormatError, match=r"missing tensor 'layers\.0\.post_attention_layernorm\.weight'"):
        r.validate_layer(0)
    r.close()


def test_full_model_needs_embedding_norm_and_tied_head(v2, tmp_path):
    r = _rewrite(v2, tmp_path, lambda rs: [x for x in rs if x.name != "embed_tokens.weight"])
    with pytest.raises(v2.V2FormatError, match=r"missing tensor 'embed_tokens\.weight'"):
        r.validate_full_model()
    r.close()
    r = _rewrite(v2, tmp_path, lambda rs: [x for x in rs if x.name != "norm.weight"])
    with pytest.raises(v2.V2FormatError, match=r"missing tensor 'norm\.weight'"):
        r.validate_full_model()
    r.close()
    meta = {k: v for k, v in TINY_MODEL_META.items() if k != "tie_word_embeddings"}
    r = _rewrite(v2, tmp_path, lambda rs: rs, meta=meta)
    with pytest.raises(v2.V2FormatError, match="tie_word_embeddings"):
        r.validate_full_model()
    r.close()


def test_load_layer_refuses_bad_arguments(v2):
    import ctypes
    from cudalm_agent_b200 import api
    lib = api.load_library()
    with v2.V2Reader(GOLD) as r:
        assert lib.cudalm_b200_v2_layer_device_bytes(r._h, 0) % 256 == 0
        assert lib.cudalm_b200_v2_layer_device_bytes(r._h, 5) == 0
        out = v2._LayerStruct()
        err = ctypes.create_string_buffer(256)
        assert lib.cudalm_b200_v2_load_layer(r._h, 0, None, 1 << 20, None, ctypes.byref(out), err, 256) == api.ERR_NULL
        # a destination off the 256-byte boundary, and one that is too small (no copy is made)
        assert lib.cudalm_b200_v2_load_layer(r._h, 0, 0x1000 + 16, 1 << 20, None, ctypes.byref(out), err, 256) == api.ERR_MISALIGNED
        assert lib.cudalm_b200_v2_load_layer(r._h, 0, 0x1000, 1024, None, ctypes.byref(out), err, 256) == api.ERR_TOO_LARGE
        assert lib.cudalm_b200_v2_load_layer(r._h, 9, 0x1000, 1 << 20, None, ctypes.byref(out), err, 256) == 9
        assert b"layer_idx out of range" in err.value


# ---------------------------------------------------------------------------------------
# on a GPU
# ---------------------------------------------------------------------------------------

@pytest.mark.gpu
def test_layers_load_with_the_files_bytes_and_shapes(v2):
    import torch
    with v2.V2Reader(GOLD) as r:
        c = r.config
        H, I = c.hidden_size, c.intermediate_size
        want_shapes = [
            {"mlp.gate_proj": (I, H), "mlp.up_proj": (I, H), "mlp.down_proj": (H, I),
             "linear_attn.in_proj_qkv": (c.linear_conv_dim, H), "linear_attn.in_proj_z": (c.linear_value_dim, H),
             "linear_attn.in_proj_b": (c.lin_num_v_heads, H), "linear_attn.in_proj_a": (c.lin_num_v_heads, H),
             "linear_attn.out_proj": (H, c.linear_value_dim)},
            {"mlp.gate_proj": (I, H), "mlp.up_proj": (I, H), "mlp.down_proj": (H, I),
             "self_attn.q_proj": (c.q_proj_out, H), "self_attn.k_proj": (c.kv_proj_out, H),
             "self_attn.v_proj": (c.kv_proj_out, H), "self_attn.o_proj": (H, c.o_proj_in)}]
        for i in range(c.num_hidden_layers):
            layer = r.load_layer(i)
            assert layer.full_attention == c.is_full_attention(i)
            assert {k: (l.N, l.K) for k, l in layer.linears.items()} == want_shapes[i]
            for name, lin in layer.linears.items():
                assert lin.weight.data_ptr() % 256 == 0 and lin.scale.data_ptr() % 256 == 0
                assert lin.weight.cpu().numpy().tobytes() == r.host_bytes(f"layers.{i}.{name}.weight")
                assert lin.scale.cpu().view(torch.uint8).numpy().tobytes() == r.host_bytes(f"layers.{i}.{name}.scale")
            assert len(layer.aux) == (4 if layer.full_attention else 6)
            for name, t in layer.aux.items():
                assert t.cpu().view(torch.uint8).numpy().tobytes() == r.host_bytes(f"layers.{i}.{name}")
                assert tuple(t.shape) == r.find(f"layers.{i}.{name}").dims


@pytest.mark.gpu
def test_a_group_built_from_the_file_matches_the_oracle(v2, orc):
    """Every projection of the model in one grouped launch, weights straight from the file."""
    import torch
    import cudalm_agent_b200 as eng
    from helpers import check_close, from_dev, make_x, to_dev
    with v2.V2Reader(GOLD) as r:
        layers = [r.load_layer(i) for i in range(r.config.num_hidden_layers)]
        items, refs = [], []
        for layer in layers:
            for j, (name, lin) in enumerate(layer.linears.items()):
                x = make_x(orc, (2, lin.K), 31 * layer.layer_idx + j)
                y = torch.zeros((2, lin.N), dtype=torch.bfloat16, device="cuda")
                items.append((lin, to_dev(x, torch.bfloat16), y))
                W = np.frombuffer(r.host_bytes(f"layers.{layer.layer_idx}.{name}.weight"), np.uint8).reshape(lin.N, lin.K // 2)
                S = np.frombuffer(r.host_bytes(f"layers.{layer.layer_idx}.{name}.scale"), np.uint16).reshape(lin.N, lin.K // 128)
                refs.append(orc.batch_gemv_bf16(W, S, x, threads=2))
        assert len(items) == 15
        grp = eng.LinearGroup(items)
        grp.run()
        torch.cuda.synchronize()
        for (lin, _, y), want in zip(items, refs):
            check_close(orc, from_dev(y), want, f"{lin.N}x{lin.K}")
        grp.close()
        assert eng.device_status() == 0


@pytest.mark.gpu
def test_safetensors_conversion_reproduces_the_reference_converters_file(v2, tmp_path):
    """bf16 safetensors -> v2 with the projections quantized on the GPU: the same bytes
    as the reference's converter walk with its CPU quantizer and writer."""
    from safetensors.torch import save_file
    src = tiny_model_tensors()
    st = tmp_path / "model.safetensors"
    save_file({k: v.contiguous() for k, v in src.items()}, str(st))
    out = tmp_path / "converted.cudalm"
    recs = v2.convert_safetensors(str(st), str(out), v2.ModelConfig(**TINY_MODEL), dict(TINY_MODEL_META),
                                  full_model=True, prefix=CHECKPOINT_PREFIX)
    assert len(recs) == 42
    with open(GOLD, "rb") as f:
        assert out.read_bytes() == f.read()
    with v2.V2Reader(str(out)) as r:
        r.validate_full_model()
    # a subset of the layers, as the reference's per-layer conversion writes it
    part = tmp_path / "layer1.cudalm"
    v2.convert_safetensors(str(st), str(part), v2.ModelConfig(**TINY_MODEL), dict(TINY_MODEL_META),
                           layers=[1], prefix=CHECKPOINT_PREFIX)
    with v2.V2Reader(str(part)) as r:
        r.validate_layer(1)
        with pytest.raises(v2.V2FormatError, match="missing tensor"):
            r.validate_layer(0)
