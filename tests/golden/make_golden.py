"""Regenerates tests/golden/*.npz from the CUDALM reference itself.

Run where the reference tree is mounted (it is not present on GPU boxes):

    python tests/golden/make_golden.py [--ref <reference tree>] [--only model]

What is recorded, and which reference code produced it:

* quantize.npz   inputs (bf16 bits) and the outputs of the reference's Python
                 quantizer ``quantize_w4a16`` (tools/common/w4a16_quant.py:25-60),
                 imported from the reference tree and run under torch CPU.
* gemv.npz       inputs and the outputs of the reference's CPU GEMV
                 ``ref_gemv_bf16`` (tests/cuda/test_int4_gemv_bf16.cpp:54-69),
                 called through oracle/_ref/libcudalm_ref.so, which oracle/Makefile
                 compiles from the reference's own sources.
* pick.npz       bf16 logit rows with the reference's ``argmax_bf16``
                 (include/cudalm/greedy.h:28-39) result and the keep-set of its
                 top-k filter (include/cudalm/sampling.h:152-166).

* tiny_model_v2.cudalm  a whole two-layer model converted the way the reference's
                 converter does it (tools/convert_qwen35.py:181-264), written by the
                 reference's container writer (tools/common/cudalm_v2.py).

All inputs are seeded; the files are a few hundred KB in total.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import cpu_oracle as orc  # noqa: E402

BASE_SEED = 20250922


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def f16_bits(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.float16).contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def quant_cases(quantize_w4a16):
    g = torch.Generator().manual_seed(BASE_SEED + 4)
    cases = {}

    def add(name, W):
        W = W.to(torch.bfloat16).contiguous()
        packed, scale16, q, scale32 = quantize_w4a16(W)
        cases[f"{name}.w"] = bf16_bits(W)
        cases[f"{name}.packed"] = packed.numpy().copy()
        cases[f"{name}.scale"] = f16_bits(scale16)

    # the benchmark's distribution: N(0, 0.02)
    add("normal_16x1024", torch.randn(16, 1024, generator=g) * 0.02)
    add("normal_5x256", torch.randn(5, 256, generator=g) * 0.02)
    add("normal_3x3584", torch.randn(3, 3584, generator=g) * 0.02)
    # wide dynamic range between groups
    W = torch.randn(8, 512, generator=g)
    W = W * torch.logspace(-6, 3, 8).view(8, 1)
    add("logrange_8x512", W)
    # an all-zero group, an all-zero row, and a group with a single non-zero
    W = torch.randn(6, 384, generator=g) * 0.02
    W[0, 0:128] = 0
    W[2, :] = 0
    W[4, 128:256] = 0
    W[4, 200] = 0.3
    add("zero_groups_6x384", W)
    # scale underflows fp16 (amax/7 < 2^-25) while the fp32 scale is non-zero:
    # the stored scale is 0 but q keeps its non-zero values
    W = torch.randn(4, 256, generator=g) * 1e-9
    add("fp16_underflow_4x256", W)
    # fp16-subnormal scales
    W = torch.randn(4, 256, generator=g) * 3e-6
    add("fp16_subnormal_4x256", W)
    # exact .5 ties: amax = 7 so the scale is 1 and w = k + 0.5 are ties
    W = torch.zeros(2, 128)
    W[0, :15] = torch.arange(-7, 8).float()
    W[0, 15:29] = torch.arange(-7, 7).float() + 0.5
    W[0, 29] = 7.0
    W[1, :] = torch.linspace(-7, 7, 128)
    add("ties_2x128", W)
    # values large enough that the scale is large; negative extreme only
    W = -torch.rand(3, 128, generator=g) * 1000.0
    add("negative_large_3x128", W)
    # every group the same magnitude element (max|q| must be 7 everywhere)
    W = torch.full((2, 256), 0.0123)
    W[1] = -W[1]
    add("constant_2x256", W)
    return cases


def gemv_cases():
    cases = {}
    rng = np.random.default_rng(BASE_SEED)

    def add(name, W, S, x):
        y = orc.ref_gemv_bf16(W, S, x)
        cases[f"{name}.W"] = W
        cases[f"{name}.S"] = S
        cases[f"{name}.x"] = x
        cases[f"{name}.y"] = y

    def rand_scales(shape):
        return f16_bits(torch.from_numpy(
            (0.001 + 0.02 * rng.random(shape)).astype(np.float32)))

    def rand_x(K, scale=1.0):
        return orc.f32_to_bf16_bits((rng.standard_normal(K) * scale).astype(np.float32))

    # full nibble domain (0x8 = -8 included), positive scales
    for N, K in ((3, 128), (5, 256), (16, 1024), (9, 1024), (8, 2048), (4, 3584)):
        W = rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)
        add(f"random_{N}x{K}", W, rand_scales((N, K // 128)), rand_x(K))
    # all-zero weights and scales -> exact zeros
    add("zero_8x256", np.zeros((8, 128), np.uint8), np.zeros((8, 2), np.uint16),
        rand_x(256))
    # all-zero activations
    W = rng.integers(0, 256, size=(6, 512), dtype=np.uint8)
    add("zero_x_6x1024", W, rand_scales((6, 8)), np.zeros(1024, np.uint16))
    # boundary nibbles with one scale in five set to zero
    nib = np.array([0x7, 0x9, 0x8, 0x0, 0xF, 0x7, 0x8, 0xF], np.uint8)
    lo = nib[rng.integers(0, 8, size=(12, 512))]
    hi = nib[rng.integers(0, 8, size=(12, 512))]
    W = (lo | (hi << 4)).astype(np.uint8)
    S = rand_scales((12, 8))
    S[rng.random((12, 8)) < 0.2] = 0
    add("boundary_12x1024", W, S, rand_x(1024))
    # tiny activations, mixed signs
    W = rng.integers(0, 256, size=(7, 512), dtype=np.uint8)
    add("small_x_7x1024", W, rand_scales((7, 8)), rand_x(1024, 0.005))
    # activation outliers (1% x20), as the batched-decode configuration uses
    x = (rng.standard_normal(1024)).astype(np.float32)
    x[rng.random(1024) < 0.01] *= 20.0
    W = rng.integers(0, 256, size=(10, 512), dtype=np.uint8)
    add("outlier_x_10x1024", W, rand_scales((10, 8)), orc.f32_to_bf16_bits(x))
    return cases


def pick_cases():
    cases = {}
    rng = np.random.default_rng(BASE_SEED + 3)

    def add(name, logits_bits, k):
        cases[f"{name}.logits"] = logits_bits
        cases[f"{name}.argmax"] = np.array([orc.ref_argmax_bf16(logits_bits)], np.int32)
        cases[f"{name}.k"] = np.array([k], np.int32)
        cases[f"{name}.keep"] = orc.ref_topk_keep(logits_bits, k)

    add("normal_4096_k50", orc.f32_to_bf16_bits(
        (rng.standard_normal(4096) * 3).astype(np.float32)), 50)
    # heavy ties: few distinct bf16 values
    add("ties_2048_k50", orc.f32_to_bf16_bits(
        rng.integers(-3, 4, size=2048).astype(np.float32) * 0.5), 50)
    # all equal
    add("flat_300_k50", orc.f32_to_bf16_bits(np.full(300, 1.25, np.float32)), 50)
    # all negative
    add("negative_1000_k7", orc.f32_to_bf16_bits(
        (-np.abs(rng.standard_normal(1000)) - 0.5).astype(np.float32)), 7)
    # k larger than n
    add("short_20_k50", orc.f32_to_bf16_bits(
        rng.standard_normal(20).astype(np.float32)), 50)
    # +0 and -0 compare equal
    z = np.zeros(64, np.float32)
    z[::2] = -0.0
    z[10] = -1.0
    add("signed_zero_64_k5", orc.f32_to_bf16_bits(z), 5)
    # single element
    add("single_1_k1", orc.f32_to_bf16_bits(np.array([-7.5], np.float32)), 1)
    return cases


def sample_cases():
    """The reference's sample_token on full logits: per case the logits, the
    configuration, the SplitMix64 state before, and the tokens and states of
    eight consecutive draws."""
    cases = {}
    rng = np.random.default_rng(BASE_SEED + 6)
    shapes = {
        "normal_4096": (rng.standard_normal(4096) * 3).astype(np.float32),
        "ties_2048": rng.integers(-3, 4, size=2048).astype(np.float32) * 0.5,
        "peaked_1000": np.concatenate([[12.0], rng.standard_normal(999)]).astype(np.float32),
        "flat_300": np.full(300, 1.25, np.float32),
        "vocab_248320": (rng.standard_normal(248320) * 2.5).astype(np.float32),
    }
    configs = [(1.0, 50, 1.0), (0.7, 50, 0.9), (1.5, 20, 0.5), (0.05, 50, 0.95), (1.0, 1, 1.0),
               (0.0, 50, 0.9), (2.0, 50, 0.999), (1e-3, 8, 0.3)]
    for name, vals in shapes.items():
        bits = orc.f32_to_bf16_bits(vals)
        cases[f"{name}.logits"] = bits
        cfgs, toks, states = [], [], []
        for ci, (t, k, p) in enumerate(configs):
            state = (0x1234567 * (ci + 1)) ^ (len(name) << 32)
            row_t, row_s = [], [state]
            for _ in range(8):
                tok, state = orc.ref_sample_token(bits, t, k, p, state)
                row_t.append(tok)
                row_s.append(state)
            cfgs.append((t, k, p))
            toks.append(row_t)
            states.append(row_s)
        cases[f"{name}.configs"] = np.array(cfgs, np.float64)
        cases[f"{name}.tokens"] = np.array(toks, np.int32)
        cases[f"{name}.states"] = np.array(states, np.uint64)
    return cases


def v2_file_case(ref_root, quantize_w4a16):
    """A small `.cudalm` v2 file written by the reference's own Python writer
    (tools/common/cudalm_v2.py), and what it holds."""
    import torch
    sys.path.insert(0, os.path.join(ref_root, "tools", "common"))
    import cudalm_v2 as ref_v2  # the reference's writer

    g = torch.Generator().manual_seed(BASE_SEED + 7)
    w = (torch.randn(16, 256, generator=g) * 0.02).to(torch.bfloat16)
    packed, scale, _, _ = quantize_w4a16(w)
    packed = packed.contiguous().numpy().astype(np.uint8)
    scale = scale.contiguous().view(torch.int16).numpy().astype(np.uint16)
    norm = torch.randn(24, generator=g).to(torch.bfloat16).view(torch.int16).numpy().astype(np.uint16)
    a_log = torch.randn(5, generator=g).numpy().astype(np.float32)
    conv = torch.randn(2, 3, 4, generator=g).to(torch.float16).view(torch.int16).numpy().astype(np.uint16)
    tensors = [
        ref_v2.V2Tensor("layers.0.mlp.gate_proj.weight", ref_v2.DT_INT4_PACKED, packed.shape, packed.tobytes()),
        ref_v2.V2Tensor("layers.0.mlp.gate_proj.scale", ref_v2.DT_FP16_SCALE, scale.shape, scale.tobytes()),
        ref_v2.V2Tensor("layers.0.input_layernorm.weight", ref_v2.DT_BF16, norm.shape, norm.tobytes(), 2),
        ref_v2.V2Tensor("layers.0.linear_attn.A_log", ref_v2.DT_FP32, a_log.shape, a_log.tobytes(), 4),
        ref_v2.V2Tensor("layers.0.linear_attn.conv1d.weight", ref_v2.DT_FP16, conv.shape, conv.tobytes()),
    ]
    meta = {"arch": "qwen3_5", "source_dtype": "bfloat16", "generator": "make_golden.py"}
    obj = ref_v2.V2File(ref_v2.Qwen35Config.qwen35_08b(), meta, tensors)
    raw = obj.to_bytes()
    with open(os.path.join(HERE, "tiny_v2.cudalm"), "wb") as f:
        f.write(raw)
    back = ref_v2.V2File.from_bytes(raw)  # the reference's reader accepts its writer's file
    assert [t.name for t in back.tensors] == [t.name for t in tensors]
    cases = {"config_blob": np.frombuffer(obj.config.to_blob(), np.uint8),
             "meta_keys": np.array(list(meta.keys())), "meta_values": np.array(list(meta.values())),
             "names": np.array([t.name for t in tensors]),
             "dtypes": np.array([t.dtype for t in tensors], np.int32),
             "aligns": np.array([t.align for t in tensors], np.int32),
             "w_bf16": w.view(torch.int16).numpy().astype(np.uint16)}
    for i, t in enumerate(tensors):
        cases[f"dims{i}"] = np.array(t.dims, np.int64)
        cases[f"data{i}"] = np.frombuffer(t.data, np.uint8)
    return cases


def model_v2_file(ref_root, quantize_w4a16):
    """A whole two-layer model (tests/helpers.py: tiny_model_tensors) converted the way
    the reference's converter does it (tools/convert_qwen35.py:181-264: its tensor walk,
    its quantizer, its container writer), for the model-level loader and the
    safetensors conversion to be checked against."""
    import torch
    sys.path.insert(0, os.path.join(ref_root, "tools", "common"))
    sys.path.insert(0, os.path.join(os.path.dirname(HERE)))
    import cudalm_v2 as ref_v2
    from helpers import CHECKPOINT_PREFIX, TINY_MODEL, TINY_MODEL_META, tiny_model_tensors

    conf = ref_v2.Qwen35Config(**TINY_MODEL)
    assert conf.valid()
    src = tiny_model_tensors()
    tensors = []

    def raw(t):
        return t.contiguous().view(torch.uint8).reshape(-1).numpy().tobytes()

    def plain(name, dtype):
        t = src[CHECKPOINT_PREFIX + name]
        tensors.append(ref_v2.V2Tensor(name, dtype, tuple(t.shape), raw(t)))

    def w4(name):
        t = src[CHECKPOINT_PREFIX + name + ".weight"]
        packed, scale16, _q, _s32 = quantize_w4a16(t)
        n, k = t.shape
        tensors.append(ref_v2.V2Tensor(name + ".weight", ref_v2.DT_INT4_PACKED, (n, k // 2), raw(packed)))
        tensors.append(ref_v2.V2Tensor(name + ".scale", ref_v2.DT_FP16_SCALE, (n, k // 128), raw(scale16)))

    for i in range(conf.num_hidden_layers):
        L = f"layers.{i}."
        plain(L + "input_layernorm.weight", ref_v2.DT_BF16)
        if conf.is_full_attention(i):
            for p in ("q_proj", "k_proj", "v_proj", "o_proj"):
                w4(L + "self_attn." + p)
            plain(L + "self_attn.q_norm.weight", ref_v2.DT_BF16)
            plain(L + "self_attn.k_norm.weight", ref_v2.DT_BF16)
        else:
            for p in ("in_proj_qkv", "in_proj_z", "in_proj_b", "in_proj_a", "out_proj"):
                w4(L + "linear_attn." + p)
            plain(L + "linear_attn.conv1d.weight", ref_v2.DT_BF16)
            plain(L + "linear_attn.dt_bias", ref_v2.DT_BF16)
            plain(L + "linear_attn.A_log", ref_v2.DT_FP32)
            plain(L + "linear_attn.norm.weight", ref_v2.DT_FP32)
        plain(L + "post_attention_layernorm.weight", ref_v2.DT_BF16)
        for p in ("gate_proj", "up_proj", "down_proj"):
            w4(L + "mlp." + p)
    plain("norm.weight", ref_v2.DT_BF16)
    plain("embed_tokens.weight", ref_v2.DT_BF16)
    data = ref_v2.V2File(conf, dict(TINY_MODEL_META), tensors).to_bytes()
    ref_v2.V2File.from_bytes(data)  # the reference's reader accepts it
    with open(os.path.join(HERE, "tiny_model_v2.cudalm"), "wb") as f:
        f.write(data)
    return len(data)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("CUDALM_REFERENCE") or
                    os.path.join(os.path.dirname(ROOT), "reference"),
                    help="root of the CUDALM source tree (default: $CUDALM_REFERENCE, else a "
                         "directory 'reference' beside this repository)")
    ap.add_argument("--only", default="all", choices=["all", "model"],
                    help="'model': regenerate only tiny_model_v2.cudalm")
    args = ap.parse_args()
    if not os.path.isdir(os.path.join(args.ref, "tools")):
        raise SystemExit(f"no CUDALM source tree at {args.ref!r}")
    sys.path.insert(0, os.path.join(args.ref, "tools"))
    from common.w4a16_quant import quantize_w4a16  # the reference's quantizer

    if args.only == "model":
        print("tiny_model_v2.cudalm", model_v2_file(args.ref, quantize_w4a16), "bytes")
        return
    orc.build(force=True)
    if not orc.have_ref():
        raise SystemExit("oracle/_ref/libcudalm_ref.so was not built")
    np.savez_compressed(os.path.join(HERE, "quantize.npz"), **quant_cases(quantize_w4a16))
    np.savez_compressed(os.path.join(HERE, "gemv.npz"), **gemv_cases())
    np.savez_compressed(os.path.join(HERE, "pick.npz"), **pick_cases())
    np.savez_compressed(os.path.join(HERE, "sample.npz"), **sample_cases())
    np.savez_compressed(os.path.join(HERE, "tiny_v2.npz"), **v2_file_case(args.ref, quantize_w4a16))
    model_v2_file(args.ref, quantize_w4a16)
    for f in ("quantize.npz", "gemv.npz", "pick.npz", "sample.npz", "tiny_v2.npz", "tiny_v2.cudalm",
              "tiny_model_v2.cudalm"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
