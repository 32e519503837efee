"""Pins the CPU oracle to the reference.

Every oracle function is compared with golden vectors that the reference's own
code produced (tests/golden/make_golden.py records which code made which file),
with the known-answer rules the reference's tests state, and -- where the
reference bridge oracle/_ref is built -- with the reference functions directly.
"""
import numpy as np
import pytest


def test_quantize_matches_reference_quantizer(orc, golden):
    # reference tools/common/w4a16_quant.py:25-60 (outputs recorded in quantize.npz)
    g = golden.quantize
    for name in golden.names(g):
        packed, scale = orc.quantize_w4a16(g[f"{name}.w"])
        assert np.array_equal(packed, g[f"{name}.packed"]), name
        assert np.array_equal(scale, g[f"{name}.scale"]), name


def test_quantize_threads_do_not_change_bits(orc, golden):
    w = golden.quantize["normal_16x1024.w"]
    a = orc.quantize_w4a16(w, threads=1)
    b = orc.quantize_w4a16(w, threads=4)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


def test_quantize_invariants(orc, golden):
    # reference tests/cpu/test_weights_crosslang.cpp:79-107: q in [-7,7];
    # scale > 0 => max|q| == 7; scale32 == 0 => q == 0.
    # reference tools/verify_qwen35_ingestion.py:160-190: stored scale == fp16(amax/7).
    g = golden.quantize
    for name in golden.names(g):
        w = orc.bf16_bits_to_f32(g[f"{name}.w"])
        packed, scale = orc.quantize_w4a16(g[f"{name}.w"])
        q = orc.unpack_int4(packed).astype(np.int32)
        N, K = w.shape
        assert q.min() >= -7 and q.max() <= 7
        qmax = np.abs(q).reshape(N, K // 128, 128).max(axis=2)
        amax = np.abs(w).reshape(N, K // 128, 128).max(axis=2)
        scale32 = (amax / np.float32(7)).astype(np.float32)
        assert np.array_equal(scale32.astype(np.float16).view(np.uint16), scale), name
        assert np.all(qmax[scale32 > 0] == 7), name
        assert np.all(qmax[scale32 == 0] == 0), name
        # reference tools/convert_qwen35.py:311-320: |deq - w| <= 0.51 * scale32
        deq = q.reshape(N, K // 128, 128) * scale32[:, :, None]
        err = np.abs(deq - w.reshape(N, K // 128, 128))
        assert np.all(err <= 0.51 * scale32[:, :, None] + 1e-30), name


def test_fp16_underflow_keeps_nonzero_q(orc, golden):
    # reference tools/verify_qwen35_ingestion.py:243-260: the zero test is on the
    # fp32 scale, so a group whose scale underflows fp16 stores 0 but keeps q.
    g = golden.quantize
    packed, scale = orc.quantize_w4a16(g["fp16_underflow_4x256.w"])
    assert np.all(scale == 0)
    assert np.abs(orc.unpack_int4(packed)).max() == 7


def test_pack_unpack_full_domain(orc):
    # reference tests/cpu/test_weight_file.cpp:212-224
    L = orc.lib()
    for lo in range(-8, 8):
        for hi in range(-8, 8):
            b = L.orc_pack_byte(lo, hi)
            assert L.orc_unpack_lo(b) == lo and L.orc_unpack_hi(b) == hi
    if orc.have_ref():
        R = orc.ref()
        for b in range(256):
            assert R.ref_cpu_unpack_lo(b) == L.orc_unpack_lo(b)
            assert R.ref_cpu_unpack_hi(b) == L.orc_unpack_hi(b)


def test_gemv_matches_reference_cpu_gemv_bitwise(orc, golden):
    # reference tests/cuda/test_int4_gemv_bf16.cpp:54-69 (outputs in gemv.npz)
    g = golden.gemv
    for name in golden.names(g):
        y = orc.gemv_bf16(g[f"{name}.W"], g[f"{name}.S"], g[f"{name}.x"])
        assert np.array_equal(y, g[f"{name}.y"]), name


def test_gemv_zero_group_is_exact_zero(orc, golden):
    # reference tests/cuda/test_int4_gemv_bf16.cpp:146-176
    g = golden.gemv
    y = orc.gemv_bf16(g["zero_8x256.W"], g["zero_8x256.S"], g["zero_8x256.x"])
    assert np.all(y == 0)


def test_batch_rows_equal_single_calls(orc, golden):
    # reference include/cudalm/kernels/batch_decode.h:50-63: per row identical
    g = golden.gemv
    W, S = g["random_16x1024.W"], g["random_16x1024.S"]
    rng = np.random.default_rng(7)
    x = orc.f32_to_bf16_bits(rng.standard_normal((5, 1024)).astype(np.float32))
    for threads in (1, 3):
        y = orc.batch_gemv_bf16(W, S, x, threads=threads)
        for b in range(5):
            assert np.array_equal(y[b], orc.gemv_bf16(W, S, x[b]))


def test_gemv_against_live_reference(orc):
    if not orc.have_ref():
        pytest.skip("oracle/_ref not built here")
    rng = np.random.default_rng(11)
    for N, K in ((33, 1024), (4, 3584), (17, 128)):
        W = rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)
        S = (0.001 + 0.02 * rng.random((N, K // 128))).astype(np.float16).view(np.uint16)
        x = orc.f32_to_bf16_bits(rng.standard_normal(K).astype(np.float32))
        assert np.array_equal(orc.gemv_bf16(W, S, x), orc.ref_gemv_bf16(W, S, x))


def _bf(xs):
    from oracle import cpu_oracle
    return cpu_oracle.f32_to_bf16_bits(np.array(xs, np.float32))


def test_argmax_known_answers(orc):
    # the cases of reference tests/cpu/test_greedy_argmax.cpp:28-71
    assert orc.argmax_bf16(_bf([1.0, 5.0, 3.0, 2.0, -100.0])) == 1
    assert orc.argmax_bf16(_bf([-5.0, -1.0, -3.0, -2.0, -9.0])) == 1
    assert orc.argmax_bf16(_bf([3.0, 1.0, 2.0, 3.0, 3.0])) == 0
    assert orc.argmax_bf16(_bf([1.0, 0.5, 2.5, 2.5, -1.0])) == 2
    assert orc.argmax_bf16(_bf([-7.5])) == 0
    two = _bf([0.1 + 1e-7, 0.1])
    assert two[0] == two[1]
    assert orc.argmax_bf16(two) == 0


def test_topk_known_answers(orc):
    # reference tests/cpu/test_sampling.cpp:120-160 and :437-490
    idx, _ = orc.topk_bf16(_bf([5.0, 4.0, 3.0, 2.0, 1.0]), 2)
    assert list(idx) == [0, 1]
    idx, _ = orc.topk_bf16(_bf([3.0, 3.0, 2.0]), 1)
    assert list(idx) == [0]
    idx, _ = orc.topk_bf16(_bf([5.0, 4.0, 3.0, 2.0, 1.0]), 1000)
    assert list(idx) == [0, 1, 2, 3, 4]
    idx, _ = orc.topk_bf16(_bf([5.0, 5.0, 5.0, 5.0]), 1)
    assert list(idx) == [0]
    idx, _ = orc.topk_bf16(_bf([-1.5, 3.25, -0.25, 3.25, -4.0]), 1)
    assert list(idx) == [1]
    idx, _ = orc.topk_bf16(_bf([2.0, 2.0, 1.0, 1.0]), 3)
    assert list(idx) == [0, 1, 2]


def test_pick_matches_reference(orc, golden):
    # reference include/cudalm/greedy.h:28-39, include/cudalm/sampling.h:152-166
    g = golden.pick
    for name in golden.names(g):
        logits = g[f"{name}.logits"]
        k = int(g[f"{name}.k"][0])
        assert orc.argmax_bf16(logits) == int(g[f"{name}.argmax"][0]), name
        idx, val = orc.topk_bf16(logits, k)
        keep = np.zeros(logits.size, bool)
        keep[idx] = True
        assert np.array_equal(keep, g[f"{name}.keep"]), name
        assert idx[0] == int(g[f"{name}.argmax"][0]), name
        # order: value descending, ties by ascending id
        v = orc.bf16_bits_to_f32(val)
        for a in range(len(idx) - 1):
            assert v[a] > v[a + 1] or (v[a] == v[a + 1] and idx[a] < idx[a + 1]), name
        assert np.array_equal(val, logits[idx])


def sample_case_names(golden):
    return sorted({k.split(".")[0] for k in golden.sample.files})


def test_sampling_on_candidate_list_matches_reference_sample_token(orc, golden):
    # the reference's sample_token on FULL logits (recorded by make_golden.py) against the
    # oracle's restatement on the top-50 candidate list: tokens and RNG states, eight
    # consecutive draws per configuration (CUDALM include/cudalm/sampling.h:131-234)
    for name in sample_case_names(golden):
        logits = golden.sample[f"{name}.logits"]
        idx, val = orc.topk_bf16(logits, 50)
        for (t, k, p), toks, states in zip(golden.sample[f"{name}.configs"],
                                           golden.sample[f"{name}.tokens"],
                                           golden.sample[f"{name}.states"]):
            state = int(states[0])
            for j in range(8):
                tok, state = orc.sample_from_topk(idx, val, float(np.float32(t)), int(k),
                                                  float(np.float32(p)), state)
                assert tok == int(toks[j]), (name, t, k, p, j)
                assert state == int(states[j + 1]), (name, t, k, p, j)


def test_sampling_rejects_what_a_candidate_list_cannot_answer(orc):
    idx = np.arange(10, dtype=np.int32)
    val = orc.f32_to_bf16_bits(np.linspace(2, 1, 10).astype(np.float32))
    assert orc.sample_from_topk(idx, val, 1.0, 0, 1.0, 1)[0] == -1    # top-k disabled: whole vocabulary
    assert orc.sample_from_topk(idx, val, 1.0, 11, 1.0, 1)[0] == -1   # more than the list holds
    tok, state = orc.sample_from_topk(idx, val, 0.0, 5, 0.5, 77)      # greedy: entry 0, no draw
    assert (tok, state) == (0, 77)


def test_silu_mul_and_add_rounding_order(orc):
    # reference src/kernels/qwen35_kernels.cu:442-476: silu is rounded to bf16
    # first, then multiplied; add rounds once.
    rng = np.random.default_rng(5)
    g = rng.standard_normal(4096).astype(np.float32) * 4
    u = rng.standard_normal(4096).astype(np.float32)
    gb, ub = orc.f32_to_bf16_bits(g), orc.f32_to_bf16_bits(u)
    gf, uf = orc.bf16_bits_to_f32(gb), orc.bf16_bits_to_f32(ub)
    s = orc.bf16_bits_to_f32(orc.f32_to_bf16_bits(
        (gf / (np.float32(1) + np.exp(-gf, dtype=np.float32))).astype(np.float32)))
    want = orc.f32_to_bf16_bits((s * uf).astype(np.float32))
    got = orc.silu_mul_bf16(gb, ub)
    # expf differs from numpy's exp by at most an ulp, which can flip a bf16
    # rounding only rarely; demand near-total agreement and 1-ulp otherwise
    diff = np.abs(got.astype(np.int32) - want.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 0.01
    assert np.array_equal(orc.add_bf16(gb, ub),
                          orc.f32_to_bf16_bits((gf + uf).astype(np.float32)))


def test_scalar_conversions_match_numpy(orc):
    L = orc.lib()
    rng = np.random.default_rng(3)
    vals = np.concatenate([
        rng.standard_normal(2000).astype(np.float32) * 10.0 ** rng.integers(-9, 5, 2000),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 2.0 ** -25, 2.0 ** -24,
                  6.1e-5, 5.97e-8, 3e-8], np.float32)]).astype(np.float32)
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = np.array([L.orc_f32_to_f16(float(v)) for v in vals], np.uint16)
    assert np.array_equal(got, want)
    allh = np.arange(0, 0x7C00, 37, dtype=np.uint16)
    back = np.array([L.orc_f16_to_f32(int(h)) for h in allh], np.float32)
    assert np.array_equal(back, allh.view(np.float16).astype(np.float32))
    b = np.array([L.orc_f32_to_bf16(float(v)) for v in vals], np.uint16)
    assert np.array_equal(b, orc.f32_to_bf16_bits(vals))
