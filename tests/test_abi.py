"""The C-ABI library without a GPU: it loads, exports every symbol the header
declares, and rejects bad arguments on the host before touching a device."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from cudalm_agent_b200 import build, load_library
    build.build_library()
    return load_library()


def header_symbols():
    text = open(os.path.join(ROOT, "include", "cudalm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cudalm_b200_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    from cudalm_agent_b200.api import SIGNATURES
    names = header_symbols()
    assert len(names) >= 18
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
        assert n in SIGNATURES, f"{n} has no ctypes signature"
    assert set(SIGNATURES) == set(names)


def test_status_strings(lib):
    for code in range(0, 9):
        assert lib.cudalm_b200_status_string(code)
    assert lib.cudalm_b200_status_string(0) == b"ok"
    assert b"sm_100a" in lib.cudalm_b200_build_info()


def test_host_side_rejections(lib):
    # CUDALM aborts on these (src/kernels/int4_gemv_bf16.cu:224-226,
    # src/kernels/batch_decode.cu:650-653); the ABI returns a status instead.
    p = ctypes.c_void_p(4096)
    f = lib.cudalm_b200_int4_gemv_bf16
    assert f(None, p, p, p, 16, 128, None) == 2
    assert f(p, p, p, None, 16, 128, None) == 2
    assert f(p, p, p, p, 0, 128, None) == 1
    assert f(p, p, p, p, 16, 0, None) == 1
    assert f(p, p, p, p, 16, 192, None) == 1
    b = lib.cudalm_b200_batch_int4_gemv_bf16
    assert b(p, p, p, p, 16, 128, 0, None) == 1
    q = lib.cudalm_b200_quantize_w4a16
    assert q(None, 4, 128, p, p, None) == 2
    assert q(p, 4, 100, p, p, None) == 1
    assert q(ctypes.c_void_p(4098), 4, 128, p, p, None) == 3
    g = lib.cudalm_b200_gate_up_bf16
    assert g(p, p, p, p, p, p, p, 16, 128, 0, None) == 1
    lm = lib.cudalm_b200_lm_head_topk
    assert lm(p, p, p, 100, 128, 1, 65, 0, None, p, p, p, p, 1 << 30, None) == 7
    assert lm(p, p, p, 100, 128, 1, 50, 0, None, p, p, p, None, 0, None) == 8
    assert lm(p, p, p, 100, 128, 1, 50, 0, None, p, p, p, p, 16, None) == 8
    mg = lib.cudalm_b200_topk_merge
    assert mg(p, p, 64, 1, 64, p, p, p, None) == 7
    assert lib.cudalm_b200_linear_multi(None, 1, None) == 2
    assert lib.cudalm_b200_group_run(None, None) == 2
    assert lib.cudalm_b200_kernel_regs(b"no_such_kernel") == -1


def test_workspace_size_formula(lib):
    f = lib.cudalm_b200_lm_head_workspace_bytes
    small = f(1000, 1024, 1, 50, 0)
    with_logits = f(1000, 1024, 1, 50, 1)
    assert with_logits - small >= 2000 and small > 0
    assert f(248320, 1024, 32, 50, 1) >= 32 * 248320 * 2
    # rows beyond one pass reuse the same workspace
    assert f(1000, 1024, 64, 50, 1) == f(1000, 1024, 32, 50, 1)


def test_python_layer_refuses_cpu_tensors():
    import torch
    from cudalm_agent_b200 import int4_gemv_bf16, quantize_w4a16
    with pytest.raises(ValueError):
        int4_gemv_bf16(torch.zeros(4, 64, dtype=torch.uint8), torch.zeros(4, 1, dtype=torch.float16),
                       torch.zeros(128, dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        quantize_w4a16(torch.zeros(4, 128, dtype=torch.bfloat16))


def test_shard_rows_cover_the_vocabulary():
    from cudalm_agent_b200 import shard_rows
    for vocab in (248320, 1000, 31, 16):
        for world in (1, 2, 4, 8):
            prev = 0
            for r in range(world):
                lo, hi = shard_rows(vocab, world, r)
                assert lo == prev and lo <= hi
                assert lo % 16 == 0
                prev = hi
            assert prev == vocab
    assert shard_rows(248320, 8, 3) == (93120, 124160)
