"""GPU numerics beyond the parity gate: accuracy against an exact (fp64) sum,
the activation range the kernels accept, and the reference's full cross of input
classes, shapes, seeds and batch widths
(CUDALM tests/cuda/test_w4a16_qwen35_optimized.cpp:76-171,456-480).
"""
import numpy as np
import pytest

from helpers import BASE_SEED, _ordinal, check_close, from_dev, make_x, raw_weights, to_dev

pytestmark = pytest.mark.gpu

CENSUS = [(16, 1024), (512, 1024), (1024, 2048), (1024, 3584), (2048, 1024), (3584, 1024),
          (4096, 1024), (6144, 1024)]
EDGE = [(1, 128), (3, 128), (5, 256), (9, 1024), (15, 1024), (1023, 1024)]


@pytest.fixture(scope="module")
def eng():
    import torch
    import cudalm_agent_b200 as eng
    assert torch.cuda.is_available()
    eng.load_library()
    yield eng
    assert eng.device_status() == 0, "a device-side wait ran out during the tests"


class _Path:
    """Forces one of the kernels for calls of any size."""

    def __init__(self, eng, name):
        self.eng, self.name = eng, name

    def __enter__(self):
        e = self.eng
        self.prev_direct = e.set_direct_path_max_bytes(1 << 40 if self.name == "lean" else 0)
        self.prev_rows = e.set_tensor_path_min_rows(1 if self.name == "tensor" else 1 << 30)
        return self

    def __exit__(self, *exc):
        self.eng.set_direct_path_max_bytes(self.prev_direct)
        self.eng.set_tensor_path_min_rows(self.prev_rows)


def _run(eng, W, S, x, misalign_weight=False):
    import torch
    Wd = to_dev(W)
    if misalign_weight:  # a weight base off 16 bytes takes the one-warp-per-row kernel
        buf = torch.empty(W.size + 1, dtype=torch.uint8, device="cuda")
        Wd = buf[1:].view(W.shape)
        Wd.copy_(to_dev(W))
    xd = to_dev(x, torch.bfloat16)
    if x.ndim == 1:
        y = eng.int4_gemv_bf16(Wd, to_dev(S, torch.float16), xd)
    else:
        y = eng.batch_int4_gemv_bf16(Wd, to_dev(S, torch.float16), xd)
    torch.cuda.synchronize()
    return from_dev(y)


def _exact(orc, W, S, x):
    """The sums in double precision (products are exact in it) and the sum of the
    terms' magnitudes, per output."""
    q = orc.unpack_int4(W).astype(np.float64)
    N, K = q.shape
    s = S.view(np.float16).astype(np.float64)
    xs = orc.bf16_bits_to_f32(x).astype(np.float64).reshape(-1, K)
    out = np.empty((xs.shape[0], N))
    mag = np.empty_like(out)
    for m in range(xs.shape[0]):
        t = q.reshape(N, K // 128, 128) * xs[m].reshape(K // 128, 128)
        out[m] = (t.sum(-1) * s).sum(-1)
        mag[m] = (np.abs(t).sum(-1) * np.abs(s)).sum(-1)
    return out, mag


def _bf16_ulp(v):
    a = np.maximum(np.abs(v), 2.0 ** -126)
    return 2.0 ** (np.floor(np.log2(a)) - 7)


@pytest.mark.parametrize("path,M", [("lean", 1), ("streaming", 1), ("slow", 1), ("lean", 8),
                                    ("streaming", 8), ("streaming", 16), ("tensor", 32)])
def test_no_less_accurate_than_the_cpu_reference(eng, orc, path, M):
    """|gpu - exact| <= |cpu_ref - exact| + 1/2 bf16 ulp, element by element, where
    exact is the double-precision sum; a few fp32 roundings of the terms' magnitude
    are allowed on top, which only matters for outputs that cancel to almost zero
    (there both fp32 sums are noise and neither is the better one)."""
    for N, K in CENSUS:
        W, S = raw_weights(N, K, BASE_SEED + 11 * N + K)
        x = make_x(orc, (M, K) if M > 1 else (K,), BASE_SEED + N + M, "normal")
        with _Path(eng, path):
            got = _run(eng, W, S, x, misalign_weight=(path == "slow"))
        cpu = orc.batch_gemv_bf16(W, S, x.reshape(-1, K), threads=8)
        exact, mag = _exact(orc, W, S, x)
        e_gpu = np.abs(orc.bf16_bits_to_f32(got).astype(np.float64).reshape(exact.shape) - exact)
        e_cpu = np.abs(orc.bf16_bits_to_f32(cpu).astype(np.float64).reshape(exact.shape) - exact)
        allow = e_cpu + 0.5 * _bf16_ulp(exact) + 8 * 2.0 ** -24 * mag
        worst = (e_gpu - allow).max()
        assert worst <= 0, f"{path} M={M} {N}x{K}: {np.count_nonzero(e_gpu > allow)} outputs, worst excess {worst:.3g}"
        # and on the whole the GPU's sums are at least as close to exact as the CPU's serial ones
        assert e_gpu.mean() <= e_cpu.mean() * 1.02 + 1e-12, (path, N, K, e_gpu.mean(), e_cpu.mean())


def _class_fixture(orc, N, K, B, kind, seed):
    """Weights, scales and activations of one input class of the reference's test."""
    wkind = {"random": "random", "zero": "zero", "small": "small", "mixedsign": "random",
             "boundary": "boundary"}[kind]
    xkind = {"random": "normal", "zero": "zero", "small": "small", "mixedsign": "normal",
             "boundary": "normal"}[kind]
    W, S = raw_weights(N, K, seed, wkind)
    x = make_x(orc, (B, K), seed ^ 0x5bd1e995, xkind)
    return W, S, x


@pytest.mark.parametrize("path", ["lean", "streaming", "tensor"])
def test_input_class_cross(eng, orc, path):
    """Every shape x seed x input class x batch width B = 1, 2, 3 of the reference's
    kernel test, on each kernel that takes such calls."""
    seeds = (0x51ed, 0x1234abcd, 0x9e3779b9, 0xcafebabe) if path != "tensor" else (0x51ed, 0xcafebabe)
    for N, K in CENSUS + EDGE:
        for seed in seeds:
            for kind in ("random", "zero", "small", "mixedsign", "boundary"):
                for B in (1, 2, 3):
                    W, S, x = _class_fixture(orc, N, K, B, kind, (seed + 131 * N + K) & 0x7fffffff)
                    with _Path(eng, path):
                        got = _run(eng, W, S, x if B > 1 else x[0]).reshape(B, N)
                    want = orc.batch_gemv_bf16(W, S, x, threads=8)
                    for b in range(B):
                        check_close(orc, got[b], want[b], f"{path} {kind} {N}x{K} B={B} row {b}")
                    if kind == "zero":
                        assert np.all((got & 0x7FFF) == 0)
                    if kind == "boundary":
                        # outputs of rows whose groups all have scale 0 are exact zeros
                        dead = ~S.view(np.float16).astype(bool).any(axis=1)
                        assert np.all((got[:, dead] & 0x7FFF) == 0)


def _same_class(orc, got_bits, want_bits, label):
    """Non-finite outputs must agree in kind (NaN, +inf, -inf); finite ones meet the
    benchmark's gate max|err| <= 1e-2 * RMS (or are the neighbouring bf16 value).  The
    reference's absolute tolerance of 1e-2 presumes outputs of order one and is left
    out here, where the outputs are of order 2^60 or 2^-60."""
    gb, wb = np.asarray(got_bits, np.uint16).ravel(), np.asarray(want_bits, np.uint16).ravel()
    g = orc.bf16_bits_to_f32(gb).astype(np.float64)
    w = orc.bf16_bits_to_f32(wb).astype(np.float64)
    assert np.array_equal(np.isnan(g), np.isnan(w)), label
    assert np.array_equal(np.isposinf(g), np.isposinf(w)), label
    assert np.array_equal(np.isneginf(g), np.isneginf(w)), label
    fin = np.isfinite(w)
    if not fin.any():
        return
    rms = np.sqrt(np.mean(w[fin] * w[fin]))
    over = np.abs(g[fin] - w[fin]) > 1e-2 * rms
    neighbours = np.abs(_ordinal(gb[fin]) - _ordinal(wb[fin])) <= 1
    assert not (over & ~neighbours).any(), label
    assert over.mean() <= 5e-3, label


@pytest.mark.parametrize("path", ["lean", "streaming", "tensor", "slow"])
def test_activation_range(eng, orc, path):
    """Legal inputs are never rejected (CUDALM include/cudalm/kernels/int4_gemv_bf16.h:40-45):
    activations of any magnitude a bf16 holds, infinities and NaNs give what the CPU
    reference gives."""
    rng = np.random.default_rng(4242)
    M = 3 if path != "slow" else 1
    for N, K in ((512, 1024), (1024, 3584), (37, 256)):
        W, S = raw_weights(N, K, 606 + N)
        base = rng.standard_normal((M, K)).astype(np.float32)
        cases = {
            "huge": base * np.float32(2.0 ** 62),
            "huger": base * np.float32(2.0 ** 100),
            "tiny": base * np.float32(2.0 ** -56),
            "tinier": base * np.float32(2.0 ** -100),
            "mixed magnitudes": base * (2.0 ** rng.integers(-40, 40, size=(M, K))).astype(np.float32),
        }
        one_inf = base.copy()
        one_inf[:, 5] = np.inf
        one_nan = base.copy()
        one_nan[0, 77] = np.nan
        cases["one +inf"] = one_inf
        cases["one nan"] = one_nan
        for name, xf in cases.items():
            x = orc.f32_to_bf16_bits(xf)
            with _Path(eng, path):
                got = _run(eng, W, S, x if M > 1 else x[0], misalign_weight=(path == "slow"))
            want = orc.batch_gemv_bf16(W, S, x, threads=4)
            _same_class(orc, got.reshape(M, N), want, f"{path} {name} {N}x{K}")
