"""Seeded random shapes through every entry point that projects: each result against the
CPU oracle under the same gate as the fixed-shape tests, the fused forms against the
unfused sequence of this library bit for bit, and twice the same bits on two runs.
The shapes are drawn so that every kernel is met: the lean kernel (few rows, few bytes),
the streaming kernel, the tensor-memory kernel with and without a split K, the one-warp
fallback (K > 4096 or a weight base off 16 bytes)."""
import numpy as np
import pytest

from helpers import check_close, from_dev, make_x, raw_weights, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng():
    import torch
    import cudalm_agent_b200 as eng
    assert torch.cuda.is_available()
    eng.load_library()
    yield eng
    assert eng.device_status() == 0, "a device-side wait ran out during the tests"

KINDS = ["random", "boundary", "small"]
XKINDS = ["normal", "outlier", "uniform", "rmsnorm"]


def _cases(n, seed):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(n):
        N = int(rng.choice([rng.integers(1, 64), rng.integers(64, 1200), rng.integers(1200, 6200)]))
        K = 128 * int(rng.choice([rng.integers(1, 9), rng.integers(9, 33), rng.integers(33, 41)]))
        M = int(rng.choice([1, rng.integers(2, 9), rng.integers(9, 17), rng.integers(17, 65)]))
        out.append((N, K, M, KINDS[i % 3], XKINDS[i % 4], int(rng.integers(0, 2))))
    return out


@pytest.mark.parametrize("N,K,M,kind,xkind,offset", _cases(36, 77))
def test_random_projection(eng, orc, N, K, M, kind, xkind, offset):
    import torch
    W, S = raw_weights(N, K, 9000 + N + K + M, kind)
    x = make_x(orc, (M, K), 9001 + N + M, xkind)
    want = orc.batch_gemv_bf16(W, S, x, threads=8)
    dS, dx = to_dev(S, torch.float16), to_dev(x, torch.bfloat16)
    if offset:
        # a weight base one byte off any alignment: the slow kernel's domain
        raw = torch.empty(W.size + 16, dtype=torch.uint8, device="cuda")
        dW = raw[1:1 + W.size].view(N, K // 2)
        dW.copy_(to_dev(W))
    else:
        dW = to_dev(W)
    got = eng.batch_int4_gemv_bf16(dW, dS, dx) if M > 1 else eng.int4_gemv_bf16(dW, dS, dx[0]).view(1, N)
    torch.cuda.synchronize()
    a = from_dev(got)
    check_close(orc, a, want, f"{N}x{K} M={M} {kind}/{xkind} off={offset}")
    again = eng.batch_int4_gemv_bf16(dW, dS, dx) if M > 1 else eng.int4_gemv_bf16(dW, dS, dx[0]).view(1, N)
    torch.cuda.synchronize()
    assert np.array_equal(a, from_dev(again)), "two runs differ"
    if offset:
        return
    lin = eng.W4A16Linear(dW, dS)
    res = make_x(orc, (M, N), 9002 + N, "normal")
    out = eng.linear_residual_bf16(lin, dx if M > 1 else dx[0], to_dev(res if M > 1 else res[0], torch.bfloat16))
    torch.cuda.synchronize()
    # The residual form may run on another kernel than the plain call (it wants N a multiple
    # of 8 on the tensor-memory kernel), i.e. another summation order: its projection may
    # then sit one bf16 step from the plain one on a few values, never more.
    r = from_dev(out).reshape(M, N)
    alt = [orc.add_bf16(res, (a.astype(np.int32) + d).astype(np.uint16)) for d in (0, 1, -1)]
    ok = (r == alt[0]) | (r == alt[1]) | (r == alt[2])
    assert ok.all(), f"residual form: {(~ok).sum()} values are not res + projection within one step"
    assert (r != alt[0]).mean() <= 0.01, f"residual form differs on {(r != alt[0]).sum()} of {r.size}"
    W2, S2 = raw_weights(N, K, 9003 + N + K, kind)
    up = eng.W4A16Linear(to_dev(W2), to_dev(S2, torch.float16))
    b = from_dev(eng.batch_int4_gemv_bf16(up.weight, up.scale, dx) if M > 1
                 else eng.int4_gemv_bf16(up.weight, up.scale, dx[0]).view(1, N))
    fused = eng.gate_up_silu_bf16(lin, up, dx if M > 1 else dx[0])
    torch.cuda.synchronize()
    want_f = orc.silu_mul_bf16(a, b)
    f = from_dev(fused).reshape(M, N)
    # the device's expf may differ from the host's by one bf16 step of silu on a few values
    diff = f != want_f
    assert diff.mean() <= 0.005, f"fused gate/up differs on {diff.sum()} of {diff.size}"
    assert eng.device_status() == 0


def _pick_cases(n, seed):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(n):
        N = int(rng.choice([rng.integers(8, 200), rng.integers(200, 5000), rng.integers(5000, 60000)]))
        K = 128 * int(rng.integers(1, 17))
        M = int(rng.choice([1, rng.integers(2, 9), rng.integers(9, 17), rng.integers(17, 41)]))
        k = int(rng.choice([1, 8, 50, 64]))
        out.append((N, K, M, k, i % 3 == 0))
    return out


@pytest.mark.parametrize("N,K,M,k,ties", _pick_cases(18, 78))
def test_random_vocabulary_pick(eng, orc, N, K, M, k, ties):
    """The token pick on random vocabularies: argmax and top-k follow the reference's
    ordering rule on the device's logits (lists padded with -1 past the vocabulary), with
    heavy ties (few distinct weight rows) in every third case, with and without a logits
    buffer, and on consecutive calls (the workspace must come back clean)."""
    import torch
    W, S = raw_weights(N, K, 9100 + N + K, "small" if ties else "random")
    if ties:
        W[:] = W[np.arange(N) % 7]
        S[:] = S[np.arange(N) % 7]
    x = make_x(orc, (M, K), 9101 + M, "rmsnorm")
    lin = eng.W4A16Linear(to_dev(W), to_dev(S, torch.float16))
    dx = to_dev(x, torch.bfloat16)
    head = eng.LmHead(lin, top_k=k, id_offset=17, max_rows=max(M, 1), keep_logits=True)
    bare = eng.LmHead(lin, top_k=k, id_offset=17, max_rows=max(M, 1))
    for _ in range(2):
        argmax, idx, val = head.forward(dx)
        a2, i2, v2 = bare.forward(dx)
        torch.cuda.synchronize()
        logits = from_dev(head.logits[:M])
        check_close(orc, logits, orc.batch_gemv_bf16(W, S, x, threads=8), f"logits {N}x{K} M={M}")
        gi, gv, ga = from_dev(idx), from_dev(val), from_dev(argmax)
        for m in range(M):
            wi, wv = orc.topk_bf16(logits[m], k)
            n = len(wi)
            assert np.array_equal(gi[m][:n] - 17, wi), (N, K, M, k, m)
            assert np.array_equal(gv[m][:n], wv), (N, K, M, k, m)
            assert np.all(gi[m][n:] == -1)
            assert int(ga[m]) - 17 == orc.argmax_bf16(logits[m])
        assert np.array_equal(from_dev(i2), gi) and np.array_equal(from_dev(v2), gv)
        assert np.array_equal(from_dev(a2), ga)
    assert eng.device_status() == 0
