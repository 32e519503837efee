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


@pytest.mark.parametrize("seed", range(8))
def test_random_group(eng, orc, seed):
    """Grouped launches over random sets of projections (2 to 60 of them, K from 128 to
    4096, rows 1 to 64 per projection, the same or different row counts inside a group):
    every output against the oracle, the same bits on a second run, and against the
    projection's own call on the same kernel class (lean kernel off, so that a single call
    of up to 16 rows streams as the group does): the same bits when the group's row counts
    are equal, within one bf16 step on at most one value in a thousand otherwise."""
    import torch
    rng = np.random.default_rng(500 + seed)
    count = int(rng.integers(2, 61))
    big_m = seed % 4 == 3          # every fourth group: the tensor-memory kernel
    same_m = seed % 2 == 0
    m_all = int(rng.integers(17, 65)) if big_m else int(rng.integers(1, 17))
    items, refs, raws = [], [], []
    for i in range(count):
        N = int(rng.choice([rng.integers(1, 40), rng.integers(40, 900), rng.integers(900, 4200)]))
        K = 128 * int(rng.choice([rng.integers(1, 9), rng.integers(9, 33)]))
        M = m_all if same_m else (int(rng.integers(17, 65)) if big_m else int(rng.integers(1, 17)))
        W, S = raw_weights(N, K, 9200 + 100 * seed + i, KINDS[i % 3])
        x = make_x(orc, (M, K), 9300 + 100 * seed + i, XKINDS[i % 4])
        lin = eng.W4A16Linear(to_dev(W), to_dev(S, torch.float16))
        y = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
        items.append((lin, to_dev(x, torch.bfloat16), y))
        refs.append(orc.batch_gemv_bf16(W, S, x, threads=8))
        raws.append((W, S, x))
    grp = eng.LinearGroup(items)
    grp.run()
    torch.cuda.synchronize()
    first = [from_dev(y) for _, _, y in items]
    for i, (got, want) in enumerate(zip(first, refs)):
        check_close(orc, got, want, f"group {seed} item {i} {items[i][0].N}x{items[i][0].K} M={items[i][1].shape[0]}")
    grp.run()
    torch.cuda.synchronize()
    for a, (_, _, y) in zip(first, items):
        assert np.array_equal(a, from_dev(y)), "second run differs"
    prev = eng.set_direct_path_max_bytes(0)
    try:
        for i in range(0, count, max(1, count // 6)):
            lin, dx, _ = items[i]
            single = eng.batch_int4_gemv_bf16(lin.weight, lin.scale, dx)
            torch.cuda.synchronize()
            # (a projection whose K the tensor-memory kernel splits when it is launched
            # alone sums in another order than inside a launch with many tiles)
            if not big_m:
                # A group that no single launch takes (its longest K with its largest row
                # count does not fit the rings) runs its projections one by one, where the
                # small ones take the lean kernel, whose sums are grouped otherwise:
                # measured, one or two values in 10,000 then sit on the neighbouring bf16
                # value.  Never more.  (Row counts alone change nothing: 1, 3, 8, 9 and 16
                # rows of one projection give the same bits row for row.)
                sg = from_dev(single)
                d = np.abs(sg.astype(np.int32) - first[i].astype(np.int32))
                assert d.max() <= 1 and (d > 0).mean() <= 1e-3, \
                    f"item {i} differs from its own call: {(d > 0).sum()} of {d.size}, max step {d.max()}"
                if same_m:
                    assert d.max() == 0, f"item {i}: equal row counts, yet other bits than its own call"
            else:
                check_close(orc, from_dev(single), first[i], f"item {i} against its own call")
    finally:
        eng.set_direct_path_max_bytes(prev)
    grp.close()
    assert eng.device_status() == 0


@pytest.mark.parametrize("N,K", [(4015, 1024), (3546, 2048), (100, 384)])
def test_a_row_does_not_depend_on_its_batch(eng, orc, N, K):
    """CUDALM's batch test holds every row of a batched call to the single call's result
    (tests/cuda/test_qwen35_batch_kernels.cpp:88-134).  Here a row's bits are the same
    whether it is projected alone or with 2, 7, 8 or 15 others, on the streaming kernel and
    (up to 8 rows) on the lean kernel; with 17 rows and more the tensor-memory kernel, whose
    sums are grouped otherwise, gives the same bits for 17, 40 and 64 rows."""
    import torch
    W, S = raw_weights(N, K, 9400 + N)
    x = make_x(orc, (64, K), 9401 + K, "outlier")
    dW, dS = to_dev(W), to_dev(S, torch.float16)

    def rows(M):
        dx = to_dev(x[:M], torch.bfloat16)
        y = eng.batch_int4_gemv_bf16(dW, dS, dx) if M > 1 else eng.int4_gemv_bf16(dW, dS, dx[0]).view(1, N)
        torch.cuda.synchronize()
        return from_dev(y)

    for lean in (0, 1 << 40):
        prev = eng.set_direct_path_max_bytes(lean)
        try:
            base = rows(16 if lean == 0 else 8)
            for M in ((1, 3, 8, 9) if lean == 0 else (1, 3, 7)):
                assert np.array_equal(rows(M), base[:M]), f"{M} rows, lean kernel {'on' if lean else 'off'}"
        finally:
            eng.set_direct_path_max_bytes(prev)
    base = rows(64)
    for M in (17, 40):
        assert np.array_equal(rows(M), base[:M]), f"{M} rows on the tensor-memory kernel"
