"""The allocation-free vocabulary projection (cudalm_b200_lm_head_topk_static).

It serves callers that cannot allocate device memory when they need a token pick
-- a server whose pools own the whole GPU, a decode loop where cudaMalloc is
forbidden because it synchronises the device -- by keeping its scratch in a fixed
array inside the library.  Here it is called through the C ABI twice in a row
with different activations and must reproduce, bit for bit, what the
workspace-taking entry point returns for the same inputs: the pick is integer
work, so the tolerance is zero, and the second call shows that what the first
left in the shared array does no harm.

The file sorts last on purpose: a run that stops at the first failure has then
already run every other test.
"""
import numpy as np
import pytest

from helpers import from_dev, make_weights, make_x, to_dev

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_workspace_entry_twice():
    import torch
    import cudalm_agent_b200 as eng
    from oracle import cpu_oracle as orc
    orc.build()
    eng.load_library()

    N, K, M, k = 20000, 1024, 6, 50
    _, W, S = make_weights(orc, N, K, 4242)
    lin = eng.W4A16Linear(to_dev(W), to_dev(S, torch.float16))
    assert eng.lm_head_static_scratch_bytes() >= 600_000

    ref_head = eng.LmHead(lin, top_k=k, id_offset=7, max_rows=M, keep_logits=True)
    logits = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    argmax = torch.empty(M, dtype=torch.int32, device="cuda")
    idx = torch.empty((M, k), dtype=torch.int32, device="cuda")
    val = torch.empty((M, k), dtype=torch.bfloat16, device="cuda")

    # one warm-up call: the first call on a device looks up the array's address (and loads
    # the kernels), which is allowed to cost memory; the calls after it are not
    x0 = to_dev(make_x(orc, (M, K), 9, "rmsnorm"), torch.bfloat16)
    eng.lm_head_topk_static(lin, x0, logits, argmax, idx, val, id_offset=7)
    big = torch.empty((32, N), dtype=torch.bfloat16, device="cuda")  # logits of the 32-row call below
    x32 = to_dev(make_x(orc, (32, K), 10, "rmsnorm"), torch.bfloat16)
    i32 = torch.empty((32, k), dtype=torch.int32, device="cuda")
    v32 = torch.empty((32, k), dtype=torch.bfloat16, device="cuda")
    a32 = torch.empty(32, dtype=torch.int32, device="cuda")
    eng.lm_head_topk_static(lin, x32, big, a32, i32, v32, id_offset=7)  # the tensor-memory kernel's first use
    torch.cuda.synchronize()
    # free device memory as the driver sees it: a cudaMalloc inside the library would show
    # here, which torch's own allocator statistics cannot see
    free_before = torch.cuda.mem_get_info()[0]
    eng.lm_head_topk_static(lin, x0, logits, argmax, idx, val, id_offset=7)
    eng.lm_head_topk_static(lin, x32, big, a32, i32, v32, id_offset=7)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] >= free_before, "the allocation-free entry allocated device memory"
    for call, (seed, rows) in enumerate(((1, M), (2, 3))):
        x = to_dev(make_x(orc, (rows, K), seed, "rmsnorm"), torch.bfloat16)
        want = [from_dev(t).copy() for t in ref_head.forward(x)]
        want_logits = from_dev(ref_head.logits[:rows]).copy()
        for t in (logits, argmax, idx, val):
            t.fill_(0)
        eng.lm_head_topk_static(lin, x, logits, argmax, idx, val, id_offset=7)
        torch.cuda.synchronize()
        assert np.array_equal(from_dev(argmax)[:rows], want[0]), f"call {call}: argmax"
        assert np.array_equal(from_dev(idx)[:rows], want[1]), f"call {call}: top-k ids"
        assert np.array_equal(from_dev(val)[:rows], want[2]), f"call {call}: top-k values"
        assert np.array_equal(from_dev(logits)[:rows], want_logits), f"call {call}: logits"
        # and the pick follows the reference's ordering rule on those logits
        for m in range(rows):
            wi, wv = orc.topk_bf16(want_logits[m], k)
            assert np.array_equal(from_dev(idx)[m] - 7, wi)
    assert eng.device_status() == 0


def test_static_entry_rejects_what_it_cannot_hold():
    import ctypes
    import cudalm_agent_b200 as eng
    lib = eng.load_library()
    p = ctypes.c_void_p(4096)
    f = lib.cudalm_b200_lm_head_topk_static
    # more than 32 activation rows: the fixed array has no room
    assert f(p, p, p, 1000, 1024, 33, 50, 0, p, p, p, p, None) == 7
    # the logits buffer is an output of this entry point, never scratch
    assert f(p, p, p, 1000, 1024, 1, 50, 0, None, p, p, p, None) == 2
