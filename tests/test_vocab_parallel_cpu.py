"""The multi-rank half of the vocabulary-parallel lm_head, on CPU: world_size 2
and 4 gloo ranks (tests/vocab_parallel_worker.py), plus the host-side merge and
its validation of what ranks send (failure detection without touching a GPU)."""
import os
import socket
import subprocess
import sys

import pytest
import torch

from cudalm_agent_b200.vocab_parallel import TopKMergeError, merge_topk_host

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return str(s.getsockname()[1])


def _run(world, mode):
    port = _free_port()
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "vocab_parallel_worker.py"),
                               str(r), str(world), port, mode],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(world)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out = "timeout"
        outs.append((p.returncode, out))
    return outs


@pytest.mark.parametrize("world", [2, 4])
def test_ranks_agree_with_single_rank_pick(world, orc):
    for rc, out in _run(world, "ok"):
        assert rc == 0, out


def test_short_list_is_detected_on_every_rank(orc):
    for rc, out in _run(2, "short"):
        assert rc == 3 and "short list" in out, out


def _lists(vals_by_rank, ids_by_rank):
    li = [torch.tensor(i, dtype=torch.int32) for i in ids_by_rank]
    lv = [torch.tensor(v, dtype=torch.float32).to(torch.bfloat16) for v in vals_by_rank]
    return li, lv


def test_merge_orders_by_value_then_global_id():
    # the tie at 2.0 spans both ranks: the lower global id (3) comes first
    li, lv = _lists([[[2.0, 1.0]], [[2.0, 0.5]]], [[[7, 1]], [[3, 9]]])
    argmax, idx, val = merge_topk_host(li, lv, 2)
    assert idx.tolist() == [[3, 7]] and argmax.tolist() == [3]
    assert val.float().tolist() == [[2.0, 2.0]]


def test_merge_rejects_bad_input():
    li, lv = _lists([[[2.0, 1.0]], [[2.0, 0.5]]], [[[7, 1]], [[3, 9]]])
    with pytest.raises(TopKMergeError, match="no list"):
        merge_topk_host([li[0], None], [lv[0], None], 2)
    with pytest.raises(TopKMergeError, match="shape"):
        merge_topk_host([li[0], li[1][:, :1]], [lv[0], lv[1][:, :1]], 2)
    with pytest.raises(TopKMergeError, match="twice"):
        merge_topk_host([li[0], li[0]], [lv[0], lv[0]], 2)
    with pytest.raises(TopKMergeError, match="outside"):
        merge_topk_host(li, lv, 2, blocks=[(0, 8), (8, 16)])
    li[1][0, 1] = -1
    with pytest.raises(TopKMergeError, match="short"):
        merge_topk_host(li, lv, 2, blocks=[(0, 8), (0, 16)])
    # padding is legal when the block is smaller than k
    merge_topk_host(li, lv, 2, blocks=[(0, 8), (3, 4)])
