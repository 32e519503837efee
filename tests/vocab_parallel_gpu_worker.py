"""One rank of the GPU test of the vocabulary-parallel lm_head (launched by
tests/test_gpu_multi.py under torch.distributed.run, one rank per GPU).

Every rank builds the same quantized vocabulary matrix, keeps its own block of rows,
and runs the pick with the peer exchange and with the all-gather; both must equal the
CPU oracle's pick over the whole vocabulary (ids, values and order) for 1, 5 and 32
activation rows, with ties across the blocks' borders.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import cudalm_agent_b200 as eng  # noqa: E402
from oracle import cpu_oracle as orc  # noqa: E402
from helpers import from_dev, make_x, raw_weights, to_dev  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    orc.build()
    vocab, K, k = 20000, 512, 50
    W, S = raw_weights(vocab, K, 4242)
    # identical rows on both sides of every block border: ties that only global ids break
    for r in range(1, world):
        lo, _ = eng.shard_rows(vocab, world, r)
        W[lo:lo + 4] = W[lo - 4:lo]
        S[lo:lo + 4] = S[lo - 4:lo]
    lo, hi = eng.shard_rows(vocab, world, rank)
    lin = eng.W4A16Linear(to_dev(W[lo:hi]), to_dev(S[lo:hi], torch.float16))
    for M in (1, 5, 32):
        x = make_x(orc, (M, K), 4300 + M, "rmsnorm")
        dx = to_dev(x, torch.bfloat16)
        logits = orc.batch_gemv_bf16(W, S, x, threads=8)
        for mode in ("peer", "collective"):
            head = eng.VocabParallelLmHead(eng.LmHead(lin, top_k=k, id_offset=lo, max_rows=M), exchange=mode)
            for _ in range(3):  # epochs advance; every call must give the same pick
                argmax, idx, val = head.forward(dx)
            torch.cuda.synchronize()
            assert eng.device_status() == 0, (rank, mode, M)
            got_idx, got_val, got_arg = from_dev(idx), from_dev(val), from_dev(argmax)
            head.close()
            for m in range(M):
                # the device's logits may differ from the CPU's by a bf16 step; the pick is
                # held to the rule on the CPU logits where those agree on the top-k values
                wi, wv = orc.topk_bf16(logits[m], k)
                if np.array_equal(got_val[m], wv):
                    assert np.array_equal(got_idx[m], wi), (rank, mode, M, m)
                    assert int(got_arg[m]) == int(wi[0])
                else:
                    assert len(set(got_idx[m].tolist()) - set(wi.tolist())) <= 2, (rank, mode, M, m)
                assert np.all(np.diff(orc.bf16_bits_to_f32(got_val[m]).astype(np.float64)) <= 0)
        dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("vocabulary-parallel pick on", world, "GPUs: ok")


if __name__ == "__main__":
    main()
