"""One rank of the CPU (gloo) test of the vocabulary-parallel pick.

Each rank owns a contiguous block of vocabulary rows, computes its block's
logits and local top-k with the CPU oracle, all-gathers the candidate lists and
merges them on the host; every rank must end with the single-rank pick.
Usage: vocab_parallel_worker.py RANK WORLD PORT MODE   (MODE: ok | short)
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from cudalm_agent_b200.vocab_parallel import (TopKMergeError, gather_packed,  # noqa: E402
                                              merge_topk_host, shard_rows, unpack_candidates)
from oracle import cpu_oracle as orc  # noqa: E402
from helpers import make_x, raw_weights  # noqa: E402


def main():
    rank, world, port, mode = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    vocab, K, M, k = 1000, 256, 3, 50
    W, S = raw_weights(vocab, K, 99)          # every rank builds the same matrix
    x = make_x(orc, (M, K), 98, "rmsnorm")
    # heavy ties: quantise the activations coarsely so equal logits occur across blocks
    full = orc.batch_gemv_bf16(W, S, x)
    full = orc.f32_to_bf16_bits(np.round(orc.bf16_bits_to_f32(full) * 4) / 4)
    lo, hi = shard_rows(vocab, world, rank)
    idx = np.full((M, k), -1, np.int32)
    val = np.full((M, k), 0xFF80, np.uint16)
    for m in range(M):
        i, v = orc.topk_bf16(full[m, lo:hi], k)
        idx[m, :len(i)] = i + lo
        val[m, :len(i)] = v
    if mode == "short" and rank == world - 1:
        idx[:, -1] = -1                           # a rank that lost an entry
    # the packed form one all-gather carries: ids int32 [M][k], then values bf16 [M][k]
    packed = torch.from_numpy(np.concatenate([idx.view(np.int32).ravel(),
                                              val.ravel().view(np.int32)]))
    gi, gv = unpack_candidates(gather_packed(packed), M, k)
    blocks = [shard_rows(vocab, world, r) for r in range(world)]
    try:
        argmax, midx, mval = merge_topk_host(list(gi), list(gv), k, blocks)
    except TopKMergeError as e:
        print(f"rank {rank}: merge refused: {e}")
        dist.destroy_process_group()
        sys.exit(3 if mode == "short" else 1)
    for m in range(M):
        wi, wv = orc.topk_bf16(full[m], k)
        assert np.array_equal(midx[m].numpy(), wi), (rank, m)
        assert np.array_equal(mval[m].view(torch.int16).numpy().view(np.uint16), wv), (rank, m)
        assert int(argmax[m]) == orc.argmax_bf16(full[m])
    dist.destroy_process_group()
    print(f"rank {rank}: ok")


if __name__ == "__main__":
    main()
