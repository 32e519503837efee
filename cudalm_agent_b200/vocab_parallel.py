"""Vocabulary-parallel lm_head: each rank owns a contiguous block of vocabulary
rows, picks its local top-k with global token ids, and one all-gather of the
candidate lists (k ids + k values per activation row per rank) lets every rank
merge to the same final pick.

The merge order is (value descending, id ascending) on *global* ids, so the
result equals the single-GPU result exactly, ties included (CUDALM
include/cudalm/greedy.h:28-39, include/cudalm/sampling.h:152-166).

``merge_topk_host`` is the same merge on the host, with validation of what the
ranks sent (a missing or short list, an id outside the sender's block, an id sent
twice); it backs the CPU tests of the multi-rank path and is the check a caller
can run when a rank is suspected of having failed.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_rows(vocab: int, world: int, rank: int) -> Tuple[int, int]:
    """Rows ``[lo, hi)`` of rank ``rank``: contiguous blocks whose sizes differ
    by at most one m-tile (16 rows), every block a multiple of 16 except the last."""
    tiles = (vocab + 15) // 16
    lo_t = tiles * rank // world
    hi_t = tiles * (rank + 1) // world
    return min(lo_t * 16, vocab), min(hi_t * 16, vocab)


class TopKMergeError(ValueError):
    """The gathered candidate lists are not what healthy ranks would send."""


def merge_topk_host(lists_idx: Sequence[torch.Tensor], lists_val: Sequence[torch.Tensor], k: int,
                    blocks: Optional[Sequence[Tuple[int, int]]] = None
                    ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Merges per-rank ``[M, k]`` lists on the host.  Returns
    ``(argmax [M], idx [M, k], val [M, k])``.  Raises ``TopKMergeError`` when a
    list is missing (None), has the wrong shape, repeats an id, or holds an id
    outside its sender's block (``blocks[r] = (lo, hi)``)."""
    if len(lists_idx) == 0 or len(lists_idx) != len(lists_val):
        raise TopKMergeError("no candidate lists, or ids/values count differ")
    M = None
    for r, (li, lv) in enumerate(zip(lists_idx, lists_val)):
        if li is None or lv is None:
            raise TopKMergeError(f"rank {r} sent no list")
        if li.dim() != 2 or li.shape[1] != k or tuple(lv.shape) != tuple(li.shape):
            raise TopKMergeError(f"rank {r} sent a list of shape {tuple(li.shape)}, want [M, {k}]")
        M = li.shape[0] if M is None else M
        if li.shape[0] != M:
            raise TopKMergeError(f"rank {r} sent {li.shape[0]} rows, others {M}")
        real = li >= 0
        if blocks is not None:
            lo, hi = blocks[r]
            if bool(((li < lo) | (li >= hi))[real].any()):
                raise TopKMergeError(f"rank {r} sent an id outside its block [{lo}, {hi})")
            want = min(k, hi - lo)
            if bool((real.sum(dim=1) != want).any()):
                raise TopKMergeError(f"rank {r} sent a short list")
    idx = torch.cat([t.cpu().to(torch.int64) for t in lists_idx], dim=1)
    val = torch.cat([t.cpu() for t in lists_val], dim=1)
    out_idx = torch.full((M, k), -1, dtype=torch.int32)
    out_val = torch.full((M, k), float("-inf"), dtype=torch.bfloat16)
    for m in range(M):
        real = idx[m] >= 0
        ids = idx[m][real]
        if ids.unique().numel() != ids.numel():
            raise TopKMergeError(f"row {m}: an id was sent twice")
        v = val[m][real].float()
        # value descending, then id ascending: sort by id first, then stable by value
        order = torch.argsort(ids, stable=True)
        order = order[torch.argsort(-v[order], stable=True)]
        n = min(k, order.numel())
        out_idx[m, :n] = ids[order[:n]].to(torch.int32)
        out_val[m, :n] = val[m][real][order[:n]]
    return out_idx[:, 0].clone(), out_idx, out_val


def gather_packed(packed: torch.Tensor, group=None) -> torch.Tensor:
    """All-gathers one rank's packed candidate buffer (int32, see
    ``api.packed_words``) into ``[world, words]`` with ONE collective.  int32 is
    carried by every backend, which is what lets the multi-rank logic be tested
    with gloo on CPU."""
    world = dist.get_world_size(group)
    out = torch.empty((world, packed.numel()), dtype=torch.int32, device=packed.device)
    dist.all_gather_into_tensor(out.view(-1), packed.contiguous().view(-1), group=group)
    return out


def unpack_candidates(gathered: torch.Tensor, rows: int, k: int):
    """``[world, words]`` -> per-rank lists of ids int32 ``[rows, k]`` and values
    bf16 ``[rows, k]`` (host-side form, for ``merge_topk_host``)."""
    n = rows * k
    ids = [g[:n].view(rows, k) for g in gathered]
    vals = [g[n:].contiguous().view(torch.bfloat16)[:n].view(rows, k) for g in gathered]
    return ids, vals


class VocabParallelLmHead:
    """Rank-local half of the vocabulary-parallel lm_head.

    ``local`` is an ``LmHead`` over this rank's rows with ``id_offset`` set to
    the block's first token id.  ``forward(x)`` runs the local pick, all-gathers
    the packed ``[max_rows, k]`` ids and values (one collective) and merges on
    the device.
    """

    def __init__(self, local, group: Optional[dist.ProcessGroup] = None):
        from .api import LmHead
        assert isinstance(local, LmHead)
        self.local = local
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self._gathered = torch.empty((self.world, local.packed.numel()), dtype=torch.int32,
                                     device=local.packed.device)

    def forward(self, x: torch.Tensor):
        from .api import topk_merge_packed
        argmax, idx, val = self.local.forward(x)
        if self.world == 1:
            return argmax, idx, val
        dist.all_gather_into_tensor(self._gathered.view(-1), self.local.packed, group=self.group)
        return topk_merge_packed(self._gathered, self.local.max_rows, idx.shape[0], self.local.top_k)
