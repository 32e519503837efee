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


class PeerExchange:
    """This rank's exchange buffer and its peers' buffers mapped over CUDA IPC, for
    ``cudalm_b200_topk_exchange_merge``: the candidate lists cross NVLink as plain
    stores from the kernel that also merges them, with no collective launch.  All
    ranks of ``group`` must sit on one node, each on its own GPU.

    The device-side wait for the peers is bounded (``set_exchange_timeout_ns``).  When it
    runs out, ``device_status()`` reads 5 and the affected rows come back as id -1 and
    value -inf.  After that the ranks' epochs no longer agree: ``close()`` this object
    on every rank and build a new one before the next call."""

    def __init__(self, words_per_list: int, rows_cap: int, top_k: int,
                 group: Optional[dist.ProcessGroup] = None):
        import ctypes
        from . import api
        self._lib = api.load_library()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.words, self.rows_cap, self.top_k = words_per_list, rows_cap, top_k
        nbytes = int(self._lib.cudalm_b200_exchange_bytes(self.world, words_per_list))
        if nbytes == 0:
            raise ValueError(f"no peer exchange for {self.world} ranks")
        # Every rank goes through the same collectives whether or not a step failed
        # locally, and all ranks raise together: a rank that cannot map a peer must not
        # leave the others waiting.
        local = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        st = self._lib.cudalm_b200_exchange_create(nbytes, ctypes.byref(local), handle)
        self._local = local if st == 0 else None
        handles: List[Optional[bytes]] = [None] * self.world
        dist.all_gather_object(handles, handle.raw if st == 0 else None, group=group)
        self._ptrs = (ctypes.c_void_p * self.world)()
        self._opened: List[ctypes.c_void_p] = []
        ok = st == 0 and all(h is not None for h in handles)
        if ok:
            for r, h in enumerate(handles):
                if r == self.rank:
                    self._ptrs[r] = local.value
                    continue
                peer = ctypes.c_void_p()
                if self._lib.cudalm_b200_exchange_open(h, ctypes.byref(peer)) != 0:
                    ok = False
                    break
                self._opened.append(peer)
                self._ptrs[r] = peer.value
        verdicts: List[Optional[bool]] = [None] * self.world
        dist.all_gather_object(verdicts, ok, group=group)  # also: every buffer is mapped everywhere
        if not all(verdicts):
            self._release()
            bad = [r for r, v in enumerate(verdicts) if not v]
            raise RuntimeError(f"peer exchange: ranks {bad} could not create or map the buffers")

    def merge(self, packed: torch.Tensor, M: int):
        """The merged pick of ``M`` rows from every rank's packed candidates."""
        from . import api
        dev = packed.device
        argmax = torch.empty(M, dtype=torch.int32, device=dev)
        idx = torch.empty((M, self.top_k), dtype=torch.int32, device=dev)
        val = torch.empty((M, self.top_k), dtype=torch.bfloat16, device=dev)
        api._check("topk_exchange_merge", self._lib.cudalm_b200_topk_exchange_merge(
            api._ptr(packed), self._ptrs, self.rank, self.world, self.words, self.rows_cap, M,
            self.top_k, api._ptr(argmax), api._ptr(idx), api._ptr(val), api._stream()))
        return argmax, idx, val

    def forward(self, head, x: torch.Tensor):
        """Projection, local pick, exchange and merge of one rank in two launches
        (``head``: this rank's ``LmHead``).  Returns None when the rows do not fit one
        pass; the caller then runs ``head.forward`` and ``merge``."""
        from . import api
        M = 1 if x.dim() == 1 else int(x.shape[0])
        dev = x.device
        argmax = torch.empty(M, dtype=torch.int32, device=dev)
        idx = torch.empty((M, self.top_k), dtype=torch.int32, device=dev)
        val = torch.empty((M, self.top_k), dtype=torch.bfloat16, device=dev)
        rows = head.rows
        st = self._lib.cudalm_b200_lm_head_topk_exchange(
            api._ptr(rows.weight), api._ptr(rows.scale), api._ptr(x), rows.N, rows.K, M, self.top_k,
            head.id_offset, api._ptr(head.logits), api._ptr(head.packed), self.rows_cap,
            api._ptr(head.workspace), head.workspace.numel(), self._ptrs, self.rank, self.world,
            self.words, api._ptr(argmax), api._ptr(idx), api._ptr(val), api._stream())
        if st == 6:  # UNSUPPORTED
            return None
        api._check("lm_head_topk_exchange", st)
        return argmax, idx, val

    def _release(self) -> None:
        for peer in self._opened:
            self._lib.cudalm_b200_exchange_close(peer)
        if self._local is not None:
            self._lib.cudalm_b200_exchange_destroy(self._local)
        self._local, self._opened = None, []

    def close(self) -> None:
        """Unmaps the peers' buffers and frees this rank's (after a barrier: no peer
        may still be storing into it)."""
        if self._local is None:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self._release()


class VocabParallelLmHead:
    """Rank-local half of the vocabulary-parallel lm_head.

    ``local`` is an ``LmHead`` over this rank's rows with ``id_offset`` set to
    the block's first token id.  ``forward(x)`` runs the local pick, then either
    exchanges the packed ``[max_rows, k]`` ids and values over peer memory inside
    the merge kernel (``exchange="peer"``: ranks of one node) or all-gathers them
    (``exchange="collective"``: one collective, any backend) and merges on the device.
    """

    def __init__(self, local, group: Optional[dist.ProcessGroup] = None,
                 exchange: str = "collective"):
        from .api import LmHead
        assert isinstance(local, LmHead)
        if exchange not in ("collective", "peer"):
            raise ValueError("exchange is 'collective' or 'peer'")
        self.local = local
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self._gathered = torch.empty((self.world, local.packed.numel()), dtype=torch.int32,
                                     device=local.packed.device)
        self.peer = None
        if exchange == "peer" and self.world > 1:
            self.peer = PeerExchange(local.packed.numel(), local.max_rows, local.top_k, group)

    def forward(self, x: torch.Tensor):
        from .api import topk_merge_packed
        M = 1 if x.dim() == 1 else int(x.shape[0])
        # the peer exchange takes up to 32 rows per call; more rows go through the all-gather
        use_peer = self.peer is not None and M <= 32
        if use_peer:
            fused = self.peer.forward(self.local, x)
            if fused is not None:
                return fused
        argmax, idx, val = self.local.forward(x)
        if self.world == 1:
            return argmax, idx, val
        if use_peer:
            return self.peer.merge(self.local.packed, idx.shape[0])
        dist.all_gather_into_tensor(self._gathered.view(-1), self.local.packed, group=self.group)
        return topk_merge_packed(self._gathered, self.local.max_rows, idx.shape[0], self.local.top_k)

    def close(self) -> None:
        if self.peer is not None:
            self.peer.close()
            self.peer = None
