"""Splitting a set of variable-length sequences over GPUs and into micro-batches.

The encoder path needs no exchange between sequences (attention never crosses a
sequence, GEMMs are row-wise), so multi-GPU execution is plain sharding: every
GPU holds a full weight replica and receives a subset of the sequences, chosen
so that the estimated cost per GPU is balanced.  No collective is involved.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import numpy as np


def sequence_cost(length, hidden: int = 768) -> float:
    """Algorithmic flops of one layer for one sequence: GEMMs 24*L*H^2 plus
    attention 4*H*L^2."""
    length = np.asarray(length, dtype=np.float64)
    return 24.0 * length * hidden * hidden + 4.0 * hidden * length * length


def lpt_shards(lengths: Sequence[int], n_shards: int, hidden: int = 768) -> List[np.ndarray]:
    """Longest-processing-time greedy: sort by cost descending, give each sequence
    to the currently lightest shard.  Returns, per shard, the indices of its
    sequences (ascending).  Deterministic; every index appears exactly once."""
    lengths = np.asarray(lengths, dtype=np.int64)
    if n_shards <= 0:
        raise ValueError("n_shards must be positive")
    cost = sequence_cost(lengths, hidden)
    order = np.argsort(-cost, kind="stable")
    load = np.zeros(n_shards, dtype=np.float64)
    members: List[List[int]] = [[] for _ in range(n_shards)]
    for i in order:
        s = int(np.argmin(load))
        members[s].append(int(i))
        load[s] += cost[i]
    return [np.array(sorted(m), dtype=np.int64) for m in members]


@dataclass
class MicroBatch:
    seq_ids: np.ndarray      # indices into the caller's sequence list
    cu_seqlens: np.ndarray   # int32 [n+1]
    max_len: int
    tokens: int


def micro_batches(lengths: Sequence[int], seq_ids: Sequence[int], token_budget: int,
                  mix: bool = True) -> List[MicroBatch]:
    """Cut the sequences `seq_ids` into micro-batches of at most `token_budget` packed tokens; inside a
    micro-batch the sequences are ordered longest first.  Zero-length sequences are kept (they produce no
    work and no output rows).

    mix=True (default): the fewest micro-batches the budget allows, all with about the same token count and
    the same mix of lengths (the length-sorted sequences are dealt out in snake order).  The attention
    kernel hands its (sequence, query tile, head) items to a fixed set of persistent CTAs in snake order
    too; with long and short sequences in every micro-batch the cheap items fill the last round, where a
    micro-batch of equal lengths leaves part of the CTAs idle (8.5 % against 4.4 % over the mean load on
    1024 lengths uniform in [16, 1024]).
    mix=False: greedy fill in length order, so that a micro-batch holds sequences of similar length."""
    lengths = np.asarray(lengths, dtype=np.int64)
    ids = np.asarray(seq_ids, dtype=np.int64)
    if token_budget <= 0:
        raise ValueError("token_budget must be positive")
    order = ids[np.argsort(-lengths[ids], kind="stable")]
    for i in order:
        if int(lengths[i]) > token_budget:
            raise ValueError(f"sequence {int(i)} has {int(lengths[i])} tokens, more than the budget {token_budget}")
    if mix and len(order) > 0:
        total = int(lengths[order].sum())
        n = max(1, -(-total // token_budget))
        while True:
            bins: List[List[int]] = [[] for _ in range(n)]
            tok = np.zeros(n, dtype=np.int64)
            for k, i in enumerate(order):
                r, c = divmod(k, n)
                b = c if r % 2 == 0 else n - 1 - c
                bins[b].append(int(i))
                tok[b] += lengths[i]
            if tok.max() <= token_budget:
                return [_finish(lengths, b) for b in bins if b]
            n += 1
    out: List[MicroBatch] = []
    cur: List[int] = []
    tok = 0
    for i in order:
        L = int(lengths[i])
        if cur and tok + L > token_budget:
            out.append(_finish(lengths, cur))
            cur, tok = [], 0
        cur.append(int(i))
        tok += L
    if cur:
        out.append(_finish(lengths, cur))
    return out


def _finish(lengths, cur) -> MicroBatch:
    ls = lengths[np.array(cur, dtype=np.int64)]
    cu = np.zeros(len(cur) + 1, dtype=np.int32)
    np.cumsum(ls, out=cu[1:])
    return MicroBatch(np.array(cur, dtype=np.int64), cu, int(ls.max()) if len(ls) else 0, int(cu[-1]))
