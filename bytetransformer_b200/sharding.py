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


def micro_batches(lengths: Sequence[int], seq_ids: Sequence[int], token_budget: int) -> List[MicroBatch]:
    """Cut the sequences `seq_ids` into micro-batches of at most `token_budget`
    packed tokens.  Sequences are taken longest first so that a micro-batch holds
    sequences of similar length (keeps the attention grid dense); zero-length
    sequences are kept (they produce no work and no output rows)."""
    lengths = np.asarray(lengths, dtype=np.int64)
    ids = np.asarray(seq_ids, dtype=np.int64)
    if token_budget <= 0:
        raise ValueError("token_budget must be positive")
    order = ids[np.argsort(-lengths[ids], kind="stable")]
    out: List[MicroBatch] = []
    cur: List[int] = []
    tok = 0
    for i in order:
        L = int(lengths[i])
        if L > token_budget:
            raise ValueError(f"sequence {int(i)} has {L} tokens, more than the budget {token_budget}")
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
