"""Host-side handling of a failed shard in a multi-GPU run.

The encoder path shards by sequence with no exchange between ranks, so a rank that fails takes nothing
with it but its own sequences: the survivors split those among themselves and carry on.  Nothing here
touches a GPU.  Ranks learn of a failure between steps, on the host, through a key-value store (the
`torch.distributed` TCP store): a rank whose step raised reports itself; a rank that stopped reporting
progress is presumed dead after a timeout.  No collective is involved, so no rank ever blocks in one
waiting for a rank that is gone.

  board = ShardBoard(rank, world)                       # MASTER_ADDR / MASTER_PORT (+1) from the environment
  shards = lpt_shards(lengths, world)
  for step in range(steps):
      gone = board.failed_ranks()
      if gone - known: shards = reshard_after_failure(lengths, shards, gone); known = gone
      try: run(shards[rank]); board.heartbeat(step)
      except Exception as e: board.report_failure(repr(e), step); break
"""
from __future__ import annotations

import os
import time
from typing import Dict, Iterable, List, Optional, Sequence, Set

import numpy as np

from .sharding import sequence_cost


def reshard_after_failure(lengths: Sequence[int], shards: Sequence[np.ndarray], failed: Iterable[int],
                          hidden: int = 768) -> List[np.ndarray]:
    """New shards after the ranks in `failed` are gone: their sequences go to the surviving ranks,
    longest-processing-time first onto the currently lightest survivor (the survivors keep what they had).
    Deterministic: every survivor computes the same answer from the same inputs.  Failed ranks get an
    empty shard.  Raises if no rank survives."""
    lengths = np.asarray(lengths, dtype=np.int64)
    failed = set(int(f) for f in failed)
    n = len(shards)
    survivors = [r for r in range(n) if r not in failed]
    if not survivors:
        raise RuntimeError("every rank has failed: nothing left to run the sequences on")
    cost = sequence_cost(lengths, hidden)
    members: Dict[int, List[int]] = {r: [int(i) for i in shards[r]] for r in survivors}
    load = {r: float(cost[members[r]].sum()) if members[r] else 0.0 for r in survivors}
    orphans = sorted((int(i) for r in failed if r < n for i in shards[r]), key=lambda i: (-cost[i], i))
    for i in orphans:
        r = min(survivors, key=lambda s: (load[s], s))
        members[r].append(i)
        load[r] += float(cost[i])
    return [np.array(sorted(members[r]), dtype=np.int64) if r in members else np.zeros(0, dtype=np.int64)
            for r in range(n)]


class ShardBoard:
    """What the ranks tell one another between steps, through a key-value store."""

    def __init__(self, rank: int, world: int, store=None, port_offset: int = 1, timeout_s: float = 60.0):
        self.rank, self.world = int(rank), int(world)
        if store is None:
            import datetime
            from torch.distributed import TCPStore
            host = os.environ.get("MASTER_ADDR", "127.0.0.1")
            port = int(os.environ.get("MASTER_PORT", "29511")) + port_offset
            store = TCPStore(host, port, self.world, is_master=(self.rank == 0),
                             timeout=datetime.timedelta(seconds=timeout_s), wait_for_workers=True)
        self.store = store

    # ------------------------------------------------------------------ progress and failure
    def heartbeat(self, step: int) -> None:
        self.store.set(f"hb/{self.rank}", f"{int(step)}:{time.time():.3f}")

    def report_failure(self, reason: str = "", step: int = -1) -> None:
        """`step`: the step this rank did not finish (-1 = not known).  A survivor that has already run that step
        runs it again for the sequences it takes over; one that has not, simply runs them as part of it."""
        self.store.set(f"failed/{self.rank}", f"{int(step)}:{reason or 'failed'}")

    def failure_step(self, rank: int) -> int:
        """The step rank `rank` reported as unfinished, or -1 (not failed, or not known)."""
        v = self._get(f"failed/{int(rank)}")
        if v is None:
            return -1
        try:
            return int(v.split(":", 1)[0])
        except ValueError:
            return -1

    def _get(self, key: str) -> Optional[str]:
        # (check first: a plain get() would wait for the key)
        if not self.store.check([key]):
            return None
        return self.store.get(key).decode()

    def failed_ranks(self, stale_after_s: Optional[float] = None) -> Set[int]:
        """Ranks that reported a failure, plus (with `stale_after_s`) ranks whose last heartbeat is older
        than that many seconds."""
        gone = set()
        now = time.time()
        for r in range(self.world):
            if self._get(f"failed/{r}") is not None:
                gone.add(r)
            elif stale_after_s is not None and r != self.rank:
                hb = self._get(f"hb/{r}")
                if hb is not None and now - float(hb.split(":")[1]) > stale_after_s:
                    gone.add(r)
        return gone

    # ------------------------------------------------------------------ results without a collective
    def publish(self, key: str, value: str) -> None:
        self.store.set(f"{key}/{self.rank}", value)

    def collect(self, key: str, ranks: Iterable[int], timeout_s: float = 60.0) -> Dict[int, str]:
        """Values the given ranks published under `key`; waits (bounded) for those still missing."""
        out: Dict[int, str] = {}
        deadline = time.time() + timeout_s
        todo = [int(r) for r in ranks]
        while todo:
            for r in list(todo):
                v = self._get(f"{key}/{r}")
                if v is not None:
                    out[r] = v
                    todo.remove(r)
            if todo:
                if time.time() > deadline:
                    raise TimeoutError(f"ranks {todo} never published {key!r}")
                time.sleep(0.02)
        return out
