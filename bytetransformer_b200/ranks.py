"""Rank plumbing for multi-GPU runs: one process per GPU, launched by torchrun.

The encoder path has no exchange step, so the only cross-rank operations are the
ones a benchmark or a driver needs around the work: a barrier, a maximum (timing
is the slowest rank's) and a sum (tokens, bytes, launches).  `nccl` on GPUs,
`gloo` on CPU (tests)."""
from __future__ import annotations

import os
from typing import Optional

import torch


class Ranks:
    def __init__(self, backend: Optional[str] = None, device: Optional[torch.device] = None):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.device = device
        self.dist = None
        self.backend = None
        if self.world > 1:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29511")
            backend = backend or ("nccl" if (device is not None and device.type == "cuda") else "gloo")
            kw = {}
            if backend == "nccl" and device is not None:
                kw["device_id"] = device
            dist.init_process_group(backend, rank=self.rank, world_size=self.world, **kw)
            self.backend = backend
            self.dist = dist

    def _tensor(self, values):
        dev = self.device if (self.backend == "nccl" and self.device is not None) else torch.device("cpu")
        return torch.tensor(values, dtype=torch.float64, device=dev)

    def barrier(self):
        if self.device is not None and self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        if self.dist is not None:
            self.dist.barrier()
        if self.device is not None and self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    def max(self, value: float) -> float:
        if self.dist is None:
            return float(value)
        t = self._tensor([value])
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum(self, *values):
        if self.dist is None:
            return [float(v) for v in values]
        t = self._tensor(list(values))
        self.dist.all_reduce(t)
        return [float(v) for v in t.tolist()]

    def close(self):
        if self.dist is not None:
            self.dist.barrier()
            self.dist.destroy_process_group()
            self.dist = None
