"""Running a set of sequences through the encoder on one GPU, micro-batch by
micro-batch, either with inputs already resident in device memory or end to end
from pinned host buffers (host->device copy, compute, device->host copy
overlapped on three streams).

One process drives one GPU.  For several GPUs every process takes the shard that
`sharding.lpt_shards` gives its rank; there is no communication between ranks.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from .encoder import Encoder
from .sharding import MicroBatch, micro_batches

TOKEN_BUDGET_UNIT = 148 * 128     # one 128-row GEMM tile per SM and tile column
DEFAULT_TOKEN_BUDGET = TOKEN_BUDGET_UNIT
MAX_TOKEN_BUDGET_UNITS = 4


def pick_token_budget(total_tokens: int, min_batches: int = 4) -> int:
    """Token budget of a micro-batch for a rank that holds `total_tokens`: the largest of 1..4 x 18,944
    that still leaves at least `min_batches` micro-batches (else 18,944).

    Larger launches amortise each kernel's first and last wave (measured on B200, BERT-base, 556,500 tokens on
    one GPU: 3.72 / 3.86 / 3.89 / 3.93 M tokens/s at 1 / 2 / 3 / 4 units; the GEMM kernels gain 8 %, the
    attention kernel nothing), while the end-to-end path overlaps its host copies with the compute of the
    neighbouring micro-batches and so wants several of them: the first copy in and the last copy out are
    exposed.  With four: the benchmark's 556,500 tokens are cut with a budget of 75,776 on one and two GPUs,
    37,888 on four and 18,944 on eight; with `min_batches=1` (resident inputs) always 75,776.  (Measured on four GPUs: two micro-batches of 69.6k tokens per rank
    instead of four of 34.8k give +2 % with resident inputs and -3 % end to end.)"""
    best = 1
    for k in range(1, MAX_TOKEN_BUDGET_UNITS + 1):
        if -(-int(total_tokens) // (k * TOKEN_BUDGET_UNIT)) >= min_batches:
            best = k
    return best * TOKEN_BUDGET_UNIT


class PackedRunner:
    def __init__(self, enc: Encoder, lengths: Sequence[int], seq_ids: Sequence[int],
                 token_budget: int = 0, mix: bool = False, min_batches: int = 4):
        """`token_budget` 0 = pick_token_budget() of this rank's tokens with at least `min_batches` micro-batches:
        4 (default) for run_host, whose copies hide behind the neighbouring micro-batches' compute; 1 for a runner
        that only serves run_device, where nothing is overlapped and the largest launch is the fastest (on eight
        GPUs a rank's 69.6k tokens of the benchmark then go through in one launch per kernel instead of four).
        `mix` False (default): micro-batches are
        filled to the budget one after the other in length order, so all but the last hold a whole number of
        148 x 128-token waves of GEMM tiles (measured on one B200: +0.6 % over equal micro-batches, 30 waves per
        GEMM and step instead of 32; the attention kernel takes the same time either way); True: equal
        micro-batches with the same mix of lengths (sharding.micro_batches)."""
        self.enc = enc
        self.device = enc.device
        self.hidden = enc.hidden
        if token_budget <= 0:
            ids = np.asarray(seq_ids, dtype=np.int64)
            token_budget = pick_token_budget(int(np.asarray(lengths, dtype=np.int64)[ids].sum()) if len(ids) else 0,
                                             min_batches=max(1, int(min_batches)))
            token_budget = max(token_budget, int(np.asarray(lengths)[ids].max()) if len(ids) else 1)
        self.token_budget = int(token_budget)
        self.batches: List[MicroBatch] = micro_batches(lengths, seq_ids, token_budget, mix=mix)
        self.tokens = int(sum(mb.tokens for mb in self.batches))
        self.max_tokens = max([mb.tokens for mb in self.batches] + [1])
        self.max_batch = max([len(mb.seq_ids) for mb in self.batches] + [1])
        with torch.cuda.device(self.device):
            self.workspace = torch.empty(enc.packed_workspace_bytes(self.max_batch, self.max_tokens),
                                         dtype=torch.int8, device=self.device)
            self.cu_dev = [torch.from_numpy(mb.cu_seqlens).to(self.device) for mb in self.batches]

    # ------------------------------------------------------------ device-resident
    def make_device_inputs(self, seed: int = 0):
        g = torch.Generator(device="cpu").manual_seed(seed)
        xs = []
        for mb in self.batches:
            xs.append(torch.randn(max(mb.tokens, 1), self.hidden, generator=g).half().to(self.device)[:mb.tokens])
        outs = [torch.empty_like(x) for x in xs]
        return xs, outs

    def run_device(self, xs, outs):
        """One pass over every micro-batch; inputs and outputs stay in device memory."""
        for mb, cu, x, o in zip(self.batches, self.cu_dev, xs, outs):
            if mb.tokens == 0:
                continue
            self.enc.forward_packed(x, cu, mb.max_len, out=o, workspace=self.workspace)

    # ----------------------------------------------------------------- end to end
    def make_host_inputs(self, seed: int = 0):
        g = torch.Generator(device="cpu").manual_seed(seed)
        xs, outs = [], []
        for mb in self.batches:
            x = torch.randn(max(mb.tokens, 1), self.hidden, generator=g).half()[:mb.tokens].contiguous().pin_memory()
            xs.append(x)
            outs.append(torch.empty_like(x).pin_memory())
        return xs, outs

    def _e2e_state(self):
        if getattr(self, "_e2e", None) is None:
            with torch.cuda.device(self.device):
                st = {
                    "in": [torch.empty(self.max_tokens, self.hidden, dtype=torch.float16, device=self.device) for _ in range(2)],
                    "out": [torch.empty(self.max_tokens, self.hidden, dtype=torch.float16, device=self.device) for _ in range(2)],
                    "s_in": torch.cuda.Stream(self.device), "s_out": torch.cuda.Stream(self.device),
                    "ev_in": [torch.cuda.Event() for _ in range(2)], "ev_cmp": [torch.cuda.Event() for _ in range(2)],
                    "ev_out": [torch.cuda.Event() for _ in range(2)], "ev_free_in": [torch.cuda.Event() for _ in range(2)],
                    # whether a buffer pair has been used before: kept ACROSS calls, because the first copies of a
                    # call are enqueued while the last micro-batches of the call before may still be computing
                    "used": [False, False],
                }
            self._e2e = st
        return self._e2e

    def run_host(self, xs_host, outs_host):
        """One pass from pinned host inputs to pinned host outputs.  Copies run on
        their own streams and overlap the compute of the neighbouring micro-batches
        (two device buffers each way).  Returns (h2d_bytes, d2h_bytes)."""
        st = self._e2e_state()
        cmp_stream = torch.cuda.current_stream(self.device)
        h2d = d2h = 0
        used = st["used"]
        for i, (mb, cu, xh, oh) in enumerate(zip(self.batches, self.cu_dev, xs_host, outs_host)):
            if mb.tokens == 0:
                continue
            k = i & 1
            xin = st["in"][k][:mb.tokens]
            xout = st["out"][k][:mb.tokens]
            with torch.cuda.stream(st["s_in"]):
                if used[k]:
                    st["s_in"].wait_event(st["ev_free_in"][k])     # compute that read this buffer is done
                xin.copy_(xh, non_blocking=True)
                st["ev_in"][k].record(st["s_in"])
            cmp_stream.wait_event(st["ev_in"][k])
            if used[k]:
                cmp_stream.wait_event(st["ev_out"][k])             # previous D2H from this out buffer is done
            self.enc.forward_packed(xin, cu, mb.max_len, out=xout, workspace=self.workspace)
            st["ev_cmp"][k].record(cmp_stream)
            st["ev_free_in"][k].record(cmp_stream)
            with torch.cuda.stream(st["s_out"]):
                st["s_out"].wait_event(st["ev_cmp"][k])
                oh.copy_(xout, non_blocking=True)
                st["ev_out"][k].record(st["s_out"])
            used[k] = True
            h2d += xh.numel() * 2 + cu.numel() * 0
            d2h += oh.numel() * 2
        cmp_stream.wait_stream(st["s_out"])
        return h2d, d2h
