"""CPU, world_size 2 over gloo: the host-side multi-rank flow of the benchmark —
every rank takes its LPT shard, cuts micro-batches, the union covers the workload
exactly once, and the cross-rank reductions (max time, summed tokens) are right.
No GPU and no collective on the data path are involved."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys, json
    sys.path.insert(0, %r)
    import numpy as np
    from bytetransformer_b200.ranks import Ranks
    from bytetransformer_b200.sharding import lpt_shards, micro_batches
    from bytetransformer_b200.workloads import lengths_for
    r = Ranks(backend="gloo")
    lengths = lengths_for("whole_box_1024x1024")
    mine = lpt_shards(lengths, r.world)[r.rank]
    mbs = micro_batches(lengths, mine, 148 * 128)
    my_tokens = sum(mb.tokens for mb in mbs)
    my_seqs = sum(len(mb.seq_ids) for mb in mbs)
    r.barrier()
    tokens, seqs, idsum = r.sum(my_tokens, my_seqs, float(np.concatenate([mb.seq_ids for mb in mbs]).sum()))
    slowest = r.max(10.0 + r.rank)          # pretend rank k took 10+k ms
    if r.rank == 0:
        print(json.dumps({"world": r.world, "tokens": tokens, "seqs": seqs, "idsum": idsum, "slowest": slowest,
                          "my_tokens": my_tokens}))
    r.close()
""") % ROOT


def test_two_ranks_cover_the_workload_once(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stdout + r.stderr
    import json
    line = [l for l in r.stdout.splitlines() if l.startswith("{")][-1]
    d = json.loads(line)
    assert d["world"] == 2
    assert d["tokens"] == 556500 and d["seqs"] == 1024
    assert d["idsum"] == sum(range(1024))
    assert d["slowest"] == 11.0                        # the maximum over ranks, not rank 0's own time
    assert abs(d["my_tokens"] - 556500 / 2) < 0.005 * 556500
