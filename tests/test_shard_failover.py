"""CPU: a rank that fails between steps loses nothing but time - the survivors learn of it on the host
(key-value store, no collective) and split its sequences among themselves (bytetransformer_b200/failover.py).
Three worker processes stand in for three GPUs; the work of a step is a stub that records which sequences
were run.  The failure is a Python exception raised by rank 1's step function; no GPU is involved."""
import json
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reshard_keeps_survivors_and_places_every_orphan_once():
    from bytetransformer_b200.failover import reshard_after_failure
    from bytetransformer_b200.sharding import lpt_shards, sequence_cost
    from bytetransformer_b200.workloads import lengths_for
    lengths = lengths_for("whole_box_1024x1024")
    shards = lpt_shards(lengths, 8)
    new = reshard_after_failure(lengths, shards, {2, 5})
    assert len(new[2]) == 0 and len(new[5]) == 0
    assert sorted(np.concatenate(new).tolist()) == list(range(1024))          # everything exactly once
    for r in (0, 1, 3, 4, 6, 7):
        assert set(shards[r].tolist()) <= set(new[r].tolist())                # survivors keep what they had
    cost = [sequence_cost(lengths[s]).sum() for s in new if len(s)]
    assert max(cost) / (sum(cost) / 6) < 1.01                                  # and stay balanced
    assert all(np.array_equal(a, b) for a, b in zip(new, reshard_after_failure(lengths, shards, [5, 2])))  # deterministic
    with pytest.raises(RuntimeError):
        reshard_after_failure(lengths, shards, range(8))


WORKER = textwrap.dedent("""
    import os, sys, json, time
    sys.path.insert(0, %r)
    import numpy as np
    from bytetransformer_b200.failover import ShardBoard, reshard_after_failure
    from bytetransformer_b200.sharding import lpt_shards
    from bytetransformer_b200.workloads import lengths_for
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    board = ShardBoard(rank, world)
    lengths = lengths_for("b16_s512")                  # 16 sequences
    shards = lpt_shards(lengths, world)
    steps, fail_step = 4, 2
    done = []                                           # (step, sequence) pairs this rank completed
    known = set()
    alive = True
    for step in range(steps):
        # ---- between steps: has anybody failed?  (ranks proceed in lock step here so that the test is
        # deterministic: everyone waits for everyone's heartbeat or failure notice of the previous step)
        if step > 0:
            deadline = time.time() + 60
            while True:
                gone = board.failed_ranks()
                seen = [r for r in range(world) if r in gone or int((board._get(f"hb/{r}") or "-1:0").split(":")[0]) >= step - 1]
                if len(seen) == world: break
                assert time.time() < deadline
                time.sleep(0.01)
            if gone - known:
                new = reshard_after_failure(lengths, shards, gone)
                for r in gone - known:
                    # A step the failed rank did not finish and this rank has already run is run again for the
                    # sequences it takes over; if this rank has not run it yet (the failed rank was ahead), the
                    # new shard simply includes them.
                    f = board.failure_step(r)
                    lost = set(int(i) for i in shards[r])
                    if 0 <= f < step:
                        done += [(s, i) for s in range(f, step) for i in new[rank].tolist() if i in lost]
                shards, known = new, set(gone)
        try:
            if rank == 1 and step == fail_step:
                raise RuntimeError("injected failure of rank 1 (host side)")
            done += [(step, int(i)) for i in shards[rank]]
            board.heartbeat(step)
        except RuntimeError as e:
            board.report_failure(repr(e), step)
            alive = False
            break
    board.publish("done", json.dumps(done))
    if rank == 0:
        res = board.collect("done", range(world))
        print(json.dumps({"done": {str(r): json.loads(v) for r, v in res.items()}, "n": len(lengths), "steps": steps}))
    else:
        board.collect("done", [0])                     # keep the store's clients alive until rank 0 has everything
    time.sleep(0.2)
""") % ROOT


def test_three_ranks_one_fails_between_steps(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    procs = []
    for rank in range(3):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="3", MASTER_ADDR="127.0.0.1", MASTER_PORT="29561")
        procs.append(subprocess.Popen([sys.executable, str(script)], stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                                      text=True, env=env, cwd=ROOT))
    outs = [p.communicate(timeout=300) for p in procs]
    for p, (o, e) in zip(procs, outs):
        assert p.returncode == 0, o + e
    d = json.loads([l for l in outs[0][0].splitlines() if l.startswith("{")][-1])
    n, steps = d["n"], d["steps"]
    count = {}
    for r, pairs in d["done"].items():
        for step, seq in pairs:
            count[(step, seq)] = count.get((step, seq), 0) + 1
    # every sequence was run exactly once in every step, failure or not
    assert sorted(count) == [(s, i) for s in range(steps) for i in range(n)]
    assert set(count.values()) == {1}
    # rank 1 did steps 0 and 1 only; after that the others carried its sequences
    assert {s for s, _ in d["done"]["1"]} == {0, 1}
    assert len([1 for s, _ in d["done"]["0"] if s == 3]) + len([1 for s, _ in d["done"]["2"] if s == 3]) == n
