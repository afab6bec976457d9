"""CPU: sequence sharding over GPUs and micro-batching (bytetransformer_b200/sharding.py)."""
import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

from bytetransformer_b200.sharding import lpt_shards, micro_batches, sequence_cost
from bytetransformer_b200.workloads import BERT_BASE, lengths_for, total_flops


def test_whole_box_workload_is_seeded_and_sized():
    l = lengths_for("whole_box_1024x1024")
    assert len(l) == 1024 and l.min() >= 16 and l.max() <= 1024
    assert int(l.sum()) == 556500                       # pinned: the bench reports this token count
    assert np.array_equal(l, lengths_for("whole_box_1024x1024"))
    assert abs(total_flops(l, BERT_BASE) / 1e12 - 108.8) < 0.1


@pytest.mark.parametrize("n", [1, 2, 4, 8])
def test_lpt_shards_partition_and_balance(n):
    l = lengths_for("whole_box_1024x1024")
    shards = lpt_shards(l, n)
    allidx = np.concatenate(shards)
    assert sorted(allidx.tolist()) == list(range(1024))           # every sequence exactly once
    cost = [sequence_cost(l[s]).sum() for s in shards]
    assert max(cost) / (sum(cost) / n) < 1.005                    # <= 0.5 % imbalance -> >= 7.9x of 8x possible


@given(st.lists(st.integers(0, 1024), min_size=1, max_size=200), st.integers(1, 8))
@settings(max_examples=60, deadline=None)
def test_lpt_property(lengths, n):
    shards = lpt_shards(lengths, n)
    assert len(shards) == n
    assert sorted(np.concatenate(shards).tolist()) == list(range(len(lengths)))


@given(st.lists(st.integers(0, 1024), min_size=1, max_size=300), st.integers(1024, 20000))
@settings(max_examples=60, deadline=None)
def test_micro_batches_property(lengths, budget):
    ids = list(range(len(lengths)))
    mbs = micro_batches(lengths, ids, budget)
    seen = np.concatenate([mb.seq_ids for mb in mbs]).tolist()
    assert sorted(seen) == ids                                     # nothing lost, nothing duplicated
    for mb in mbs:
        ls = np.asarray(lengths)[mb.seq_ids]
        assert mb.tokens == int(ls.sum()) <= budget
        assert mb.cu_seqlens.dtype == np.int32 and mb.cu_seqlens[0] == 0
        assert np.array_equal(np.diff(mb.cu_seqlens), ls)
        assert mb.max_len == (int(ls.max()) if len(ls) else 0)


def test_micro_batch_rejects_oversized_sequence():
    with pytest.raises(ValueError):
        micro_batches([5000], [0], 4096)


def test_token_budget_grows_with_the_rank_s_tokens_but_keeps_several_micro_batches():
    from bytetransformer_b200.runner import TOKEN_BUDGET_UNIT, pick_token_budget
    assert pick_token_budget(0) == TOKEN_BUDGET_UNIT
    assert pick_token_budget(10_000) == TOKEN_BUDGET_UNIT
    # the benchmark workload on 1 / 2 / 4 / 8 GPUs
    assert pick_token_budget(556_500) == 4 * TOKEN_BUDGET_UNIT
    assert pick_token_budget(278_250) == 4 * TOKEN_BUDGET_UNIT
    assert pick_token_budget(139_125) == 2 * TOKEN_BUDGET_UNIT
    assert pick_token_budget(69_563) == TOKEN_BUDGET_UNIT
    for total in (556_500, 278_250, 139_125, 69_563, 10_000_000):
        b = pick_token_budget(total)
        assert -(-total // b) >= 4
        # inputs resident in device memory (nothing to overlap): the largest launch whatever the total
        assert pick_token_budget(total, min_batches=1) == 4 * TOKEN_BUDGET_UNIT
