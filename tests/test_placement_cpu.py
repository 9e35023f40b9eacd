"""Replica placement for skewed expert loads (host arithmetic, no GPU)."""

import pytest

from b12x_b200.moe.placement import PATTERN, plan_expert_replicas


def _zipf(n, s=1.2):
    return [1.0 / (i + 1) ** s for i in range(n)]


@pytest.mark.parametrize("world,experts", [(8, 8), (4, 8), (2, 8), (8, 64), (4, 128)])
def test_plan_flattens_zipf_loads_and_is_consistent(world, experts):
    loads = _zipf(experts)
    total = sum(loads)
    frac = [x / total for x in loads]
    per = experts // world
    before = max(sum(frac[r * per:(r + 1) * per]) for r in range(world)) * world
    plan = plan_expert_replicas(loads, world, 1)
    after = max(plan.rank_loads(frac)) * world
    assert after <= before + 1e-9
    assert after - 1.0 < 0.4 * (before - 1.0)          # one spare slot per rank removes most of the imbalance
    if experts == 8:
        assert after < 1.15
    ranks, local = plan.pattern_tables()
    assert len(ranks) == len(local) == experts * PATTERN
    for e, holders in enumerate(plan.holders):
        assert sum(h[2] for h in holders) == PATTERN and all(h[2] > 0 for h in holders)
        assert holders[0][0] == e // per and holders[0][1] == e % per           # the owner keeps a share
        assert len({h[0] for h in holders}) == len(holders)                       # one entry per rank
        for rank, slot, _share in holders[1:]:
            assert plan.extra[rank][slot - per] == e                              # copies sit in the spare slots
        row = list(zip(ranks[e * PATTERN:(e + 1) * PATTERN], local[e * PATTERN:(e + 1) * PATTERN]))
        for rank, slot, share in holders:
            assert row.count((rank, slot)) == share
    assert all(len(x) <= 1 for x in plan.extra)


def test_uniform_loads_need_no_copies_and_no_slots_means_no_copies():
    plan = plan_expert_replicas([1.0] * 16, 4, 2)
    assert all(len(x) == 0 for x in plan.extra)
    assert all(h == ((e // 4, e % 4, PATTERN),) for e, h in enumerate(plan.holders))
    plan = plan_expert_replicas(_zipf(8), 8, 0)
    assert all(len(x) == 0 for x in plan.extra)
    with pytest.raises(ValueError):
        plan_expert_replicas([1.0] * 7, 2, 1)


def test_same_loads_give_the_same_plan():
    a = plan_expert_replicas(_zipf(8), 8, 1)
    b = plan_expert_replicas(_zipf(8), 8, 1)
    assert a == b
