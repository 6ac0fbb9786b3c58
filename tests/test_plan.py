"""Static sharding plan: every leaf placed exactly once, expert leaves sharded by expert, owners balanced by optimizer cost."""

import math

import pytest

from lyra_b200.parallel.runtime import Plan, _owner_cost
from lyra_b200.variants import model_variant


@pytest.mark.parametrize("world", [2, 4, 8])
def test_lyra_medium_plan_is_complete_and_balanced(world):
    m = model_variant("lyra-medium")
    plan = Plan.build(m, world)
    paths = set(plan.specs)
    assert set(plan.owner) | plan.replicated | plan.expert == paths
    assert not (set(plan.owner) & plan.replicated) and not (set(plan.owner) & plan.expert) and not (plan.replicated & plan.expert)
    assert all(p.split("/")[-1].startswith(("mlp_up", "mlp_down")) for p in plan.expert)
    cost = [0.0] * world
    for path, r in plan.owner.items():
        cost[r] += _owner_cost(path, plan.specs[path])
    assert max(cost) / min(cost) < 1.05, cost            # Newton-Schulz time per owner within 5 %
    # the two embedding tables (Adam, cheap) must not count like Muon matrices of the same size
    emb_owner = {r for p, r in plan.owner.items() if p.split("/")[-1] in ("emb", "unemb")}
    sizes = [sum(math.prod(plan.specs[p].shape) for p, r in plan.owner.items() if r == k) for k in range(world)]
    if world >= 4:
        assert max(sizes[r] for r in emb_owner) == max(sizes)


def test_single_rank_plan_replicates_everything():
    plan = Plan.build(model_variant("tiny"), 1)
    assert not plan.owner and not plan.expert and plan.replicated == set(plan.specs)
