"""Native planners: pipeline schedules, static memory plan, strategy search."""
import numpy as np
import pytest

from mindspore_b200.parallel import planner as P


def _check_schedule(steps, micro, chunks=1):
    fwd = [(m, c) for k, m, c in steps if k == P.FORWARD]
    bwd = [(m, c) for k, m, c in steps if k == P.BACKWARD]
    assert sorted(fwd) == sorted(bwd) == sorted((m, c) for m in range(micro) for c in range(chunks))
    seen = set()
    for k, m, c in steps:
        if k == P.FORWARD:
            seen.add((m, c))
        else:
            assert (m, c) in seen, "backward before forward"


def test_gpipe_and_1f1b_orders():
    g = P.pipeline_schedule(4, 0, 8, scheduler="gpipe")
    assert [s[0] for s in g] == [0] * 8 + [1] * 8
    for stage in range(4):
        s = P.pipeline_schedule(4, stage, 8, scheduler="1f1b")
        _check_schedule(s, 8)
        assert P.pipeline_peak_activations(s) == 4 - stage      # 1F1B bounds live activations by stages - stage
        assert P.pipeline_peak_activations(P.pipeline_schedule(4, stage, 8, scheduler="gpipe")) == 8
    last = P.pipeline_schedule(4, 3, 4)
    assert last == [(0, 0, 0), (1, 0, 0), (0, 1, 0), (1, 1, 0), (0, 2, 0), (1, 2, 0), (0, 3, 0), (1, 3, 0)]


def test_interleaved_schedule():
    for stage in range(2):
        s = P.pipeline_schedule(2, stage, 4, chunks=2)
        _check_schedule(s, 4, 2)
    with pytest.raises(ValueError):
        P.pipeline_schedule(4, 0, 6, chunks=2)
    with pytest.raises(ValueError):
        P.pipeline_schedule(2, 5, 4)


def test_memory_plan_reuses_and_never_overlaps():
    rng = np.random.RandomState(0)
    n = 200
    starts = rng.randint(0, 100, n)
    ends = starts + rng.randint(0, 20, n)
    sizes = (rng.randint(1, 64, n) * 1024).tolist()
    offs, total = P.memory_plan(sizes, starts.tolist(), ends.tolist())
    assert P.memory_plan_conflicts(sizes, starts.tolist(), ends.tolist(), offs) == 0
    assert total < sum(sizes) * 0.5           # lifetimes are short: the arena must be far below the plain sum
    assert all(o % 512 == 0 for o in offs)


def test_memory_plan_contiguity_group():
    sizes, starts, ends = [1000, 2000, 3000, 500], [0, 0, 0, 5], [3, 3, 3, 9]
    offs, total = P.memory_plan(sizes, starts, ends, groups=[7, 7, 7, -1], align=256)
    assert offs[1] == offs[0] + 1024 and offs[2] == offs[1] + 2048      # members back to back (aligned sizes)
    assert P.memory_plan_conflicts(sizes, starts, ends, offs) == 0


def test_chain_dp_matches_brute_force():
    rng = np.random.RandomState(3)
    ncand = [3, 4, 2, 5, 3]
    op = [rng.rand(n).tolist() for n in ncand]
    edge = [rng.rand(ncand[i], ncand[i + 1]).tolist() for i in range(len(ncand) - 1)]
    choice, total = P.chain_dp_search(op, edge)
    import itertools
    best = min(itertools.product(*[range(n) for n in ncand]),
               key=lambda c: sum(op[i][c[i]] for i in range(5)) + sum(edge[i][c[i]][c[i + 1]] for i in range(4)))
    assert tuple(choice) == best
    assert abs(total - (sum(op[i][best[i]] for i in range(5)) + sum(edge[i][best[i]][best[i + 1]] for i in range(4)))) < 1e-12


def test_sharding_propagation_follows_cheapest_edges():
    # chain 0 - 1 - 2 with node 0 pinned to candidate 1; identity-like costs make neighbours follow it
    cost = [[0.0 if a == b else 1.0 for b in range(3)] for a in range(3)]
    out = P.propagate_strategies([3, 3, 3], [1, -1, -1], [(0, 1), (1, 2)], [cost, cost])
    assert out == [1, 1, 1]
    out = P.propagate_strategies([3, 3, 3], [-1, -1, 2], [(0, 1), (1, 2)], [cost, cost])
    assert out == [2, 2, 2]
    assert P.propagate_strategies([2, 2], [-1, -1], [(0, 1)], [[[0, 1], [1, 0]]]) == [0, 0]
