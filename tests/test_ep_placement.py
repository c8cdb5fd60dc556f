"""Host logic of the expert placement used by the peer-memory expert-parallel path:
every expert is served by exactly one rank or replicated on all of them, local indices are
dense, the sharded experts come first, and a skewed load ends up balanced."""
import importlib

import numpy as np
import pytest


@pytest.fixture(scope="module")
def ep():
    return importlib.import_module("qwen4-thor_b200.ep")


def _zipf_counts(E, rows, s, seed):
    rng = np.random.default_rng(seed)
    p = 1.0 / np.arange(1, E + 1) ** s
    p /= p.sum()
    counts = np.minimum(rng.multinomial(rows, p), rows // 10)   # top-k routing caps an expert at one row per token
    return counts[rng.permutation(E)]


@pytest.mark.parametrize("world,hot", [(2, 0), (2, 32), (4, 16), (8, 32), (8, 0)])
def test_placement_tables_are_consistent(ep, world, hot):
    E = 512
    counts = _zipf_counts(E, 327680, 1.1, seed=world + hot)
    experts, tables = ep.plan_placement(counts, world, hot)
    REPL = 1 << 30
    hot_set = set(np.argsort(-counts, kind="stable")[:hot].tolist())
    for r in range(world):
        t = tables[r]
        assert t.dtype == np.int32 and t.shape == (E,)
        served = [e for e in range(E) if t[e] >= 0]
        assert sorted(served) == sorted(experts[r])
        # local indices are dense and follow the list order; replicated experts come last
        for idx, e in enumerate(experts[r]):
            assert (t[e] & ~REPL) == idx
            assert bool(t[e] & REPL) == (e in hot_set)
        assert all(e in hot_set for e in experts[r][len(experts[r]) - hot:])
    for e in range(E):
        owners = [r for r in range(world) if tables[r][e] >= 0]
        assert len(owners) == (world if e in hot_set else 1)


def test_replication_balances_a_skewed_router(ep):
    """Three experts that nearly every token selects cannot be spread evenly over two ranks by
    sharding; replicated, their rows stay with the tokens' ranks."""
    world = 2
    counts = np.array([1000, 1000, 1000] + [10] * 13)

    def worst_over_mean(hot):
        experts, _ = ep.plan_placement(counts, world, hot)
        hot_set = set(np.argsort(-counts, kind="stable")[:hot].tolist())
        # rows of a replicated expert stay with the token's rank: an even share each
        load = [sum(counts[e] / world if e in hot_set else counts[e] for e in lst) for lst in experts]
        return max(load) / (sum(load) / world)

    assert worst_over_mean(0) > 1.25
    assert worst_over_mean(3) < 1.01


@pytest.mark.parametrize("world,hot", [(2, 3), (8, 32), (4, 0)])
def test_owner_table_matches_placement(ep, world, hot):
    """The table the selective publish step uses: a sharded expert names its one serving rank,
    a replicated expert is marked -1 (served where the token lives)."""
    E = 512
    counts = _zipf_counts(E, 100000, 1.1, seed=7 * world + hot)
    experts, tables = ep.plan_placement(counts, world, hot)
    owner = ep.owner_table(tables)
    assert owner.dtype == np.int32 and owner.shape == (E,)
    REPL = 1 << 30
    for e in range(E):
        serving = [r for r in range(world) if tables[r][e] >= 0]
        if tables[0][e] >= 0 and tables[0][e] & REPL:
            assert owner[e] == -1 and len(serving) == world
        else:
            assert serving == [int(owner[e])]
    assert int((owner < 0).sum()) == hot
