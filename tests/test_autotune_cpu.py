"""Autotuner host logic with a scripted timer and a dummy kernel (no GPU)."""

import json
from types import SimpleNamespace
from unittest.mock import patch

import pytest
import torch

from helpers import make_graph, random_edges
from turbo_gnn_b200._autotune import (
    AutotuneConfig,
    TunableKernel,
    TunableParam,
    _build_combinations,
    _InlineAutotuneCache,
    with_autotune,
)
from turbo_gnn_b200._kernels import GATv2AggrKernel, GraphTransformerAggrKernel, ReductionAggrKernel


class Doubler(TunableKernel):
    """x * factor; `speed` is the tunable whose value the scripted timer rewards."""

    def __init__(self, factor=2):
        super().__init__()
        self.factor = factor
        self.speed = 0
        self.calls = []

    def _execute(self, graph, x, **kwargs):
        if self.speed == 13:
            raise RuntimeError("Wrong int value")
        self.calls.append((graph, self.speed))
        return x * self.factor

    def get_tunable_forward_kernel_params(self):
        return [TunableParam("speed", [1, 13, 5, 3], default=0)]

    def get_tunable_forward_graph_params(self):
        return [TunableParam("forward_huge_degree_threshold_quantile", [-1, 0.5], default=-1)]


def scripted_timer(kernel):
    def fake(fn, warmup=10, iters=50):
        fn()  # invalid configurations raise here, like a real timed call
        graph, speed = kernel.calls[-1]
        ms = 10.0 / speed + (0.0 if graph.forward_heavy_nodes.numel() else 0.5)
        return SimpleNamespace(iters=iters, ms_per_iter=ms)

    return fake


@pytest.fixture(autouse=True)
def _fresh_singletons():
    TunableKernel._shared_instances.clear()
    yield
    TunableKernel._shared_instances.clear()


@pytest.fixture
def graph():
    return make_graph(random_edges(60, 500, 4), 60, torch.int64, quantile=0.9, device="cpu")


def test_build_combinations():
    assert _build_combinations([]) == [{}]
    combos = _build_combinations([TunableParam("a", [1, 2], 1), TunableParam("b", ["x"], "x")])
    assert combos == [{"a": 1, "b": "x"}, {"a": 2, "b": "x"}]


def test_inline_autotune_picks_fastest_and_skips_invalid(graph):
    k = Doubler()
    x = torch.ones(60, 4)
    with patch("turbo_gnn_b200._timer.time_callable", scripted_timer(k)):
        result = k._inline_autotune(x, graph, AutotuneConfig(warmup=1, iters=1))
    assert result["kernel_config"] == {"speed": 5}
    assert result["graph_repr"].forward_heavy_nodes.numel() > 0  # the 0.5-quantile split won
    assert k.speed == 5 and k._is_autotuning is False and k._is_tuned


def test_call_with_autotune_caches_per_graph_and_feature_width(graph):
    k = Doubler()
    x = torch.ones(60, 4)
    with patch("turbo_gnn_b200._timer.time_callable", scripted_timer(k)) as _:
        out = k(graph, x, autotune=True, autotune_config=AutotuneConfig(1, 1))
        assert torch.equal(out, x * 2)
        tuned_calls = len(k.calls)
        k(graph, x, autotune=True)
        assert len(k.calls) == tuned_calls + 1  # cache hit: one execution, no search
        k(graph, torch.ones(60, 8), autotune=True, autotune_config=AutotuneConfig(1, 1))
        assert len(k.calls) > tuned_calls + 2  # other feature width: searched again
    assert torch.equal(k(graph, x), x * 2)  # plain call path


def test_cache_tiers():
    cache = _InlineAutotuneCache()
    g = make_graph(random_edges(30, 100, 1), 30, torch.int64, device="cpu")
    assert cache.lookup(g, 16) is None
    cache.store(g, 16, {"kernel_config": {"a": 1}, "graph_repr": g})
    assert cache.lookup(g, 16)["kernel_config"] == {"a": 1}
    assert cache.lookup(g, 32) is None
    g.forward_indptr = g.forward_indptr.clone()  # same object, other CSR storage
    assert cache.lookup(g, 16) is None


def test_with_autotune_decorator_routes_init_and_exec_kwargs(graph):
    seen = {}

    class Scaled(Doubler):
        def _execute(self, graph, x, **kwargs):
            seen.update(kwargs)
            return super()._execute(graph, x)

    @with_autotune(Scaled, init_params=("factor",))
    def op(graph, x, bias=0, factor=2):
        return x * factor + bias

    x = torch.ones(60, 4)
    assert torch.equal(op(graph, x, bias=1, factor=3), x * 3 + 1)  # autotune off: the function itself
    inst = Scaled._get_or_create(factor=3)
    with patch("turbo_gnn_b200._timer.time_callable", scripted_timer(inst)):
        out = op(graph, x, bias=1, factor=3, autotune=True, autotune_config=AutotuneConfig(1, 1))
    assert torch.equal(out, x * 3)
    assert seen == {"bias": 1}  # init kwargs are not forwarded to _execute
    assert Scaled._get_or_create(factor=3) is inst and Scaled._get_or_create(factor=4) is not inst


def test_disk_cache_round_trip(graph, tmp_path):
    cfg = AutotuneConfig(warmup=1, iters=1, cache_dir=str(tmp_path))
    x = torch.ones(60, 4)
    k = Doubler()
    with patch("turbo_gnn_b200._timer.time_callable", scripted_timer(k)):
        k._inline_autotune(x, graph, cfg)
    files = list(tmp_path.glob("Doubler_*.json"))
    assert len(files) == 1
    saved = json.loads(files[0].read_text())
    assert saved["kernel_config"] == {"speed": 5} and saved["graph_config"] == {
        "forward_huge_degree_threshold_quantile": 0.5}
    fresh = Doubler()

    def boom(*a, **k):
        raise AssertionError("the search must not run when a disk entry exists")

    with patch("turbo_gnn_b200._timer.time_callable", boom):
        result = fresh._inline_autotune(x, graph, cfg)
    assert fresh.speed == 5 and result["graph_repr"].forward_heavy_nodes.numel() > 0


def test_kernel_classes_expose_reference_attribute_names():
    r = ReductionAggrKernel(reduce="max", warps_per_block=4)
    assert (r.reduce, r.forward_warps_per_block, r.forward_edges_per_block_heavy_nodes) == ("max", 4, 128)
    assert {p.name for p in r.get_tunable_forward_graph_params()} == {"forward_huge_degree_threshold_quantile"}
    g = GATv2AggrKernel(forward_light_warps=2)
    assert g.forward_light_warps == 2 and g.backward_grad_A_reduce_row_chunk_size == 512
    assert "forward_heavy_warps" in {p.name for p in g.get_tunable_forward_kernel_params()}
    t = GraphTransformerAggrKernel()
    assert (t.forward_light_warps, t.forward_heavy_warps, t.backward_light_warps) == (4, 8, 1)
    assert {p.name for p in t.get_tunable_backward_graph_params()} == {"backward_huge_degree_threshold_quantile"}
    assert ReductionAggrKernel._get_or_create(reduce="min") is not ReductionAggrKernel._get_or_create(reduce="max")


# ---- search strategies (host logic) ---------------------------------------------------------------


def _objective(cfg):
    # separable with one interaction; unique minimum at a=3, b="x", c=16, d=2
    return abs(cfg["a"] - 3) * 2.0 + (0.0 if cfg["b"] == "x" else 1.5) + abs(cfg["c"] - 16) / 8 + (cfg["d"] - 2) ** 2 \
        + (0.7 if (cfg["a"] == 3 and cfg["b"] == "y") else 0.0)


_SPACE = {"a": [0, 1, 2, 3, 4, 5], "b": ["x", "y", "z"], "c": [1, 2, 4, 8, 16, 32], "d": [0, 1, 2, 3, 4]}


def test_grid_search_visits_every_combination_once():
    from turbo_gnn_b200._search import GridSearch

    grid = GridSearch(_SPACE)
    seen = []
    while (cfg := grid.ask()) is not None:
        seen.append(tuple(cfg.values()))
        grid.tell(cfg, _objective(cfg))
    assert grid.size == 6 * 3 * 6 * 5 == len(seen) == len(set(seen))
    assert grid.best()[0] == {"a": 3, "b": "x", "c": 16, "d": 2}


def test_tpe_finds_the_optimum_in_a_fraction_of_the_grid_and_is_reproducible():
    from turbo_gnn_b200._search import TPESearch

    def run(seed):
        tpe = TPESearch(_SPACE, seed=seed, n_startup=10)
        asked = []
        for _ in range(120):  # grid: 540
            cfg = tpe.ask()
            assert cfg is not None
            asked.append(tuple(cfg.values()))
            tpe.tell(cfg, _objective(cfg) if cfg["d"] != 4 else float("inf"))  # d=4: an invalid launch parameter
        assert len(set(asked)) == len(asked)  # never the same combination twice
        return asked, tpe.best()

    asked, best = run(0)
    assert best[1] <= 0.5 and best[0]["a"] == 3 and best[0]["b"] == "x"
    assert run(0)[0] == asked  # same seed, same trajectory
    hits = sum(run(s)[1][1] == 0.0 for s in range(5))
    assert hits >= 3  # the exact optimum in most runs with 22 % of the grid


def test_tpe_exhausts_small_spaces_and_then_stops():
    from turbo_gnn_b200._search import TPESearch, make_search

    tpe = TPESearch({"p": [1, 2], "q": ["a", "b", "c"]}, seed=1, n_startup=2)
    got = []
    while (cfg := tpe.ask()) is not None:
        got.append((cfg["p"], cfg["q"]))
        tpe.tell(cfg, float(cfg["p"]))
    assert sorted(got) == [(p, q) for p in (1, 2) for q in "abc"]
    assert type(make_search("tpe", {"p": [1, 2]}, max_trials=8)).__name__ == "GridSearch"  # max_trials covers the grid
    assert type(make_search("tpe", _SPACE, max_trials=50)).__name__ == "TPESearch"
    with pytest.raises(ValueError):
        make_search("anneal", _SPACE, max_trials=5)


def test_autotune_with_tpe_trial_limit_and_trial_records(tmp_path):
    graph = make_graph(random_edges(60, 500, 3), 60, device="cpu")
    kern = Doubler()
    x = torch.ones(60, 8)
    cfg = AutotuneConfig(warmup=0, iters=1, cache_dir=str(tmp_path), search="tpe", max_trials=5, seed=3)
    with patch("turbo_gnn_b200._autotune._timer.time_callable", scripted_timer(kern)):
        kern._inline_autotune(x, graph, cfg)
    records = list((tmp_path / "trials").glob("*.json"))
    assert len(records) == 5  # one JSON record per timed trial, failures included
    timed = len(kern.calls)
    # a second search with the same seed replays the records instead of timing again
    kern2 = Doubler()
    with patch("turbo_gnn_b200._autotune._timer.time_callable", scripted_timer(kern2)):
        import os

        for f in tmp_path.glob("Doubler_*.json"):
            os.remove(f)  # drop the winner file so that the search itself runs again
        kern2._inline_autotune(x, graph, cfg)
    assert len(kern2.calls) == 0 and timed >= 4
    assert kern2.speed == kern.speed
