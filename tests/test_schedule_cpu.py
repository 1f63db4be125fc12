"""The three-tier schedule: every edge of every row is covered exactly once."""

import pytest
import torch

from helpers import make_graph, random_edges
from turbo_gnn_b200 import _schedule


@pytest.mark.parametrize("chunk,hub_min", [(32, 64), (64, 100), (2048, 4096)])
def test_tiers_partition_rows_and_chunks_cover_hub_rows(chunk, hub_min):
    n = 400
    ei = random_edges(n, 4000, 3, hubs=3, hub_degree=350)
    g = make_graph(ei, n, torch.int32, quantile=0.9, device="cpu")
    s = _schedule.split_tiers(g.forward_indptr, g.forward_light_nodes, g.forward_heavy_nodes, chunk, hub_min)
    rows = torch.cat([s.light, s.heavy, s.hub]).long()
    assert sorted(rows.tolist()) == list(range(n))
    ptr = g.forward_indptr.long()
    deg = ptr[1:] - ptr[:-1]
    assert bool((deg[s.hub.long()] >= hub_min).all()) and bool((deg[s.heavy.long()] < hub_min).all())
    assert s.hub_part_ptr[0].item() == 0 and s.hub_part_ptr[-1].item() == s.num_chunks == s.chunk_hub.numel()
    covered = torch.zeros(int(ptr[-1]), dtype=torch.int32)
    for c in range(s.num_chunks):
        k = int(s.chunk_hub[c])
        row = int(s.hub[k])
        e0 = int(ptr[row]) + (c - int(s.hub_part_ptr[k])) * chunk
        e1 = min(e0 + chunk, int(ptr[row + 1]))
        assert e0 < e1
        covered[e0:e1] += 1
    for row in s.hub.tolist():
        assert bool((covered[int(ptr[row]): int(ptr[row + 1])] == 1).all())
    # light rows are ordered longest first
    ld = deg[s.light.long()]
    assert bool((ld[:-1] >= ld[1:]).all())


def test_cache_hits_on_same_tensors_and_misses_on_new_ones():
    n = 100
    g = make_graph(random_edges(n, 800, 1), n, torch.int64, quantile=0.9, device="cpu")
    a = _schedule.get_schedule(g.forward_indptr, g.forward_light_nodes, g.forward_heavy_nodes)
    b = _schedule.get_schedule(g.forward_indptr, g.forward_light_nodes, g.forward_heavy_nodes)
    assert a is b
    c = _schedule.get_schedule(g.forward_indptr, g.forward_light_nodes, g.forward_heavy_nodes, chunk_edges=64)
    assert c is not a
    r = g.repartition(forward_huge_degree_threshold_quantile=0.5)
    d = _schedule.get_schedule(r.forward_indptr, r.forward_light_nodes, r.forward_heavy_nodes)
    assert d is not a


def test_automatic_thresholds_follow_the_work_per_warp_slot():
    chunk, hub_min, cta_min = _schedule.auto_thresholds(114_000_000, torch.device("cpu"))
    fair = 114_000_000 // (148 * 16)
    assert cta_min == fair // 2 and hub_min == 4 * fair and chunk % 32 == 0 and 1024 <= chunk <= 32768
    chunk, hub_min, cta_min = _schedule.auto_thresholds(10_000, torch.device("cpu"))
    assert (chunk, hub_min, cta_min) == (1024, 2048, 64)
    # small graph: every heavy-list row is shorter than cta_min_degree and runs warp-per-row
    n = 300
    g = make_graph(random_edges(n, 3000, 5, hubs=2, hub_degree=200), n, torch.int32, quantile=0.9, device="cpu")
    s = _schedule.split_tiers(g.forward_indptr, g.forward_light_nodes, g.forward_heavy_nodes)
    assert s.heavy.numel() == 2 and s.hub.numel() == 0 and s.light.numel() == n - 2  # only the two long rows get CTAs
    # explicit thresholds restore the plain light / heavy / hub split
    s = _schedule.split_tiers(g.forward_indptr, g.forward_light_nodes, g.forward_heavy_nodes, 64, 100)
    assert s.light.numel() == g.forward_light_nodes.numel() and s.hub.numel() == 2
    s = _schedule.split_tiers(g.forward_indptr, g.forward_light_nodes, g.forward_heavy_nodes, 64, 100,
                              cta_min_degree=50)
    assert s.light.numel() > g.forward_light_nodes.numel() and s.hub.numel() == 2


def test_bad_chunk_size_raises_runtime_error():
    g = make_graph(random_edges(50, 300, 2), 50, torch.int32, device="cpu")
    with pytest.raises(RuntimeError):
        _schedule.split_tiers(g.forward_indptr, g.forward_light_nodes, g.forward_heavy_nodes, chunk_edges=48)


def test_auto_tiles_rule():
    from turbo_gnn_b200 import _schedule as S

    # 233k nodes x 2 KB gathered per edge, mean degree 492: 477 MB -> 8 tiles
    assert S.auto_tiles(232_965, 232_965, 114_585_574, 2048) == 8
    # the same graph cut into 8 row shards keeps the column footprint and the row length
    assert S.auto_tiles(28_673, 8 * 29_344, 14_321_060, 2048) == 8
    # short rows, or a gathered matrix that fits L2: one pass
    assert S.auto_tiles(169_343, 169_343, 2_460_000, 2048) == 1
    assert S.auto_tiles(20_000, 20_000, 10_000_000, 2048) == 1
    assert S.auto_tiles(4_194_304, 4_194_304, 65_000_000, 512) == 1
    assert S.auto_tiles(0, 10, 0, 2048) == 1
    # one gathered 1 KB row per edge on the same graph (238 MB): 4 tiles
    assert S.auto_tiles(232_965, 232_965, 114_585_574, 1024) == 4


def test_tile_table_on_host():
    import torch
    from turbo_gnn_b200 import _schedule as S

    indptr = torch.tensor([0, 3, 3, 7, 8], dtype=torch.int32)
    indices = torch.tensor([0, 5, 9, 1, 2, 3, 8, 4], dtype=torch.int32)
    table = S.build_tile_ptr(indptr, indices, 10, 2).view(3, 4)  # tiles [0,5) and [5,10)
    assert table.dtype == torch.int32
    assert table.tolist() == [[0, 3, 3, 7], [1, 3, 6, 8], [3, 3, 7, 8]]
    sched = S.split_tiers(indptr, torch.arange(4, dtype=torch.int32), torch.zeros(0, dtype=torch.int32))
    same = S.with_column_tiles(sched, indptr, indices, 10, 2048, tiles=1)
    assert same is sched and same.num_tiles == 1
    tiled = S.with_column_tiles(sched, indptr, indices, 10, 2048, tiles=2)
    assert tiled.num_tiles == 2 and tiled.tile_ptr.numel() == 12 and tiled.light is sched.light
