"""Process-group tables of the 3D grid (pure function, no processes)."""
import pytest


def test_sixteen_ranks_tp2_pp4_tables():
    """16 GPUs, TP 2, PP 4 (the layout example documented for Megatron-style grids): DP = 2."""
    from easyllm_b200.parallel.grid import grid_layout
    g = grid_layout(16, tp=2, pp=4)
    assert (g.tp, g.pp, g.dp) == (2, 4, 2)
    assert g.dp_groups == [[0, 2], [1, 3], [4, 6], [5, 7], [8, 10], [9, 11], [12, 14], [13, 15]]
    assert g.tp_groups == [[0, 1], [2, 3], [4, 5], [6, 7], [8, 9], [10, 11], [12, 13], [14, 15]]
    assert g.pp_groups == [[0, 4, 8, 12], [1, 5, 9, 13], [2, 6, 10, 14], [3, 7, 11, 15]]
    assert g.emb_groups == [[0, 12], [1, 13], [2, 14], [3, 15]]
    assert g.mp_groups == [[0, 1, 4, 5, 8, 9, 12, 13], [2, 3, 6, 7, 10, 11, 14, 15]]
    # rank = pp * (DP * TP) + dp * TP + tp
    for rank in range(16):
        pp, dp, tp = g.coords(rank)
        assert rank == pp * 4 + dp * 2 + tp


def test_every_rank_is_in_exactly_one_group_of_each_kind():
    from easyllm_b200.parallel.grid import grid_layout
    for world, tp, pp in ((8, 2, 1), (8, 4, 2), (8, 8, 1), (8, 1, 1), (12, 2, 3), (4, 1, 4)):
        g = grid_layout(world, tp, pp)
        for groups in (g.dp_groups, g.tp_groups, g.pp_groups, g.mp_groups):
            flat = sorted(r for grp in groups for r in grp)
            assert flat == list(range(world)), (world, tp, pp)
        assert all(len(grp) == g.dp for grp in g.dp_groups) and all(len(grp) == tp for grp in g.tp_groups)
        assert all(len(grp) == pp for grp in g.pp_groups)
    with pytest.raises(ValueError):
        grid_layout(6, tp=4, pp=1)
    clamped = grid_layout(2, tp=8, pp=1)                  # sizes larger than the world are clamped, as in the reference
    assert (clamped.tp, clamped.dp) == (2, 1)
