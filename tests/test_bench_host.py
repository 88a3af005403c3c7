"""Host-side pieces of the benchmarks (no GPU): the puzzle bench.py builds itself, and the exchange schedules the
collective benchmark times."""
import numpy as np
import pytest

import bench
import bench_collective
import bench_optimizer
import bench_variants


def test_bench_builds_the_trainers_cyclic_puzzle(oracle):
    # bench.py must not import the oracle on its product path, so it restates the built-in puzzle (tool:117-140)
    for state_len, moves in ((72, 18), (24, 5)):
        m, t = bench.cyclic_puzzle(state_len, moves)
        om, ot = oracle.cyclic_puzzle(state_len, moves)
        assert np.array_equal(m, om) and np.array_equal(t, ot)


def test_collective_schedules_cover_every_parameter_once():
    params = 15460289
    bucket = (4 << 20) // 4
    ranges, launches = bench_collective.p888_schedule(bucket)
    assert len(ranges) == 35 and len(launches) == 47           # the reference trainer's schedule at 4 MB buckets
    assert ranges[0][0] + ranges[0][1] == params and ranges[-1] == (0, 72 * 72 * 2560 + 2560)
    for chosen in (launches, sum(bench_collective.trainer_schedule(bucket), [])):
        covered = sorted(chosen)
        assert covered[0][0] == 0 and sum(c for _, c in covered) == params
        assert all(covered[i][0] + covered[i][1] == covered[i + 1][0] for i in range(len(covered) - 1))
    early, fused = bench_collective.trainer_schedule(bucket)
    assert early == [ranges[-1]] and len(fused) == 4 and all(c <= bucket for _, c in fused)


def test_variant_table_is_consistent():
    for name, v in bench_variants.VARIANTS.items():
        s = v["shape"]
        assert s["state_len"] == 72 and s["hd1"] <= 4096 and s["hd2"] <= 512 and s["residual_blocks"] <= 32, name
        assert not v["cross_entropy"] or s["output_dim"] >= 29          # one logit per walk depth 1..29


def test_optimizer_bench_gradient_kinds():
    n = 100000
    g = bench_optimizer.gradient("normal", n)
    assert g.dtype == np.float32 and np.isfinite(g).all() and np.abs(g).max() <= 1e-4
    z = bench_optimizer.gradient("half_of_columns_zero", n)
    frac = float((z == 0).mean())
    assert 0.4 < frac < 0.6
    rows = n // 2560
    zero_cols = (z[:rows * 2560].reshape(rows, 2560) == 0).all(axis=0)  # whole columns, not scattered elements
    assert 0.4 < float(zero_cols.mean()) < 0.6
    live = np.tile(~zero_cols, rows)
    assert np.array_equal(z[:rows * 2560][live], g[:rows * 2560][live])
    assert not bench_optimizer.gradient("all_zero", n).any()
    d = bench_optimizer.gradient("zeros_and_denormals", n)
    tiny = np.float32(1.1754944e-38)
    assert (np.signbit(d) & (d == 0)).any() and ((np.abs(d) > 0) & (np.abs(d) < tiny)).any()
    with pytest.raises(ValueError):
        bench_optimizer.gradient("other", 8)
