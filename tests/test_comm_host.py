"""Host logic of the gradient exchange: range scheduling (pure Python) and a world_size-2 run over
gloo on CPU that checks the data-parallel result against a single-process computation."""
import os
import socket

import numpy as np
import pytest

from multigputrainmlp_b200.comm import GradientRangeScheduler


def p888_ranges():
    """The 35 gradient-ready ranges of the p888 model in notification order
    (native/cuda/mlp_backward.cu:1364,1385,1402,1427,1506)."""
    h1, h2, r, inp = 2560, 224, 16, 72 * 72
    in_w = inp * h1
    hidden = in_w + h1
    rbase = hidden + h1 * h2 + h2
    blk = 2 * (h2 * h2 + h2)
    out = [(rbase + r * blk, h2 + 1)]
    for k in range(r - 1, -1, -1):
        out.append((rbase + k * blk + h2 * h2 + h2, h2 * h2 + h2))
        out.append((rbase + k * blk, h2 * h2 + h2))
    out.append((hidden, h1 * h2 + h2))
    out.append((0, in_w + h1))
    return out


def run_scheduler(lag, bucket_bytes=4 << 20, whole_tail=True):
    launches, waits = [], []
    sched = GradientRangeScheduler(lambda off, cnt: launches.append((off, cnt)), lambda: waits.append(len(launches)),
                                   bucket_params=bucket_bytes // 4, expected_ranges=35, lag=lag, whole_tail=whole_tail)
    sched.begin_step()
    seen_before = []
    for i, (off, cnt) in enumerate(p888_ranges()):
        assert sched.on_ready(i, off, cnt) == 0
        seen_before.append(len(launches))
    sched.finish()
    return sched, launches, waits, seen_before


def test_schedule_matches_reference_chunking():
    sched, launches, waits, _ = run_scheduler(lag=0, whole_tail=False)
    # 35 ranges; at 4 MiB buckets the embedding range (13 273 600 floats) needs 13 chunks: 47 launches
    assert sched.scheduled_ranges == 35 and sched.scheduled_chunks == 47 == len(launches)
    assert launches[0] == (15460064, 225)
    assert launches[-13][0] == 0 and sum(c for _, c in launches[-13:]) == 72 * 72 * 2560 + 2560
    assert all(c <= (4 << 20) // 4 for _, c in launches)
    assert sum(c for _, c in launches) == 15460289  # every parameter exactly once
    covered = sorted(launches)
    assert all(covered[i][0] + covered[i][1] == covered[i + 1][0] for i in range(len(covered) - 1))


def test_fused_update_is_held_back_one_notification():
    sched, launches, waits, seen_before = run_scheduler(lag=1)
    # the range still pending when backward ends (the embedding table) goes out whole: 34 chunks + 1 instead of + 13
    assert sched.scheduled_chunks == 35 and launches[-1] == (0, 72 * 72 * 2560 + 2560)
    ranges = p888_ranges()
    # after notification i only ranges 0..i-1 may have been launched: the GEMM that still reads the
    # weights of range i is enqueued between notification i and i+1
    for i in range(35):
        launched = seen_before[i]
        assert launched == sum(-(-ranges[j][1] // ((4 << 20) // 4)) for j in range(i))
    assert len(waits) == 35  # one producer event per flush


def test_default_schedule_launches_at_once_and_keeps_the_closing_range_whole():
    sched, launches, waits, seen_before = run_scheduler(lag=0)
    ranges = p888_ranges()
    assert sched.scheduled_chunks == 35 and launches[-1] == (0, 72 * 72 * 2560 + 2560)
    # range i is launched inside notification i (the engine announces it after the last reader of its weights) ...
    assert seen_before[:34] == list(range(1, 35)) and launches[:34] == ranges[:34]
    # ... except the one that closes backward, which finish() sends unchunked
    assert seen_before[34] == 34


def test_early_blocks_go_out_whole_and_the_closing_call_sends_the_rest():
    # the engine computes the embedding gradient in row blocks and announces every finished block but the last through its
    # early-range hook; the closing gradient-ready call still names the whole range, as the reference does
    launches, waits = [], []
    sched = GradientRangeScheduler(lambda off, cnt: launches.append((off, cnt)), lambda: waits.append(len(launches)),
                                   bucket_params=(4 << 20) // 4, expected_ranges=35)
    ranges = p888_ranges()
    half = 36 * 72 * 2560                                  # 36 of the 72 positions: the README's --input-grad-position-tile
    for step in range(2):                                  # the second step starts clean
        launches.clear()
        sched.begin_step()
        for i in range(34):
            assert sched.on_ready(i, *ranges[i]) == 0
        assert sched.on_early(34, 0, half) == 0
        assert launches[-1] == (0, half) and len(launches) == 35   # at once and whole: 6 635 520 floats in one launch
        assert sched.on_ready(34, *ranges[34]) == 0
        assert len(launches) == 35                          # what is left waits for finish() ...
        sched.finish()
        assert launches[-1] == (half, ranges[34][1] - half)  # ... and goes out whole: second block + input bias
        assert sched.scheduled_ranges == 35 and sched.scheduled_chunks == 36
        assert sum(c for _, c in launches) == 15460289      # every parameter exactly once
        covered = sorted(launches)
        assert all(covered[i][0] + covered[i][1] == covered[i + 1][0] for i in range(len(covered) - 1))
    # a hook that announced everything leaves nothing for the closing call
    sched.begin_step()
    for i in range(34):
        assert sched.on_ready(i, *ranges[i]) == 0
    assert sched.on_early(34, 0, half) == 0 and sched.on_early(34, half, ranges[34][1] - half) == 0
    n = len(launches)
    assert sched.on_ready(34, *ranges[34]) == 0
    sched.finish()
    assert len(launches) == n and sched.on_early(34, 0, 0) == 1


def test_touching_ranges_are_joined_into_bucket_sized_launches():
    # the engine's order: output layer, blocks 15..0 (fc2 then fc1), the embedding range through the early hook once its
    # GEMM is enqueued (before the weight-gradient GEMMs in the engine, here after the ranges for simplicity), hidden layer
    bucket = (4 << 20) // 4
    launches = []
    sched = GradientRangeScheduler(lambda off, cnt: launches.append((off, cnt)), lambda: None, bucket_params=bucket, expected_ranges=35,
                                   coalesce=True)
    ranges = p888_ranges()
    for step in range(2):
        launches.clear()
        sched.begin_step()
        assert sched.on_early(34, *ranges[34]) == 0
        for i in range(35):
            assert sched.on_ready(i, *ranges[i]) == 0
        sched.finish()
        assert launches[0] == ranges[34]
        rest = launches[1:]
        assert len(rest) == 3                               # 34 ranges (2.18 M floats) in three launches instead of 34
        assert all(c <= bucket for _, c in rest)
        assert sum(c for _, c in launches) == 15460289
        covered = sorted(launches)
        assert all(covered[i][0] + covered[i][1] == covered[i + 1][0] for i in range(len(covered) - 1))
    # ranges that do not touch are never joined, and a joined launch never exceeds the bucket
    launches.clear()
    sched = GradientRangeScheduler(lambda off, cnt: launches.append((off, cnt)), lambda: None, bucket_params=100, coalesce=True)
    sched.begin_step()
    for off, cnt in [(900, 60), (860, 40), (800, 60), (100, 50), (150, 50), (300, 10)]:
        assert sched.on_ready(0, off, cnt) == 0
    sched.finish()
    assert launches == [(860, 100), (800, 60), (100, 100), (300, 10)]


def test_scheduler_rejects_unexpected_ranges():
    sched = GradientRangeScheduler(lambda o, c: None, lambda: None, expected_ranges=3)
    sched.begin_step()
    assert sched.on_ready(0, 0, 10) == 0
    assert sched.on_ready(5, 0, 10) == 1
    assert sched.on_ready(1, 0, 0) == 1
    with pytest.raises(RuntimeError):
        sched.finish()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _gloo_worker(rank, world, port, ranges, params, out_dir):
    import torch
    import torch.distributed as dist
    from oracle import load_oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    orc = load_oracle()
    rng = np.random.default_rng(100 + rank)
    w = np.linspace(-0.1, 0.1, params).astype(np.float32)
    m = np.zeros(params, np.float32)
    v = np.zeros(params, np.float32)
    for step in (1, 2):
        grad = (rng.standard_normal(params) * 1e-3).astype(np.float32)  # each rank's own batch gradient
        g_t = torch.from_numpy(grad)

        def launch(off, cnt):
            view = g_t[off:off + cnt]
            dist.all_reduce(view, op=dist.ReduceOp.SUM)
            view.mul_(1.0 / world)
            assert orc.adamw(w[off:off + cnt], grad[off:off + cnt], m[off:off + cnt], v[off:off + cnt], step=step, lr=1e-3) == 0

        sched = GradientRangeScheduler(launch, lambda: None, bucket_params=4096, expected_ranges=len(ranges), lag=1)
        sched.begin_step()
        for i, (off, cnt) in enumerate(ranges):
            assert sched.on_ready(i, off, cnt) == 0
        sched.finish()
    np.save(os.path.join(out_dir, f"w{rank}.npy"), w)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_training_matches_single_process(tmp_path, oracle):
    import torch.multiprocessing as mp
    params = 20000
    ranges = [(15000, 5000), (9000, 6000), (0, 9000)]  # backward order: last layer first
    port = _free_port()
    mp.spawn(_gloo_worker, args=(2, port, ranges, params, str(tmp_path)), nprocs=2, join=True)
    w0 = np.load(tmp_path / "w0.npy")
    w1 = np.load(tmp_path / "w1.npy")
    assert np.array_equal(w0, w1)  # replicas stay identical
    # single-process restatement: average in rank order, then AdamW over all parameters
    rngs = [np.random.default_rng(100), np.random.default_rng(101)]
    w = np.linspace(-0.1, 0.1, params).astype(np.float32)
    m = np.zeros(params, np.float32)
    v = np.zeros(params, np.float32)
    for step in (1, 2):
        grads = [(r.standard_normal(params) * 1e-3).astype(np.float32) for r in rngs]
        avg = oracle.allreduce_average(grads)
        assert oracle.adamw(w, avg, m, v, step=step, lr=1e-3) == 0
    assert np.array_equal(w, w0)
