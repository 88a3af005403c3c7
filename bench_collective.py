#!/usr/bin/env python
"""Collective microbenchmark: the gradient exchange fused with AdamW, per bucket size and on the real
p888 schedule, against NCCL + scale + AdamW (the reference's scheme) and against the NVLink link rate.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        bench.py --workload collective --gpus N [--steps K --warmup W]

What is measured (native/cuda/allreduce_nccl.cu:120-150 + native/cuda/adamw.cu:35-46 are what it replaces):
  * flat fp32 gradient buffer of the full p888 parameter count (15 460 289 floats, 61.84 MB), values ~ N(0, 1e-3)
    from a fixed-seed host generator, different on every rank;
  * buckets of 256 KB ... 64 MB: one timed pass walks the whole buffer in buckets of that size (the last one
    ragged), so consecutive launches touch different memory and a pass moves 4 x 62 MB through HBM (> L2);
  * the reference trainer's schedule (native/tools/mgt_native_train_smoke.cu:494-523): output layer, 32 block ranges,
    hidden layer, embedding range, each cut into --bucket-bytes chunks, in backward order (47 launches);
  * this trainer's schedule: the embedding range first and whole, the other ranges joined where they touch (5 launches) -
    the headline value of the line;
  * 17 statistics vectors of 2 x 224 floats (one-shot exchange, no update): the latency of a tiny collective.
  bus GB/s = 2 (W-1)/W * bytes / time, device-timed with CUDA events, max over ranks.
Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

P888 = dict(state_len=72, state_value_pad=72, hd1=2560, hd2=224, residual_blocks=16, output_dim=1)
NVLINK_GBS_PER_DIRECTION = 900.0        # nominal, per GPU
NVLINK_MEASURED_PEER_COPY_GBS = 770.0   # peer copy measured on this pool's B200s


def p888_schedule(bucket_params: int):
    """(offset, count) of every exchange launch of one p888 step, in the order backward announces the ranges."""
    L, V, H1, H2, R, OUT = 72, 72, 2560, 224, 16, 1
    in_bias = L * V * H1
    hidden_w = in_bias + H1
    hidden_b = hidden_w + H1 * H2
    res = hidden_b + H2
    block = 2 * (H2 * H2 + H2)
    out_w = res + R * block
    ranges = [(out_w, H2 * OUT + OUT)]
    for k in reversed(range(R)):
        fc1 = res + k * block
        fc2 = fc1 + H2 * H2 + H2
        ranges += [(fc2, H2 * H2 + H2), (fc1, H2 * H2 + H2)]
    ranges += [(hidden_w, H1 * H2 + H2), (0, in_bias + H1)]
    launches = []
    for off, cnt in ranges:
        while cnt > 0:
            c = min(cnt, bucket_params)
            launches.append((off, c))
            off += c
            cnt -= c
    return ranges, launches


def trainer_schedule(bucket_params: int):
    """What the trainer and bench.py launch for one p888 step: the embedding range whole and first (it comes through the
    engine's early-range hook, exchange only, its AdamW follows backward), then the other 34 ranges in backward order,
    joined where they touch into launches of at most one bucket (GradientRangeScheduler with coalesce=True)."""
    from multigputrainmlp_b200.comm import GradientRangeScheduler
    ranges, _ = p888_schedule(bucket_params)
    early, fused = [], []
    sched = GradientRangeScheduler(lambda off, cnt: fused.append((off, cnt)), lambda: None, bucket_params=bucket_params,
                                   expected_ranges=len(ranges), coalesce=True, launch_early=lambda off, cnt: early.append((off, cnt)))
    sched.begin_step()
    for i, (off, cnt) in enumerate(ranges[:-1]):
        if i == 0:
            sched.on_ready(i, off, cnt)   # the output layer is announced long before the embedding gradient is complete
            continue
        if i == 1:
            sched.on_early(len(ranges) - 1, *ranges[-1])
        sched.on_ready(i, off, cnt)
    sched.on_ready(len(ranges) - 1, *ranges[-1])
    sched.finish()
    return early, fused


def run(args) -> dict:
    import torch
    import torch.distributed as dist
    import multigputrainmlp_b200 as mgt
    from multigputrainmlp_b200.comm import PeerBackend, default_id_file

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        raise SystemExit("--workload collective needs at least 2 ranks (torchrun --nproc-per-node N)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    params = mgt.CudaMlpShape(**P888).param_count
    id_file = default_id_file() + ".coll"
    if rank == 0 and os.path.exists(id_file):
        os.remove(id_file)
    dist.barrier()
    backend = PeerBackend(local_rank, world, rank, id_file, params)
    grad = backend.gradient_tensor(dev)
    host = (np.random.default_rng(1000 + rank).standard_normal(params) * 1e-3).astype(np.float32)
    grad_src = torch.from_numpy(host).to(dev)
    grad_nccl = torch.empty_like(grad_src)
    w = torch.linspace(-0.05, 0.05, params, device=dev)
    w_half = w.half()
    m = torch.zeros(params, device=dev)
    v = torch.zeros(params, device=dev)
    steps, warmup = args.steps, max(args.warmup, 3)
    step_no = [0]

    def adam_cfg(count):
        step_no[0] += 1
        return mgt.AdamWKernelConfig(count, step_no[0], 1e-4)

    def sync():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    def timed(fn) -> float:
        """ms per call of fn (one pass), device-timed: max over ranks, median over passes; the gradient buffer is refilled outside the timing"""
        for _ in range(warmup):
            grad.copy_(grad_src)
            fn()
        times = []
        for _ in range(steps):
            grad.copy_(grad_src)
            grad_nccl.copy_(grad_src)
            sync()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        # per pass the slowest rank counts; over the passes the median (single passes three to five times slower than
        # the rest turn up on shared NVSwitch fabric, for NCCL and for the peer kernels alike)
        t = torch.tensor(times, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.median().item())

    def fused_pass(launches):
        def go():
            for off, cnt in launches:
                st = backend.allreduce_average_adamw(off, cnt, adam_cfg(params), w, w_half, m, v)
                assert st == 0, st
        return go

    def nccl_pass(launches):
        inv = 1.0 / world

        def go():
            for off, cnt in launches:
                view = grad_nccl[off:off + cnt]
                dist.all_reduce(view, op=dist.ReduceOp.SUM)
                view.mul_(inv)
                cfg = adam_cfg(cnt)
                st = mgt.launch_adamw_kernel_with_half_mirror(cfg, w[off:off + cnt], w_half[off:off + cnt], view, m[off:off + cnt], v[off:off + cnt])
                assert st == 0, st
        return go

    def bus(bytes_moved, ms):
        return 2.0 * (world - 1) / world * bytes_moved / (ms * 1e-3) / 1e9

    rows = []
    for bucket_bytes in (256 << 10, 1 << 20, 4 << 20, 16 << 20, 64 << 20):
        bp = bucket_bytes // 4
        launches = [(off, min(bp, params - off)) for off in range(0, params, bp)]
        # offsets of later buckets are multiples of 4 floats only when bp is: all sizes here are
        f_ms = timed(fused_pass(launches))
        n_ms = timed(nccl_pass(launches))
        rows.append({"bucket_bytes": bucket_bytes, "launches_per_pass": len(launches), "fused_ms_per_pass": f_ms, "nccl_adamw_ms_per_pass": n_ms,
                     "fused_bus_gbs": bus(params * 4, f_ms), "nccl_adamw_bus_gbs": bus(params * 4, n_ms)})
    ranges, launches = p888_schedule(args.bucket_bytes // 4)
    sched_f = timed(fused_pass(launches))
    sched_n = timed(nccl_pass(launches))
    early, joined = trainer_schedule(args.bucket_bytes // 4)

    def trainer_pass():
        for off, cnt in early:
            assert backend.allreduce_average(off, cnt) == 0
        for off, cnt in joined:
            assert backend.allreduce_average_adamw(off, cnt, adam_cfg(params), w, w_half, m, v) == 0
        for off, cnt in early:   # the deferred update of the early range
            assert mgt.launch_adamw_kernel_with_half_mirror(adam_cfg(cnt), w[off:off + cnt], w_half[off:off + cnt], grad[off:off + cnt], m[off:off + cnt], v[off:off + cnt]) == 0

    trainer_ms = timed(trainer_pass)
    whole = [(0, params)]
    whole_f = timed(fused_pass(whole))
    whole_n = timed(nccl_pass(whole))
    emb = [ranges[-1]]
    emb_f = timed(fused_pass(emb))

    # statistics vectors: 17 one-shot exchanges of 2 x 224 floats, no optimizer step
    stat_launches = [(i * 448, 448) for i in range(17)]

    def stats_fused():
        for off, cnt in stat_launches:
            assert backend.allreduce_average(off, cnt) == 0

    def stats_nccl():
        for off, cnt in stat_launches:
            view = grad_nccl[off:off + cnt]
            dist.all_reduce(view, op=dist.ReduceOp.SUM)
            view.mul_(1.0 / world)

    stat_f = timed(stats_fused)
    stat_n = timed(stats_nccl)
    st, code = backend.check()
    assert st == 0, f"communicator status {code}"
    sync()
    line = {
        "metric": "fused gradient allreduce + AdamW bus GB/s (the trainer's p888 schedule, device-timed, max over ranks)",
        "value": bus(params * 4, trainer_ms), "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": trainer_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "collective microbench: flat fp32 gradient of the full p888 parameter count, N(0,1e-3), fused exchange + AdamW",
                   "gradient_floats": params, "gradient_bytes": params * 4, "bucket_bytes": args.bucket_bytes, "ranges": len(ranges),
                   "launches": len(launches), "l2": "a pass walks 4 arrays x 62 MB (larger than L2); the buffer is refilled between passes"},
        "trainer_schedule": {"fused_ms": trainer_ms, "fused_bus_gbs": bus(params * 4, trainer_ms), "exchange_launches": len(early) + len(joined),
                             "note": "embedding range first and whole (exchange only, AdamW after the others), the other 34 ranges joined into bucket-sized launches"},
        "reference_schedule": {"fused_ms": sched_f, "nccl_scale_adamw_ms": sched_n, "fused_bus_gbs": bus(params * 4, sched_f),
                     "nccl_scale_adamw_bus_gbs": bus(params * 4, sched_n), "speedup": sched_n / sched_f},
        "whole_buffer": {"fused_ms": whole_f, "nccl_scale_adamw_ms": whole_n, "fused_bus_gbs": bus(params * 4, whole_f),
                         "nccl_scale_adamw_bus_gbs": bus(params * 4, whole_n)},
        "embedding_range": {"floats": emb[0][1], "fused_ms": emb_f, "fused_bus_gbs": bus(emb[0][1] * 4, emb_f)},
        "buckets": rows,
        "stat_vectors": {"count": 17, "floats_each": 448, "one_shot_us_each": stat_f * 1e3 / 17, "nccl_us_each": stat_n * 1e3 / 17},
        "nvlink_gbs_per_direction": {"nominal": NVLINK_GBS_PER_DIRECTION, "measured_peer_copy": NVLINK_MEASURED_PEER_COPY_GBS},
        "frac_of_link": {"of_nominal": bus(params * 4, trainer_ms) / NVLINK_GBS_PER_DIRECTION, "of_measured": bus(params * 4, trainer_ms) / NVLINK_MEASURED_PEER_COPY_GBS},
        "gpu_launches": int(backend.launch_count),
    }
    backend.close()
    dist.barrier()
    dist.destroy_process_group()
    return line if rank == 0 else {}


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--bucket-bytes", type=int, default=4 << 20)
    out = run(ap.parse_args())
    if out:
        print(json.dumps(out), flush=True)
