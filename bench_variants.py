#!/usr/bin/env python
"""Training-step benchmark of the configurations beside the headline one (the options the reference does not have).

    python bench.py --workload variant --variant p888_bn            # the p888 model with batch normalisation
    python bench.py --workload variant --variant wide               # hd1 4096, hd2 512, 32 blocks, 29 per-depth logits,
                                                                    # bfloat16 operands, cross-entropy, batch 131072, wd 0.01
    python -m torch.distributed.run ... bench.py --gpus N --workload variant --variant wide [--batch-norm]

Same measurement as the headline line: walk kernel -> loss + gradients -> gradient exchange fused with AdamW (N > 1) or
AdamW (N = 1); K steps between CUDA events, max over ranks; inputs are generated on the device every step and the
activation tape of a step is far larger than L2. With batch normalisation at N > 1 the statistics of every layer are
averaged over the ranks by a second communicator on the compute stream. Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

VARIANTS = {
    "p888_bn": dict(shape=dict(state_len=72, state_value_pad=72, hd1=2560, hd2=224, residual_blocks=16, output_dim=1), batch=53248,
                    bf16=False, cross_entropy=False, batch_norm=True, weight_decay=0.0,
                    workload="p888 training step with batch normalisation of the hidden layer and of every block (statistics over all ranks)"),
    "wide": dict(shape=dict(state_len=72, state_value_pad=72, hd1=4096, hd2=512, residual_blocks=32, output_dim=29), batch=131072,
                 bf16=True, cross_entropy=True, batch_norm=False, weight_decay=0.01,
                 workload="wide/deep variant: hd1 4096, hd2 512, 32 blocks, 29 per-depth logits, bfloat16 operands, cross-entropy on depth - 1"),
}
SEED = 1234
LR = 1e-4


def run(args) -> dict:
    import torch
    import multigputrainmlp_b200 as mgt
    from multigputrainmlp_b200.comm import OverlappedGradientExchange, PeerBackend, default_id_file

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    v = dict(VARIANTS[args.variant])
    if args.batch_norm:
        v["batch_norm"] = True
    batch = args.variant_batch or v["batch"]
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    shape = mgt.CudaMlpShape(**v["shape"])
    out_dim, h2, blocks = shape.output_dim, shape.hd2, shape.residual_blocks
    params = shape.param_count
    nbn = mgt.bn_param_count(shape) if v["batch_norm"] else 0
    total = params + nbn
    idx = np.arange(params, dtype=np.int64)
    w_host = np.concatenate([((idx % 29 - 14) * 0.0001).astype(np.float32), np.zeros(nbn, np.float32)])
    if nbn:
        w_host[params:].reshape(blocks + 1, 2, h2)[:, 0, :] = 1.0
    w = torch.from_numpy(w_host).to(dev)
    w_half = w.half()
    m = torch.zeros(total, device=dev)
    vv = torch.zeros(total, device=dev)
    loss = torch.zeros(1, device=dev)
    engine = mgt.Engine(local_rank)
    assert engine.set_train_options(bf16=v["bf16"], cross_entropy=v["cross_entropy"], batch_norm=v["batch_norm"]) == 0
    backend = stats_backend = exchange = None
    if world > 1:
        id_file = default_id_file() + ".variant"
        for suffix in ("", ".bn"):
            if rank == 0 and os.path.exists(id_file + suffix):
                os.remove(id_file + suffix)
        dist.barrier()
        backend = PeerBackend(local_rank, world, rank, id_file, total)
        grad = backend.gradient_tensor(dev)
        exchange = OverlappedGradientExchange(backend, dev, bucket_bytes=args.bucket_bytes, residual_blocks=blocks, fused_adamw=True,
                                              extra_ranges=1 if nbn else 0)
        assert engine.set_early_range_hook(exchange.early_callback) == 0
    else:
        grad = torch.zeros(total, device=dev)
    running = None
    if nbn:
        running = torch.zeros(blocks + 1, 2, h2, device=dev)
        running[:, 1, :] = 1.0
        if world > 1:
            stats_backend = PeerBackend(local_rank, world, rank, id_file + ".bn", 2 * h2)
            stats_buffer = stats_backend.gradient_tensor(dev)

            def stats_exchange(user, ptr, count, stream):
                return stats_backend.allreduce_average(0, int(count), stream=int(stream) if stream else 0)

            assert engine.set_batch_norm_state(running, 0.1, world, stats_buffer, stats_exchange) == 0
        else:
            assert engine.set_batch_norm_state(running, 0.1, 1) == 0
    moves_h = np.zeros((18, 80), np.uint8)
    for mv in range(18):
        moves_h[mv, :72] = (np.arange(72) + mv + 1) % 72          # the trainer's built-in cyclic shifts (tool:117-140)
    target_h = np.zeros(80, np.uint8)
    target_h[:72] = np.arange(72)
    moves_d = torch.from_numpy(moves_h).to(dev)
    target_d = torch.from_numpy(target_h).to(dev)
    states = torch.zeros(batch, 80, dtype=torch.uint8, device=dev)
    depth = torch.zeros(batch, device=dev)
    labels = depth if out_dim == 1 else torch.zeros(batch * out_dim, device=dev)
    meta = torch.zeros(batch, 16, dtype=torch.uint8, device=dev)
    ws_floats = mgt.mlp_loss_grad_workspace_floats(shape, batch, batch_norm=bool(nbn))
    assert ws_floats > 0
    workspace = torch.empty(ws_floats, device=dev)
    walk_cfg = mgt.RandomWalkKernelConfig(batch, 1, 29)
    other = [0]

    def step(s, profile=None):
        assert mgt.launch_random_walk_kernel(walk_cfg, SEED, 0, s, rank, moves_d, target_d, states, depth, meta) == 0
        other[0] += 1
        if out_dim > 1:
            assert mgt.launch_expand_scalar_labels(depth, batch, out_dim, labels) == 0
            other[0] += 1
        cfg = mgt.AdamWKernelConfig(total, s + 1, LR, weight_decay=v["weight_decay"])
        if exchange is not None:
            exchange.begin_step(cfg, w, w_half, m, vv)
        st = engine.launch_mlp_loss_grad(shape, w, w_half, states, labels, batch, loss, grad, workspace, ws_floats, profile=profile,
                                         input_grad_position_tile=36, gradient_ready=exchange.callback if exchange is not None else None)
        assert st == 0, mgt.status_name(st)
        if exchange is not None:
            exchange.finish_step()
        else:
            assert mgt.launch_adamw_kernel_with_half_mirror(cfg, w, w_half, grad, m, vv) == 0
            other[0] += 1

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    warmup = max(3, args.warmup)
    for s in range(warmup):
        step(s)
    barrier()
    st, code = engine.check()
    assert st == 0, f"device status {code}"
    launches0 = engine.launch_count + other[0] + (backend.launch_count if backend else 0) + (stats_backend.launch_count if stats_backend else 0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for s in range(args.steps):
        step(warmup + s)
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_step = float(ms.item())
    launches = engine.launch_count + other[0] + (backend.launch_count if backend else 0) + (stats_backend.launch_count if stats_backend else 0) - launches0
    for b in (backend, stats_backend):
        if b is not None:
            st, code = b.check()
            assert st == 0, f"communicator status {code}"
    final_loss = float(loss.item())
    prof = mgt.BackwardProfile()
    step(warmup + args.steps, profile=prof)
    torch.cuda.synchronize()
    stage_ms = {n: round(getattr(prof, n), 4) for n, _ in prof._fields_}
    # replicas must still agree (N > 1): the same two checksums of the weights on every rank
    replicas_identical = None
    if world > 1:
        sums = torch.stack([w.double().sum(), (w.double() * torch.arange(total, device=dev, dtype=torch.float64).remainder(251.0)).sum()])
        gathered = [torch.zeros_like(sums) for _ in range(world)]
        dist.all_gather(gathered, sums)
        replicas_identical = all(bool(torch.equal(g, gathered[0])) for g in gathered)
    h1 = shape.hd1
    flop = 3 * (2 * h1 * h2 + 4 * blocks * h2 * h2 + 2 * h2 * out_dim) + 2 * 72 * h1   # as the headline line counts it
    line = {
        "metric": "training candidates/sec (device-timed, max over ranks)", "value": batch * world / (ms_step * 1e-3), "unit": "candidates/s",
        "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16" if v["bf16"] else "f16", "data": "synthetic",
        "config": {"workload": v["workload"], "variant": args.variant, "batch_per_rank": batch, **v["shape"], "batch_norm": bool(nbn),
                   "loss": "cross_entropy" if v["cross_entropy"] else "mse", "weight_decay": v["weight_decay"], "parallelism": f"dp{world}",
                   "l2": "inputs larger than L2 (activation tapes of several GB per step)"},
        "gpu_launches": int(launches), "stage_ms": stage_ms, "final_loss": final_loss, "replicas_identical": replicas_identical,
        "step_tflops_algorithmic": flop * batch / (ms_step * 1e-3) / 1e12,
        "workspace_gb": ws_floats * 4 / 1e9,
    }
    for b in (backend, stats_backend):
        if b is not None:
            b.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return line if rank == 0 else {}
