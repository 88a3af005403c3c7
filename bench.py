#!/usr/bin/env python
"""Headline benchmark: training candidates/s of the full p888 training step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is exactly what the reference trainer times between its step_start and step_stop events
(native/tools/mgt_native_train_smoke.cu:769-846): on-GPU random-walk generation -> forward, MSE
loss, backward -> gradient average over ranks -> AdamW with fp16 mirror. Configuration: physical
p888 model (state 72x72, hd1 2556->2560, hd2 218->224, 16 residual blocks, output 1), batch
53 248 per rank, fp16 linears with fp32 accumulate and fp32 master weights, seed 1234, the
trainer's built-in cyclic-shift puzzle and deterministic initial weights (synthetic data: the
training set is generated on the fly, there is no dataset).

One process per GPU (torchrun sets RANK/LOCAL_RANK/WORLD_SIZE). Rank 0 prints ONE JSON line.
`--impl reference` times the reference's own CPU implementation of the same step on the host
cores instead (rank 0 only), on a bounded sample of the batch.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "training candidates/sec (device-timed, max over ranks)"
UNIT = "candidates/s"
P888 = dict(state_len=72, state_value_pad=72, hd1=2560, hd2=224, residual_blocks=16, output_dim=1)
BATCH = 53248
SEED = 1234
LR = 1e-4
FLOP_PER_CANDIDATE = 13_444_416          # 3*(2*H1*H2 + 4R*H2^2 + 2*H2*OUT) + 2*L*H1 at the physical dims
EMB_ALGO_FLOP_PER_CANDIDATE = 72 * 2560   # the embedding forward counted as the sparse work it is (72 row adds)
EMB_EXEC_FLOP_PER_CANDIDATE = 2 * (72 * 72 + 1) * 2560  # what the one-hot GEMM executes on the tensor cores
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from an ncu capture (not measured by
# this run: the source is named in the output next to the figure)
EMB_FWD_DRAM_BYTES_PER_LAUNCH = 268_568_064
EMB_FWD_DRAM_SOURCE = ("ncu dram__bytes_read.sum + dram__bytes_write.sum, one launch at batch 53248 (32.9 MB read + 235.7 MB written: "
                       "the [hd1][B] activation and its sign words), single-pass capture of 2026-11-25, profiles/training_step_p888_launch_list.md")
README_P888_FLAGS = ["--batch-size", "53248", "--k-min", "1", "--k-max", "29", "--hd1", "2556", "--hd2", "218", "--nrd", "16",
                     "--input-grad-fp16", "1", "--input-grad-position-tile", "36", "--linear-fp16", "1", "--write-artifacts", "0",
                     "--allreduce-bucket-bytes", "4194304"]  # the reference README's p888 command (README.md:48-64)


def cyclic_puzzle(state_len: int = 72, move_count: int = 18):
    """The trainer's built-in puzzle (native/tools/mgt_native_train_smoke.cu:117-140): move m maps i -> (i + m + 1) mod
    state_len (unused moves are the identity), the target is the identity; pad bytes are zero."""
    moves = np.zeros((18, 80), np.uint8)
    for mv in range(18):
        moves[mv, :state_len] = (np.arange(state_len) + mv + 1) % state_len if mv < move_count else np.arange(state_len)
    target = np.zeros(80, np.uint8)
    target[:state_len] = np.arange(state_len)
    return moves, target


def workload_config(n_gpus: int) -> dict:
    return {
        "workload": "p888 training step: walk gen -> fwd/loss/bwd -> grad average -> AdamW (headline configuration, %s)" % ("one rank" if n_gpus == 1 else "%d ranks" % n_gpus),
        "batch_per_rank": BATCH, "global_batch": BATCH * n_gpus, "hd1": 2556, "physical_hd1": 2560, "hd2": 218,
        "physical_hd2": 224, "nrd": 16, "output_dim": 1, "k_min": 1, "k_max": 29, "seed": SEED,
        "precision": "fp16 operands, fp32 accumulate, fp32 master weights", "parallelism": "dp%d" % n_gpus,
        "l2": "inputs larger than L2 (1.5 GB activation tape per step, 126 MB L2)",
    }


def load_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "tflops_burst": p["bf16_tflops"], "tflops_sustained": p["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops_burst": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML queries (read-only) every
    10 ms from a thread of this process, or `nvidia-smi -lms 100` when the NVML module is missing."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index: int, uuid: str | None = None):
        self.rows = []          # (time, sm_mhz, set of active reasons)
        self.smax = None
        self.proc = None
        self.stop_flag = threading.Event()
        self.thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            try:  # CUDA_VISIBLE_DEVICES renumbers CUDA devices, NVML keeps the board order: go by UUID when it is known
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode() if isinstance(uuid, str) else uuid)
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.smax = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._poll_nvml, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read_smi, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _poll_nvml(self):
        n = self.nvml
        masks = {"hw_slowdown": getattr(n, "nvmlClocksEventReasonHwSlowdown", 0x8), "hw_thermal_slowdown": getattr(n, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(n, "nvmlClocksEventReasonSwThermalSlowdown", 0x20), "sw_power_cap": getattr(n, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        get_reasons = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(n, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self.stop_flag.is_set():
            try:
                mhz = float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                bits = int(get_reasons(self.handle))
                self.rows.append((time.time(), mhz, {name for name, mask in masks.items() if bits & mask}))
            except Exception:
                pass
            time.sleep(0.01)

    def _read_smi(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                self.smax = float(parts[1])
                self.rows.append((time.time(), float(parts[0]), {name for name, val in zip(self.NAMES, parts[3:7]) if val.lower().startswith("active")}))
            except ValueError:
                continue

    def stop(self, t0: float, t1: float) -> dict:
        if self.thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock sampling unavailable"]}
        time.sleep(0.05 if self.proc is None else 0.15)
        self.stop_flag.set()
        if self.proc is not None:
            self.proc.terminate()
        inside = [r for r in self.rows if t0 <= r[0] <= t1] or self.rows[-3:]  # very short regions: take what was seen
        sm = [r[1] for r in inside]
        reasons = set()
        for r in inside:
            reasons |= r[2]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": self.smax, "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
def run_reference_cpu(args, steps: int, warmup: int) -> dict:
    """The reference's own CPU path (GenerateRandomWalksCpu + CpuMlpLossAndGrad + CpuAdamWStep) on the
    host cores. Its code is single-threaded, so the harness runs one sample slice per core with its
    own gradient buffer, as a data-parallel CPU run would."""
    from oracle import MlpShape, load_oracle, load_reference

    ref = load_reference()
    orc = load_oracle()
    kind = "reference" if ref is not None else "port"
    impl = ref if ref is not None else orc
    shape = MlpShape(**P888)
    params = shape.param_count
    cores = min(os.cpu_count() or 1, 64)  # one 62 MB gradient buffer per thread: bounded on purpose
    per_core = args.cpu_samples_per_core
    idx = np.arange(params, dtype=np.int64)
    weights = ((idx % 29 - 14) * 0.0001).astype(np.float64).astype(np.float32)
    moves, target = orc.cyclic_puzzle(72, 18)
    grads = [np.zeros(params, np.float32) for _ in range(cores)]
    m = np.zeros(params, np.float32)
    v = np.zeros(params, np.float32)
    sample = cores * per_core

    def one_step(step: int) -> float:
        t0 = time.perf_counter()
        st, states, labels, _ = impl.random_walks(moves, target, seed=SEED, epoch=0, step=step, rank=0, k_min=1, k_max=29, samples=sample)
        assert st == 0
        out = [None] * cores

        def work(c):
            lo = c * per_core
            out[c] = impl.loss_grad(shape, weights, states[lo:lo + per_core], labels[lo:lo + per_core].reshape(-1, 1))
            grads[c][:] = out[c][2]

        threads = [threading.Thread(target=work, args=(c,)) for c in range(cores)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        total = grads[0].copy()
        for c in range(1, cores):
            total += grads[c]
        total *= 1.0 / cores
        t_grad = time.perf_counter() - t0
        t1 = time.perf_counter()
        impl.adamw(weights, total, m, v, step=step + 1, lr=LR)
        t_adam = time.perf_counter() - t1
        # the optimizer runs once per full batch: charge the sample its share of that cost
        return t_grad + t_adam * (sample / BATCH)

    for s in range(warmup):
        one_step(s)
    times = [one_step(warmup + s) for s in range(steps)]
    sec = float(np.mean(times))
    value = sample / sec
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": workload_config(max(1, args.gpus)),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind,
                         "sample": f"{sample} samples of the batch per step ({per_core} per core, {cores} threads), optimizer cost scaled by {sample}/{BATCH}"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    return line



# ------------------------------------------------------------------------------------------------
def check_gradient_exchange(torch, dist, mgt, backend, dev, world, params, bucket_bytes, state):
    """Correctness of the multi-GPU data plane, checked where the number is produced (after the timed regions):
      avg_bit_exact       the peer exchange on the trainer's real range schedule equals the rank-order sum times 1/W
                          bit for bit (what ncclAllReduce(sum) + ScaleKernel define, native/cuda/allreduce_nccl.cu:130-148);
      replicas_identical  weights, fp16 mirror and both AdamW moments have the same checksums on every rank after the
                          timed steps (identical replicas are what lets the reference skip a broadcast);
      fused_vs_nccl_rel_l2  one fused exchange+AdamW step against NCCL allreduce + scale + AdamW kernel from the same state."""
    from bench_collective import p888_schedule
    w, w_half, m, v = state
    out = {}

    def checksums(t):
        bits = t.view(torch.int32) if t.dtype == torch.float32 else t.view(torch.int16)
        x = bits.to(torch.int64)
        weights = (torch.arange(x.numel(), device=dev, dtype=torch.int64) % 65521) + 1
        return [int(x.sum().item()), int((x * weights).sum().item())]

    mine = torch.tensor([c for t in (w, w_half, m, v) for c in checksums(t)], device=dev, dtype=torch.int64)
    everyone = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(everyone, mine)
    out["replicas_identical"] = bool(all(torch.equal(everyone[0], e) for e in everyone))

    grad = backend.gradient_tensor(dev)
    gen = torch.Generator(device=dev).manual_seed(4242 + dist.get_rank())
    pattern = torch.randn(params, device=dev, generator=gen) * 1e-3
    ranges, launches = p888_schedule(max(1, bucket_bytes // 4))
    grad.copy_(pattern)
    torch.cuda.synchronize()
    dist.barrier()
    for off, cnt in launches:
        st = backend.allreduce_average(off, cnt)
        assert st == 0, st
    st, code = backend.check()
    assert st == 0, f"communicator status {code}"
    inputs = [torch.empty_like(pattern) for _ in range(world)]
    dist.all_gather(inputs, pattern)
    expected = inputs[0].clone()
    for r in range(1, world):
        expected += inputs[r]
    expected *= torch.tensor(1.0, dtype=torch.float32).div(float(world)).item()
    out["avg_bit_exact"] = bool(torch.equal(grad, expected))
    out["avg_ranges"] = len(ranges)
    out["avg_launches"] = len(launches)
    del inputs

    # one optimizer step both ways from the same state
    w0, h0, m0, v0 = w.clone(), w_half.clone(), m.clone(), v.clone()
    cfg = mgt.AdamWKernelConfig(params, 7, LR)
    grad.copy_(pattern)
    torch.cuda.synchronize()
    dist.barrier()
    for off, cnt in launches:
        st = backend.allreduce_average_adamw(off, cnt, cfg, w, w_half, m, v)
        assert st == 0, st
    st, code = backend.check()
    assert st == 0, f"communicator status {code}"
    g2 = pattern.clone()
    dist.all_reduce(g2, op=dist.ReduceOp.SUM)
    g2.mul_(1.0 / world)
    st = mgt.launch_adamw_kernel_with_half_mirror(cfg, w0, h0, g2, m0, v0)
    assert st == 0, st
    torch.cuda.synchronize()
    num = (w.double() - w0.double()).pow(2).sum().sqrt().item()
    den = w0.double().pow(2).sum().sqrt().item()
    out["fused_vs_nccl_rel_l2"] = num / max(den, 1e-30)
    out["fused_vs_nccl_mirror_equal_fraction"] = float((w_half == h0).float().mean().item())
    flags = torch.tensor([int(out["avg_bit_exact"]), int(out["replicas_identical"]), int(out["fused_vs_nccl_rel_l2"] <= 1e-6)], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)  # a check holds only if it holds on every rank
    out["avg_bit_exact"], out["replicas_identical"] = bool(flags[0].item()), bool(flags[1].item())
    out["ok"] = bool(flags.min().item() == 1)
    return out


def run_gpu_trainers_side_by_side(world: int, steps: int) -> dict:
    """The reference's own GPU trainer (unmodified sources compiled for sm_100 with the cuBLASLt/NCCL of the image, built
    by oracle/Makefile into oracle/_ref) and bin/mgt_native_train on the README's p888 command, one process per GPU, timed
    by the reference's throughput formula (kaggle/kernel/run_ranks_2xt4.sh:95-115). A checker leg like cpu_baseline: it runs
    outside the timed regions and nothing of it is on the product path."""
    import tempfile
    from multigputrainmlp_b200.launch import TRAINER, launch
    ref_bin = os.path.join(ROOT, "oracle", "_ref", "mgt_native_train_ref")
    if not os.path.exists(ref_bin) or not os.path.exists(TRAINER):
        return {"unavailable": "oracle/_ref/mgt_native_train_ref or bin/mgt_native_train not built"}
    flags = README_P888_FLAGS + ["--steps", str(steps)]
    out = {"flags": " ".join(flags), "world_size": world}
    with tempfile.TemporaryDirectory(prefix="mgt_bench_") as tmp:
        for name, binary in (("reference", ref_bin), ("ours", TRAINER)):
            summary = launch(world, os.path.join(tmp, name), flags, trainer=binary, timeout=600)
            if summary.get("status") != "ok":
                return {"unavailable": f"{name} trainer run failed: {summary.get('status')} exit codes {summary.get('exit_codes')}"}
            steady = summary["steady_steps"]
            out[name] = {"candidates_s": summary["avg_throughput_states_s"], "ms_per_step": float(np.mean([s["max_rank_ms"] for s in steady])),
                         "final_loss_rank0": steady[-1]["rank_losses"][0], "steps_timed": len(steady)}
    out["ratio"] = out["ours"]["candidates_s"] / out["reference"]["candidates_s"]
    a, b = out["reference"]["final_loss_rank0"], out["ours"]["final_loss_rank0"]
    out["final_loss_rel_diff"] = abs(a - b) / max(abs(a), 1e-30)
    return out


def claim_stdout():
    """stdout carries ONE JSON line and nothing else: libraries write banners there (NCCL prints its version at the first
    collective), so file descriptor 1 is pointed at stderr for the rest of the process and the line goes to the returned
    file, which is the original stdout."""
    sys.stdout.flush()
    original = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    return original


# ------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--comm", default="peer", choices=["peer", "nccl"], help="gradient exchange at N>1: the library's NVLink peer kernels, or NCCL + AdamW (the reference's scheme, for comparison)")
    ap.add_argument("--bucket-bytes", type=int, default=4 << 20)
    ap.add_argument("--no-early-range", action="store_true", help="N>1: exchange the embedding range when backward has ended instead of under the weight-gradient GEMMs")
    ap.add_argument("--early-fused", action="store_true", help="N>1: also run the AdamW update of the early range under the weight-gradient GEMMs (default: after backward)")
    ap.add_argument("--batch", type=int, default=BATCH, help=argparse.SUPPRESS)  # smaller batches are for ncu captures only
    ap.add_argument("--cpu-samples-per-core", type=int, default=384)
    ap.add_argument("--steps-cpu", type=int, default=2)
    ap.add_argument("--warmup-cpu", type=int, default=1)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-reference-gpu", action="store_true", help="skip the side-by-side run of the reference's GPU trainer and bin/mgt_native_train")
    ap.add_argument("--reference-gpu-steps", type=int, default=30)
    ap.add_argument("--workload", default="step", choices=["step", "collective", "variant", "optimizer"],
                    help="step: the p888 training step (headline); collective: the gradient-exchange microbenchmark (bench_collective.py, needs >= 2 "
                         "ranks); variant: a training step with the options the reference does not have (bench_variants.py, see --variant); "
                         "optimizer: the AdamW kernel alone on gradients with and without exact zeros (bench_optimizer.py)")
    ap.add_argument("--variant", default="p888_bn", choices=["p888_bn", "wide"],
                    help="p888_bn: the p888 model with batch normalisation; wide: hd1 4096, hd2 512, 32 blocks, 29 logits, bfloat16, cross-entropy, batch 131072")
    ap.add_argument("--batch-norm", action="store_true", help="--workload variant: batch normalisation also in a variant that has none by default")
    ap.add_argument("--variant-batch", type=int, default=0, help=argparse.SUPPRESS)
    args = ap.parse_args()
    out = claim_stdout()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank == 0:
            print(json.dumps(run_reference_cpu(args, args.steps, args.warmup)), file=out, flush=True)
        return

    if args.workload in ("collective", "variant", "optimizer"):
        if args.workload == "collective":
            import bench_collective as other
        elif args.workload == "optimizer":
            import bench_optimizer as other
        else:
            import bench_variants as other
        line = other.run(args)
        if line:
            print(json.dumps(line), file=out, flush=True)
        return

    import torch
    import multigputrainmlp_b200 as mgt

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        host_group = dist.new_group(backend="gloo")  # for waits during which no rank may keep a kernel spinning on its GPU
    batch = args.batch
    shape = mgt.CudaMlpShape(**P888)
    params = shape.param_count
    idx = np.arange(params, dtype=np.int64)
    w_host = ((idx % 29 - 14) * 0.0001).astype(np.float64).astype(np.float32)  # tool:648-650
    w = torch.from_numpy(w_host).to(dev)
    w_half = w.half()
    m = torch.zeros(params, device=dev)
    v = torch.zeros(params, device=dev)
    loss = torch.zeros(1, device=dev)
    backend = None
    exchange = None
    from multigputrainmlp_b200.comm import NcclBackend, OverlappedGradientExchange, PeerBackend, default_id_file
    if world > 1 and args.comm == "nccl":
        grad = torch.zeros(params, device=dev)
        backend = NcclBackend(grad, world)
        exchange = OverlappedGradientExchange(backend, dev, bucket_bytes=args.bucket_bytes, residual_blocks=16, fused_adamw=False)
    elif world > 1:
        import torch.distributed as dist
        id_file = default_id_file()
        if rank == 0 and os.path.exists(id_file):
            os.remove(id_file)  # a stale id file of an earlier run must not be picked up
        dist.barrier()
        backend = PeerBackend(local_rank, world, rank, id_file, params)
        grad = backend.gradient_tensor(dev)
        exchange = OverlappedGradientExchange(backend, dev, bucket_bytes=args.bucket_bytes, residual_blocks=16, fused_adamw=True,
                                              early_update_after_backward=not args.early_fused)
    else:
        grad = torch.zeros(params, device=dev)
    moves_h, target_h = cyclic_puzzle(72, 18)
    puzzle_pinned = torch.from_numpy(np.concatenate([moves_h.reshape(-1), target_h.reshape(-1)])).pin_memory()
    puzzle_dev = torch.empty_like(puzzle_pinned, device=dev)
    puzzle_dev.copy_(puzzle_pinned)
    moves_d = puzzle_dev[: 18 * 80]
    target_d = puzzle_dev[18 * 80:]
    states = torch.zeros(batch, 80, dtype=torch.uint8, device=dev)
    labels = torch.zeros(batch, device=dev)
    meta = torch.zeros(batch, 16, dtype=torch.uint8, device=dev)
    ws_floats = mgt.mlp_loss_grad_workspace_floats(shape, batch)
    workspace = torch.empty(ws_floats, device=dev)
    engine = mgt.Engine(local_rank)
    if exchange is not None and not args.no_early_range:
        assert engine.set_early_range_hook(exchange.early_callback) == 0
    walk_cfg = mgt.RandomWalkKernelConfig(batch, 1, 29)
    loss_pinned = torch.zeros(1).pin_memory()
    other_launches = 0

    def step(s: int, profile=None, marks=None):
        nonlocal other_launches

        def mark():
            if marks is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append(ev)

        mark()
        st = mgt.launch_random_walk_kernel(walk_cfg, SEED, 0, s, rank, moves_d, target_d, states, labels, meta)
        assert st == 0, st
        mark()
        cfg = mgt.AdamWKernelConfig(params, s + 1, LR)
        if exchange is not None:
            exchange.begin_step(cfg, w, w_half, m, v)
        st = engine.launch_mlp_loss_grad(shape, w, w_half, states, labels, batch, loss, grad, workspace, ws_floats,
                                         profile=profile, input_grad_position_tile=36,
                                         gradient_ready=exchange.callback if exchange is not None else None)
        assert st == 0, mgt.status_name(st)
        other_launches += 1
        mark()
        if exchange is not None:
            exchange.finish_step()
        if exchange is None or not exchange.fused:
            st = mgt.launch_adamw_kernel_with_half_mirror(cfg, w, w_half, grad, m, v)
            assert st == 0, st
            other_launches += 1
        mark()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
            torch.cuda.synchronize()

    for s in range(args.warmup):
        step(s)
    barrier()
    st, code = engine.check()
    assert st == 0, f"device status {code}"

    # ---- device-timed region: K steps, resident inputs --------------------------------------
    try:
        gpu_uuid = "GPU-" + str(torch.cuda.get_device_properties(local_rank).uuid)
    except Exception:
        gpu_uuid = None
    sampler = ClockSampler(local_rank, gpu_uuid) if rank == 0 else None
    if sampler is not None:
        time.sleep(0.3)
    launches0 = engine.launch_count + other_launches
    peer_comm = isinstance(backend, PeerBackend)
    comm_launches0 = backend.launch_count if peer_comm else 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_wall0 = time.time()
    e0.record()
    for s in range(args.steps):
        step(args.warmup + s)
    e1.record()
    barrier()
    t_wall1 = time.time()
    ms_total = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(ms_total, op=dist.ReduceOp.MAX)
    ms_step = float(ms_total.item()) / args.steps
    launches = engine.launch_count + other_launches - launches0
    if peer_comm:
        launches += backend.launch_count - comm_launches0
        st, code = backend.check()
        assert st == 0, f"communicator status {code}"
    clocks = sampler.stop(t_wall0, t_wall1) if sampler is not None else None
    final_loss = float(loss.item())
    st, code = engine.check()
    assert st == 0, f"device status {code}"

    # ---- end to end through the public call, as the reference trainer's loop runs it: the step's
    # host inputs (puzzle definition, 1520 B pinned) go to the device, the step runs, the loss (4 B)
    # comes back and the host waits for it, every step (tool:836-851).
    barrier()
    t0 = time.perf_counter()
    e2e_steps = max(3, args.steps // 2)
    for s in range(e2e_steps):
        puzzle_dev.copy_(puzzle_pinned, non_blocking=True)
        step(args.warmup + args.steps + s)
        loss_pinned.copy_(loss, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e2e_sec = torch.tensor([(time.perf_counter() - t0) / e2e_steps], device=dev)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(e2e_sec, op=dist.ReduceOp.MAX)
    e2e_value = batch * world / float(e2e_sec.item())

    # ---- roofline of the dominant kernel (embedding-forward one-hot GEMM), timed live with CUDA events
    # on the launching stream by the engine's stage timer, outside the timed region above.
    peaks = load_peaks()
    prof = mgt.BackwardProfile()
    emb_ms, grad_ms = [], []
    for s in range(3):
        step(args.warmup + args.steps + e2e_steps + s, profile=prof)
        emb_ms.append(prof.input_forward_ms)
        grad_ms.append(prof.input_grad_ms)
    stage_ms = {n: round(getattr(prof, n), 4) for n, _ in prof._fields_}
    # where a step's time goes on the compute stream (outside the timed region; the stage timer is off here): the walk
    # kernel, forward + backward (with the overlapped part of the exchange beside it), and what is left after backward
    # has ended - the exchange's tail and the optimizer work that was not overlapped.
    spans = np.zeros(3)
    timeline_steps = 5
    for s in range(timeline_steps):
        marks = []
        step(args.warmup + args.steps + e2e_steps + 3 + s, marks=marks)
        torch.cuda.synchronize()
        spans += np.array([marks[i].elapsed_time(marks[i + 1]) for i in range(3)])
    spans_t = torch.tensor(spans / timeline_steps, device=dev)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(spans_t, op=dist.ReduceOp.MAX)
    timeline_ms = dict(zip(("walk", "forward_backward", "after_backward"), (round(float(x), 4) for x in spans_t.tolist())))
    emb = float(np.median(emb_ms))
    algo_tflops = EMB_ALGO_FLOP_PER_CANDIDATE * batch / (emb * 1e-3) / 1e12
    exec_tflops = EMB_EXEC_FLOP_PER_CANDIDATE * batch / (emb * 1e-3) / 1e12
    roofline = {
        "kernel": "umma_gemm_kernel<one-hot forward> (embedding layer)", "bound": "tensor", "achieved": algo_tflops,
        "peak": peaks["tflops_burst"], "unit": "TFLOP/s", "frac": algo_tflops / peaks["tflops_burst"],
        "traffic": EMB_FWD_DRAM_BYTES_PER_LAUNCH if batch == BATCH else None,
        "traffic_source": EMB_FWD_DRAM_SOURCE if batch == BATCH else None,
        "peak_source": peaks["source"] + " (cuBLAS bf16 burst)", "ms_per_launch": emb,
        "executed_tflops": exec_tflops, "executed_frac": exec_tflops / peaks["tflops_burst"],
        "note": "achieved counts the 72 row-adds per candidate the layer needs; executed counts the dense one-hot MMA work",
    }

    # the other single-kernel stages, same live timer: algorithmic work of the stage / its time, against the measured peaks
    grad_t = float(np.median(grad_ms))
    tower_fwd_bytes = batch * (224 * 4 + 16 * 2 * 224 * 2 + 17 * 32 + 224 * 4)   # state in, 32 fp16 tape entries, sign bits, state out
    hidden_fwd_bytes = batch * (2560 * 2 + 224 * 4 + 224 * 2) + 2560 * 224 * 2    # a1 in, x fp32 + fp16 out, weights
    roofline_other = [
        {"kernel": "umma_gemm_kernel<one-hot gradient> (embedding table gradient)", "bound": "tensor", "ms_per_launch": grad_t,
         "achieved": EMB_ALGO_FLOP_PER_CANDIDATE * batch / (grad_t * 1e-3) / 1e12, "executed_tflops": 2 * 72 * 72 * 2560 * batch / (grad_t * 1e-3) / 1e12,
         "peak": peaks["tflops_burst"], "unit": "TFLOP/s", "executed_frac": 2 * 72 * 72 * 2560 * batch / (grad_t * 1e-3) / 1e12 / peaks["tflops_burst"]},
        {"kernel": "tower_chain_kernel<forward> (16 residual blocks)", "bound": "hbm", "ms_per_launch": stage_ms["residual_forward_ms"],
         "achieved": tower_fwd_bytes / (stage_ms["residual_forward_ms"] * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
         "frac": tower_fwd_bytes / (stage_ms["residual_forward_ms"] * 1e-3) / 1e9 / peaks["hbm_gbs"]},
        {"kernel": "umma_gemm_kernel (hidden layer forward)", "bound": "hbm", "ms_per_launch": stage_ms["hidden_forward_ms"],
         "achieved": hidden_fwd_bytes / (stage_ms["hidden_forward_ms"] * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
         "frac": hidden_fwd_bytes / (stage_ms["hidden_forward_ms"] * 1e-3) / 1e9 / peaks["hbm_gbs"]},
    ]

    comm_check = None
    if world > 1 and args.comm == "peer" and batch == BATCH:
        import torch.distributed as dist
        comm_check = check_gradient_exchange(torch, dist, mgt, backend, dev, world, params, args.bucket_bytes, (w, w_half, m, v))
    barrier()
    reference_gpu = None
    if not args.no_reference_gpu and batch == BATCH:
        # rank 0 starts the trainer processes on all GPUs; the other ranks wait on the host (a NCCL barrier would keep a
        # kernel polling on their GPUs and time-slice with the trainers)
        if rank == 0:
            reference_gpu = run_gpu_trainers_side_by_side(world, max(3, min(args.steps, args.reference_gpu_steps)))
        if world > 1:
            import torch.distributed as dist
            dist.barrier(group=host_group)

    if rank != 0:
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
            dist.destroy_process_group()
        if comm_check is not None and not comm_check["ok"]:
            sys.exit(1)
        return

    value = batch * world / (ms_step * 1e-3)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "config": workload_config(world), "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(puzzle_pinned.numel()), "d2h_bytes_per_step": 4},
        "gpu_launches": int(launches), "roofline": roofline, "roofline_other": roofline_other if batch == BATCH else None, "comm": (args.comm if world > 1 else "none"),
        "step_tflops_algorithmic": FLOP_PER_CANDIDATE * value / world / 1e12,
        "step_frac_of_fp16_peak": FLOP_PER_CANDIDATE * value / world / 1e12 / peaks["tflops_sustained"],
        "stage_ms": stage_ms, "timeline_ms": timeline_ms, "final_loss": final_loss, "comm_check": comm_check, "reference_gpu": reference_gpu,
    }
    if batch != BATCH:
        line["config"]["batch_per_rank"] = batch
        line["config"]["note"] = "reduced batch: profiler capture only, not a benchmark value"
    if not args.no_cpu_baseline and world == 1:
        cpu = run_reference_cpu(args, args.steps_cpu, args.warmup_cpu)
        line["cpu_baseline"] = cpu["cpu_baseline"]
    print(json.dumps(line), file=out, flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    if comm_check is not None and not comm_check["ok"]:
        sys.exit(1)


if __name__ == "__main__":
    main()
