"""One-node multi-rank launcher for bin/mgt_native_train: one process per GPU, file rendezvous, and the
reference's throughput summary.

    python -m multigputrainmlp_b200.launch --gpus 8 --run-dir runs/p888 -- --steps 200 --batch-size 53248 \\
        --k-min 1 --k-max 29 --hd1 2556 --hd2 218 --nrd 16 --write-artifacts 0

plays the role of the reference's kaggle/kernel/run_ranks_2xt4.sh:50-78: rank r gets --device-id r --global-rank r
--local-rank r --world-size N --output-dir <run-dir>/rank<r> --nccl-id-file <run-dir>/nccl.id, its stdout goes to
<run-dir>/rank<r>.stdout, and when all ranks have ended the per-step rows of every rank's profile.jsonl are folded
into <run-dir>/throughput_summary.json with the formula of that script (:95-115): for every step all ranks logged,
step 0 excluded, throughput = sum over ranks of batch_states * 1000 / max over ranks of milliseconds; the headline is the
mean over those steps.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
from typing import Dict, List, Sequence

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRAINER = os.path.join(ROOT, "bin", "mgt_native_train")
PER_RANK_FLAGS = ("--output-dir", "--device-id", "--world-size", "--global-rank", "--local-rank", "--nccl-id-file")


def throughput_summary(rank_rows: Sequence[Sequence[dict]]) -> dict:
    """rank_rows[r] = the parsed profile.jsonl rows of rank r. Same keys as the reference's summary."""
    summary: Dict[str, object] = {"world_size": len(rank_rows), "steady_steps": [], "status": "ok"}
    if rank_rows and rank_rows[0]:
        first = rank_rows[0][0]
        summary["input_grad_backend"] = first.get("input_grad_backend")
        summary["input_grad_position_tile"] = first.get("input_grad_position_tile")
        summary["batch_states_per_rank"] = first.get("batch_states")
    steady: List[dict] = []
    if rank_rows:
        by_step = [{int(row["step"]): row for row in rows} for rows in rank_rows]
        common = sorted(set.intersection(*(set(d) for d in by_step)))
        for step in common:
            if step == 0:  # carries the one-time set-up cost
                continue
            rows = [d[step] for d in by_step]
            batch = sum(int(r["batch_states"]) for r in rows)
            slowest = max(float(r["milliseconds"]) for r in rows)
            steady.append({
                "step": step, "global_batch_states": batch, "max_rank_ms": slowest, "throughput_states_s": batch * 1000.0 / slowest,
                "rank_ms": [float(r["milliseconds"]) for r in rows], "rank_losses": [float(r["loss"]) for r in rows],
                "overlap_chunks": [int(r.get("overlap_chunks", 0)) for r in rows],
            })
    summary["steady_steps"] = steady
    if steady:
        values = [s["throughput_states_s"] for s in steady]
        summary["avg_throughput_states_s"] = sum(values) / len(values)
        summary["min_throughput_states_s"] = min(values)
        summary["max_throughput_states_s"] = max(values)
    else:
        summary["status"] = "no_steady_steps"
    return summary


def rank_command(rank: int, world: int, run_dir: str, trainer_flags: Sequence[str], trainer: str = TRAINER) -> List[str]:
    cmd = [trainer, "--output-dir", os.path.join(run_dir, f"rank{rank}"), "--device-id", str(rank), "--world-size", str(world),
           "--global-rank", str(rank), "--local-rank", str(rank)]
    if world > 1:
        cmd += ["--nccl-id-file", os.path.join(run_dir, "nccl.id")]
    return cmd + list(trainer_flags)


def launch(gpus: int, run_dir: str, trainer_flags: Sequence[str], trainer: str = TRAINER, timeout: float | None = None) -> dict:
    clash = [f for f in trainer_flags if f in PER_RANK_FLAGS]
    if clash:
        raise ValueError(f"set by the launcher, not by the caller: {clash}")
    os.makedirs(run_dir, exist_ok=True)
    id_file = os.path.join(run_dir, "nccl.id")
    if os.path.exists(id_file):
        os.remove(id_file)  # a stale rendezvous file would be read by the new ranks
    procs = []
    for rank in range(gpus):
        out = open(os.path.join(run_dir, f"rank{rank}.stdout"), "w")
        procs.append((subprocess.Popen(rank_command(rank, gpus, run_dir, trainer_flags, trainer), stdout=out, stderr=subprocess.STDOUT), out))
    codes = []
    for proc, out in procs:
        try:
            codes.append(proc.wait(timeout=timeout))
        except subprocess.TimeoutExpired:
            proc.kill()  # the process started above, by its own handle
            codes.append(-9)
        out.close()
    rank_rows = []
    for rank in range(gpus):
        path = os.path.join(run_dir, f"rank{rank}", "profile.jsonl")
        rows = [json.loads(line) for line in open(path)] if os.path.exists(path) else []
        rank_rows.append([r for r in rows if r])
    summary = throughput_summary(rank_rows)
    summary["exit_codes"] = codes
    if any(codes):
        summary["status"] = "rank_failed"
    with open(os.path.join(run_dir, "throughput_summary.json"), "w") as f:
        json.dump(summary, f, indent=2)
    return summary


def main(argv: Sequence[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    rest: List[str] = []
    if "--" in argv:
        cut = argv.index("--")
        argv, rest = argv[:cut], argv[cut + 1:]
    ap = argparse.ArgumentParser(prog="python -m multigputrainmlp_b200.launch", description=__doc__.split("\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--run-dir", required=True)
    ap.add_argument("--timeout", type=float, default=None)
    args = ap.parse_args(argv)
    summary = launch(args.gpus, args.run_dir, rest, timeout=args.timeout)
    print("rank_launch_ok world_size=%d" % args.gpus if summary["status"] == "ok" else "rank_launch_failed status=%s" % summary["status"])
    print("throughput_summary=", json.dumps(summary, sort_keys=True), flush=True)
    return 0 if summary["status"] == "ok" else 1


if __name__ == "__main__":
    sys.exit(main())
