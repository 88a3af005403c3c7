"""The mgt_native_train binary: process contract of the reference trainer (flags in, files out)
and numerical parity of whole training runs against the CPU oracle."""
import json
import os
import subprocess

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from helpers import rel_l2, trainer_init_weights  # noqa: E402
from oracle import MlpShape  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "bin", "mgt_native_train")
BASE = ["--device-id", "0", "--world-size", "1", "--global-rank", "0", "--local-rank", "0"]


def run(out_dir, *flags, check=True):
    cmd = [BIN, "--output-dir", str(out_dir), *BASE, *[str(f) for f in flags]]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    if check:
        assert res.returncode == 0, res.stderr + res.stdout
    return res


def oracle_training(oracle, *, hd1, hd2, nrd, out, batch, steps, k_min, k_max, seed=1234, lr=1e-4, wd=0.0, world=1, start=None, puzzle=None):
    """The reference trainer's loop on the CPU oracle (fp16 data flow), `world` ranks averaged in rank order."""
    shape = MlpShape(72, 72, hd1, hd2, nrd, out)
    moves, target = oracle.cyclic_puzzle(72, 18) if puzzle is None else puzzle
    w = trainer_init_weights(shape.param_count) if start is None else start[0].copy()
    m = np.zeros_like(w) if start is None else start[1].copy()
    v = np.zeros_like(w) if start is None else start[2].copy()
    losses = []
    for step in range(steps):
        grads, rank_losses = [], []
        for rank in range(world):
            _, states, labels, _ = oracle.random_walks(moves, target, seed=seed, epoch=0, step=step, rank=rank, k_min=k_min, k_max=k_max, samples=batch)
            lab = np.repeat(labels.reshape(-1, 1), out, axis=1)  # ExpandScalarLabelsKernel (tool:74-80)
            st, loss, grad = oracle.loss_grad_mixed(shape, w, states, np.ascontiguousarray(lab))
            assert st == 0
            grads.append(grad)
            rank_losses.append(loss)
        avg = oracle.allreduce_average(grads) if world > 1 else grads[0]
        assert oracle.adamw(w, avg, m, v, step=step + 1, lr=lr, wd=wd) == 0
        losses.append(rank_losses)
    return w, m, v, losses


def read_profile(path):
    return [json.loads(line) for line in open(path)]


def test_smoke_run_writes_the_reference_file_set(tmp_path, oracle):
    # ctest native_train_smoke + native_train_artifacts (native/CMakeLists.txt:177,191; tests/scripts/check_native_train_artifacts.sh)
    d = tmp_path / "smoke"
    res = run(d, "--steps", 2)
    assert res.stdout.strip().splitlines()[-1].startswith("native_train_smoke_ok loss=")
    for rel in ("train.log", "metadata.env", "layers.json", "linear_ops.json", "profile.jsonl", "weights/manifest.json", "weights/weights.f32.bin",
                "weights/input_weight_hxk.fp16", "weights/input_bias.fp16", "weights/hidden_weight_hxk.fp16", "weights/hidden_bias.fp16",
                "weights/residual0_fc1_weight_hxk.fp16", "weights/residual0_fc1_bias.fp16", "weights/residual0_fc2_weight_hxk.fp16",
                "weights/residual0_fc2_bias.fp16", "weights/output_weight_hxk.fp16", "weights/output_bias.fp16", "checkpoint/manifest.json",
                "checkpoint/state.f32.bin"):
        assert os.path.getsize(d / rel) > 0, rel
    man = open(d / "weights" / "manifest.json").read()
    for needle in ('"format": "stream1_weights"', '"dtype": "fp16"', '"num_classes": 72', '"hd1": 8', '"hd2": 8', '"original_hd1": 5', '"original_hd2": 3', '"nrd": 1'):
        assert needle in man
    cman = open(d / "checkpoint" / "manifest.json").read()
    assert '"format": "mgt_train_checkpoint"' in cman and '"sections": ["weights", "adam_m", "adam_v"]' in cman
    env = open(d / "metadata.env").read()
    for needle in ("OUTPUT_DIM=1", "HD1=5", "HD2=3", "NCCL_ENABLED=", "RESUME_CHECKPOINT=0", "INPUT_GRAD_BACKEND=dense_one_hot_half_gemm"):
        assert needle in env
    rows = read_profile(d / "profile.jsonl")
    assert len(rows) == 2 and all(k in rows[0] for k in ("milliseconds", "memory_bytes", "input_grad_backend", "batch_states", "loss", "bw_input_grad_ms"))
    assert rows[0]["batch_states"] == 64 and rows[0]["status"] == "ok"
    log = open(d / "train.log").read().splitlines()
    assert "phase=start batch_states=64 hd1=5 physical_hd1=8 hd2=3 physical_hd2=8 nrd=1 k_min=1 k_max=9" in log[0] and "phase=train loss=" in log[1]
    ops = json.load(open(d / "linear_ops.json"))
    assert ops["op_count"] == 14 and {"backend", "m"} <= set(ops["linear_ops"][0])

    # numerical parity of the whole run with the oracle: losses per step, final weights / m / v
    w, m, v, losses = oracle_training(oracle, hd1=8, hd2=8, nrd=1, out=1, batch=64, steps=2, k_min=1, k_max=9)
    for row, want in zip(rows, losses):
        assert abs(row["loss"] - want[0]) <= 1e-3 * abs(want[0])
    state = np.fromfile(d / "checkpoint" / "state.f32.bin", np.float32)
    p = w.size
    assert state.size == 3 * p
    assert rel_l2(state[:p], w) <= 1e-3 and rel_l2(state[p:2 * p], m) <= 1e-3 and rel_l2(state[2 * p:], v) <= 2e-3

    # ctest native_train_resume_smoke: restart from the checkpoint (step counter restarts, as in the reference)
    d2 = tmp_path / "resume"
    run(d2, "--steps", 1, "--resume-checkpoint", d / "checkpoint")
    assert "RESUME_CHECKPOINT=1" in open(d2 / "metadata.env").read() and "resumed=1" in open(d2 / "train.log").read()
    w2, _, _, losses2 = oracle_training(oracle, hd1=8, hd2=8, nrd=1, out=1, batch=64, steps=1, k_min=1, k_max=9,
                                        start=(state[:p], state[p:2 * p], state[2 * p:]))
    got = np.fromfile(d2 / "checkpoint" / "state.f32.bin", np.float32)[:p]
    assert rel_l2(got, w2) <= 1e-3
    assert abs(read_profile(d2 / "profile.jsonl")[0]["loss"] - losses2[0][0]) <= 1e-3 * abs(losses2[0][0])


@pytest.mark.parametrize("extra,out_dim", [((), 1), (("--write-artifacts", 0), 1), (("--lt-workspace-bytes", 1048576, "--write-artifacts", 0), 1),
                                           (("--output-dim", 3, "--write-artifacts", 0), 3), (("--output-dim", 128), 128)])
def test_profile_runs_of_the_reference_ctest_list(tmp_path, oracle, extra, out_dim):
    # native/CMakeLists.txt:181-186
    d = tmp_path / "run"
    batch = 17 if out_dim == 1 else 8
    run(d, "--steps", 1, "--batch-size", batch, "--k-min", 2, "--k-max", 5, "--hd1", 7, "--hd2", 4, "--backward-profile", 1, *extra)
    env = open(d / "metadata.env").read()
    assert f"OUTPUT_DIM={out_dim}\n" in env and "INPUT_GRAD_BACKEND=dense_one_hot_half_gemm\n" in env
    assert json.load(open(d / "layers.json"))["output_dim"] == out_dim
    row = read_profile(d / "profile.jsonl")[0]
    assert row["input_grad_backend"] == "dense_one_hot_half_gemm" and row["bw_input_forward_ms"] > 0
    assert os.path.exists(d / "weights" / "manifest.json") == ("--write-artifacts" not in extra)
    _, _, _, losses = oracle_training(oracle, hd1=8, hd2=8, nrd=1, out=out_dim, batch=batch, steps=1, k_min=2, k_max=5)
    assert abs(row["loss"] - losses[0][0]) <= 1e-3 * abs(losses[0][0])


def test_bad_command_lines_exit_1(tmp_path):
    for flags in (["--no-such-flag", "1"], ["--steps"], ["--steps", "0"], ["--k-min", "9", "--k-max", "2"], ["--state-len", "100"], ["--device-id", "99"]):
        res = subprocess.run([BIN, "--output-dir", str(tmp_path / "x"), *flags], capture_output=True, text=True, timeout=120)
        assert res.returncode == 1, flags
    res = subprocess.run([BIN, "--bogus", "1"], capture_output=True, text=True)
    assert res.stderr.startswith("usage: mgt_native_train")


def test_medium_model_training_run_tracks_the_oracle(tmp_path, oracle):
    d = tmp_path / "med"
    run(d, "--steps", 3, "--batch-size", 512, "--k-min", 1, "--k-max", 29, "--hd1", 250, "--hd2", 60, "--nrd", 2, "--lr", 0.001, "--weight-decay", 0.01,
        "--input-grad-position-tile", 36, "--persistent-half-weights", 0)
    env = open(d / "metadata.env").read()
    assert "PHYSICAL_HD1=256\n" in env and "PHYSICAL_HD2=64\n" in env and "INPUT_GRAD_BACKEND=position_tiled_one_hot_half_gemm\n" in env
    w, m, v, losses = oracle_training(oracle, hd1=256, hd2=64, nrd=2, out=1, batch=512, steps=3, k_min=1, k_max=29, lr=1e-3, wd=0.01)
    rows = read_profile(d / "profile.jsonl")
    for row, want in zip(rows, losses):
        assert abs(row["loss"] - want[0]) <= 1e-3 * abs(want[0])
    state = np.fromfile(d / "checkpoint" / "state.f32.bin", np.float32)
    p = w.size
    assert rel_l2(state[:p], w) <= 1e-3 and rel_l2(state[p:2 * p], m) <= 2e-3


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_run_keeps_replicas_identical(tmp_path, oracle):
    # kaggle/kernel/run_ranks_2xt4.sh:50-78: one process per rank, rendezvous through --nccl-id-file
    id_file = tmp_path / "nccl.id"
    procs = []
    for rank in range(2):
        cmd = [BIN, "--output-dir", str(tmp_path / f"rank{rank}"), "--steps", 3, "--device-id", rank, "--world-size", 2, "--global-rank", rank, "--local-rank", rank,
               "--batch-size", 256, "--k-min", 1, "--k-max", 29, "--hd1", 128, "--hd2", 32, "--nrd", 2, "--lr", 0.001, "--nccl-id-file", str(id_file),
               "--allreduce-bucket-bytes", 65536]
        procs.append(subprocess.Popen([str(c) for c in cmd], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                                      env=dict(os.environ, NCCL_NVLS_ENABLE="0")))
    outs = [p.communicate(timeout=300) for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    states = [np.fromfile(tmp_path / f"rank{r}" / "checkpoint" / "state.f32.bin", np.float32) for r in range(2)]
    assert np.array_equal(states[0], states[1])  # replicas bit-identical
    w, m, v, losses = oracle_training(oracle, hd1=128, hd2=32, nrd=2, out=1, batch=256, steps=3, k_min=1, k_max=29, lr=1e-3, world=2)
    p = w.size
    assert rel_l2(states[0][:p], w) <= 1e-3
    for r in range(2):
        rows = read_profile(tmp_path / f"rank{r}" / "profile.jsonl")
        assert rows[0]["overlap_allreduce"] == 1 and rows[0]["overlap_ranges"] == 7 and rows[0]["rank"] == r
        for row, want in zip(rows, losses):
            assert abs(row["loss"] - want[r]) <= 1e-3 * abs(want[r])
        assert "WORLD_SIZE=2\n" in open(tmp_path / f"rank{r}" / "metadata.env").read()


def test_resume_step_continues_the_run_bit_for_bit(tmp_path):
    # --resume-step 1 / --checkpoint-period-steps (beyond the reference's flags): 3 + 3 steps in two runs, the second
    # resumed from the periodic checkpoint of the first, end in the very state of 6 steps in one run
    common = ["--batch-size", 640, "--k-min", 1, "--k-max", 29, "--hd1", 128, "--hd2", 64, "--nrd", 2, "--lr", 0.001]
    run(tmp_path / "whole", "--steps", 6, *common)
    run(tmp_path / "first", "--steps", 4, "--checkpoint-period-steps", 3, *common)
    # the periodic checkpoint of step 3 was overwritten by the final one of step 4; make the 3-step one explicitly
    run(tmp_path / "three", "--steps", 3, *common)
    assert open(tmp_path / "three" / "checkpoint" / "step.txt").read().strip() == "3"
    assert open(tmp_path / "first" / "checkpoint" / "step.txt").read().strip() == "4"
    run(tmp_path / "second", "--steps", 3, "--resume-checkpoint", tmp_path / "three" / "checkpoint", "--resume-step", 1, *common)
    whole = np.fromfile(tmp_path / "whole" / "checkpoint" / "state.f32.bin", dtype=np.float32)
    second = np.fromfile(tmp_path / "second" / "checkpoint" / "state.f32.bin", dtype=np.float32)
    assert np.array_equal(whole, second)
    steps = [r["step"] for r in read_profile(tmp_path / "second" / "profile.jsonl")]
    assert steps == [3, 4, 5]
    losses_whole = [r["loss"] for r in read_profile(tmp_path / "whole" / "profile.jsonl")]
    losses_second = [r["loss"] for r in read_profile(tmp_path / "second" / "profile.jsonl")]
    assert losses_whole[3:] == losses_second
    # the reference's behaviour stays the default: the step count restarts
    run(tmp_path / "restart", "--steps", 2, "--resume-checkpoint", tmp_path / "three" / "checkpoint", *common)
    assert [r["step"] for r in read_profile(tmp_path / "restart" / "profile.jsonl")] == [0, 1]
    res = run(tmp_path / "bad", "--steps", 1, "--resume-checkpoint", tmp_path / "nowhere", "--resume-step", 1, *common, check=False)
    assert res.returncode != 0


def test_puzzle_from_files_drives_the_walks(tmp_path, oracle):
    # --puzzle-json / --target-bin (beyond the reference trainer, which only knows its built-in cyclic shifts): a random
    # generator set in the reference loader's file format; the run must follow the oracle trained on those moves
    import multigputrainmlp_b200 as mgt
    rng = np.random.default_rng(21)
    perms = [rng.permutation(72) for _ in range(18)]
    jp = tmp_path / "puzzle.json"
    jp.write_text(json.dumps({"group_id": 888, "state_len": 72, "move_count": 18, "moves": [[int(v) for v in p] for p in perms]}))
    tp = tmp_path / "target.bin"
    tp.write_bytes(bytes(range(72)))
    st, moves, target = mgt.load_puzzle_definition(jp, tp)
    assert st == 0
    cfg = dict(hd1=64, hd2=32, nrd=2, out=1, batch=512, steps=3, k_min=1, k_max=29, lr=1e-3)
    run(tmp_path / "run", "--steps", 3, "--batch-size", 512, "--k-min", 1, "--k-max", 29, "--hd1", 64, "--hd2", 32, "--nrd", 2, "--lr", 0.001,
        "--puzzle-json", jp, "--target-bin", tp)
    w, m, v, losses = oracle_training(oracle, puzzle=(moves, target), **cfg)
    got = [r["loss"] for r in read_profile(tmp_path / "run" / "profile.jsonl")]
    for a, b in zip(got, losses):
        assert abs(a - b[0]) <= 1e-3 * abs(b[0])
    state = np.fromfile(tmp_path / "run" / "checkpoint" / "state.f32.bin", dtype=np.float32)
    p = w.size
    # the first moment is linear in the gradients; the weights themselves are looser here: random generators visit every
    # table row with a few samples, and where such a tiny gradient component changes sign Adam moves the weight the other way
    assert rel_l2(state[p:2 * p], m) <= 2e-3
    assert rel_l2(state[:p], w) <= 5e-2
    # and it is a different run from the built-in puzzle
    run(tmp_path / "builtin", "--steps", 3, "--batch-size", 512, "--k-min", 1, "--k-max", 29, "--hd1", 64, "--hd2", 32, "--nrd", 2, "--lr", 0.001)
    builtin = np.fromfile(tmp_path / "builtin" / "checkpoint" / "state.f32.bin", dtype=np.float32)
    table = 72 * 72 * 64  # depths, hence step-0 losses, do not depend on the moves; which table rows get gradients does
    assert rel_l2(builtin[p:p + table], m[:table]) > 0.5
    assert run(tmp_path / "bad", "--steps", 1, "--puzzle-json", jp, check=False).returncode != 0
