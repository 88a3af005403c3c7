"""The one-node launcher: command lines per rank and the reference's throughput formula
(kaggle/kernel/run_ranks_2xt4.sh:50-115). Host logic; the GPU run is at the end."""
import json
import os

import pytest

from multigputrainmlp_b200.launch import TRAINER, launch, rank_command, throughput_summary


def rows(ms, batch=100, loss=1.0):
    return [{"step": s, "milliseconds": m, "batch_states": batch, "loss": loss + s, "overlap_chunks": 3, "input_grad_backend": "x",
             "input_grad_position_tile": 36} for s, m in enumerate(ms)]


def test_summary_follows_the_reference_formula():
    # two ranks, three steps; step 0 is excluded, every step counts the slower rank
    s = throughput_summary([rows([50.0, 10.0, 20.0]), rows([60.0, 12.5, 16.0])])
    assert s["world_size"] == 2 and s["status"] == "ok" and s["batch_states_per_rank"] == 100
    assert [x["step"] for x in s["steady_steps"]] == [1, 2]
    assert s["steady_steps"][0]["max_rank_ms"] == 12.5 and s["steady_steps"][0]["throughput_states_s"] == 200 * 1000.0 / 12.5
    assert s["steady_steps"][1]["throughput_states_s"] == 200 * 1000.0 / 20.0
    assert s["avg_throughput_states_s"] == (16000.0 + 10000.0) / 2 and s["min_throughput_states_s"] == 10000.0
    assert s["steady_steps"][1]["rank_losses"] == [3.0, 3.0] and s["steady_steps"][1]["overlap_chunks"] == [3, 3]


def test_summary_uses_only_steps_every_rank_logged():
    s = throughput_summary([rows([5.0, 10.0, 20.0, 30.0]), rows([5.0, 10.0])])
    assert [x["step"] for x in s["steady_steps"]] == [1]
    assert throughput_summary([rows([5.0])])["status"] == "no_steady_steps"
    assert throughput_summary([])["status"] == "no_steady_steps"


def test_rank_command_lines():
    cmd = rank_command(3, 8, "runs/x", ["--steps", "2"])
    assert cmd[0] == TRAINER and cmd[-2:] == ["--steps", "2"]
    flags = dict(zip(cmd[1:-2:2], cmd[2:-2:2]))
    assert flags == {"--output-dir": os.path.join("runs/x", "rank3"), "--device-id": "3", "--world-size": "8", "--global-rank": "3",
                     "--local-rank": "3", "--nccl-id-file": os.path.join("runs/x", "nccl.id")}
    assert "--nccl-id-file" not in rank_command(0, 1, "runs/x", [])
    with pytest.raises(ValueError):
        launch(1, "runs/x", ["--device-id", "0"])


@pytest.mark.gpu
def test_launcher_runs_the_trainer(tmp_path):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    world = 2 if torch.cuda.device_count() >= 2 else 1
    s = launch(world, str(tmp_path / "run"), ["--steps", "3", "--batch-size", "256", "--hd1", "64", "--hd2", "32", "--nrd", "1", "--write-artifacts", "0"],
               timeout=300)
    assert s["status"] == "ok" and s["exit_codes"] == [0] * world and s["world_size"] == world
    assert [x["step"] for x in s["steady_steps"]] == [1, 2] and s["avg_throughput_states_s"] > 0
    assert json.load(open(tmp_path / "run" / "throughput_summary.json"))["world_size"] == world
    assert "native_train_smoke_ok" in open(tmp_path / "run" / "rank0.stdout").read()
