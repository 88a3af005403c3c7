"""The `mgt` front end (configuration file -> rank binary), after the reference's own launcher tests:
crates/trainer-cli/tests/config_contract.rs and native_artifacts.rs (a fake rank binary that echoes its flags)."""
import os
import stat

import pytest

from multigputrainmlp_b200 import mgt_cli
from multigputrainmlp_b200.mgt_cli import ConfigError, TrainerConfig

pytestmark = pytest.mark.skipif(mgt_cli.tomllib is None, reason="needs tomllib (Python 3.11+)")


def test_p888_default_matches_static_contract():
    cfg = TrainerConfig()
    assert (cfg.group_id, cfg.target_id, cfg.state_len, cfg.state_storage_len, cfg.state_alignment) == (888, 0, 72, 80, 16)
    assert (cfg.state_value_pad, cfg.move_count, cfg.output_dim, cfg.hd1, cfg.hd2, cfg.hidden_alignment) == (72, 18, 1, 2556, 218, 8)
    assert (cfg.batch_states_per_rank, cfg.walkers, cfg.gradient_carousel_slots) == (100_000, 34_482, 3)
    assert (cfg.input_grad_partial_chunks, cfg.input_grad_positions_per_block) == (1, 1)
    assert not cfg.input_grad_fp16 and not cfg.linear_fp16 and cfg.allreduce_bucket_bytes == 4 * 1024 * 1024
    cfg.validate()


def test_state_padding_and_rejections():
    cfg = TrainerConfig(group_id=123, target_id=7, state_len=31, state_alignment=16, state_value_pad=11, move_count=5, hd1=33, hd2=37)
    assert cfg.state_storage_len == 32
    cfg.validate()
    for change, word in ((dict(output_dim=2), "output_dim"), (dict(state_alignment=10), "state_alignment"), (dict(k_min=0), "walk depth"),
                         (dict(batch_size=2 ** 32), "batch_size"), (dict(adam_beta1=1.0), "adam_beta1"), (dict(learning_rate=0.0), "learning_rate")):
        with pytest.raises(ConfigError, match=word):
            TrainerConfig(**change).validate()


def test_default_config_toml_round_trips(capsys):
    assert mgt_cli.main(["print-default-config"]) == 0
    text = capsys.readouterr().out
    assert "hd1 = 2556" in text and "learning_rate = 0.0001" in text and "input_grad_fp16 = false" in text
    assert f"base_seed = {0x0888_0000_0000_0001}" in text
    parsed = TrainerConfig.from_toml(text)
    assert parsed == TrainerConfig()
    with pytest.raises(ConfigError, match="missing field `hd2`"):
        TrainerConfig.from_toml(text.replace("hd2 = 218\n", ""))
    with pytest.raises(ConfigError, match="linear_fp16"):
        TrainerConfig.from_toml(text.replace("linear_fp16 = false", "linear_fp16 = 3"))


def test_validate_config_command(tmp_path, capsys):
    path = tmp_path / "c.toml"
    path.write_text(TrainerConfig().to_toml())
    assert mgt_cli.main(["validate-config", str(path)]) == 0
    assert capsys.readouterr().out.strip() == "config_ok"
    path.write_text(TrainerConfig(output_dim=3).to_toml())
    assert mgt_cli.main(["validate-config", str(path)]) == 1
    assert "output_dim must be 1" in capsys.readouterr().err
    assert mgt_cli.main(["bogus"]) == 2


FAKE_RANK_BINARY = r"""#!/usr/bin/env bash
set -euo pipefail
out=""
declare -A seen
order=""
while [ "$#" -gt 0 ]; do
  seen["$1"]="$2"; order="$order $1"
  if [ "$1" = "--output-dir" ]; then out="$2"; fi
  shift 2
done
mkdir -p "$out/weights" "$out/checkpoint"
{ echo "MODEL_MODE=MLP2RB"; echo "OUTPUT_DIM=1"; for k in "${!seen[@]}"; do echo "FLAG${k}=${seen[$k]}"; done; echo "ORDER=$order"; } > "$out/metadata.env"
echo '{"output_dim": 1}' > "$out/layers.json"
echo "rank=0 phase=train steps=${seen[--steps]}" > "$out/train.log"
echo '{"milliseconds":1.0}' > "$out/profile.jsonl"
if [ "${FAKE_SKIP_WEIGHTS:-0}" != "1" ]; then
  echo '{"format":"stream1_weights"}' > "$out/weights/manifest.json"; printf 'weights' > "$out/weights/weights.f32.bin"
fi
echo '{"format":"mgt_train_checkpoint"}' > "$out/checkpoint/manifest.json"; printf 'checkpoint' > "$out/checkpoint/state.f32.bin"
echo "fake native ok"
"""


def _fake_binary(tmp_path):
    path = tmp_path / "fake_native_train.sh"
    path.write_text(FAKE_RANK_BINARY)
    path.chmod(path.stat().st_mode | stat.S_IEXEC)
    return str(path)


def test_training_entry_invokes_native_rank_binary(tmp_path, capsys):
    cfg = TrainerConfig(state_len=31, state_alignment=16, state_value_pad=11, move_count=5, hidden_alignment=8, gradient_carousel_slots=4,
                        input_grad_partial_chunks=1, input_grad_fp16=True, linear_fp16=True, allreduce_bucket_bytes=1_048_576,
                        learning_rate=0.0003, weight_decay=0.0)
    cfg.validate()
    out = tmp_path / "run"
    env = {"PATH": os.environ["PATH"], "MGT_NATIVE_TRAIN_BIN": _fake_binary(tmp_path), "MGT_TRAIN_STEPS": "2", "MGT_TRAIN_BATCH_SIZE": "17",
           "MGT_TRAIN_HD1": "7", "MGT_TRAIN_HD2": "4", "MGT_GLOBAL_RANK": "3", "MGT_NCCL_ID_FILE": "/tmp/x.id"}
    mgt_cli.run_training(cfg, str(out), env)
    assert capsys.readouterr().out.strip() == "native_training_ok"
    meta = dict(line.split("=", 1) for line in open(out / "metadata.env").read().splitlines())
    assert meta["MODEL_MODE"] == "MLP2RB" and meta["FLAG--hd1"] == "7" and meta["FLAG--hd2"] == "4" and meta["FLAG--steps"] == "2"
    assert meta["FLAG--batch-size"] == "17" and meta["FLAG--state-len"] == "31" and meta["FLAG--state-value-count"] == "11"
    assert meta["FLAG--gradient-carousel-slots"] == "4" and meta["FLAG--input-grad-fp16"] == "1" and meta["FLAG--linear-fp16"] == "1"
    assert meta["FLAG--overlap-allreduce"] == "1" and meta["FLAG--allreduce-bucket-bytes"] == "1048576" and meta["FLAG--lr"] == "0.0003"
    assert meta["FLAG--weight-decay"] == "0" and meta["FLAG--seed"] == str(0x0888_0000_0000_0001)
    # ranks: local rank and device follow the global rank unless set (native.rs:13-16)
    assert meta["FLAG--global-rank"] == meta["FLAG--local-rank"] == meta["FLAG--device-id"] == "3" and meta["FLAG--nccl-id-file"] == "/tmp/x.id"
    # the reference's flag order (native.rs:63-134)
    assert meta["ORDER"].split()[:8] == ["--output-dir", "--steps", "--device-id", "--world-size", "--global-rank", "--local-rank", "--group-id", "--target-id"]
    assert meta["ORDER"].split()[-2:] == ["--write-artifacts", "--nccl-id-file"]
    snap = open(out / "config.snapshot.toml").read()
    assert "state_storage_len = 32\nnum_classes = 11\n" in snap and 'base_seed = "0x0888000000000001"' in snap
    assert "learning_rate = 0.0003\nweight_decay = 0\nadam_beta1 = 0.9\nadam_beta2 = 0.999\nadam_eps = 0.00000001\n" in snap
    assert "overlap_allreduce = true\n" in snap
    assert open(out / "native.stdout").read().strip() == "fake native ok"


def test_missing_outputs_and_bad_overrides_are_errors(tmp_path):
    cfg = TrainerConfig()
    base = {"PATH": os.environ["PATH"], "MGT_NATIVE_TRAIN_BIN": _fake_binary(tmp_path), "MGT_TRAIN_STEPS": "1"}
    with pytest.raises(ConfigError, match="weights"):
        mgt_cli.run_training(cfg, str(tmp_path / "a"), {**base, "FAKE_SKIP_WEIGHTS": "1"})
    mgt_cli.run_training(cfg, str(tmp_path / "b"), {**base, "FAKE_SKIP_WEIGHTS": "1", "MGT_WRITE_ARTIFACTS": "0"})  # nothing to require then
    with pytest.raises(ConfigError, match="MGT_TRAIN_STEPS"):
        mgt_cli.run_training(cfg, str(tmp_path / "c"), {**base, "MGT_TRAIN_STEPS": "0"})
    with pytest.raises(ConfigError, match="MGT_LINEAR_FP16"):
        mgt_cli.run_training(cfg, str(tmp_path / "d"), {**base, "MGT_LINEAR_FP16": "maybe"})
    with pytest.raises(ConfigError, match="unsigned integer"):
        mgt_cli.run_training(cfg, str(tmp_path / "e"), {**base, "MGT_TRAIN_HD1": "-3"})
    with pytest.raises(ConfigError, match="K_MIN"):
        mgt_cli.run_training(cfg, str(tmp_path / "f"), {**base, "MGT_TRAIN_K_MIN": "9", "MGT_TRAIN_K_MAX": "3"})
