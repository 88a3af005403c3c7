"""`mgt`: the configuration-file front end of the trainer.

    python -m multigputrainmlp_b200.mgt_cli print-default-config
    python -m multigputrainmlp_b200.mgt_cli validate-config CONFIG.toml
    python -m multigputrainmlp_b200.mgt_cli train CONFIG.toml OUTPUT_DIR

Stands where the reference's Rust command line stands (crates/trainer-cli/src/main.rs:41-46): the same three
subcommands, the same TOML keys, defaults and validation messages (config.rs:5-145), the same MGT_* environment
overrides and the same flag list handed to the rank binary (native.rs:13-134), the same config.snapshot.toml,
native.stdout/native.stderr and required-output check (native.rs:8-11,137-153). It starts ONE rank process
(`bin/mgt_native_train`, or whatever MGT_NATIVE_TRAIN_BIN names); several ranks are started by `launch.py`.
No arithmetic happens here. There is no Rust toolchain in this build's image, hence Python; nothing on the
training path depends on this module.
"""
from __future__ import annotations

import os
import subprocess
import sys
from dataclasses import dataclass, fields
from typing import Dict, List, Sequence

try:
    import tomllib
except ModuleNotFoundError:  # Python < 3.11
    tomllib = None

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEFAULT_TRAINER = os.path.join(ROOT, "bin", "mgt_native_train")
U32_MAX = 2 ** 32 - 1


class ConfigError(ValueError):
    pass


@dataclass
class TrainerConfig:
    """crates/trainer-cli/src/config.rs:5-36; the defaults are p888_default() (config.rs:39-72)."""
    group_id: int = 888
    target_id: int = 0
    state_len: int = 72
    state_alignment: int = 16
    state_value_pad: int = 72
    move_count: int = 18
    output_dim: int = 1
    hd1: int = 2556
    hd2: int = 218
    residual_blocks: int = 16
    hidden_alignment: int = 8
    batch_size: int = 100_000
    walkers: int = 34_482
    k_min: int = 1
    k_max: int = 29
    epochs: int = 32692
    learning_rate: float = 0.0001
    weight_decay: float = 0.0
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_eps: float = 1.0e-8
    base_seed: int = 0x0888_0000_0000_0001
    checkpoint_period_steps: int = 4096
    weight_export_period_steps: int = 4096
    gradient_carousel_slots: int = 3
    input_grad_partial_chunks: int = 1
    input_grad_positions_per_block: int = 1
    input_grad_fp16: bool = False
    linear_fp16: bool = False
    allreduce_bucket_bytes: int = 4 * 1024 * 1024

    @property
    def state_storage_len(self) -> int:
        a = self.state_alignment
        return self.state_len if a == 0 else (self.state_len + a - 1) // a * a

    @property
    def batch_states_per_rank(self) -> int:
        return self.batch_size

    def validate(self) -> None:
        """config.rs:82-145, same order and wording."""
        def pow2(v):
            return v != 0 and (v & (v - 1)) == 0
        checks = [
            (self.state_len == 0, "state_len must be positive"),
            (not pow2(self.state_alignment), "state_alignment must be a non-zero power of two"),
            (self.state_value_pad == 0, "state_value_pad must be positive"),
            (self.move_count == 0, "move_count must be positive"),
            (self.output_dim != 1, "output_dim must be 1 for the current native trainer"),
            (self.hd1 == 0 or self.hd2 == 0, "hidden dimensions must be positive"),
            (not pow2(self.hidden_alignment), "hidden_alignment must be a non-zero power of two"),
            (self.batch_size == 0 or self.batch_size > U32_MAX, "batch_size must fit into u32 and be positive"),
            (self.walkers == 0, "walkers must be positive"),
            (self.k_min == 0 or self.k_min > self.k_max, "invalid walk depth range"),
            (self.epochs == 0 or self.epochs > U32_MAX, "epochs must fit into u32 and be positive"),
            (self.learning_rate <= 0.0, "learning_rate must be positive"),
            (self.weight_decay < 0.0, "weight_decay must be non-negative"),
            (not 0.0 <= self.adam_beta1 < 1.0, "adam_beta1 must be in [0, 1)"),
            (not 0.0 <= self.adam_beta2 < 1.0, "adam_beta2 must be in [0, 1)"),
            (self.adam_eps <= 0.0, "adam_eps must be positive"),
            (self.gradient_carousel_slots == 0, "gradient_carousel_slots must be positive"),
            (self.input_grad_partial_chunks == 0, "input_grad_partial_chunks must be positive"),
            (self.input_grad_positions_per_block == 0, "input_grad_positions_per_block must be positive"),
            (self.allreduce_bucket_bytes == 0, "allreduce_bucket_bytes must be positive"),
        ]
        for bad, message in checks:
            if bad:
                raise ConfigError(message)

    def to_toml(self) -> str:
        """What `mgt print-default-config` prints: one `key = value` line per field, in declaration order."""
        lines = []
        for f in fields(self):
            v = getattr(self, f.name)
            if isinstance(v, bool):
                lines.append(f"{f.name} = {'true' if v else 'false'}")
            elif isinstance(v, float):
                lines.append(f"{f.name} = {_toml_float(v)}")
            else:
                lines.append(f"{f.name} = {v}")
        return "\n".join(lines) + "\n"

    @classmethod
    def from_toml(cls, text: str) -> "TrainerConfig":
        """Every key is required and unknown keys are ignored, as serde's derive does for the reference struct."""
        if tomllib is None:
            raise ConfigError("this Python has no tomllib (needs 3.11 or newer)")
        try:
            data = tomllib.loads(text)
        except tomllib.TOMLDecodeError as e:
            raise ConfigError(f"TOML parse error: {e}") from None
        values = {}
        for f in fields(cls):
            if f.name not in data:
                raise ConfigError(f"missing field `{f.name}`")
            v = data[f.name]
            if f.type == "bool":
                if not isinstance(v, bool):
                    raise ConfigError(f"invalid type for `{f.name}`: expected a boolean")
            elif f.type == "float":
                if isinstance(v, bool) or not isinstance(v, (int, float)):
                    raise ConfigError(f"invalid type for `{f.name}`: expected a float")
                v = float(v)
            else:
                if isinstance(v, bool) or not isinstance(v, int) or v < 0:
                    raise ConfigError(f"invalid type for `{f.name}`: expected an unsigned integer")
            values[f.name] = v
        return cls(**values)


def _f32_text(x: float) -> str:
    """The reference prints floats as Rust's `{}` of an f32: the shortest decimal that reads back as the same 32-bit value,
    never in exponent form, no trailing ".0" ("0.0001", "0", "0.00000001")."""
    import numpy as np
    return np.format_float_positional(np.float32(x), unique=True, trim="-")


def _toml_float(v: float) -> str:
    text = _f32_text(v)
    return text if "." in text else text + ".0"  # TOML wants a fractional part on a float


def config_snapshot(cfg: TrainerConfig) -> str:
    """config.snapshot.toml (native.rs:229-265): derived state_storage_len, `num_classes` for the value count, the seed
    as a quoted hexadecimal string, overlap_allreduce always true."""
    def b(x):
        return "true" if x else "false"

    f = _f32_text
    return (
        f"group_id = {cfg.group_id}\ntarget_id = {cfg.target_id}\nstate_len = {cfg.state_len}\nstate_alignment = {cfg.state_alignment}\n"
        f"state_storage_len = {cfg.state_storage_len}\nnum_classes = {cfg.state_value_pad}\nmove_count = {cfg.move_count}\n"
        f"output_dim = {cfg.output_dim}\nhd1 = {cfg.hd1}\nhd2 = {cfg.hd2}\nresidual_blocks = {cfg.residual_blocks}\n"
        f"hidden_alignment = {cfg.hidden_alignment}\nbatch_size = {cfg.batch_size}\nwalkers = {cfg.walkers}\nk_min = {cfg.k_min}\n"
        f"k_max = {cfg.k_max}\nepochs = {cfg.epochs}\nlearning_rate = {f(cfg.learning_rate)}\nweight_decay = {f(cfg.weight_decay)}\n"
        f"adam_beta1 = {f(cfg.adam_beta1)}\nadam_beta2 = {f(cfg.adam_beta2)}\nadam_eps = {f(cfg.adam_eps)}\n"
        f"base_seed = \"0x{cfg.base_seed:016x}\"\ncheckpoint_period_steps = {cfg.checkpoint_period_steps}\n"
        f"weight_export_period_steps = {cfg.weight_export_period_steps}\ngradient_carousel_slots = {cfg.gradient_carousel_slots}\n"
        f"input_grad_partial_chunks = {cfg.input_grad_partial_chunks}\ninput_grad_positions_per_block = {cfg.input_grad_positions_per_block}\n"
        f"input_grad_fp16 = {b(cfg.input_grad_fp16)}\nlinear_fp16 = {b(cfg.linear_fp16)}\noverlap_allreduce = true\n"
        f"allreduce_bucket_bytes = {cfg.allreduce_bucket_bytes}\n")


def _env_uint(env: Dict[str, str], name: str, default: int, limit: int) -> int:
    if name not in env:
        return default
    text = env[name]
    if not text.isdigit() or int(text) > limit:
        raise ConfigError(f"{name} must be an unsigned integer")
    return int(text)


def _env_float(env: Dict[str, str], name: str, default: float) -> float:
    if name not in env:
        return default
    try:
        return float(env[name])
    except ValueError:
        raise ConfigError(f"{name} must be a float") from None


def _env_bool(env: Dict[str, str], name: str, default: bool) -> bool:
    if name not in env:
        return default
    if env[name] in ("1", "true", "yes", "on"):
        return True
    if env[name] in ("0", "false", "no", "off"):
        return False
    raise ConfigError(f"{name} must be one of 1,0,true,false,yes,no,on,off")


def resolve_native_binary(env: Dict[str, str]) -> str:
    """MGT_NATIVE_TRAIN_BIN wins (native.rs:158-161); otherwise this repository's own trainer."""
    if "MGT_NATIVE_TRAIN_BIN" in env:
        return env["MGT_NATIVE_TRAIN_BIN"]
    if os.path.exists(DEFAULT_TRAINER):
        return DEFAULT_TRAINER
    raise ConfigError("native trainer binary not found; set MGT_NATIVE_TRAIN_BIN or build mgt_native_train")


def native_command(cfg: TrainerConfig, output_dir: str, env: Dict[str, str]) -> List[str]:
    """The rank binary's command line (native.rs:13-134): configuration values with their MGT_* overrides, flags in
    the reference's order."""
    u32, u64 = U32_MAX, 2 ** 64 - 1
    world_size = _env_uint(env, "MGT_WORLD_SIZE", 1, u32)
    global_rank = _env_uint(env, "MGT_GLOBAL_RANK", 0, u32)
    local_rank = _env_uint(env, "MGT_LOCAL_RANK", global_rank, u32)
    device_id = _env_uint(env, "MGT_DEVICE_ID", local_rank, u32)
    steps = _env_uint(env, "MGT_TRAIN_STEPS", cfg.epochs, u64)
    batch_size = _env_uint(env, "MGT_TRAIN_BATCH_SIZE", cfg.batch_states_per_rank, u64)
    k_min = _env_uint(env, "MGT_TRAIN_K_MIN", cfg.k_min, u32)
    k_max = _env_uint(env, "MGT_TRAIN_K_MAX", cfg.k_max, u32)
    pairs = [
        ("--output-dir", output_dir), ("--steps", steps), ("--device-id", device_id), ("--world-size", world_size),
        ("--global-rank", global_rank), ("--local-rank", local_rank),
        ("--group-id", _env_uint(env, "MGT_GROUP_ID", cfg.group_id, u32)),
        ("--target-id", _env_uint(env, "MGT_TARGET_ID", cfg.target_id, u32)),
        ("--state-len", _env_uint(env, "MGT_STATE_LEN", cfg.state_len, u32)),
        ("--state-value-count", _env_uint(env, "MGT_STATE_VALUE_COUNT", cfg.state_value_pad, u32)),
        ("--move-count", _env_uint(env, "MGT_MOVE_COUNT", cfg.move_count, u32)),
        ("--state-alignment", _env_uint(env, "MGT_STATE_ALIGNMENT", cfg.state_alignment, u32)),
        ("--batch-size", batch_size), ("--k-min", k_min), ("--k-max", k_max),
        ("--walkers", _env_uint(env, "MGT_WALKERS", cfg.walkers, u32)),
        ("--hd1", _env_uint(env, "MGT_TRAIN_HD1", cfg.hd1, u32)),
        ("--hd2", _env_uint(env, "MGT_TRAIN_HD2", cfg.hd2, u32)),
        ("--nrd", _env_uint(env, "MGT_TRAIN_NRD", cfg.residual_blocks, u32)),
        ("--output-dim", _env_uint(env, "MGT_OUTPUT_DIM", cfg.output_dim, u32)),
        ("--hidden-alignment", _env_uint(env, "MGT_HIDDEN_ALIGNMENT", cfg.hidden_alignment, u32)),
        ("--gradient-carousel-slots", _env_uint(env, "MGT_GRADIENT_CAROUSEL_SLOTS", cfg.gradient_carousel_slots, u32)),
        ("--input-grad-partial-chunks", _env_uint(env, "MGT_INPUT_GRAD_PARTIAL_CHUNKS", cfg.input_grad_partial_chunks, u32)),
        ("--input-grad-positions-per-block", _env_uint(env, "MGT_INPUT_GRAD_POSITIONS_PER_BLOCK", cfg.input_grad_positions_per_block, u32)),
        ("--input-grad-fp16", int(_env_bool(env, "MGT_INPUT_GRAD_FP16", cfg.input_grad_fp16))),
        ("--linear-fp16", int(_env_bool(env, "MGT_LINEAR_FP16", cfg.linear_fp16))),
        ("--overlap-allreduce", int(_env_bool(env, "MGT_OVERLAP_ALLREDUCE", True))),
        ("--allreduce-bucket-bytes", _env_uint(env, "MGT_ALLREDUCE_BUCKET_BYTES", cfg.allreduce_bucket_bytes, u64)),
        ("--seed", _env_uint(env, "MGT_SEED", cfg.base_seed, u64)),
        ("--lr", _f32_text(_env_float(env, "MGT_LR", cfg.learning_rate))),
        ("--weight-decay", _f32_text(_env_float(env, "MGT_WEIGHT_DECAY", cfg.weight_decay))),
        ("--write-artifacts", int(_env_bool(env, "MGT_WRITE_ARTIFACTS", True))),
    ]
    if steps == 0 or steps > U32_MAX or batch_size == 0 or batch_size > U32_MAX:
        raise ConfigError("MGT_TRAIN_STEPS and MGT_TRAIN_BATCH_SIZE must be positive u32 values")
    if k_min == 0 or k_min > k_max:
        raise ConfigError("invalid MGT_TRAIN_K_MIN/MGT_TRAIN_K_MAX range")
    cmd = [resolve_native_binary(env)]
    for flag, value in pairs:
        cmd += [flag, str(value)]
    if "MGT_NCCL_ID_FILE" in env:
        cmd += ["--nccl-id-file", env["MGT_NCCL_ID_FILE"]]
    if "MGT_RESUME_CHECKPOINT" in env:
        cmd += ["--resume-checkpoint", env["MGT_RESUME_CHECKPOINT"]]
    return cmd


def _require_file(path: str) -> None:
    if not os.path.exists(path):
        raise ConfigError(f"missing artifact {path}")
    if not os.path.isfile(path) or os.path.getsize(path) == 0:
        raise ConfigError(f"artifact {path} is empty or not a file")


def run_training(cfg: TrainerConfig, output_dir: str, env: Dict[str, str] | None = None) -> None:
    """native.rs:6-156."""
    env = dict(os.environ) if env is None else env
    os.makedirs(output_dir, exist_ok=True)
    with open(os.path.join(output_dir, "config.snapshot.toml"), "w") as f:
        f.write(config_snapshot(cfg))
    cmd = native_command(cfg, output_dir, env)
    try:
        res = subprocess.run(cmd, capture_output=True, env=env)
    except OSError as e:
        raise ConfigError(f"failed to launch native trainer {cmd[0]}: {e}") from None
    with open(os.path.join(output_dir, "native.stdout"), "wb") as f:
        f.write(res.stdout)
    with open(os.path.join(output_dir, "native.stderr"), "wb") as f:
        f.write(res.stderr)
    if res.returncode != 0:
        raise ConfigError(f"native trainer failed with status {res.returncode}")
    for name in ("metadata.env", "layers.json", "train.log", "profile.jsonl"):
        _require_file(os.path.join(output_dir, name))
    if "--write-artifacts" in cmd and cmd[cmd.index("--write-artifacts") + 1] == "1":
        for parts in (("weights", "manifest.json"), ("weights", "weights.f32.bin"), ("checkpoint", "manifest.json"), ("checkpoint", "state.f32.bin")):
            _require_file(os.path.join(output_dir, *parts))
    print("native_training_ok")


def main(argv: Sequence[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    usage = "usage: mgt <print-default-config | validate-config PATH | train CONFIG OUTPUT_DIR>"
    try:
        if argv == ["print-default-config"]:
            print(TrainerConfig().to_toml())
        elif len(argv) == 2 and argv[0] == "validate-config":
            TrainerConfig.from_toml(open(argv[1]).read()).validate()
            print("config_ok")
        elif len(argv) == 3 and argv[0] == "train":
            cfg = TrainerConfig.from_toml(open(argv[1]).read())
            cfg.validate()
            run_training(cfg, argv[2])
        else:
            print(usage, file=sys.stderr)
            return 2
    except (ConfigError, OSError) as e:
        print(f"Error: {e}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
