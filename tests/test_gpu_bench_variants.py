"""The variant benchmarks (bench.py --workload variant) keep running: one short step loop each on one GPU, at a small
batch; the line must carry the contract's keys and a finite loss."""
import json
import math
import os
import subprocess
import sys

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("flags,dtype,launch_floor", [(["--variant", "p888_bn", "--variant-batch", "2048"], "f16", 150),
                                                      (["--variant", "wide", "--variant-batch", "1024"], "bf16", 150),
                                                      (["--variant", "wide", "--batch-norm", "--variant-batch", "1024"], "bf16", 300)])
def test_variant_line(flags, dtype, launch_floor):
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--workload", "variant", "--steps", "2", "--warmup", "3", *flags],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1, res.stdout                     # stdout carries the JSON line and nothing else
    line = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "dtype", "data", "config", "gpu_launches"):
        assert key in line, key
    assert line["dtype"] == dtype and line["n_gpus"] == 1 and line["value"] > 0
    assert math.isfinite(line["final_loss"]) and line["final_loss"] > 0
    assert line["gpu_launches"] >= launch_floor            # a layered step is hundreds of this library's launches


def test_optimizer_line_does_not_depend_on_zeros():
    """bench.py --workload optimizer: exact zeros in the gradient (dead units, padding columns) must not slow the AdamW
    kernel down - they once sent nearly every warp down the slow path of division and square root (0.117 against 0.080 ms)."""
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--workload", "optimizer", "--steps", "5", "--warmup", "3"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1, res.stdout
    line = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "dtype", "data", "config", "roofline", "gpu_launches"):
        assert key in line, key
    kinds = line["gradient_kinds"]
    assert set(kinds) == {"normal", "half_of_columns_zero", "all_zero", "zeros_and_denormals"}
    base = kinds["normal"]["ms"]
    assert base > 0 and line["gpu_launches"] == 20
    assert kinds["half_of_columns_zero"]["ms"] <= 1.15 * base
    assert kinds["all_zero"]["ms"] <= 1.15 * base
