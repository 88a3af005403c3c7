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
