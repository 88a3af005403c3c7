"""The C-ABI library loads and exports every symbol include/mgt_b200.h declares (no GPU needed)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "mgt_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(mgt_[a-z0-9_]+)\s*\(", text))
    names -= {n for n in names if n.endswith(("_fn", "_t"))}
    return sorted(names)


def test_library_exports_every_declared_symbol():
    from multigputrainmlp_b200 import _lib
    lib = _lib.load()
    names = declared_functions()
    assert len(names) >= 25
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_only_declared_symbols_are_exported():
    import subprocess
    from multigputrainmlp_b200 import _lib
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True).stdout
    exported = {line.split()[-1] for line in out.splitlines() if " T " in line}
    ours = {n for n in exported if n.startswith("mgt_")}
    assert ours == set(declared_functions())


def test_host_side_validation_without_gpu():
    import multigputrainmlp_b200 as mgt
    assert mgt.status_name(0) == "ok" and mgt.status_name(3) == "capacity_exceeded" and mgt.status_name(7) == "device_timeout"
    assert mgt.validate_random_walk_kernel_config(mgt.RandomWalkKernelConfig(8, 1, 9)) == 0
    assert mgt.validate_random_walk_kernel_config(mgt.RandomWalkKernelConfig(8, 9, 1)) == 1
    assert mgt.validate_cuda_mlp_shape(mgt.CudaMlpShape(72, 72, 2560, 224, 16, 1)) == 0
    assert mgt.validate_cuda_mlp_shape(mgt.CudaMlpShape(72, 72, 4097, 224, 16, 1)) == 1   # native/cuda/mlp_forward.cu:7-9
    assert mgt.validate_cuda_mlp_shape(mgt.CudaMlpShape(72, 72, 16, 513, 1, 1)) == 1
    assert mgt.validate_cuda_mlp_shape(mgt.CudaMlpShape(72, 72, 16, 16, 33, 1)) == 1
    assert mgt.CudaMlpShape(72, 72, 2560, 224, 16, 1).param_count == 15460289
    assert mgt.CudaMlpShape(72, 72, 256, 64, 2, 1).param_count == 1360513
    assert mgt.CudaMlpShape(72, 72, 4096, 512, 32, 29).param_count == 40160285
    assert mgt.mlp_loss_grad_workspace_floats(mgt.CudaMlpShape(72, 72, 2560, 224, 16, 1), 53248) * 4 < 3 * 1024**3  # reference: ~6.8 GB
    assert mgt.validate_adamw_kernel_config(mgt.AdamWKernelConfig(8, 1, 1e-3)) == 0
    assert mgt.validate_adamw_kernel_config(mgt.AdamWKernelConfig(8, 1, 1e-3, weight_decay=-1.0)) == 1


def test_walk_launch_refuses_misaligned_arrays_before_any_launch():
    # host-side argument checks only: nothing reaches the device (there is none here)
    import multigputrainmlp_b200 as mgt
    cfg = mgt.RandomWalkKernelConfig(8, 1, 9)
    good = dict(moves=0x10000, target=0x20000, states=0x30000, labels=0x40000, meta=0x50000)
    for name, bad in (("moves", 0x10001), ("target", 0x20002), ("states", 0x30008), ("labels", 0x40002), ("meta", 0x50004)):
        a = dict(good)
        a[name] = bad
        assert mgt.launch_random_walk_kernel(cfg, 1, 0, 0, 0, a["moves"], a["target"], a["states"], a["labels"], a["meta"], stream=0) == 1, name
    assert mgt.launch_random_walk_kernel(mgt.RandomWalkKernelConfig(0, 1, 9), 1, 0, 0, 0, *good.values(), stream=0) == 1


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "multigputrainmlp_b200")
    for dirpath, _, files in os.walk(pkg):
        for name in files:
            if name.endswith((".py", ".cu", ".cuh", ".cpp", ".hpp", ".h")):
                text = open(os.path.join(dirpath, name)).read()
                assert "oracle" not in text.lower(), f"{name} mentions the oracle"
