#!/usr/bin/env python
"""The AdamW kernel alone, on gradients with and without exact zeros.

    python bench.py --workload optimizer [--steps K --warmup W]

The full p888 parameter count (15 460 289 fp32 weights + fp16 mirror, 30 bytes per parameter through HBM), one launch of
`mgt_launch_adamw_with_half_mirror` per timed iteration between CUDA events, a buffer larger than L2 written before every
launch. Four gradients: all normal numbers; half of the 2560 hidden-layer columns exactly zero (units whose ReLU never
opens, padding columns: what a real step produces); all zero; zeros, negative zeros and denormals mixed in. Exact zeros
used to send nearly every warp down the slow path of the correctly rounded division and square root; the line shows
whether the kernel still depends on the data. `value` is the slowest of the first three kinds; denormal operands still
take the slow path (a moment of a unit that died decays through that range for about 150 steps) and are listed beside
it. One GPU; prints ONE JSON line.
"""
from __future__ import annotations

import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

PARAMS = 15460289
BYTES_PER_PARAM = 30  # w, m, v read and written, gradient read, fp16 mirror written
MODES = ("normal", "half_of_columns_zero", "all_zero", "zeros_and_denormals")


def gradient(mode: str, params: int = PARAMS) -> np.ndarray:
    """Deterministic gradient of the given kind (numpy only: the host test checks the kinds)."""
    idx = np.arange(params, dtype=np.uint64)
    h = (idx * np.uint64(0x9E3779B97F4A7C15)) >> np.uint64(40)
    g = (1e-4 * ((h % np.uint64(2001)).astype(np.float32) - 1000.0) / 1000.0).astype(np.float32)
    if mode == "half_of_columns_zero":
        col = idx % np.uint64(2560)
        g[((col * np.uint64(2654435761)) >> np.uint64(7)) & np.uint64(1) == 1] = 0.0
    elif mode == "all_zero":
        g[:] = 0.0
    elif mode == "zeros_and_denormals":
        k = h % np.uint64(7)
        for kind, value in enumerate((0.0, -0.0, 1e-41, -3e-39, 1e-20)):
            g[k == kind] = np.float32(value)
    elif mode != "normal":
        raise ValueError(mode)
    return g


def run(args) -> dict:
    import torch
    import multigputrainmlp_b200 as mgt

    if int(os.environ.get("WORLD_SIZE", "1")) > 1 and int(os.environ.get("RANK", "0")) != 0:
        return {}
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU fallback")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    idx = np.arange(PARAMS, dtype=np.int64)
    w0 = torch.from_numpy(((idx % 29 - 14) * 0.0001).astype(np.float32)).to(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    w_half = torch.zeros(PARAMS, dtype=torch.half, device=dev)
    out, launches = {}, 0
    for mode in MODES:
        g = torch.from_numpy(gradient(mode)).to(dev)
        w = w0.clone()
        m = torch.zeros(PARAMS, device=dev)
        v = torch.zeros(PARAMS, device=dev)
        times = []
        for it in range(warmup + steps):
            flush.fill_(it & 255)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            st = mgt.launch_adamw_kernel_with_half_mirror(mgt.AdamWKernelConfig(PARAMS, it + 1, 1e-4), w, w_half, g, m, v)
            e1.record()
            assert st == 0, mgt.status_name(st)
            torch.cuda.synchronize()
            if it >= warmup:
                times.append(e0.elapsed_time(e1))
                launches += 1
        ms = float(np.median(times))
        out[mode] = {"ms": round(ms, 4), "gbs": round(PARAMS * BYTES_PER_PARAM / ms * 1e-6, 1)}
        assert bool(torch.isfinite(w).all())
    peaks = {}
    try:
        import json
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except (OSError, ValueError):
        pass
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    worst = max(out[mode]["ms"] for mode in MODES[:3])
    return {
        "metric": "AdamW + fp16 mirror, HBM GB/s on the slowest of normal / half-zero / all-zero gradients (device-timed, one launch per iteration)",
        "value": round(PARAMS * BYTES_PER_PARAM / worst * 1e-6, 1), "unit": "GB/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": worst, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "optimizer microbench: AdamW on %d parameters" % PARAMS, "l2": "256 MB written before every launch"},
        "gradient_kinds": out,
        "roofline": {"bound": "hbm", "achieved": round(PARAMS * BYTES_PER_PARAM / worst * 1e-6, 1), "peak": hbm, "unit": "GB/s",
                     "frac": round(PARAMS * BYTES_PER_PARAM / worst * 1e-6 / hbm, 4), "traffic": None,
                     "peak_source": "measured (copy)" if "hbm_gbs" in peaks else "fallback"},
        "gpu_launches": launches,
    }
