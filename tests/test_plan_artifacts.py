"""Host-side plan numbers against the reference's BuildTrainPlan (golden fixture) and the byte
format of the output files (metadata.env, layers.json, linear_ops.json, weights/, checkpoint/)."""
import ctypes as C
import json
import os

import numpy as np
import pytest

from multigputrainmlp_b200 import _lib


def _argv(flags: dict):
    items = []
    for k, v in flags.items():
        items += [k.encode(), str(v).encode()]
    arr = (C.c_char_p * len(items))(*items)
    return len(items), arr


def plan_summary(**flags):
    lib = _lib.load()
    n, arr = _argv({"--" + k.replace("_", "-"): v for k, v in flags.items()})
    out = (C.c_uint64 * 16)()
    st = lib.mgt_plan_summary(n, arr, out, 16)
    keys = ["padded_state_dim", "physical_hd1", "physical_hd2", "blocks", "linear_ops", "gradient_buckets", "total_params", "total_bytes",
            "total_rank_bytes", "training_scratch_bytes", "logical_params", "fits_state_record", "states_bytes", "layout_allreduce_bytes",
            "walkers", "state_capacity_bytes"]
    return st, dict(zip(keys, [int(x) for x in out]))


P888 = dict(hd1=2556, hd2=218, nrd=16, k_max=29)


def test_plan_numbers_match_reference_golden(golden):
    g = golden.plan
    keys = [str(k) for k in g["keys"]]
    cases = {
        "p888": dict(batch_size=100000, **P888),
        "p888_b53248_w8": dict(batch_size=53248, world_size=8, global_rank=3, **P888),
        "synthetic": dict(state_len=31, state_value_count=37, move_count=11, hd1=64, hd2=33, nrd=2, batch_size=1234, allreduce_bucket_bytes=4096),
        "tiny": dict(state_len=17, state_value_count=9, hd1=31, hd2=19, nrd=2, batch_size=512),
        "config0": dict(hd1=256, hd2=64, nrd=2, batch_size=1024),
        "config3": dict(hd1=4096, hd2=512, nrd=32, output_dim=29, batch_size=131072),
    }
    for name, flags in cases.items():
        st, got = plan_summary(**flags)
        assert st == 0, name
        want = dict(zip(keys, [int(x) for x in g[name]]))
        for k, v in want.items():
            assert got[k] == v, (name, k, got[k], v)
    # numbers the reference's own tests pin (native/tests/test_train_plan.cpp, test_model_layout.cpp)
    st, p = plan_summary(batch_size=100000, **P888)
    assert (p["padded_state_dim"], p["physical_hd2"], p["blocks"], p["linear_ops"], p["total_params"]) == (80, 224, 70, 104, 15460289)
    assert p["total_bytes"] % 64 == 0 and p["fits_state_record"] == 1 and p["layout_allreduce_bytes"] == 3 * p["total_bytes"]
    st, p = plan_summary(state_len=31, state_value_count=37, move_count=11, hd1=64, hd2=33, nrd=2, batch_size=1234, allreduce_bucket_bytes=4096)
    assert (p["padded_state_dim"], p["physical_hd2"], p["blocks"], p["states_bytes"]) == (32, 40, 14, 1234 * 32) and p["gradient_buckets"] >= 2


def test_linear_op_manifest_matches_reference(golden):
    lib = _lib.load()
    rows = golden.plan["p888_linear_ops_b32768"]
    n, arr = _argv({"--hd1": 2556, "--hd2": 218, "--nrd": 16, "--batch-size": 32768})
    for i in range(104):
        out = (C.c_uint32 * 14)()
        assert lib.mgt_plan_linear_op(n, arr, i, out, 14) == 0
        assert [int(x) for x in out] == [int(x) for x in rows[i]], i
    out = (C.c_uint32 * 14)()
    assert lib.mgt_plan_linear_op(n, arr, 104, out, 14) == 1
    # the large-K candidate class (native/tests/test_train_plan.cpp:103-113); such a state does not fit the 80-byte record
    n, arr = _argv({"--state-len": 128, "--state-value-count": 64, "--hd1": 4097, "--hd2": 513, "--nrd": 1, "--batch-size": 16384})
    assert lib.mgt_plan_linear_op(n, arr, 13, out, 14) == 0
    assert (out[9], out[6], out[7], out[8]) == (3, 8192, 4104, 16384)


def test_invalid_configurations_are_rejected():
    # native/tests/test_train_plan.cpp:119-133 and the option parser (tool:525-613)
    for flags in (dict(state_len=0), dict(output_dim=0), dict(gradient_carousel_slots=0), dict(k_min=5, k_max=2), dict(steps=0),
                  dict(world_size=2, global_rank=2), dict(state_alignment=12), dict(allreduce_bucket_bytes=6), dict(lr=0), dict(batch_size=0)):
        st, _ = plan_summary(**flags)
        assert st == 1, flags
    lib = _lib.load()
    out = (C.c_uint64 * 16)()
    for bad in ([b"--no-such-flag", b"1"], [b"--steps"], [b"--steps", b"abc"], [b"--linear-fp16", b"maybe"]):
        arr = (C.c_char_p * len(bad))(*bad)
        assert lib.mgt_plan_summary(len(bad), arr, out, 16) == 1
    for good in ([b"--linear-fp16", b"off"], [b"--write-artifacts", b"yes"], [b"--overlap-allreduce", b"false"]):
        arr = (C.c_char_p * len(good))(*good)
        assert lib.mgt_plan_summary(len(good), arr, out, 16) == 0


def test_plan_files_format(tmp_path):
    lib = _lib.load()
    flags = {"--batch-size": 8, "--k-min": 2, "--k-max": 5, "--hd1": 7, "--hd2": 4, "--output-dim": 3, "--input-grad-positions-per-block": 2,
             "--world-size": 2, "--global-rank": 1, "--local-rank": 1, "--device-id": 1}
    n, arr = _argv(flags)
    assert lib.mgt_plan_write_files(n, arr, str(tmp_path).encode(), 1, 1, 0) == 0
    env = dict(line.split("=", 1) for line in open(tmp_path / "metadata.env").read().splitlines())
    assert list(env)[:6] == ["MODEL_MODE", "OUTPUT_DIM", "WORLD_SIZE", "GLOBAL_RANK", "LOCAL_RANK", "DEVICE_ID"] and list(env)[-1] == "NUM_PARAMETERS"
    assert env["MODEL_MODE"] == "MLP2RB" and env["OUTPUT_DIM"] == "3" and env["HD1"] == "7" and env["PHYSICAL_HD1"] == "8" and env["HD2"] == "4"
    assert env["INPUT_GRAD_BACKEND"] == "position_group_owner_write" and env["NCCL_ENABLED"] == "1" and env["RESUME_CHECKPOINT"] == "0"
    assert env["NUM_CLASSES"] == "72" and env["GLOBAL_RANK"] == "1" and env["OVERLAP_ALLREDUCE"] == "1" and len(env) == 30
    params = 72 * 72 * 8 + 8 + 8 * 8 + 8 + 2 * (8 * 8 + 8) + 8 * 3 + 3
    assert env["NUM_PARAMETERS"] == str(params)
    layers = json.load(open(tmp_path / "layers.json"))
    assert layers == {"model_mode": "MLP2RB", "output_dim": 3, "state_len": 72, "state_storage_len": 80, "num_classes": 72, "hd1": 7,
                      "physical_hd1": 8, "hd2": 4, "physical_hd2": 8, "nrd": 1, "artifacts_written": True, "num_parameters": params}
    assert open(tmp_path / "layers.json").read().startswith('{\n  "model_mode": "MLP2RB",\n  "output_dim": 3,\n')
    ops = json.load(open(tmp_path / "linear_ops.json"))
    assert ops["format"] == "mgt_linear_ops_v1" and ops["op_count"] == len(ops["linear_ops"]) == 14
    first = open(tmp_path / "linear_ops.json").read().splitlines()[4]
    assert first == ('    {"op_id": 0, "phase": "forward", "role": "input_embedding", "block_index": 0, "transpose_a": "N", "transpose_b": "N", '
                     '"m": 8, "n": 8, "k": 72, "lhs_rows": 8, "lhs_cols": 72, "rhs_rows": 72, "rhs_cols": 8, "output_rows": 8, "output_cols": 8, '
                     '"backend": "custom_kernel", "tensor_core_eligible": true, "logical_tail_masked": true},')
    # back-end names the reference reports for its flags (tool:93-102)
    for extra, name in (({}, "dense_one_hot_half_gemm"), ({"--input-grad-fp16": 0}, "dense_one_hot_float_gemm"),
                        ({"--input-grad-partial-chunks": 2}, "position_chunked_owner_write"),
                        ({"--input-grad-position-tile": 36}, "position_tiled_one_hot_half_gemm"),
                        ({"--input-grad-position-tile": 36, "--input-grad-fp16": 0}, "position_tiled_one_hot_float_gemm")):
        n, arr = _argv(extra)
        assert lib.mgt_plan_write_files(n, arr, str(tmp_path / "b").encode(), 0, 0, 0) == 0
        assert f"INPUT_GRAD_BACKEND={name}\n" in open(tmp_path / "b" / "metadata.env").read()


def test_export_converter_matches_trainer_converter(oracle):
    lib = _lib.load()
    lib.mgt_export_float_to_fp16.restype = C.c_uint16
    lib.mgt_export_float_to_fp16.argtypes = [C.c_float]
    rng = np.random.default_rng(2)
    xs = np.concatenate([rng.standard_normal(3000).astype(np.float32) * s for s in (1e-9, 1e-6, 1e-3, 1.0, 1e3, 1e5)])
    xs = np.concatenate([xs, np.array([0.0, -0.0, 65504.0, 65520.0, 1e30, -1e30, 2.0**-24, 2.0**-25, 3.0 * 2.0**-26, np.inf], np.float32)])
    got = np.array([lib.mgt_export_float_to_fp16(float(x)) for x in xs], np.uint16)
    assert np.array_equal(got, oracle.export_fp16(xs))


def test_weights_and_checkpoint_files(tmp_path):
    lib = _lib.load()
    flags = {"--hd1": 5, "--hd2": 3, "--nrd": 1, "--steps": 2, "--weight-decay": 0.01}
    n, arr = _argv(flags)
    params = 72 * 72 * 8 + 8 + 8 * 8 + 8 + 2 * (8 * 8 + 8) + 8 + 1
    i = np.arange(params, dtype=np.int64)
    w = ((i % 29 - 14) * 0.0001).astype(np.float64).astype(np.float32)
    m = (w * 0.5).astype(np.float32)
    v = (w * w).astype(np.float32)
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    lib.mgt_write_run_artifacts.argtypes = [C.c_int32, C.c_void_p, C.c_char_p, C.c_void_p, C.c_void_p, C.c_void_p]
    assert lib.mgt_write_run_artifacts(n, arr, str(tmp_path).encode(), p(w), p(m), p(v)) == 0
    wd, cd = tmp_path / "weights", tmp_path / "checkpoint"
    man = json.load(open(wd / "manifest.json"))
    assert man == {"format": "stream1_weights", "version": 1, "state_len": 72, "num_classes": 72, "logical_num_classes": 72, "hd1": 8, "hd2": 8,
                   "original_hd1": 5, "original_hd2": 3, "hidden_alignment": 8, "nrd": 1, "output_dim": 1, "dtype": "fp16",
                   "normalization": "none", "layout": "row-major input activations times weight_hxk", "flat_debug_weights": "weights.f32.bin"}
    assert np.array_equal(np.fromfile(wd / "weights.f32.bin", np.float32), w)
    sizes = {"input_weight_hxk": 5184 * 8, "input_bias": 8, "hidden_weight_hxk": 64, "hidden_bias": 8, "residual0_fc1_weight_hxk": 64,
             "residual0_fc1_bias": 8, "residual0_fc2_weight_hxk": 64, "residual0_fc2_bias": 8, "output_weight_hxk": 8, "output_bias": 1}
    for name, count in sizes.items():
        assert os.path.getsize(wd / f"{name}.fp16") == 2 * count, name
    table = np.fromfile(wd / "input_weight_hxk.fp16", np.float16).reshape(5184, 8)
    assert np.allclose(table.astype(np.float32), w[: 5184 * 8].reshape(5184, 8), atol=1e-7, rtol=1e-3)
    fc2 = np.fromfile(wd / "residual0_fc2_weight_hxk.fp16", np.float16)
    off = 5184 * 8 + 8 + 64 + 8 + 64 + 8
    assert np.allclose(fc2.astype(np.float32), w[off:off + 64], atol=1e-7, rtol=1e-3)
    cman = json.load(open(cd / "manifest.json"))
    assert cman["format"] == "mgt_train_checkpoint" and cman["step"] == 2 and cman["sections"] == ["weights", "adam_m", "adam_v"]
    assert cman["params_per_section"] == params and cman["physical_hd1"] == 8 and cman["hd1"] == 5 and cman["optimizer"] == "AdamW"
    assert '"weight_decay": 0.01,' in open(cd / "manifest.json").read()
    state = np.fromfile(cd / "state.f32.bin", np.float32)
    assert np.array_equal(state, np.concatenate([w, m, v]))
    w2, m2, v2 = np.zeros_like(w), np.zeros_like(w), np.zeros_like(w)
    lib.mgt_read_checkpoint.argtypes = [C.c_char_p, C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p]
    assert lib.mgt_read_checkpoint(str(cd).encode(), params, p(w2), p(m2), p(v2)) == 0
    assert np.array_equal(w2, w) and np.array_equal(m2, m) and np.array_equal(v2, v)
    assert lib.mgt_read_checkpoint(str(tmp_path / "nope").encode(), params, p(w2), p(m2), p(v2)) == 6
    assert lib.mgt_read_checkpoint(str(cd).encode(), params + 1, p(np.zeros(params + 1, np.float32)), p(np.zeros(params + 1, np.float32)), p(np.zeros(params + 1, np.float32))) == 6


def test_exported_weight_files_rebuild_the_model(tmp_path, oracle):
    # What the downstream consumer does with weights/ (tool:241-348): every tensor is a row-major [inputs][outputs] fp16
    # file named in a fixed order, "row-major input activations times weight_hxk". Rebuilding the flat parameter vector
    # from the files alone and running the forward pass must reproduce the fp32 model up to the fp16 rounding.
    from oracle import MlpShape
    lib = _lib.load()
    hd1, hd2, nrd, out = 16, 8, 2, 3
    n, arr = _argv({"--hd1": hd1, "--hd2": hd2, "--nrd": nrd, "--output-dim": out})
    shape = MlpShape(72, 72, hd1, hd2, nrd, out)
    rng = np.random.default_rng(12)
    w = (rng.standard_normal(shape.param_count) * 0.05).astype(np.float32)
    zeros = np.zeros_like(w)
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    lib.mgt_write_run_artifacts.argtypes = [C.c_int32, C.c_void_p, C.c_char_p, C.c_void_p, C.c_void_p, C.c_void_p]
    assert lib.mgt_write_run_artifacts(n, arr, str(tmp_path).encode(), p(w), p(zeros), p(zeros)) == 0
    man = json.load(open(tmp_path / "weights" / "manifest.json"))
    assert (man["hd1"], man["hd2"], man["nrd"], man["output_dim"], man["dtype"]) == (hd1, hd2, nrd, out, "fp16")
    names = ["input_weight_hxk", "input_bias", "hidden_weight_hxk", "hidden_bias"]
    for k in range(man["nrd"]):
        names += [f"residual{k}_fc1_weight_hxk", f"residual{k}_fc1_bias", f"residual{k}_fc2_weight_hxk", f"residual{k}_fc2_bias"]
    names += ["output_weight_hxk", "output_bias"]
    bits = np.concatenate([np.fromfile(tmp_path / "weights" / f"{name}.fp16", np.uint16) for name in names])
    assert bits.size == shape.param_count
    # the files hold exactly the trainer's software conversion of every parameter, tensors in parameter order
    lib.mgt_export_float_to_fp16.restype = C.c_uint16
    lib.mgt_export_float_to_fp16.argtypes = [C.c_float]
    assert np.array_equal(bits, np.array([lib.mgt_export_float_to_fp16(float(x)) for x in w], np.uint16))
    rebuilt = bits.view(np.float16).astype(np.float32)
    # That converter (tool:215-229) ORs the rounded mantissa into the exponent field, so a value that rounds up to a power
    # of two with an odd half exponent comes out halved; it is reproduced literally. Everything else is fp16 rounding.
    off = np.abs(rebuilt - w) > 2.0 ** -11 * np.abs(w) + 1e-7
    assert off.sum() <= 1e-3 * w.size
    ieee = w[off].astype(np.float16)
    assert np.all((ieee.view(np.uint16) & 0x3FF) == 0) and np.all(((ieee.view(np.uint16) >> 10) & 1) == 0)  # IEEE result 2^e, carried into an even exponent
    assert np.allclose(rebuilt[off], 0.5 * ieee.astype(np.float32))
    states = rng.integers(0, 72, (40, 80)).astype(np.uint8)
    states[:, 72:] = 0
    expect = w.copy()
    expect[off] = rebuilt[off]
    st_a, y_files = oracle.forward(shape, rebuilt, states)
    st_b, y_f32 = oracle.forward(shape, expect, states)
    assert st_a == 0 and st_b == 0
    assert np.max(np.abs(y_files - y_f32)) <= 5e-3 * max(1.0, np.max(np.abs(y_f32)))


# the reference checkout: MGT_REFERENCE_DIR if set, else a directory `reference` beside this repository
REF_SCRIPTS = os.path.join(os.environ.get("MGT_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "..", "reference"),
                           "native", "tests", "scripts")


@pytest.mark.skipif(not os.path.exists(os.path.join(REF_SCRIPTS, "check_native_train_artifacts.sh")),
                    reason="the reference checkout (with its contract scripts) is not present")
def test_reference_artifact_script_accepts_our_files(tmp_path):
    """native/tests/scripts/check_native_train_artifacts.sh, run UNCHANGED (ctest native_train_artifacts, CMakeLists.txt:191)
    over a run directory written by the trainer's own writers and formatters for the flags of ctest native_train_smoke
    (defaults: hd1 5, hd2 3, nrd 1). The GPU suite runs the same script over a directory bin/mgt_native_train wrote, where
    a GPU and the checkout are both present; this leg needs neither a GPU nor the trainer's step loop."""
    import subprocess

    class Rec(C.Structure):
        _fields_ = [("step", C.c_uint32), ("loss", C.c_float), ("step_ms", C.c_float), ("walk_ms", C.c_float), ("backward_ms", C.c_float),
                    ("allreduce_ms", C.c_float), ("adam_ms", C.c_float), ("memory_bytes", C.c_uint64), ("overlap_ranges", C.c_uint32),
                    ("overlap_chunks", C.c_uint32), ("backward_stage_ms", C.c_float * 7)]

    lib = _lib.load()
    flags = {"--steps": 2, "--device-id": 0, "--world-size": 1, "--global-rank": 0, "--local-rank": 0}
    n, arr = _argv(flags)
    run = tmp_path / "native-train-smoke-run"
    assert lib.mgt_plan_write_files(n, arr, str(run).encode(), 1, 1, 0) == 0
    params = 72 * 72 * 8 + 8 + 8 * 8 + 8 + 2 * (8 * 8 + 8) + 8 + 1
    i = np.arange(params, dtype=np.int64)
    w = ((i % 29 - 14) * 0.0001).astype(np.float64).astype(np.float32)
    zeros = np.zeros(params, np.float32)
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    lib.mgt_write_run_artifacts.argtypes = [C.c_int32, C.c_void_p, C.c_char_p, C.c_void_p, C.c_void_p, C.c_void_p]
    assert lib.mgt_write_run_artifacts(n, arr, str(run).encode(), p(w), p(zeros), p(zeros)) == 0
    lib.mgt_format_step_record.argtypes = [C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_char_p, C.c_char_p, C.c_char_p, C.c_uint32]
    start, line, row = (C.create_string_buffer(8192) for _ in range(3))
    with open(run / "train.log", "w") as log, open(run / "profile.jsonl", "w") as prof:
        for step in range(2):
            rec = Rec(step, 30.5 - step, 1.25, 0.02, 1.0, 0.0, 0.1, 123456789, 0, 0, (C.c_float * 7)(*[0.1] * 7))
            assert lib.mgt_format_step_record(n, arr, C.byref(rec), 0, 1, 0, start if step == 0 else None, line, row, 8192) == 0
            if step == 0:
                log.write(start.value.decode())
            log.write(line.value.decode())
            prof.write(row.value.decode())
    for text in open(run / "profile.jsonl"):
        json.loads(text)  # every row is one JSON object
    res = subprocess.run(["bash", os.path.join(REF_SCRIPTS, "check_native_train_artifacts.sh"), str(run)], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    assert lib.mgt_format_step_record(n, arr, C.byref(rec), 0, 1, 0, None, line, row, 8) == 3  # capacity_exceeded
