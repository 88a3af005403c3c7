"""Our mgt_native_train against the UNMODIFIED reference GPU trainer: per-step losses against the committed
fixture (losses the reference binary wrote on a B200), and - when the reference binary is present beside the
oracle - a live side-by-side run comparing losses, final weights and optimizer state, and step time."""
import json
import os
import subprocess

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from helpers import rel_l2  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
OURS = os.path.join(ROOT, "bin", "mgt_native_train")
REF = os.path.join(ROOT, "oracle", "_ref", "mgt_native_train_ref")
GOLDEN = os.path.join(ROOT, "tests", "golden", "reference_gpu_losses.json")
BASE = ["--device-id", "0", "--world-size", "1", "--global-rank", "0", "--local-rank", "0"]
TOL = 1e-3  # per-step loss, weights and optimizer state: 1e-3 relative (fp16 operands, fp32 accumulate)


def run(binary, out_dir, flags):
    res = subprocess.run([binary, "--output-dir", str(out_dir), *BASE, *[str(f) for f in flags]], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr + res.stdout
    return [json.loads(line) for line in open(os.path.join(out_dir, "profile.jsonl"))]


@pytest.mark.parametrize("case", ["p888", "small_out1", "small_out3"])
def test_losses_match_reference_gpu_fixture(tmp_path, case):
    golden = json.load(open(GOLDEN))["cases"][case]
    rows = run(OURS, tmp_path, ["--write-artifacts", "0", *golden["flags"]])
    want = np.array(golden["loss"])
    got = np.array([r["loss"] for r in rows])
    assert got.shape == want.shape
    assert np.max(np.abs(got - want) / np.abs(want)) <= TOL, (got, want)


@pytest.mark.skipif(not os.path.exists(REF), reason="reference GPU trainer not built (make -C oracle ref_gpu)")
@pytest.mark.parametrize("flags", [
    ["--steps", 6, "--batch-size", 1536, "--k-min", 1, "--k-max", 29, "--hd1", 256, "--hd2", 64, "--nrd", 2, "--lr", 0.001],
    ["--steps", 10, "--batch-size", 53248, "--k-min", 1, "--k-max", 29, "--hd1", 2556, "--hd2", 218, "--nrd", 16,
     "--input-grad-fp16", 1, "--input-grad-position-tile", 36, "--linear-fp16", 1],
    # the reference's ctest native_train_input_grad_float_backend, and its TF32 linears (our fp32 path is the more exact one)
    ["--steps", 6, "--batch-size", 1536, "--k-min", 1, "--k-max", 29, "--hd1", 256, "--hd2", 64, "--nrd", 2, "--lr", 0.001, "--input-grad-fp16", 0],
    ["--steps", 6, "--batch-size", 1536, "--k-min", 1, "--k-max", 29, "--hd1", 256, "--hd2", 64, "--nrd", 2, "--lr", 0.001, "--linear-fp16", 0,
     "--input-grad-fp16", 0],
], ids=["small", "p888", "small_ig_fp32", "small_all_fp32"])
def test_side_by_side_with_reference_binary(tmp_path, flags):
    ref_rows = run(REF, tmp_path / "ref", ["--write-artifacts", 1, *flags])
    our_rows = run(OURS, tmp_path / "ours", ["--write-artifacts", 1, *flags])
    assert len(ref_rows) == len(our_rows)
    assert [r["input_grad_backend"] for r in ref_rows] == [r["input_grad_backend"] for r in our_rows]
    for a, b in zip(ref_rows, our_rows):
        assert abs(a["loss"] - b["loss"]) <= TOL * abs(a["loss"]), (a["step"], a["loss"], b["loss"])
    # final weights, m, v as the two binaries checkpoint them (checkpoint/state.f32.bin: w | m | v)
    ref_state = np.fromfile(tmp_path / "ref" / "checkpoint" / "state.f32.bin", dtype=np.float32)
    our_state = np.fromfile(tmp_path / "ours" / "checkpoint" / "state.f32.bin", dtype=np.float32)
    assert ref_state.shape == our_state.shape and ref_state.size % 3 == 0
    p = ref_state.size // 3
    for name, lo in (("weights", 0), ("m", p), ("v", 2 * p)):
        assert rel_l2(our_state[lo:lo + p], ref_state[lo:lo + p]) <= TOL, name
    # the exported fp16 weight files are what the downstream consumer reads
    for fname in sorted(os.listdir(tmp_path / "ref" / "weights")):
        if fname.endswith(".fp16"):
            a = np.fromfile(tmp_path / "ref" / "weights" / fname, dtype=np.float16).astype(np.float32)
            b = np.fromfile(tmp_path / "ours" / "weights" / fname, dtype=np.float16).astype(np.float32)
            assert a.shape == b.shape, fname
            # Adam divides by sqrt(v): where a gradient component is near zero the update direction amplifies the last
            # bits of the gradient, and after ten steps of lr 1e-4 the updates are as large as the 1e-4-scale initial
            # weights. The whole state agrees to 1e-3 (above); single small tensors get a looser per-file bound.
            assert rel_l2(b, a) <= (1e-2 if a.size >= 4096 else 5e-2), fname
    ref_ms = float(np.median([r["milliseconds"] for r in ref_rows[1:]]))
    our_ms = float(np.median([r["milliseconds"] for r in our_rows[1:]]))
    print(f"\nstep time: reference {ref_ms:.3f} ms, this library {our_ms:.3f} ms ({ref_ms / our_ms:.2f}x)")
    if flags[3] == 53248:
        assert our_ms < ref_ms  # the headline configuration must not be slower than the reference on the same GPU


@pytest.mark.skipif(not os.path.exists(REF), reason="reference GPU trainer not built (make -C oracle ref_gpu)")
def test_two_hundred_steps_track_the_reference(tmp_path):
    """The README's p888 command for its full 200 steps, both binaries, same seeds: every per-step loss within the stated
    1e-3. (The trainer's initial weights sit on a 1e-4 lattice and stay near it for the first dozens of Adam steps, so many
    pre-activations cancel to zero up to rounding; which of those pass the ReLU in backward is decided by the sign of an
    fp32 rounding residue. The masks are therefore taken from the fp32 values, as the reference takes them - with masks
    from the fp16-rounded activations the two runs drifted apart by up to 1.4e-3 around step 40.)"""
    flags = ["--steps", 200, "--batch-size", 53248, "--k-min", 1, "--k-max", 29, "--hd1", 2556, "--hd2", 218, "--nrd", 16,
             "--input-grad-fp16", 1, "--input-grad-position-tile", 36, "--linear-fp16", 1, "--write-artifacts", 0]
    ref = np.array([r["loss"] for r in run(REF, tmp_path / "ref", flags)])
    ours = np.array([r["loss"] for r in run(OURS, tmp_path / "ours", flags)])
    assert ref.shape == ours.shape == (200,)
    rel = np.abs(ours - ref) / np.abs(ref)
    print(f"\n200 steps: worst {rel.max():.2e} at step {int(rel.argmax())}, steps over 1e-3: {int((rel > 1e-3).sum())}, "
          f"median {np.median(rel):.2e}, last 100 worst {rel[100:].max():.2e}")
    assert rel.max() <= TOL
    assert np.median(rel) <= 1e-4
