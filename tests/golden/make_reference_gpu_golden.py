"""Regenerates tests/golden/reference_gpu_losses.json: per-step losses written by the UNMODIFIED reference GPU
trainer (oracle/_ref/mgt_native_train_ref, built by `make -C oracle ref_gpu` from the reference's sources) on a
B200. Needs a GPU; run from the repository root:

    python tests/golden/make_reference_gpu_golden.py

The cases are the reference README's p888 command (README.md:48-64) and two small configurations of the ctest
family (native/CMakeLists.txt:177-186).
"""
import json
import os
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REF = os.path.join(ROOT, "oracle", "_ref", "mgt_native_train_ref")
BASE = ["--device-id", "0", "--world-size", "1", "--global-rank", "0", "--local-rank", "0", "--write-artifacts", "0"]

CASES = {
    "p888": ["--steps", "30", "--batch-size", "53248", "--k-min", "1", "--k-max", "29", "--hd1", "2556", "--hd2", "218", "--nrd", "16",
             "--input-grad-fp16", "1", "--input-grad-position-tile", "36", "--linear-fp16", "1"],
    "small_out1": ["--steps", "12", "--batch-size", "2048", "--k-min", "1", "--k-max", "29", "--hd1", "256", "--hd2", "64", "--nrd", "2",
                   "--lr", "0.001"],
    "small_out3": ["--steps", "8", "--batch-size", "1000", "--k-min", "2", "--k-max", "9", "--hd1", "120", "--hd2", "96", "--nrd", "3",
                   "--output-dim", "3", "--lr", "0.001"],
}


def main():
    if not os.path.exists(REF):
        sys.exit("build the reference trainer first: make -C oracle ref_gpu")
    out = {"generator": "tests/golden/make_reference_gpu_golden.py", "binary": "reference mgt_native_train (tools/mgt_native_train_smoke.cu), sm_100 build",
           "cases": {}}
    for name, flags in CASES.items():
        with tempfile.TemporaryDirectory() as tmp:
            subprocess.run([REF, "--output-dir", tmp, *BASE, *flags], check=True, capture_output=True, timeout=600)
            rows = [json.loads(line) for line in open(os.path.join(tmp, "profile.jsonl"))]
        out["cases"][name] = {"flags": flags, "loss": [r["loss"] for r in rows]}
        print(name, len(rows), "steps, last loss", rows[-1]["loss"])
    with open(os.path.join(ROOT, "tests", "golden", "reference_gpu_losses.json"), "w") as f:
        json.dump(out, f, indent=1)


if __name__ == "__main__":
    main()
