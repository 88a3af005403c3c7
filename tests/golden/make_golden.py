"""Regenerates tests/golden/*.npz from the reference's own CPU code.

Run where the reference checkout is present (it compiles the reference sources into
oracle/_ref/libmgt_ref.so through oracle/Makefile):

    python tests/golden/make_golden.py

The fixtures are small, committed, and never hand-edited.
  walks.npz   : states/labels/meta of GenerateRandomWalksCpu for several (seed, epoch, step, rank, k-range)
  mlp.npz     : loss + full gradient of CpuMlpLossAndGrad and outputs of CpuMlpForward on the
                reference tests' deterministic inputs (test_mlp_cpu_ref.cpp, test_cuda_mlp_backward_cpu_compare.cpp)
  adamw.npz   : CpuAdamWStep results for three consecutive steps
  plan.npz    : planner numbers of BuildTrainPlan for the configurations the reference tests use
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import MlpShape, build_oracle, load_oracle, load_reference  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))

WALK_CASES = [
    # seed, epoch, step, rank, k_min, k_max, samples
    (1234, 0, 0, 0, 1, 29, 64),
    (1234, 0, 1, 0, 1, 29, 64),
    (1234, 0, 0, 1, 1, 29, 64),
    (1234, 0, 1, 1, 1, 29, 64),
    (1234, 5, 7, 2, 1, 9, 64),
    (0, 0, 0, 0, 1, 29, 256),
    (0xDEADBEEFCAFEF00D, 3, 199, 7, 5, 5, 33),
]


def compare_case_inputs(shape: MlpShape, samples: int):
    """Deterministic inputs of test_cuda_mlp_backward_cpu_compare.cpp:29-41."""
    p = shape.param_count
    i = np.arange(p, dtype=np.int64)
    weights = (((i * 7) % 29 - 14) * 0.00325).astype(np.float32)
    labels = np.zeros((samples, shape.output_dim), np.float32)
    states = np.zeros((samples, 80), np.uint8)
    for s in range(samples):
        for o in range(shape.output_dim):
            labels[s, o] = np.float32(((s * 3 + o * 5 + shape.output_dim) % 17) - 8) * np.float32(0.0625)
        for k in range(shape.state_len):
            states[s, k] = (k * 3 + s * 5 + shape.output_dim) % shape.state_value_pad
    return weights, states, labels


def cpu_ref_case_inputs():
    """Inputs of test_mlp_cpu_ref.cpp:7-27."""
    shape = MlpShape(4, 8, 5, 3, 1, 1)
    i = np.arange(shape.param_count, dtype=np.int64)
    weights = ((i % 11 - 5) * 0.01).astype(np.float32)
    states = np.zeros((2, 80), np.uint8)
    for s in range(2):
        for k in range(4):
            states[s, k] = (k + s) % 8
    labels = np.array([[1.0], [3.0]], np.float32)
    return shape, weights, states, labels


def main():
    build_oracle(with_reference=True)
    ref = load_reference()
    assert ref is not None, "reference checkout missing"
    orc = load_oracle()
    moves, target = orc.cyclic_puzzle(72, 18)

    walks = {"cases": np.array(WALK_CASES, dtype=np.uint64), "moves": moves, "target": target}
    for idx, (seed, epoch, step, rank, kmin, kmax, n) in enumerate(WALK_CASES):
        st, states, labels, meta = ref.random_walks(moves, target, seed=seed, epoch=epoch, step=step, rank=rank,
                                                    k_min=kmin, k_max=kmax, samples=n)
        assert st == 0
        walks[f"states_{idx}"] = states
        walks[f"labels_{idx}"] = labels
        walks[f"depth_{idx}"] = meta["depth"]
        walks[f"last_move_{idx}"] = meta["last_move"]
        walks[f"rng_{idx}"] = meta["rng_counter"]
    np.savez_compressed(os.path.join(OUT, "walks.npz"), **walks)

    mlp = {}
    shape, w, s, l = cpu_ref_case_inputs()
    st, out = ref.forward(shape, w, s)
    assert st == 0
    st, loss, grad = ref.loss_grad(shape, w, s, l)
    assert st == 0
    mlp["kat_shape"] = np.array([4, 8, 5, 3, 1, 1], np.uint32)
    mlp["kat_outputs"] = out
    mlp["kat_loss"] = np.float32(loss)
    mlp["kat_grad"] = grad
    cases = [((4, 8, 5, 3, 1, 1), 8), ((4, 8, 5, 3, 1, 3), 8), ((6, 8, 9, 7, 2, 11), 10),
             ((72, 72, 64, 32, 2, 1), 16)]
    mlp["cmp_cases"] = np.array([list(c[0]) + [c[1]] for c in cases], np.uint32)
    for idx, (dims, n) in enumerate(cases):
        shape = MlpShape(*dims)
        w, s, l = compare_case_inputs(shape, n)
        st, loss, grad = ref.loss_grad(shape, w, s, l)
        assert st == 0
        st, out = ref.forward(shape, w, s)
        mlp[f"cmp_loss_{idx}"] = np.float32(loss)
        mlp[f"cmp_grad_{idx}"] = grad
        mlp[f"cmp_out_{idx}"] = out
    np.savez_compressed(os.path.join(OUT, "mlp.npz"), **mlp)

    rng = np.random.default_rng(7)
    n = 1024
    w = rng.standard_normal(n).astype(np.float32) * 0.1
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    adam = {"w0": w.copy()}
    for step in (1, 2, 3):
        g = (rng.standard_normal(n) * 1e-3).astype(np.float32)
        adam[f"g_{step}"] = g
        assert ref.adamw(w, g, m, v, step=step, lr=1e-3, wd=0.01 if step == 3 else 0.0) == 0
        adam[f"w_{step}"] = w.copy()
        adam[f"m_{step}"] = m.copy()
        adam[f"v_{step}"] = v.copy()
    np.savez_compressed(os.path.join(OUT, "adamw.npz"), **adam)

    plan = {}
    configs = {
        "p888": dict(),
        "p888_b53248_w8": dict(batch=53248, world=8),
        "synthetic": dict(state_len=31, value_count=37, move_count=11, hd1=64, hd2=33, nrd=2, batch=1234, bucket_bytes=4096),
        "tiny": dict(state_len=17, value_count=9, hd1=31, hd2=19, nrd=2, batch=512),
        "config0": dict(hd1=256, hd2=64, nrd=2, batch=1024),
        "config3": dict(hd1=4096, hd2=512, nrd=32, output_dim=29, batch=131072),
    }
    for name, kw in configs.items():
        st, numbers = ref.plan_numbers(**kw)
        assert st == 0, name
        plan[name] = np.array([numbers[k] for k in sorted(numbers)], np.uint64)
    plan["keys"] = np.array(sorted(numbers))
    rows = []
    for i in range(104):
        st, row = ref.plan_linear_op(i, batch=32768)
        assert st == 0
        rows.append(row)
    plan["p888_linear_ops_b32768"] = np.array(rows, np.uint32)
    np.savez_compressed(os.path.join(OUT, "plan.npz"), **plan)
    print("golden fixtures written to", OUT)


if __name__ == "__main__":
    main()
