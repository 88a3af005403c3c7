"""Batch normalisation in the loss+gradient engine (opt-in; the reference has none) against the CPU oracle's
restatement, which is pinned by finite differences (tests/test_oracle.py). Statistics over several ranks are tested
on ONE GPU: the ranks are host threads with an engine and a stream each, and the statistics exchange is done on the
host between them (no kernel ever waits for another)."""
import threading

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

import multigputrainmlp_b200 as mgt  # noqa: E402
from helpers import rel_l2  # noqa: E402
from oracle import MlpShape  # noqa: E402

DEV = "cuda:0"


def make_case(oracle, dims, n, seed, scale=0.05):
    shape = MlpShape(*dims)
    rng = np.random.default_rng(seed)
    if shape.state_len == 72:
        moves, target = oracle.cyclic_puzzle(72, 18)
        _, states, depth, _ = oracle.random_walks(moves, target, seed=seed, epoch=0, step=0, rank=0, k_min=1, k_max=29, samples=n)
    else:
        states = np.zeros((n, 80), np.uint8)
        states[:, :shape.state_len] = rng.integers(0, shape.state_value_pad, (n, shape.state_len))
        depth = rng.integers(1, 30, n).astype(np.float32)
    nbn = oracle.bn_param_count(shape)
    w = (rng.standard_normal(shape.param_count + nbn) * scale).astype(np.float32)
    bn = w[shape.param_count:].reshape(shape.residual_blocks + 1, 2, shape.hd2)
    bn[:, 0, :] = 1.0 + 0.2 * rng.standard_normal((shape.residual_blocks + 1, shape.hd2))   # gamma
    bn[:, 1, :] = 0.1 * rng.standard_normal((shape.residual_blocks + 1, shape.hd2))         # beta
    labels = np.ascontiguousarray(np.repeat(depth.reshape(-1, 1), shape.output_dim, axis=1).astype(np.float32))
    if shape.output_dim < 29:
        labels = np.minimum(labels, shape.output_dim)
    return shape, w, states, labels


def cshape_of(shape):
    return mgt.CudaMlpShape(shape.state_len, shape.state_value_pad, shape.hd1, shape.hd2, shape.residual_blocks, shape.output_dim)


def run_bn_engine(eng, shape, w, states, labels, *, stream=None, callback=None, running=None, device=DEV):
    cshape = cshape_of(shape)
    total = shape.param_count + mgt.bn_param_count(cshape)
    assert w.size == total
    b = states.shape[0]
    with torch.cuda.stream(stream) if stream is not None else torch.cuda.stream(torch.cuda.current_stream()):
        dw = torch.from_numpy(w).to(device)
        ds = torch.from_numpy(states).to(device)
        dl = torch.from_numpy(np.ascontiguousarray(labels)).to(device)
        loss = torch.zeros(1, device=device)
        grad = torch.full((total,), float("nan"), device=device)
        floats = mgt.mlp_loss_grad_workspace_floats(cshape, b, batch_norm=True)
        assert floats > mgt.mlp_loss_grad_workspace_floats(cshape, b)
        ws = torch.empty(floats, device=device)
        ws.fill_(float("nan"))
        st = eng.launch_mlp_loss_grad(cshape, dw, None, ds, dl, b, loss, grad, ws, floats, gradient_ready=callback, stream=stream)
        assert st == 0, mgt.status_name(st)
        (stream or torch.cuda.current_stream()).synchronize()
    st, code = eng.check()
    assert st == 0, f"device status {code}"
    return float(loss.item()), grad.cpu().numpy()


def sections(shape):
    p = shape.param_count
    in_w = shape.state_len * shape.state_value_pad * shape.hd1
    hid_end = in_w + shape.hd1 + shape.hd1 * shape.hd2 + shape.hd2
    return {"embedding": (0, in_w + shape.hd1), "hidden": (in_w + shape.hd1, hid_end), "tail": (hid_end, p), "scale_shift": (p, None)}


def assert_close(shape, loss_g, grad_g, loss_o, grad_o, grad_exact, tol):
    """Normalised values crowd around zero, where the 16-bit rounding of an operand decides which side of a ReLU a value
    falls on: two correct realisations of the same rounding model then differ by about as much as the model differs
    from exact arithmetic (2 % of the gradient norm for random weights). The bound is therefore `tol` plus that distance,
    overall and per section; the `smooth` cases keep every ReLU open, which makes it tight (1e-4 ... 1e-3) where the
    normalisation's own terms live (the tower and the scale/shift gradients)."""
    assert np.isfinite(grad_g).all()
    assert abs(loss_g - loss_o) <= tol * max(abs(loss_o), 1e-6), (loss_g, loss_o)
    model = rel_l2(grad_o, grad_exact)
    assert rel_l2(grad_g, grad_o) <= tol + model, (rel_l2(grad_g, grad_o), model)
    for name, (lo, hi) in sections(shape).items():
        if np.abs(grad_o[lo:hi]).max() > 0:
            model = rel_l2(grad_o[lo:hi], grad_exact[lo:hi])
            assert rel_l2(grad_g[lo:hi], grad_o[lo:hi]) <= 2 * tol + 1.5 * model, (name, rel_l2(grad_g[lo:hi], grad_o[lo:hi]), model)


def keep_relus_open(shape, w):
    """Biases that keep every ReLU of the network open on these inputs (so that no rounding can flip one)."""
    w = w.copy()
    p, h1, h2, r = shape.param_count, shape.hd1, shape.hd2, shape.residual_blocks
    in_w = shape.state_len * shape.state_value_pad * h1
    w[in_w:in_w + h1] = 3.0
    tower = in_w + h1 + h1 * h2 + h2
    for k in range(r):
        b1 = tower + k * 2 * (h2 * h2 + h2) + h2 * h2
        w[b1:b1 + h2] = 12.0
    bn = w[p:].reshape(r + 1, 2, h2)
    bn[:, 0, :] = 0.3 + 0.05 * np.sin(np.arange(h2))
    bn[:, 1, :] = 3.0
    return w


CASES = [
    ((72, 72, 128, 224, 3, 1), 600, False, False, False),     # the p888 tower width
    ((72, 72, 128, 224, 3, 1), 600, False, False, True),
    ((72, 72, 64, 64, 2, 5), 257, False, True, False),        # cross-entropy, a ragged last row tile
    ((72, 72, 64, 64, 2, 5), 257, False, False, True),
    ((72, 72, 40, 24, 1, 1), 100, False, False, False),
    ((6, 8, 9, 7, 2, 11), 40, False, False, False),           # widths that are no multiple of four: ragged column quads
    ((6, 8, 9, 7, 2, 11), 40, False, False, True),
    ((72, 72, 96, 224, 2, 29), 300, True, True, False),       # bfloat16 + cross-entropy
    ((72, 72, 64, 32, 0, 1), 128, False, False, False),       # no residual blocks: the hidden layer's normalisation alone
]


@pytest.mark.parametrize("dims,n,bf16,ce,smooth", CASES)
def test_batch_norm_matches_the_oracle(oracle, dims, n, bf16, ce, smooth):
    shape, w, states, labels = make_case(oracle, dims, n, seed=31)
    if smooth:
        w = keep_relus_open(shape, w)
    if not ce and shape.output_dim > 1:
        labels = labels * 0.1
    st, loss_o, grad_o, stats_o = oracle.loss_grad_ex(shape, w, states, labels, bf16=bf16, cross_entropy=ce, batch_norm=True)
    assert st == 0
    st, _, grad_exact, _ = oracle.loss_grad_ex(shape, w, states, labels, half_linear=False, half_input_grad=False, cross_entropy=ce, batch_norm=True)
    assert st == 0
    seen = []
    eng = mgt.Engine(0)
    try:
        assert eng.set_train_options(bf16=bf16, cross_entropy=ce, batch_norm=True) == 0
        running = torch.zeros(shape.residual_blocks + 1, 2, shape.hd2, device=DEV)
        running[:, 1, :] = 1.0
        assert eng.set_batch_norm_state(running, momentum=0.25, world_size=1) == 0
        loss_g, grad_g = run_bn_engine(eng, shape, w, states, labels, callback=lambda u, i, off, cnt, s: seen.append((i, off, cnt)) or 0)
    finally:
        eng.close()
    assert_close(shape, loss_g, grad_g, loss_o, grad_o, grad_exact, tol=8e-3 if bf16 else 1e-3)
    # one more announcement than the reference makes: the scale/shift range, last
    assert len(seen) == 2 * shape.residual_blocks + 4
    assert seen[-1] == (2 * shape.residual_blocks + 3, shape.param_count, oracle.bn_param_count(shape))
    assert seen[-2][1] == 0
    # running statistics: (1 - momentum) * initial + momentum * batch, the variance unbiased
    r = running.cpu().numpy()
    unbias = n / (n - 1.0)
    np.testing.assert_allclose(r[:, 0, :], 0.25 * stats_o[:, 0, :], rtol=2e-2 if bf16 else 5e-3, atol=2e-3)
    np.testing.assert_allclose(r[:, 1, :], 0.75 + 0.25 * unbias * stats_o[:, 1, :], rtol=2e-2 if bf16 else 5e-3, atol=2e-3)


def test_batch_norm_is_scale_invariant(oracle):
    # the property that sets batch normalisation apart: scaling the weights AND the bias that feed a normalised layer
    # leaves loss and all other gradients unchanged (up to eps), and the scaled layer's own gradient shrinks by the factor
    shape, w, states, labels = make_case(oracle, (72, 72, 64, 64, 1, 1), 256, seed=32)
    in_w = 72 * 72 * 64
    lo, hi = in_w + 64, in_w + 64 + 64 * 64 + 64     # hidden weight + bias
    w2 = w.copy()
    w2[lo:hi] *= 2.0                                  # a power of two: the 16-bit rounding of the operands scales with it
    eng = mgt.Engine(0)
    try:
        assert eng.set_train_options(batch_norm=True, bn_eps=1e-12) == 0
        la, ga = run_bn_engine(eng, shape, w, states, labels)
        lb, gb = run_bn_engine(eng, shape, w2, states, labels)
    finally:
        eng.close()
    assert abs(la - lb) <= 1e-5 * abs(la)
    assert rel_l2(gb[lo:hi] * 2.0, ga[lo:hi]) <= 1e-4
    rest = np.r_[0:lo, hi:w.size]
    assert rel_l2(gb[rest], ga[rest]) <= 1e-4


def test_statistics_over_two_ranks_equal_one_rank_with_the_joint_batch(oracle):
    # data parallel with synchronised statistics: each rank normalises with the statistics of ALL samples, and the
    # rank-averaged gradient equals the gradient of the joint batch
    dims, n = (72, 72, 64, 96, 2, 1), 192
    shape, w, states, labels = make_case(oracle, dims, 2 * n, seed=33)
    st, loss_o, grad_o, _ = oracle.loss_grad_ex(shape, w, states, labels, batch_norm=True)
    assert st == 0
    st, _, grad_exact, _ = oracle.loss_grad_ex(shape, w, states, labels, half_linear=False, half_input_grad=False, batch_norm=True)
    assert st == 0
    world = 2
    barrier = threading.Barrier(world)
    slots = [None] * world
    results = [None] * world
    errors = []

    def rank_main(rank):
        try:
            torch.cuda.set_device(0)
            stream = torch.cuda.Stream(device=DEV)
            eng = mgt.Engine(0)
            exchange_buffer = torch.zeros(2 * shape.hd2, device=DEV)
            calls = [0]

            def exchange(user, ptr, count, s):
                # host-side average: wait for this rank's numbers, meet the other rank, average, write back
                assert int(count) == 2 * shape.hd2 and int(ptr) == exchange_buffer.data_ptr()
                stream.synchronize()
                slots[rank] = exchange_buffer.cpu().numpy().copy()
                barrier.wait(timeout=60)
                mean = (slots[0] + slots[1]) * 0.5
                barrier.wait(timeout=60)
                with torch.cuda.stream(stream):
                    exchange_buffer.copy_(torch.from_numpy(mean))
                calls[0] += 1
                return 0

            try:
                assert eng.set_train_options(batch_norm=True) == 0
                assert eng.set_batch_norm_state(None, 0.1, world, exchange_buffer, exchange) == 0
                part = slice(rank * n, (rank + 1) * n)
                results[rank] = run_bn_engine(eng, shape, w, states[part], labels[part], stream=stream)
                assert calls[0] == 2 * (shape.residual_blocks + 1)
            finally:
                eng.close()
        except BaseException as exc:  # noqa: BLE001
            errors.append(exc)
            barrier.abort()

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=180)
    assert not errors, errors
    loss_avg = 0.5 * (results[0][0] + results[1][0])
    grad_avg = 0.5 * (results[0][1].astype(np.float64) + results[1][1].astype(np.float64))
    assert_close(shape, loss_avg, grad_avg.astype(np.float32), loss_o, grad_o, grad_exact, tol=1e-3)
    # and NOT what two ranks with their own statistics give (the test would pass with a hook that does nothing otherwise)
    eng = mgt.Engine(0)
    try:
        assert eng.set_train_options(batch_norm=True) == 0
        local = [run_bn_engine(eng, shape, w, states[r * n:(r + 1) * n], labels[r * n:(r + 1) * n]) for r in range(world)]
    finally:
        eng.close()
    local_avg = 0.5 * (local[0][1].astype(np.float64) + local[1][1].astype(np.float64))
    assert rel_l2(local_avg.astype(np.float32), grad_o) > 3 * (1e-3 + rel_l2(grad_o, grad_exact))


def test_batch_norm_option_errors():
    cshape = mgt.CudaMlpShape(8, 8, 16, 16, 2, 1)
    eng = mgt.Engine(0)
    try:
        assert eng.set_train_options(batch_norm=True, bn_eps=0.0) == 1
        assert eng.set_train_options(batch_norm=True) == 0
        n = 32
        total = cshape.param_count + mgt.bn_param_count(cshape)
        assert mgt.bn_param_count(cshape) == 2 * 3 * 16
        t = torch.zeros(total, device=DEV)
        st8 = torch.zeros(n, 80, dtype=torch.uint8, device=DEV)
        small = mgt.mlp_loss_grad_workspace_floats(cshape, n)
        ws = torch.zeros(small, device=DEV)
        assert eng.launch_mlp_loss_grad(cshape, t, None, st8, t, n, t, t, ws, small) == 3               # the workspace of the plain flow is too small
        assert eng.launch_mlp_loss_grad(cshape, t, None, st8, t, n, t, t, ws, small, use_half_linear=False) == 1
        buf = torch.zeros(32, device=DEV)
        assert eng.set_batch_norm_state(None, 0.1, 2, buf, None) == 1                                   # a buffer without an exchange
        assert eng.set_batch_norm_state(None, 1.5, 1) == 1
        assert eng.set_batch_norm_state(None, 0.1, 0) == 1
    finally:
        eng.close()


# ---- the trainer binary with --batch-norm 1 ------------------------------------------------------------------------------
import json  # noqa: E402
import os  # noqa: E402
import subprocess  # noqa: E402

from helpers import trainer_init_weights  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "bin", "mgt_native_train")


def run_trainer(out_dir, *flags, rank=0, world=1, check=True, wait=True):
    cmd = [BIN, "--output-dir", str(out_dir), "--device-id", rank, "--world-size", world, "--global-rank", rank, "--local-rank", rank, *flags]
    if not wait:
        return subprocess.Popen([str(c) for c in cmd], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    res = subprocess.run([str(c) for c in cmd], capture_output=True, text=True, timeout=300)
    if check:
        assert res.returncode == 0, res.stderr + res.stdout
    return res


def oracle_bn_training(oracle, shape, *, batch, steps, k_max, lr, momentum, eps=1e-5, world=1, seed=1234):
    """The trainer's loop on the CPU oracle with batch normalisation over the joint batch of all ranks."""
    moves, target = oracle.cyclic_puzzle(72, 18)
    p, nbn = shape.param_count, oracle.bn_param_count(shape)
    w = np.concatenate([trainer_init_weights(p), np.zeros(nbn, np.float32)])
    w[p:].reshape(-1, 2, shape.hd2)[:, 0, :] = 1.0
    m, v = np.zeros_like(w), np.zeros_like(w)
    running = np.zeros((shape.residual_blocks + 1, 2, shape.hd2), np.float32)
    running[:, 1, :] = 1.0
    losses = []
    n = batch * world
    for step in range(steps):
        parts = [oracle.random_walks(moves, target, seed=seed, epoch=0, step=step, rank=r, k_min=1, k_max=k_max, samples=batch) for r in range(world)]
        states = np.concatenate([q[1] for q in parts])
        labels = np.concatenate([q[2] for q in parts]).reshape(-1, 1)
        st, loss, grad, stats = oracle.loss_grad_ex(shape, w, states, labels, batch_norm=True, bn_eps=eps)
        assert st == 0
        assert oracle.adamw(w, grad, m, v, step=step + 1, lr=lr) == 0
        running[:, 0, :] = (1 - momentum) * running[:, 0, :] + momentum * stats[:, 0, :]
        running[:, 1, :] = (1 - momentum) * running[:, 1, :] + momentum * stats[:, 1, :] * (n / (n - 1.0))
        losses.append(loss)
    return w, running, losses


def read_bn_state(run_dir, nbn):
    raw = np.fromfile(run_dir / "checkpoint" / "batch_norm.f32.bin", np.float32)
    assert raw.size == 4 * nbn
    return {name: raw[i * nbn:(i + 1) * nbn] for i, name in enumerate(("scale_shift", "adam_m", "adam_v", "running_stats"))}


def test_trainer_with_batch_norm_tracks_the_oracle_and_exports_folded_weights(tmp_path, oracle):
    shape = MlpShape(72, 72, 256, 64, 2, 1)
    cshape = cshape_of(shape)
    common = ["--batch-size", 512, "--k-min", 1, "--k-max", 29, "--hd1", 256, "--hd2", 64, "--nrd", 2, "--lr", 0.001, "--batch-norm", 1, "--bn-momentum", 0.2]
    d = tmp_path / "bn"
    run_trainer(d, "--steps", 3, *common)
    w, running, losses = oracle_bn_training(oracle, shape, batch=512, steps=3, k_max=29, lr=1e-3, momentum=0.2)
    rows = [json.loads(line) for line in open(d / "profile.jsonl")]
    for row, want in zip(rows, losses):
        assert abs(row["loss"] - want) <= 2e-3 * abs(want), (row["loss"], want)
    p, nbn = shape.param_count, oracle.bn_param_count(shape)
    state = np.fromfile(d / "checkpoint" / "state.f32.bin", np.float32)
    assert state.size == 3 * p                                           # the reference's checkpoint keeps its format
    bn = read_bn_state(d, nbn)
    # AdamW's first steps move every parameter by about lr whatever the gradient's size, so a sign flip of a near-zero
    # gradient shows as 2 * lr: compare against the distance travelled
    travelled = np.abs(w[:p] - trainer_init_weights(p)).max()
    # (the biases in front of a normalisation are left out: their true gradient is zero, what arrives is rounding noise
    # of either sign, and AdamW turns it into steps of +-lr)
    checked = np.ones(p, bool)
    hidden_b = 72 * 72 * 256 + 256 + 256 * 64
    checked[hidden_b:hidden_b + 64] = False
    for k in range(2):
        b2 = hidden_b + 64 + k * 2 * (64 * 64 + 64) + 64 * 64 + 64 + 64 * 64
        checked[b2:b2 + 64] = False
    diff = np.abs(state[:p] - w[:p])[checked]
    # (and a gradient at the edge of fp16 underflow is zero in one realisation and tiny in the other: no step against
    # a full one. Few elements are affected, each by at most the distance travelled.)
    assert np.quantile(diff, 0.99) <= 0.35 * travelled and diff.max() <= 1.1 * travelled, (np.quantile(diff, 0.99), diff.max(), travelled)
    assert rel_l2(state[:p][checked], w[:p][checked]) <= 0.2
    assert np.abs(bn["scale_shift"] - w[p:]).max() <= 0.7 * travelled
    np.testing.assert_allclose(bn["running_stats"].reshape(running.shape), running, rtol=2e-2, atol=2e-3)
    meta = json.load(open(d / "checkpoint" / "batch_norm.json"))
    assert meta["layers"] == 3 and meta["width"] == 64 and meta["section_floats"] == nbn
    # weights/ holds the folded network (no normalisation left), from the very code the library exports
    exported = np.fromfile(d / "weights" / "weights.f32.bin", np.float32)
    folded = mgt.fold_batch_norm(cshape, state[:p], bn["scale_shift"], bn["running_stats"], 1e-5)
    assert np.array_equal(exported, folded) and not np.array_equal(exported, state[:p])
    # 2 + 1 steps through a checkpoint end in the state of 3 steps in one run, normalisation state included
    run_trainer(tmp_path / "two", "--steps", 2, *common)
    run_trainer(tmp_path / "third", "--steps", 1, "--resume-checkpoint", tmp_path / "two" / "checkpoint", "--resume-step", 1, *common)
    assert np.array_equal(np.fromfile(tmp_path / "third" / "checkpoint" / "state.f32.bin", np.float32), state)
    again = read_bn_state(tmp_path / "third", nbn)
    assert all(np.array_equal(again[k], bn[k]) for k in bn)
    # a checkpoint without the normalisation state cannot be resumed with --batch-norm 1; bad values are refused
    run_trainer(tmp_path / "plain", "--steps", 1, *common[:-4])
    res = run_trainer(tmp_path / "bad", "--steps", 1, "--resume-checkpoint", tmp_path / "plain" / "checkpoint", *common, check=False)
    assert res.returncode != 0
    assert run_trainer(tmp_path / "bad2", "--steps", 1, *common, "--bn-eps", 0, check=False).returncode != 0
    assert run_trainer(tmp_path / "bad3", "--steps", 1, *common, "--linear-fp16", 0, check=False).returncode != 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_normalise_with_joint_statistics(tmp_path, oracle):
    shape = MlpShape(72, 72, 128, 32, 2, 1)
    id_file = tmp_path / "nccl.id"
    flags = ["--steps", 3, "--batch-size", 256, "--k-min", 1, "--k-max", 29, "--hd1", 128, "--hd2", 32, "--nrd", 2, "--lr", 0.001, "--batch-norm", 1,
             "--nccl-id-file", id_file]
    procs = [run_trainer(tmp_path / f"rank{r}", *flags, rank=r, world=2, wait=False) for r in range(2)]
    outs = [q.communicate(timeout=300) for q in procs]
    assert all(q.returncode == 0 for q in procs), outs
    nbn = oracle.bn_param_count(shape)
    states = [np.fromfile(tmp_path / f"rank{r}" / "checkpoint" / "state.f32.bin", np.float32) for r in range(2)]
    bns = [read_bn_state(tmp_path / f"rank{r}", nbn) for r in range(2)]
    assert np.array_equal(states[0], states[1]) and all(np.array_equal(bns[0][k], bns[1][k]) for k in bns[0])   # replicas bit-identical
    w, running, losses = oracle_bn_training(oracle, shape, batch=256, steps=3, k_max=29, lr=1e-3, momentum=0.1, world=2)
    np.testing.assert_allclose(bns[0]["running_stats"].reshape(running.shape), running, rtol=2e-2, atol=2e-3)   # statistics of BOTH ranks' samples
    rows = [[json.loads(line) for line in open(tmp_path / f"rank{r}" / "profile.jsonl")] for r in range(2)]
    assert rows[0][0]["overlap_ranges"] == 8                                                                     # 2 * 2 + 3 and the scale/shift range
    for i, want in enumerate(losses):
        got = 0.5 * (rows[0][i]["loss"] + rows[1][i]["loss"])    # each rank reports the loss of its own samples
        assert abs(got - want) <= 2e-3 * abs(want), (got, want)
