"""GPU parity of the loss+gradient engine (forward, loss, backward) against the CPU oracle's
restatement of the reference's fp16 data flow, through the C ABI."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

import multigputrainmlp_b200 as mgt  # noqa: E402
from helpers import compare_case_inputs, mixed_case_inputs, rel_l2, trainer_init_weights  # noqa: E402
from oracle import MlpShape  # noqa: E402

DEV = "cuda:0"


@pytest.fixture(scope="module")
def engine():
    e = mgt.Engine(0)
    yield e
    e.close()


def run_engine(engine, shape: MlpShape, w, states, labels, persistent_mirror=True, callback=None, profile=None):
    w = np.ascontiguousarray(w[:shape.param_count])
    cshape = mgt.CudaMlpShape(shape.state_len, shape.state_value_pad, shape.hd1, shape.hd2, shape.residual_blocks, shape.output_dim)
    b = states.shape[0]
    dw = torch.from_numpy(w).to(DEV)
    dh = dw.half() if persistent_mirror else None
    ds = torch.from_numpy(states).to(DEV)
    dl = torch.from_numpy(np.ascontiguousarray(labels)).to(DEV)
    loss = torch.zeros(1, device=DEV)
    grad = torch.full((shape.param_count,), float("nan"), device=DEV)
    floats = mgt.mlp_loss_grad_workspace_floats(cshape, b)
    assert floats > 0
    ws = torch.empty(floats, device=DEV)
    ws.fill_(float("nan"))  # the engine must not depend on the workspace's previous contents
    st = engine.launch_mlp_loss_grad(cshape, dw, dh, ds, dl, b, loss, grad, ws, floats, gradient_ready=callback, profile=profile)
    assert st == 0, mgt.status_name(st)
    st, code = engine.check()
    assert st == 0, f"device status {code}"
    return float(loss.item()), grad.cpu().numpy()


def check_against_oracle(oracle, engine, shape, w, states, labels, tol=1e-3, section_tol=None, **kw):
    st, loss_o, grad_o = oracle.loss_grad_mixed(shape, w, states, labels)
    assert st == 0
    loss_g, grad_g = run_engine(engine, shape, w, states, labels, **kw)
    assert np.isfinite(grad_g).all()
    # tolerance of the headline metric: per-step loss and gradients within 1e-3 relative (norm-wise)
    assert abs(loss_g - loss_o) <= tol * max(abs(loss_o), 1e-6), (loss_g, loss_o)
    assert rel_l2(grad_g, grad_o) <= tol, rel_l2(grad_g, grad_o)
    # per-section check so that a small block cannot hide behind the embedding table
    in_w = shape.state_len * shape.state_value_pad * shape.hd1
    sections = {"embedding": (0, in_w), "input_bias": (in_w, in_w + shape.hd1),
                "hidden": (in_w + shape.hd1, in_w + shape.hd1 + shape.hd1 * shape.hd2 + shape.hd2),
                "tail": (in_w + shape.hd1 + shape.hd1 * shape.hd2 + shape.hd2, shape.param_count)}
    for name, (lo, hi) in sections.items():
        if np.abs(grad_o[lo:hi]).max() > 0:
            assert rel_l2(grad_g[lo:hi], grad_o[lo:hi]) <= (section_tol or 3 * tol), (name, rel_l2(grad_g[lo:hi], grad_o[lo:hi]))
    return loss_g, grad_g, loss_o, grad_o


@pytest.mark.parametrize("dims,n", [((8, 8, 16, 16, 2, 1), 32), ((8, 8, 16, 16, 2, 3), 32), ((8, 8, 16, 16, 2, 17), 32), ((5, 8, 8, 8, 1, 128), 16)])
def test_reference_mixed_precision_cases(oracle, engine, dims, n):
    # shapes and inputs of native/tests/cuda/test_cuda_mlp_backward_mixed_precision_error.cu
    shape = MlpShape(*dims)
    w, s, l = mixed_case_inputs(shape, n)
    loss_g, grad_g, _, _ = check_against_oracle(oracle, engine, shape, w, s, l)
    # and the reference's own envelope against the true-fp32 CPU reference
    _, loss_ref, grad_ref = oracle.loss_grad(shape, w, s, l)
    assert abs(loss_ref - loss_g) <= 2e-3 + 2e-2 * max(abs(loss_ref), abs(loss_g))
    assert rel_l2(grad_g, grad_ref) <= 8e-2 and np.abs(grad_g - grad_ref).max() <= 2e-2


@pytest.mark.parametrize("dims,n", [((4, 8, 5, 3, 1, 1), 8), ((4, 8, 5, 3, 1, 3), 8), ((6, 8, 9, 7, 2, 11), 10), ((72, 72, 40, 24, 0, 1), 300)])
def test_odd_shapes_and_no_mirror(oracle, engine, dims, n):
    # unaligned hidden sizes (the reference's cpu-compare shapes) go through the padded fp16 weight copy
    shape = MlpShape(*dims)
    w, s, l = compare_case_inputs(shape, n)
    check_against_oracle(oracle, engine, shape, w, s, l, persistent_mirror=False)


def test_walk_batch_medium_model(oracle, engine):
    moves, target = oracle.cyclic_puzzle(72, 18)
    _, states, labels, _ = oracle.random_walks(moves, target, seed=1234, epoch=0, step=0, rank=0, k_min=1, k_max=29, samples=700)
    shape = MlpShape(72, 72, 256, 64, 2, 1)
    rng = np.random.default_rng(1)
    w = (rng.standard_normal(shape.param_count) * 0.03).astype(np.float32)
    order = []
    def cb(user, ready_id, off, count, stream):
        order.append((ready_id, off, count))
        return 0
    check_against_oracle(oracle, engine, shape, w, states, labels.reshape(-1, 1), callback=cb)
    # gradient-ready notifications: native/cuda/mlp_backward.cu:1364,1385,1402,1427,1506
    h1, h2, r = 256, 64, 2
    in_w = 72 * 72 * h1
    hidden = in_w + h1
    rbase = hidden + h1 * h2 + h2
    blk = 2 * (h2 * h2 + h2)
    want = [(0, rbase + r * blk, h2 + 1)]
    for k in (1, 0):
        want.append((len(want), rbase + k * blk + h2 * h2 + h2, h2 * h2 + h2))
        want.append((len(want), rbase + k * blk, h2 * h2 + h2))
    want.append((len(want), hidden, h1 * h2 + h2))
    want.append((len(want), 0, in_w + h1))
    assert order == want


def _walk_case(oracle, dims, n, seed):
    moves, target = oracle.cyclic_puzzle(72, 18)
    _, states, labels, _ = oracle.random_walks(moves, target, seed=seed, epoch=0, step=0, rank=0, k_min=1, k_max=29, samples=n)
    shape = MlpShape(*dims)
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal(shape.param_count) * 0.03).astype(np.float32)
    lab = labels.reshape(-1, 1).astype(np.float32)
    if shape.output_dim > 1:
        lab = np.repeat(lab, shape.output_dim, axis=1) * np.linspace(0.5, 1.5, shape.output_dim, dtype=np.float32)
    return shape, w, states, np.ascontiguousarray(lab)


# hidden widths the fused residual-tower kernels take (multiples of 32 up to 256), ragged last tiles included
@pytest.mark.parametrize("dims,n", [((72, 72, 128, 224, 3, 1), 900), ((72, 72, 64, 256, 2, 1), 300), ((72, 72, 64, 96, 5, 3), 260),
                                     ((72, 72, 64, 160, 1, 1), 128)])
def test_residual_tower_fused(oracle, engine, dims, n):
    shape, w, states, labels = _walk_case(oracle, dims, n, seed=77)
    check_against_oracle(oracle, engine, shape, w, states, labels)


def test_reference_hard_caps(oracle, engine):
    # hd1 4096, hd2 512 are the reference's compile-time caps (native/cuda/mlp_forward.cu:7-9); 29 outputs as in the
    # depth-classification variant; hd2 > 256 takes the per-layer residual path
    shape, w, states, labels = _walk_case(oracle, (72, 72, 4096, 512, 2, 29), 96, seed=3)
    check_against_oracle(oracle, engine, shape, w * 0.3, states, labels)


def test_residual_tower_layered_matches_fused(oracle, engine, monkeypatch):
    # the per-layer GEMM path (taken for other widths) on a width both paths accept
    shape, w, states, labels = _walk_case(oracle, (72, 72, 64, 64, 3, 1), 500, seed=5)
    loss_f, grad_f = run_engine(engine, shape, w, states, labels)
    monkeypatch.setenv("MGT_RESIDUAL_PATH", "layered")
    layered = mgt.Engine(0)
    try:
        check_against_oracle(oracle, layered, shape, w, states, labels)
        loss_l, grad_l = run_engine(layered, shape, w, states, labels)
    finally:
        layered.close()
    assert abs(loss_f - loss_l) <= 1e-5 * abs(loss_l)
    assert rel_l2(grad_f, grad_l) <= 1e-4


def test_trainer_init_weights_first_step(oracle, engine):
    # the trainer's deterministic initial weights (tool:648-650) on a walk batch, physical dims of a padded model
    moves, target = oracle.cyclic_puzzle(72, 18)
    _, states, labels, _ = oracle.random_walks(moves, target, seed=1234, epoch=0, step=0, rank=0, k_min=1, k_max=29, samples=384)
    shape = MlpShape(72, 72, 128, 32, 3, 1)
    w = trainer_init_weights(shape.param_count)
    prof = mgt.BackwardProfile()
    check_against_oracle(oracle, engine, shape, w, states, labels.reshape(-1, 1), profile=prof)
    assert prof.input_forward_ms > 0 and prof.input_grad_ms > 0


@pytest.mark.parametrize("weights", ["trainer_init", "random"])
def test_physical_p888_shape(oracle, engine, weights):
    # the headline model at its physical dims (72 x 72 -> 2560 -> 224, 16 blocks, 1 output: 15 460 289 parameters) on a walk
    # batch the oracle finishes in seconds: the 224-wide fused tower at its full depth, the 2560-wide embedding and hidden layers
    moves, target = oracle.cyclic_puzzle(72, 18)
    _, states, labels, _ = oracle.random_walks(moves, target, seed=1234, epoch=0, step=3, rank=0, k_min=1, k_max=29, samples=512)
    shape = MlpShape(72, 72, 2560, 224, 16, 1)
    assert shape.param_count == 15_460_289
    if weights == "trainer_init":
        w = trainer_init_weights(shape.param_count)
    else:
        # He-like scales per layer keep the activations O(1) through 16 blocks (a flat 0.03 would overflow fp16 here)
        rng = np.random.default_rng(11)
        w = np.empty(shape.param_count, np.float32)
        in_w = 72 * 72 * 2560
        w[:in_w] = rng.standard_normal(in_w) * 0.08
        w[in_w:in_w + 2560] = rng.standard_normal(2560) * 0.05
        lo = in_w + 2560
        w[lo:lo + 2560 * 224 + 224] = rng.standard_normal(2560 * 224 + 224) * 0.02
        lo += 2560 * 224 + 224
        w[lo:] = rng.standard_normal(shape.param_count - lo) * 0.04
    # With the trainer's 1e-4-scale initial weights the stated 1e-3 holds. With O(1) random weights 33 fp16-rounded layers
    # amplify every last-bit difference in summation order: the rounding-point model itself sits 4.2e-3 (gradient rel-L2;
    # 2.2e-2 on the embedding table, whose gradient is a sum of fp16-rounded dz1 rows) from the true-fp32 reference on
    # this case. Two correct fp16 realisations then agree only to that order, so the GPU result is held to the model
    # within 5e-3 overall and, section by section, to 1.5 x the model's own distance from fp32.
    base = 72 * 72 * 2560 + 2560 + 2560 * 224 + 224
    blk = 2 * (224 * 224 + 224)
    lab = labels.reshape(-1, 1)
    if weights == "trainer_init":
        loss_g, grad_g, loss_o, grad_o = check_against_oracle(oracle, engine, shape, w, states, lab)
        for k in range(16):  # every residual block on its own: weights and biases of fc1/fc2 of block k
            lo, hi = base + k * blk, base + (k + 1) * blk
            if np.abs(grad_o[lo:hi]).max() > 0:
                assert rel_l2(grad_g[lo:hi], grad_o[lo:hi]) <= 3e-3, (k, rel_l2(grad_g[lo:hi], grad_o[lo:hi]))
        return
    loss_g, grad_g, loss_o, grad_o = check_against_oracle(oracle, engine, shape, w, states, lab, tol=5e-3, section_tol=1.0)
    assert abs(loss_g - loss_o) <= 1e-3 * abs(loss_o)
    _, loss_f, grad_f = oracle.loss_grad(shape, w, states, lab)
    in_w = 72 * 72 * 2560
    sections = [("embedding", 0, in_w), ("input_bias", in_w, in_w + 2560), ("hidden", in_w + 2560, base)]
    sections += [(f"block{k}", base + k * blk, base + (k + 1) * blk) for k in range(16)] + [("output", base + 16 * blk, shape.param_count)]
    for name, lo, hi in sections:
        model_error = rel_l2(grad_o[lo:hi], grad_f[lo:hi])
        assert rel_l2(grad_g[lo:hi], grad_o[lo:hi]) <= 1.5 * model_error + 1e-4, (name, rel_l2(grad_g[lo:hi], grad_o[lo:hi]), model_error)
        assert rel_l2(grad_g[lo:hi], grad_f[lo:hi]) <= 1.5 * model_error + 1e-4, (name, rel_l2(grad_g[lo:hi], grad_f[lo:hi]), model_error)


# ---- options the reference does not have (pinned by the oracle's finite-difference tests, not by the reference) ----------
def _options_case(oracle, dims, n, seed, scale=0.03):
    moves, target = oracle.cyclic_puzzle(72, 18)
    _, states, depth, _ = oracle.random_walks(moves, target, seed=seed, epoch=0, step=0, rank=0, k_min=1, k_max=29, samples=n)
    shape = MlpShape(*dims)
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal(shape.param_count) * scale).astype(np.float32)
    labels = np.ascontiguousarray(np.repeat(depth.reshape(-1, 1), shape.output_dim, axis=1).astype(np.float32))  # what ExpandScalarLabels writes
    return shape, w, states, labels


def _check_option_case(oracle, shape, w, states, labels, *, bf16, cross_entropy, tol):
    eng = mgt.Engine(0)
    try:
        assert eng.set_train_options(bf16=bf16, cross_entropy=cross_entropy) == 0
        loss_g, grad_g = run_engine(eng, shape, w, states, labels)
    finally:
        eng.close()
    st, loss_o, grad_o, _ = oracle.loss_grad_ex(shape, w, states, labels, bf16=bf16, cross_entropy=cross_entropy)
    assert st == 0 and np.isfinite(grad_g).all()
    assert abs(loss_g - loss_o) <= tol * max(abs(loss_o), 1e-6), (loss_g, loss_o)
    assert rel_l2(grad_g, grad_o) <= tol, rel_l2(grad_g, grad_o)
    # and against exact arithmetic: no further from it than the rounding model is
    st, loss_f, grad_f, _ = oracle.loss_grad_ex(shape, w, states, labels, half_linear=False, half_input_grad=False, cross_entropy=cross_entropy)
    model_error = rel_l2(grad_o, grad_f)
    assert rel_l2(grad_g, grad_f) <= 1.5 * model_error + 1e-4, (rel_l2(grad_g, grad_f), model_error)
    return loss_g, grad_g


@pytest.mark.parametrize("dims,n", [((72, 72, 128, 224, 3, 29), 600), ((72, 72, 64, 64, 2, 5), 257), ((72, 72, 40, 24, 1, 29), 100)])
def test_cross_entropy_on_depth(oracle, dims, n):
    shape, w, states, labels = _options_case(oracle, dims, n, seed=21)
    if shape.output_dim < 29:
        labels = np.minimum(labels, shape.output_dim)
    loss, _ = _check_option_case(oracle, shape, w, states, labels, bf16=False, cross_entropy=True, tol=2e-3)
    assert 0.5 * np.log(shape.output_dim) < loss < 2.0 * np.log(shape.output_dim)  # near-uniform logits at these weight scales


@pytest.mark.parametrize("dims,n", [((72, 72, 128, 224, 3, 1), 500), ((72, 72, 64, 96, 2, 3), 260), ((72, 72, 40, 24, 1, 1), 100)])
def test_bfloat16_operands(oracle, dims, n):
    # 8 bits of mantissa: a last-bit flip is 2^-9 of the value, so two correct realisations agree to a few 1e-3
    shape, w, states, labels = _options_case(oracle, dims, n, seed=22)
    _check_option_case(oracle, shape, w, states, labels, bf16=True, cross_entropy=False, tol=8e-3)


def test_wide_deep_variant_bf16_cross_entropy(oracle):
    # hd1 4096, hd2 512 (the reference's compile-time caps, per-layer residual path), 29 per-depth logits, bfloat16, cross-entropy
    shape, w, states, labels = _options_case(oracle, (72, 72, 4096, 512, 2, 29), 96, seed=23, scale=0.01)
    _check_option_case(oracle, shape, w, states, labels, bf16=True, cross_entropy=True, tol=8e-3)


def test_option_errors(engine):
    cshape = mgt.CudaMlpShape(8, 8, 16, 16, 2, 1)
    t = torch.zeros(4096, device=DEV)
    floats = mgt.mlp_loss_grad_workspace_floats(cshape, 32)
    big = torch.zeros(floats, device=DEV)
    st8 = torch.zeros(32, 80, dtype=torch.uint8, device=DEV)
    eng = mgt.Engine(0)
    try:
        assert eng.set_train_options(cross_entropy=True) == 0
        assert eng.launch_mlp_loss_grad(cshape, t, None, st8, t, 32, t, t, big, floats) == 1            # one output has no classes
        assert eng.set_train_options(bf16=True) == 0
        assert eng.launch_mlp_loss_grad(cshape, t, None, st8, t, 32, t, t, big, floats, use_half_linear=False) == 1  # options need the tensor-core flow
        assert eng.set_train_options() == 0
    finally:
        eng.close()


def test_argument_errors(engine):
    cshape = mgt.CudaMlpShape(8, 8, 16, 16, 2, 1)
    t = torch.zeros(4096, device=DEV)
    floats = mgt.mlp_loss_grad_workspace_floats(cshape, 32)
    big = torch.zeros(floats, device=DEV)
    st8 = torch.zeros(32, 80, dtype=torch.uint8, device=DEV)
    args = (cshape, t, None, st8, t, 32, t, t)
    assert engine.launch_mlp_loss_grad(*args, big, floats - 1) == 3                      # capacity_exceeded (mlp_backward.cu:1256)
    assert engine.launch_mlp_loss_grad(*args, big, floats, input_grad_partial_chunks=0) == 1
    assert engine.launch_mlp_loss_grad(*args, big, floats, input_grad_positions_per_block=0) == 1
    assert engine.launch_mlp_loss_grad(cshape, None, None, st8, t, 32, t, t, big, floats) == 1
    assert engine.launch_mlp_loss_grad(mgt.CudaMlpShape(8, 8, 5000, 16, 2, 1), t, None, st8, t, 32, t, t, big, floats) == 1  # hd1 > 4096
    assert mgt.mlp_loss_grad_workspace_floats(mgt.CudaMlpShape(73, 8, 16, 16, 2, 1), 32) == 0
    assert mgt.validate_cuda_mlp_shape(mgt.CudaMlpShape(72, 72, 4096, 512, 32, 29)) == 0
