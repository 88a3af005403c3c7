"""use_half_linear / use_half_input_grad = 0 (the trainer's --linear-fp16 0 / --input-grad-fp16 0) through the C ABI.

fp32 linears are checked against the reference's fp32 CPU code at the tolerances of the reference's own GPU-vs-CPU
test (native/tests/cuda/test_cuda_mlp_backward_cpu_compare.cpp:92-99: same shapes, same data, loss 1e-5, gradients
2e-5 absolute + relative); the mixed combinations against the oracle's fp16 data-flow model."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

import multigputrainmlp_b200 as mgt  # noqa: E402
from helpers import compare_case_inputs, rel_l2  # noqa: E402
from oracle import MlpShape  # noqa: E402

DEV = "cuda:0"


@pytest.fixture(scope="module")
def engine():
    e = mgt.Engine(0)
    yield e
    e.close()


def run(engine, shape, w, states, labels, half_ig, half_lin, callback=None):
    cshape = mgt.CudaMlpShape(shape.state_len, shape.state_value_pad, shape.hd1, shape.hd2, shape.residual_blocks, shape.output_dim)
    b = states.shape[0]
    dw = torch.from_numpy(w).to(DEV)
    ds = torch.from_numpy(states).to(DEV)
    dl = torch.from_numpy(np.ascontiguousarray(labels)).to(DEV)
    loss = torch.zeros(1, device=DEV)
    grad = torch.full((shape.param_count,), float("nan"), device=DEV)
    floats = mgt.mlp_loss_grad_workspace_floats(cshape, b, 1, half_ig, half_lin)
    assert floats > 0
    ws = torch.full((floats,), float("nan"), device=DEV)
    st = engine.launch_mlp_loss_grad(cshape, dw, dw.half(), ds, dl, b, loss, grad, ws, floats, use_half_input_grad=half_ig,
                                     use_half_linear=half_lin, gradient_ready=callback)
    assert st == 0, mgt.status_name(st)
    st, code = engine.check()
    assert st == 0, code
    return float(loss.item()), grad.cpu().numpy()


# the three shapes of the reference's CUDA-vs-CPU comparison and its data generators
@pytest.mark.parametrize("dims,n", [((4, 8, 5, 3, 1, 1), 8), ((4, 8, 5, 3, 1, 3), 8), ((6, 8, 9, 7, 2, 11), 10)])
@pytest.mark.parametrize("half_ig", [False, True])
def test_fp32_linears_at_the_reference_tolerance(reference, oracle, engine, dims, n, half_ig):
    shape = MlpShape(*dims)
    w, states, labels = compare_case_inputs(shape, n)
    cpu = reference if reference is not None else oracle
    st, loss_o, grad_o = cpu.loss_grad(shape, w, states, labels)
    assert st == 0
    loss_g, grad_g = run(engine, shape, w, states, labels, half_ig, False)
    assert abs(loss_g - loss_o) <= 1e-5 + 1e-5 * abs(loss_o)
    if not half_ig:
        assert np.all(np.abs(grad_g - grad_o) <= 2e-5 + 2e-5 * np.abs(grad_o))
    else:  # the table gradient's operand is rounded to fp16 first
        assert rel_l2(grad_g, grad_o) <= 1e-3


def test_fp32_linears_walk_batch_and_notifications(oracle, engine):
    moves, target = oracle.cyclic_puzzle(72, 18)
    _, states, labels, _ = oracle.random_walks(moves, target, seed=7, epoch=0, step=0, rank=0, k_min=1, k_max=29, samples=333)
    shape = MlpShape(72, 72, 96, 40, 2, 1)
    w = (np.random.default_rng(3).standard_normal(shape.param_count) * 0.03).astype(np.float32)
    order = []

    def cb(user, ready_id, off, count, stream):
        order.append((ready_id, off, count))
        return 0
    st, loss_o, grad_o = oracle.loss_grad(shape, w, states, labels.reshape(-1, 1))
    loss_g, grad_g = run(engine, shape, w, states, labels.reshape(-1, 1), False, False, callback=cb)
    assert abs(loss_g - loss_o) <= 1e-5 * abs(loss_o)
    assert rel_l2(grad_g, grad_o) <= 1e-5
    assert [o[0] for o in order] == list(range(2 * 2 + 3)) and order[-1][1] == 0 and order[-1][2] == 72 * 72 * 96 + 96


def test_fp16_linears_with_fp32_table_gradient(oracle, engine):
    # --input-grad-fp16 0 with fp16 linears (the reference's ctest native_train_input_grad_float_backend)
    moves, target = oracle.cyclic_puzzle(72, 18)
    _, states, labels, _ = oracle.random_walks(moves, target, seed=11, epoch=0, step=0, rank=0, k_min=1, k_max=29, samples=500)
    shape = MlpShape(72, 72, 128, 64, 2, 1)
    w = (np.random.default_rng(5).standard_normal(shape.param_count) * 0.03).astype(np.float32)
    st, loss_o, grad_o = oracle.loss_grad_mixed(shape, w, states, labels.reshape(-1, 1))
    loss_f, grad_f = run(engine, shape, w, states, labels.reshape(-1, 1), False, True)
    loss_h, grad_h = run(engine, shape, w, states, labels.reshape(-1, 1), True, True)
    assert loss_f == loss_h  # the forward pass is the same
    assert rel_l2(grad_f, grad_o) <= 1e-3
    table = 72 * 72 * 128
    assert np.array_equal(grad_f[table + 128:], grad_h[table + 128:])  # only the table (and its bias sum) take the other route
    assert rel_l2(grad_f[:table], grad_h[:table]) <= 1e-3
