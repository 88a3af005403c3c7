"""mgt_fold_batch_norm (host code, no GPU): a network with batch normalisation, evaluated with fixed statistics, equals
the folded network without normalisation. The oracle provides both sides: its batch-norm path normalises with the
statistics of the batch in flight, so folding with exactly those statistics must reproduce its loss."""
import numpy as np
import pytest

import multigputrainmlp_b200 as mgt
from oracle import MlpShape


@pytest.mark.parametrize("dims,n", [((8, 8, 16, 12, 2, 1), 48), ((6, 8, 9, 7, 3, 4), 40), ((8, 8, 16, 8, 0, 1), 32)])
def test_folded_network_reproduces_the_normalised_one(oracle, dims, n):
    shape = MlpShape(*dims)
    cshape = mgt.CudaMlpShape(*dims)
    rng = np.random.default_rng(5)
    nbn = oracle.bn_param_count(shape)
    assert nbn == mgt.bn_param_count(cshape)
    w = (rng.standard_normal(shape.param_count + nbn) * 0.2).astype(np.float32)
    bn = w[shape.param_count:].reshape(shape.residual_blocks + 1, 2, shape.hd2)
    bn[:, 0, :] = 1.0 + 0.3 * rng.standard_normal(bn[:, 0, :].shape)
    states = np.zeros((n, 80), np.uint8)
    states[:, :shape.state_len] = rng.integers(0, shape.state_value_pad, (n, shape.state_len))
    labels = rng.standard_normal((n, shape.output_dim)).astype(np.float32)
    eps = 1e-5
    st, loss_bn, _, stats = oracle.loss_grad_ex(shape, w, states, labels, half_linear=False, half_input_grad=False, batch_norm=True, bn_eps=eps)
    assert st == 0
    folded = mgt.fold_batch_norm(cshape, w[:shape.param_count], w[shape.param_count:], stats, eps)
    st, loss_folded, _ = oracle.loss_grad(shape, folded, states, labels)
    assert st == 0
    assert abs(loss_folded - loss_bn) <= 2e-5 * abs(loss_bn)
    # only the layers that a normalisation follows change: hidden weight + bias and every fc2 weight + bias
    h1, h2 = shape.hd1, shape.hd2
    changed = np.flatnonzero(folded != w[:shape.param_count])
    hidden_lo = shape.state_len * shape.state_value_pad * h1 + h1
    tower = hidden_lo + h1 * h2 + h2
    allowed = np.zeros(shape.param_count, bool)
    allowed[hidden_lo:tower] = True
    for k in range(shape.residual_blocks):
        fc2 = tower + k * 2 * (h2 * h2 + h2) + h2 * h2 + h2
        allowed[fc2:fc2 + h2 * h2 + h2] = True
    assert allowed[changed].all() and changed.size > 0.9 * allowed.sum()


def test_fold_argument_errors():
    cshape = mgt.CudaMlpShape(8, 8, 16, 12, 2, 1)
    p, n = cshape.param_count, mgt.bn_param_count(cshape)
    w, ss, rs = np.zeros(p, np.float32), np.ones(n, np.float32), np.ones(n, np.float32)
    with pytest.raises(mgt.MgtError):
        mgt.fold_batch_norm(cshape, w, ss, rs, eps=0.0)
    with pytest.raises(mgt.MgtError):
        mgt.fold_batch_norm(cshape, w[:-1], ss, rs)
    with pytest.raises(mgt.MgtError):
        mgt.fold_batch_norm(mgt.CudaMlpShape(73, 8, 16, 12, 2, 1), w, ss, rs)
