"""Shared deterministic input builders (the reference tests' own generators)."""
import numpy as np

from oracle import MlpShape


def compare_case_inputs(shape: MlpShape, samples: int):
    """native/tests/cuda/test_cuda_mlp_backward_cpu_compare.cpp:29-41"""
    i = np.arange(shape.param_count, dtype=np.int64)
    weights = (((i * 7) % 29 - 14) * 0.00325).astype(np.float32)
    labels = np.zeros((samples, shape.output_dim), np.float32)
    states = np.zeros((samples, 80), np.uint8)
    for s in range(samples):
        for o in range(shape.output_dim):
            labels[s, o] = np.float32(((s * 3 + o * 5 + shape.output_dim) % 17) - 8) * np.float32(0.0625)
        for k in range(shape.state_len):
            states[s, k] = (k * 3 + s * 5 + shape.output_dim) % shape.state_value_pad
    return weights, states, labels


def mixed_case_inputs(shape: MlpShape, samples: int):
    """native/tests/cuda/test_cuda_mlp_backward_mixed_precision_error.cu:36-50"""
    i = np.arange(shape.param_count, dtype=np.int64)
    weights = (((i * 5 + shape.output_dim) % 31 - 15) * 0.0015).astype(np.float32)
    labels = np.zeros((samples, shape.output_dim), np.float32)
    states = np.zeros((samples, 80), np.uint8)
    for s in range(samples):
        for o in range(shape.output_dim):
            labels[s, o] = np.float32(((s + 3 * o) % 7) - 3) * np.float32(0.125)
        for k in range(shape.state_len):
            states[s, k] = (s + 3 * k + shape.output_dim) % shape.state_value_pad
    return weights, states, labels


def trainer_init_weights(param_count: int):
    """native/tools/mgt_native_train_smoke.cu:648-650"""
    i = np.arange(param_count, dtype=np.int64)
    return ((i % 29 - 14) * 0.0001).astype(np.float64).astype(np.float32)


def rel_l2(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    return float(np.sqrt(((a - b) ** 2).sum() / max((b ** 2).sum(), 1e-30)))
