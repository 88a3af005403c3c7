"""Host-side mirror of the reference's launch API (namespace mgt_cuda) over the C ABI.

Names follow the reference: RandomWalkKernelConfig / LaunchRandomWalkKernel
(native/cuda/mgt_cuda/random_walk_kernel.cuh), CudaMlpShape / MlpLossGradWorkspaceFloats /
LaunchMlpLossGrad... (native/cuda/mgt_cuda/mlp_backward.cuh), AdamWKernelConfig /
LaunchAdamWKernel[WithHalfMirror] (native/cuda/mgt_cuda/adamw.cuh). Functions return the
reference's status codes as ints; device buffers are torch CUDA tensors owned by the caller.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

from . import _lib

STATUS = {0: "ok", 1: "invalid_config", 2: "invalid_puzzle", 3: "capacity_exceeded", 4: "cuda_failure",
          5: "nccl_failure", 6: "io_failure", 7: "device_timeout"}


class MgtError(RuntimeError):
    def __init__(self, status: int, what: str):
        super().__init__(f"{what}: status {status} ({STATUS.get(status, 'unknown')})")
        self.status = status


def status_name(status: int) -> str:
    return _lib.load().mgt_status_name(status).decode()


def _ptr(t):
    if t is None:
        return None
    if hasattr(t, "data_ptr"):
        return C.c_void_p(t.data_ptr())
    return C.c_void_p(int(t))


def _stream(stream):
    if stream is None:
        import torch
        stream = torch.cuda.current_stream()
    return C.c_void_p(stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream))


class _WalkCfg(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("sample_count", "k_min", "k_max", "move_count", "state_len", "state_storage_len")]


class _Shape(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("state_len", "state_value_pad", "hd1", "hd2", "residual_blocks", "output_dim")]


class _Adam(C.Structure):
    _fields_ = [("param_count", C.c_uint64), ("step", C.c_uint64), ("learning_rate", C.c_float), ("beta1", C.c_float),
                ("beta2", C.c_float), ("eps", C.c_float), ("weight_decay", C.c_float)]


class BackwardProfile(C.Structure):
    """mgt_cuda::MlpBackwardProfile (native/cuda/mgt_cuda/mlp_backward.cuh:11-19)."""
    _fields_ = [(n, C.c_float) for n in ("input_forward_ms", "hidden_forward_ms", "residual_forward_ms", "output_ms",
                                         "residual_backward_ms", "hidden_backward_ms", "input_grad_ms")]


@dataclass
class RandomWalkKernelConfig:
    sample_count: int = 0
    k_min: int = 0
    k_max: int = 0
    move_count: int = 18
    state_len: int = 72
    state_storage_len: int = 80

    def c(self):
        return _WalkCfg(self.sample_count, self.k_min, self.k_max, self.move_count, self.state_len, self.state_storage_len)


@dataclass
class CudaMlpShape:
    state_len: int
    state_value_pad: int
    hd1: int
    hd2: int
    residual_blocks: int
    output_dim: int = 1

    def c(self):
        return _Shape(self.state_len, self.state_value_pad, self.hd1, self.hd2, self.residual_blocks, self.output_dim)

    @property
    def param_count(self) -> int:
        shape = self.c()
        return int(_lib.load().mgt_mlp_param_count(C.byref(shape)))


@dataclass
class AdamWKernelConfig:
    param_count: int
    step: int
    learning_rate: float
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.0

    def c(self):
        return _Adam(self.param_count, self.step, self.learning_rate, self.beta1, self.beta2, self.eps, self.weight_decay)


def launch_expand_scalar_labels(scalar_labels, sample_count: int, output_dim: int, expanded_labels, stream=None) -> int:
    """ExpandScalarLabelsKernel (native/tools/mgt_native_train_smoke.cu:74-80): labels[b][o] = scalar[b] for every output."""
    return int(_lib.load().mgt_launch_expand_scalar_labels(_ptr(scalar_labels), sample_count, output_dim, _ptr(expanded_labels), _stream(stream)))


def validate_random_walk_kernel_config(config: RandomWalkKernelConfig) -> int:
    cfg = config.c()
    return int(_lib.load().mgt_validate_random_walk_config(C.byref(cfg)))


def launch_random_walk_kernel(config, base_seed, epoch, step, global_rank, device_moves, device_target, device_states,
                              device_labels, device_meta, stream=None) -> int:
    cfg = config.c()
    return int(_lib.load().mgt_launch_random_walk(C.byref(cfg), base_seed & (2**64 - 1), epoch, step, global_rank,
                                                  _ptr(device_moves), _ptr(device_target), _ptr(device_states),
                                                  _ptr(device_labels), _ptr(device_meta), _stream(stream)))


def load_puzzle_definition(group_json: str, target_bin: str, group_id: int = 888, state_len: int = 72, move_count: int = 18):
    """LoadPuzzleDefinition (native/src/puzzle_io.cpp:48-97): returns (status, moves[18][80] uint8, target[80] uint8)."""
    import numpy as np
    moves = np.zeros((18, 80), np.uint8)
    target = np.zeros(80, np.uint8)
    lib = _lib.load()
    lib.mgt_load_puzzle_definition.argtypes = [C.c_char_p, C.c_char_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p]
    st = int(lib.mgt_load_puzzle_definition(str(group_json).encode(), str(target_bin).encode(), group_id, state_len, move_count,
                                            moves.ctypes.data_as(C.c_void_p), target.ctypes.data_as(C.c_void_p)))
    return st, moves, target


def validate_cuda_mlp_shape(shape: CudaMlpShape) -> int:
    s = shape.c()
    return int(_lib.load().mgt_validate_mlp_shape(C.byref(s)))


class _TrainOptions(C.Structure):
    """mgt_train_options_t"""
    _fields_ = [("operand_format", C.c_int32), ("loss_kind", C.c_int32), ("batch_norm", C.c_int32), ("bn_eps", C.c_float)]


def mlp_loss_grad_workspace_floats(shape, sample_count, input_grad_partial_chunks=1, use_half_input_grad=True,
                                   use_half_linear=True, batch_norm=False) -> int:
    s = shape.c()
    lib = _lib.load()
    if not batch_norm:
        return int(lib.mgt_mlp_loss_grad_workspace_floats(C.byref(s), sample_count, input_grad_partial_chunks,
                                                          int(use_half_input_grad), int(use_half_linear)))
    opt = _TrainOptions(0, 0, 1, 1e-5)
    lib.mgt_mlp_loss_grad_workspace_floats_with_options.restype = C.c_uint64
    lib.mgt_mlp_loss_grad_workspace_floats_with_options.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_int32, C.c_int32, C.c_void_p]
    return int(lib.mgt_mlp_loss_grad_workspace_floats_with_options(C.byref(s), sample_count, input_grad_partial_chunks,
                                                                   int(use_half_input_grad), int(use_half_linear), C.byref(opt)))


def bn_param_count(shape) -> int:
    """mgt_bn_param_count: floats of batch-norm scale/shift that follow the reference's parameters (2 * (blocks + 1) * hd2)."""
    s = shape.c()
    lib = _lib.load()
    lib.mgt_bn_param_count.restype = C.c_uint64
    lib.mgt_bn_param_count.argtypes = [C.c_void_p]
    return int(lib.mgt_bn_param_count(C.byref(s)))


def fold_batch_norm(shape, weights, scale_shift, running_stats, eps: float = 1e-5):
    """mgt_fold_batch_norm on host arrays: a copy of `weights` (the reference's layout) with the normalisation folded into
    the hidden layer and into every block's fc2, using the running statistics. Raises MgtError on a bad argument."""
    import numpy as np
    s = shape.c()
    lib = _lib.load()
    out = np.array(weights, dtype=np.float32, copy=True).ravel()
    ss = np.ascontiguousarray(scale_shift, dtype=np.float32).ravel()
    rs = np.ascontiguousarray(running_stats, dtype=np.float32).ravel()
    n = bn_param_count(shape)
    if out.size != shape.param_count or ss.size != n or rs.size != n:
        raise MgtError(1, "fold_batch_norm: array sizes")
    lib.mgt_fold_batch_norm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float]
    st = int(lib.mgt_fold_batch_norm(C.byref(s), out.ctypes.data_as(C.c_void_p), ss.ctypes.data_as(C.c_void_p), rs.ctypes.data_as(C.c_void_p), eps))
    if st != 0:
        raise MgtError(st, "fold_batch_norm")
    return out


STATS_EXCHANGE_FN = C.CFUNCTYPE(C.c_int32, C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p)
GRADIENT_READY_FN = C.CFUNCTYPE(C.c_int32, C.c_void_p, C.c_uint32, C.c_uint64, C.c_uint64, C.c_void_p)


class Engine:
    """Owner of the opaque engine handle (stands where the reference passes cuBLAS handles)."""

    def __init__(self, device_id: int = 0):
        self._lib = _lib.load()
        handle = C.c_void_p()
        st = self._lib.mgt_engine_create(device_id, C.byref(handle))
        if st != 0:
            raise MgtError(st, "mgt_engine_create")
        self.handle = handle

    def close(self):
        if getattr(self, "handle", None):
            self._lib.mgt_engine_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def launch_count(self) -> int:
        return int(self._lib.mgt_engine_launch_count(self.handle))

    def check(self, stream=None):
        code = C.c_int32(0)
        st = int(self._lib.mgt_engine_check(self.handle, _stream(stream), C.byref(code)))
        return st, int(code.value)

    def set_train_options(self, bf16: bool = False, cross_entropy: bool = False, batch_norm: bool = False, bn_eps: float = 1e-5) -> int:
        """mgt_engine_set_train_options: bfloat16 operands, cross-entropy on depth - 1, batch normalisation (defaults = the reference)."""
        opt = _TrainOptions(int(bf16), int(cross_entropy), int(batch_norm), float(bn_eps))
        self._lib.mgt_engine_set_train_options.argtypes = [C.c_void_p, C.c_void_p]
        return int(self._lib.mgt_engine_set_train_options(self.handle, C.byref(opt)))

    def set_batch_norm_state(self, running_stats=None, momentum: float = 0.1, world_size: int = 1, exchange_buffer=None, exchange=None) -> int:
        """mgt_engine_set_batch_norm_state. `exchange(user, device_pointer, float_count, stream) -> status` must enqueue an
        in-place average of the buffer over all ranks on `stream`; `exchange_buffer` is a device tensor or a raw pointer."""
        cb = STATS_EXCHANGE_FN(exchange) if exchange is not None else None
        self._stats_keepalive = (cb, running_stats, exchange_buffer)
        buf = exchange_buffer if isinstance(exchange_buffer, int) or exchange_buffer is None else _ptr(exchange_buffer)
        self._lib.mgt_engine_set_batch_norm_state.argtypes = [C.c_void_p, C.c_void_p, C.c_float, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p]
        return int(self._lib.mgt_engine_set_batch_norm_state(self.handle, _ptr(running_stats), momentum, world_size, buf,
                                                             C.cast(cb, C.c_void_p) if cb is not None else None, None))

    def set_early_range_hook(self, fn=None) -> int:
        """mgt_engine_set_early_range_hook: fn(user, ready_id, offset, count, stream) -> status, or None to remove it."""
        cb = GRADIENT_READY_FN(fn) if fn is not None else None
        self._early_keepalive = cb
        self._lib.mgt_engine_set_early_range_hook.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        return int(self._lib.mgt_engine_set_early_range_hook(self.handle, C.cast(cb, C.c_void_p) if cb is not None else None, None))

    def launch_mlp_loss_grad(self, shape, device_weights, device_weights_half, device_states, device_labels, sample_count,
                             device_loss, device_grad, workspace, workspace_floats, input_grad_partial_chunks=1,
                             input_grad_positions_per_block=1, use_half_input_grad=True, use_half_linear=True,
                             profile=None, gradient_ready=None, stream=None, input_grad_position_tile=0) -> int:
        """LaunchMlpLossGrad...ExternalHalf (native/cuda/mgt_cuda/mlp_backward.cuh:224-287)."""
        s = shape.c()
        cb = GRADIENT_READY_FN(gradient_ready) if gradient_ready is not None else None
        self._keepalive = cb
        return int(self._lib.mgt_launch_mlp_loss_grad(
            self.handle, C.byref(s), _ptr(device_weights), _ptr(device_weights_half), _ptr(device_states), _ptr(device_labels),
            sample_count, _ptr(device_loss), _ptr(device_grad), _ptr(workspace), workspace_floats, input_grad_partial_chunks,
            input_grad_positions_per_block, int(use_half_input_grad), int(use_half_linear),
            C.byref(profile) if profile is not None else None, C.cast(cb, C.c_void_p) if cb is not None else None, None,
            _stream(stream), input_grad_position_tile))

    def debug_gemm(self, a, lda, a_mn_major, b, ldb, b_mn_major, d, m, n, k, splits=1, partial=None, stream=None) -> int:
        return int(self._lib.mgt_debug_gemm(self.handle, _ptr(a), lda, int(a_mn_major), _ptr(b), ldb, int(b_mn_major), _ptr(d),
                                            m, n, k, splits, _ptr(partial), _stream(stream)))


def validate_adamw_kernel_config(config: AdamWKernelConfig) -> int:
    cfg = config.c()
    return int(_lib.load().mgt_validate_adamw_config(C.byref(cfg)))


def launch_adamw_kernel(config, device_weights, device_grad, device_m, device_v, stream=None) -> int:
    cfg = config.c()
    return int(_lib.load().mgt_launch_adamw(C.byref(cfg), _ptr(device_weights), _ptr(device_grad), _ptr(device_m),
                                            _ptr(device_v), _stream(stream)))


def launch_adamw_kernel_with_half_mirror(config, device_weights, device_weights_half, device_grad, device_m, device_v,
                                         stream=None) -> int:
    cfg = config.c()
    return int(_lib.load().mgt_launch_adamw_with_half_mirror(C.byref(cfg), _ptr(device_weights), _ptr(device_weights_half),
                                                             _ptr(device_grad), _ptr(device_m), _ptr(device_v), _stream(stream)))


def launch_float_to_half(device_values, count, device_half, stream=None) -> int:
    return int(_lib.load().mgt_launch_float_to_half(_ptr(device_values), count, _ptr(device_half), _stream(stream)))
