"""ctypes bindings for the CPU oracle (oracle.cpp) and for the reference's own CPU library
behind the C shim (ref_shim.cpp). Test infrastructure only."""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
STATE_STORAGE_LEN = 80
MAX_MOVES = 18

WALK_META_DTYPE = np.dtype([("depth", "<u4"), ("last_move", "<u4"), ("rng_counter", "<u8")])


@dataclass(frozen=True)
class MlpShape:
    state_len: int
    state_value_pad: int
    hd1: int
    hd2: int
    residual_blocks: int
    output_dim: int = 1

    def as_array(self):
        return (C.c_uint32 * 6)(self.state_len, self.state_value_pad, self.hd1, self.hd2,
                                self.residual_blocks, self.output_dim)

    @property
    def param_count(self) -> int:
        block = 2 * (self.hd2 * self.hd2 + self.hd2)
        return (self.state_len * self.state_value_pad * self.hd1 + self.hd1 + self.hd1 * self.hd2 + self.hd2
                + self.residual_blocks * block + self.hd2 * self.output_dim + self.output_dim)


def _p(a, ctype=C.c_void_p):
    return a.ctypes.data_as(ctype)


def build_oracle(with_reference: bool = True) -> None:
    """Compile liboracle.so and, if the reference checkout exists, libmgt_ref.so."""
    target = "all" if with_reference else "oracle"
    subprocess.run(["make", "-s", "-C", HERE, target], check=True)


class Oracle:
    """The restatement in oracle.cpp."""

    def __init__(self, lib):
        self.lib = lib
        lib.orc_mix64.restype = C.c_uint64
        lib.orc_mix64.argtypes = [C.c_uint64]
        lib.orc_mlp_param_count.restype = C.c_uint64
        lib.orc_half_to_float.restype = C.c_float
        lib.orc_half_to_float.argtypes = [C.c_uint16]
        lib.orc_float_to_half_rn.restype = C.c_uint16
        lib.orc_float_to_half_rn.argtypes = [C.c_float]
        lib.orc_export_float_to_fp16.restype = C.c_uint16
        lib.orc_export_float_to_fp16.argtypes = [C.c_float]

    def mix64(self, x: int) -> int:
        return int(self.lib.orc_mix64(C.c_uint64(x & (2**64 - 1))))

    def cyclic_puzzle(self, state_len=72, move_count=18):
        moves = np.zeros((MAX_MOVES, STATE_STORAGE_LEN), np.uint8)
        target = np.zeros(STATE_STORAGE_LEN, np.uint8)
        self.lib.orc_build_cyclic_puzzle(C.c_uint32(state_len), C.c_uint32(move_count), C.c_uint32(MAX_MOVES),
                                         _p(moves), _p(target))
        return moves, target

    def random_walks(self, moves, target, *, seed, epoch, step, rank, k_min, k_max, samples,
                     move_count=18, state_len=72, state_storage_len=80):
        states = np.zeros((samples, STATE_STORAGE_LEN), np.uint8)
        labels = np.zeros(samples, np.float32)
        meta = np.zeros(samples, WALK_META_DTYPE)
        st = self.lib.orc_random_walks(_p(np.ascontiguousarray(moves)), _p(np.ascontiguousarray(target)),
                                       C.c_uint32(move_count), C.c_uint32(state_len), C.c_uint32(state_storage_len),
                                       C.c_uint64(seed), C.c_uint64(epoch), C.c_uint64(step), C.c_uint32(rank),
                                       C.c_uint32(k_min), C.c_uint32(k_max), C.c_uint32(samples),
                                       _p(states), _p(labels), _p(meta))
        return st, states, labels, meta

    def param_count(self, shape: MlpShape) -> int:
        return int(self.lib.orc_mlp_param_count(shape.as_array()))

    def forward(self, shape, weights, states):
        b = states.shape[0]
        out = np.zeros((b, shape.output_dim), np.float32)
        st = self.lib.orc_mlp_forward(shape.as_array(), _p(weights), _p(states), C.c_uint32(b), _p(out))
        return st, out

    def loss_grad(self, shape, weights, states, labels):
        b = states.shape[0]
        loss = C.c_float(0)
        grad = np.zeros(shape.param_count, np.float32)
        st = self.lib.orc_mlp_loss_grad(shape.as_array(), _p(weights), _p(states), _p(labels), C.c_uint32(b),
                                        C.byref(loss), _p(grad))
        return st, float(loss.value), grad

    def loss_grad_mixed(self, shape, weights, states, labels, half_linear=True, half_input_grad=True):
        b = states.shape[0]
        loss = C.c_float(0)
        grad = np.zeros(shape.param_count, np.float32)
        st = self.lib.orc_mlp_loss_grad_mixed(shape.as_array(), _p(weights), _p(states), _p(labels), C.c_uint32(b),
                                              C.c_int(int(half_linear)), C.c_int(int(half_input_grad)),
                                              C.byref(loss), _p(grad))
        return st, float(loss.value), grad

    def bn_param_count(self, shape) -> int:
        self.lib.orc_bn_param_count.restype = C.c_uint64
        return int(self.lib.orc_bn_param_count(shape.as_array()))

    def loss_grad_ex(self, shape, weights, states, labels, *, half_linear=True, half_input_grad=True, bf16=False,
                     cross_entropy=False, batch_norm=False, bn_eps=1e-5):
        """orc_mlp_loss_grad_ex: the options the reference does not have (bfloat16 operands, cross-entropy on depth - 1,
        batch normalisation). With batch_norm the weights carry gamma/beta behind the reference's parameters.
        Returns (status, loss, grad, stats) with stats[layer][0|1][hd2] = batch mean / variance (None without batch norm)."""
        class Opt(C.Structure):
            _fields_ = [("half_linear", C.c_int), ("half_input_grad", C.c_int), ("operand_format", C.c_int), ("loss_kind", C.c_int),
                        ("batch_norm", C.c_int), ("bn_eps", C.c_float)]
        opt = Opt(int(half_linear), int(half_input_grad), int(bf16), int(cross_entropy), int(batch_norm), float(bn_eps))
        b = states.shape[0]
        total = shape.param_count + (self.bn_param_count(shape) if batch_norm else 0)
        assert weights.size == total, (weights.size, total)
        loss = C.c_float(0)
        grad = np.zeros(total, np.float32)
        stats = np.zeros((shape.residual_blocks + 1, 2, shape.hd2), np.float32) if batch_norm else None
        st = self.lib.orc_mlp_loss_grad_ex(shape.as_array(), _p(weights), _p(states), _p(np.ascontiguousarray(labels, np.float32)), C.c_uint32(b),
                                           C.byref(opt), C.byref(loss), _p(grad), _p(stats) if stats is not None else None)
        return st, float(loss.value), grad, stats

    def float_to_bf16(self, a):
        a = np.asarray(a, np.float32).ravel()
        return np.array([self.lib.orc_float_to_bf16_rn(C.c_float(float(x))) for x in a], np.uint16)

    def adamw(self, w, g, m, v, *, step, lr, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.0, half_mirror=None):
        hp = _p(half_mirror) if half_mirror is not None else None
        return self.lib.orc_adamw_step(_p(w), _p(g), _p(m), _p(v), C.c_uint64(w.size), C.c_uint64(step),
                                       C.c_float(lr), C.c_float(beta1), C.c_float(beta2), C.c_float(eps),
                                       C.c_float(wd), hp)

    def float_to_half(self, a):
        a = np.asarray(a, np.float32).ravel()
        return np.array([self.lib.orc_float_to_half_rn(C.c_float(float(x))) for x in a], np.uint16)

    def export_fp16(self, a):
        a = np.asarray(a, np.float32).ravel()
        return np.array([self.lib.orc_export_float_to_fp16(C.c_float(float(x))) for x in a], np.uint16)

    def allreduce_average(self, grads):
        world = len(grads)
        n = grads[0].size
        out = np.zeros(n, np.float32)
        arr = (C.c_void_p * world)(*[g.ctypes.data for g in grads])
        self.lib.orc_allreduce_average(arr, C.c_uint32(world), C.c_uint64(n), _p(out))
        return out


class Reference:
    """The reference's own CPU code, compiled from its sources (oracle/_ref/libmgt_ref.so)."""

    def __init__(self, lib):
        self.lib = lib
        lib.ref_param_count.restype = C.c_uint64

    def random_walks(self, moves, target, *, seed, epoch, step, rank, k_min, k_max, samples):
        states = np.zeros((samples, STATE_STORAGE_LEN), np.uint8)
        labels = np.zeros(samples, np.float32)
        meta = np.zeros(samples, WALK_META_DTYPE)
        st = self.lib.ref_random_walks(_p(np.ascontiguousarray(moves)), _p(np.ascontiguousarray(target)),
                                       C.c_uint64(seed), C.c_uint64(epoch), C.c_uint64(step), C.c_uint32(rank),
                                       C.c_uint32(k_min), C.c_uint32(k_max), C.c_uint32(samples),
                                       _p(states), _p(labels), _p(meta))
        return st, states, labels, meta

    def load_puzzle(self, group_json, target_bin):
        """LoadPuzzleDefinition of the reference: (status, moves[18][80], target[80])."""
        moves = np.zeros((MAX_MOVES, STATE_STORAGE_LEN), np.uint8)
        target = np.zeros(STATE_STORAGE_LEN, np.uint8)
        st = int(self.lib.ref_load_puzzle(str(group_json).encode(), str(target_bin).encode(), _p(moves), _p(target)))
        return st, moves, target

    def param_count(self, shape):
        return int(self.lib.ref_param_count(shape.as_array()))

    def forward(self, shape, weights, states):
        b = states.shape[0]
        out = np.zeros((b, shape.output_dim), np.float32)
        st = self.lib.ref_mlp_forward(shape.as_array(), _p(weights), _p(states), C.c_uint32(b), _p(out))
        return st, out

    def loss_grad(self, shape, weights, states, labels):
        b = states.shape[0]
        loss = C.c_float(0)
        grad = np.zeros(shape.param_count, np.float32)
        st = self.lib.ref_mlp_loss_grad(shape.as_array(), _p(weights), _p(states), _p(labels), C.c_uint32(b),
                                        C.byref(loss), _p(grad))
        return st, float(loss.value), grad

    def adamw(self, w, g, m, v, *, step, lr, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.0):
        return self.lib.ref_adamw(_p(w), _p(g), _p(m), _p(v), C.c_uint64(w.size), C.c_uint64(step), C.c_float(lr),
                                  C.c_float(beta1), C.c_float(beta2), C.c_float(eps), C.c_float(wd))

    def plan_numbers(self, *, state_len=72, value_count=72, move_count=18, state_alignment=16, hd1=2556, hd2=218,
                     nrd=16, output_dim=1, hidden_alignment=8, batch=100000, bucket_bytes=4 << 20, world=1):
        out = (C.c_uint64 * 10)()
        st = self.lib.ref_plan_numbers(C.c_uint32(state_len), C.c_uint32(value_count), C.c_uint32(move_count),
                                       C.c_uint32(state_alignment), C.c_uint32(hd1), C.c_uint32(hd2), C.c_uint32(nrd),
                                       C.c_uint32(output_dim), C.c_uint32(hidden_alignment), C.c_uint32(batch),
                                       C.c_uint64(bucket_bytes), C.c_uint32(world), out)
        keys = ["padded_state_dim", "physical_hd1", "physical_hd2", "blocks", "linear_ops", "gradient_buckets",
                "total_params", "total_bytes", "total_rank_bytes", "training_scratch_bytes"]
        return st, dict(zip(keys, [int(x) for x in out]))

    def plan_linear_op(self, index, *, state_len=72, value_count=72, hd1=2556, hd2=218, nrd=16, output_dim=1,
                       batch=100000):
        out = (C.c_uint32 * 14)()
        st = self.lib.ref_plan_linear_op(C.c_uint32(state_len), C.c_uint32(value_count), C.c_uint32(hd1),
                                         C.c_uint32(hd2), C.c_uint32(nrd), C.c_uint32(output_dim), C.c_uint32(batch),
                                         C.c_uint32(index), out)
        return st, [int(x) for x in out]


def load_oracle(build: bool = True) -> Oracle:
    path = os.path.join(HERE, "_build", "liboracle.so")
    if build and not os.path.exists(path):
        build_oracle(with_reference=False)
    return Oracle(C.CDLL(path))


def load_reference():
    """Returns the reference binding, or None when oracle/_ref was never built."""
    path = os.path.join(HERE, "_ref", "libmgt_ref.so")
    if not os.path.exists(path):
        return None
    return Reference(C.CDLL(path))
