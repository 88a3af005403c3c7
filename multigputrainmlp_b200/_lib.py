"""Loads the native library. There is no CPU or PyTorch fallback: if libmgt_b200.so is missing
or cannot be loaded, importing the API fails loudly."""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "_native", "libmgt_b200.so")

_lib = None


class NativeLibraryMissing(RuntimeError):
    pass


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise NativeLibraryMissing(
                f"{LIB_PATH} not found. Build it with `python -m multigputrainmlp_b200.build` "
                "(nvcc, sm_100a). This package has no CPU fallback.")
        _lib = C.CDLL(LIB_PATH)
        _declare(_lib)
    return _lib


def _declare(lib: C.CDLL) -> None:
    u32, u64, i32, f32, vp = C.c_uint32, C.c_uint64, C.c_int32, C.c_float, C.c_void_p
    lib.mgt_status_name.restype = C.c_char_p
    lib.mgt_status_name.argtypes = [i32]
    lib.mgt_version.restype = C.c_char_p
    lib.mgt_validate_random_walk_config.argtypes = [vp]
    lib.mgt_launch_random_walk.argtypes = [vp, u64, u64, u64, u32, vp, vp, vp, vp, vp, vp]
    lib.mgt_launch_expand_scalar_labels.argtypes = [vp, u32, u32, vp, vp]
    lib.mgt_validate_mlp_shape.argtypes = [vp]
    lib.mgt_mlp_param_count.restype = u64
    lib.mgt_mlp_param_count.argtypes = [vp]
    lib.mgt_engine_create.argtypes = [i32, C.POINTER(vp)]
    lib.mgt_engine_destroy.argtypes = [vp]
    lib.mgt_engine_check.argtypes = [vp, vp, C.POINTER(i32)]
    lib.mgt_engine_launch_count.restype = u64
    lib.mgt_engine_launch_count.argtypes = [vp]
    lib.mgt_mlp_loss_grad_workspace_floats.restype = u64
    lib.mgt_mlp_loss_grad_workspace_floats.argtypes = [vp, u32, u32, i32, i32]
    lib.mgt_launch_mlp_loss_grad.argtypes = [vp, vp, vp, vp, vp, vp, u32, vp, vp, vp, u64, u32, u32, i32, i32, vp, vp, vp, vp, u32]
    lib.mgt_validate_adamw_config.argtypes = [vp]
    lib.mgt_launch_adamw.argtypes = [vp, vp, vp, vp, vp, vp]
    lib.mgt_launch_adamw_with_half_mirror.argtypes = [vp, vp, vp, vp, vp, vp, vp]
    lib.mgt_launch_float_to_half.argtypes = [vp, u64, vp, vp]
    lib.mgt_debug_gemm.argtypes = [vp, vp, u32, i32, vp, u32, i32, vp, u32, u32, u32, u32, vp, vp]
