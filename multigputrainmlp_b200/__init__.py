"""B200-native (sm_100a) training step of the residual-MLP puzzle trainer.

The product is the native library ``_native/libmgt_b200.so`` (C ABI in ``include/mgt_b200.h``) and
the ``mgt_native_train`` binary. This package is the thin host-side mirror of the reference's
launch API (same names, argument meaning and status codes) over that C ABI, used by the tests
and the benchmark. PyTorch appears only as the owner of device memory and streams.
"""
from .api import (  # noqa: F401
    STATUS,
    AdamWKernelConfig,
    BackwardProfile,
    CudaMlpShape,
    Engine,
    MgtError,
    RandomWalkKernelConfig,
    launch_adamw_kernel,
    launch_adamw_kernel_with_half_mirror,
    launch_float_to_half,
    launch_random_walk_kernel,
    load_puzzle_definition,
    mlp_loss_grad_workspace_floats,
    bn_param_count,
    fold_batch_norm,
    launch_expand_scalar_labels,
    status_name,
    validate_adamw_kernel_config,
    validate_cuda_mlp_shape,
    validate_random_walk_kernel_config,
)
