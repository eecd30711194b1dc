"""Operator layer: same module and function names as the reference's ``operators`` package
for the functions on the activation-compression path."""
from . import compress_function  # noqa: F401
from . import rmsnorm_kernels  # noqa: F401
from . import softmax_kernels  # noqa: F401
from . import rope_kernels  # noqa: F401
from . import triton_fuse_lora_silu_hadamard_forward_kernels  # noqa: F401
from . import triton_fuse_lora_silu_hadamard_backward_kernels  # noqa: F401
