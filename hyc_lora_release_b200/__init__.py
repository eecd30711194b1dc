"""B200-native activation-compression hot path of HyC-LoRA.

The compute lives in ``lib/libhyc.so`` (hand-written sm_100a CUDA behind a C ABI, see
``include/hyc.h``).  This package is the thin host side: it mirrors the operator API of the
reference (``operators/compress_function.py`` and friends) and forwards device pointers.
There is no CPU or PyTorch fallback: importing the package without the built library, or
calling an operator with a non-CUDA tensor, raises.
"""
from . import _lib  # noqa: F401  (loads libhyc.so; raises ImportError if it is missing)

__all__ = ["operators", "mlp"]
__version__ = "0.1.0"
