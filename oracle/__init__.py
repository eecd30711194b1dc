"""CPU oracle for the HyC-LoRA activation-compression hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory; it exists so that the CUDA kernels can be checked against a plain
CPU restatement of the reference algorithm.  Only the test-suite, the smoke
check and the CPU-baseline leg of the benchmark may import it.

Every function cites the reference file:line it restates (paths relative to the
HyC-LoRA-release project root).

Pinning status
--------------
* REF mode (per-channel scale, interleaved 32-column pack, channel outliers,
  zero-point variant, softmax threshold prune, fused LoRA-SiLU-Hadamard
  forward/backward): pinned by fixtures under ``tests/golden`` that were
  produced by executing the reference's own source (its pure-PyTorch
  statistics functions as-is, and its Triton kernels under the Triton CPU
  interpreter); see ``tests/golden/make_golden.py``.
* GROUP mode (64-wide groups with scale + zero-point) and TOPK mode (per-row
  top-k + grouped remainder) have NO reference implementation.  Their
  definition lives here and is the specification for the CUDA side:
  **parity unpinned** for those two modes.
"""
from .quant import *          # noqa: F401,F403
from .group import *          # noqa: F401,F403
from .softmax_map import *    # noqa: F401,F403
from .fused_mlp import *      # noqa: F401,F403
