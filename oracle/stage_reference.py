"""Stage the reference's pure-PyTorch compress path for the timed CPU baseline (test infrastructure).

    python oracle/stage_reference.py [/path/to/HyC-LoRA-release]

The reference is a tree of Python scripts without a package or a build step, so "building" its CPU implementation
of the path means placing the files that implement it -- ``operators/compress_function.py`` and the module it
imports, ``operators/compress_function_kernel.py`` -- UNCHANGED under ``oracle/_ref/operators/``.  That folder is
kept out of version control (it is an output, like a compiled library); the benchmark's reference arm and its
``cpu_baseline`` leg import ``get_statistics_softmax``, ``compression_softmax`` and ``decompression_softmax``
(compress_function.py:30-32, 309-317) from there and time them on the host cores.  The two fused-kernel modules
travel along so that the benchmark can also time the reference's own Triton kernels on the GPU it runs on (a
reported comparison line).  Nothing else may use the staged files.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
FILES = ("compress_function.py", "compress_function_kernel.py",
         "triton_fuse_lora_silu_hadamard_forward_kernels.py", "triton_fuse_lora_silu_hadamard_backward_kernels.py")


def stage(reference_root=None):
    """-> the staged folder, or None when no checkout is reachable."""
    ref = reference_root or os.environ.get("HYC_REFERENCE") or os.path.join(os.sep, "root", "reference")
    src = os.path.join(ref, "operators")
    if not all(os.path.isfile(os.path.join(src, f)) for f in FILES):
        return None
    dst = os.path.join(HERE, "_ref", "operators")
    os.makedirs(dst, exist_ok=True)
    for f in FILES:
        shutil.copyfile(os.path.join(src, f), os.path.join(dst, f))
    return os.path.dirname(dst)


if __name__ == "__main__":
    out = stage(sys.argv[1] if len(sys.argv) > 1 else None)
    print(out or "no reference checkout found")
