"""ctypes binding of libhyc.so.  One entry per declaration of include/hyc.h."""
import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libhyc.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        "libhyc.so is not built (%s). Build it with `python hyc_lora_release_b200/build.py`; "
        "there is no fallback implementation." % LIB_PATH)

_cdll = ctypes.CDLL(LIB_PATH)

_p, _i, _l, _f, _z = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_size_t

SIGNATURES = {
    "hyc_strerror": (ctypes.c_char_p, [_i]),
    "hyc_last_cuda_error": (_i, []),
    "hyc_version": (_i, []),
    "hyc_colstats_scale": (_i, [_p, _i, _i, _l, _i, _p, _i, _p, _p, _p]),
    "hyc_channel_norm_topk": (_i, [_p, _i, _i, _l, _i, _p, _p, _p]),
    "hyc_quant_pack": (_i, [_p, _l, _i, _l, _p, _p, _p, _i, _p, _p, _i, _p]),
    "hyc_unpack_dequant": (_i, [_p, _l, _i, _p, _p, _p, _i, _p, _p, _l, _i, _p]),
    "hyc_group_quant_pack": (_i, [_p, _l, _i, _l, _p, _p, _p, _i, _p]),
    "hyc_group_unpack_dequant": (_i, [_p, _l, _i, _p, _p, _p, _l, _i, _p]),
    "hyc_softmax_prune_workspace_bytes": (_z, [_l]),
    "hyc_softmax_prune_count": (_i, [_p, _l, _f, _p, _z, _p]),
    "hyc_softmax_prune_fill": (_i, [_p, _l, _f, _p, _p, _p, _l, _p]),
    "hyc_softmax_prune_restore": (_i, [_p, _p, _l, _p, _l, _p]),
    "hyc_softmax_prune_restore_counted": (_i, [_p, _p, _p, _l, _p, _l, _p]),
    "hyc_softmax_prune_static": (_i, [_p, _l, _f, _p, _p, _l, _p, _p]),
    "hyc_softmax_prune_tiled_directory_bytes": (_z, [_l]),
    "hyc_softmax_prune_tiled": (_i, [_p, _l, _f, _p, _l, _p, _p, _p]),
    "hyc_softmax_prune_tiled_restore": (_i, [_p, _l, _p, _p, _l, _p]),
    "hyc_softmax_topk_compress": (_i, [_p, _l, _i, _i, _p, _p, _p, _p, _p, _i, _p]),
    "hyc_softmax_fwd_topk_save": (_i, [_p, _f, _p, _l, _l, _l, _i, _i, _l, _i, _i, _p, _p, _p, _p, _p, _p, _i, _p]),
    "hyc_softmax_topk_restore": (_i, [_p, _p, _i, _p, _p, _p, _l, _i, _p, _i, _p]),
    "hyc_softmax_topk_restore_bwd": (_i, [_p, _p, _i, _p, _p, _p, _l, _i, _p, _p, _i, _f, _p]),
    "hyc_fused_lora_silu_hadamard_fwd": (_i, [_p] * 11 + [_l, _i, _i, _i, _p]),
    "hyc_fused_lora_silu_hadamard_bwd": (_i, [_p] * 12 + [_l, _i, _i, _i, _p]),
    "hyc_dequant_lora_add": (_i, [_p, _p, _p, _p, _p, _l, _i, _i, _i, _p]),
    "hyc_rmsnorm_fwd": (_i, [_p, _p, _f, _p, _p, _l, _i, _p]),
    "hyc_rmsnorm_bwd": (_i, [_p, _p, _p, _p, _p, _l, _i, _p]),
    "hyc_rmsnorm_fwd_save": (_i, [_p, _p, _f, _l, _i, _p, _p, _i, _p, _p, _p, _p, _p, _p, _i, _p]),
    "hyc_rmsnorm_bwd_packed": (_i, [_p, _p, _p, _p, _i, _p, _p, _p, _p, _p, _l, _i, _i, _p]),
    "hyc_softmax_bwd": (_i, [_p, _p, _p, _l, _i, _f, _p]),
    "hyc_softmax_fwd_scale_mask": (_i, [_p, _f, _p, _l, _l, _l, _i, _i, _p, _l, _i, _p]),
    "hyc_rope": (_i, [_p, _l, _p, _l, _p, _p, _l, _i, _l, _i, _i, _i, _i, _p]),
    "hyc_lora_grad_a_workspace_bytes": (_z, [_i, _i, _i]),
    "hyc_lora_grad_a_dequant": (_i, [_p, _p, _p, _l, _i, _i, _i, _i, _p, _p, _z, _p]),
    "hyc_dequant_nf4": (_i, [_p, _p, _p, _p, _p, _p, _i, _f, _l, _i, _p, _p]),
    "hyc_gemm_bf16_tcgen05": (_i, [_p, _p, _i, _i, _i, _i, _p, _p, _i, _p, _p, _i,
                                   _p, _p, _l, _l, _p, _p, _l, _l, _p, _p, _p, _p]),
    "hyc_mlp_gateup_fwd_tcgen05": (_i, [_p, _p, _p, _i, _i, _i, _p, _p, _l, _l, _p, _p, _l, _l,
                                        _p, _p, _p, _p, _p, _p, _p, _i, _p, _p]),
    "hyc_linear_lora_save_fwd_tcgen05": (_i, [_p, _p, _i, _i, _i, _p, _p, _l, _l, _p, _p, _p, _p, _i, _p, _p]),
    "hyc_mlp_graddown_bwd_tcgen05": (_i, [_p, _p, _i, _i, _i, _p, _p, _i, _p, _p, _l, _l, _p, _p, _l, _l,
                                          _p, _p, _p, _p, _p, _p, _l, _p, _p, _p, _i, _p, _p]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(_cdll, _name)
    _fn.restype = _res
    _fn.argtypes = _args

_pending = threading.local()


class _DeviceGuardedLibrary:
    """The library's entry points launch on the CURRENT device.  Every call site passes ``stream_of(t)``, which
    notes the device of ``t``; the call then runs with that device current, so a tensor on cuda:1 is never paired
    with a launch (or the built-in scratch) of cuda:0."""

    def __getattr__(self, name):
        fn = getattr(_cdll, name)

        def call(*args):
            dev = getattr(_pending, "device", None)      # kept: a stream handle may serve several calls in a row
            if dev is not None and dev != torch.cuda.current_device():
                with torch.cuda.device(dev):
                    return fn(*args)
            return fn(*args)
        call.__name__ = name
        setattr(self, name, call)
        return call


lib = _DeviceGuardedLibrary()


class HycError(RuntimeError):
    pass


def check(code, what):
    if code != 0:
        msg = lib.hyc_strerror(code).decode()
        extra = ""
        if code == -6:
            extra = " [cudaError %d]" % lib.hyc_last_cuda_error()
        raise HycError("%s: %s%s" % (what, msg, extra))


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    if t is None:
        return None
    return ctypes.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)     # the handle without building a Stream object


def stream_of(t):
    """torch's current stream on the device of ``t``; also notes that device for the call that follows."""
    idx = t.device.index
    _pending.device = idx
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(idx))
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def require_cuda(*tensors):
    """All given tensors (None entries skipped) must be CUDA tensors on ONE device."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("this operator runs only on CUDA tensors (sm_100a kernels); there is no CPU path")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError("the tensors of one call live on different devices (%s and %s)" % (dev, t.device))
