"""Generate tests/golden/ref_layer_golden.pt by RUNNING THE REFERENCE'S OWN FUSED DECODER LAYER on a CUDA GPU.

    python tests/golden/make_layer_golden.py /path/to/HyC-LoRA-release [output.pt]

Needs a GPU and the HyC-LoRA-release checkout; the fixture it writes is committed, so the test-suite itself
never needs the checkout.  What runs, unchanged: ``models/llama/fused_llama_layer_intra_inter_full_fuse.py``
(module + autograd function, :29-708) and its Mistral twin, on the cases of ``layer_case.py`` (7 iterations:
5 calibration + 2 with frozen statistics, forward + backward each), in two arms, each in a process of its own:

  triton  the layer imports the reference's own ``operators`` package; its Triton kernels are compiled by the
          installed Triton for the GPU at hand.  One module is NOT the reference's in this arm:
          ``operators.rmsnorm_kernels`` is this package's, because the reference's backward kernel spins on a
          lock without a limit (operators/rmsnorm_kernels.py:103-113), which has no place on a shared GPU; that
          kernel is pinned through the CPU interpreter instead (make_golden.py).  And one call is adapted: the
          layer hands ``triton_fuse_silu_backward`` the LoRA-B factors as transposed views
          (``lora_B.weight.T``, :638-639 of the layer), but that kernel steps through B with
          ``b1_ptrs + i * (BLOCK_SIZE_N // elem_per_position)`` (backward_kernels.py:96-97), which is only right
          for a unit column stride; the forward wrapper makes them contiguous itself ("must keep b1, b2
          contiguous", forward_kernels.py:164-166), the backward wrapper does not, and for q_bit < 8 the
          recomputed gate/up values of every second sub-block then use the wrong columns of B.  This arm passes
          contiguous copies, as the forward wrapper does.
  triton_raw  the same without that adaptation (the reference exactly as it runs): kept for iteration 6 of the
          Llama case, to show what the stride slip costs.
  hyc     ``sys.modules["operators"]`` and its sub-modules are replaced by ``hyc_lora_release_b200.operators``
          before the layer is imported: the reference's layer code then runs on libhyc, operator by operator.
          (``operators.silu_kernels``, which the layer imports and never calls, stays the reference's.)

``bitsandbytes`` is absent here: stub modules give ``dequantize_nf4(w, state) = w``, and the frozen weights are
plain bf16 matrices with ``quant_state = None``.  The fixture holds, per family and arm, y, grad_x and the 14
LoRA gradients of iterations 0 and 6 and the calibrated ``static_value``; inputs and weights are re-created
from seeds by ``layer_case.build``.
"""
import importlib.util
import os
import subprocess
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
for p in (ROOT, HERE):
    if p not in sys.path:
        sys.path.insert(0, p)


def _stub_bitsandbytes():
    bnb = types.ModuleType("bitsandbytes")
    bnbf = types.ModuleType("bitsandbytes.functional")
    bnbnn = types.ModuleType("bitsandbytes.nn")
    bnbmod = types.ModuleType("bitsandbytes.nn.modules")
    bnbf.dequantize_nf4 = lambda w, quant_state=None: w
    bnbmod.Linear4bit = type("Linear4bit", (), {})
    bnbnn.modules = bnbmod
    bnb.nn = bnbnn
    bnb.functional = bnbf
    sys.modules.update({"bitsandbytes": bnb, "bitsandbytes.functional": bnbf, "bitsandbytes.nn": bnbnn,
                        "bitsandbytes.nn.modules": bnbmod})


def _load_by_path(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def run_arm(ref, arm, family, out_path):
    import torch
    import layer_case
    _stub_bitsandbytes()
    sys.path.insert(0, ref)
    import hyc_lora_release_b200.operators as hyc_ops
    if arm in ("triton", "triton_raw"):
        sys.modules["operators.rmsnorm_kernels"] = hyc_ops.rmsnorm_kernels
    else:
        sys.modules["operators"] = hyc_ops
        for name in ("compress_function", "rmsnorm_kernels", "softmax_kernels", "rope_kernels",
                     "triton_fuse_lora_silu_hadamard_forward_kernels", "triton_fuse_lora_silu_hadamard_backward_kernels"):
            sys.modules["operators." + name] = getattr(hyc_ops, name)
        _load_by_path("operators.silu_kernels", os.path.join(ref, "operators", "silu_kernels.py"))
    if family == "llama":
        from models.llama.fused_llama_layer_intra_inter_full_fuse import FusedLlamaLayerIntraInterFullFuse as Layer
    else:
        from models.mistral.fused_mistral_layer_intra_inter_full_fuse import FusedMistralLayerIntraInterFullFuse as Layer
    if arm == "triton":
        mod = sys.modules[Layer.__module__]
        raw_bwd = mod.triton_fuse_silu_backward

        def bwd_contiguous_b(xa1, b1, q1, s1, xa2, b2, q2, s2, grad_o, quantize_bit=8):
            return raw_bwd(xa1, b1.contiguous(), q1, s1, xa2, b2.contiguous(), q2, s2, grad_o, quantize_bit)
        mod.triton_fuse_silu_backward = bwd_contiguous_b
    case = layer_case.build(family)
    layer = Layer()
    layer.set_hyclora_config(types.SimpleNamespace(q_bit=case["q_bit"], **layer_case.CONFIG))
    res = layer_case.run_iterations(layer, case, torch.device("cuda", 0))
    torch.cuda.synchronize()
    import triton
    res["meta"] = dict(arm=arm, family=family, torch=torch.__version__, triton=triton.__version__,
                       gpu=torch.cuda.get_device_name(0))
    torch.save(res, out_path)


def _report(a, b):
    import torch
    a, b = a.float().flatten(), b.float().flatten()
    scale = b.abs().max().clamp(min=1e-30)
    return float((a - b).abs().max() / scale), float(torch.nn.functional.cosine_similarity(a, b, dim=0))


def main():
    ref = os.path.abspath(sys.argv[1])
    assert os.path.isdir(os.path.join(ref, "operators")), "pass the path of the HyC-LoRA-release checkout"
    if len(sys.argv) > 3 and sys.argv[2] == "--arm":
        arm, family, out_path = sys.argv[3], sys.argv[4], sys.argv[5]
        run_arm(ref, arm, family, out_path)
        return
    import torch
    dst = sys.argv[2] if len(sys.argv) > 2 else os.path.join(HERE, "ref_layer_golden.pt")
    out, log = {}, []
    for family in ("llama", "mistral"):
        out[family] = {}
        for arm in ("triton", "hyc") + (("triton_raw",) if family == "llama" else ()):
            tmp = "%s.%s.%s.tmp" % (dst, family, arm)
            r = subprocess.run([sys.executable, os.path.abspath(__file__), ref, "--arm", arm, family, tmp],
                               capture_output=True, text=True)
            if r.returncode != 0:
                out[family][arm] = dict(error=(r.stderr or r.stdout)[-3000:])
                log.append("%s/%s FAILED:\n%s" % (family, arm, out[family][arm]["error"]))
                continue
            out[family][arm] = torch.load(tmp, weights_only=False)
            os.remove(tmp)
        # Mistral and the raw arm: only the steady-state iteration is kept (the fixture stays small)
        for arm in out[family]:
            if family == "mistral" or arm == "triton_raw":
                out[family][arm].pop(0, None)
        t = out[family].get("triton", {})
        for other in ("hyc", "triton_raw"):
            h = out[family].get(other, {})
            for it in (0, 6):
                if it in t and it in h:
                    for k in sorted(t[it]):
                        log.append("%s it %d %-12s %s vs triton: max rel err %.3e cosine %.6f" % ((family, it, k, other) + _report(h[it][k], t[it][k])))
        if "static_value" in t and "static_value" in out[family].get("hyc", {}):
            for k, v in t["static_value"].items():
                for kk, vv in v.items():
                    hv = out[family]["hyc"]["static_value"][k][kk]
                    if vv.dtype == torch.int64:
                        log.append("%s static %s.%s triton %s hyc %s" % (family, k, kk, vv.tolist(), hv.tolist()))
                    else:
                        log.append("%s static %-10s %-6s hyc vs triton: max rel err %.3e cosine %.6f" % ((family, k, kk) + _report(hv, vv)))
    torch.save(out, dst)
    log.append("wrote %s %d bytes" % (dst, os.path.getsize(dst)))
    print("\n".join(log))
    with open(os.path.splitext(dst)[0] + "_report.txt", "w") as f:
        f.write("\n".join(log) + "\n")


if __name__ == "__main__":
    main()
