"""The fused decoder layer against the reference's OWN layer code (tests/golden/ref_layer_golden.pt, written by
tests/golden/make_layer_golden.py: models/llama/fused_llama_layer_intra_inter_full_fuse.py and the Mistral twin run
unchanged on a B200, 5 calibration + 2 steady-state iterations, forward + backward).

CPU part: the arms of the fixture against each other (the reference's layer on its own Triton operators vs the
same layer code with this package's operators swapped in) and the CPU oracle's restatement of the layer against
the reference's results.  GPU part (marked gpu): this package's layer module against the same results.

Bounds.  Outputs: max |err| <= 1e-2 * max|ref|, cosine > 0.999.  Gradients: cosine > 0.999; their largest single
deviation is allowed 6e-2 of the tensor's maximum, because they are computed from 4-bit codes of COMPUTED tensors
(projection outputs, the attention output, the gate/up branches): where two implementations' GEMM sums differ in
the last bf16 bit a code flips, and one flipped code moves one element by 1/15 of its channel's range.  The
operator-level tests bound that effect exactly (codes of an emitted tensor are compared bit for bit)."""
import os
import sys
import types

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import layer_case  # noqa: E402

BF16 = torch.bfloat16
GRADS = ["grad_x"] + ["grad_%s%s" % (ab, n) for n in layer_case.PROJ for ab in "ab"]


@pytest.fixture(scope="module")
def fixture():
    return torch.load(os.path.join(HERE, "golden", "ref_layer_golden.pt"), weights_only=False)


def err_cos(a, b):
    a, b = a.float().cpu().flatten(), b.float().cpu().flatten()
    scale = b.abs().max().clamp(min=1e-30)
    return float((a - b).abs().max() / scale), float(torch.nn.functional.cosine_similarity(a, b, dim=0))


def check_record(got, want, what):
    e, c = err_cos(got["y"], want["y"])
    assert e <= 1e-2 and c > 0.999, (what, "y", e, c)
    for k in GRADS:
        e, c = err_cos(got[k], want[k])
        assert c > 0.999 and e <= 6e-2, (what, k, e, c)


def test_operator_swap_matches_the_reference_operators(fixture):
    """INTEGRATION.md's operator swap, executed: the reference's layer code on libhyc gives the reference's results."""
    for fam, its in (("llama", (0, 6)), ("mistral", (6,))):
        t, h = fixture[fam]["triton"], fixture[fam]["hyc"]
        assert "error" not in t and "error" not in h
        for it in its:
            check_record(h[it], t[it], (fam, it))
        for name, entry in t["static_value"].items():
            for key, v in entry.items():
                hv = h["static_value"][name][key]
                if v.dtype == torch.int64:
                    assert torch.equal(v, hv), (fam, name)
                else:
                    e, c = err_cos(hv, v)
                    assert e <= 1e-2 and c > 0.9999, (fam, name, key, e, c)


def test_transposed_lora_b_slip_of_the_reference_is_visible(fixture):
    """The reference's backward wrapper hands its kernel transposed views of the LoRA-B factors, which the kernel's
    pointer arithmetic does not support (see make_layer_golden.py): run exactly as it is, the reference's gradients
    are far from the ones it computes with contiguous factors.  This package follows the contiguous form."""
    t, raw = fixture["llama"]["triton"][6], fixture["llama"]["triton_raw"][6]
    assert err_cos(raw["y"], t["y"])[1] > 0.9999                      # forward untouched
    assert err_cos(raw["grad_adown"], t["grad_adown"])[1] < 0.99      # backward is not
    assert err_cos(raw["grad_x"], t["grad_x"])[1] < 0.999


def _static_for_oracle(sv):
    c = lambda v: v.to(BF16)
    return dict(attention=dict(x_idx=sv["x"]["outlier_channel_index"], x_scale=c(sv["x"]["scale"]),
                               x_norm_1_scale=c(sv["x_norm_1"]["scale"]), q_scale=c(sv["q"]["scale"]),
                               k_scale=c(sv["k"]["scale"]), v_scale=c(sv["v"]["scale"]), o_scale=c(sv["o"]["scale"]),
                               a_threshold=sv["a"]["outlier"].float()),
                mlp=dict(x_medium_idx=sv["x_medium"]["outlier_channel_index"], x_medium_scale=c(sv["x_medium"]["scale"]),
                         gate_scale=c(sv["gate"]["scale"]), up_scale=c(sv["up"]["scale"]),
                         x_norm_2_scale=c(sv["x_norm_2"]["scale"])))


@pytest.mark.parametrize("family,it", [("llama", 0), ("llama", 6), ("mistral", 6)])
def test_oracle_layer_matches_the_reference_layer(fixture, family, it):
    from oracle.attention import ref_layer_backward, ref_layer_forward
    case = layer_case.build(family)
    t = fixture[family]["triton"]
    static = None if it < layer_case.CONFIG["iteration_threshold"] else _static_for_oracle(t["static_value"])
    y, saved = ref_layer_forward(case["xs"][it], case["p"], case["cos"], case["sin"], case["mask"], case["heads"], case["d"],
                                 case["kv"], case["q_bit"], layer_case.CONFIG["layernorm_outlier_ratio"],
                                 layer_case.CONFIG["softmax_outlier_ratio"], map_mode="prune", static=static)
    g = ref_layer_backward(case["grad_y"], saved, case["p"], case["cos"], case["sin"], case["heads"], case["d"], case["kv"],
                           case["q_bit"])
    got = dict(y=y, grad_x=g["grad_x"])
    for n in layer_case.PROJ:           # the oracle keeps [in, r] / [r, out]; the fixture the weights' layout
        got["grad_a" + n] = g["grad_a" + n].t()
        got["grad_b" + n] = g["grad_b" + n].t()
    check_record(got, t[it], (family, it))


@pytest.mark.gpu
@pytest.mark.parametrize("family", ["llama", "mistral"])
def test_layer_module_matches_the_reference_layer(fixture, family):
    """This package's fused layer (norm + saves in one pass, GEMM epilogues that pack the codes, restore fused with its
    consumer) driven exactly like the reference's module, against the reference's results."""
    from hyc_lora_release_b200.layer import FusedLlamaLayerIntraInterFullFuse, FusedMistralLayerIntraInterFullFuse
    case = layer_case.build(family)
    layer = (FusedLlamaLayerIntraInterFullFuse if family == "llama" else FusedMistralLayerIntraInterFullFuse)()
    layer.set_hyclora_config(types.SimpleNamespace(q_bit=case["q_bit"], **layer_case.CONFIG))
    layer.check_kernel_status = True
    res = layer_case.run_iterations(layer, case, torch.device("cuda", 0))
    t = fixture[family]["triton"]
    for it in layer_case.RECORDED:
        if it in t:
            check_record(res[it], t[it], (family, it))
    for name, entry in t["static_value"].items():
        for key, v in entry.items():
            hv = res["static_value"][name][key]
            if v.dtype == torch.int64:
                assert torch.equal(v, hv.cpu()), (family, name)
            else:
                e, c = err_cos(hv, v)
                assert e <= 1e-2 and c > 0.9999, (family, name, key, e, c)
