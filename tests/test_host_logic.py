"""Host-side logic that needs no device: the calibration running mean."""
import torch

from hyc_lora_release_b200.operators.compress_function import (
    head_to_hidden_shape, hidden_to_head_shape, update_dict)


def test_update_dict_matches_reference(golden):
    d = golden["update_dict"]
    old = {"outlier_channel_index": None, "scale": None}
    for it, new in enumerate(d["history"]):
        old = update_dict(old, {k: v.clone() for k, v in new.items()}, it)
    assert torch.equal(old["outlier_channel_index"], d["final"]["outlier_channel_index"])
    assert torch.equal(old["scale"], d["final"]["scale"])


def test_head_hidden_roundtrip():
    x = torch.arange(2 * 3 * 8, dtype=torch.float32).reshape(2, 3, 8)
    assert torch.equal(head_to_hidden_shape(hidden_to_head_shape(x, 4)), x)
