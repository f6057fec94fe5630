"""weight_quant / UniformWeights (setup only; ti_torch.py:77-85, 334-339) against the reference's own functions under
one seed.  Runs on the CPU: both sides are plain torch host code; the reference's Python comes from oracle/_ref."""
import numpy as np
import pytest
import torch

from oracle import make_ref, ref_harness

if not (make_ref.available() or ref_harness.default_ref_dir()):
    pytest.skip("the reference's Python is not available (python -m oracle.make_ref <checkout>)", allow_module_level=True)


@pytest.fixture(scope="module")
def ours():
    from niti_b200 import ti_torch
    saved = ti_torch.GPU
    ti_torch.GPU = "cpu"
    yield ti_torch
    ti_torch.GPU = saved


@pytest.mark.parametrize("size", [(128, 3, 3, 3), (64, 3, 3, 32), (10, 512), (7, 33)])
def test_uniform_weights_match_the_reference(ours, size):
    H = ref_harness.load()
    with H.active():
        torch.manual_seed(1234)
        want_w, want_e = H.ti_torch.UniformWeights(torch.Size(size))
        torch.manual_seed(99)
        want_nw, want_ne = H.ti_torch.NormalWeight(torch.Size(size))
    torch.manual_seed(1234)
    got_w, got_e = ours.UniformWeights(torch.Size(size))
    torch.manual_seed(99)
    got_nw, got_ne = ours.NormalWeight(torch.Size(size))
    assert got_w.dtype == torch.int8 and torch.equal(got_w, want_w) and int(got_e) == int(want_e)
    assert torch.equal(got_nw, want_nw) and int(got_ne) == int(want_ne)


def test_weight_quant_edge_values(ours):
    H = ref_harness.load()
    for vals in ([0.5, -0.25, 0.125], [1.0, -1.0], [3e-3, -7e-3, 6.9e-3], [127.0, 1.0]):
        x = torch.tensor(vals, dtype=torch.float32)
        with H.active():
            want_w, want_e = H.ti_torch.weight_quant(x.clone())
        got_w, got_e = ours.weight_quant(x.clone())
        assert torch.equal(got_w, want_w) and int(got_e) == int(want_e), vals
