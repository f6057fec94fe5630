"""The reference's UNMODIFIED ti_torch.py on the GPU, its four extension modules served by niti_b200/compat.

The reference's TiConv2d / TiLinear / TiMaxpool2d / TiReLU forward and backward (their own Python: transposes, pads,
act_calc / err_calc / grad_calc in torch, weight_update) run on cuda:0 and call cutlassconv_cuda, int8mm_cuda,
int8pool_cuda and int8conv_cuda from niti_b200/compat, i.e. this library's kernels through the C ABI.  The results
must equal tests/golden/layers.npz, which the same Python produced on the CPU over exact integer stand-ins.
Only two shims are kept from the CPU harness: torch-1.7 truncating ``//`` and injected random words."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from oracle import make_ref, ref_harness  # noqa: E402

if not make_ref.available():
    pytest.skip("oracle/_ref is absent (python -m oracle.make_ref <checkout of the reference>)", allow_module_level=True)

import niti_b200.compat as compat  # noqa: E402

DEV = "cuda:0"


def t8(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


@pytest.fixture(scope="module")
def H():
    torch.cuda.set_device(0)
    return ref_harness.load(device="cuda", extension_dir=compat.path())


def test_reference_layers_on_the_b200_kernels(H, golden_dir):
    g = np.load(os.path.join(golden_dir, "layers.npz"))
    T = H.ti_torch
    N, Hh, W, C, K = 4, 8, 8, 16, 32
    with H.active(grad_bitwidth=5):
        conv = T.TiConv2d(C, K)
        conv.weight, conv.weight_exp = t8(g["w"]), torch.tensor(-9.0)
        y, ye = conv.forward((t8(g["x"]), torch.tensor(-5.0)))
        e, ee = conv.backward((t8(g["err"]), 0))
        assert np.array_equal(y.cpu().numpy(), g["conv_y"]) and int(ye) == g["conv_y_exp"]
        assert np.array_equal(e.cpu().numpy(), g["conv_e"]) and int(ee) == g["conv_e_exp"]
        assert np.array_equal(conv.grad_int32acc.cpu().numpy().astype(np.int32), g["conv_g32"])
        assert np.array_equal(conv.weight.cpu().numpy(), g["conv_w_new"])
        # first layer: conv2d_weight_int8 -> int8conv_cuda.group_conv
        c1 = T.TiConv2d(3, K, first_layer=True)
        c1.weight, c1.weight_exp = t8(g["w3"]), torch.tensor(-8.0)
        y, ye = c1.forward((t8(g["x3"]), torch.tensor(-6.0)))
        c1.backward((t8(g["err"]), 0))
        assert np.array_equal(y.cpu().numpy(), g["conv1_y"]) and int(ye) == g["conv1_y_exp"]
        assert np.array_equal(c1.grad_int32acc.cpu().numpy().astype(np.int32), g["conv1_g32"])
        assert np.array_equal(c1.weight.cpu().numpy(), g["conv1_w_new"])
        lin = T.TiLinear(256, 10)
        lin.weight, lin.weight_exp = t8(g["lin_w"]), torch.tensor(-9.0)
        y, ye = lin.forward((t8(g["lin_a"]), torch.tensor(-3.0)))
        e, ee = lin.backward((t8(g["lin_err"]), 0))
        assert np.array_equal(y.cpu().numpy(), g["lin_y"]) and int(ye) == g["lin_y_exp"]
        assert np.array_equal(e.cpu().numpy(), g["lin_e"]) and int(ee) == g["lin_e_exp"]
        assert np.array_equal(lin.grad_int32acc.cpu().numpy().astype(np.int32), g["lin_g32"])
        assert np.array_equal(lin.weight.cpu().numpy(), g["lin_w_new"])
        pool = T.TiMaxpool2d(2, 2)
        y, _ = pool.forward((t8(g["pool_x"]), 0))
        e, _ = pool.backward((t8(g["pool_dy"]), 0))
        assert np.array_equal(y.cpu().numpy(), g["pool_y"]) and np.array_equal(e.cpu().numpy(), g["pool_dx"])


def test_weight_gradient_in_its_conv_disguise_at_a_tensor_core_size(H):
    """ti_torch.py:429-432 at a size the tcgen05 weight-gradient kernel takes (batch and channels multiples of 16): the
    shim recognises the image-sized filters and must agree with the generic forward kernel on the same call."""
    from niti_b200 import ops
    from oracle import niti_oracle as O
    rng = np.random.default_rng(3)
    x = rng.integers(-127, 128, size=(16, 8, 8, 32)).astype(np.int8)
    err = rng.integers(-127, 128, size=(16, 8, 8, 48)).astype(np.int8)
    with H.active():
        got = H.ti_torch.conv2d_int8(t8(x).transpose(0, 3).contiguous(), t8(err).transpose(0, 3).contiguous(), 1, 1).transpose(0, 3).contiguous()
    assert np.array_equal(got.cpu().numpy(), O.conv_wgrad(x, err, 3, 3, 1).astype(np.int32))
    direct = ops.conv_fprop_acc(t8(x).transpose(0, 3).contiguous(), t8(err).transpose(0, 3).contiguous(), 1, 1)[0]
    assert torch.equal(direct.transpose(0, 3).contiguous(), got)


def test_extension_contracts():
    import sys
    sys.path.insert(0, compat.path())
    try:
        import cutlassconv_cuda
        import int8mm_cuda
    finally:
        sys.path.remove(compat.path())
    a = torch.zeros((4, 8), dtype=torch.int8)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        int8mm_cuda.int8_mm(a, a.t())
    b = torch.zeros((4, 8, 8, 32), dtype=torch.int8, device=DEV)
    with pytest.raises(RuntimeError, match="contiguous"):
        cutlassconv_cuda.sp_conv(b.transpose(1, 2), torch.zeros((16, 3, 3, 32), dtype=torch.int8, device=DEV), 1, 1)
    for name in ("cutlassconv_cuda", "int8mm_cuda", "int8pool_cuda", "int8conv_cuda"):
        sys.modules.pop(name, None)
