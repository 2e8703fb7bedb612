"""The convolution oracle: the reference's one vector (helium/tests/tensor_ops.rs:379-397), torch as a second
opinion on forward and both gradients for every geometry the model of resnet-train uses, and the planner's
geometry / refusals (no GPU needed for planning)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import helium_b200 as hb
from helium_b200 import ir
from helpers import O


def test_reference_conv_simple_vector():
    x = np.array([1.0, 2.0]).reshape(1, 1, 1, 2)
    w = np.array([10.0, 20.0, 30.0, 40.0]).reshape(2, 1, 1, 2)
    y = O.conv2d(x, w)
    assert y.shape == (1, 1, 1, 2)
    assert np.array_equal(y.reshape(-1), [50.0, 110.0])


GEOMS = [  # (H, W, C, K, R, S, stride): every layer geometry of resnet-train/src/model.rs:9-83,112-247, shrunk in H, W
    (20, 20, 3, 8, 7, 7, 2), (12, 12, 8, 16, 1, 1, 2), (12, 12, 8, 16, 3, 3, 2), (6, 6, 16, 16, 3, 3, 1), (7, 7, 16, 24, 1, 1, 1),
    (9, 11, 8, 8, 3, 3, 1), (10, 14, 8, 8, 3, 3, 2),
]


@pytest.mark.parametrize("geom", GEOMS)
def test_conv_oracle_matches_torch(geom):
    H, W, C, K, R, S, st = geom
    r = np.random.default_rng(5)
    x = r.standard_normal((2, H, W, C)); w = r.standard_normal((K, R, S, C))
    (P, Q), pad = O.conv_geometry((H, W), (R, S), (st, st))
    tx = torch.from_numpy(x).permute(0, 3, 1, 2).requires_grad_(True)
    tw = torch.from_numpy(w).permute(0, 3, 1, 2).requires_grad_(True)
    ty = F.conv2d(tx, tw, stride=st, padding=tuple(pad))[:, :, :P, :Q]     # torch keeps a last partial window the reference drops
    y = O.conv2d(x, w, (st, st))
    assert y.shape == (2, P, Q, K)
    assert np.allclose(y, ty.detach().permute(0, 2, 3, 1).numpy(), rtol=1e-10, atol=1e-10)
    dy = r.standard_normal(y.shape)
    ty.backward(torch.from_numpy(dy).permute(0, 3, 1, 2))
    assert np.allclose(O.conv2d_backward_data(dy, w, (H, W), (st, st)), tx.grad.permute(0, 2, 3, 1).numpy(), rtol=1e-10, atol=1e-10)
    assert np.allclose(O.conv2d_backward_filter(dy, x, (R, S), (st, st)), tw.grad.permute(0, 2, 3, 1).numpy(), rtol=1e-10, atol=1e-10)


def test_conv_planning_without_a_device():
    p = hb.Plan.conv2d(None, "fwd", batch=128, in_hw=(56, 56), in_channels=64, out_channels=64, kernel=(3, 3), stride=1)
    assert "implicit GEMM" in p.description and "[128,56,56,64] -> [128,56,56,64]" in p.description
    assert p.out_shapes[0] == (128, 56, 56, 64)
    p = hb.Plan.conv2d(None, "fwd", batch=128, in_hw=(56, 56), in_channels=64, out_channels=128, kernel=(3, 3), stride=2, stats=True)
    assert p.out_shapes == [(128, 28, 28, 128), (2, 128)] and p.workspace_bytes > 0
    p = hb.Plan.conv2d(None, "bwd_data", batch=4, in_hw=(56, 56), in_channels=64, out_channels=128, kernel=(3, 3), stride=2)
    assert "4 passes" in p.description and p.out_shapes[0] == (4, 56, 56, 64)
    p = hb.Plan.conv2d(None, "bwd_filter", batch=4, in_hw=(56, 56), in_channels=64, out_channels=128, kernel=(3, 3), stride=2)
    assert p.out_shapes[0] == (128, 3, 3, 64) and p.workspace_bytes >= 128 * 9 * 64 * 4
    # a 1x1 stride-2 data gradient leaves three of four pixels untouched: zero-filled, no fusion
    with pytest.raises(hb.HeliumError, match="zero-filled"):
        hb.Plan.conv2d(None, "bwd_data", batch=4, in_hw=(56, 56), in_channels=64, out_channels=128, kernel=(1, 1), stride=2, resid=True)
    with pytest.raises(hb.HeliumError, match="multiples of 8"):
        hb.Plan.conv2d(None, "fwd", batch=4, in_hw=(224, 224), in_channels=3, out_channels=32, kernel=(7, 7), stride=2)
    with pytest.raises(hb.HeliumError, match="dilation"):
        hb.Plan.conv2d(None, "fwd", batch=4, in_hw=(8, 8), in_channels=8, out_channels=8, kernel=(3, 3), dilation=2)
