"""he_reduce_sum_f32_noalloc against the planned reduction (he_plan_pointwise + he_launch with a workspace).

Collected last on purpose: the entry point keeps its partial sums in one array inside the library, so
this file checks that it works both as the first thing a process does and after every other test has
used the device.
"""
import ctypes as C

import numpy as np
import pytest

import helium_b200 as hb
from helium_b200 import ir
from helium_b200._lib import lib
from helpers import O

pytestmark = pytest.mark.gpu

MAX_PARTIALS = 65536      # HE_NOALLOC_MAX_PARTIALS in include/helium_b200.h
TOL = 1e-5                # f32 sums: rel-L2 against the existing entry point and against the f64 oracle


def _noalloc(x_dev, groups, group_size):
    import torch
    out = torch.full((groups,), float("nan"), dtype=torch.float32, device=x_dev.device)
    rc = lib.he_reduce_sum_f32_noalloc(C.c_void_p(x_dev.data_ptr()), C.c_void_p(out.data_ptr()), groups, group_size,
                                       C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.he_last_error_string().decode()
    torch.cuda.synchronize()
    return out.cpu().numpy()


def _planned(ctx, x_dev, groups, group_size):
    import torch
    g = ir.Graph()
    x = g.new_input([groups, group_size], ir.F32)
    g.new_output(g.reduce(ir.RED_SUM, x, 1))
    plan = hb.Plan.pointwise(ctx, g)
    outs = plan.launch([x_dev])
    torch.cuda.synchronize()
    return outs[0].cpu().numpy().reshape(-1), g


@pytest.mark.parametrize("groups,group_size", [
    (1, 1 << 20),        # one group, 256 slices
    (3, 70000),          # ragged last slice
    (64, 5000),          # two slices per group
    (7, 3000),           # one slice: written straight to the output
    (1000, 100),         # short groups
    (16, 4096 * 4096),   # 65536 partials: exactly the capacity
])
def test_matches_planned_reduction_twice(ctx, groups, group_size):
    import torch
    gen = torch.Generator(device="cuda").manual_seed(41)
    x_dev = torch.randn((groups, group_size), dtype=torch.float32, device="cuda", generator=gen) + 0.25
    want, g = _planned(ctx, x_dev, groups, group_size)
    first = _noalloc(x_dev, groups, group_size)
    # second call in a row: the array still holds the first call's partials, the result must not care
    x2_dev = x_dev * 0.5 + 1.0
    want2, _ = _planned(ctx, x2_dev, groups, group_size)
    second = _noalloc(x2_dev, groups, group_size)
    again = _noalloc(x_dev, groups, group_size)
    assert O.rel_l2(first.astype(np.float64), want.astype(np.float64)) <= TOL
    assert O.rel_l2(second.astype(np.float64), want2.astype(np.float64)) <= TOL
    assert np.array_equal(first, again)            # fixed summation order
    exact = x_dev.double().sum(dim=1).cpu().numpy()   # f64 checker, independent of both entry points
    assert O.rel_l2(first.astype(np.float64), exact) <= TOL


def test_after_a_larger_call_leaves_stale_partials(ctx):
    """A small call right after a big one reads none of the big call's leftovers."""
    import torch
    big = torch.ones((8, 1 << 20), dtype=torch.float32, device="cuda") * 3.0
    assert np.array_equal(_noalloc(big, 8, 1 << 20), np.full(8, 3.0 * (1 << 20), dtype=np.float32))
    small = torch.ones((2, 8192), dtype=torch.float32, device="cuda")
    assert np.array_equal(_noalloc(small, 2, 8192), np.full(2, 8192.0, dtype=np.float32))


def test_refuses_shapes_beyond_the_scratch(ctx):
    import torch
    x = torch.zeros(16, dtype=torch.float32, device="cuda")   # never read: the call is refused before any launch
    out = torch.zeros(16, dtype=torch.float32, device="cuda")
    groups, group_size = 70000, 5000                          # 2 slices per group -> 140000 partials
    rc = lib.he_reduce_sum_f32_noalloc(C.c_void_p(x.data_ptr()), C.c_void_p(out.data_ptr()), groups, group_size, None)
    assert rc == -4                                           # HE_ERR_WORKSPACE
    msg = lib.he_last_error_string().decode()
    assert "140000" in msg and str(MAX_PARTIALS) in msg
    rc = lib.he_reduce_sum_f32_noalloc(C.c_void_p(x.data_ptr()), C.c_void_p(out.data_ptr()), 1 << 20, 1 << 12, None)
    assert rc == -2 and "2^31" in lib.he_last_error_string().decode()
    rc = lib.he_reduce_sum_f32_noalloc(None, C.c_void_p(out.data_ptr()), 4, 4, None)
    assert rc == -1
