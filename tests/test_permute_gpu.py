"""permute_dims kernels against the oracle: bit-exact, every kernel variant, ragged and empty shapes,
the benchmark shapes at full size."""
import numpy as np
import pytest

import helium_b200 as hb
from helium_b200 import ir
from helpers import O, rng

pytestmark = pytest.mark.gpu


def _permute_case(ctx, shape, perm, dtype, reference_compat=False, misalign=False):
    """perm[k] = input axis placed at output position k."""
    import torch
    nd = {ir.F32: np.float32, ir.BF16: np.uint16, ir.F16: np.uint16, ir.U32: np.uint32}[dtype]
    r = rng(hash((tuple(shape), tuple(perm))) % (1 << 31))
    total = int(np.prod(shape))
    x = r.integers(0, 1 << 16, size=total, dtype=np.uint32).astype(nd).reshape(shape) if nd != np.float32 else \
        r.standard_normal(shape, dtype=np.float32)
    strides = [0] * len(shape)
    s = 1
    for k in reversed(range(len(shape))):
        strides[perm[k]] = s
        s *= shape[perm[k]]
    want = O.permute(x, strides)
    plan = hb.Plan.permute(ctx, list(shape), strides, dtype)
    tdt = {np.float32: torch.float32, np.uint16: torch.int16, np.uint32: torch.int32}[nd]
    pad = 1 if misalign else 0   # shifts both pointers off 16-byte alignment
    xin_buf = torch.empty(total + pad, dtype=tdt, device="cuda")
    out_buf = torch.full((total + pad + 8,), -1, dtype=tdt, device="cuda")
    xin = xin_buf[pad:pad + total]
    xin.copy_(torch.from_numpy(x.reshape(-1).view({np.float32: np.float32, np.uint16: np.int16, np.uint32: np.int32}[nd])))
    plan.launch_ptrs([xin.data_ptr()], [out_buf[pad:].data_ptr()])
    torch.cuda.synchronize()
    got = out_buf[pad:pad + total].cpu().numpy().view(nd)
    assert np.array_equal(got, want.view(nd)), plan.description
    # canary after the output must be untouched
    assert (out_buf[pad + total:].cpu().numpy() == -1).all(), "wrote past the end: " + plan.description
    return plan.description


@pytest.mark.parametrize("dtype", [ir.F32, ir.BF16])
@pytest.mark.parametrize("shape,perm", [
    ((64, 48), (1, 0)),                 # plain 2-D transpose, vector path
    ((7, 13), (1, 0)),                  # ragged: scalar path
    ((5, 64, 8), (2, 0, 1)),            # small inner dim (the [4096,4096,8] family)
    ((3, 16, 40, 24), (0, 2, 3, 1)),    # NCHW -> NHWC
    ((3, 40, 24, 16), (0, 3, 1, 2)),    # NHWC -> NCHW
    ((4, 6, 10, 32), (1, 0, 2, 3)),     # inner axis preserved: row gather, 16-byte units
    ((4, 6, 10, 9), (2, 1, 0, 3)),      # inner axis preserved, element units
    ((2, 3, 4, 5, 6), (4, 2, 0, 3, 1)),
    ((1, 256, 1, 96), (3, 1, 0, 2)),    # singleton dims
    ((130, 264), (1, 0)),               # partial tiles in both directions
    ((32, 64, 16, 4), (0, 2, 3, 1)),
])
def test_permutations(ctx, shape, perm, dtype):
    _permute_case(ctx, shape, perm, dtype)


def test_unaligned_pointers_use_the_scalar_kernels(ctx):
    _permute_case(ctx, (64, 48), (1, 0), ir.F32, misalign=True)
    _permute_case(ctx, (4, 6, 10, 32), (1, 0, 2, 3), ir.BF16, misalign=True)


def test_empty_and_identity(ctx):
    import torch
    plan = hb.Plan.permute(ctx, [4, 0, 8], [0, 8, 1], ir.F32)
    plan.launch_ptrs([0], [0])  # nothing is touched
    x = torch.arange(24, dtype=torch.float32, device="cuda").reshape(2, 3, 4)
    plan = hb.Plan.permute(ctx, [2, 3, 4], [12, 4, 1], ir.F32)
    (y,) = plan.launch([x])
    assert torch.equal(y.reshape(-1), x.reshape(-1))


def test_reference_stride_convention(ctx):
    # out_strides computed the reference's way (permute_dims.rs:158-172) place the data of a
    # 3-cycle in the inverse permutation's layout; the kernel must follow the strides it is given.
    import torch
    x = rng(5).standard_normal((6, 10, 4), dtype=np.float32)
    swaps = [(1, 2), (0, 1)]
    st = hb.permute_output_strides(list(x.shape), swaps, True)
    assert st == O.output_strides_reference(swaps, x.shape)
    plan = hb.Plan.permute(ctx, list(x.shape), st, ir.F32)
    (y,) = plan.launch([torch.from_numpy(x).cuda()])
    assert np.array_equal(y.cpu().numpy().reshape(-1), O.permute(x, st))


@pytest.mark.parametrize("shape,swaps,dtype", [
    ((4096, 4096, 8), [(1, 2), (0, 1)], ir.F32),        # the f32 benchmark permutation
    ((64, 256, 56, 56), [(1, 2), (2, 3)], ir.BF16),     # the permute half of config 2a
    ((2048, 128, 128, 32), [(0, 3)], ir.F32),           # helium/examples/permute_dim_benchmark.rs:13-38
])
def test_full_size_shapes(ctx, shape, swaps, dtype):
    """Full benchmark sizes: checked on the device with torch.permute as the index oracle (bit moves
    only, so equality is exact) plus an involution property: permuting back restores the input."""
    import torch
    tdt = torch.float32 if dtype == ir.F32 else torch.bfloat16
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(shape, generator=g, device="cuda", dtype=torch.float32).to(tdt)
    st = hb.permute_output_strides(list(shape), swaps)
    plan = hb.Plan.permute(ctx, list(shape), st, dtype)
    (y,) = plan.launch([x])
    ref = x
    for a, b in swaps:
        ref = ref.transpose(a, b)
    assert torch.equal(y.reshape(-1), ref.contiguous().reshape(-1)), plan.description
    # back again
    out_shape = list(ref.shape)
    back_st = hb.permute_output_strides(out_shape, list(reversed(swaps)))
    plan2 = hb.Plan.permute(ctx, out_shape, back_st, dtype)
    (z,) = plan2.launch([y.reshape(out_shape)])
    assert torch.equal(z.reshape(-1), x.reshape(-1)), plan2.description
