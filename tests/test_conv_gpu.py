"""Implicit-GEMM convolutions (forward, data gradient, filter gradient) against the oracle on the same bf16
input bits: every layer geometry of the model in resnet-train/src/model.rs:9-83,112-247 at batch 4, the 7x7/2
head and one 3x3 layer at batch 128, odd image sizes, and the fused epilogues.  Tolerance: rel-L2 <= 1e-2 for
bf16 outputs, <= 1e-5 for the f32 statistics relative to the oracle's sums of the same stored values."""
import numpy as np
import pytest

import helium_b200 as hb
from helium_b200 import ir
from helpers import O, bf16_normal, rng, storage_to_torch, torch_to_storage

pytestmark = pytest.mark.gpu


def _dec(bits, shape):
    return O.decode(bits, ir.BF16, shape)


def _launch(ctx, plan, ins_bits_or_f32):
    import torch
    tin = []
    for a in ins_bits_or_f32:
        tin.append(storage_to_torch(a, ir.BF16) if a.dtype == np.uint16 else torch.from_numpy(np.ascontiguousarray(a)).cuda())
    outs = plan.launch(tin)
    torch.cuda.synchronize()
    ctx.poll()
    return [torch_to_storage(t, dt) for t, dt in zip(outs, plan.out_dtypes)]


# (H, W, C, K, R, S, stride): head (RGB padded to 8 channels), then per segment: 1x1/2 shortcut, 3x3/2, 3x3, and the 1x1 tail
MODEL_LAYERS = [(224, 224, 8, 32, 7, 7, 2)]
for c, hw in ((32, 112), (64, 56), (128, 28), (256, 14)):
    MODEL_LAYERS += [(hw, hw, c, 2 * c, 1, 1, 2), (hw, hw, c, 2 * c, 3, 3, 2), (hw // 2, hw // 2, 2 * c, 2 * c, 3, 3, 1)]
MODEL_LAYERS += [(7, 7, 512, 1000, 1, 1, 1)]


def _case(batch, geom, seed):
    H, W, C, K, R, S, st = geom
    r = rng(seed)
    x = bf16_normal(r, (batch, H, W, C))
    w = bf16_normal(r, (K, R, S, C), 1.0 / np.sqrt(R * S * C))
    (P, Q), _ = O.conv_geometry((H, W), (R, S), (st, st))
    dy = bf16_normal(r, (batch, P, Q, K))
    return x, w, dy, (P, Q)


@pytest.mark.parametrize("geom", MODEL_LAYERS, ids=lambda g: "x".join(map(str, g)))
def test_model_layers_batch4(ctx, geom):
    H, W, C, K, R, S, st = geom
    batch = 4
    x, w, dy, (P, Q) = _case(batch, geom, 11)
    kw = dict(batch=batch, in_hw=(H, W), in_channels=C, out_channels=K, kernel=(R, S), stride=st)
    xv, wv, dyv = _dec(x, x.shape), _dec(w, w.shape), _dec(dy, dy.shape)
    plan = hb.Plan.conv2d(ctx, "fwd", **kw)
    (y,) = _launch(ctx, plan, [x, w])
    err = O.rel_l2(_dec(y, (batch, P, Q, K)), O.conv2d(xv, wv, (st, st)))
    assert err <= 1e-2, (err, plan.description)
    plan = hb.Plan.conv2d(ctx, "bwd_data", **kw)
    (dx,) = _launch(ctx, plan, [dy, w])
    err = O.rel_l2(_dec(dx, x.shape), O.conv2d_backward_data(dyv, wv, (H, W), (st, st)))
    assert err <= 1e-2, (err, plan.description)
    plan = hb.Plan.conv2d(ctx, "bwd_filter", **kw)
    (dw,) = _launch(ctx, plan, [dy, x])
    err = O.rel_l2(_dec(dw, w.shape), O.conv2d_backward_filter(dyv, xv, (R, S), (st, st)))
    assert err <= 1e-2, (err, plan.description)
    (dw2,) = _launch(ctx, plan, [dy, x])
    assert np.array_equal(dw, dw2), "the split-K fold must be bit-stable"


@pytest.mark.parametrize("geom", [(9, 11, 8, 24, 3, 3, 1), (10, 14, 16, 8, 3, 3, 2), (13, 7, 72, 136, 3, 3, 1), (5, 5, 8, 8, 5, 5, 1),
                                  (12, 12, 8, 16, 1, 1, 2)], ids=lambda g: "x".join(map(str, g)))
def test_ragged_geometries(ctx, geom):
    """Image sizes that no patch divides, channel counts off the 64 grid, odd sizes under a stride of two."""
    H, W, C, K, R, S, st = geom
    batch = 3
    x, w, dy, (P, Q) = _case(batch, geom, 12)
    kw = dict(batch=batch, in_hw=(H, W), in_channels=C, out_channels=K, kernel=(R, S), stride=st)
    xv, wv, dyv = _dec(x, x.shape), _dec(w, w.shape), _dec(dy, dy.shape)
    (y,) = _launch(ctx, hb.Plan.conv2d(ctx, "fwd", **kw), [x, w])
    assert O.rel_l2(_dec(y, (batch, P, Q, K)), O.conv2d(xv, wv, (st, st))) <= 1e-2
    (dx,) = _launch(ctx, hb.Plan.conv2d(ctx, "bwd_data", **kw), [dy, w])
    assert O.rel_l2(_dec(dx, x.shape), O.conv2d_backward_data(dyv, wv, (H, W), (st, st))) <= 1e-2
    (dw,) = _launch(ctx, hb.Plan.conv2d(ctx, "bwd_filter", **kw), [dy, x])
    assert O.rel_l2(_dec(dw, w.shape), O.conv2d_backward_filter(dyv, xv, (R, S), (st, st))) <= 1e-2


def test_fused_epilogues(ctx):
    """Forward: bias + residual + batch statistics.  Backward: extra gradient branch + rectifier gate + the two
    sums of batch norm's backward."""
    batch, H, W, C, K = 4, 28, 28, 64, 128
    geom = (H, W, C, K, 3, 3, 1)
    x, w, dy, (P, Q) = _case(batch, geom, 13)
    r = rng(14)
    bias = (r.standard_normal(K) * 0.1).astype(np.float32)
    resid = bf16_normal(r, (batch, P, Q, K))
    kw = dict(batch=batch, in_hw=(H, W), in_channels=C, out_channels=K, kernel=(3, 3), stride=1)
    plan = hb.Plan.conv2d(ctx, "fwd", bias=True, resid=True, stats=True, **kw)
    y, st = _launch(ctx, plan, [x, w, bias, resid])
    want = O.conv2d(_dec(x, x.shape), _dec(w, w.shape)) + bias.astype(np.float64) + _dec(resid, resid.shape)
    assert O.rel_l2(_dec(y, want.shape), want) <= 1e-2, plan.description
    # the statistics are sums of the f32 values before the bf16 rounding of the stored tile
    assert O.rel_l2(st.reshape(2, K)[0], want.reshape(-1, K).sum(0)) <= 1e-3
    assert O.rel_l2(st.reshape(2, K)[1], (want * want).reshape(-1, K).sum(0)) <= 1e-5 * 100
    # backward
    gx = bf16_normal(r, (batch, H, W, C))
    scale = (r.random(C) + 0.5).astype(np.float32); shift = (r.standard_normal(C) * 0.3).astype(np.float32)
    extra = bf16_normal(r, (batch, H, W, C))
    plan = hb.Plan.conv2d(ctx, "bwd_data", resid=True, gate=True, stats=True, **kw)
    dx, st = _launch(ctx, plan, [dy, w, extra, gx, scale, shift])
    gxv = _dec(gx, gx.shape)
    g = O.conv2d_backward_data(_dec(dy, dy.shape), _dec(w, w.shape), (H, W)) + _dec(extra, extra.shape)
    mask = (gxv.astype(np.float32) * scale + shift) > 0
    g = np.where(mask, g, 0.0)
    assert O.rel_l2(_dec(dx, g.shape), g) <= 1e-2, plan.description
    assert O.rel_l2(st.reshape(2, C)[0], g.reshape(-1, C).sum(0)) <= 1e-3
    assert O.rel_l2(st.reshape(2, C)[1], (g * gxv).reshape(-1, C).sum(0)) <= 1e-3
    dx2, st2 = _launch(ctx, plan, [dy, w, extra, gx, scale, shift])
    assert np.array_equal(dx, dx2) and np.array_equal(st, st2)


@pytest.mark.parametrize("geom", [(224, 224, 8, 32, 7, 7, 2), (56, 56, 64, 64, 3, 3, 1)], ids=lambda g: "x".join(map(str, g)))
def test_batch128_layers(ctx, geom):
    """The head and a 3x3 layer at the benchmark batch.  Forward and data gradient are checked on 3 sampled images
    (each image is independent); the filter gradient, which sums over all 128 images, against a float32 torch
    convolution backward on the CPU over the whole batch."""
    import torch
    import torch.nn.functional as F
    H, W, C, K, R, S, st = geom
    batch = 128
    x, w, dy, (P, Q) = _case(batch, geom, 15)
    kw = dict(batch=batch, in_hw=(H, W), in_channels=C, out_channels=K, kernel=(R, S), stride=st)
    sel = [0, 77, 127]
    xv, wv, dyv = _dec(x[sel], (3, H, W, C)), _dec(w, w.shape), _dec(dy[sel], (3, P, Q, K))
    (y,) = _launch(ctx, hb.Plan.conv2d(ctx, "fwd", **kw), [x, w])
    assert O.rel_l2(_dec(y.reshape(batch, P, Q, K)[sel], (3, P, Q, K)), O.conv2d(xv, wv, (st, st))) <= 1e-2
    (dx,) = _launch(ctx, hb.Plan.conv2d(ctx, "bwd_data", **kw), [dy, w])
    assert O.rel_l2(_dec(dx.reshape(batch, H, W, C)[sel], (3, H, W, C)), O.conv2d_backward_data(dyv, wv, (H, W), (st, st))) <= 1e-2
    plan = hb.Plan.conv2d(ctx, "bwd_filter", **kw)
    (dw,) = _launch(ctx, plan, [dy, x])
    tx = torch.from_numpy(O.bf16_bits_to_f32(x)).permute(0, 3, 1, 2)
    tdy = torch.from_numpy(O.bf16_bits_to_f32(dy)).permute(0, 3, 1, 2)
    pad = (R // 2, S // 2)
    tw = torch.zeros((K, C, R, S), requires_grad=True)
    F.conv2d(tx, tw, stride=st, padding=pad)[:, :, :P, :Q].backward(tdy)
    want = tw.grad.permute(0, 2, 3, 1).numpy().astype(np.float64)
    err = O.rel_l2(_dec(dw, w.shape), want)
    assert err <= 1e-2, (err, plan.description)


def test_reference_conv_vector_through_the_c_abi(ctx):
    """helium/tests/tensor_ops.rs:379-397 (`conv_simple`: x = [1, 2], w = [[10, 20], [30, 40]], 1 x 1, Same ->
    [50, 110]) replayed on the GPU.  The kernels take channel counts that are multiples of 8 (a 16-byte pixel for
    TMA), so the two channels are zero-padded to eight on both sides; every value is exact in bf16 and f16."""
    for dt in (ir.BF16, ir.F16):
        x = np.zeros((1, 1, 1, 8)); x[0, 0, 0, :2] = [1.0, 2.0]
        w = np.zeros((8, 1, 1, 8)); w[0, 0, 0, :2] = [10.0, 20.0]; w[1, 0, 0, :2] = [30.0, 40.0]
        plan = hb.Plan.conv2d(ctx, "fwd", batch=1, in_hw=(1, 1), in_channels=8, out_channels=8, kernel=(1, 1), stride=1, dtype=dt,
                              out_dtype=ir.F32)
        import torch
        tin = [storage_to_torch(O.encode(x, dt), dt), storage_to_torch(O.encode(w, dt), dt)]
        (y,) = plan.launch(tin)
        torch.cuda.synchronize()
        ctx.poll()
        assert y.shape == (1, 1, 1, 8)
        assert y.reshape(-1).tolist() == [50.0, 110.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0]


@pytest.mark.parametrize("geom", [(12, 12, 16, 24, 3, 3, 1), (14, 10, 8, 16, 3, 3, 2)], ids=lambda g: "x".join(map(str, g)))
def test_f16_convolutions(ctx, geom):
    """The same three kernels on f16 images and filters (tcgen05 kind::f16 with the f16 operand format), f32 outputs
    so that only the products' input rounding and the f32 accumulation order separate them from the oracle."""
    import torch
    H, W, C, K, R, S, st = geom
    batch = 3
    r = rng(15)
    f16 = lambda shape, s=1.0: O.encode(r.standard_normal(shape) * s, ir.F16)
    (P, Q), _ = O.conv_geometry((H, W), (R, S), (st, st))
    x, w, dy = f16((batch, H, W, C)), f16((K, R, S, C), 1.0 / np.sqrt(R * S * C)), f16((batch, P, Q, K))
    dec = lambda b, shape: O.decode(b, ir.F16, shape)
    kw = dict(batch=batch, in_hw=(H, W), in_channels=C, out_channels=K, kernel=(R, S), stride=st, dtype=ir.F16, out_dtype=ir.F32)
    def run(kind, ins):
        plan = hb.Plan.conv2d(ctx, kind, **kw)
        (o,) = plan.launch([storage_to_torch(a, ir.F16) for a in ins])
        torch.cuda.synchronize()
        ctx.poll()
        return o.cpu().numpy().astype(np.float64)
    xv, wv, dyv = dec(x, (batch, H, W, C)), dec(w, (K, R, S, C)), dec(dy, (batch, P, Q, K))
    assert O.rel_l2(run("fwd", [x, w]), O.conv2d(xv, wv, (st, st))) <= 1e-5
    assert O.rel_l2(run("bwd_data", [dy, w]), O.conv2d_backward_data(dyv, wv, (H, W), (st, st))) <= 1e-5
    assert O.rel_l2(run("bwd_filter", [dy, x]), O.conv2d_backward_filter(dyv, xv, (R, S), (st, st))) <= 1e-5


@pytest.mark.parametrize("case", [(2, 20, 20, 3, 7, 7, 2, 152), (3, 9, 13, 4, 5, 5, 1, 104), (1, 300, 6, 2, 3, 3, 2, 24), (2, 16, 16, 8, 1, 1, 1, 8)],
                         ids=lambda c: "x".join(map(str, c)))
def test_patch_matrix(ctx, case):
    """he_im2col_nhwc against a direct numpy gather: cols[n, p, q, (r * S + s) * C + c] = x[n, p st + r - R/2,
    q st + s - S/2, c], zero outside the image and in the padding columns -- bit for bit (it only moves values)."""
    import ctypes as C
    import torch
    from helium_b200._lib import check, lib
    n, h, w, c, R, S, st, pitch = case
    r = rng(16)
    x = bf16_normal(r, (n, h, w, c))
    P, Q = h // st, w // st
    want = np.zeros((n, P, Q, pitch), dtype=np.uint16)
    for rr in range(R):
        for ss in range(S):
            for p in range(P):
                hh = p * st + rr - R // 2
                if not 0 <= hh < h:
                    continue
                for q in range(Q):
                    ww = q * st + ss - S // 2
                    if 0 <= ww < w:
                        want[:, p, q, (rr * S + ss) * c:(rr * S + ss + 1) * c] = x[:, hh, ww, :]
    tx = storage_to_torch(x, ir.BF16)
    cols = torch.full((n, P, Q, pitch), 7.0, dtype=torch.bfloat16, device="cuda")
    check(lib.he_im2col_nhwc(tx.data_ptr(), cols.data_ptr(), n, h, w, c, R, S, st, pitch, C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    assert np.array_equal(cols.view(torch.int16).cpu().numpy().view(np.uint16), want)
