"""Guard bands around every output and workspace (compute-sanitizer is closed on this pool, so this is the
memory checker): each kernel family runs on shapes that are not multiples of its tiles, every output buffer and the
workspace sit between 4 KiB bands of a known pattern, the workspace is exactly `workspace_bytes` long, and after the
launch both bands of every buffer must be untouched and no output may still hold the fill pattern everywhere.
Values are checked by the parity tests; this file only checks where the kernels write."""
import ctypes as C

import numpy as np
import pytest

import helium_b200 as hb
from helium_b200 import ir
from helium_b200._lib import check, lib
from helium_b200.configs import graph_c3, graph_linear

pytestmark = pytest.mark.gpu

BAND = 4096          # bytes on each side
PATTERN = 0x5A


class Guarded:
    """`nbytes` of device memory between two bands; the payload starts 256-byte aligned."""

    def __init__(self, nbytes: int):
        import torch
        self.n = int(nbytes)
        self.buf = torch.full((2 * BAND + self.n + 256,), PATTERN, dtype=torch.uint8, device="cuda")
        base = self.buf.data_ptr() + BAND
        self.off = BAND + (-base) % 256
        self.ptr = self.buf.data_ptr() + self.off

    def payload(self):
        return self.buf[self.off:self.off + self.n]

    def assert_bands(self, what: str):
        lo = self.buf[:self.off]
        hi = self.buf[self.off + self.n:]
        assert bool((lo == PATTERN).all()), f"{what}: wrote before the buffer"
        assert bool((hi == PATTERN).all()), f"{what}: wrote past the end of the buffer"

    def assert_written(self, what: str):
        if self.n >= 64:
            assert not bool((self.payload() == PATTERN).all()), f"{what}: the output was never written"


def _nbytes(shape, dt):
    n = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
    if dt == ir.BOOL:
        return (n + 31) // 32 * 4
    return n * {ir.F32: 4, ir.U32: 4, ir.BF16: 2, ir.F16: 2}[dt]


def _rand_input(shape, dt, scale=1.0):
    import torch
    n = max(1, int(np.prod(shape, dtype=np.int64)))
    if dt == ir.U32:
        return torch.randint(0, 1000, (n,), dtype=torch.int32, device="cuda")
    if dt == ir.BOOL:
        return torch.randint(0, 2 ** 31 - 1, ((n + 31) // 32,), dtype=torch.int32, device="cuda")
    t = torch.randn(n, device="cuda") * scale
    return t.to({ir.F32: torch.float32, ir.BF16: torch.bfloat16, ir.F16: torch.float16}[dt])


def _run_plan(ctx, plan, graph_or_inputs, what):
    """Launches `plan` on random inputs with guarded outputs and a guarded, exactly sized workspace."""
    import torch
    ins = graph_or_inputs
    outs = [Guarded(_nbytes(s, d)) for s, d in zip(plan.out_shapes, plan.out_dtypes)]
    ws = Guarded(plan.workspace_bytes) if plan.workspace_bytes else None
    for _ in range(2):     # twice: stale partials of the first launch must not change where the second writes
        plan.launch_ptrs([t.data_ptr() for t in ins], [o.ptr for o in outs], ws.ptr if ws else 0)
    torch.cuda.synchronize()
    ctx.poll()
    for i, o in enumerate(outs):
        o.assert_bands(f"{what}: output {i} ({plan.description})")
        o.assert_written(f"{what}: output {i} ({plan.description})")
    if ws:
        ws.assert_bands(f"{what}: workspace ({plan.description})")


def _graph_inputs(g, scale=None):
    return [_rand_input(g.nodes[i].shape, g.nodes[i].dtype, (scale or {}).get(k, 1.0)) for k, i in enumerate(g.inputs)]


# ---- fused matmul -----------------------------------------------------------------------------------------------
MATMULS = {
    "plain_ragged": lambda: graph_linear(129, 257, 131, bias=False),
    "bias_gelu_z_odd_pitch": lambda: graph_linear(200, 136, 72, bias=True, act=ir.UN_GELU, store_z=True),
    "resid_colsum": lambda: graph_linear(300, 264, 96, bias=True, resid=True, colsum="y"),
    "transposed_operands": lambda: graph_linear(130, 72, 200, bias=True, a_t=True, b_t=True),
    "batched": lambda: graph_linear(70, 40, 136, bias=False, batch=3),
    "f32_simt": lambda: graph_linear(33, 17, 29, bias=True, dtype=ir.F32),
    "readme_graph": lambda: graph_c3(136, 264, 72),
    "readme_graph_pair_kernel": lambda: graph_c3(392, 520, 136),
}


@pytest.mark.parametrize("name", sorted(MATMULS))
def test_fused_matmul(ctx, name):
    try:
        g = MATMULS[name]()
    except TypeError as e:       # a builder argument this tree does not have
        pytest.skip(str(e))
    plan = hb.Plan.fused_matmul(ctx, g)
    _run_plan(ctx, plan, _graph_inputs(g), name)


def test_fused_matmul_interpreted_epilogue_and_reductions(ctx):
    g = ir.Graph()
    a = g.new_input([150, 72], ir.BF16); b = g.new_input([72, 264], ir.BF16)
    t = g.unary(ir.UN_SIN, g.matmul(a, b))
    g.new_output(t)
    g.new_output(g.reduce(ir.RED_SUM, t, 1))
    g.new_output(g.reduce(ir.RED_MAX, g.swap_dims(t, 0, 1), 1))
    plan = hb.Plan.fused_matmul(ctx, g)
    _run_plan(ctx, plan, _graph_inputs(g), "interpreted epilogue")


def test_fused_matmul_mainloop_rewrites(ctx, monkeypatch):
    for mode in ("fused", "materialise"):
        monkeypatch.setenv("HE_GEMM_MAINLOOP", mode)
        g = ir.Graph()
        a = g.new_input([392, 136], ir.BF16); m = g.new_input([392, 136], ir.BF16); b = g.new_input([136, 264], ir.BF16)
        g.new_output(g.matmul(g.binary(ir.BIN_MUL, g.unary(ir.UN_RELU, a), m), b))
        plan = hb.Plan.fused_matmul(ctx, g)
        _run_plan(ctx, plan, _graph_inputs(g), "relu * mask, " + mode)
        g = ir.Graph()
        a = g.new_input([264, 72], ir.BF16); b = g.new_input([72, 136], ir.BF16)
        g.new_output(g.matmul(g.unary(ir.UN_TANH, a), g.unary(ir.UN_MUL_CONST, b, 0.5)))
        plan = hb.Plan.fused_matmul(ctx, g)
        _run_plan(ctx, plan, _graph_inputs(g), "generic chains, " + mode)


def test_fused_matmul_8bit(ctx, monkeypatch):
    monkeypatch.setenv("HE_GEMM_F8", "native")
    for shape, ta, tb in (((2, 136, 200, 1001), False, False), ((1, 392, 264, 72), True, True)):
        bt, m, n, k = shape
        g = ir.Graph()
        a = g.new_input([bt, k, m] if ta else [bt, m, k], ir.BF16)
        b = g.new_input([bt, n, k] if tb else [bt, k, n], ir.BF16)
        g.new_output(g.matmul(g.swap_dims(a, 1, 2) if ta else a, g.swap_dims(b, 1, 2) if tb else b, ir.prec_f8(ir.PREC_F8_F32)))
        plan = hb.Plan.fused_matmul(ctx, g)
        assert "f8f6f4" in plan.description
        _run_plan(ctx, plan, _graph_inputs(g), "8-bit multiplication")


# ---- pointwise, permute ----------------------------------------------------------------------------------------
def _pointwise_graphs():
    out = {}
    g = ir.Graph()
    x = g.new_input([5, 13], ir.BF16); y = g.new_input([13], ir.F32)
    g.new_output(g.unary(ir.UN_TANH, g.binary(ir.BIN_ADD, x, g.broadcast_to(y, [5, 13]))))
    out["elementwise_ragged"] = g
    g = ir.Graph()
    x = g.new_input([1001], ir.BF16)
    g.new_output(g.unary(ir.UN_RELU, x))
    out["catalogue_with_tail"] = g
    g = ir.Graph()
    x = g.new_input([37, 45], ir.F32); y = g.new_input([37, 45], ir.F32)
    g.new_output(g.compare(ir.CMP_LT, x, y))
    out["bool_output"] = g
    g = ir.Graph()
    x = g.new_input([3, 70001], ir.F32)
    g.new_output(g.reduce(ir.RED_SUM, g.unary(ir.UN_EXP, g.unary(ir.UN_MUL_CONST, x, 0.1)), 1))
    g.new_output(g.reduce(ir.RED_MAX, x, 1))
    out["reduce_cta_slices"] = g
    g = ir.Graph()
    x = g.new_input([1000, 96], ir.BF16)
    g.new_output(g.reduce(ir.RED_SUM, g.swap_dims(g.unary(ir.UN_RELU, x), 0, 1), 1))
    out["reduce_columns"] = g
    g = ir.Graph()
    x = g.new_input([300, 7], ir.F32)
    g.new_output(g.reduce(ir.RED_MEAN, x, 1))
    out["reduce_warp_per_group"] = g
    g = ir.Graph()
    x = g.new_input([3, 24, 9, 7], ir.BF16); s = g.new_input([24], ir.F32); b = g.new_input([24], ir.F32)
    t = g.binary(ir.BIN_ADD, g.binary(ir.BIN_MUL, x, g.broadcast_to(g.reshape(s, [24, 1, 1]), [3, 24, 9, 7])),
                 g.broadcast_to(g.reshape(b, [24, 1, 1]), [3, 24, 9, 7]))
    g.new_output(g.swap_dims(g.swap_dims(g.unary(ir.UN_RELU, t), 1, 2), 2, 3))
    out["affine_relu_permute"] = g
    return out


@pytest.mark.parametrize("jit", [True, False], ids=["specialised", "interpreter"])
@pytest.mark.parametrize("name", sorted(_pointwise_graphs()))
def test_pointwise(ctx, monkeypatch, name, jit):
    if jit:
        monkeypatch.delenv("HE_PW_JIT", raising=False)
    else:
        monkeypatch.setenv("HE_PW_JIT", "0")
    g = _pointwise_graphs()[name]
    plan = hb.Plan.pointwise(ctx, g)
    _run_plan(ctx, plan, _graph_inputs(g), name)


@pytest.mark.parametrize("shape,perm", [((7, 13), (1, 0)), ((5, 64, 8), (2, 0, 1)), ((3, 16, 40, 24), (0, 2, 3, 1)), ((130, 264), (1, 0))])
@pytest.mark.parametrize("dt", [ir.F32, ir.BF16])
def test_permute(ctx, shape, perm, dt):
    rank = len(shape)
    strides = [0] * rank
    s = 1
    for k in range(rank - 1, -1, -1):
        strides[perm[k]] = s
        s *= shape[perm[k]]
    plan = hb.Plan.permute(ctx, list(shape), strides, dt)
    _run_plan(ctx, plan, [_rand_input(shape, dt)], "permute")


# ---- convolutions and the training kernels ----------------------------------------------------------------------
@pytest.mark.parametrize("geom", [(9, 11, 8, 24, 3, 3, 1), (10, 14, 16, 8, 3, 3, 2), (13, 7, 72, 136, 3, 3, 1), (12, 12, 8, 16, 1, 1, 2)],
                         ids=lambda g_: "x".join(map(str, g_)))
def test_convolutions(ctx, geom):
    H, W, Cin, K, R, S, st = geom
    batch = 3
    P, Q = H // st, W // st
    kw = dict(batch=batch, in_hw=(H, W), in_channels=Cin, out_channels=K, kernel=(R, S), stride=st)
    x = _rand_input((batch, H, W, Cin), ir.BF16); w = _rand_input((K, R, S, Cin), ir.BF16, 0.1); dy = _rand_input((batch, P, Q, K), ir.BF16)
    bias = _rand_input((K,), ir.F32); resid = _rand_input((batch, P, Q, K), ir.BF16)
    _run_plan(ctx, hb.Plan.conv2d(ctx, "fwd", bias=True, resid=True, stats=True, **kw), [x, w, bias, resid], "conv forward")
    gx = _rand_input((batch, H, W, Cin), ir.BF16); sc = _rand_input((Cin,), ir.F32); sh = _rand_input((Cin,), ir.F32)
    extra = _rand_input((batch, H, W, Cin), ir.BF16)
    if R == 1 and st == 2:
        # a 1 x 1 / 2 data gradient leaves input pixels no tap reaches (zero-filled): fused epilogues are refused there
        with pytest.raises(hb.HeliumError):
            hb.Plan.conv2d(ctx, "bwd_data", resid=True, gate=True, stats=True, **kw)
        _run_plan(ctx, hb.Plan.conv2d(ctx, "bwd_data", **kw), [dy, w], "conv data gradient")
    else:
        _run_plan(ctx, hb.Plan.conv2d(ctx, "bwd_data", resid=True, gate=True, stats=True, **kw), [dy, w, extra, gx, sc, sh], "conv data gradient")
    _run_plan(ctx, hb.Plan.conv2d(ctx, "bwd_filter", **kw), [dy, x], "conv filter gradient")


def test_training_kernels(ctx):
    import torch
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    pixels, ch = 3 * 9 * 11, 24
    nb = lambda n, dt: _nbytes((n,), dt)
    x = _rand_input((pixels, ch), ir.BF16); g = _rand_input((pixels, ch), ir.BF16); e = _rand_input((pixels, ch), ir.BF16)
    scale = _rand_input((ch,), ir.F32); shift = _rand_input((ch,), ir.F32)
    ws = Guarded(lib.he_bn_workspace_bytes(pixels, ch))
    # y = relu(x * scale + shift) with the statistics of y
    y = Guarded(nb(pixels * ch, ir.BF16)); stats = Guarded(nb(2 * ch, ir.F32))
    check(lib.he_bn_apply(x.data_ptr(), y.ptr, scale.data_ptr(), shift.data_ptr(), pixels, ch, 1, stats.ptr, ws.ptr, st))
    # backward: plain with the column sums of its output, and masked with its two sums
    coef = _rand_input((3 * ch,), ir.F32)
    out1 = Guarded(nb(pixels * ch, ir.BF16)); sums1 = Guarded(nb(ch, ir.F32))
    check(lib.he_bn_backward_apply(g.data_ptr(), x.data_ptr(), e.data_ptr(), out1.ptr, coef.data_ptr(), None, None, None, sums1.ptr, ws.ptr,
                                   pixels, ch, st))
    out2 = Guarded(nb(pixels * ch, ir.BF16)); sums2 = Guarded(nb(2 * ch, ir.F32))
    check(lib.he_bn_backward_apply(g.data_ptr(), x.data_ptr(), None, out2.ptr, coef.data_ptr(), x.data_ptr(), scale.data_ptr(), shift.data_ptr(),
                                   sums2.ptr, ws.ptr, pixels, ch, st))
    cs = Guarded(nb(ch, ir.F32))
    check(lib.he_colsum_bf16(x.data_ptr(), cs.ptr, ws.ptr, pixels, ch, st))
    # patch matrix of a 3-channel image
    n, h, w = 2, 21, 19
    img = _rand_input((n, h, w, 3), ir.BF16)
    cols = Guarded(nb(n * (h // 2) * (w // 2) * 152, ir.BF16))
    check(lib.he_im2col_nhwc(img.data_ptr(), cols.ptr, n, h, w, 3, 7, 7, 2, 152, st))
    # pooled softmax cross entropy
    batch, pos, classes = 5, 6, 37
    logits = _rand_input((batch, pos, classes), ir.BF16)
    labels = torch.randint(0, classes, (batch,), dtype=torch.int32, device="cuda")
    loss = Guarded(nb(batch, ir.F32)); dlog = Guarded(nb(batch * pos * classes, ir.BF16))
    check(lib.he_pool_softmax_ce(logits.data_ptr(), labels.data_ptr(), loss.ptr, dlog.ptr, batch, pos, classes, st))
    # SGD with momentum on a length that is no multiple of any vector width
    nw = 1003
    wgt = Guarded(nb(nw, ir.F32)); avg = Guarded(nb(nw, ir.F32)); w16 = Guarded(nb(nw, ir.BF16))
    wgt.payload().view(torch.float32).normal_(); avg.payload().view(torch.float32).zero_()
    grad = _rand_input((nw,), ir.BF16)
    check(lib.he_sgd_momentum(wgt.ptr, avg.ptr, grad.data_ptr(), ir.BF16, w16.ptr, nw, 0.01, 0.9, 1, st))
    torch.cuda.synchronize()
    ctx.poll()
    for name, buf in (("bn_apply y", y), ("bn_apply statistics", stats), ("bn_backward out", out1), ("bn_backward column sums", sums1),
                      ("bn_backward masked out", out2), ("bn_backward masked sums", sums2), ("colsum", cs), ("patch matrix", cols),
                      ("loss", loss), ("dlogits", dlog), ("weights", wgt), ("momentum", avg), ("bf16 weights", w16), ("bn workspace", ws)):
        buf.assert_bands(name)
        if name not in ("bn workspace",):
            buf.assert_written(name)
