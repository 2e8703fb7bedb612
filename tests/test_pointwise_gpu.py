"""Pointwise kernels (both tiers) against the oracle."""
import numpy as np
import pytest

import helium_b200 as hb
from helium_b200 import ir
from helpers import O, graph_affine_relu_permute, rng, storage_to_torch, torch_to_storage

pytestmark = pytest.mark.gpu


def _run(ctx, graph, inputs):
    import torch
    plan = hb.Plan.pointwise(ctx, graph)
    ins = [storage_to_torch(a, graph.nodes[i].dtype) for a, i in zip(inputs, graph.inputs)]
    outs = plan.launch(ins)
    torch.cuda.synchronize()
    return [torch_to_storage(t, graph.nodes[o].dtype) for t, o in zip(outs, graph.outputs)], plan


def _close(graph, got, want, tol):
    for o, g_, w_ in zip(graph.outputs, got, want):
        node = graph.nodes[o]
        if node.dtype in (ir.BOOL, ir.U32):
            n_words = (node.num_elements + 31) // 32 if node.dtype == ir.BOOL else node.num_elements
            assert np.array_equal(np.asarray(g_).reshape(-1)[:n_words], np.asarray(w_).reshape(-1)[:n_words])
        else:
            a = O.decode(g_, node.dtype, node.shape).reshape(-1)
            b = O.decode(w_, node.dtype, node.shape).reshape(-1)
            assert np.allclose(a, b, rtol=tol, atol=tol), float(np.abs(a - b).max())


@pytest.mark.parametrize("shape", [(2, 8, 3, 8), (3, 16, 7, 8), (2, 256, 8, 8), (1, 24, 5, 3)])
@pytest.mark.parametrize("x_dtype,p_dtype", [(ir.BF16, ir.F32), (ir.F32, ir.F32), (ir.F16, ir.F16), (ir.BF16, ir.BF16)])
def test_affine_relu_permute_tier2(ctx, shape, x_dtype, p_dtype):
    n, c, h, w = shape
    g = graph_affine_relu_permute(n, c, h, w, x_dtype, p_dtype)
    r = rng(11)
    x = r.standard_normal(shape, dtype=np.float32)
    s = r.random(c, dtype=np.float32) + 0.5
    b = r.standard_normal(c, dtype=np.float32) * 0.1
    ins = [O.encode(x.astype(np.float64), x_dtype), O.encode(s.astype(np.float64), p_dtype), O.encode(b.astype(np.float64), p_dtype)]
    got, plan = _run(ctx, g, ins)
    assert "tier 2" in plan.description
    want = O.evaluate(g, ins)
    a = O.decode(got[0], x_dtype, (n, h, w, c)).reshape(-1)
    bb = O.decode(want[0], x_dtype, (n, h, w, c)).reshape(-1)
    # one fused multiply-add then one rounding: the f64 oracle can differ only on double-rounding ties
    ulp = {ir.BF16: 2.0 ** -8, ir.F16: 2.0 ** -11, ir.F32: 2.0 ** -23}[x_dtype]
    assert np.all(np.abs(a - bb) <= ulp * np.maximum(np.abs(bb), 1e-30) * 1.01 + 1e-38)
    assert np.mean(a != bb) < 1e-3
    # zeros of the relu must be exact
    assert np.array_equal(a == 0, bb == 0)


def test_config_2a_full_size(ctx):
    """The fused affine + relu + layout change at its benchmark size: [64,256,56,56] bf16; checked against the numpy oracle."""
    g = graph_affine_relu_permute(64, 256, 56, 56)
    r = rng(1)
    x = O.f32_to_bf16_bits(r.standard_normal((64, 256, 56, 56), dtype=np.float32))
    s = r.random(256, dtype=np.float32) + 0.5
    b = r.standard_normal(256, dtype=np.float32) * 0.1
    got, plan = _run(ctx, g, [x, s, b])
    want = O.affine_relu_nchw_to_nhwc(x, s, b).reshape(-1)
    assert "tier 2" in plan.description
    assert np.array_equal(got[0].reshape(-1), want), plan.description


def test_interpreter_mixed_graph(ctx):
    g = ir.Graph()
    x = g.new_input([33, 17, 5], ir.BF16)
    y = g.new_input([17, 1], ir.F32)
    yb = g.broadcast_to(y, [33, 17, 5])
    t = g.binary(ir.BIN_ADD, g.unary(ir.UN_TANH, x), g.binary(ir.BIN_MUL, yb, g.unary(ir.UN_SIGMOID, x)))
    g.new_output(t)                                        # bf16
    g.new_output(g.cast(g.unary(ir.UN_EXP, t), ir.F32))    # f32
    g.new_output(g.compare(ir.CMP_GT, t, yb))              # bool, bit-packed
    g.new_output(g.swap_dims(g.cast(t, ir.F16), 0, 2))     # would break the equal-size rule? no: same count
    r = rng(12)
    ins = [O.f32_to_bf16_bits(r.standard_normal((33, 17, 5), dtype=np.float32)), r.standard_normal((17, 1), dtype=np.float32)]
    got, plan = _run(ctx, g, ins)
    assert "tier 1" in plan.description
    want = O.evaluate(g, ins)
    _close(g, got[:2] + got[3:], want[:2] + want[3:], 1e-2)
    # the comparison may flip where t == yb up to rounding; demand equality away from ties
    tv = O.decode(want[0], ir.BF16, (33, 17, 5)).reshape(-1)
    yv = np.broadcast_to(ins[1].reshape(1, 17, 1), (33, 17, 5)).reshape(-1)
    far = np.abs(tv - yv) > 1e-2 * np.maximum(1.0, np.abs(yv))
    gb = O.unpack_bools(got[2], tv.size)
    wb = O.unpack_bools(want[2], tv.size)
    assert np.array_equal(gb[far], wb[far])


@pytest.mark.parametrize("shape,depth,op", [
    ((256, 10), 1, ir.RED_MAX), ((256, 10), 1, ir.RED_SUM), ((256, 10), 2, ir.RED_SUM),
    ((2, 1000, 100), 2, ir.RED_SUM), ((2, 1000, 100), 3, ir.RED_MEAN), ((7, 5000), 1, ir.RED_MIN),
    ((3, 70000), 1, ir.RED_SUM), ((1, 1 << 20), 2, ir.RED_MEAN),
])
def test_reductions(ctx, shape, depth, op):
    g = ir.Graph()
    x = g.new_input(list(shape), ir.F32)
    g.new_output(g.reduce(op, g.binary(ir.BIN_MUL, x, x), depth))
    ins = [rng(13).standard_normal(shape, dtype=np.float32)]
    got, plan = _run(ctx, g, ins)
    want = O.evaluate(g, ins)
    a, b = got[0].reshape(-1).astype(np.float64), want[0].reshape(-1).astype(np.float64)
    assert O.rel_l2(a, b) <= 1e-5, (O.rel_l2(a, b), plan.description)   # f32 reductions: rel-L2 <= 1e-5
    # bit-stable across launches (fixed summation order; helium/tests/stress_test.rs:38 asks for this)
    got2, _ = _run(ctx, g, ins)
    assert np.array_equal(got[0], got2[0])


def test_softmax_cross_entropy_pieces(ctx):
    """The reductions of config 1's loss: row max, row sum of exp, and the scalar loss."""
    g = ir.Graph()
    z = g.new_input([256, 10], ir.F32)
    t = g.new_input([256, 10], ir.F32)
    m = g.new_input([256, 1], ir.F32)
    zs = g.binary(ir.BIN_ADD, z, g.unary(ir.UN_NEG, g.broadcast_to(m, [256, 10])))
    e = g.unary(ir.UN_EXP, zs)
    g.new_output(g.reduce(ir.RED_SUM, e, 1))
    r = rng(14)
    zv = r.standard_normal((256, 10), dtype=np.float32) * 3
    onehot = np.eye(10, dtype=np.float32)[r.integers(0, 10, 256)]
    ins = [zv, onehot, zv.max(1, keepdims=True)]
    got, _ = _run(ctx, g, ins)
    want = O.evaluate(g, ins)
    assert O.rel_l2(got[0], want[0]) <= 1e-5


_DENSE = {
    "relu": (1, lambda g, i: g.unary(ir.UN_RELU, i[0])),
    "gelu": (1, lambda g, i: g.unary(ir.UN_GELU, i[0])),
    "add": (2, lambda g, i: g.binary(ir.BIN_ADD, i[0], i[1])),
    "mul": (2, lambda g, i: g.binary(ir.BIN_MUL, i[1], i[0])),
    "add_relu": (2, lambda g, i: g.unary(ir.UN_RELU, g.binary(ir.BIN_ADD, i[0], i[1]))),
    "relu_mul": (2, lambda g, i: g.binary(ir.BIN_MUL, g.unary(ir.UN_RELU, i[0]), i[1])),
    "fma": (3, lambda g, i: g.binary(ir.BIN_ADD, g.binary(ir.BIN_MUL, i[0], i[1]), i[2])),
    "sgd": (2, lambda g, i: g.binary(ir.BIN_ADD, i[0], g.unary(ir.UN_NEG, g.binary(ir.BIN_MUL, i[1], g.constant(0.01, list(g.nodes[i[1]].shape)))))),
}


@pytest.mark.parametrize("dtype", [ir.F32, ir.BF16, ir.F16])
@pytest.mark.parametrize("name", sorted(_DENSE))
def test_dense_elementwise_tier(ctx, name, dtype):
    """The hand-written dense kernels against the oracle, on a size with a ragged last CTA, and against
    the interpreter they replace (reached here through a tensor that is not 16-byte aligned)."""
    import torch
    n_in, build = _DENSE[name]
    shape = [257, 264]
    g = ir.Graph()
    ins = [g.new_input(shape, dtype) for _ in range(n_in)]
    g.new_output(build(g, ins))
    r = rng(77)
    host = [O.encode(r.standard_normal(shape), dtype) for _ in range(n_in)]
    plan = hb.Plan.pointwise(ctx, g)
    assert "tier 2 (dense elementwise" in plan.description
    tin = [storage_to_torch(a, dtype) for a in host]
    (out,) = plan.launch(tin)
    torch.cuda.synchronize()
    got = torch_to_storage(out, dtype)
    want = O.evaluate(g, host)[0]
    a, b = O.decode(got, dtype, shape), O.decode(want, dtype, shape)
    tol = 1e-6 if dtype == ir.F32 else 1e-2
    assert O.rel_l2(a, b) <= tol
    # same plan, misaligned first input: the launch falls back to the interpreter; results must agree
    # bit for bit with the dense kernel (same operation order, one rounding)
    pad = torch.empty(tin[0].numel() + 8, dtype=tin[0].dtype, device="cuda")
    shifted = pad[1:1 + tin[0].numel()].view(tin[0].shape)
    shifted.copy_(tin[0])
    out2 = torch.empty_like(out)
    plan.launch_ptrs([shifted.data_ptr()] + [t.data_ptr() for t in tin[1:]], [out2.data_ptr()])
    torch.cuda.synchronize()
    if name != "gelu":   # erff is evaluated by the same libm routine in both tiers, but contraction around it may differ
        assert torch.equal(out.view(torch.int16 if dtype != ir.F32 else torch.int32), out2.view(torch.int16 if dtype != ir.F32 else torch.int32))
    else:
        assert O.rel_l2(O.decode(torch_to_storage(out2, dtype), dtype, shape), b) <= tol


@pytest.mark.parametrize("shape,dtype", [((300, 520), ir.F32), ((4096, 1024), ir.BF16), ((3, 129, 64), ir.F32), ((70, 33), ir.F32)])
def test_transposed_reductions_use_column_mode(ctx, shape, dtype):
    """helium's bias gradient: swap_dims -> reduce_sum(depth 1) -> reshape.  The reduction reads through
    the swapped view with lanes along the contiguous axis; results as the oracle's, bit-stable."""
    g = ir.Graph()
    x = g.new_input(list(shape), dtype)
    y = g.binary(ir.BIN_MUL, x, x)
    r = len(shape)
    red = g.reduce(ir.RED_SUM, g.swap_dims(y, r - 2, r - 1), 1)
    g.new_output(g.reshape(red, list(shape[:-2]) + [shape[-1]]))
    ins = [O.encode(rng(17).standard_normal(shape), dtype)]
    got, plan = _run(ctx, g, ins)
    if shape[-1] >= 32:
        assert "column mode" in plan.description, plan.description
    want = O.evaluate(g, ins)
    assert O.rel_l2(got[0].reshape(-1).astype(np.float64), want[0].reshape(-1).astype(np.float64)) <= 1e-5
    got2, _ = _run(ctx, g, ins)
    assert np.array_equal(got[0], got2[0])


@pytest.mark.parametrize("shape,axes,dtype", [((300, 520), [0], ir.F32), ((1024, 512), [0], ir.BF16), ((4, 129, 64), [1], ir.F32),
                                              ((4, 64, 33), [0], ir.F16), ((5, 32, 48), [0, 2], ir.F32), ((8, 1, 16), [0], ir.F32),
                                              ((6, 7, 8, 9), [1, 2], ir.F32)])
@pytest.mark.parametrize("op", [ir.RED_SUM, ir.RED_MAX, ir.RED_MEAN])
def test_rank_kept_reductions_over_any_axes(ctx, shape, axes, dtype, op):
    """The playground's Reduction{axes} (helium-playground/src/opgraph.rs:397-413) over dims that are not the
    trailing ones, as a kernel of its own: planned as swaps to a trailing reduction, results as the oracle's in the
    order of the kept dims, bit-stable, next to an elementwise output of the same kernel."""
    g = ir.Graph()
    x = g.new_input(list(shape), dtype)
    y = g.unary(ir.UN_TANH, x)
    g.new_output(g.reduce_axes(op, y, axes))
    ins = [O.encode(rng(23).standard_normal(shape), dtype)]
    got, plan = _run(ctx, g, ins)
    want = O.evaluate(g, ins)
    assert got[0].size == want[0].size
    assert O.rel_l2(got[0].reshape(-1).astype(np.float64), want[0].reshape(-1).astype(np.float64)) <= 1e-5, plan.description
    got2, _ = _run(ctx, g, ins)
    assert np.array_equal(got[0], got2[0])


@pytest.mark.parametrize("shape,dtype", [((4096, 1024), ir.BF16), ((300, 520), ir.F32), ((3, 513, 64), ir.F16), ((8192, 4096), ir.BF16)])
def test_dense_column_sum_kernel(ctx, shape, dtype):
    """Bias gradient of a plain tensor (swap_dims -> reduce_sum -> reshape with nothing in front):
    the hand-written column-sum kernel, against the oracle and against the column-mode interpreter
    (reached through a misaligned input)."""
    import torch
    g = ir.Graph()
    x = g.new_input(list(shape), dtype)
    r = len(shape)
    g.new_output(g.reshape(g.reduce(ir.RED_SUM, g.swap_dims(x, r - 2, r - 1), 1), list(shape[:-2]) + [shape[-1]]))
    plan = hb.Plan.pointwise(ctx, g)
    assert "dense column-sum kernel" in plan.description, plan.description
    host = O.encode(rng(19).standard_normal(shape), dtype)
    want = O.evaluate(g, [host])[0].reshape(-1).astype(np.float64)
    t = storage_to_torch(host, dtype)
    (out,) = plan.launch([t])
    torch.cuda.synchronize()
    assert O.rel_l2(out.cpu().numpy().reshape(-1).astype(np.float64), want) <= 1e-5
    pad = torch.empty(t.numel() + 8, dtype=t.dtype, device="cuda")
    shifted = pad[1:1 + t.numel()].view(t.shape)
    shifted.copy_(t)
    out2 = torch.empty_like(out)
    ws = torch.empty(plan.workspace_bytes + 256, dtype=torch.uint8, device="cuda")
    plan.launch_ptrs([shifted.data_ptr()], [out2.data_ptr()], (ws.data_ptr() + 255) // 256 * 256)
    torch.cuda.synchronize()
    assert O.rel_l2(out2.cpu().numpy().reshape(-1).astype(np.float64), want) <= 1e-5


def _random_pointwise_graph(r):
    """A random pointwise DAG over a 3-D iteration space: broadcasts of lower-rank inputs, swaps, casts,
    unary / binary / compare / select nodes, then either a store or a trailing reduction."""
    pick = lambda xs: xs[int(r.integers(0, len(xs)))]
    shape = [int(pick([1, 2, 3, 5, 8, 16, 33])) for _ in range(3)]
    g = ir.Graph()
    dts = [ir.F32, ir.BF16, ir.F16]
    vals = []
    for _ in range(int(r.integers(1, 4))):
        form = int(r.integers(0, 4))
        dt = pick(dts)
        if form == 0:
            vals.append(g.new_input(shape, dt))
        elif form == 1:      # row vector broadcast over the leading dims
            vals.append(g.broadcast_to(g.new_input([shape[2]], dt), shape))
        elif form == 2:      # tensor stored with its last two dims swapped
            vals.append(g.swap_dims(g.new_input([shape[0], shape[2], shape[1]], dt), 1, 2))
        else:                # column vector [s1, 1] broadcast along the last dim
            vals.append(g.broadcast_to(g.new_input([shape[1], 1], dt), shape))
    for _ in range(int(r.integers(2, 9))):
        kind = int(r.integers(0, 6))
        a = pick(vals)
        if kind <= 1:
            vals.append(g.unary(pick([ir.UN_RELU, ir.UN_NEG, ir.UN_TANH, ir.UN_SIGMOID, ir.UN_SIN, ir.UN_COS]), a))
        elif kind <= 3:
            vals.append(g.binary(pick([ir.BIN_ADD, ir.BIN_MUL, ir.BIN_MIN, ir.BIN_MAX, ir.BIN_SUB]), a, pick(vals)))
        elif kind == 4:
            vals.append(g.cast(a, pick(dts)))
        else:
            c = g.compare(pick([ir.CMP_LT, ir.CMP_GE, ir.CMP_NE]), a, pick(vals))
            vals.append(g.select(a, pick(vals), c))
    out = vals[-1]
    tail = int(r.integers(0, 4))
    if tail == 0:
        out = g.reduce(pick([ir.RED_SUM, ir.RED_MAX, ir.RED_MIN, ir.RED_MEAN]), out, int(r.integers(1, 4)))
    elif tail == 1:
        out = g.swap_dims(out, 0, 2)
    g.new_output(out)
    return g


@pytest.mark.parametrize("seed", range(40))
def test_random_pointwise_graphs(ctx, seed):
    r = rng(3000 + seed)
    g = _random_pointwise_graph(r)
    ins = [O.encode(r.standard_normal(g.nodes[i].shape), g.nodes[i].dtype) for i in g.inputs]
    got, plan = _run(ctx, g, ins)
    want = O.evaluate(g, ins)
    node = g.nodes[g.outputs[0]]
    a, b = O.decode(got[0], node.dtype, node.shape).reshape(-1), O.decode(want[0], node.dtype, node.shape).reshape(-1)
    tol = 1e-5 if node.dtype == ir.F32 else 1e-2
    assert np.allclose(a, b, rtol=tol, atol=tol), (float(np.abs(a - b).max()), plan.description)
