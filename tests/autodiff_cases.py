"""The known-answer gradients of helium/tests/autodiff.rs, as op graphs.

Each case records the forward ops and the backward ops that helium's front end would append for them
(helium/src/tensor.rs: `broadcast_to` :83-142, `relu` :374-387, `max` / `min` :389-435, `pow` :344-358,
`reduce_sum` / `reduce_mean` :481-516, `reduce_min` / `reduce_max` :518-580; scalar multiplication and
`Tensor * Tensor` give `flow * other`), starting from a flow of ones.  The expected values are the
literals of the reference's assertions.  test_autodiff_cpu.py pins the oracle on them,
test_autodiff_gpu.py runs the same graphs through the host runtime on the GPU.
"""
from __future__ import annotations

import numpy as np

from helium_b200 import ir


def _f32(v):
    return np.asarray(v, dtype=np.float32)


def _ones(g, shape):
    return g.constant(1.0, shape)


def _scalar_like(g, value, shape):
    """Tensor::from_scalar(value).broadcast_to(shape): a [1] constant widened to `shape`."""
    c = g.constant(value, [1])
    return c if list(shape) == [1] else g.broadcast_to(c, shape)


def _mask_select(g, mask, true_case, false_case):
    """RawTensor::select(true_case, false_case) (helium/src/raw_tensor.rs:541-566): Op::Select{lhs: false, rhs: true}."""
    return g.select(false_case, true_case, mask)


def case_simple():
    g = ir.Graph()
    p = g.new_input([1], ir.F32)
    _ = g.binary(ir.BIN_MUL, p, _scalar_like(g, 3.0, [1]))
    flow = _ones(g, [1])
    g.new_output(g.binary(ir.BIN_MUL, flow, _scalar_like(g, 3.0, [1])))
    return "simple", "autodiff.rs:7-13", g, [_f32([2.0])], [_f32([3.0])]


def case_autodiff_scalar():
    g = ir.Graph()
    p1 = g.new_input([1], ir.F32); p2 = g.new_input([1], ir.F32); x = g.new_input([1], ir.F32)
    a = g.binary(ir.BIN_MUL, x, p1)
    two = _scalar_like(g, 2.0, [1])
    c = g.binary(ir.BIN_POW, a, two)
    _ = g.binary(ir.BIN_MUL, c, p2)
    flow = _ones(g, [1])
    g_p2 = g.binary(ir.BIN_MUL, c, flow)
    flow_c = g.binary(ir.BIN_MUL, p2, flow)
    # pow backward w.r.t. the base: b * a.pow(b - 1) * flow
    bm1 = g.binary(ir.BIN_ADD, two, g.constant(-1.0, [1]))
    flow_a = g.binary(ir.BIN_MUL, g.binary(ir.BIN_MUL, two, g.binary(ir.BIN_POW, a, bm1)), flow_c)
    g_p1 = g.binary(ir.BIN_MUL, x, flow_a)
    g.new_output(g_p1); g.new_output(g_p2)
    return "autodiff_scalar", "autodiff.rs:16-33", g, [_f32([10.0]), _f32([8.0]), _f32([2.0])], [_f32([640.0]), _f32([400.0])]


def case_reduce_sum_mean():
    g = ir.Graph()
    p = g.new_input([10], ir.F32); x = g.new_input([10], ir.F32)
    prod = g.binary(ir.BIN_MUL, x, p)
    _ = g.reduce(ir.RED_SUM, prod, 1); _ = g.reduce(ir.RED_MEAN, prod, 1)
    outs = []
    for mean in (False, True):
        flow = g.binary(ir.BIN_MUL, _ones(g, [1]), _scalar_like(g, 3.0, [1]))    # through `* 3.0`
        flow = g.broadcast_to(g.reshape(flow, [1]), [10])                          # reduce backward
        if mean:
            flow = g.binary(ir.BIN_MUL, flow, g.constant(float(np.float32(1.0) / np.float32(10.0)), [10]))
        outs.append(g.binary(ir.BIN_MUL, x, flow))                                 # through `input * param`
    for o in outs:
        g.new_output(o)
    return ("reduce_sum_mean", "autodiff.rs:36-62", g, [_f32([10.0] * 10), _f32([2.0] * 10)],
            [_f32([6.0] * 10), _f32([0.6] * 10)])


def case_broadcast():
    g = ir.Graph()
    p = g.new_input([20, 1], ir.F32); x = g.new_input([2, 20, 2], ir.F32)
    pb = g.broadcast_to(p, [2, 20, 2])
    y = g.reduce(ir.RED_SUM, g.binary(ir.BIN_MUL, pb, x), 3)
    assert g.nodes[y].shape == (1,)
    flow = g.broadcast_to(g.reshape(_ones(g, [1]), [1, 1, 1]), [2, 20, 2])         # reduce_sum backward
    flow = g.binary(ir.BIN_MUL, x, flow)                                           # w.r.t. the broadcast operand
    # broadcast_to backward: the broadcast axes (2 and the new leading axis 0) go last, are summed, and the
    # permutation is undone (tensor.rs:110-139)
    t = g.swap_dims(flow, 0, 1)                                                     # [20, 2, 2]
    t = g.reshape(g.reduce(ir.RED_SUM, t, 2), [20, 1, 1])
    t = g.swap_dims(t, 0, 1)                                                        # [1, 20, 1]
    g.new_output(g.reshape(t, [20, 1]))
    return "broadcast", "autodiff.rs:65-76", g, [_f32(np.ones((20, 1))), _f32(np.full((2, 20, 2), 2.0))], [_f32(np.full((20, 1), 8.0))]


def _reduce_extreme(which):
    g = ir.Graph()
    p = g.new_input([6], ir.F32); x = g.new_input([6], ir.F32)
    prod = g.binary(ir.BIN_MUL, p, x)
    red = ir.RED_MIN if which == "min" else ir.RED_MAX
    ext = g.broadcast_to(g.reshape(g.reduce(red, prod, 1), [1]), [6])
    mask = g.compare(ir.CMP_EQ, ext, prod)
    # the reference counts matches in F32 for min and in F16 for max (tensor.rs:535, :565)
    cnt = g.cast(mask, ir.F32 if which == "min" else ir.F16)
    num = g.broadcast_to(g.reshape(g.reduce(ir.RED_SUM, cnt, 1), [1]), [6])
    share = _mask_select(g, mask, g.unary(ir.UN_RECIP, num), g.constant(0.0, [6]))
    flow = g.binary(ir.BIN_MUL, share, g.broadcast_to(g.reshape(_ones(g, [1]), [1]), [6]))
    g.new_output(g.binary(ir.BIN_MUL, x, flow))                                    # through `param * x`
    want = [0.25, 0, 0, 0, 0, 0.25] if which == "min" else [0, 0, 1.5, 1.5, 0, 0]
    line = "autodiff.rs:79-96" if which == "min" else "autodiff.rs:99-116"
    return f"reduce_{which}", line, g, [_f32([1.0] * 6), _f32([0.5, 2.0, 3.0, 3.0, 2.0, 0.5])], [_f32(want)]


def case_relu():
    g = ir.Graph()
    p = g.new_input([4], ir.F32); x = g.new_input([4], ir.F32)
    xp = g.binary(ir.BIN_MUL, x, p)
    _ = g.reduce(ir.RED_SUM, g.unary(ir.UN_RELU, xp), 1)
    flow = g.broadcast_to(g.reshape(_ones(g, [1]), [1]), [4])
    zero, one = g.constant(0.0, [4]), g.constant(1.0, [4])
    gate = g.cast(_mask_select(g, g.compare(ir.CMP_LT, xp, zero), zero, one), ir.F32)
    flow = g.binary(ir.BIN_MUL, gate, flow)
    g.new_output(g.binary(ir.BIN_MUL, x, flow))
    return "relu", "autodiff.rs:153-160", g, [_f32([1.0, 2.0, 3.0, -4.0]), _f32([1.0, -1.0, 5.0, -10.0])], [_f32([1.0, 0.0, 5.0, -10.0])]


def _max_min(which, a_val, b_val, ga, gb, line):
    g = ir.Graph()
    a = g.new_input([1], ir.F32); b = g.new_input([1], ir.F32)
    _ = g.binary(ir.BIN_MAX if which == "max" else ir.BIN_MIN, a, b)
    flow = g.binary(ir.BIN_MUL, _ones(g, [1]), _scalar_like(g, 2.0, [1]))
    cmp_op = ir.CMP_GT if which == "max" else ir.CMP_LT

    def grad(data, other):
        ones, zeros, halves = g.constant(1.0, [1]), g.constant(0.0, [1]), g.constant(0.5, [1])
        strict = g.compare(cmp_op, data, other)
        equal = g.compare(ir.CMP_EQ, data, other)
        return g.binary(ir.BIN_MUL, _mask_select(g, strict, ones, _mask_select(g, equal, halves, zeros)), flow)

    g.new_output(grad(a, b)); g.new_output(grad(b, a))
    return f"{which}_{a_val}_{b_val}", line, g, [_f32([a_val]), _f32([b_val])], [_f32([ga]), _f32([gb])]


def cases():
    return [
        case_simple(), case_autodiff_scalar(), case_reduce_sum_mean(), case_broadcast(),
        _reduce_extreme("min"), _reduce_extreme("max"), case_relu(),
        _max_min("max", 1.5, 0.5, 2.0, 0.0, "autodiff.rs:163-171"),
        _max_min("max", -0.5, 2.5, 0.0, 2.0, "autodiff.rs:174-182"),
        _max_min("max", -0.5, -0.5, 1.0, 1.0, "autodiff.rs:185-193"),
        _max_min("min", -1.5, 0.5, 2.0, 0.0, "autodiff.rs:196-204"),
        _max_min("min", 0.5, -2.5, 0.0, 2.0, "autodiff.rs:207-215"),
        _max_min("min", -0.5, -0.5, 1.0, 1.0, "autodiff.rs:218-226"),
    ]
