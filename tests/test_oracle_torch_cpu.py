"""Second opinion on the oracle's reading of the playground ops, from torch on the CPU.

The reference never executes Gelu, Drelu, Sub / Div, the *Constant ops, reductions inside a fused
matmul or mainloop fusion in a test, so no vector of its own pins the oracle there.  The one
independent statement of those ops in the reference is the mapping to torch expressions that
helium-playground/src/torch_synthesizer.rs:31-87 emits (`F.gelu`, `torch.tanh`, `x ** c`,
`torch.where(rhs > 0, lhs, 0)`, `sum(dim=2 | 1 | (1, 2) | (0, 1, 2), keepdim=True)`,
`torch.transpose(x, 1, 2)`, implicit broadcasts).  This file evaluates graphs with exactly that mapping
in float64 and compares every output with oracle.evaluate before its final rounding, at 1e-6.
gelu' has no torch spelling in the reference (its autodiff of Gelu is `todo!()`, autodiff.rs:63-65); it
is checked against torch.autograd's derivative of F.gelu.
"""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from helium_b200 import configs, ir
from helium_b200.mlp_block import mlp_block_graphs, mlp_block_inputs
from helpers import O

TOL = 1e-6


def torch_evaluate(graph, inputs):
    """Values (float64 tensors) of every node, computed the way torch_synthesizer.rs spells each op."""
    vals = {}
    it = iter(inputs)
    for i, n in enumerate(graph.nodes):
        shape = tuple(n.shape)
        x = [vals[j] for j in n.inputs]
        if n.kind == ir.OP_INPUT:
            v = torch.from_numpy(np.ascontiguousarray(O.decode(next(it), n.dtype, shape)))
        elif n.kind == ir.OP_CONSTANT:      # torch.full(shape, value)
            v = torch.full(shape, float(O._const_value(n.const_bits, n.dtype)), dtype=torch.float64)
        elif n.kind == ir.OP_MATMUL:        # torch.matmul(a, b)
            v = torch.matmul(x[0], x[1])
        elif n.kind == ir.OP_UNARY:
            c = float(np.array([n.const_bits], dtype=np.uint32).view(np.float32)[0])
            a = x[0]
            if n.sub_op == ir.UN_NEG: v = torch.neg(a)
            elif n.sub_op == ir.UN_RELU: v = F.relu(a)
            elif n.sub_op == ir.UN_GELU: v = F.gelu(a)
            elif n.sub_op == ir.UN_TANH: v = torch.tanh(a)
            elif n.sub_op == ir.UN_EXP: v = torch.exp(a)
            elif n.sub_op == ir.UN_LOG: v = torch.log(a)
            elif n.sub_op == ir.UN_SQRT: v = torch.sqrt(a)
            elif n.sub_op == ir.UN_ADD_CONST: v = a + c
            elif n.sub_op == ir.UN_MUL_CONST: v = a * c
            elif n.sub_op == ir.UN_POW_CONST: v = a ** c
            elif n.sub_op == ir.UN_DGELU:
                leaf = a.detach().clone().requires_grad_(True)
                (v,) = torch.autograd.grad(F.gelu(leaf).sum(), leaf)
            elif n.sub_op == ir.UN_SIGMOID: v = torch.sigmoid(a)
            elif n.sub_op == ir.UN_RECIP: v = torch.reciprocal(a)
            else: raise NotImplementedError(n.sub_op)
        elif n.kind == ir.OP_BINARY:
            a, b = x[0], x[1].reshape(x[0].shape)
            if n.sub_op == ir.BIN_ADD: v = a + b
            elif n.sub_op == ir.BIN_SUB: v = a - b
            elif n.sub_op == ir.BIN_MUL: v = a * b
            elif n.sub_op == ir.BIN_DIV: v = a / b
            elif n.sub_op == ir.BIN_POW: v = a ** b
            elif n.sub_op == ir.BIN_DRELU: v = torch.where(b > 0, a, torch.tensor(0.0, dtype=torch.float64))
            else: raise NotImplementedError(n.sub_op)
        elif n.kind == ir.OP_REDUCE:        # tensor.sum(dim=..., keepdim=True)
            assert n.sub_op == ir.RED_SUM
            dims = tuple(d for d in range(x[0].dim()) if (n.axes >> d) & 1)
            v = x[0].sum(dim=dims, keepdim=True).reshape(shape)
        elif n.kind == ir.OP_BROADCAST:     # implicit in torch
            v = x[0].reshape((1,) * (len(shape) - x[0].dim()) + tuple(x[0].shape)).expand(shape)
        elif n.kind == ir.OP_SWAP_DIMS:     # torch.transpose
            v = torch.transpose(x[0], n.axis_a, n.axis_b)
        elif n.kind == ir.OP_RESHAPE:
            v = x[0].contiguous().reshape(shape)
        elif n.kind == ir.OP_CAST:
            v = x[0]
        else:
            raise NotImplementedError(n.kind)
        vals[i] = v
    return vals


def _check(graph, inputs, what):
    _, ours = O.evaluate(graph, inputs, return_all=True)
    theirs = torch_evaluate(graph, inputs)
    for o in graph.outputs:
        a = np.asarray(ours[o], dtype=np.float64)
        b = theirs[o].detach().numpy()
        err = O.rel_l2(a, b)
        assert err <= TOL, f"{what}: output node {o} {graph.nodes[o].shape}: rel-L2 {err:.3e}"


@pytest.mark.parametrize("with_e", [False, True])
def test_readme_graph_matches_the_torch_mapping(with_e):
    m, n, k = 96, 160, 64
    _check(configs.graph_c3(m, n, k, with_e), configs.c3_inputs(m, n, k, with_e), "README graph")


def test_mlp_block_graphs_match_the_torch_mapping():
    tokens, d, ff = 64, 48, 96
    graphs = mlp_block_graphs(tokens, d, ff)
    h = mlp_block_inputs(tokens, d, ff)
    r = configs.rng(5)
    z = configs.bf16_normal(r, (tokens, ff))
    hh = configs.bf16_normal(r, (tokens, ff))
    dz = configs.bf16_normal(r, (tokens, ff))
    feeds = {"H": [h["X"], h["W1"], h["b1"]], "O": [hh, h["W2"], h["b2"], h["X"]], "dZ": [h["dO"], h["W2"], z],
             "dW1": [h["X"], dz], "dW2": [hh, h["dO"]], "dX": [dz, h["W1"], h["dO"]]}
    for name, g in graphs.items():
        _check(g, feeds[name], f"MLP block GEMM {name}")


def test_playground_only_ops_match_the_torch_mapping():
    """Sub, Div, Pow, PowConstant (2 and a non-integer exponent), AddConstant, MulConstant, Exp, Ln, Sqrt, Neg,
    Drelu and the four reduction depths, on a [2, 24, 40] tensor."""
    b, m, n = 2, 24, 40
    g = ir.Graph()
    x = g.new_input([b, m, n], ir.F32)
    y = g.new_input([b, m, n], ir.F32)
    p = g.unary(ir.UN_ADD_CONST, g.unary(ir.UN_MUL_CONST, g.unary(ir.UN_TANH, x), 0.5), 1.5)       # in [1, 2]
    outs = [
        g.binary(ir.BIN_SUB, x, y), g.binary(ir.BIN_DIV, x, p), g.binary(ir.BIN_POW, p, y),
        g.unary(ir.UN_POW_CONST, x, 2.0), g.unary(ir.UN_POW_CONST, p, 1.7), g.unary(ir.UN_EXP, g.unary(ir.UN_NEG, p)),
        g.unary(ir.UN_LOG, p), g.unary(ir.UN_SQRT, p), g.binary(ir.BIN_DRELU, x, y), g.unary(ir.UN_GELU, x),
        g.unary(ir.UN_DGELU, x),
        g.reduce_axes(ir.RED_SUM, g.binary(ir.BIN_MUL, x, y), [2]),           # Rows    -> [b, m, 1]
        g.reduce_axes(ir.RED_SUM, g.binary(ir.BIN_MUL, x, y), [1]),           # Columns -> [b, 1, n]
        g.reduce_axes(ir.RED_SUM, g.unary(ir.UN_GELU, x), [1, 2]),            # Item    -> [b, 1, 1]
        g.reduce_axes(ir.RED_SUM, g.binary(ir.BIN_DRELU, x, y), [0, 1, 2]),   # Batch   -> [1, 1, 1]
        g.transpose(g.binary(ir.BIN_SUB, x, y)),
    ]
    for o in outs:
        g.new_output(o)
    r = configs.rng(17)
    ins = [r.standard_normal((b, m, n), dtype=np.float32) for _ in range(2)]
    _check(g, ins, "playground ops")
