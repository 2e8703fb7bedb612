"""Pointwise graphs outside the hand-written catalogue, shared by the CPU (compiles) and GPU (same bits as the
interpreter, oracle parity) tests of the plan-time specialised kernels."""
from helium_b200 import ir

UNARY = [ir.UN_RECIP, ir.UN_NEG, ir.UN_EXP, ir.UN_SIN, ir.UN_COS, ir.UN_TAN, ir.UN_SIGMOID, ir.UN_TANH, ir.UN_RELU,
         ir.UN_SQRT, ir.UN_LOG, ir.UN_GELU, ir.UN_DGELU]
BINARY = [ir.BIN_ADD, ir.BIN_MUL, ir.BIN_MIN, ir.BIN_MAX, ir.BIN_SUB, ir.BIN_DIV, ir.BIN_DRELU, ir.BIN_POW]


def _graph(shape, dts, build):
    g = ir.Graph()
    ins = [g.new_input(list(shape), d) for d in dts]
    outs = build(g, ins)
    for o in outs if isinstance(outs, (list, tuple)) else [outs]:
        g.new_output(o)
    return g


def cases(shape=(37, 24)):
    """(name, graph, positive_inputs): `positive_inputs` asks for inputs in (0.1, 3) (log, sqrt, pow, div)."""
    out = []
    for op in UNARY:
        for dt in (ir.F32, ir.BF16, ir.F16):
            # exp(x) alone would be in the catalogue's neighbourhood; chain two ops so the program is never catalogue
            out.append((f"unary{op}_{dt}", _graph(shape, [dt], lambda g, i, op=op: g.unary(ir.UN_TANH, g.unary(op, i[0]))),
                        op in (ir.UN_SQRT, ir.UN_LOG, ir.UN_RECIP)))
    for op in BINARY:
        for dts in ((ir.F32, ir.F32), (ir.BF16, ir.F32), (ir.F16, ir.BF16)):
            out.append((f"binary{op}_{dts[0]}{dts[1]}",
                        _graph(shape, dts, lambda g, i, op=op: g.unary(ir.UN_NEG, g.binary(op, i[0], i[1]))), op in (ir.BIN_DIV, ir.BIN_POW)))
    # constants, scale-and-shift chains, mul + add that the compiler contracts and ones it must not (two uses)
    def chain(g, i):
        t = g.binary(ir.BIN_MUL, i[0], i[1])
        u = g.binary(ir.BIN_ADD, t, i[2])            # contracted to one fma
        v = g.binary(ir.BIN_ADD, t, g.unary(ir.UN_MUL_CONST, u, 0.3))   # t has two uses
        return [g.unary(ir.UN_ADD_CONST, v, -1.25), g.unary(ir.UN_POW_CONST, u, 2.0), g.unary(ir.UN_POW_CONST, g.unary(ir.UN_RELU, u), 1.5)]
    out.append(("chain_f32", _graph(shape, [ir.F32] * 3, chain), False))
    out.append(("chain_bf16", _graph(shape, [ir.BF16] * 3, chain), False))
    # broadcasts: row vector, column vector, scalar; a transposing view of a second tensor
    def bcast(g, i):
        n, m = shape
        row = g.new_input([m], ir.BF16); col = g.new_input([n], ir.F32); sc = g.new_input([1], ir.F32)
        t = g.binary(ir.BIN_ADD, i[0], g.broadcast_to(row, [n, m]))
        t = g.binary(ir.BIN_MUL, t, g.broadcast_to(g.reshape(col, [n, 1]), [n, m]))
        return g.unary(ir.UN_SIGMOID, g.binary(ir.BIN_SUB, t, g.broadcast_to(sc, [n, m])))
    out.append(("broadcasts", _graph(shape, [ir.F32], bcast), False))
    def transposed(g, i):
        n, m = shape
        y = g.new_input([m, n], ir.F16)
        return g.unary(ir.UN_GELU, g.binary(ir.BIN_ADD, i[0], g.swap_dims(y, 0, 1)))
    out.append(("transposed_operand", _graph(shape, [ir.BF16], transposed), False))
    def outer_swap(g, i):
        # [4, 6, 16] read through a swap of its two outer dims plus a row vector: runs of 8 along the last dim
        x = g.new_input([6, 4, 16], ir.BF16); row = g.new_input([16], ir.F32); colv = g.new_input([4, 1, 1], ir.F16)
        t = g.binary(ir.BIN_ADD, g.swap_dims(x, 0, 1), g.broadcast_to(row, [4, 6, 16]))
        return g.unary(ir.UN_TANH, g.binary(ir.BIN_MUL, t, g.broadcast_to(colv, [4, 6, 16])))
    out.append(("outer_swap_runs", _graph(shape, [], outer_swap), False))
    # compare / select / conversions through bool and u32 values held in registers (no bool tensors in memory)
    def select(g, i):
        c = g.compare(ir.CMP_GT, i[0], i[1])
        s = g.select(i[0], i[1], c)
        return g.binary(ir.BIN_MUL, s, g.unary(ir.UN_EXP, g.unary(ir.UN_NEG, g.binary(ir.BIN_MUL, i[1], i[1]))))
    out.append(("compare_select", _graph(shape, [ir.F32, ir.F32], select), False))
    def casts(g, i):
        u = g.cast(g.unary(ir.UN_RELU, g.unary(ir.UN_MUL_CONST, i[0], 100.0)), ir.U32)
        return [g.cast(g.binary(ir.BIN_ADD, u, g.cast(g.unary(ir.UN_RELU, i[1]), ir.U32)), ir.F32), g.cast(g.cast(i[1], ir.BOOL), ir.BF16)]
    out.append(("casts", _graph(shape, [ir.F32, ir.BF16], casts), False))
    # the bench program
    out.append(("gelu_add_mul_bf16", _graph(shape, [ir.BF16] * 3, lambda g, i: g.binary(ir.BIN_MUL, g.unary(ir.UN_GELU, g.binary(ir.BIN_ADD, i[0], i[1])), i[2])), False))
    return out
