"""Seeded random op graphs for the planners: a few matmuls with pointwise chains, shared operands, transposes,
broadcast rows and column sums between them.  Everything is [S, S] bf16 (matmul results are scaled and cast back),
so any value can feed any op and magnitudes stay near one."""
from __future__ import annotations

import numpy as np

from helium_b200 import configs, ir


def random_graph(seed: int, size: int = 128, n_ops: int = 12, flavour: str = "bf16"):
    """flavour "bf16": [S, S] bf16 tensors, bf16 x bf16 -> f32 matmuls; "f32": everything f32, f32 matmuls;
    "batched": [3, S, S] bf16 tensors and batched matmuls (transposes swap the last two dims); "f16_select": f16
    tensors, f16 x f16 -> f32 matmuls, elementwise max / min and compare -> select chains."""
    r = np.random.default_rng(1000 + seed)
    g = ir.Graph()
    S = size
    dt = ir.F32 if flavour == "f32" else ir.F16 if flavour == "f16_select" else ir.BF16
    prec = ir.PREC_F32_F32 if flavour == "f32" else ir.PREC_F16_F32 if flavour == "f16_select" else ir.PREC_BF16_F32
    full = [3, S, S] if flavour == "batched" else [S, S]
    pool = [g.new_input(full, dt) for _ in range(3)]
    row = g.new_input([S], dt)
    reductions = []
    matmuls = 0
    pick = lambda: pool[int(r.integers(len(pool)))] if r.random() < 0.5 else pool[-1 - int(r.integers(min(3, len(pool))))]
    for k in range(n_ops):
        u = r.random()
        if u < 0.25 and matmuls < 3:
            a, b = pick(), pick()
            mm = g.matmul(a, b, prec)
            pool.append(g.cast(g.unary(ir.UN_MUL_CONST, mm, const=float(1.0 / np.sqrt(S))), dt))
            matmuls += 1
        elif u < 0.50:
            op = [ir.UN_RELU, ir.UN_NEG, ir.UN_TANH, ir.UN_MUL_CONST, ir.UN_ADD_CONST][int(r.integers(5))]
            pool.append(g.unary(op, pick(), const=0.5))
        elif u < 0.62 and flavour == "f16_select":
            # where(a > b, a, b * 0.5): compare -> bool tensor -> select (op.rs:422-445)
            a, b = pick(), pick()
            pool.append(g.select(g.unary(ir.UN_MUL_CONST, b, const=0.5), a, g.compare(ir.CMP_GT, a, b)))
        elif u < 0.75:
            op = [ir.BIN_ADD, ir.BIN_MUL, ir.BIN_SUB, ir.BIN_MAX, ir.BIN_MIN][int(r.integers(5 if flavour == "f16_select" else 3))]
            pool.append(g.binary(op, pick(), pick()))
        elif u < 0.85:
            pool.append(g.binary(ir.BIN_ADD, pick(), g.broadcast_to(row, full)))
        elif u < 0.93:
            pool.append(g.transpose(pick()))
        else:
            reductions.append(g.reduce_axes([ir.RED_SUM, ir.RED_MAX, ir.RED_MEAN][int(r.integers(3))] if flavour != "bf16" else ir.RED_SUM,
                                            pick(), [len(full) - 2]))
    if matmuls == 0:
        pool.append(g.cast(g.matmul(pool[-1], pool[0], prec), dt))
    outs = [pool[-1]] + reductions
    extra = pool[3 + int(r.integers(len(pool) - 3))]
    if extra not in outs:
        outs.append(extra)
    for o in outs:
        g.new_output(o)
    if flavour == "f16_select":
        ins = [(r.standard_normal(full) * 0.5).astype(np.float16) for _ in range(3)] + [(r.standard_normal(S) * 0.5).astype(np.float16)]
    elif flavour == "f32":
        ins = [(r.standard_normal(full) * 0.5).astype(np.float32) for _ in range(3)] + [(r.standard_normal(S) * 0.5).astype(np.float32)]
    else:
        ins = [configs.bf16_normal(r, tuple(full), 0.5) for _ in range(3)] + [configs.bf16_normal(r, (S,), 0.5)]
    return g, ins


def oracle_by_plan(g, ins, plan_text, evaluate):
    """Evaluates `g` the way a plan executes it: one oracle evaluation per instruction of `plan_text` (the listing
    of heh_graph_plan_text), on the stored -- rounded -- tensors that earlier instructions wrote, with everything
    inside an instruction kept unrounded, as a kernel keeps it in registers (pointwise/jit.rs:488-504).  A node
    computed in several instructions is evaluated in each.  Returns the storage arrays of the graph outputs."""
    import re
    stored = {i: a for i, a in zip(g.inputs, ins)}
    for m in re.finditer(r"tier=\d nodes=\[([\d,]*)\] in=\[([\d,]*)\] out=\[([\d,]*)\]", plan_text):
        f = lambda t: [int(v) for v in t.split(",") if v]
        nodes, reads, writes = f(m.group(1)), f(m.group(2)), f(m.group(3))
        sub = ir.Graph()
        index = {}
        for r_ in reads:
            index[r_] = sub.new_input(g.nodes[r_].shape, g.nodes[r_].dtype)
        for n in sorted(nodes):
            src = g.nodes[n]
            index[n] = sub._add(ir.Node(src.kind, src.dtype, src.shape, sub_op=src.sub_op, inputs=tuple(index[i] for i in src.inputs),
                                        const_bits=src.const_bits, axis_a=src.axis_a, axis_b=src.axis_b, axes=src.axes))
        for w in writes:
            sub.new_output(index[w])
        outs = evaluate(sub, [stored[r_] for r_ in reads])
        for w, o in zip(writes, outs):
            stored[w] = o
    return [stored[o] for o in g.outputs]
