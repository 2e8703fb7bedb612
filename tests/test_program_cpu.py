"""Validates the host-side pointwise compiler without a GPU: the program the library would run is
dumped through he_debug_dump_program, executed by the numpy emulator in helpers.py (same view
arithmetic, including the magic-number division) and compared with the oracle."""
import numpy as np
import pytest

from helpers import O, emulate_program, ir, rng
from test_oracle_golden import kat_cases


def _check(graph, inputs, tol=2e-6):
    want = O.evaluate(graph, inputs)
    got, prog = emulate_program(graph, inputs)
    for o, w, gt in zip(graph.outputs, want, got):
        node = graph.nodes[o]
        if node.dtype in (ir.BOOL, ir.U32):
            assert np.array_equal(np.asarray(w).reshape(-1), np.asarray(gt).reshape(-1))
        else:
            a = O.decode(w, node.dtype, node.shape).reshape(-1)
            b = O.decode(gt, node.dtype, node.shape).reshape(-1)
            assert np.allclose(a, b, rtol=tol, atol=tol), (np.abs(a - b).max(), prog.n_instr)
    return prog


@pytest.mark.parametrize("case", kat_cases(), ids=lambda c: c[0])
def test_program_matches_oracle_on_reference_vectors(case):
    _, _, graph, inputs, _, _ = case
    _check(graph, inputs)


def test_broadcast_swap_reshape_chain():
    g = ir.Graph()
    x = g.new_input([3, 4, 5], ir.F32)
    s = g.new_input([4], ir.F32)
    sb = g.broadcast_to(g.reshape(s, [4, 1]), [3, 4, 5])
    y = g.swap_dims(g.binary(ir.BIN_MUL, x, sb), 0, 2)          # [5,4,3]
    y = g.reshape(y, [20, 3])                                    # reshape of a permuted view
    y = g.swap_dims(y, 0, 1)                                     # [3,20]
    g.new_output(y)
    r = rng(1)
    ins = [r.standard_normal((3, 4, 5), dtype=np.float32), r.standard_normal(4, dtype=np.float32)]
    prog = _check(g, ins)
    assert prog.n_instr <= 4


def test_index_math_matches_reference_snapshot_case():
    # the graph of the reference's snapshot test (pointwise/jit.rs:752-803): bf16 [5,10,10] ^ f16 [1,10]
    g = ir.Graph()
    a = g.new_input([5, 10, 10], ir.BF16)
    b = g.new_input([1, 10], ir.F16)
    bb = g.broadcast(b, 3, [(0, 5), (1, 10)])
    g.new_output(g.binary(ir.BIN_POW, a, bb))
    r = rng(2)
    ins = [O.f32_to_bf16_bits(np.abs(r.standard_normal((5, 10, 10), dtype=np.float32)) + 0.5),
           (np.abs(r.standard_normal((1, 10), dtype=np.float32)) + 0.5).astype(np.float16)]
    _check(g, ins, tol=1e-2)  # bf16 output


def test_bool_and_u32_paths():
    g = ir.Graph()
    x = g.new_input([7, 9], ir.F32)
    y = g.new_input([7, 9], ir.F32)
    lt = g.compare(ir.CMP_LT, x, y)
    ge = g.compare(ir.CMP_GE, x, g.constant(0.0, [7, 9]))
    both = g.binary(ir.BIN_AND, lt, ge)
    g.new_output(both)
    g.new_output(g.cast(both, ir.U32))
    g.new_output(g.select(x, y, both))
    r = rng(3)
    ins = [r.standard_normal((7, 9), dtype=np.float32), r.standard_normal((7, 9), dtype=np.float32)]
    _check(g, ins)


def test_mean_reduction_scale_and_groups():
    g = ir.Graph()
    x = g.new_input([6, 5, 7], ir.BF16)
    g.new_output(g.reduce(ir.RED_MEAN, g.unary(ir.UN_EXP, x), 2))
    ins = [O.f32_to_bf16_bits(rng(4).standard_normal((6, 5, 7), dtype=np.float32))]
    prog = _check(g, ins, tol=1e-5)
    assert prog.group_size == 35 and prog.n_reductions == 1


def test_fma_contraction_is_applied_once():
    g = ir.Graph()
    x = g.new_input([64], ir.F32); s = g.new_input([64], ir.F32); b = g.new_input([64], ir.F32)
    g.new_output(g.binary(ir.BIN_ADD, g.binary(ir.BIN_MUL, x, s), b))
    r = rng(5)
    ins = [r.standard_normal(64, dtype=np.float32) for _ in range(3)]
    prog = _check(g, ins)
    ops = [prog.instr[i].op for i in range(prog.n_instr)]
    assert ops.count(6) == 1 and 3 not in ops  # one PW_FMA, no separate float binary


def test_register_reuse_keeps_footprint_small():
    g = ir.Graph()
    x = g.new_input([128], ir.F32)
    t = x
    for _ in range(40):
        t = g.unary(ir.UN_TANH, g.binary(ir.BIN_ADD, t, x))
    g.new_output(t)
    prog = _check(g, [rng(6).standard_normal(128, dtype=np.float32)], tol=1e-5)
    regs = {prog.instr[i].dst for i in range(prog.n_instr)}
    assert len(regs) <= 3


def test_c2a_graph_views():
    from helpers import graph_affine_relu_permute
    g = graph_affine_relu_permute(2, 8, 3, 5)
    r = rng(7)
    ins = [O.f32_to_bf16_bits(r.standard_normal((2, 8, 3, 5), dtype=np.float32)),
           (r.random(8, dtype=np.float32) + 0.5), r.standard_normal(8, dtype=np.float32) * 0.1]
    want = O.affine_relu_nchw_to_nhwc(ins[0], ins[1], ins[2]).reshape(-1)
    got, _ = emulate_program(g, ins)
    assert np.array_equal(got[0].reshape(-1), want)
    assert np.array_equal(O.evaluate(g, ins)[0].reshape(-1), want)
