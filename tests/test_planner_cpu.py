"""Host-side planner logic that needs no GPU: symbol table of the C ABI, tier selection, catalogue
matching, permutation normalisation and error behaviour."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import helium_b200 as hb
from helium_b200 import ir
from helium_b200._lib import SIGNATURES, HeliumError, lib
from helpers import ROOT, canonical_text, graph_affine_relu_permute, graph_c3, graph_linear


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "helium_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(heh?_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations parsed"
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert declared == set(SIGNATURES), declared ^ set(SIGNATURES)


def test_no_device_is_a_loud_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(HeliumError) as e:
        hb.Context(0)
    assert "no CPU path" in str(e.value)
    plan = hb.Plan.permute(None, [4, 8], [1, 4], ir.F32)
    with pytest.raises(HeliumError) as e:
        plan.launch_ptrs([0], [0], 0, stream=0)
    assert "no CPU path" in str(e.value)


def test_permute_plans_for_benchmark_shapes():
    st = hb.permute_output_strides([4096, 4096, 8], [(1, 2), (0, 1)])
    assert st == [4096, 1, 4096 * 4096]
    d = hb.Plan.permute(None, [4096, 4096, 8], st, ir.F32).description
    assert "tile 8x512" in d and "16-byte vectors" in d
    d = hb.Plan.permute(None, [2048, 128, 128, 32], hb.permute_output_strides([2048, 128, 128, 32], [(0, 3)]), ir.F32).description
    assert "tile" in d
    # inner axis preserved -> row gather; identity -> memcpy
    assert "row gather" in hb.Plan.permute(None, [8, 16, 32], [32, 256, 1], ir.F32).description
    assert "memcpy" in hb.Plan.permute(None, [8, 16, 32], [512, 32, 1], ir.BF16).description
    assert "empty" in hb.Plan.permute(None, [8, 0, 32], [0, 32, 1], ir.BF16).description


def test_permute_rejects_non_permutation_strides():
    with pytest.raises(HeliumError):
        hb.Plan.permute(None, [4, 8], [1, 5], ir.F32)
    with pytest.raises(HeliumError):
        hb.Plan.permute(None, [4, 8], [1, 4], ir.BOOL)


def test_reference_compat_strides_reproduce_reference_unit_test():
    # helium/src/cuda/instr/permute_dims.rs:179-188
    assert hb.permute_output_strides([100, 1000], [(0, 1)], True) == [1, 100]
    assert hb.permute_output_strides([32, 64, 16, 4], [(3, 2), (2, 1)], True) == [4096, 1, 256, 64]
    assert hb.permute_output_strides([32, 64, 16, 4], [(3, 2), (2, 1)], False) == [4096, 16, 1, 1024]


def test_pointwise_tiers():
    g = graph_affine_relu_permute(64, 256, 56, 56)
    assert hb.plan_supported(g, 0) == 2
    d = hb.Plan.pointwise(None, g).description
    assert "tier 2" in d and "fused affine" in d and "tile 64x" in d
    # same graph with the multiplication operands swapped still matches
    g2 = ir.Graph()
    x = g2.new_input([4, 16, 8, 8], ir.BF16); s = g2.new_input([16], ir.BF16)
    sb = g2.broadcast_to(g2.reshape(s, [16, 1, 1]), [4, 16, 8, 8])
    g2.new_output(g2.swap_dims(g2.binary(ir.BIN_MUL, sb, x), 1, 3))
    assert hb.plan_supported(g2, 0) == 2
    # no permutation -> interpreter
    g3 = ir.Graph()
    x = g3.new_input([4, 16], ir.F32)
    g3.new_output(g3.unary(ir.UN_TANH, x))
    assert hb.plan_supported(g3, 0) == 1
    # a reduction that is not a leaf is refused (pointwise.rs:159-163)
    g4 = ir.Graph()
    x = g4.new_input([4, 16], ir.F32)
    g4.new_output(g4.unary(ir.UN_EXP, g4.reduce(ir.RED_SUM, x, 1)))
    assert hb.plan_supported(g4, 0) == 0
    # outputs of different sizes are refused (pointwise.rs:135-147)
    g5 = ir.Graph()
    x = g5.new_input([4, 16], ir.F32); y = g5.new_input([4], ir.F32)
    g5.new_output(g5.unary(ir.UN_EXP, x)); g5.new_output(g5.unary(ir.UN_EXP, y))
    assert hb.plan_supported(g5, 0) == 0


def test_permute_chain_support_query():
    g = ir.Graph()
    x = g.new_input([8, 16, 32], ir.F32)
    g.new_output(g.swap_dims(g.swap_dims(x, 1, 2), 0, 1))
    assert hb.plan_supported(g, 1) == 2
    g2 = ir.Graph()
    x = g2.new_input([8, 16], ir.F32)
    g2.new_output(g2.swap_dims(g2.unary(ir.UN_EXP, x), 0, 1))
    assert hb.plan_supported(g2, 1) == 0


def test_reduce_plan_shapes():
    g = ir.Graph()
    x = g.new_input([2, 1000, 100], ir.F32)
    g.new_output(g.reduce(ir.RED_SUM, x, 2))
    p = hb.Plan.pointwise(None, g)
    assert "CTA slices" in p.description and p.workspace_bytes > 0
    g = ir.Graph()
    x = g.new_input([256, 10], ir.F32)
    g.new_output(g.reduce(ir.RED_MAX, x, 1))
    p = hb.Plan.pointwise(None, g)
    assert "warp per group" in p.description and p.workspace_bytes == 0


def test_c3_graph_matches_the_hand_written_epilogue():
    for with_e in (False, True):
        g = graph_c3(256, 512, 128, with_e=with_e)
        assert hb.plan_supported(g, 2) == 2
        p = hb.Plan.fused_matmul(None, g)
        assert "README graph" in p.description and "mainloop 3" in p.description
        assert p.workspace_bytes >= (2 * 2 * 512 + 4) * 4
    text = canonical_text(graph_c3(256, 512, 128))
    assert text.count("red0@") == 3 and "u7(" in text and "b18f(" in text


def test_c3_match_is_insensitive_to_operand_order():
    # rebuild z1 as bias + acc and the gate product in the other order
    m, n, k = 128, 256, 64
    g = graph_c3(m, n, k)
    # swap the operands of every commutative binary op
    for node in g.nodes:
        if node.kind == ir.OP_BINARY and node.sub_op in (ir.BIN_ADD, ir.BIN_MUL):
            a, b = node.inputs
            if g.nodes[a].shape == g.nodes[b].shape and g.nodes[a].dtype == g.nodes[b].dtype:
                node.inputs = (b, a)
    assert hb.plan_supported(g, 2) == 2


@pytest.mark.parametrize("kw", [
    dict(bias=False, act=None),
    dict(bias=True, act=ir.UN_GELU, store_z=True),
    dict(bias=True, resid=True),
    dict(bias=False, resid=True, colsum="resid"),
    dict(bias=False, act=None, gate="dgelu", colsum="y"),
    dict(bias=True, act=ir.UN_RELU, a_t=True, b_t=True),
    dict(bias=False, act=None, out_dtype=ir.F32),
])
def test_flex_catalogue_matches(kw):
    g = graph_linear(256, 512, 128, **kw)
    assert hb.plan_supported(g, 2) == 2, canonical_text(g)
    p = hb.Plan.fused_matmul(None, g)
    assert "flex" in p.description
    if kw.get("a_t"):
        assert "M-major A" in p.description and "K-major B" in p.description
    else:
        assert "K-major A" in p.description and "N-major B" in p.description


def test_unmatched_epilogue_goes_to_interpreter_tier():
    g = ir.Graph()
    a = g.new_input([128, 64], ir.BF16); b = g.new_input([64, 256], ir.BF16)
    t = g.matmul(a, b)
    g.new_output(g.cast(g.unary(ir.UN_SIN, g.unary(ir.UN_EXP, t)), ir.BF16))
    assert hb.plan_supported(g, 2) == 1
    assert "interpreted epilogue" in hb.Plan.fused_matmul(None, g).description


def test_matmul_refusals():
    # K not a multiple of 8 breaks the TMA pitch rule: small problems with plain epilogues fall to the SIMT
    # kernel, anything richer or larger runs on tcgen05 over a pitch-padded copy of the operand
    g = ir.Graph()
    a = g.new_input([128, 100], ir.BF16); b = g.new_input([100, 256], ir.BF16)
    g.new_output(g.matmul(a, b))
    assert "SIMT" in hb.Plan.fused_matmul(None, g).description
    g = ir.Graph()
    a = g.new_input([128, 100], ir.BF16); b = g.new_input([100, 256], ir.BF16)
    g.new_output(g.unary(ir.UN_TANH, g.matmul(a, b)))
    plan = hb.Plan.fused_matmul(None, g)
    assert "tcgen05" in plan.description and "A copied to a 16-byte pitch" in plan.description and "B copied" not in plan.description
    assert plan.workspace_bytes >= 128 * 104 * 2
    # an operand expression runs in the kernel's mainloop when its repetition is short (small N here) ...
    g = ir.Graph()
    a = g.new_input([128, 64], ir.BF16); b = g.new_input([64, 256], ir.BF16)
    g.new_output(g.matmul(g.unary(ir.UN_EXP, a), b))
    assert hb.plan_supported(g, 2) == 2
    assert "generic mainloop rewrite" in hb.Plan.fused_matmul(None, g).description
    # ... and as a pre-pass that writes the operand once when the GEMM is long (tier 1)
    g = ir.Graph()
    a = g.new_input([4096, 4096], ir.BF16); b = g.new_input([4096, 4096], ir.BF16)
    g.new_output(g.matmul(g.unary(ir.UN_EXP, a), b))
    assert hb.plan_supported(g, 2) == 1
    assert "operand A evaluated by a pre-pass" in hb.Plan.fused_matmul(None, g).description
    # ... unless it hides a reduction or another matmul
    g = ir.Graph()
    a = g.new_input([128, 64], ir.BF16); b = g.new_input([64, 256], ir.BF16)
    g.new_output(g.matmul(g.broadcast_to(g.reduce(ir.RED_SUM, a, 1), [128, 64]), b))
    assert hb.plan_supported(g, 2) == 0
    # f32 operands use the SIMT kernel
    g = ir.Graph()
    a = g.new_input([256, 784], ir.F32); b = g.new_input([784, 512], ir.F32)
    g.new_output(g.matmul(a, b, ir.PREC_TF32_F32))
    assert "SIMT" in hb.Plan.fused_matmul(None, g).description


def test_invalid_descriptors_are_rejected_with_a_message():
    g = ir.Graph()
    x = g.new_input([4, 4], ir.F32)
    bad = g.unary(ir.UN_EXP, x)
    g.nodes[bad].shape = (4, 5)
    g.new_output(bad)
    with pytest.raises(HeliumError) as e:
        hb.Plan.pointwise(None, g)
    assert "unary output descriptor" in str(e.value)


def test_mlp_block_plans_at_full_size():
    """configs[3]: all six GEMMs of the transformer MLP block map onto hand-written tcgen05 kernels."""
    import helium_b200 as hb
    from helium_b200.mlp_block import flops_per_token, mlp_block_graphs
    graphs = mlp_block_graphs(8192, 4096, 16384)
    assert set(graphs) == {"H", "O", "dZ", "dW1", "dW2", "dX"}
    for name, g in graphs.items():
        assert hb.plan_supported(g, 2) == 2, name
        d = hb.Plan.fused_matmul(None, g).description
        assert "tcgen05" in d and "flex" in d, (name, d)
    assert "K-major B" in hb.Plan.fused_matmul(None, graphs["dZ"]).description
    assert "M-major A" in hb.Plan.fused_matmul(None, graphs["dW1"]).description
    assert flops_per_token(4096, 16384) * 8192 == 6 * 2 * 8192 * 4096 * 16384


def test_dense_elementwise_programs_are_tier_2():
    """Short dense programs hit the hand-written elementwise kernels; anything else stays on the interpreter."""
    import helium_b200 as hb
    def tier(build, dts, shape=(64, 128)):
        g = ir.Graph()
        ins = [g.new_input(list(shape), d) for d in dts]
        g.new_output(build(g, ins))
        return hb.plan_supported(g, 0)
    assert tier(lambda g, i: g.unary(ir.UN_RELU, i[0]), [ir.BF16]) == 2
    assert tier(lambda g, i: g.binary(ir.BIN_MUL, g.unary(ir.UN_RELU, i[0]), i[1]), [ir.BF16, ir.BF16]) == 2
    assert tier(lambda g, i: g.binary(ir.BIN_ADD, i[0], g.unary(ir.UN_NEG, g.binary(ir.BIN_MUL, i[1], g.constant(0.01, [64, 128])))), [ir.F32, ir.F32]) == 2
    # mixed dtypes, a broadcast operand, or an op outside the catalogue: interpreter tier
    assert tier(lambda g, i: g.binary(ir.BIN_ADD, i[0], i[1]), [ir.BF16, ir.F32]) == 1
    assert tier(lambda g, i: g.unary(ir.UN_EXP, i[0]), [ir.F32]) == 1
    g = ir.Graph()
    x = g.new_input([64, 128], ir.F32); b = g.new_input([128], ir.F32)
    g.new_output(g.binary(ir.BIN_ADD, x, g.broadcast_to(b, [64, 128])))
    assert hb.plan_supported(g, 0) == 1


def test_every_precision_setting_is_accepted_at_or_above_its_minimum():
    """helium-ir/src/opgraph/op/precision.rs:36-96: seven settings; the node's dtype is the accumulator
    type; the setting is a minimum, so the 8-bit and f16-accumulate requests plan onto the same kernels
    as the operand dtype's own setting."""
    cases = [(ir.F32, ir.PREC_F32_F32), (ir.F32, ir.PREC_TF32_F32), (ir.BF16, ir.PREC_BF16_F32), (ir.F16, ir.PREC_F16_F32),
             (ir.F16, ir.PREC_F16_F16), (ir.BF16, ir.prec_f8(ir.PREC_F8_F32, ir.F8_E4M3, ir.F8_E5M2)),
             (ir.F16, ir.prec_f8(ir.PREC_F8_F16, ir.F8_E5M2, ir.F8_E5M2)), (ir.F32, ir.prec_f8(ir.PREC_F8_F32))]
    for dt, prec in cases:
        g = ir.Graph()
        a = g.new_input([256, 512], dt); b = g.new_input([512, 384], dt)
        t = g.matmul(a, b, prec)
        assert g.nodes[t].dtype == (ir.F16 if (prec & 0xff) in (ir.PREC_F16_F16, ir.PREC_F8_F16) else ir.F32)
        g.new_output(t)
        assert hb.plan_supported(g, 2) == 2, hex(prec)
        d = hb.Plan.fused_matmul(None, g).description
        assert ("SIMT" in d) == (dt == ir.F32), d
    # accumulator type and mode bits are validated
    for bad_dtype, prec in [(ir.F32, ir.PREC_F16_F16), (ir.F16, ir.PREC_BF16_F32), (ir.F32, 7), (ir.F32, ir.PREC_BF16_F32 | (1 << 8)),
                            (ir.F32, ir.PREC_F8_F32 | (2 << 8))]:
        g = ir.Graph()
        a = g.new_input([64, 64], ir.F16); b = g.new_input([64, 64], ir.F16)
        t = g.matmul(a, b, ir.PREC_F16_F32)
        g.nodes[t].sub_op = prec
        g.nodes[t].dtype = bad_dtype
        g.new_output(t)
        with pytest.raises(HeliumError):
            hb.Plan.fused_matmul(None, g)


def test_8bit_multiplication_goes_native_from_4_gflop(monkeypatch):
    """MulF8Accum* requests: small products stay at the operand precision (the setting is a minimum), large ones
    run tcgen05 kind::f8f6f4 on 8-bit copies of the operands; the environment switch forces either."""
    def plan(m, n, k, dt=ir.BF16, prec=None):
        g = ir.Graph()
        a = g.new_input([m, k], dt); b = g.new_input([k, n], dt)
        g.new_output(g.matmul(a, b, prec if prec is not None else ir.prec_f8(ir.PREC_F8_F32, ir.F8_E4M3, ir.F8_E5M2)))
        return hb.Plan.fused_matmul(None, g)
    monkeypatch.delenv("HE_GEMM_F8", raising=False)
    big = plan(4096, 4096, 4096)
    assert "kind::f8f6f4" in big.description and "A E4M3, B E5M2" in big.description
    assert big.workspace_bytes >= 2 * 4096 * 4096
    assert "f8f6f4" not in plan(256, 256, 256).description
    assert "f8f6f4" not in plan(4096, 4096, 4096, prec=ir.PREC_BF16_F32).description
    assert "kind::f8f6f4" in plan(4096, 4096, 4096, dt=ir.F32).description
    monkeypatch.setenv("HE_GEMM_F8", "operand")
    assert "f8f6f4" not in plan(4096, 4096, 4096).description
    monkeypatch.setenv("HE_GEMM_F8", "native")
    assert "kind::f8f6f4" in plan(256, 264, 1001).description
