"""Pins the CPU oracle on the known-answer vectors of the reference's own tests.

Each case names the reference test it restates (file:line in caelunshun/helium).  The same graphs
are replayed through the CUDA library in tests/test_kat_gpu.py, so oracle and kernels are held to
the same vectors.
"""
import numpy as np
import pytest

from helpers import O, ir

F32 = ir.F32


def f32(a):
    return np.asarray(a, dtype=np.float32)


def bf16(a):
    return O.f32_to_bf16_bits(np.asarray(a, dtype=np.float32))


def f16(a):
    return np.asarray(a, dtype=np.float16)


def run(graph, inputs):
    return O.evaluate(graph, inputs)


# ---- the cases; also imported by the GPU test ------------------------------------------------------
def kat_cases():
    """Yields (name, reference location, graph, inputs, expected f32 values per output, tolerance)."""
    cases = []

    # helium/tests/tensor_ops.rs:18-26 add_simple: f32 2.0 + bf16 1.0 -> 3.0
    g = ir.Graph(); a = g.new_input([50, 2], F32); b = g.new_input([50, 2], ir.BF16)
    g.new_output(g.binary(ir.BIN_ADD, a, b))
    cases.append(("add_simple", "tensor_ops.rs:18", g, [f32(np.full((50, 2), 2.0)), bf16(np.ones((50, 2)))], [np.full(100, 3.0)], 0))

    # tensor_ops.rs:28-36 add_with_broadcast: [[3]*5]*5 + broadcast([1.0]) -> 4
    g = ir.Graph(); a = g.new_input([5, 5], F32); b = g.new_input([1], F32)
    g.new_output(g.binary(ir.BIN_ADD, a, g.broadcast_to(b, [5, 5])))
    cases.append(("add_with_broadcast", "tensor_ops.rs:28", g, [f32(np.full((5, 5), 3.0)), f32([1.0])], [np.full(25, 4.0)], 0))

    # tensor_ops.rs:38-46 multiply: 2 * bf16(3) -> 6
    g = ir.Graph(); a = g.new_input([50, 2], F32); b = g.new_input([50, 2], ir.BF16)
    g.new_output(g.binary(ir.BIN_MUL, a, b))
    cases.append(("multiply", "tensor_ops.rs:38", g, [f32(np.full((50, 2), 2.0)), bf16(np.full((50, 2), 3.0))], [np.full(100, 6.0)], 0))

    # tensor_ops.rs:48-56 divide: a / b is a * recip(b): 6 / bf16(2) -> 3
    g = ir.Graph(); a = g.new_input([50, 2], F32); b = g.new_input([50, 2], ir.BF16)
    g.new_output(g.binary(ir.BIN_MUL, a, g.unary(ir.UN_RECIP, b)))
    cases.append(("divide", "tensor_ops.rs:48", g, [f32(np.full((50, 2), 6.0)), bf16(np.full((50, 2), 2.0))], [np.full(100, 3.0)], 0))

    # tensor_ops.rs:58-66 multiply_by_scalar: x * constant(3)
    g = ir.Graph(); a = g.new_input([50, 2], F32)
    g.new_output(g.binary(ir.BIN_MUL, a, g.constant(3.0, [50, 2])))
    cases.append(("multiply_by_scalar", "tensor_ops.rs:58", g, [f32(np.full((50, 2), 2.0))], [np.full(100, 6.0)], 0))

    # tensor_ops.rs:78-85 recip
    g = ir.Graph(); a = g.new_input([50, 2], F32)
    g.new_output(g.unary(ir.UN_RECIP, a))
    cases.append(("recip", "tensor_ops.rs:78", g, [f32(np.full((50, 2), 2.0))], [np.full(100, 0.5)], 0))

    # tensor_ops.rs:87-100 complex_operation_chain: (a + b) * recip(c - d) / 2 + a = 0.4
    g = ir.Graph()
    a, b, c, d = (g.new_input([50, 2], F32) for _ in range(4))
    cd = g.binary(ir.BIN_ADD, c, g.unary(ir.UN_NEG, d))
    t = g.binary(ir.BIN_MUL, g.binary(ir.BIN_ADD, a, b), g.unary(ir.UN_RECIP, cd))
    t = g.binary(ir.BIN_MUL, t, g.unary(ir.UN_RECIP, g.constant(2.0, [50, 2])))
    g.new_output(g.binary(ir.BIN_ADD, t, a))
    ins = [f32(np.full((50, 2), v)) for v in (1.0, 2.0, 0.5, 3.0)]
    cases.append(("complex_operation_chain", "tensor_ops.rs:87", g, ins, [np.full(100, 0.4)], 1e-6))

    # tensor_ops.rs:102-111 reduce_sum: [25,4] of 10 -> all 1000; per row 40
    for tag, depth, exp in (("all", 2, np.array([1000.0])), ("rows", 1, np.full(25, 40.0))):
        g = ir.Graph(); x = g.new_input([25, 4], F32)
        g.new_output(g.reduce(ir.RED_SUM, x, depth))
        cases.append((f"reduce_sum_{tag}", "tensor_ops.rs:102", g, [f32(np.full((25, 4), 10.0))], [exp], 0))

    # tensor_ops.rs:113-122 reduce_mean
    for tag, depth, exp in (("all", 2, np.array([10.0])), ("rows", 1, np.full(25, 10.0))):
        g = ir.Graph(); x = g.new_input([25, 4], F32)
        g.new_output(g.reduce(ir.RED_MEAN, x, depth))
        cases.append((f"reduce_mean_{tag}", "tensor_ops.rs:113", g, [f32(np.full((25, 4), 10.0))], [exp], 1e-06))

    # tensor_ops.rs:124-138 reduce_max and :140-159 reduce_min on 1..12 as [3,4]
    seq = f32(np.arange(1, 13).reshape(3, 4))
    for tag, depth, exp in (("all", 2, np.array([12.0])), ("rows", 1, np.array([4.0, 8.0, 12.0]))):
        g = ir.Graph(); x = g.new_input([3, 4], F32)
        g.new_output(g.reduce(ir.RED_MAX, x, depth))
        cases.append((f"reduce_max_{tag}", "tensor_ops.rs:124", g, [seq], [exp], 0))
    for tag, depth, exp in (("all", 2, np.array([1.0])), ("rows", 1, np.array([1.0, 5.0, 9.0]))):
        g = ir.Graph(); x = g.new_input([3, 4], F32)
        g.new_output(g.reduce(ir.RED_MIN, x, depth))
        cases.append((f"reduce_min_{tag}", "tensor_ops.rs:140", g, [seq], [exp], 0))

    # tensor_ops.rs:161-174 reduce_large: [2,1000,100], first half 1.0, second half 2.0
    data = f32(np.concatenate([np.ones(100_000), np.full(100_000, 2.0)]).reshape(2, 1000, 100))
    for tag, depth, exp in (("all", 3, np.array([300_000.0])), ("rows", 2, np.array([100_000.0, 200_000.0]))):
        g = ir.Graph(); x = g.new_input([2, 1000, 100], F32)
        g.new_output(g.reduce(ir.RED_SUM, x, depth))
        cases.append((f"reduce_large_{tag}", "tensor_ops.rs:161", g, [data], [exp], 0))

    # tensor_ops.rs:320-332 broadcast: [[1],[2]] -> [2,2,4]
    g = ir.Graph(); x = g.new_input([2, 1], F32)
    g.new_output(g.broadcast_to(x, [2, 2, 4]))
    cases.append(("broadcast", "tensor_ops.rs:320", g, [f32([[1.0], [2.0]])], [np.array([1, 1, 1, 1, 2, 2, 2, 2] * 2, dtype=np.float64)], 0))

    # tensor_ops.rs:334-341 reshape
    g = ir.Graph(); x = g.new_input([4], F32)
    g.new_output(g.reshape(x, [2, 2]))
    cases.append(("reshape", "tensor_ops.rs:334", g, [f32([1, 2, 3, 4])], [np.array([1.0, 2, 3, 4])], 0))

    # tensor_ops.rs:343-359 transpose of [2,2,3]
    g = ir.Graph(); x = g.new_input([2, 2, 3], F32)
    g.new_output(g.transpose(x))
    cases.append(("transpose", "tensor_ops.rs:343", g, [f32(np.arange(1, 13).reshape(2, 2, 3))],
                  [np.array([1, 4, 2, 5, 3, 6, 7, 10, 8, 11, 9, 12], dtype=np.float64)], 0))

    # tensor_ops.rs:361-377 swap_dims(1, 2) of [2,2,2,2]
    g = ir.Graph(); x = g.new_input([2, 2, 2, 2], F32)
    g.new_output(g.swap_dims(x, 1, 2))
    cases.append(("swap_dims", "tensor_ops.rs:361", g, [f32(np.arange(1, 17).reshape(2, 2, 2, 2))],
                  [np.array([1, 2, 5, 6, 3, 4, 7, 8, 9, 10, 13, 14, 11, 12, 15, 16], dtype=np.float64)], 0))

    # tensor_ops.rs:399-403 relu
    g = ir.Graph(); x = g.new_input([4], F32)
    g.new_output(g.unary(ir.UN_RELU, x))
    cases.append(("relu", "tensor_ops.rs:399", g, [f32([-1.0, -0.5, 1.0, 0.0])], [np.array([0.0, 0.0, 1.0, 0.0])], 0))

    # tensor_ops.rs:405-410 test_2d_tensor_swap
    g = ir.Graph(); x = g.new_input([2, 3], F32)
    g.new_output(g.swap_dims(x, 0, 1))
    cases.append(("2d_swap", "tensor_ops.rs:405", g, [f32([[1, 2, 3], [4, 5, 6]])], [np.array([1.0, 4, 2, 5, 3, 6])], 0))

    # tensor_ops.rs:412-421 test_3d_tensor_swap
    cube = f32(np.arange(1, 9).reshape(2, 2, 2))
    g = ir.Graph(); x = g.new_input([2, 2, 2], F32)
    g.new_output(g.swap_dims(x, 0, 1)); g.new_output(g.swap_dims(x, 1, 2))
    cases.append(("3d_swap", "tensor_ops.rs:412", g, [cube], [np.array([1.0, 2, 5, 6, 3, 4, 7, 8]), np.array([1.0, 3, 2, 4, 5, 7, 6, 8])], 0))

    # tensor_ops.rs:423-434 test_chained_swaps: (0,1) then (1,2) then (0,2)
    g = ir.Graph(); x = g.new_input([2, 2, 2], F32)
    g.new_output(g.swap_dims(g.swap_dims(g.swap_dims(x, 0, 1), 1, 2), 0, 2))
    cases.append(("chained_swaps", "tensor_ops.rs:423", g, [cube], [np.array([1.0, 3, 2, 4, 5, 7, 6, 8])], 0))

    # tensor_ops.rs:436-442 same-dimension swap, :444-450 different sizes, :452-458 singleton
    g = ir.Graph(); x = g.new_input([2, 2, 2], F32)
    g.new_output(g.swap_dims(x, 1, 1))
    cases.append(("same_dim_swap", "tensor_ops.rs:436", g, [cube], [np.arange(1, 9, dtype=np.float64)], 0))
    g = ir.Graph(); x = g.new_input([2, 1, 3], F32)
    g.new_output(g.swap_dims(x, 1, 2))
    cases.append(("different_sized", "tensor_ops.rs:444", g, [f32(np.arange(1, 7).reshape(2, 1, 3))], [np.arange(1, 7, dtype=np.float64)], 0))
    g = ir.Graph(); x = g.new_input([1, 2, 2, 1], F32)
    g.new_output(g.swap_dims(x, 0, 3))
    cases.append(("singleton_swap", "tensor_ops.rs:452", g, [f32(np.arange(1, 5).reshape(1, 2, 2, 1))], [np.arange(1, 5, dtype=np.float64)], 0))

    # tensor_ops.rs:475-486 constant
    g = ir.Graph()
    g.new_output(g.constant(10.0, [10, 20], F32))
    cases.append(("constant_f32", "tensor_ops.rs:475", g, [], [np.full(200, 10.0)], 0))
    g = ir.Graph()
    g.new_output(g.constant(200.0, [2, 3], ir.BF16))
    cases.append(("constant_bf16", "tensor_ops.rs:482", g, [], [np.full(6, 200.0)], 0))

    # tensor_ops.rs:488-495 max, :497-503 min against constant(-1)
    g = ir.Graph(); b = g.new_input([3], F32)
    g.new_output(g.binary(ir.BIN_MAX, g.constant(-1.0, [3]), b))
    cases.append(("max", "tensor_ops.rs:488", g, [f32([-3.0, -1.0, 2.0])], [np.array([-1.0, -1.0, 2.0])], 0))
    g = ir.Graph(); b = g.new_input([3], F32)
    g.new_output(g.binary(ir.BIN_MIN, g.constant(-1.0, [3]), b))
    cases.append(("min", "tensor_ops.rs:497", g, [f32([-3.0, -1.0, 2.0])], [np.array([-3.0, -1.0, -1.0])], 0))

    # helium/tests/autodiff.rs relu backward: select(x < 0, 0, 1) * flow (tensor.rs:374-387)
    g = ir.Graph(); x = g.new_input([4], F32); flow = g.new_input([4], F32)
    neg = g.compare(ir.CMP_LT, x, g.constant(0.0, [4]))
    mask = g.select(g.constant(1.0, [4]), g.constant(0.0, [4]), neg)
    g.new_output(g.binary(ir.BIN_MUL, mask, flow))
    cases.append(("relu_backward", "tensor.rs:374", g, [f32([-1.0, 2.0, -3.0, 4.0]), f32([10.0, 20.0, 30.0, 40.0])],
                  [np.array([0.0, 20.0, 0.0, 40.0])], 0))
    return cases


def matmul_kat_cases():
    """(name, location, graph, inputs, expected, abs tolerance) for the matmul vectors."""
    cases = []
    # tensor_ops.rs:176-187 matmul_simple (operands and result transposed): 2*I x [[1,2,3],[2,4,6]]^T
    g = ir.Graph(); a = g.new_input([3, 3], F32); b = g.new_input([2, 3], F32)
    g.new_output(g.transpose(g.matmul(g.transpose(a), g.transpose(b), ir.PREC_TF32_F32)))
    cases.append(("matmul_simple", "tensor_ops.rs:176", g, [f32(2 * np.eye(3)), f32([[1, 2, 3], [2, 4, 6]])],
                  [np.array([2.0, 4, 6, 4, 8, 12])], 1e-6))
    # tensor_ops.rs:189-210 matmul_bf16: [[1,2],[3,4]]^2 = [7,10,15,22]
    g = ir.Graph(); a = g.new_input([2, 2], ir.BF16); b = g.new_input([2, 2], ir.BF16)
    g.new_output(g.matmul(a, b, ir.PREC_BF16_F32))
    m = np.array([[1.0, 2], [3, 4]])
    cases.append(("matmul_bf16", "tensor_ops.rs:189", g, [bf16(m), bf16(m)], [np.array([7.0, 10, 15, 22])], 1e-3))
    # tensor_ops.rs:212-242 matmul_f16 with transposed operands
    g = ir.Graph(); a = g.new_input([2, 3], ir.F16); b = g.new_input([3, 2], ir.F16)
    g.new_output(g.transpose(g.matmul(g.transpose(a), g.transpose(b), ir.PREC_F16_F32)))
    cases.append(("matmul_f16", "tensor_ops.rs:212", g, [f16([[1, 2, 3], [4, 5, 6]]), f16([[1, 2], [3, 4], [5, 6]])],
                  [np.array([9.0, 12, 15, 19, 26, 33, 29, 40, 51])], 1e-3))
    # tensor_ops.rs:244-252 matmul_large_matrices: ones[100,100] x 0.5[100,100] = 50
    g = ir.Graph(); a = g.new_input([100, 100], F32); b = g.new_input([100, 100], F32)
    g.new_output(g.matmul(a, b, ir.PREC_TF32_F32))
    cases.append(("matmul_large", "tensor_ops.rs:244", g, [f32(np.ones((100, 100))), f32(np.full((100, 100), 0.5))],
                  [np.full(10000, 50.0)], 1e-3))
    # tensor_ops.rs:254-318 matmul_batched (bf16, transposed operands and result)
    a0 = np.arange(1, 13, dtype=np.float64).reshape(2, 2, 3)
    b0 = np.arange(1, 13, dtype=np.float64).reshape(2, 3, 2)
    g = ir.Graph(); a = g.new_input([2, 2, 3], ir.BF16); b = g.new_input([2, 3, 2], ir.BF16)
    g.new_output(g.transpose(g.matmul(g.transpose(a), g.transpose(b), ir.PREC_BF16_F32)))
    exp = np.array([9.0, 12, 15, 19, 26, 33, 29, 40, 51, 129, 144, 159, 163, 182, 201, 197, 220, 243])
    cases.append(("matmul_batched", "tensor_ops.rs:254", g, [bf16(a0), bf16(b0)], [exp], 1e-2))
    return cases


@pytest.mark.parametrize("case", kat_cases() + matmul_kat_cases(), ids=lambda c: c[0])
def test_oracle_matches_reference_vector(case):
    name, where, graph, inputs, expected, tol = case
    outs = run(graph, inputs)
    assert len(outs) == len(expected)
    for o, storage, exp in zip(graph.outputs, outs, expected):
        node = graph.nodes[o]
        got = O.decode(storage, node.dtype, node.shape).reshape(-1)
        if tol == 0:
            assert np.array_equal(got, exp), f"{name} ({where})"
        else:
            assert np.allclose(got, exp, rtol=0, atol=tol * max(1.0, np.abs(exp).max())), f"{name} ({where})"


def test_output_strides_reference_golden():
    # helium/src/cuda/instr/permute_dims.rs:179-188
    assert O.output_strides_reference([(0, 1)], [100, 1000]) == [1, 100]
    assert O.output_strides_reference([(3, 2), (2, 1)], [32, 64, 16, 4]) == [4096, 1, 256, 64]


def test_output_strides_semantic_vs_reference():
    # self-inverse chains agree; the 3-cycle of the golden vector does not (reference yields the inverse)
    assert O.output_strides_semantic([(0, 1)], [100, 1000]) == [1, 100]
    assert O.output_strides_semantic([(3, 2), (2, 1)], [32, 64, 16, 4]) == [4096, 16, 1, 1024]
    x = np.arange(2 * 3 * 4, dtype=np.float32).reshape(2, 3, 4)
    swaps = [(1, 2), (0, 1)]
    want = np.swapaxes(np.swapaxes(x, 1, 2), 0, 1).reshape(-1)
    assert np.array_equal(O.permute(x, O.output_strides_semantic(swaps, x.shape)), want)
    inv = O.permute(x, O.output_strides_reference(swaps, x.shape))
    assert np.array_equal(inv, np.transpose(x, (1, 2, 0)).reshape(-1))  # the inverse permutation's layout


def test_bool_packing_roundtrip():
    g = np.random.default_rng(0)
    v = g.random(77) < 0.5
    w = O.pack_bools(v)
    assert w.dtype == np.uint32 and w.size == 3
    assert np.array_equal(O.unpack_bools(w, 77), v)
    assert (int(w[0]) & 1) == int(v[0])  # LSB first (pointwise/jit.rs:235-237)


def test_bf16_rounding_is_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38], dtype=np.float32)
    bits = O.f32_to_bf16_bits(x)
    back = O.bf16_bits_to_f32(bits)
    assert back[0] == 1.0
    assert back[1] == 1.0            # exactly half-way between 1.0 and 1.0078125 -> even
    assert back[2] == 1.015625       # half-way between 1.0078125 and 1.015625 -> even (odd mantissa rounds up)
    assert back[3] == -2.5


# ---- committed golden fixtures (tests/golden/golden_v1.npz, written by tests/golden/make_golden.py) ----
def golden_cases():
    import importlib.util
    import os
    here = os.path.dirname(os.path.abspath(__file__))
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(here, "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    fixtures = np.load(os.path.join(here, "golden", "golden_v1.npz"))
    return [(name, g, ins, [fixtures[f"{name}/{k}"] for k in range(len(g.outputs))]) for name, (g, ins) in mod.cases().items()]


def compare_with_golden(graph, got, want, f32_tol=1e-5, half_tol=1e-2, exact_moves=False):
    """f32 outputs: rel-L2 <= f32_tol; bf16/f16 outputs: rel-L2 <= half_tol; pure data movement: bit-exact."""
    for o, g_, w_ in zip(graph.outputs, got, want):
        node = graph.nodes[o]
        if exact_moves:
            assert np.array_equal(np.asarray(g_).reshape(-1), np.asarray(w_).reshape(-1))
            continue
        a = O.decode(g_, node.dtype, node.shape)
        b = O.decode(w_, node.dtype, node.shape)
        tol = f32_tol if node.dtype == ir.F32 else half_tol
        assert O.rel_l2(a, b) <= tol, (node.shape, O.rel_l2(a, b))


@pytest.mark.parametrize("case", golden_cases(), ids=lambda c: c[0])
def test_golden_fixtures(case):
    """The oracle reproduces its committed outputs (f64 sums may differ in the last bits between BLAS builds)."""
    name, g, ins, want = case
    got = O.evaluate(g, ins)
    compare_with_golden(g, got, want, f32_tol=1e-6, half_tol=2e-3, exact_moves=name.startswith("permute"))


def test_f8_rounding_known_answers():
    """E4M3 (bias 7, 3 mantissa bits, largest finite 448) and E5M2 (bias 15, 2 mantissa bits, largest
    finite 57344), helium-ir/src/opgraph/op/precision.rs:100-108: nearest-even, ties, subnormals,
    saturation."""
    from oracle import oracle as O
    x = np.array([0.0, 1.0, 1.0625, 1.1875, 17.0, 448.0, 500.0, -1000.0, 2.0 ** -9, 2.0 ** -10, 0.3, 3.7])
    e4 = np.array([0.0, 1.0, 1.0, 1.25, 16.0, 448.0, 448.0, -448.0, 2.0 ** -9, 0.0, 0.3125, 3.75])
    e5 = np.array([0.0, 1.0, 1.0, 1.25, 16.0, 448.0, 512.0, -1024.0, 2.0 ** -9, 2.0 ** -10, 0.3125, 3.5])
    assert np.array_equal(O.round_to_f8(x, O.F8_E4M3), e4)
    assert np.array_equal(O.round_to_f8(x, O.F8_E5M2), e5)
    assert np.array_equal(O.round_to_f8(np.array([6.0e4, 1.0e6, 2.0 ** -16, 2.0 ** -17]), O.F8_E5M2), np.array([57344.0, 57344.0, 2.0 ** -16, 0.0]))
    # every value of either format is a fixed point
    for mode in (O.F8_E4M3, O.F8_E5M2):
        g = O.round_to_f8(np.linspace(-500, 500, 20001), mode)
        assert np.array_equal(O.round_to_f8(g, mode), g)
        assert len(np.unique(g)) <= 256
