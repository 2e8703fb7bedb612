"""Plan-time specialised pointwise kernels on the GPU: for every program family the specialised kernel gives the
same bits as the interpreter (the tier the oracle parity tests were written against) and stays within the
oracle's tolerance; sizes with a ragged tail, a tensor that breaks the 16-byte rule (interpreter fallback), and
the bench program at a size beyond L2."""
import numpy as np
import pytest

import helium_b200 as hb
from helium_b200 import ir
from helpers import O, rng, storage_to_torch, torch_to_storage
from jit_cases import cases

pytestmark = pytest.mark.gpu

SPECIALISED = "specialised at plan time with NVRTC"


def _inputs(graph, positive, seed):
    r = rng(seed)
    ins = []
    for i in graph.inputs:
        n = graph.nodes[i]
        x = r.standard_normal(n.shape, dtype=np.float32) * 1.5
        if positive:
            x = np.abs(x) % 2.9 + 0.1
        flat = x.reshape(-1)
        if not positive and flat.size >= 8:
            flat[:8] = [0.0, -0.0, 1.0, -1.0, 1e-30, -1e30, 88.0, -104.0]   # zeros, huge, exp overflow / underflow
        ins.append(O.encode(x.astype(np.float64), n.dtype))
    return ins


def _launch(ctx, graph, ins, jit, monkeypatch):
    import torch
    if jit:
        monkeypatch.delenv("HE_PW_JIT", raising=False)
    else:
        monkeypatch.setenv("HE_PW_JIT", "0")
    plan = hb.Plan.pointwise(ctx, graph)
    tin = [storage_to_torch(a, graph.nodes[i].dtype) for a, i in zip(ins, graph.inputs)]
    outs = plan.launch(tin)
    torch.cuda.synchronize()
    ctx.poll()
    return [torch_to_storage(t, graph.nodes[o].dtype) for t, o in zip(outs, graph.outputs)], plan


ALL = cases((37, 24)) + [(n + "_ragged", g, p) for n, g, p in cases((5, 13))]


@pytest.mark.parametrize("name,graph,positive", ALL, ids=[c[0] for c in ALL])
def test_same_bits_as_the_interpreter_and_oracle_parity(ctx, monkeypatch, name, graph, positive):
    ins = _inputs(graph, positive, 5)
    got, plan = _launch(ctx, graph, ins, True, monkeypatch)
    assert SPECIALISED in plan.description
    ref, plan0 = _launch(ctx, graph, ins, False, monkeypatch)
    assert "interpreter, " in plan0.description
    for a, b in zip(got, ref):
        assert np.array_equal(np.asarray(a).view(np.uint8), np.asarray(b).view(np.uint8)), name
    want = O.evaluate(graph, ins)
    for o, g_, w_ in zip(graph.outputs, got, want):
        node = graph.nodes[o]
        a = O.decode(g_, node.dtype, node.shape).reshape(-1)
        b = O.decode(w_, node.dtype, node.shape).reshape(-1)
        tol = {ir.BF16: 1e-2, ir.F16: 2e-3, ir.F32: 2e-5}[node.dtype]
        ok = np.isfinite(b)
        assert np.allclose(a[ok], b[ok], rtol=tol, atol=tol), (name, float(np.abs(a[ok] - b[ok]).max()))


def test_unaligned_tensor_takes_the_interpreter(ctx):
    import torch
    g = ir.Graph()
    x = g.new_input([1024], ir.F32)
    g.new_output(g.unary(ir.UN_TANH, g.unary(ir.UN_EXP, x)))
    plan = hb.Plan.pointwise(ctx, g)
    assert SPECIALISED in plan.description
    base = torch.randn(1025, device="cuda")
    aligned = base[:1024].clone()
    out_a = plan.launch([aligned])[0]
    out_u = torch.empty(1024, device="cuda")
    plan.launch_ptrs([base.data_ptr() + 4], [out_u.data_ptr()])      # 4-byte offset: breaks the 16-byte rule
    out_ref = plan.launch([base[1:].clone()])[0]
    torch.cuda.synchronize()
    ctx.poll()
    assert torch.equal(out_u, out_ref)
    assert torch.allclose(out_a, torch.tanh(torch.exp(aligned)), rtol=1e-5, atol=1e-6)


def test_bench_program_beyond_l2(ctx, monkeypatch):
    """gelu(a + b) * c on 32 Mi bf16 elements: oracle parity on a sample, equality with the interpreter on all."""
    import torch
    n = 1 << 25
    g = ir.Graph()
    a, b, c = (g.new_input([n], ir.BF16) for _ in range(3))
    g.new_output(g.binary(ir.BIN_MUL, g.unary(ir.UN_GELU, g.binary(ir.BIN_ADD, a, b)), c))
    tin = [torch.randn(n, device="cuda").bfloat16() for _ in range(3)]
    plan = hb.Plan.pointwise(ctx, g)
    assert SPECIALISED in plan.description
    out = plan.launch(tin)[0]
    monkeypatch.setenv("HE_PW_JIT", "0")
    out0 = hb.Plan.pointwise(ctx, g).launch(tin)[0]
    torch.cuda.synchronize()
    ctx.poll()
    assert torch.equal(out.view(torch.int16), out0.view(torch.int16))
    f = [t[:4096].double() for t in tin]
    want = torch.nn.functional.gelu(f[0] + f[1]) * f[2]
    assert torch.allclose(out[:4096].double(), want, rtol=1e-2, atol=1e-2)


def _reduce_graph(shape, depth, dt, column=False):
    g = ir.Graph()
    a = g.new_input(list(shape), dt); b = g.new_input(list(shape), dt)
    t = g.binary(ir.BIN_MUL, g.unary(ir.UN_TANH, a), b)
    if column:
        t = g.swap_dims(t, 0, 1)
    g.new_output(g.reduce(ir.RED_SUM, t, depth))
    g.new_output(g.reduce(ir.RED_MAX, t, depth))
    g.new_output(g.reduce(ir.RED_MEAN, g.unary(ir.UN_RELU, t), depth))
    return g


@pytest.mark.parametrize("shape,depth,column", [((256, 10), 1, False), ((3, 70001), 1, False), ((64, 33, 7), 2, False),
                                                ((1 << 20,), 1, False), ((1000, 96), 1, True), ((37, 5), 2, False)],
                         ids=["warp_per_group", "cta_slices_multi", "cta_slices_one", "one_group", "column_mode", "tiny"])
@pytest.mark.parametrize("dt", [ir.F32, ir.BF16])
def test_reductions_with_prologues(ctx, monkeypatch, shape, depth, column, dt):
    """Reductions over a pointwise prologue: the specialised reduction kernel walks and combines exactly like the
    interpreter's (same bits, every launch mode), and both sit within the oracle's f32 tolerance."""
    g = _reduce_graph(shape, depth, dt, column)
    ins = _inputs(g, False, 9)
    got, plan = _launch(ctx, g, ins, True, monkeypatch)
    assert SPECIALISED in plan.description, plan.description
    ref, plan0 = _launch(ctx, g, ins, False, monkeypatch)
    assert "interpreter" in plan0.description
    for a, b in zip(got, ref):
        assert np.array_equal(np.asarray(a).view(np.uint8), np.asarray(b).view(np.uint8))
    want = O.evaluate(g, ins)
    for o, g_, w_ in zip(g.outputs, got, want):
        node = g.nodes[o]
        a = O.decode(g_, node.dtype, node.shape).reshape(-1)
        b = O.decode(w_, node.dtype, node.shape).reshape(-1)
        assert np.allclose(a, b, rtol=2e-5, atol=2e-5 * max(1.0, float(np.abs(b).max()))), float(np.abs(a - b).max())
