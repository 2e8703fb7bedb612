"""Replays the reference's known-answer vectors (see test_oracle_golden.py for file:line) through
the C ABI on the GPU."""
import numpy as np
import pytest

import helium_b200 as hb
from helium_b200 import ir
from helpers import O, storage_to_torch, torch_to_storage
from test_oracle_golden import kat_cases, matmul_kat_cases

pytestmark = pytest.mark.gpu


def _run_pointwise(ctx, graph, inputs):
    plan = hb.Plan.pointwise(ctx, graph)
    ins = [storage_to_torch(a, graph.nodes[i].dtype) for a, i in zip(inputs, graph.inputs)]
    outs = plan.launch(ins)
    import torch
    torch.cuda.synchronize()
    return [torch_to_storage(t, graph.nodes[o].dtype) for t, o in zip(outs, graph.outputs)]


@pytest.mark.parametrize("case", kat_cases(), ids=lambda c: c[0])
def test_pointwise_family_vectors(ctx, case):
    name, where, graph, inputs, expected, tol = case
    outs = _run_pointwise(ctx, graph, inputs)
    for o, storage, exp in zip(graph.outputs, outs, expected):
        node = graph.nodes[o]
        got = O.decode(storage, node.dtype, node.shape).reshape(-1)
        if tol == 0:
            assert np.array_equal(got, exp), f"{name} ({where})"
        else:
            assert np.allclose(got, exp, rtol=0, atol=tol * max(1.0, np.abs(exp).max())), f"{name} ({where})"


@pytest.mark.parametrize("case", matmul_kat_cases(), ids=lambda c: c[0])
def test_matmul_vectors(ctx, case):
    """The reference evaluates transpose(matmul(transpose(a), transpose(b))) as matmul + separate
    swap kernels; here the operand transposes fold into the matmul and the result transpose, when
    present, is a second (permute) launch."""
    import torch
    name, where, graph, inputs, expected, tol = case
    out_node = graph.outputs[0]
    last = graph.nodes[out_node]
    g2 = ir.Graph(nodes=list(graph.nodes), outputs=[])
    if last.kind == ir.OP_SWAP_DIMS:
        mm = last.inputs[0]
        g2.nodes = g2.nodes[:out_node]
        g2.outputs = [mm]
    else:
        g2.outputs = [out_node]
    plan = hb.Plan.fused_matmul(ctx, g2)
    ins = [storage_to_torch(a, graph.nodes[i].dtype) for a, i in zip(inputs, graph.inputs)]
    (c,) = plan.launch(ins)
    if last.kind == ir.OP_SWAP_DIMS:
        shp = list(g2.nodes[g2.outputs[0]].shape)
        r = len(shp)
        st = hb.permute_output_strides(shp, [(r - 2, r - 1)])
        pp = hb.Plan.permute(ctx, shp, st, ir.F32)
        (c,) = pp.launch([c])
    torch.cuda.synchronize()
    got = c.float().cpu().numpy().reshape(-1)
    assert np.allclose(got, expected[0], rtol=0, atol=tol * max(1.0, np.abs(expected[0]).max())), f"{name} ({where})"


from test_oracle_golden import compare_with_golden, golden_cases  # noqa: E402


@pytest.mark.parametrize("case", golden_cases(), ids=lambda c: c[0])
def test_golden_fixtures_on_device(ctx, case):
    """The committed golden outputs (tests/golden) through the C ABI: pointwise / permute cases as
    pointwise plans, matmul cases as fused matmul plans, the training step through the host runtime."""
    import torch
    name, g, ins, want = case
    tin = [storage_to_torch(a, g.nodes[i].dtype) for a, i in zip(ins, g.inputs)]
    if name == "mlp_train_step":
        touts = [torch.zeros(g.nodes[o].shape, dtype=torch.float32, device="cuda") for o in g.outputs]
        ex = hb.Executor(ctx, hb.HostGraph(g), tin, touts, capture=True)
        ex.run(); ex.run()
    elif any(n.kind == ir.OP_MATMUL for n in g.nodes):
        touts = hb.Plan.fused_matmul(ctx, g).launch(tin)
    else:
        touts = hb.Plan.pointwise(ctx, g).launch(tin)
    torch.cuda.synchronize()
    ctx.poll()
    got = [torch_to_storage(t, g.nodes[o].dtype) for t, o in zip(touts, g.outputs)]
    if name == "affine_relu_nhwc":
        # one f32 fma then one rounding vs the f64 oracle: double-rounding ties may differ by one ulp
        a, b = np.asarray(got[0]).reshape(-1).astype(np.int64), np.asarray(want[0]).reshape(-1).astype(np.int64)
        assert np.abs(a - b).max() <= 1 and np.mean(a != b) < 1e-3
    else:
        compare_with_golden(g, got, want, exact_moves=name.startswith("permute"))
