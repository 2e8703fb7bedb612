"""The bounded device-side waits of the tensor-core matmul kernels, made to run out on purpose.

The failure is injected on the host: `he_debug_plan_fault_injection` tells the plan's TMA producers to
stay silent and shortens the wait limit to 20 ms, so the MMA thread's first wait for operands gives up.
Nothing traps, faults or spins without bound: the kernel records the wait site, every role leaves its
loop, TMEM is freed in the normal teardown and the launch completes.  The test checks the whole chain:
launch returns HE_OK, the poll reports HE_ERR_DEVICE_TIMEOUT with the wait site, the status word is
cleared by the poll, and the same plan on the same context then computes the right result."""
import time

import numpy as np
import pytest

import helium_b200 as hb
from helium_b200 import ir
from helpers import O, bf16_normal, graph_linear, rng, storage_to_torch

pytestmark = pytest.mark.gpu

HE_ERR_DEVICE_TIMEOUT = -5


@pytest.mark.parametrize("m,n,k,kernel", [(128, 256, 64, "128x"), (512, 512, 256, "2-CTA")])
def test_operand_wait_runs_out_and_context_survives(ctx, m, n, k, kernel):
    import torch
    g = graph_linear(m, n, k, bias=False)
    r = rng(91)
    a, b = bf16_normal(r, (m, k)), bf16_normal(r, (k, n), 1.0 / np.sqrt(k))
    ins = [storage_to_torch(a, ir.BF16), storage_to_torch(b, ir.BF16)]
    plan = hb.Plan.fused_matmul(ctx, g)
    assert kernel in plan.description, plan.description
    ctx.poll()   # clean slate

    plan.fault_injection(wait_limit_us=20_000, withhold_loads=True)
    t0 = time.perf_counter()
    outs = plan.launch(ins)          # HE_OK: the failure happens on the device
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert dt < 1.0, f"the launch took {dt:.3f} s: the waits did not stop at their 20 ms limit"
    with pytest.raises(hb.HeliumError) as ei:
        ctx.poll()
    assert ei.value.status == HE_ERR_DEVICE_TIMEOUT
    # site 3 = the MMA thread waiting for a full operand stage, site 4 = an epilogue warp waiting for the
    # accumulator that those operands would have produced; both start waiting at launch and whichever
    # reaches the limit first records itself (stage / buffer 0 in both cases)
    assert "site 3 detail 0" in ei.value.message or "site 4 detail 0" in ei.value.message, ei.value.message
    ctx.poll()   # the poll cleared the status word

    plan.fault_injection(wait_limit_us=0, withhold_loads=False)
    outs = plan.launch(ins, outs)
    torch.cuda.synchronize()
    ctx.poll()
    want = O.evaluate(g, [a, b])[0]
    node = g.nodes[g.outputs[0]]
    got = outs[0].float().cpu().numpy().reshape(-1).astype(np.float64)
    assert O.rel_l2(got, O.decode(want, node.dtype, node.shape).reshape(-1)) <= 1e-2


def test_plans_without_device_waits_refuse_the_hook(ctx):
    g = ir.Graph()
    x = g.new_input([64], ir.F32)
    g.new_output(g.unary(ir.UN_RELU, x))
    plan = hb.Plan.pointwise(ctx, g)
    with pytest.raises(hb.HeliumError) as ei:
        plan.fault_injection(1000, True)
    assert ei.value.status == -2
