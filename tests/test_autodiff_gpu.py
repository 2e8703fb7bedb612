"""The known-answer gradients of helium/tests/autodiff.rs through the host runtime on the GPU: each graph
(forward ops plus the backward ops helium's front end appends, autodiff_cases.py) is planned, fused and
executed by the C++ mini-host and compared with the literals the reference asserts."""
import numpy as np
import pytest

import helium_b200 as hb
from autodiff_cases import cases
from helium_b200 import ir
from helpers import storage_to_torch, torch_to_storage

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("capture", [False, True])
@pytest.mark.parametrize("case", cases(), ids=lambda c: c[0])
def test_reference_gradients_on_the_gpu(ctx, case, capture):
    import torch
    name, where, g, ins, want = case
    tin = [storage_to_torch(a, g.nodes[i].dtype) for a, i in zip(ins, g.inputs)]
    touts = [torch.zeros(g.nodes[o].shape, dtype=torch.float32, device="cuda") for o in g.outputs]
    ex = hb.Executor(ctx, hb.HostGraph(g), tin, touts, capture=capture)
    ex.run()
    torch.cuda.synchronize()
    ctx.poll()
    for t, o, w in zip(touts, g.outputs, want):
        got = torch_to_storage(t, ir.F32).reshape(-1).astype(np.float64)
        # assert_ulps_eq! in the reference: a few f32 ulps
        assert np.allclose(got, np.asarray(w, dtype=np.float64).reshape(-1), rtol=5e-7, atol=0), (name, where, got, w)
