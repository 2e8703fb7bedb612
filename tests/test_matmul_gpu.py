"""Fused matmul (tcgen05 core, mainloop + epilogue fusion, SIMT fallback) against the oracle.

Tolerances (the path's stated bar): rel-L2 <= 1e-2 for bf16/f16 outputs, <= 1e-5 for f32 outputs
of contractions and reductions, measured against the f64 oracle on the same input bits."""
import numpy as np
import pytest

import helium_b200 as hb
from helium_b200 import ir
from helpers import (O, bf16_bernoulli, bf16_normal, graph_c3, graph_linear, rng, storage_to_torch, torch_to_storage)

pytestmark = pytest.mark.gpu

TOL = {ir.BF16: 1e-2, ir.F16: 1e-2, ir.F32: 1e-5}


def _run(ctx, graph, inputs):
    import torch
    plan = hb.Plan.fused_matmul(ctx, graph)
    ins = [storage_to_torch(a, graph.nodes[i].dtype) for a, i in zip(inputs, graph.inputs)]
    outs = plan.launch(ins)
    torch.cuda.synchronize()
    ctx.poll()  # a bounded wait that gave up would surface here as HE_ERR_DEVICE_TIMEOUT
    return [torch_to_storage(t, graph.nodes[o].dtype) for t, o in zip(outs, graph.outputs)], plan


def _gen(graph, seed, scale=None):
    r = rng(seed)
    ins = []
    for k, i in enumerate(graph.inputs):
        n = graph.nodes[i]
        std = 1.0 if scale is None else scale.get(k, 1.0)
        v = r.standard_normal(n.shape, dtype=np.float32) * np.float32(std)
        ins.append(O.encode(v.astype(np.float64), n.dtype))
    return ins


def _compare(graph, got, want, desc):
    for o, g_, w_ in zip(graph.outputs, got, want):
        node = graph.nodes[o]
        a = O.decode(g_, node.dtype, node.shape)
        b = O.decode(w_, node.dtype, node.shape)
        err = O.rel_l2(a, b)
        assert err <= TOL[node.dtype], f"rel-L2 {err:.3e} > {TOL[node.dtype]} for output {o} {node.shape}: {desc}"


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 512), (256, 512, 128), (384, 768, 320),
                                   (200, 264, 136), (8, 8, 8), (1000, 40, 72), (136, 1000, 4096)])
@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, False), (True, True)])
def test_plain_matmul_bf16(ctx, m, n, k, a_t, b_t):
    g = graph_linear(m, n, k, bias=False, a_t=a_t, b_t=b_t, out_dtype=ir.F32)
    ins = _gen(g, 21, {1: 1.0 / np.sqrt(k)})
    got, plan = _run(ctx, g, ins)
    assert "tcgen05" in plan.description
    _compare(g, got, O.evaluate(g, ins), plan.description)


def test_matmul_f16_and_bf16_outputs(ctx):
    for dt in (ir.F16, ir.BF16):
        g = graph_linear(256, 256, 256, bias=True, act=ir.UN_RELU, dtype=dt)
        ins = _gen(g, 22, {1: 1 / 16.0})
        got, plan = _run(ctx, g, ins)
        _compare(g, got, O.evaluate(g, ins), plan.description)


def test_batched_matmul(ctx):
    g = graph_linear(136, 264, 72, bias=False, batch=3, out_dtype=ir.F32)
    ins = _gen(g, 23, {1: 1 / 8.0})
    got, plan = _run(ctx, g, ins)
    _compare(g, got, O.evaluate(g, ins), plan.description)


@pytest.mark.parametrize("kw", [
    dict(bias=True, act=ir.UN_GELU, store_z=True),                 # config 4 forward GEMM 1
    dict(bias=True, resid=True),                                   # config 4 forward GEMM 2
    dict(bias=False, resid=True, colsum="resid"),                  # dX = dZ W1^T + dOut, db2 = colsum(dOut)
    dict(bias=False, gate="dgelu", colsum="y", b_t=True),          # dZ = (dOut W2^T) * gelu'(Z), db1 = colsum(dZ)
    dict(bias=False, a_t=True),                                    # dW = X^T dZ
    dict(bias=True, act=ir.UN_TANH, gate="mul"),
    dict(bias=False, act=None, gate="drelu", out_dtype=ir.F32),
])
@pytest.mark.parametrize("m,n,k", [(256, 512, 192), (200, 136, 64)])
def test_flex_epilogues(ctx, kw, m, n, k):
    g = graph_linear(m, n, k, **kw)
    ins = _gen(g, 24, {1: 1.0 / np.sqrt(k)})
    got, plan = _run(ctx, g, ins)
    assert "flex" in plan.description
    _compare(g, got, O.evaluate(g, ins), plan.description)
    got2, _ = _run(ctx, g, ins)
    for x, y in zip(got, got2):
        assert np.array_equal(x, y), "results must be bit-stable across launches"


def test_mainloop_relu_mask(ctx):
    for (m, n, k) in [(128, 256, 64), (256, 264, 200), (512, 512, 1024)]:
        g = ir.Graph()
        a = g.new_input([m, k], ir.BF16); mk = g.new_input([m, k], ir.BF16); b = g.new_input([k, n], ir.BF16)
        g.new_output(g.matmul(g.binary(ir.BIN_MUL, g.unary(ir.UN_RELU, a), mk), b))
        r = rng(25)
        ins = [bf16_normal(r, (m, k)), bf16_bernoulli(r, (m, k)), bf16_normal(r, (k, n), 1 / np.sqrt(k))]
        got, plan = _run(ctx, g, ins)
        assert "mainloop 3" in plan.description
        _compare(g, got, O.evaluate(g, ins), plan.description)


from helpers import c3_inputs as _c3_inputs  # noqa: E402


@pytest.mark.parametrize("m,n,k,with_e", [(128, 256, 64, False), (256, 512, 128, False), (384, 520, 200, True), (1024, 1024, 1024, False)])
def test_readme_graph(ctx, m, n, k, with_e):
    g = graph_c3(m, n, k, with_e)
    ins = _c3_inputs(m, n, k, with_e)
    got, plan = _run(ctx, g, ins)
    assert "README graph" in plan.description
    _compare(g, got, O.evaluate(g, ins), plan.description)
    got2, _ = _run(ctx, g, ins)
    for x, y in zip(got, got2):
        assert np.array_equal(x, y), "reductions must be bit-stable across launches"


def test_readme_graph_with_saturating_biases(ctx):
    """The README epilogue where tanh saturates and relu switches: the product is zero (A = 0) and b1 / b2
    carry zeros of both signs, tiny values, the bulk and +-3 ... +-200, so z1 = b1 and t = tanh(b2) exactly
    as the oracle sees them."""
    m, n, k = 256, 512, 128
    g = graph_c3(m, n, k, False)
    ins = _c3_inputs(m, n, k, False)
    vals = np.array([0.0, -0.0, 1e-20, -1e-20, 0.01, -0.01, 0.5, -0.5, 1.0, -1.0, 3.0, -3.0, 8.0, -8.0, 12.0, -12.0,
                     45.0, -45.0, 90.0, -90.0, 200.0, -200.0, 0.25, -0.25], dtype=np.float64)
    ins[0] = O.encode(np.zeros((1, m, k)), ir.BF16)
    ins[3] = O.encode(np.resize(vals, (1, 1, n)), ir.BF16)
    ins[4] = O.encode(np.resize(np.roll(vals, 5), (1, 1, n)), ir.BF16)
    got, plan = _run(ctx, g, ins)
    assert "README graph" in plan.description
    _compare(g, got, O.evaluate(g, ins), plan.description)


def _readme_oracle_full(ins, m, n):
    """Every row of the README graph through the C oracle (bf16 products, f32 accumulate, the epilogue in
    f32 as the graph spells it, sums in f64): (loss, db2, db1, gt bits, gz1 bits, z1)."""
    from oracle import oracle_c as OC
    a, mk_ml, b, b1, b2, mk, y = [x.reshape(x.shape[-2], x.shape[-1]) for x in ins]
    acc = OC.gemm_bf16(a, b, mk_ml, 0, m)
    out = OC.c3_epilogue(acc, mk, y, b1.reshape(-1), b2.reshape(-1), 1.0 / n, 0, m)
    acc += O.bf16_bits_to_f32(b1.reshape(1, -1))     # z1 = C + b1, the argument of the relu switch
    return out + (acc,)


def _check_readme_outputs(got, ref, ins, m, n, what):
    loss, db2, db1, gt, gz1 = got
    l_ref, db2_ref, db1_ref, gt_ref, gz_ref, z1 = ref
    dec = lambda bits: O.bf16_bits_to_f32(np.asarray(bits).reshape(m, n)).astype(np.float64)
    for name, mine, want in (("gt", gt, gt_ref), ("gz1", gz1, gz_ref)):
        err = O.rel_l2(dec(mine), dec(want))
        assert err <= 1e-2, f"{what}: {name} rel-L2 {err:.3e}"
    # DB1 sums gz1 = (z1 > 0 ? gu : 0), which jumps at z1 = 0.  Two f32 accumulations of the same 4096-term dot
    # product differ by ~1e-6, so among 16.7 M elements a handful with |z1| below that may legally switch the
    # other way, each moving one column sum by a whole element (~3e-4 of the vector's norm).  Those elements
    # are identified from the oracle's z1; for them the kernel's stored value must be one of the two legal
    # outcomes (0, or the oracle's value had the switch been on), and the reference sum takes the kernel's
    # choice.  Everything else is compared as is.
    amb = np.argwhere(np.abs(z1) <= 4e-6 * max(1.0, float(np.abs(z1).max())))
    assert len(amb) <= max(64, int(1e-4 * m * n)), f"{what}: {len(amb)} elements next to the relu switch"
    db1_ref = np.array(db1_ref, dtype=np.float64)
    gz_mine, gz_want = dec(gz1), dec(gz_ref)
    b1v, b2v = [O.bf16_bits_to_f32(ins[k].reshape(-1)).astype(np.float64) for k in (3, 4)]
    mkv, yv = [O.bf16_bits_to_f32(ins[k].reshape(m, n)) for k in (5, 6)]
    for i, j in amb:
        # u ~ 0 here, so d = mask - y and the switched-on value is g * (t - mask)
        t = np.tanh(float(z1[i, j]) - b1v[j] + b2v[j])
        on = (float(mkv[i, j]) - float(yv[i, j])) * 2.0 / n * (t - float(mkv[i, j]))
        assert gz_mine[i, j] == 0.0 or abs(gz_mine[i, j] - on) <= 1e-2 * abs(on) + 1e-12, (what, i, j, gz_mine[i, j], on)
        db1_ref[j] += gz_mine[i, j] - gz_want[i, j]
    # the three reductions against the oracle's own f64 sums, at the f32 tolerance
    for name, mine, want in (("DB2", db2, db2_ref), ("DB1", db1, db1_ref), ("LOSS", loss, np.array([l_ref]))):
        err = O.rel_l2(np.asarray(mine, dtype=np.float64).reshape(-1), np.asarray(want, dtype=np.float64).reshape(-1))
        assert err <= 1e-5, f"{what}: {name} rel-L2 {err:.3e} ({len(amb)} elements next to the relu switch)"


def test_readme_graph_full_size_against_c_oracle(ctx):
    """The README fused matmul at its benchmark size, 4096^3: ALL rows go through the C oracle (the numpy
    oracle would take minutes); both stored tiles are compared over the whole matrix at 1e-2, and LOSS, DB1,
    DB2 against the oracle's f64 sums at 1e-5."""
    m = n = k = 4096
    g = graph_c3(m, n, k, False)
    ins = _c3_inputs(m, n, k, False)
    got, plan = _run(ctx, g, ins)
    _check_readme_outputs(got, _readme_oracle_full(ins, m, n), ins, m, n, plan.description)


@pytest.mark.parametrize("m,n,k,repeats", [(4096, 4096, 4096, 50), (8192, 512, 4096, 20)])
def test_in_kernel_mainloop_fusion_at_scale(ctx, monkeypatch, m, n, k, repeats):
    """The in-kernel mainloop rewrite (transform warps of both CTAs of a pair hand their tiles to the leader's
    MMA thread through a cluster-remote mbarrier arrive) forced on at sizes where the planner would
    materialise instead: parity against the C oracle on every row, then repeated launches that must give
    the same bits every time -- a lost or early hand-off would show up as a changed tile."""
    import torch
    monkeypatch.setenv("HE_GEMM_MAINLOOP", "fused")   # read at plan time
    g = graph_c3(m, n, k, False)
    ins = _c3_inputs(m, n, k, False)
    plan = hb.Plan.fused_matmul(ctx, g)
    assert "mainloop rewrite in shared memory" in plan.description, plan.description
    t_ins = [storage_to_torch(a, g.nodes[i].dtype) for a, i in zip(ins, g.inputs)]
    outs = plan.launch(t_ins)
    torch.cuda.synchronize()
    ctx.poll()
    first = [t.clone() for t in outs]
    got = [torch_to_storage(t, g.nodes[o].dtype) for t, o in zip(outs, g.outputs)]
    _check_readme_outputs(got, _readme_oracle_full(ins, m, n), ins, m, n, plan.description)
    for it in range(repeats):
        plan.launch(t_ins, outs)
        if it % 10 == 9:
            for a, b in zip(first, outs):
                assert torch.equal(a.view(torch.int32) if a.dtype == torch.float32 else a.view(torch.int16),
                                   b.view(torch.int32) if b.dtype == torch.float32 else b.view(torch.int16)), f"launch {it + 1} changed a result"
    torch.cuda.synchronize()
    ctx.poll()
    for a, b in zip(first, outs):
        assert torch.equal(a.view(torch.int32) if a.dtype == torch.float32 else a.view(torch.int16),
                           b.view(torch.int32) if b.dtype == torch.float32 else b.view(torch.int16))


def test_interpreted_epilogue(ctx):
    for (m, n, k) in [(128, 256, 64), (200, 264, 136)]:
        g = ir.Graph()
        a = g.new_input([m, k], ir.BF16); b = g.new_input([k, n], ir.BF16); s = g.new_input([m, 1], ir.F32)
        t = g.matmul(a, b)
        t = g.binary(ir.BIN_MUL, g.unary(ir.UN_SIN, t), g.broadcast_to(s, [m, n]))
        g.new_output(g.cast(t, ir.BF16))
        g.new_output(g.unary(ir.UN_SIGMOID, t))
        ins = _gen(g, 26, {1: 1.0 / np.sqrt(k)})
        got, plan = _run(ctx, g, ins)
        assert "interpreted" in plan.description
        _compare(g, got, O.evaluate(g, ins), plan.description)


def test_simt_paths(ctx):
    # f32 operands (config 1 shapes), and bf16 shapes that break the TMA pitch rule (4097-style)
    for (m, n, k, dt, bias, act) in [(256, 512, 784, ir.F32, True, ir.UN_RELU), (256, 10, 512, ir.F32, True, None),
                                     (129, 257, 131, ir.BF16, False, None), (2, 2, 2, ir.BF16, False, None)]:
        g = graph_linear(m, n, k, bias=bias, act=act, dtype=dt, out_dtype=ir.F32)
        ins = _gen(g, 27, {1: 1.0 / np.sqrt(k)})
        got, plan = _run(ctx, g, ins)
        assert "SIMT" in plan.description
        _compare(g, got, O.evaluate(g, ins), plan.description)


@pytest.mark.parametrize("dt,out_dt", [(ir.BF16, ir.BF16), (ir.BF16, ir.F32), (ir.F16, ir.F16), (ir.F16, ir.F32)])
def test_matmul_4097_cubed_stays_on_the_tensor_cores(ctx, dt, out_dt):
    """The shape and the acceptance rule of the reference's own GEMM test (helium-kernel-generator/tests/
    matmul.rs:160-190: 4097 x 4097 x 4097, entries uniform in [0, 1); per element |expected - actual| <= 1e-3 or
    relative error <= 1e-2, matmul.rs:140-147).  No row pitch here is a multiple of 16 bytes, so both operands
    go through the pitch-padding copy and the product still runs on tcgen05.  320 rows (the last one, which
    sits alone in its tile, among them) are checked against a float64 product of the same input bits."""
    n = 4097
    g = graph_linear(n, n, n, bias=False, dtype=dt, out_dtype=out_dt)
    r = rng(4097)
    ins = [O.encode(r.random((n, n), dtype=np.float32).astype(np.float64), dt) for _ in range(2)]
    got, plan = _run(ctx, g, ins)
    assert "tcgen05" in plan.description and "copied to a 16-byte pitch" in plan.description, plan.description
    rows = np.unique(np.concatenate([r.choice(n, 319, replace=False), [n - 1]]))
    a = O.decode(ins[0], dt, (n, n))[rows]
    want = a @ O.decode(ins[1], dt, (n, n))
    mine = O.decode(got[0], out_dt, (n, n))[rows]
    bad = ~((np.abs(mine - want) <= 1e-3) | (np.abs(mine - want) <= 1e-2 * np.maximum(np.abs(mine), np.abs(want))))
    assert not bad.any(), (int(bad.sum()), plan.description)
    # With all-positive entries the rounding errors of the 4097 f32 accumulation steps do not cancel (the tensor
    # core's accumulator rounds towards zero), which leaves a relative bias of ~1e-5 in f32 outputs; the
    # reference's own criterion for this test is the per-element one above.
    err = O.rel_l2(mine, want)
    assert err <= (1e-4 if out_dt == ir.F32 else 1e-2), (err, plan.description)


def test_odd_pitches_with_fused_epilogues(ctx):
    """Ragged operands with epilogues beyond what the SIMT kernel offers (these were refused before the
    pitch-padding copy existed): bias + GELU with the pre-activation kept, and a gated column sum."""
    for kw in (dict(bias=True, act=ir.UN_GELU, store_z=True), dict(bias=False, gate="dgelu", colsum="y", b_t=True),
               dict(bias=False, a_t=True, resid=True)):
        m, n, k = 1029, 517, 1003
        g = graph_linear(m, n, k, **kw)
        ins = _gen(g, 77, {1: 1.0 / np.sqrt(k)})
        got, plan = _run(ctx, g, ins)
        assert "tcgen05" in plan.description and "16-byte pitch" in plan.description, plan.description
        _compare(g, got, O.evaluate(g, ins), plan.description)


def test_simt_scale_accumulate_epilogues(ctx):
    """The SGD update of a weight gradient, w + (-(g * lr)) (helium/src/optimizer/sgd.rs), and the
    partial forms greedy fusion passes through, as epilogues of the f32 SIMT kernel (with and without
    the cluster split of K)."""
    for (m, n, k) in [(784, 512, 256), (512, 10, 256), (70, 33, 19)]:
        for form in range(5):
            g = ir.Graph()
            a = g.new_input([k, m], ir.F32); b = g.new_input([k, n], ir.F32)
            w = g.new_input([m, n], ir.F32); s = g.new_input([m, n], ir.F32)
            t = g.matmul(g.transpose(a), b, ir.PREC_TF32_F32)
            t = g.binary(ir.BIN_MUL, t, s if form == 0 else g.constant(0.01, [m, n]))
            if form in (2, 3):
                t = g.unary(ir.UN_NEG, t)
            if form in (3, 4):
                t = g.binary(ir.BIN_ADD, w, t)
            g.new_output(t)
            ins = _gen(g, 61 + form, {1: 1.0 / np.sqrt(k)})
            got, plan = _run(ctx, g, ins)
            assert "SIMT" in plan.description and "scale/accumulate" in plan.description
            _compare(g, got, O.evaluate(g, ins), plan.description)


def test_low_precision_requests_are_served_at_or_above_their_minimum(ctx):
    """MulF16AccumF16 and MulF8Accum{F32,F16} (helium-ir/src/opgraph/op/precision.rs:56-81).  The setting
    is a minimum (precision.rs:3-9): the product is taken at the operand dtype with f32 accumulation, so
    the result must match the operand-precision oracle to the usual tolerance, and must be closer to it
    than the narrowest legal reading (operands rounded to their F8Mode) is."""
    for dt, prec, epi in [(ir.F16, ir.PREC_F16_F16, False), (ir.F16, ir.PREC_F16_F16, True),
                          (ir.BF16, ir.prec_f8(ir.PREC_F8_F32, ir.F8_E4M3, ir.F8_E5M2), False),
                          (ir.BF16, ir.prec_f8(ir.PREC_F8_F32, ir.F8_E4M3, ir.F8_E4M3), True),
                          (ir.F16, ir.prec_f8(ir.PREC_F8_F16, ir.F8_E5M2, ir.F8_E4M3), False),
                          (ir.F32, ir.prec_f8(ir.PREC_F8_F32), False)]:
        m, n, k = 264, 392, 520
        g = ir.Graph()
        a = g.new_input([m, k], dt); b = g.new_input([k, n], dt); bias = g.new_input([n], ir.F32)
        t = g.matmul(a, b, prec)
        if epi:
            t = g.cast(g.unary(ir.UN_RELU, g.binary(ir.BIN_ADD, t, g.broadcast_to(bias, [m, n]))), dt)
        g.new_output(t)
        ins = _gen(g, 71, {1: 1.0 / np.sqrt(k)})
        got, plan = _run(ctx, g, ins)
        want = O.evaluate(g, ins)
        _compare(g, got, want, plan.description)
        if (prec & 0xff) in (ir.PREC_F8_F32, ir.PREC_F8_F16):
            node = g.nodes[g.outputs[0]]
            dec = lambda x: O.decode(x, node.dtype, node.shape)
            narrow = O.evaluate(g, ins, f8_quantise=True)
            assert O.rel_l2(dec(got[0]), dec(want[0])) < 0.1 * O.rel_l2(dec(narrow[0]), dec(want[0])), plan.description


@pytest.mark.parametrize("dt", [ir.BF16, ir.F16, ir.F32])
@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
def test_native_8bit_multiplication(ctx, monkeypatch, dt, ta, tb):
    """MulF8AccumF32 served by tcgen05 kind::f8f6f4 (forced at a test size): both operands are rounded to their
    F8Mode once, products of 8-bit floats are exact in f32, so the result must match the oracle's narrowest legal
    reading (operands rounded to E4M3 / E5M2, f64 accumulation) to f32 accumulation error -- and it must NOT match
    the operand-precision reading.  All four operand layouts, a batch, K off every vector rule, saturating values,
    a fused bias + relu epilogue."""
    monkeypatch.setenv("HE_GEMM_F8", "native")
    bt, m, n, k = 2, 264, 392, 1000 + (1 if dt == ir.F32 else 0)
    for ma, mb, epi in [(ir.F8_E4M3, ir.F8_E4M3, False), (ir.F8_E5M2, ir.F8_E4M3, True), (ir.F8_E4M3, ir.F8_E5M2, False)]:
        g = ir.Graph()
        a = g.new_input([bt, k, m] if ta else [bt, m, k], dt)
        b = g.new_input([bt, n, k] if tb else [bt, k, n], dt)
        bias = g.new_input([n], ir.F32)
        t = g.matmul(g.swap_dims(a, 1, 2) if ta else a, g.swap_dims(b, 1, 2) if tb else b, ir.prec_f8(ir.PREC_F8_F32, ma, mb))
        if epi:
            t = g.unary(ir.UN_RELU, g.binary(ir.BIN_ADD, t, g.broadcast_to(bias, [bt, m, n])))
        g.new_output(t)
        ins = _gen(g, 91, {})
        # a few values beyond both formats' ranges and below their subnormals
        av = O.decode(ins[0], dt, g.nodes[g.inputs[0]].shape).copy()
        av.reshape(-1)[:6] = [500.0, -6.0e4, 6.2e4, 2.0 ** -10, -2.0 ** -17, 0.0]
        ins[0] = O.encode(av, dt)
        got, plan = _run(ctx, g, ins)
        assert "kind::f8f6f4" in plan.description, plan.description
        node = g.nodes[g.outputs[0]]
        dec = lambda x: O.decode(x, node.dtype, node.shape)
        narrow = O.evaluate(g, ins, f8_quantise=True)
        wide = O.evaluate(g, ins)
        err = O.rel_l2(dec(got[0]), dec(narrow[0]))
        assert err <= 2e-6, (err, plan.description)
        assert O.rel_l2(dec(got[0]), dec(wide[0])) > 1e-3


@pytest.mark.parametrize("m", [100, 392])
def test_native_8bit_with_other_epilogue_tiers(ctx, monkeypatch, m):
    """The 8-bit mainloop under the interpreted epilogue tier (an op outside the catalogue plus a row reduction), on
    the single-CTA kernel (one row tile) and on the CTA-pair kernel."""
    monkeypatch.setenv("HE_GEMM_F8", "native")
    n, k = 264, 520
    g = ir.Graph()
    a = g.new_input([m, k], ir.BF16); b = g.new_input([k, n], ir.BF16)
    t = g.unary(ir.UN_SIN, g.unary(ir.UN_MUL_CONST, g.matmul(a, b, ir.prec_f8(ir.PREC_F8_F32, ir.F8_E4M3, ir.F8_E4M3)), 0.05))
    g.new_output(t)
    g.new_output(g.reduce(ir.RED_SUM, t, 1))
    ins = _gen(g, 93, {})
    got, plan = _run(ctx, g, ins)
    assert "kind::f8f6f4" in plan.description and "interpret" in plan.description, plan.description
    narrow = O.evaluate(g, ins, f8_quantise=True)
    for o, x, y in zip(g.outputs, got, narrow):
        node = g.nodes[o]
        assert O.rel_l2(O.decode(x, node.dtype, node.shape), O.decode(y, node.dtype, node.shape)) <= 1e-5, plan.description


def test_gelu_epilogues_at_extreme_arguments(ctx):
    """GELU and gelu' in the GEMM epilogue at arguments far from the random-normal range: the product is
    zero (A = 0), so the outputs are gelu(bias[col]) and gelu'(G[row, col]) of hand-picked values --
    zeros of both signs, tiny, the bulk, the tails where erf saturates, and infinities -- checked
    element by element (f32 outputs, absolute error: the polynomial erf is good to 1.5e-7)."""
    m, n, k = 128, 256, 64
    vals = np.array([0.0, -0.0, 1e-30, -1e-30, 1e-4, -1e-4, 0.5, -0.5, 1.0, -1.0, 2.5, -2.5, 4.0, -4.0, 6.0, -6.0,
                     9.0, -9.0, 13.0, -13.0, 40.0, -40.0, 300.0, -300.0, 3.0e4, -3.0e4, np.inf, 0.25, -0.25, 3.0, -3.0, 1.5], dtype=np.float64)
    # forward: gelu(0 + bias)
    g = graph_linear(m, n, k, bias=True, act=ir.UN_GELU, dtype=ir.BF16, out_dtype=ir.F32)
    ins = _gen(g, 91)
    ins[0] = O.encode(np.zeros((m, k)), ir.BF16)
    ins[2] = O.encode(np.resize(vals, n), ir.BF16)
    got, plan = _run(ctx, g, ins)
    want = O.evaluate(g, ins)
    a = O.decode(got[0], ir.F32, (m, n)); b = O.decode(want[0], ir.F32, (m, n))
    fin = np.isfinite(b)
    assert np.array_equal(np.isfinite(a), fin), plan.description
    assert np.allclose(a[fin], b[fin], rtol=2e-6, atol=2e-6), float(np.abs(a[fin] - b[fin]).max())
    assert np.array_equal(a[~fin], b[~fin])
    # backward: (1 + 0) * gelu'(G), with the column sum
    g = graph_linear(m, n, k, bias=True, gate="dgelu", colsum="y", dtype=ir.BF16, out_dtype=ir.F32)
    ins = _gen(g, 92)
    ins[0] = O.encode(np.zeros((m, k)), ir.BF16)
    ins[2] = O.encode(np.ones(n), ir.BF16)
    gv = np.resize(vals[np.isfinite(vals)], (m, n))
    ins[3] = O.encode(gv, ir.BF16)
    got, plan = _run(ctx, g, ins)
    want = O.evaluate(g, ins)
    a = O.decode(got[0], ir.F32, (m, n)); b = O.decode(want[0], ir.F32, (m, n))
    assert np.allclose(a, b, rtol=2e-6, atol=2e-6), (plan.description, float(np.abs(a - b).max()))
    cs_a = np.asarray(got[1], dtype=np.float64).reshape(-1); cs_b = np.asarray(want[1], dtype=np.float64).reshape(-1)
    assert np.allclose(cs_a, cs_b, rtol=1e-5, atol=1e-4)


def test_mlp_block_forward_backward(ctx):
    """configs[3] at a small size: every one of the six fused GEMMs against the oracle evaluated on
    the operands that GEMM actually read (so an upstream rounding does not hide a downstream error)."""
    import torch
    from helium_b200.mlp_block import MlpBlock, mlp_block_inputs
    tokens, d, ff = 384, 256, 512
    blk = MlpBlock(ctx, tokens, d, ff)
    host = mlp_block_inputs(tokens, d, ff)
    blk.load(host)
    blk.step()
    torch.cuda.synchronize()
    ctx.poll()
    bits = lambda t: t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16) if t.dtype == torch.bfloat16 else t.cpu().numpy()
    dev = {k: bits(getattr(blk, k)) for k in ("X", "W1", "W2", "b1", "b2", "dO", "H", "Z", "O", "dZ", "dX", "dW1", "dW2", "db1", "db2")}
    cases = {
        "H": (["X", "W1", "b1"], ["H", "Z"]), "O": (["H", "W2", "b2", "X"], ["O"]),
        "dZ": (["dO", "W2", "Z"], ["dZ", "db1"]), "dW1": (["X", "dZ"], ["dW1"]),
        "dW2": (["H", "dO"], ["dW2"]), "dX": (["dZ", "W1", "dO"], ["dX", "db2"]),
    }
    for name, (ins, outs) in cases.items():
        g = blk.graphs[name]
        want = O.evaluate(g, [dev[k] for k in ins])
        _compare(g, [dev[k] for k in outs], want, f"{name}: {blk.plans[name].description}")
    assert blk.launch_count() >= 6


def test_mlp_block_full_size_sampled(ctx):
    """configs[3] at its benchmark size (8192 tokens, d 4096, ff 16384).  The numpy oracle would take
    hours, so 32 sampled output rows of every GEMM go through the C oracle's bf16 GEMM (f32
    accumulate) with the epilogue restated in f64, and the bias gradients are checked as checksums."""
    import torch
    from math import sqrt
    from scipy.special import erf
    from oracle import oracle_c as OC
    from helium_b200.mlp_block import MlpBlock, mlp_block_inputs
    T, d, ff = 8192, 4096, 16384
    blk = MlpBlock(ctx, T, d, ff)
    host = mlp_block_inputs(T, d, ff)
    blk.load(host)
    blk.step()
    torch.cuda.synchronize()
    ctx.poll()
    bits = lambda t: t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    dec = lambda b: (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    dev = {k: bits(getattr(blk, k)) for k in ("H", "Z", "O", "dZ", "dX", "dW1", "dW2")}
    r = rng(31)
    rows_t = np.sort(r.choice(T, 32, replace=False))
    close = lambda got, want, what: (O.rel_l2(got, want) <= 1e-2) or pytest.fail(f"{what}: rel-L2 {O.rel_l2(got, want):.3e}")
    gelu = lambda z: 0.5 * z * (1 + erf(z / sqrt(2)))
    dgelu = lambda z: 0.5 * (1 + erf(z / sqrt(2))) + z * np.exp(-0.5 * z * z) / sqrt(2 * np.pi)
    X, W1, W2, dO = host["X"], host["W1"], host["W2"], host["dO"]
    b1, b2 = dec(host["b1"]), dec(host["b2"])
    # H = gelu(X W1 + b1), Z kept
    z = OC.gemm_bf16(X[rows_t], W1).astype(np.float64) + b1
    close(dec(dev["Z"][rows_t]), z, "Z")
    close(dec(dev["H"][rows_t]), gelu(z), "H")
    # O = H W2 + b2 + X   (H as the kernel stored it)
    o = OC.gemm_bf16(dev["H"][rows_t], W2).astype(np.float64) + b2 + dec(X[rows_t])
    close(dec(dev["O"][rows_t]), o, "O")
    # dZ = (dO W2^T) * gelu'(Z)
    w2t = np.ascontiguousarray(W2.T)
    dz = OC.gemm_bf16(dO[rows_t], w2t).astype(np.float64) * dgelu(dec(dev["Z"][rows_t]))
    close(dec(dev["dZ"][rows_t]), dz, "dZ")
    # dX = dZ W1^T + dO
    w1t = np.ascontiguousarray(W1.T)
    dx = OC.gemm_bf16(dev["dZ"][rows_t], w1t).astype(np.float64) + dec(dO[rows_t])
    close(dec(dev["dX"][rows_t]), dx, "dX")
    # dW1 = X^T dZ (rows of dW1 are columns of X), dW2 = H^T dO
    rows_d = np.sort(r.choice(d, 32, replace=False))
    close(dec(dev["dW1"][rows_d]), OC.gemm_bf16(np.ascontiguousarray(X[:, rows_d].T), dev["dZ"]).astype(np.float64), "dW1")
    rows_f = np.sort(r.choice(ff, 32, replace=False))
    close(dec(dev["dW2"][rows_f]), OC.gemm_bf16(np.ascontiguousarray(dev["H"][:, rows_f].T), dO).astype(np.float64), "dW2")
    # bias gradients against the oracle at the f32 tolerance: db2 = colsum(dO) from the inputs; db1 =
    # colsum(dZ) over ALL 8192 rows of the oracle's own dZ (C-oracle GEMM, gelu' in f64 on the Z that the dZ
    # GEMM read, summed in f64 before any rounding) for 64 sampled columns
    db2 = blk.db2.cpu().numpy().reshape(-1).astype(np.float64)
    assert O.rel_l2(db2, dec(dO).sum(0)) <= 1e-5
    db1 = blk.db1.cpu().numpy().reshape(-1).astype(np.float64)
    cols = np.sort(r.choice(ff, 64, replace=False))
    dh_cols = OC.gemm_bf16(dO, np.ascontiguousarray(W2[cols].T)).astype(np.float64)        # [T, 64] = dO W2^T[:, cols]
    dz_cols = dh_cols * dgelu(dec(dev["Z"][:, cols]))
    err = O.rel_l2(db1[cols], dz_cols.sum(0))
    assert err <= 1e-5, f"db1 against the oracle's column sums: rel-L2 {err:.3e}"


@pytest.mark.parametrize("kw", [
    dict(bias=False),                                              # N-major B: half tiles load one 64-column box
    dict(bias=False, b_t=True),                                    # K-major B: half tiles use half of the 128-row box
    dict(bias=True, act=ir.UN_RELU, resid=True, colsum="resid"),   # column sums across full and half tiles
    dict(bias=False, a_t=True, b_t=True, out_dtype=ir.F32),
])
def test_tail_split_tiles(ctx, kw):
    """256 pair tiles on 74 SM pairs: the last 34 tiles run as 68 half-width tiles.  Every output
    element and every column sum must come out as if the tiles were whole."""
    m, n, k = 4096, 4096, 192
    g = graph_linear(m, n, k, **kw)
    ins = _gen(g, 41, {1: 1.0 / np.sqrt(k)})
    got, plan = _run(ctx, g, ins)
    assert "2-CTA" in plan.description
    _compare(g, got, O.evaluate(g, ins), plan.description)


def _generic_reduction_graph(m, n, k, batch=None, which=("cols", "rows", "all")):
    """tanh(A B + bias) stored, plus Sum reductions of pointwise expressions of it that match no
    hand-written epilogue: over rows (Columns), over columns (Rows), over everything."""
    g = ir.Graph()
    lead = [] if batch is None else [batch]
    a = g.new_input(lead + [m, k], ir.BF16)
    b = g.new_input(lead + [k, n], ir.BF16)
    bias = g.new_input([n], ir.BF16)
    w = g.new_input(lead + [m, n], ir.BF16)
    t = g.binary(ir.BIN_ADD, g.matmul(a, b, ir.PREC_BF16_F32), g.broadcast_to(bias, lead + [m, n]))
    y = g.unary(ir.UN_TANH, t)
    g.new_output(g.cast(y, ir.BF16))
    r = len(lead) + 2
    e = g.binary(ir.BIN_MUL, y, w)
    if "cols" in which:
        g.new_output(g.reduce_axes(ir.RED_SUM, e, [r - 2]))                       # [.., 1, n]
    if "rows" in which:
        g.new_output(g.reduce_axes(ir.RED_SUM, g.binary(ir.BIN_MUL, y, y), [r - 1]))   # [.., m, 1]
    if "all" in which:
        g.new_output(g.reduce_axes(ir.RED_SUM, e, list(range(r))))                # [1, .., 1]
    if "cols_batch" in which:
        g.new_output(g.reduce_axes(ir.RED_SUM, y, [0, r - 2]))                    # [1, 1, n]: batch folded in
    return g


@pytest.mark.parametrize("m,n,k,batch,which", [
    (256, 512, 128, None, ("cols", "rows", "all")),
    (200, 264, 72, None, ("cols", "rows", "all")),        # ragged tiles, one-CTA kernel for the last rows
    (640, 768, 64, None, ("rows",)),
    (128, 128, 64, None, ("cols", "all")),                 # single-CTA kernel
    (256, 256, 64, 3, ("cols", "rows", "cols_batch")),
    (4096, 4096, 64, None, ("cols", "rows", "all")),       # tail-split half tiles
])
def test_generic_epilogue_reductions(ctx, m, n, k, batch, which):
    g = _generic_reduction_graph(m, n, k, batch, which)
    ins = _gen(g, 51, {1: 1.0 / np.sqrt(k), 2: 0.1})
    got, plan = _run(ctx, g, ins)
    assert "tier 1" in plan.description and "reductions" in plan.description
    _compare(g, got, O.evaluate(g, ins), plan.description)
    got2, _ = _run(ctx, g, ins)
    for x, y in zip(got, got2):
        assert np.array_equal(x, y), "reductions must be bit-stable across launches"


def test_generic_epilogue_reduction_limits(ctx):
    g = ir.Graph()
    a = g.new_input([256, 64], ir.BF16); b = g.new_input([64, 256], ir.BF16)
    y = g.unary(ir.UN_EXP, g.matmul(a, b, ir.PREC_BF16_F32))
    for _ in range(3):
        g.new_output(g.reduce_axes(ir.RED_MAX, y, [0]))
    with pytest.raises(hb.HeliumError, match="at most two column reductions"):
        hb.Plan.fused_matmul(ctx, g)


@pytest.mark.parametrize("m,n,k,batch", [(256, 512, 128, None), (200, 264, 72, None), (136, 72, 40, 3), (4096, 4096, 64, None)])
def test_generic_epilogue_column_extrema(ctx, m, n, k, batch):
    """Max and Min over the rows of the output (one value per column), with ragged tiles whose rows
    beyond M must contribute the identity, not zero."""
    lead = [] if batch is None else [batch]
    g = ir.Graph()
    a = g.new_input(lead + [m, k], ir.BF16); b = g.new_input(lead + [k, n], ir.BF16)
    y = g.unary(ir.UN_ADD_CONST, g.unary(ir.UN_TANH, g.matmul(a, b, ir.PREC_BF16_F32)), const=3.0)   # all positive: zero would win a Min
    r = len(lead)
    g.new_output(g.reduce_axes(ir.RED_MIN, y, [r]))
    g.new_output(g.reduce_axes(ir.RED_MAX, g.unary(ir.UN_NEG, y), [r]))   # all negative: zero would win a Max
    g.new_output(g.reduce_axes(ir.RED_SUM, y, [r + 1]))
    ins = _gen(g, 83, {1: 1.0 / np.sqrt(k)})
    got, plan = _run(ctx, g, ins)
    assert "3 reductions" in plan.description
    want = O.evaluate(g, ins)
    for o, x, w in zip(g.outputs, got, want):
        x, w = np.asarray(x, dtype=np.float64).reshape(-1), np.asarray(w, dtype=np.float64).reshape(-1)
        assert np.allclose(x, w, rtol=2e-5, atol=2e-5), (g.nodes[o].shape, float(np.abs(x - w).max()))


@pytest.mark.parametrize("m,n,k", [(256, 512, 128), (200, 264, 72), (4096, 4096, 64)])
def test_generic_epilogue_mean_max_min(ctx, m, n, k):
    """Mean over rows / columns / everything (Sum scaled when the partials are folded) and Max / Min over
    columns and over everything (running extrema per thread, op-aware folds)."""
    g = ir.Graph()
    a = g.new_input([m, k], ir.BF16); b = g.new_input([k, n], ir.BF16)
    y = g.unary(ir.UN_TANH, g.matmul(a, b, ir.PREC_BF16_F32))
    g.new_output(g.reduce_axes(ir.RED_MEAN, y, [0]))          # [1, n]
    g.new_output(g.reduce_axes(ir.RED_MAX, y, [1]))           # [m, 1]
    g.new_output(g.reduce_axes(ir.RED_MIN, y, [0, 1]))        # [1, 1]
    g.new_output(g.reduce_axes(ir.RED_MEAN, g.binary(ir.BIN_MUL, y, y), [0, 1]))
    ins = _gen(g, 81, {1: 1.0 / np.sqrt(k)})
    got, plan = _run(ctx, g, ins)
    assert "4 reductions" in plan.description
    want = O.evaluate(g, ins)
    for o, x, w in zip(g.outputs, got, want):
        node = g.nodes[o]
        x, w = np.asarray(x, dtype=np.float64).reshape(-1), np.asarray(w, dtype=np.float64).reshape(-1)
        # extrema of a bf16-operand matmul are exact picks of values that carry the GEMM's rounding: 1e-5 relative to their scale
        assert np.allclose(x, w, rtol=2e-5, atol=2e-5), (node.shape, float(np.abs(x - w).max()))


def test_operand_side_pointwise_prologues(ctx):
    """Operand expressions the mainloop rewrite does not cover (here: a broadcast vector inside A's expression;
    any Constant / Unary / Binary / cast / reshape / swap chain is legal, generators/matmul.rs:234-264) are
    evaluated once into the workspace by a pointwise plan, while B's unary chain is applied in the kernel;
    the oracle rounds each operand once, where the plan does."""
    m, n, k = 256, 384, 128
    g = ir.Graph()
    x = g.new_input([m, k], ir.BF16); s = g.new_input([k], ir.BF16); y = g.new_input([m, k], ir.BF16)
    w = g.new_input([n, k], ir.BF16); bias = g.new_input([n], ir.BF16)
    a = g.binary(ir.BIN_ADD, g.binary(ir.BIN_MUL, x, g.broadcast_to(s, [m, k])), g.unary(ir.UN_TANH, y))     # A = x * s + tanh(y)
    b = g.unary(ir.UN_MUL_CONST, g.unary(ir.UN_SIGMOID, g.transpose(w)), 0.5)                                  # B = 0.5 * sigmoid(w^T)
    t = g.binary(ir.BIN_ADD, g.matmul(a, b, ir.PREC_BF16_F32), g.broadcast_to(bias, [m, n]))
    g.new_output(g.cast(g.unary(ir.UN_RELU, t), ir.BF16))
    ins = _gen(g, 61, {1: 0.5, 3: 1.0})
    plan = hb.Plan.fused_matmul(ctx, g)
    assert "operand A evaluated by a pre-pass" in plan.description and "generic mainloop rewrite" in plan.description, plan.description
    assert hb.plan_supported(g, 2) == 1
    got, _ = _run(ctx, g, ins)
    mm = [i for i, nd in enumerate(g.nodes) if nd.kind == ir.OP_MATMUL][0]
    want = O.evaluate(g, ins, round_nodes=list(g.nodes[mm].inputs[:2]))
    _compare(g, got, want, plan.description)
    # f32 operands take the SIMT GEMM; the prologue works the same way
    g = ir.Graph()
    a = g.new_input([96, 40], ir.F32); b = g.new_input([40, 24], ir.F32)
    g.new_output(g.matmul(g.binary(ir.BIN_MUL, a, a), g.unary(ir.UN_EXP, b), ir.PREC_TF32_F32))
    ins = _gen(g, 62, {1: 0.3})
    got, plan = _run(ctx, g, ins)
    assert "SIMT" in plan.description and "pre-pass" in plan.description
    _compare(g, got, O.evaluate(g, ins), plan.description)


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 264, 200), (512, 384, 1024), (1024, 512, 512)])
def test_generic_mainloop_fusion(ctx, monkeypatch, m, n, k):
    """Operand-side chains beyond relu * mask applied inside the kernel (the transform warps rewrite the tile in
    shared memory): unary chains with constants on A, a chain with a second tensor, a chain on B, transposed
    operands, f16.  The oracle rounds the operand once, where the kernel does."""
    monkeypatch.setenv("HE_GEMM_MAINLOOP", "fused")
    cases = []
    # A = tanh(x) * 0.5 + 0.25
    g = ir.Graph()
    x = g.new_input([m, k], ir.BF16); w = g.new_input([k, n], ir.BF16)
    a = g.unary(ir.UN_ADD_CONST, g.unary(ir.UN_MUL_CONST, g.unary(ir.UN_TANH, x), 0.5), 0.25)
    g.new_output(g.cast(g.matmul(a, w), ir.BF16))
    cases.append(("unary chain on A", g))
    # A = sigmoid(x) + e   (second tensor added), bias + relu epilogue
    g = ir.Graph()
    x = g.new_input([m, k], ir.BF16); e = g.new_input([m, k], ir.BF16); w = g.new_input([k, n], ir.BF16); bias = g.new_input([n], ir.BF16)
    a = g.binary(ir.BIN_ADD, g.unary(ir.UN_SIGMOID, x), e)
    t = g.binary(ir.BIN_ADD, g.matmul(a, w), g.broadcast_to(bias, [m, n]))
    g.new_output(g.cast(g.unary(ir.UN_RELU, t), ir.BF16))
    cases.append(("second tensor on A", g))
    # A = neg(x) * mk with A stored transposed; B = gelu(w) stored [n, k]
    g = ir.Graph()
    x = g.new_input([k, m], ir.BF16); mk = g.new_input([k, m], ir.BF16); w = g.new_input([n, k], ir.BF16)
    a = g.transpose(g.binary(ir.BIN_MUL, g.unary(ir.UN_NEG, x), mk))
    b = g.transpose(g.unary(ir.UN_GELU, w))
    g.new_output(g.matmul(a, b))
    cases.append(("A and B chains, transposed", g))
    # f16, B = exp(w * 0.1)
    g = ir.Graph()
    x = g.new_input([m, k], ir.F16); w = g.new_input([k, n], ir.F16)
    b = g.unary(ir.UN_EXP, g.unary(ir.UN_MUL_CONST, w, 0.1))
    g.new_output(g.cast(g.matmul(x, b, ir.PREC_F16_F32), ir.F16))
    cases.append(("f16 chain on B", g))
    for what, g in cases:
        ins = _gen(g, 33, {i: 0.5 for i in range(4)})
        plan = hb.Plan.fused_matmul(ctx, g)
        assert "generic mainloop rewrite" in plan.description and "pre-pass" not in plan.description, (what, plan.description)
        assert hb.plan_supported(g, 2) == 2
        got, _ = _run(ctx, g, ins)
        mm = [i for i, nd in enumerate(g.nodes) if nd.kind == ir.OP_MATMUL][0]
        want = O.evaluate(g, ins, round_nodes=list(g.nodes[mm].inputs[:2]))
        _compare(g, got, want, f"{what}: {plan.description}")
        got2, _ = _run(ctx, g, ins)
        for p_, q_ in zip(got, got2):
            assert np.array_equal(p_, q_), what


def test_helium_style_bias_gradient_fuses(ctx):
    """helium's front end writes a bias gradient as swap_dims -> Reduce{depth 1} -> reshape
    (tensor.rs:83-142); the planner rewrites that leaf to a reduction over the rows of the epilogue
    value, so it lands in the same hand-written column-sum epilogue as the playground spelling."""
    m, n, k = 384, 512, 128
    g = ir.Graph()
    do = g.new_input([m, k], ir.BF16); w = g.new_input([n, k], ir.BF16); z = g.new_input([m, n], ir.BF16)
    dz = g.binary(ir.BIN_MUL, g.matmul(do, g.transpose(w), ir.PREC_BF16_F32), g.unary(ir.UN_DGELU, z))
    g.new_output(g.cast(dz, ir.BF16))
    g.new_output(g.reshape(g.reduce(ir.RED_SUM, g.transpose(dz), 1), [n]))
    ins = _gen(g, 71, {1: 1.0 / np.sqrt(k)})
    got, plan = _run(ctx, g, ins)
    assert "tier 2" in plan.description and "colsum=2" in plan.description
    _compare(g, got, O.evaluate(g, ins), plan.description)
    # through the host runtime the three ops (matmul, gate, bias-gradient chain) become one instruction
    text = hb.HostGraph(g).plan_text()
    assert sum("FusedMatmul" in ln for ln in text.splitlines()) == 1 and "Pointwise" not in text and "Permute" not in text, text


def _random_linear_case(r):
    """One random fused-linear configuration within what graph_linear can express."""
    pick = lambda xs: xs[int(r.integers(0, len(xs)))]
    m = int(pick([8, 72, 128, 200, 256, 392, 520, 1024, 2304]))
    n = int(pick([8, 40, 128, 264, 512, 776, 1280]))
    k = int(pick([8, 64, 136, 320, 1024]))
    kw = dict(bias=bool(r.integers(0, 2)), a_t=bool(r.integers(0, 2)), b_t=bool(r.integers(0, 2)))
    kw["act"] = pick([None, ir.UN_RELU, ir.UN_GELU, ir.UN_TANH])
    kw["resid"] = bool(r.integers(0, 2))
    kw["gate"] = pick([None, None, "mul", "dgelu", "drelu"])
    kw["store_z"] = bool(r.integers(0, 2)) and kw["act"] is not None
    kw["colsum"] = pick([None, None, "y", "resid" if kw["resid"] else None])
    kw["batch"] = pick([None, None, 2, 3])
    kw["dtype"] = pick([ir.BF16, ir.BF16, ir.F16])
    kw["out_dtype"] = pick([None, ir.F32])
    return m, n, k, kw


@pytest.mark.parametrize("seed", range(24))
def test_random_fused_linear_configurations(ctx, seed):
    """Seeded sweep over shapes (ragged, batched, tiny), operand majors, dtypes and epilogue pieces:
    whatever tier the planner picks, the numbers must be the oracle's."""
    r = rng(1000 + seed)
    m, n, k, kw = _random_linear_case(r)
    g = graph_linear(m, n, k, **kw)
    ins = _gen(g, 2000 + seed, {1: 1.0 / np.sqrt(k)})
    try:
        plan = hb.Plan.fused_matmul(ctx, g)
    except hb.HeliumError as e:
        pytest.fail(f"refused: {e}")
    got, plan = _run(ctx, g, ins)
    _compare(g, got, O.evaluate(g, ins), f"{(m, n, k, kw)}: {plan.description}")
