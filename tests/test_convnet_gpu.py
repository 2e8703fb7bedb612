"""One training step of the resnet-train network on the GPU against the float64 torch reference
(oracle/convnet_torch.py) on the same bf16 image and filter bits: loss, every parameter gradient, and the updated
parameters after two optimiser steps (the first takes avg = g, the second the exponential average).
Tolerance: the activations are bf16 between kernels (as in the reference run), so gradients are compared at
rel-L2 <= 5e-2 per tensor and the loss at 1e-2; biases and batch-norm gradients of the last layers, which
see the least accumulated rounding, are held to 2e-2."""
import numpy as np
import pytest

import helium_b200 as hb
from helium_b200 import convnet
from helpers import O

pytestmark = pytest.mark.gpu


def _setup(ctx, batch, hw, classes):
    import torch
    net = convnet.ConvNet(ctx, batch, image_hw=hw, classes=classes)
    params = convnet.init_params(4, classes)
    # non-trivial biases / gammas / betas so that their gradients matter
    r = np.random.default_rng(9)
    for n, k, shape in net.spec:
        if k == "bias":
            params[n] = (r.standard_normal(shape) * 0.05).astype(np.float32)
        elif k == "gamma":
            params[n] = (1.0 + r.standard_normal(shape) * 0.1).astype(np.float32)
        elif k == "beta":
            params[n] = (r.standard_normal(shape) * 0.1).astype(np.float32)
    net.load_params(params)
    bits, labels = convnet.synthetic_batch(batch, hw, classes)
    net.acts["x0"].view(torch.int16).copy_(torch.from_numpy(bits.view(np.int16)))
    net.labels.copy_(torch.from_numpy(labels))
    return net, params, bits, labels


def _device_grads(net):
    out = {}
    for n, k, shape in net.spec:
        src = net.GW[n] if k == "conv" else net.GV[n]
        out[n] = src.float().cpu().numpy().astype(np.float64)
    out["head.w"] = convnet.head_to_filter(out["head.w"])      # [32,1,1,152] over the patch matrix -> [32,7,7,3]
    return out


def _as_reference(params):
    """The device's parameters in the reference's shapes: the stem filter back as [32, 7, 7, 3]."""
    out = dict(params)
    out["head.w"] = convnet.head_to_filter(params["head.w"])
    return out


def test_training_step_matches_the_reference_model(ctx):
    """Loss, gradients and updated parameters of two steps.  The yardstick for the gradients is the reference itself
    run with bf16 storage emulated (oracle/convnet_torch.py): its distance from the exact float64 gradients is the
    noise floor of any bf16 run of this network (batch statistics over a few hundred values amplify the 0.4 %
    rounding of the activations to tens of percent in the first layers).  The GPU must stay within 1.5 x that
    floor plus 1 % for every tensor.  Convolution biases in front of a batch norm have a gradient of exactly zero
    (the norm removes the mean); for those the device value must be small against the filter gradient's scale."""
    import torch
    from oracle import convnet_torch as CT
    batch, hw, classes, lr = 16, 96, 40, 0.05
    net, params, bits, labels = _setup(ctx, batch, hw, classes)
    def averages_to_host():
        out = {}
        for n, k, shape in net.spec:
            flat = net.avg_conv if k == "conv" else net.avg_vec
            out[n] = flat[net.offs[n]: net.offs[n] + int(np.prod(shape))].view(shape).cpu().numpy().astype(np.float64)
        return out

    for step in range(2):
        # the reference starts every step from the device's own state, so that one step is compared at a time
        old_p = _as_reference(net.params_to_host())
        old_avg = None if step == 0 else _as_reference(averages_to_host())
        net.step(lr)
        torch.cuda.synchronize()
        ctx.poll()
        assert net.launches > 100
        loss = float(net.loss.sum().item())
        grads = _device_grads(net)
        new_p = _as_reference(net.params_to_host())
        _, noisy, _, _ = CT.training_step(old_p, bits, labels, classes, lr, 0.9, old_avg, emulate_bf16=True)
        ref_loss, exact, ref_p, _ = CT.training_step(old_p, bits, labels, classes, lr, 0.9, old_avg)
        assert abs(loss - ref_loss) <= 5e-3 * abs(ref_loss), (step, loss, ref_loss)
        report = []
        for n, k, shape in net.spec:
            g, rg, ng = grads[n], exact[n], noisy[n]
            cut = lambda a: a
            upd_dev, upd_ref = cut(old_p[n].astype(np.float64) - new_p[n]), cut(old_p[n].astype(np.float64) - ref_p[n])
            if k == "bias" and n != "tail.b":
                wref = exact[n[:-1] + "w"]
                bound = 0.05 * np.abs(wref).max() * np.prod(wref.shape[1:])
                assert np.abs(g).max() <= bound and np.abs(upd_dev).max() <= lr * bound, (step, n)
                continue
            err, floor = O.rel_l2(cut(g), cut(rg)), O.rel_l2(cut(ng), cut(rg))
            report.append((n, err, floor))
            assert err <= 1.5 * floor + 1e-2, (step, n, err, floor)
            # the optimiser step (the second one exercises the exponential average): same yardstick on the update
            uerr = O.rel_l2(upd_dev, upd_ref)
            assert uerr <= 1.5 * floor + 2e-2, (step, n, uerr, floor)
        print(f"step {step}: loss {loss:.5f} vs {ref_loss:.5f}; gradient error / bf16 floor: " +
              " ".join(f"{n}={e:.3f}/{f:.3f}" for n, e, f in report))


def test_step_is_bit_stable(ctx):
    """Two nets fed the same bytes produce the same loss and gradient bits: every reduction has a fixed order."""
    import torch
    outs = []
    for _ in range(2):
        net, _, _, _ = _setup(ctx, 8, 64, 24)
        net.step(0.01)
        torch.cuda.synchronize()
        ctx.poll()
        outs.append((net.loss.clone(), net.g_conv.clone(), net.g_vec.clone()))
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a.view(torch.int32) if a.dtype == torch.float32 else a.view(torch.int16),
                           b.view(torch.int32) if b.dtype == torch.float32 else b.view(torch.int16))


def test_graph_replay_gives_the_eager_step(ctx):
    """Three steps replayed from the captured CUDA graphs leave the same weights, gradients and loss bits as three
    eager steps from the same start (the graphs hold the same launches, nothing else)."""
    import torch
    res = []
    for use_graph in (False, True):
        net, _, _, _ = _setup(ctx, 8, 64, 24)
        for _ in range(4):                     # first step eager either way, then three eager / replayed
            net.step(0.01, graph=use_graph)
        torch.cuda.synchronize()
        ctx.poll()
        assert (net._graphs is not None) == use_graph
        res.append((net.loss.clone(), net.g_conv.clone(), net.g_vec.clone(), net.w_conv.clone(), net.w_vec.clone(), net.launches))
    bits = lambda t: t.view(torch.int32) if t.dtype == torch.float32 else t.view(torch.int16)
    for a, b in zip(res[0][:5], res[1][:5]):
        assert torch.equal(bits(a), bits(b))
    assert res[0][5] == res[1][5] > 200


def test_many_steps_leave_the_device_status_clean_and_repeat_bit_for_bit(ctx):
    """A long run of graph-replayed steps (about 2 x 10^4 convolution launches at the benchmark's layer shapes):
    no bounded wait may give up (he_ctx_poll_device_status stays clean), and the forward pass of the same weights
    and images gives the same loss bits every time.  Guards the pipelines of the multi-issuer convolution kernels:
    a parity wait that skipped a barrier phase once stopped a ring about once in 10^4 launches."""
    import torch
    net, params, bits, labels = _setup(ctx, 64, 224, 1000)
    net.step(0.0)                      # first step eager; lr 0 keeps the weights, momentum only accumulates zeros
    torch.cuda.synchronize()
    ctx.poll()
    first = net.loss.clone()
    for i in range(120):
        net.step(0.0, graph=True)
        if i % 40 == 39:
            torch.cuda.synchronize()
            ctx.poll()
            assert torch.equal(net.loss, first), i
    torch.cuda.synchronize()
    ctx.poll()
    assert torch.equal(net.loss, first)
