"""CPU reference of the convolutional network's training step, in float64 torch with autograd.

TEST INFRASTRUCTURE ONLY (imported by tests/ and by bench.py's CPU legs; never by helium_b200/).
It restates resnet-train/src/model.rs:9-83,112-247 (including the second application of bn1 in the
downsample block, model.rs:233-240), helium/src/modules/batch_norm.rs:38-65 (train mode, biased variance
E[x^2] - mean^2, eps 1e-3), helium/src/modules/conv.rs:60-67 (filter cast to the activation dtype, bias
added), helium/src/loss.rs:5-8 and helium/src/optimizer/sgd.rs:47-62.  Convolutions are torch's, which
tests/test_conv_cpu.py ties to the numpy oracle and, through it, to the reference's conv vector.
Parity pin: the reference has no test of this model, of batch norm or of the optimiser; beyond the single
convolution vector this file's agreement with the reference rests on the restated formulas (unpinned).
Rounding points of the bf16 run are NOT modelled except where noted (weights and images are the bf16 values
the device reads): the comparison tolerance covers the rest.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F


def parameter_shapes(classes: int = 1000):
    """(name, shape) of every parameter, in the model's order (the same list as helium_b200.convnet.model_spec,
    restated here so that the CPU legs need not import the package)."""
    out = [("head.w", (32, 7, 7, 3)), ("head.b", (32,))]
    c = 32
    for s in range(4):
        o = 2 * c
        p = f"seg{s}.down."
        out += [(p + "bn1.g", (c,)), (p + "bn1.b", (c,)), (p + "conv1.w", (o, 3, 3, c)), (p + "conv1.b", (o,)), (p + "bn2.g", (o,)),
                (p + "bn2.b", (o,)), (p + "conv2.w", (o, 3, 3, o)), (p + "conv2.b", (o,)), (p + "sc.w", (o, 1, 1, c)), (p + "sc.b", (o,))]
        p = f"seg{s}.basic."
        out += [(p + "bn1.g", (o,)), (p + "bn1.b", (o,)), (p + "conv1.w", (o, 3, 3, o)), (p + "conv1.b", (o,)), (p + "bn2.g", (o,)),
                (p + "bn2.b", (o,)), (p + "conv2.w", (o, 3, 3, o)), (p + "conv2.b", (o,))]
        c = o
    out += [("tail_bn.g", (c,)), ("tail_bn.b", (c,)), ("tail.w", (classes, 1, 1, c)), ("tail.b", (classes,))]
    return out


def _bf16(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float32).to(torch.bfloat16).to(torch.float64)


class _RoundBf16(torch.autograd.Function):
    """Identity that rounds to bf16 in both directions: a tensor that is stored as bf16 between two kernels."""

    @staticmethod
    def forward(ctx, x):
        return _bf16(x)

    @staticmethod
    def backward(ctx, g):
        return _bf16(g)


_EMULATE_BF16 = False


def _store(x):
    return _RoundBf16.apply(x) if _EMULATE_BF16 else x


def _conv(x, w, b, stride):
    """x NHWC, w KRSC (f64 holding bf16 values), 'Same' padding k/2, output size in/stride."""
    k = w.shape[1]
    y = F.conv2d(x.permute(0, 3, 1, 2), w.permute(0, 3, 1, 2), stride=stride, padding=k // 2)
    p, q = x.shape[1] // stride, x.shape[2] // stride
    return _store(y[:, :, :p, :q].permute(0, 2, 3, 1) + b)


def _bn(x, gamma, beta):
    mean = x.mean(dim=(0, 1, 2))
    var = (x * x).mean(dim=(0, 1, 2)) - mean * mean
    return _store((x - mean) / torch.sqrt(var + 1e-3) * gamma + beta)


def forward(params: dict, images: torch.Tensor, labels: np.ndarray, classes: int):
    """params: name -> f64 tensors requiring grad (filters already hold bf16 values).  Returns (loss, logits)."""
    P = params
    x = _conv(images, P["head.w"], P["head.b"], 2)
    for s in range(4):
        p = f"seg{s}.down."
        a = torch.relu(_bn(x, P[p + "bn1.g"], P[p + "bn1.b"]))
        sc = _conv(a, P[p + "sc.w"], P[p + "sc.b"], 2)
        a2 = torch.relu(_bn(a, P[p + "bn1.g"], P[p + "bn1.b"]))
        c1 = _conv(a2, P[p + "conv1.w"], P[p + "conv1.b"], 2)
        a3 = torch.relu(_bn(c1, P[p + "bn2.g"], P[p + "bn2.b"]))
        x = _conv(a3, P[p + "conv2.w"], P[p + "conv2.b"], 1) + sc
        p = f"seg{s}.basic."
        a = torch.relu(_bn(x, P[p + "bn1.g"], P[p + "bn1.b"]))
        c1 = _conv(a, P[p + "conv1.w"], P[p + "conv1.b"], 1)
        a2 = torch.relu(_bn(c1, P[p + "bn2.g"], P[p + "bn2.b"]))
        x = _conv(a2, P[p + "conv2.w"], P[p + "conv2.b"], 1) + x
    t = torch.relu(_bn(x, P["tail_bn.g"], P["tail_bn.b"]))
    y = _conv(t, P["tail.w"], P["tail.b"], 1)
    logits = y.mean(dim=(1, 2))
    onehot = torch.zeros((images.shape[0], classes), dtype=torch.float64)
    onehot[torch.arange(images.shape[0]), torch.from_numpy(labels.astype(np.int64))] = 1.0
    loss = -(F.log_softmax(logits, dim=1) * onehot).sum() / images.shape[0]
    return loss, logits


def training_step(params_f32: dict, image_bits: np.ndarray, labels: np.ndarray, classes: int, lr: float, momentum: float,
                  averages: dict | None, emulate_bf16: bool = False):
    """One step on f32 master parameters (numpy).  Returns (loss, grads, new_params, new_averages).
    With `emulate_bf16` every convolution and batch-norm output (and the gradient flowing back through it) is
    rounded to bf16, which is where a bf16 run stores tensors: the distance of that run's gradients from the
    exact ones is the noise floor any bf16 implementation of this step has."""
    global _EMULATE_BF16
    _EMULATE_BF16 = bool(emulate_bf16)
    try:
        return _training_step(params_f32, image_bits, labels, classes, lr, momentum, averages)
    finally:
        _EMULATE_BF16 = False


def _training_step(params_f32, image_bits, labels, classes, lr, momentum, averages):
    bits = np.ascontiguousarray(image_bits, dtype=np.uint16)
    img = torch.from_numpy((bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64))
    P = {}
    for n, v in params_f32.items():
        t = torch.from_numpy(np.asarray(v, dtype=np.float32).astype(np.float64))
        if n.endswith(".w"):
            t = _bf16(t)        # the convolution reads the filter in the activation dtype (conv.rs:63)
        P[n] = t.requires_grad_(True)
    loss, _ = forward(P, img, labels, classes)
    loss.backward()
    grads = {n: P[n].grad.numpy() for n in P}
    new_p, new_a = {}, {}
    for n, v in params_f32.items():
        g = grads[n]
        a = g if averages is None else g * (1.0 - momentum) + averages[n] * momentum
        new_a[n] = a
        new_p[n] = np.asarray(v, dtype=np.float64) - lr * a
    return float(loss.item()), grads, new_p, new_a
