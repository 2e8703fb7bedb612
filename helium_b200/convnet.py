"""The convolutional network of resnet-train as one training step over the C ABI.

Model (resnet-train/src/model.rs:9-83,112-247): 7x7/2 head 3 -> 32; four segments, each a DownsampleBlock
(c -> 2c, /2: relu(bn1(x)) feeds a 1x1/2 shortcut convolution; bn1 is applied a SECOND time, then 3x3/2, bn2,
3x3, plus the shortcut, model.rs:233-246) followed by one BasicBlock (pre-activation: bn1, relu, 3x3, bn2, relu,
3x3, plus the input, model.rs:152-164); bn + relu; 1x1 to the classes; mean over the remaining positions.
Batch norm: helium/src/modules/batch_norm.rs:32-71.  Convolutions carry a zero-initialised bias
(helium/src/modules/conv.rs:41-47) and read their f32 master weights as bf16 (conv.rs:63).  Loss:
helium/src/loss.rs:5-8.  Optimiser: helium's SGD "momentum", an exponential average (optimizer/sgd.rs:47-62).

Every tensor operation below is a call into libhelium_b200.so (he_plan_conv2d / he_launch, he_bn_*, he_add_bf16,
he_colsum_bf16, he_pool_softmax_ce, he_sgd_momentum); PyTorch only owns the device buffers and the stream.
What is fused where:
  * every batch norm's statistics come out of the epilogue of the convolution that produces its input
    (or, for the second application of bn1, out of the bn-apply kernel itself);
  * bias and the block's residual add ride in the convolution epilogue;
  * in the backward pass the rectifier mask and the two sums batch norm's backward needs ride in the epilogue
    of the data-gradient convolution, so bn backward is one affine pass dx = A g + B x + K.
The stem is the one convolution that does not read its image through TMA: three channels are a 6-byte pixel, below
the 16-byte pitch a tensor map needs and far below the 64-channel slices the tensor core consumes.  Its patch
matrix [N, 112, 112, 152] is written once per step by he_im2col_nhwc and serves both the forward pass and the
filter gradient as the input of a 1 x 1 convolution; every other convolution is implicit.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional

import numpy as np

from . import ir
from ._lib import check, lib
from .runtime import Context, Plan, _stream_ptr

HEAD_CHANNELS = 32
IMG_CHANNELS = 3
HEAD_K = 152          # 7 * 7 * 3 = 147 patch columns, padded to a multiple of 8


def filter_to_head(w: np.ndarray) -> np.ndarray:
    """[32, 7, 7, 3] stem filter -> the [32, 1, 1, 152] filter of the 1 x 1 convolution over the patch matrix."""
    out = np.zeros((w.shape[0], 1, 1, HEAD_K), dtype=w.dtype)
    out[:, 0, 0, :147] = w.reshape(w.shape[0], 147)
    return out


def head_to_filter(w: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(w.reshape(w.shape[0], HEAD_K)[:, :147]).reshape(w.shape[0], 7, 7, 3)


def model_spec(classes: int = 1000):
    """Convolutions and batch norms in parameter order: (name, kind, shape)."""
    spec = [("head.w", "conv", (HEAD_CHANNELS, 1, 1, HEAD_K)), ("head.b", "bias", (HEAD_CHANNELS,))]
    c = HEAD_CHANNELS
    for s in range(4):
        o = 2 * c
        p = f"seg{s}.down."
        spec += [(p + "bn1.g", "gamma", (c,)), (p + "bn1.b", "beta", (c,)),
                 (p + "conv1.w", "conv", (o, 3, 3, c)), (p + "conv1.b", "bias", (o,)),
                 (p + "bn2.g", "gamma", (o,)), (p + "bn2.b", "beta", (o,)),
                 (p + "conv2.w", "conv", (o, 3, 3, o)), (p + "conv2.b", "bias", (o,)),
                 (p + "sc.w", "conv", (o, 1, 1, c)), (p + "sc.b", "bias", (o,))]
        p = f"seg{s}.basic."
        spec += [(p + "bn1.g", "gamma", (o,)), (p + "bn1.b", "beta", (o,)),
                 (p + "conv1.w", "conv", (o, 3, 3, o)), (p + "conv1.b", "bias", (o,)),
                 (p + "bn2.g", "gamma", (o,)), (p + "bn2.b", "beta", (o,)),
                 (p + "conv2.w", "conv", (o, 3, 3, o)), (p + "conv2.b", "bias", (o,))]
        c = o
    spec += [("tail_bn.g", "gamma", (c,)), ("tail_bn.b", "beta", (c,)), ("tail.w", "conv", (classes, 1, 1, c)), ("tail.b", "bias", (classes,))]
    return spec


def init_params(seed: int = 4, classes: int = 1000) -> Dict[str, np.ndarray]:
    """f32 master parameters: filters ~ N(0, 1/sqrt(R S K)) (helium's "KaimingNormal", initializer.rs:29-36,48-52),
    biases 0, gamma 1, beta 0.  The stem's [32, 7, 7, 3] filter is stored as the [32, 1, 1, 152] filter of a 1 x 1
    convolution over the patch matrix (filter_to_head)."""
    r = np.random.Generator(np.random.Philox(seed))
    out = {}
    for name, kind, shape in model_spec(classes):
        if name == "head.w":
            w = (r.standard_normal((HEAD_CHANNELS, 7, 7, 3), dtype=np.float32) / np.float32(np.sqrt(7 * 7 * HEAD_CHANNELS))).astype(np.float32)
            out[name] = filter_to_head(w)
        elif kind == "conv":
            k, rr, ss, cc = shape
            out[name] = (r.standard_normal(shape, dtype=np.float32) / np.float32(np.sqrt(rr * ss * k))).astype(np.float32)
        elif kind == "gamma":
            out[name] = np.ones(shape, dtype=np.float32)
        else:
            out[name] = np.zeros(shape, dtype=np.float32)
    return out


def flops_per_image(hw: int = 224, classes: int = 1000) -> float:
    """Multiply-adds x 2 of the forward convolutions (RGB counted as 3 channels); backward costs twice that."""
    f = (hw // 2) ** 2 * 7 * 7 * IMG_CHANNELS * HEAD_CHANNELS
    c, s = HEAD_CHANNELS, hw // 2
    for _ in range(4):
        o, s2 = 2 * c, s // 2
        f += s2 * s2 * (c * o + 9 * c * o + 9 * o * o)      # shortcut, conv1, conv2 of the downsample block
        f += s2 * s2 * 2 * 9 * o * o                        # basic block
        c, s = o, s2
    f += s * s * c * classes
    return 2.0 * f


class _Bn:
    """Per-application state of a batch norm: scale / shift / mean / rstd vectors and the statistics buffer."""

    def __init__(self, torch, dev, c):
        f = lambda *s: torch.zeros(s, dtype=torch.float32, device=dev)
        self.stats, self.scale, self.shift, self.mean, self.rstd = f(2, c), f(c), f(c), f(c), f(c)
        self.bstats, self.coef = f(2, c), f(3, c)


class ConvNet:
    def __init__(self, ctx: Context, batch: int, image_hw: int = 224, classes: int = 1000, device=None, momentum: float = 0.9):
        import torch

        self.torch, self.ctx = torch, ctx
        self.N, self.hw, self.classes, self.momentum = batch, image_hw, classes, momentum
        dev = device if device is not None else torch.device("cuda", ctx.device)
        self.dev = dev
        self.spec = model_spec(classes)
        # ---- parameters: two flat groups so that the optimiser and the gradient exchange are two calls ----
        conv_names = [n for n, k, _ in self.spec if k == "conv"]
        vec_names = [n for n, k, _ in self.spec if k != "conv"]
        self.shapes = {n: s for n, _, s in self.spec}
        size = lambda n: int(np.prod(self.shapes[n]))
        pad8 = lambda v: (v + 7) // 8 * 8
        self.offs, off = {}, 0
        for n in conv_names:
            self.offs[n] = off
            off += pad8(size(n))
        self.n_conv = off
        off = 0
        for n in vec_names:
            self.offs[n] = off
            off += pad8(size(n))
        self.n_vec = off
        f32, bf16 = torch.float32, torch.bfloat16
        z = lambda n, dt: torch.zeros(n, dtype=dt, device=dev)
        self.w_conv, self.avg_conv, self.w16_conv, self.g_conv = z(self.n_conv, f32), z(self.n_conv, f32), z(self.n_conv, bf16), z(self.n_conv, bf16)
        self.w_vec, self.avg_vec, self.g_vec = z(self.n_vec, f32), z(self.n_vec, f32), z(self.n_vec, f32)
        self.g_vec2 = z(self.n_vec, f32)    # second contribution of parameters that are used twice (bn1 of the downsample blocks)
        self.first_step = True
        view = lambda flat, n: flat[self.offs[n]: self.offs[n] + size(n)].view(self.shapes[n])
        self.W16 = {n: view(self.w16_conv, n) for n in conv_names}
        self.GW = {n: view(self.g_conv, n) for n in conv_names}
        self.V = {n: view(self.w_vec, n) for n in vec_names}
        self.GV = {n: view(self.g_vec, n) for n in vec_names}
        self.GV2 = {n: view(self.g_vec2, n) for n in vec_names}
        self._view = view
        self.running: Dict[str, tuple] = {}
        # ---- activations, plans -----------------------------------------------------------------------
        self.acts: Dict[str, object] = {}
        self.plans: Dict[str, Plan] = {}
        self.bns: Dict[str, _Bn] = {}
        self._ws_bytes = 0
        self._build()
        self.ws = torch.empty(self._ws_bytes + 256, dtype=torch.uint8, device=dev)
        self.labels = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.loss = torch.zeros(batch, dtype=torch.float32, device=dev)
        self.launches = 0
        self._graphs = None       # (lr, forward+backward graph, optimiser graph, launches) once captured

    # -- construction -----------------------------------------------------------------------------------
    def _act(self, name, shape):
        t = self.torch.empty(shape, dtype=self.torch.bfloat16, device=self.dev)
        self.acts[name] = t
        return t

    def _conv_plans(self, name, hw, cin, cout, k, stride, fwd_kw, bwd_kw=None):
        kw = dict(batch=self.N, in_hw=(hw, hw), in_channels=cin, out_channels=cout, kernel=(k, k), stride=stride)
        self.plans[name + ".fwd"] = Plan.conv2d(self.ctx, "fwd", bias=True, **fwd_kw, **kw)
        self.plans[name + ".wgrad"] = Plan.conv2d(self.ctx, "bwd_filter", **kw)
        if bwd_kw is not None:
            self.plans[name + ".dgrad"] = Plan.conv2d(self.ctx, "bwd_data", **bwd_kw, **kw)
        for suffix in (".fwd", ".wgrad", ".dgrad"):
            if name + suffix in self.plans:
                self._ws_bytes = max(self._ws_bytes, self.plans[name + suffix].workspace_bytes)

    def _bn(self, name, c, pixels):
        self.bns[name] = _Bn(self.torch, self.dev, c)
        base = name.replace("#2", "")       # both applications of a shared norm update the same running statistics
        if base not in self.running:
            self.running[base] = (self.torch.zeros(c, dtype=self.torch.float32, device=self.dev),
                                  self.torch.ones(c, dtype=self.torch.float32, device=self.dev))
        self._ws_bytes = max(self._ws_bytes, lib.he_bn_workspace_bytes(pixels, c))

    def _build(self):
        N, hw = self.N, self.hw
        self._act("x0", (N, hw, hw, IMG_CHANNELS))
        s = hw // 2
        self._act("cols", (N, s, s, HEAD_K))
        self._conv_plans("head", s, HEAD_K, HEAD_CHANNELS, 1, 1, dict(stats=True))
        self._act("h", (N, s, s, HEAD_CHANNELS))
        c = HEAD_CHANNELS
        self.blocks = []
        for i in range(4):
            o, s2 = 2 * c, s // 2
            p = f"seg{i}.down"
            px, px2 = N * s * s, N * s2 * s2
            self._bn(p + ".bn1", c, px); self._bn(p + ".bn1#2", c, px); self._bn(p + ".bn2", o, px2)
            for nm, shp in ((".a", (N, s, s, c)), (".a2", (N, s, s, c)), (".sc", (N, s2, s2, o)), (".c1", (N, s2, s2, o)),
                            (".a3", (N, s2, s2, o)), (".out", (N, s2, s2, o)), (".g", (N, s2, s2, o)), (".dsc", (N, s, s, c)),
                            (".ga", (N, s, s, c)), (".gx", (N, s, s, c))):
                self._act(p + nm, shp)
            self._conv_plans(p + ".sc", s, c, o, 1, 2, dict(), dict())
            self._conv_plans(p + ".conv1", s, c, o, 3, 2, dict(stats=True), dict(gate=True, stats=True))
            self._conv_plans(p + ".conv2", s2, o, o, 3, 1, dict(resid=True, stats=True), dict(gate=True, stats=True))
            q = f"seg{i}.basic"
            self._bn(q + ".bn1", o, px2); self._bn(q + ".bn2", o, px2)
            for nm in (".a", ".c1", ".a2", ".out", ".g", ".gx"):
                self._act(q + nm, (N, s2, s2, o))
            self._conv_plans(q + ".conv1", s2, o, o, 3, 1, dict(stats=True), dict(gate=True, stats=True))
            self._conv_plans(q + ".conv2", s2, o, o, 3, 1, dict(resid=True, stats=True), dict(gate=True, stats=True))
            self.blocks.append((i, c, o, s, s2))
            c, s = o, s2
        self.final_c, self.final_s = c, s
        self._bn("tail_bn", c, N * s * s)
        self._act("t", (N, s, s, c)); self._act("y", (N, s, s, self.classes)); self._act("dy", (N, s, s, self.classes))
        self._act("tail.g", (N, s, s, c)); self._act("dlast", (N, s, s, c))
        self._conv_plans("tail", s, c, self.classes, 1, 1, dict(), dict(gate=True, stats=True))
        self.add_vec = None

    # -- parameter I/O ------------------------------------------------------------------------------------
    def load_params(self, params: Dict[str, np.ndarray]) -> None:
        torch = self.torch
        for n, k, shape in self.spec:
            t = torch.from_numpy(np.ascontiguousarray(params[n], dtype=np.float32)).to(self.dev)
            flat = self.w_conv if k == "conv" else self.w_vec
            flat[self.offs[n]: self.offs[n] + t.numel()].copy_(t.reshape(-1))
        self.w16_conv.copy_(self.w_conv.to(torch.bfloat16))   # set-up only: the step keeps this copy current itself
        self.avg_conv.zero_(); self.avg_vec.zero_()
        self.first_step = True

    def params_to_host(self) -> Dict[str, np.ndarray]:
        out = {}
        for n, k, shape in self.spec:
            flat = self.w_conv if k == "conv" else self.w_vec
            out[n] = flat[self.offs[n]: self.offs[n] + int(np.prod(shape))].view(shape).cpu().numpy()
        return out

    # -- C ABI helpers ------------------------------------------------------------------------------------
    def _st(self):
        return C.c_void_p(_stream_ptr(None))

    def _ws_ptr(self):
        return (self.ws.data_ptr() + 255) // 256 * 256

    def _launch(self, key, ins, outs):
        self.plans[key].launch_ptrs([t.data_ptr() for t in ins], [t.data_ptr() for t in outs], self._ws_ptr())
        self.launches += self.plans[key].last_launch_count

    def _bn_finalize(self, name, count, gamma, beta):
        b = self.bns[name]
        rm, rv = self.running[name.replace("#2", "")]
        check(lib.he_bn_finalize(b.stats.data_ptr(), count, gamma.data_ptr(), beta.data_ptr(), rm.data_ptr(), rv.data_ptr(),
                                 b.scale.data_ptr(), b.shift.data_ptr(), b.mean.data_ptr(), b.rstd.data_ptr(), gamma.numel(), self._st()))
        self.launches += 1

    def _bn_apply(self, name, x, y, stats_out=None):
        b = self.bns[name]
        c = x.shape[-1]
        check(lib.he_bn_apply(x.data_ptr(), y.data_ptr(), b.scale.data_ptr(), b.shift.data_ptr(), x.numel() // c, c, 1,
                              stats_out.data_ptr() if stats_out is not None else None, self._ws_ptr(), self._st()))
        self.launches += 1 + (1 if stats_out is not None else 0)

    def _bn_backward(self, name, g, x, out, gamma_name, second=False, addend=None, mask=None, colsum_to=None):
        """dx = A g + B x + K (+ addend) from the sums in bns[name].bstats; writes dgamma / dbeta into the gradient
        buffers (the second application of a shared norm goes to the second buffer).  `colsum_to` receives the
        column sums of `out`: the bias gradient of the convolution that `out` flows into next."""
        b = self.bns[name]
        c = x.shape[-1]
        pixels = x.numel() // c
        GV = self.GV2 if second else self.GV
        gam = self.V[gamma_name + ".g"]
        check(lib.he_bn_backward_coeffs(b.bstats.data_ptr(), pixels, gam.data_ptr(), b.mean.data_ptr(), b.rstd.data_ptr(), b.coef.data_ptr(),
                                        GV[gamma_name + ".g"].data_ptr(), GV[gamma_name + ".b"].data_ptr(), c, self._st()))
        if mask is None:
            check(lib.he_bn_backward_apply(g.data_ptr(), x.data_ptr(), addend.data_ptr() if addend is not None else None, out.data_ptr(),
                                           b.coef.data_ptr(), None, None, None, colsum_to.data_ptr() if colsum_to is not None else None,
                                           self._ws_ptr() if colsum_to is not None else None, pixels, c, self._st()))
            self.launches += 2 + (1 if colsum_to is not None else 0)
        else:
            mx, mb = mask   # (tensor, _Bn whose scale / shift define the rectifier) ; statistics go to that norm's bstats
            check(lib.he_bn_backward_apply(g.data_ptr(), x.data_ptr(), addend.data_ptr() if addend is not None else None, out.data_ptr(),
                                           b.coef.data_ptr(), mx.data_ptr(), mb.scale.data_ptr(), mb.shift.data_ptr(), mb.bstats.data_ptr(),
                                           self._ws_ptr(), pixels, c, self._st()))
            self.launches += 3

    def _colsum(self, x, out):
        c = x.shape[-1]
        check(lib.he_colsum_bf16(x.data_ptr(), out.data_ptr(), self._ws_ptr(), x.numel() // c, c, self._st()))
        self.launches += 2

    # -- one training step --------------------------------------------------------------------------------
    def forward(self) -> None:
        A, W, V, B = self.acts, self.W16, self.V, self.bns
        N = self.N
        check(lib.he_im2col_nhwc(A["x0"].data_ptr(), A["cols"].data_ptr(), N, self.hw, self.hw, IMG_CHANNELS, 7, 7, 2, HEAD_K, self._st()))
        self.launches += 1
        self._launch("head.fwd", [A["cols"], W["head.w"], V["head.b"]], [A["h"], B["seg0.down.bn1"].stats])
        x = A["h"]
        for (i, c, o, s, s2) in self.blocks:
            p, q = f"seg{i}.down", f"seg{i}.basic"
            px, px2 = N * s * s, N * s2 * s2
            # downsample block
            self._bn_finalize(p + ".bn1", px, V[p + ".bn1.g"], V[p + ".bn1.b"])
            self._bn_apply(p + ".bn1", x, A[p + ".a"], stats_out=B[p + ".bn1#2"].stats)
            self._launch(p + ".sc.fwd", [A[p + ".a"], W[p + ".sc.w"], V[p + ".sc.b"]], [A[p + ".sc"]])
            self._bn_finalize(p + ".bn1#2", px, V[p + ".bn1.g"], V[p + ".bn1.b"])
            self._bn_apply(p + ".bn1#2", A[p + ".a"], A[p + ".a2"])
            self._launch(p + ".conv1.fwd", [A[p + ".a2"], W[p + ".conv1.w"], V[p + ".conv1.b"]], [A[p + ".c1"], B[p + ".bn2"].stats])
            self._bn_finalize(p + ".bn2", px2, V[p + ".bn2.g"], V[p + ".bn2.b"])
            self._bn_apply(p + ".bn2", A[p + ".c1"], A[p + ".a3"])
            self._launch(p + ".conv2.fwd", [A[p + ".a3"], W[p + ".conv2.w"], V[p + ".conv2.b"], A[p + ".sc"]], [A[p + ".out"], B[q + ".bn1"].stats])
            # basic block
            xin = A[p + ".out"]
            self._bn_finalize(q + ".bn1", px2, V[q + ".bn1.g"], V[q + ".bn1.b"])
            self._bn_apply(q + ".bn1", xin, A[q + ".a"])
            self._launch(q + ".conv1.fwd", [A[q + ".a"], W[q + ".conv1.w"], V[q + ".conv1.b"]], [A[q + ".c1"], B[q + ".bn2"].stats])
            self._bn_finalize(q + ".bn2", px2, V[q + ".bn2.g"], V[q + ".bn2.b"])
            self._bn_apply(q + ".bn2", A[q + ".c1"], A[q + ".a2"])
            nxt = B["tail_bn"] if i == 3 else B[f"seg{i + 1}.down.bn1"]
            self._launch(q + ".conv2.fwd", [A[q + ".a2"], W[q + ".conv2.w"], V[q + ".conv2.b"], xin], [A[q + ".out"], nxt.stats])
            x = A[q + ".out"]
        self.x_last = x
        s = self.final_s
        self._bn_finalize("tail_bn", N * s * s, V["tail_bn.g"], V["tail_bn.b"])
        self._bn_apply("tail_bn", x, A["t"])
        self._launch("tail.fwd", [A["t"], W["tail.w"], V["tail.b"]], [A["y"]])
        check(lib.he_pool_softmax_ce(A["y"].data_ptr(), self.labels.data_ptr(), self.loss.data_ptr(), A["dy"].data_ptr(), N, s * s,
                                     self.classes, self._st()))
        self.launches += 1

    def backward(self) -> None:
        A, W, V, B, GW, GV = self.acts, self.W16, self.V, self.bns, self.GW, self.GV
        x = self.x_last
        # tail: 1x1 convolution, then relu(bn(x_last))
        self._launch("tail.wgrad", [A["dy"], A["t"]], [GW["tail.w"]])
        self._colsum(A["dy"], GV["tail.b"])
        tb = B["tail_bn"]
        self._launch("tail.dgrad", [A["dy"], W["tail.w"], x, tb.scale, tb.shift], [A["tail.g"], tb.bstats])
        self._bn_backward("tail_bn", A["tail.g"], x, A["dlast"], "tail_bn", colsum_to=GV[f"seg{self.blocks[-1][0]}.basic.conv2.b"])
        dout = A["dlast"]
        for (i, c, o, s, s2) in reversed(self.blocks):
            p, q = f"seg{i}.down", f"seg{i}.basic"
            xin = A[p + ".out"]
            # ---- basic block: out = conv2(relu(bn2(conv1(relu(bn1(xin)))))) + xin
            # (the bias gradients, column sums of each flow, come out of the pass that produced the flow)
            self._launch(q + ".conv2.wgrad", [dout, A[q + ".a2"]], [GW[q + ".conv2.w"]])
            b2 = B[q + ".bn2"]
            self._launch(q + ".conv2.dgrad", [dout, W[q + ".conv2.w"], A[q + ".c1"], b2.scale, b2.shift], [A[q + ".g"], b2.bstats])
            self._bn_backward(q + ".bn2", A[q + ".g"], A[q + ".c1"], A[q + ".gx"], q + ".bn2", colsum_to=GV[q + ".conv1.b"])   # gradient at c1
            dc1 = A[q + ".gx"]
            self._launch(q + ".conv1.wgrad", [dc1, A[q + ".a"]], [GW[q + ".conv1.w"]])
            b1 = B[q + ".bn1"]
            self._launch(q + ".conv1.dgrad", [dc1, W[q + ".conv1.w"], xin, b1.scale, b1.shift], [A[q + ".g"], b1.bstats])
            self._bn_backward(q + ".bn1", A[q + ".g"], xin, A[p + ".g"], q + ".bn1", addend=dout, colsum_to=GV[p + ".conv2.b"])   # gradient at xin (+ the skip)
            dout = A[p + ".g"]
            # ---- downsample block: out = conv2(relu(bn2(conv1(relu(bn1(a)))))) + sc(a),  a = relu(bn1(x))
            xprev = A["h"] if i == 0 else A[f"seg{i - 1}.basic.out"]
            self._launch(p + ".conv2.wgrad", [dout, A[p + ".a3"]], [GW[p + ".conv2.w"]])
            self.torch_copy(GV[p + ".sc.b"], GV[p + ".conv2.b"])       # both biases see the same flow
            self._launch(p + ".sc.wgrad", [dout, A[p + ".a"]], [GW[p + ".sc.w"]])
            self._launch(p + ".sc.dgrad", [dout, W[p + ".sc.w"]], [A[p + ".dsc"]])
            b2 = B[p + ".bn2"]
            self._launch(p + ".conv2.dgrad", [dout, W[p + ".conv2.w"], A[p + ".c1"], b2.scale, b2.shift], [A[q + ".g"], b2.bstats])
            self._bn_backward(p + ".bn2", A[q + ".g"], A[p + ".c1"], A[q + ".gx"], p + ".bn2", colsum_to=GV[p + ".conv1.b"])   # gradient at c1
            dc1 = A[q + ".gx"]
            self._launch(p + ".conv1.wgrad", [dc1, A[p + ".a2"]], [GW[p + ".conv1.w"]])
            b12, b11 = B[p + ".bn1#2"], B[p + ".bn1"]
            self._launch(p + ".conv1.dgrad", [dc1, W[p + ".conv1.w"], A[p + ".a"], b12.scale, b12.shift], [A[p + ".ga"], b12.bstats])
            # second application of bn1 (on a), plus the shortcut's gradient, masked by the first rectifier
            self._bn_backward(p + ".bn1#2", A[p + ".ga"], A[p + ".a"], A[p + ".gx"], p + ".bn1", second=True, addend=A[p + ".dsc"],
                              mask=(xprev, b11))
            if i == 0:
                # nothing upstream of the head needs a gradient: only dgamma / dbeta of the first application
                b = b11
                check(lib.he_bn_backward_coeffs(b.bstats.data_ptr(), xprev.numel() // c, V[p + ".bn1.g"].data_ptr(), b.mean.data_ptr(),
                                                b.rstd.data_ptr(), b.coef.data_ptr(), GV[p + ".bn1.g"].data_ptr(), GV[p + ".bn1.b"].data_ptr(),
                                                c, self._st()))
                self.launches += 1
                # the head still needs the gradient at its output
                check(lib.he_bn_backward_apply(A[p + ".gx"].data_ptr(), xprev.data_ptr(), None, A[p + ".ga"].data_ptr(), b.coef.data_ptr(),
                                               None, None, None, GV["head.b"].data_ptr(), self._ws_ptr(), xprev.numel() // c, c, self._st()))
                self.launches += 2
                dout = A[p + ".ga"]
            else:
                self._bn_backward(p + ".bn1", A[p + ".gx"], xprev, A[p + ".ga"], p + ".bn1", colsum_to=GV[f"seg{i - 1}.basic.conv2.b"])
                dout = A[p + ".ga"]
        self._launch("head.wgrad", [dout, A["cols"]], [GW["head.w"]])

    def torch_copy(self, dst, src):
        """Device-to-device copy of a small parameter-gradient vector (a cudaMemcpyAsync on the current stream)."""
        dst.copy_(src, non_blocking=True)

    def optimizer_step(self, lr: float) -> None:
        # parameters used twice (bn1 of the downsample blocks): add the second contribution
        check(lib.he_sgd_momentum(self.g_vec.data_ptr(), None, self.g_vec2.data_ptr(), ir.F32, None, self.n_vec, -1.0, 0.0, 1, self._st()))
        first = 1 if self.first_step else 0
        check(lib.he_sgd_momentum(self.w_conv.data_ptr(), self.avg_conv.data_ptr(), self.g_conv.data_ptr(), ir.BF16, self.w16_conv.data_ptr(),
                                  self.n_conv, lr, self.momentum, first, self._st()))
        check(lib.he_sgd_momentum(self.w_vec.data_ptr(), self.avg_vec.data_ptr(), self.g_vec.data_ptr(), ir.F32, None, self.n_vec, lr,
                                  self.momentum, first, self._st()))
        self.first_step = False
        self.launches += 3

    def step(self, lr: float = 0.01, reducer=None, graph: bool = False, mark=None) -> None:
        """Forward, backward, (gradient mean over ranks,) optimiser.  Images are in acts["x0"], labels in self.labels.
        With `graph` the ~270 launches are replayed from three CUDA graphs (forward, backward, optimiser) captured
        on the second call with this learning rate; the gradient exchange stays an ordinary call between them.
        `mark(tag)` is called on the host at the phase boundaries ("start", "forward", "backward", "end"), e.g. to
        record events on the stream."""
        mark = mark or (lambda tag: None)
        use_graphs = graph and not self.first_step
        if use_graphs and (self._graphs is None or self._graphs[0] != lr):
            self._capture(lr)
        mark("start")
        if use_graphs:
            self._graphs[1].replay()
        else:
            self.launches = 0
            self.g_vec2.zero_()
            self.forward()
        mark("forward")
        if use_graphs:
            self._graphs[2].replay()
        else:
            self.backward()
        mark("backward")
        if reducer is not None:
            reducer.reduce_bucket([self.g_conv])
            reducer.reduce_bucket([self.g_vec, self.g_vec2])
            reducer.finish()
        if use_graphs:
            self._graphs[3].replay()
            self.launches = self._graphs[4]
        else:
            self.optimizer_step(lr)
        mark("end")

    def _capture(self, lr):
        torch = self.torch
        torch.cuda.synchronize(self.dev)
        self.ctx.poll()
        gf, gb, go = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        # the step's own buffers are all allocated; capture records the launches without running them
        self.launches = 0
        with torch.cuda.graph(gf):
            self.g_vec2.zero_()
            self.forward()
        with torch.cuda.graph(gb):
            self.backward()
        with torch.cuda.graph(go):
            self.optimizer_step(lr)
        self._graphs = (lr, gf, gb, go, self.launches)


def synthetic_batch(batch: int, hw: int = 224, classes: int = 1000, seed: int = 4, shard: int = 0):
    """Images ~ N(0,1) as bf16 bits [N, hw, hw, 3] and labels uniform over the classes."""
    r = np.random.Generator(np.random.Philox(seed + 7919 * (shard + 1)))
    img = r.standard_normal((batch, hw, hw, IMG_CHANNELS), dtype=np.float32)
    b = img.view(np.uint32).astype(np.uint64)
    bits = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)
    labels = r.integers(0, classes, size=batch).astype(np.int32)
    return bits, labels
