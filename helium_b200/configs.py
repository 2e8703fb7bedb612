"""The benchmark configurations of this path as op graphs plus seeded synthetic inputs.

Graphs are built the way helium's front end would record them (helium/src/raw_tensor.rs) or, for
the fused matmul, the way the playground prints them (README.md:33-79).  Inputs are numpy storage
arrays (uint16 bit patterns for bf16) drawn from a counter-based generator (Philox) with the seed
each configuration names, so that every consumer -- kernels, oracle, CPU baseline -- reads identical
bytes.  No dataset is involved.
"""
from __future__ import annotations

import numpy as np

from . import ir


def rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(seed))


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (host-side input preparation only)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_normal(g: np.random.Generator, shape, std: float = 1.0) -> np.ndarray:
    return f32_to_bf16_bits(g.standard_normal(shape, dtype=np.float32) * np.float32(std))


def bf16_bernoulli(g: np.random.Generator, shape, p: float = 0.5) -> np.ndarray:
    return f32_to_bf16_bits((g.random(shape, dtype=np.float32) < p).astype(np.float32))


def graph_affine_relu_permute(n, c, h, w, x_dtype=ir.BF16, p_dtype=ir.F32) -> ir.Graph:
    """The fused affine + relu + layout change benchmark graph: relu(x * s_c + b_c) on NCHW, written NHWC (swap_dims(1,2).swap_dims(2,3))."""
    g = ir.Graph()
    x = g.new_input([n, c, h, w], x_dtype)
    s = g.new_input([c], p_dtype)
    b = g.new_input([c], p_dtype)
    sb = g.broadcast_to(g.reshape(s, [c, 1, 1]), [n, c, h, w])
    bb = g.broadcast_to(g.reshape(b, [c, 1, 1]), [n, c, h, w])
    y = g.unary(ir.UN_RELU, g.binary(ir.BIN_ADD, g.binary(ir.BIN_MUL, x, sb), bb))
    y = g.swap_dims(g.swap_dims(y, 1, 2), 2, 3)
    g.new_output(y)
    return g


def graph_c3(m: int, n: int, k: int, with_e: bool = False, dtype=ir.BF16):
    """The fused graph of the reference README (README.md:33-79), node numbers in comments.

    Inputs in order: A [1,m,k], Mk [1,m,k] (mainloop mask), B [1,k,n], b1 [1,1,n], b2 [1,1,n],
    M [1,m,n] (epilogue mask; the same tensor as Mk when k == n), Y [1,m,n] (, E1, E2).
    Outputs: LOSS [1,1,1], DB2 [1,1,n], DB1 [1,1,n], gt [1,m,n], gz1 [1,m,n].
    """
    inv = 1.0 / n
    g = ir.Graph()
    a = g.new_input([1, m, k], dtype)            # 22
    mk_ml = g.new_input([1, m, k], dtype)        # 9 (mainloop use)
    bmat = g.new_input([1, k, n], dtype)
    b1 = g.new_input([1, 1, n], dtype)           # 6
    b2 = g.new_input([1, 1, n], dtype)           # 8
    mk = g.new_input([1, m, n], dtype)           # 9 (epilogue use)
    y = g.new_input([1, m, n], dtype)            # 11
    a2 = g.binary(ir.BIN_MUL, g.unary(ir.UN_RELU, a), mk_ml)   # 23, 25
    acc = g.matmul(a2, bmat, ir.PREC_BF16_F32)
    n14 = n27 = acc
    if with_e:
        e1 = g.new_input([1, m, n], dtype)       # 13
        e2 = g.new_input([1, m, n], dtype)       # 26
        n14 = g.binary(ir.BIN_ADD, acc, e1)      # 14
        n27 = g.binary(ir.BIN_ADD, acc, e2)      # 27
    n16 = g.binary(ir.BIN_ADD, n14, g.broadcast(b1, 3, [(1, m)]))     # 15, 16
    n17 = g.unary(ir.UN_RELU, n16)                                     # 17
    n29 = g.binary(ir.BIN_ADD, n27, g.broadcast(b2, 3, [(1, m)]))     # 28, 29
    n30 = g.unary(ir.UN_TANH, n29)                                     # 30
    n32 = g.unary(ir.UN_ADD_CONST, g.unary(ir.UN_NEG, n17), 1.0)       # 31, 32
    n33 = g.binary(ir.BIN_MUL, n32, mk)                                # 33
    n34 = g.binary(ir.BIN_MUL, n17, n30)                               # 34
    n35 = g.binary(ir.BIN_ADD, n33, n34)                               # 35
    n36 = g.binary(ir.BIN_SUB, n35, y)                                 # 36
    n37 = g.unary(ir.UN_POW_CONST, n36, 2.0)                           # 37
    n38 = g.unary(ir.UN_MUL_CONST, n37, inv)                           # 38
    n39 = g.reduce_axes(ir.RED_SUM, n38, [0, 1, 2])                    # 39 Batch
    n41 = g.constant(1.0, [1, 1, 1])                                   # 41
    n44 = g.broadcast(g.broadcast(g.broadcast(n41, 3, [(1, m)]), 3, [(2, n)]), 3, [(0, 1)])  # 42-44
    n45 = g.unary(ir.UN_MUL_CONST, n44, inv)                           # 45
    n46 = g.constant(2.0, [1, m, n])                                   # 46
    n47 = g.constant(1.0, [1, m, n])                                   # 47
    n48 = g.binary(ir.BIN_POW, n36, n47)                               # 48
    n49 = g.binary(ir.BIN_MUL, n48, n46)                               # 49
    n50 = g.binary(ir.BIN_MUL, n49, n45)                               # 50
    n52 = g.binary(ir.BIN_MUL, n50, n30)                               # 52
    n53 = g.binary(ir.BIN_MUL, n17, n50)                               # 53
    n56 = g.unary(ir.UN_ADD_CONST, g.unary(ir.UN_NEG, g.unary(ir.UN_POW_CONST, n30, 2.0)), 1.0)  # 54-56
    n57 = g.binary(ir.BIN_MUL, n53, n56)                               # 57
    n58 = g.reduce_axes(ir.RED_SUM, n57, [1])                          # 58 Columns
    n81 = g.binary(ir.BIN_MUL, n50, mk)                                # 81
    n85 = g.binary(ir.BIN_ADD, n52, g.unary(ir.UN_NEG, n81))           # 84, 85
    n86 = g.binary(ir.BIN_DRELU, n85, n16)                             # 86
    n87 = g.reduce_axes(ir.RED_SUM, n86, [1])                          # 87 Columns
    gt = g.cast(n57, dtype)
    gz1 = g.cast(n86, dtype)
    for o in (n39, n58, n87, gt, gz1):
        g.new_output(o)
    return g


def graph_linear(m, n, k, bias=True, act=None, resid=False, store_z=False, a_t=False, b_t=False, dtype=ir.BF16,
                 out_dtype=None, gate=None, colsum=None, batch=None, precision=None):
    """act(A @ B + bias (+ resid)) (* gate(G)) with optional transposed operand storage.

    a_t: A is stored [k, m] and transposed in the graph; b_t: B stored [n, k] and transposed.
    Input order: A, B, [bias], [resid], [gate].  Output order: y, [z], [colsum]."""
    g = ir.Graph()
    lead = [] if batch is None else [batch]
    a = g.new_input(lead + ([k, m] if a_t else [m, k]), dtype)
    b = g.new_input(lead + ([n, k] if b_t else [k, n]), dtype)
    am = g.transpose(a) if a_t else a
    bm = g.transpose(b) if b_t else b
    prec = {ir.BF16: ir.PREC_BF16_F32, ir.F16: ir.PREC_F16_F32, ir.F32: ir.PREC_TF32_F32}[dtype] if precision is None else precision
    t = g.matmul(am, bm, prec)
    rnk = len(lead) + 2
    r_in = None
    if bias:
        bv = g.new_input([n], dtype)
        t = g.binary(ir.BIN_ADD, t, g.broadcast_to(bv, lead + [m, n]))
    if resid:
        r_in = g.new_input(lead + [m, n], dtype)
        t = g.binary(ir.BIN_ADD, t, r_in)
    z = t
    y = t
    if act is not None:
        y = g.unary(act, y)
    if gate is not None:
        gi = g.new_input(lead + [m, n], dtype)
        if gate == "mul":
            y = g.binary(ir.BIN_MUL, y, gi)
        elif gate == "dgelu":
            y = g.binary(ir.BIN_MUL, y, g.unary(ir.UN_DGELU, gi))
        elif gate == "drelu":
            y = g.binary(ir.BIN_DRELU, y, gi)
    od = out_dtype if out_dtype is not None else dtype
    g.new_output(g.cast(y, od))
    if store_z:
        g.new_output(g.cast(z, od))
    if colsum == "resid":
        g.new_output(g.reduce_axes(ir.RED_SUM, r_in, [rnk - 2]))
    elif colsum == "y":
        g.new_output(g.reduce_axes(ir.RED_SUM, y, [rnk - 2]))
    return g



def c2_inputs(seed: int = 1):
    """configs[1]: x bf16 [64,256,56,56] ~ N(0,1), s ~ U[0.5,1.5], b ~ N(0,0.1) per channel (f32),
    and the f32 tensor [4096,4096,8] ~ N(0,1) of the stand-alone permutation."""
    g = rng(seed)
    x = bf16_normal(g, (64, 256, 56, 56))
    s = g.random(256, dtype=np.float32) + np.float32(0.5)
    b = g.standard_normal(256, dtype=np.float32) * np.float32(0.1)
    p = g.standard_normal((4096, 4096, 8), dtype=np.float32)
    return x, s, b, p


def c3_inputs(m: int, n: int, k: int, with_e: bool = False, seed: int = 2):
    """configs[2] operands in graph_c3 input order: A ~ N(0,1), mask ~ Bernoulli(0.5), B ~ N(0,1/sqrt(k)),
    b1, b2 ~ N(0,0.02), epilogue mask (the mainloop mask when k == n), Y ~ N(0,1) (, E1, E2 ~ N(0,1))."""
    r = rng(seed)
    a = bf16_normal(r, (1, m, k))
    mk_ml = bf16_bernoulli(r, (1, m, k))
    b = bf16_normal(r, (1, k, n), 1 / np.sqrt(k))
    b1 = bf16_normal(r, (1, 1, n), 0.02)
    b2 = bf16_normal(r, (1, 1, n), 0.02)
    mk = mk_ml if k == n else bf16_bernoulli(r, (1, m, n))
    y = bf16_normal(r, (1, m, n))
    ins = [a, mk_ml, b, b1, b2, mk, y]
    if with_e:
        ins += [bf16_normal(r, (1, m, n)), bf16_normal(r, (1, m, n))]
    return ins


def graph_mlp_train_step(batch: int = 256, d_in: int = 784, d_hidden: int = 512, d_out: int = 10, lr: float = 0.01):
    """configs[0]: one SGD step of the MLP 784 -> 512 -> 10 (ReLU, softmax cross-entropy) in f32,
    recorded op by op the way helium's front end would: `Linear::forward` (modules/linear.rs:44-57),
    `cross_entropy_loss` / `log_softmax` (loss.rs:5-8, tensor.rs:584-592), the backward formulas of
    tensor.rs:316-580 (matmul: dA = flow @ B^T, dB = A^T @ flow, tensor.rs:446-447; relu:
    select(x < 0, 0, 1) * flow, tensor.rs:374-387; broadcast: sum over the broadcast axis) and
    `Sgd::step` without momentum (optimizer/sgd.rs:48).

    Inputs: x [B,d_in], targets (one-hot) [B,d_out], W1 [d_in,H], b1 [H], W2 [H,d_out], b2 [d_out].
    Outputs: loss [1], W1', b1', W2', b2'."""
    g = ir.Graph()
    F = ir.F32
    B, H, O = batch, d_hidden, d_out
    x = g.new_input([B, d_in], F)
    t = g.new_input([B, O], F)
    w1 = g.new_input([d_in, H], F)
    b1 = g.new_input([H], F)
    w2 = g.new_input([H, O], F)
    b2 = g.new_input([O], F)
    prec = ir.PREC_TF32_F32
    # forward
    z1 = g.binary(ir.BIN_ADD, g.matmul(x, w1, prec), g.broadcast_to(b1, [B, H]))
    h = g.unary(ir.UN_RELU, z1)
    z2 = g.binary(ir.BIN_ADD, g.matmul(h, w2, prec), g.broadcast_to(b2, [B, O]))
    mx = g.broadcast_to(g.reduce(ir.RED_MAX, z2, 1), [B, O])
    zs = g.binary(ir.BIN_ADD, z2, g.unary(ir.UN_NEG, mx))
    se = g.reduce(ir.RED_SUM, g.unary(ir.UN_EXP, zs), 1)                       # [B,1]
    ls = g.binary(ir.BIN_ADD, zs, g.unary(ir.UN_NEG, g.broadcast_to(g.unary(ir.UN_LOG, se), [B, O])))
    prod = g.binary(ir.BIN_MUL, ls, t)
    total = g.reduce(ir.RED_SUM, prod, 2)                                       # [1]
    loss = g.binary(ir.BIN_MUL, g.unary(ir.UN_NEG, total), g.constant(1.0 / B, [1]))
    # backward: d loss / d z2 = (softmax - t * sum(t)) / B; targets are one-hot so sum(t) = 1
    sm = g.unary(ir.UN_EXP, ls)
    dz2 = g.binary(ir.BIN_MUL, g.binary(ir.BIN_ADD, sm, g.unary(ir.UN_NEG, t)), g.constant(1.0 / B, [B, O]))
    dw2 = g.matmul(g.transpose(h), dz2, prec)                                   # [H,O]
    db2 = g.reshape(g.reduce(ir.RED_SUM, g.transpose(dz2), 1), [O])             # sum over the batch
    dh = g.matmul(dz2, g.transpose(w2), prec)                                   # [B,H]
    neg = g.compare(ir.CMP_LT, z1, g.constant(0.0, [B, H]))
    dz1 = g.binary(ir.BIN_MUL, g.select(g.constant(1.0, [B, H]), g.constant(0.0, [B, H]), neg), dh)
    dw1 = g.matmul(g.transpose(x), dz1, prec)                                   # [d_in,H]
    db1 = g.reshape(g.reduce(ir.RED_SUM, g.transpose(dz1), 1), [H])
    # SGD: w - g * lr
    def sgd(w, grad, shape):
        return g.binary(ir.BIN_ADD, w, g.unary(ir.UN_NEG, g.binary(ir.BIN_MUL, grad, g.constant(lr, shape))))
    outs = [loss, sgd(w1, dw1, [d_in, H]), sgd(b1, db1, [H]), sgd(w2, dw2, [H, O]), sgd(b2, db2, [O])]
    for o in outs:
        g.new_output(o)
    return g


def mlp_inputs(batch: int = 256, d_in: int = 784, d_hidden: int = 512, d_out: int = 10, seed: int = 0):
    """x ~ U[-1,1], labels uniform -> one-hot, weights N(0, 1/sqrt(fan_out)) (helium's "Kaiming",
    initializer.rs:29-31,48-50), biases zero."""
    r = rng(seed)
    x = (r.random((batch, d_in), dtype=np.float32) * 2 - 1).astype(np.float32)
    labels = r.integers(0, d_out, batch)
    t = np.eye(d_out, dtype=np.float32)[labels]
    w1 = (r.standard_normal((d_in, d_hidden), dtype=np.float32) / np.float32(np.sqrt(d_hidden))).astype(np.float32)
    w2 = (r.standard_normal((d_hidden, d_out), dtype=np.float32) / np.float32(np.sqrt(d_out))).astype(np.float32)
    return [x, t, w1, np.zeros(d_hidden, np.float32), w2, np.zeros(d_out, np.float32)]


def graph_mlp_block_train(tokens: int, d: int, ff: int, dtype=ir.BF16, return_nodes: bool = False):
    """configs[3] as ONE op graph, recorded the way helium's front end would record a transformer MLP
    block and its backward pass: every matmul result is cast back to the operand dtype
    (raw_tensor.rs:225-229), gradients use explicit transposes (tensor.rs:437-450) and bias
    gradients are swap_dims -> reduce_sum -> reshape (tensor.rs:83-142).

    Inputs: X [T,d], W1 [d,ff], b1 [ff], W2 [ff,d], b2 [d], dO [T,d].
    Outputs: O, dX, dW1, db1, dW2, db2.  With return_nodes the node ids of z, h and dz are returned
    too: a plan with one kernel per matmul materialises exactly those three between kernels."""
    g = ir.Graph()
    T = tokens
    x = g.new_input([T, d], dtype)
    w1 = g.new_input([d, ff], dtype)
    b1 = g.new_input([ff], dtype)
    w2 = g.new_input([ff, d], dtype)
    b2 = g.new_input([d], dtype)
    do = g.new_input([T, d], dtype)
    mm = lambda a, b: g.cast(g.matmul(a, b, ir.PREC_BF16_F32), dtype)
    z = g.binary(ir.BIN_ADD, mm(x, w1), g.broadcast_to(b1, [T, ff]))
    h = g.unary(ir.UN_GELU, z)
    o = g.binary(ir.BIN_ADD, g.binary(ir.BIN_ADD, mm(h, w2), g.broadcast_to(b2, [T, d])), x)
    dz = g.binary(ir.BIN_MUL, mm(do, g.transpose(w2)), g.unary(ir.UN_DGELU, z))
    dw2 = mm(g.transpose(h), do)
    db2 = g.reshape(g.reduce(ir.RED_SUM, g.transpose(do), 1), [d])
    dw1 = mm(g.transpose(x), dz)
    db1 = g.reshape(g.reduce(ir.RED_SUM, g.transpose(dz), 1), [ff])
    dx = g.binary(ir.BIN_ADD, mm(dz, g.transpose(w1)), do)
    for t in (o, dx, dw1, db1, dw2, db2):
        g.new_output(t)
    return (g, {"z": z, "h": h, "dz": dz}) if return_nodes else g
