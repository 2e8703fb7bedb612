"""CPU oracle for the fused-kernel hot path of caelunshun/helium.

TEST INFRASTRUCTURE ONLY.  This module restates, in numpy, what the reference's kernels compute so
that the CUDA library can be checked against it.  It is imported by tests/, by
`__graft_entry__.smoke()` and by the CPU-baseline legs of bench.py -- never by the product
(`helium_b200/`), which has no CPU path.

Parity pin: the reference is Rust + run-time generated CUDA and cannot be built or run where this
oracle was written (no Rust toolchain, no GPU).  The oracle is pinned against every known-answer
vector the reference's own tests hold for this path (tests/test_oracle_golden.py lists them with
file:line); beyond those vectors -- fused GEMM epilogues, mainloop fusion, Gelu, reductions inside
a GEMM, which the reference never tests -- parity is UNPINNED and rests on the restated semantics.

What each function follows:
  * evaluate()            helium/src/cuda/instr/pointwise/jit.rs:196-588 (per-op code generation),
                          helium-ir/src/opgraph/op.rs:52-179 (output descriptors),
                          helium-playground/src/kernel_generator.rs:363-414 and
                          helium-playground/src/torch_synthesizer.rs:31-87 (playground op meanings),
                          helium-ir/src/opgraph/op.rs:272-282 (matmul contract)
  * conv2d*()             helium-ir/src/opgraph/op/conv.rs:51-95 (geometry), helium/src/raw_tensor.rs:232-330
                          (NHWC / KRSC operands), helium/src/cuda/instr/cudnn_graph.rs:182-228 (the three
                          cuDNN operations: cross-correlation, its data and filter gradients); pinned on the
                          reference's one vector, helium/tests/tensor_ops.rs:379-397
  * permute()             helium/src/cuda/instr/permute_dims/jit.rs:15-117 (out[sum s_i c_i] = in[c])
  * output_strides_*()    helium/src/cuda/instr/permute_dims.rs:158-172
  * bit-packed bools      helium/src/cuda/instr/pointwise/jit.rs:107-114, 234-237

Arithmetic is carried out in float64 (the reference uses f32 intermediates, jit.rs:731-739); results
are rounded once to the output dtype, like the reference's `static_cast` on store (jit.rs:99-106).
"""
from __future__ import annotations

import math
from typing import Dict, Iterable, List, Optional, Sequence

import numpy as np

# ---- enum values of include/helium_b200.h ---------------------------------------------------------
F16, BF16, F32, U32, BOOL = 0, 1, 2, 3, 4
OP_INPUT, OP_CONSTANT, OP_UNARY, OP_BINARY, OP_CAST, OP_REDUCE = 0, 1, 2, 3, 4, 5
OP_BROADCAST, OP_RESHAPE, OP_SWAP_DIMS, OP_COMPARE, OP_SELECT, OP_MATMUL = 6, 7, 8, 9, 10, 11
UN_RECIP, UN_NEG, UN_EXP, UN_SIN, UN_COS, UN_TAN, UN_SIGMOID, UN_TANH, UN_RELU, UN_SQRT, UN_LOG = range(11)
UN_GELU, UN_ADD_CONST, UN_MUL_CONST, UN_POW_CONST, UN_DGELU = 16, 17, 18, 19, 20
BIN_ADD, BIN_MUL, BIN_POW, BIN_MIN, BIN_MAX, BIN_AND, BIN_OR, BIN_XOR = range(8)
BIN_SUB, BIN_DIV, BIN_DRELU = 16, 17, 18
CMP_EQ, CMP_NE, CMP_LT, CMP_LE, CMP_GT, CMP_GE = range(6)
RED_SUM, RED_MEAN, RED_MAX, RED_MIN = range(4)
PREC_F32_F32, PREC_TF32_F32, PREC_BF16_F32, PREC_F16_F32, PREC_F16_F16, PREC_F8_F32, PREC_F8_F16 = range(7)
F8_E4M3, F8_E5M2 = 0, 1

try:  # scipy is present in the image; math.erf keeps the oracle usable without it
    from scipy.special import erf as _erf
except Exception:  # pragma: no cover
    _erf = np.vectorize(math.erf)


# ---- storage formats ------------------------------------------------------------------------------
def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (uint16), NaN kept quiet."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)
    nan = np.isnan(np.asarray(x, dtype=np.float32))
    return np.where(nan, np.uint16(0x7FC0), rounded)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def pack_bools(v: np.ndarray) -> np.ndarray:
    """1 bit per element, LSB first, in little-endian u32 words."""
    flat = np.asarray(v, dtype=bool).reshape(-1)
    n = flat.size
    padded = np.zeros((n + 31) // 32 * 32, dtype=bool)
    padded[:n] = flat
    return np.packbits(padded.reshape(-1, 32), axis=1, bitorder="little").view(np.uint32).reshape(-1)


def unpack_bools(words: np.ndarray, n: int) -> np.ndarray:
    bits = np.unpackbits(np.ascontiguousarray(words, dtype=np.uint32).view(np.uint8), bitorder="little")
    return bits[:n].astype(bool)


def decode(storage: np.ndarray, dtype: int, shape: Sequence[int]) -> np.ndarray:
    """Storage array (as the device holds it) -> compute-domain array (float64 / uint32 / bool)."""
    n = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
    if dtype == BF16:
        return bf16_bits_to_f32(np.asarray(storage).view(np.uint16).reshape(-1)[:n]).astype(np.float64).reshape(shape)
    if dtype == F16:
        return np.asarray(storage).view(np.float16).reshape(-1)[:n].astype(np.float64).reshape(shape)
    if dtype == F32:
        return np.asarray(storage).view(np.float32).reshape(-1)[:n].astype(np.float64).reshape(shape)
    if dtype == U32:
        return np.asarray(storage).view(np.uint32).reshape(-1)[:n].reshape(shape)
    return unpack_bools(np.asarray(storage).view(np.uint32), n).reshape(shape)


def encode(value: np.ndarray, dtype: int) -> np.ndarray:
    """Compute-domain array -> storage array: one rounding to the tensor dtype."""
    if dtype == BF16:
        return f32_to_bf16_bits(np.asarray(value, dtype=np.float64).astype(np.float32))
    if dtype == F16:
        return np.asarray(value, dtype=np.float64).astype(np.float32).astype(np.float16)
    if dtype == F32:
        return np.asarray(value, dtype=np.float64).astype(np.float32)
    if dtype == U32:
        return np.asarray(value).astype(np.uint32)
    return pack_bools(value)


def round_to(value: np.ndarray, dtype: int) -> np.ndarray:
    """Value after a store + load round trip in `dtype`, back in the compute domain."""
    if dtype in (BF16, F16, F32):
        return decode(encode(value, dtype), dtype, value.shape)
    return value


def round_to_f8(value: np.ndarray, mode: int) -> np.ndarray:
    """Nearest-even rounding to the 8-bit float of F8Mode (helium-ir/src/opgraph/op/precision.rs:100-108),
    saturating at the largest finite value: E4M3 (bias 7, max 448) or E5M2 (bias 15, max 57344).  Only
    used to draw the error envelope of the reference's 8-bit multiplication; the library multiplies at
    the operand dtype, which the precision contract allows (precision.rs:3-9)."""
    man, emin, vmax = (3, -6, 448.0) if mode == F8_E4M3 else (2, -14, 57344.0)
    x = np.asarray(value, dtype=np.float64)
    mag = np.abs(x)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(mag > 0, mag, 1.0)))
    quantum = np.exp2(np.maximum(e, emin) - man)
    q = np.rint(mag / quantum) * quantum
    return np.sign(x) * np.minimum(q, vmax)


def _const_value(bits: int, dtype: int):
    if dtype == F32:
        return float(np.array([bits], dtype=np.uint32).view(np.float32)[0])
    if dtype == BF16:
        return float(bf16_bits_to_f32(np.array([bits], dtype=np.uint16))[0])
    if dtype == F16:
        return float(np.array([bits], dtype=np.uint16).view(np.float16)[0])
    if dtype == U32:
        return np.uint32(bits)
    return bool(bits)


def _f32bits(bits: int) -> float:
    return float(np.array([bits], dtype=np.uint32).view(np.float32)[0])


def _is_float(dt: int) -> bool:
    return dt in (F16, BF16, F32)


# ---- op semantics -----------------------------------------------------------------------------------
def _unary(op: int, x: np.ndarray, const: float) -> np.ndarray:
    with np.errstate(all="ignore"):
        if op == UN_RECIP: return 1.0 / x
        if op == UN_NEG: return -x
        if op == UN_EXP: return np.exp(x)
        if op == UN_SIN: return np.sin(x)
        if op == UN_COS: return np.cos(x)
        if op == UN_TAN: return np.tan(x)
        if op == UN_SIGMOID: return 1.0 / (1.0 + np.exp(-x))
        if op == UN_TANH: return np.tanh(x)
        if op == UN_RELU: return np.maximum(x, 0.0)
        if op == UN_SQRT: return np.sqrt(x)
        if op == UN_LOG: return np.log(x)
        if op == UN_GELU: return 0.5 * x * (1.0 + _erf(x / math.sqrt(2.0)))
        if op == UN_ADD_CONST: return x + const
        if op == UN_MUL_CONST: return x * const
        if op == UN_POW_CONST: return x * x if const == 2.0 else np.power(x, const)
        if op == UN_DGELU:
            return 0.5 * (1.0 + _erf(x / math.sqrt(2.0))) + x * np.exp(-0.5 * x * x) / math.sqrt(2.0 * math.pi)
    raise ValueError(f"unknown unary op {op}")


def _binary(op: int, a: np.ndarray, b: np.ndarray, is_float: bool) -> np.ndarray:
    with np.errstate(all="ignore"):
        if op == BIN_ADD: return a + b
        if op == BIN_MUL: return a * b
        if op == BIN_POW: return np.power(a, b)
        if op == BIN_MIN: return np.fmin(a, b) if is_float else np.minimum(a, b)
        if op == BIN_MAX: return np.fmax(a, b) if is_float else np.maximum(a, b)
        if op == BIN_AND: return a & b
        if op == BIN_OR: return a | b
        if op == BIN_XOR: return a ^ b
        if op == BIN_SUB: return a - b
        if op == BIN_DIV: return a / b
        if op == BIN_DRELU: return np.where(b > 0, a, 0.0)
    raise ValueError(f"unknown binary op {op}")


_CMP = {CMP_EQ: np.equal, CMP_NE: np.not_equal, CMP_LT: np.less, CMP_LE: np.less_equal,
        CMP_GT: np.greater, CMP_GE: np.greater_equal}


def evaluate(graph, inputs: Sequence[np.ndarray], round_nodes: Iterable[int] = (), return_all: bool = False,
             f8_quantise: bool = False):
    """Evaluates a graph (any object with `.nodes` / `.outputs` shaped like helium_b200.ir.Graph).

    `inputs[i]` is the storage array of the i-th OP_INPUT node (uint16 bits for bf16, float16,
    float32, uint32, or packed uint32 words for bool).  Returns the storage arrays of the outputs.
    `round_nodes`: node indices whose value is additionally rounded to the node dtype, to model a
    plan that materialises that tensor between two kernels.
    """
    round_nodes = set(round_nodes)
    vals: Dict[int, np.ndarray] = {}
    it = iter(inputs)
    for i, n in enumerate(graph.nodes):
        k = n.kind
        shape = tuple(n.shape)
        if k == OP_INPUT:
            v = decode(next(it), n.dtype, shape)
        elif k == OP_CONSTANT:
            c = _const_value(n.const_bits, n.dtype)
            v = np.full(shape, c, dtype=np.float64 if _is_float(n.dtype) else (np.uint32 if n.dtype == U32 else bool))
        elif k == OP_UNARY:
            v = _unary(n.sub_op, vals[n.inputs[0]], _f32bits(n.const_bits))
        elif k == OP_BINARY:
            a = vals[n.inputs[0]]
            b = vals[n.inputs[1]].reshape(a.shape)  # operands only need equal element counts
            v = _binary(n.sub_op, a, b, _is_float(n.dtype))
            if n.dtype == U32:
                v = v.astype(np.uint32)
        elif k == OP_CAST:
            a = vals[n.inputs[0]]
            src = graph.nodes[n.inputs[0]].dtype
            if _is_float(src) and _is_float(n.dtype):
                v = a  # same class: only loads / stores change (jit.rs:488-504)
            elif _is_float(src) and n.dtype == BOOL: v = a != 0.0
            elif src == BOOL and _is_float(n.dtype): v = a.astype(np.float64)
            elif _is_float(src) and n.dtype == U32:
                v = np.clip(np.trunc(np.nan_to_num(a.astype(np.float32).astype(np.float64))), 0, 4294967295).astype(np.uint32)
            elif src == U32 and _is_float(n.dtype): v = a.astype(np.float32).astype(np.float64)
            elif src == BOOL and n.dtype == U32: v = a.astype(np.uint32)
            elif src == U32 and n.dtype == BOOL: v = a != 0
            else: v = a
        elif k == OP_REDUCE:
            a = vals[n.inputs[0]]
            axes = tuple(d for d in range(a.ndim) if (n.axes >> d) & 1)
            group = int(np.prod([a.shape[d] for d in axes], dtype=np.int64))
            if n.sub_op == RED_SUM: r = a.sum(axis=axes)
            elif n.sub_op == RED_MEAN: r = (a * (1.0 / group)).sum(axis=axes)  # pre-scaled, jit.rs:413-418
            elif n.sub_op == RED_MAX: r = a.max(axis=axes) if group else np.full((), -np.inf)
            else: r = a.min(axis=axes) if group else np.full((), np.inf)
            v = np.asarray(r, dtype=np.float64).reshape(shape)
        elif k == OP_BROADCAST:
            a = vals[n.inputs[0]]
            pad = len(shape) - a.ndim
            v = np.broadcast_to(a.reshape((1,) * pad + a.shape), shape)
        elif k == OP_RESHAPE:
            v = np.ascontiguousarray(vals[n.inputs[0]]).reshape(shape)
        elif k == OP_SWAP_DIMS:
            v = np.swapaxes(vals[n.inputs[0]], n.axis_a, n.axis_b)
        elif k == OP_COMPARE:
            a = vals[n.inputs[0]]
            v = _CMP[n.sub_op](a, vals[n.inputs[1]].reshape(a.shape))
        elif k == OP_SELECT:
            a = vals[n.inputs[0]]
            v = np.where(vals[n.inputs[2]].reshape(a.shape), vals[n.inputs[1]].reshape(a.shape), a)
        elif k == OP_MATMUL:
            a, b = vals[n.inputs[0]], vals[n.inputs[1]]
            # Precision is a minimum (precision.rs:3-9): bf16 / f16 requests multiply operands rounded to
            # that type; the 8-bit requests multiply at the operand dtype unless `f8_quantise` asks for
            # the reference's narrowest legal reading (operands rounded to their F8Mode)
            kind = n.sub_op & 0xff
            if kind == PREC_BF16_F32:
                a, b = round_to(a, BF16), round_to(b, BF16)
            elif kind in (PREC_F16_F32, PREC_F16_F16):
                a, b = round_to(a, F16), round_to(b, F16)
            elif kind in (PREC_F8_F32, PREC_F8_F16) and f8_quantise:
                a, b = round_to_f8(a, (n.sub_op >> 8) & 1), round_to_f8(b, (n.sub_op >> 12) & 1)
            v = np.matmul(a, b)
        else:
            raise ValueError(f"unknown op kind {k}")
        if i in round_nodes:
            v = round_to(np.asarray(v, dtype=np.float64), n.dtype) if _is_float(n.dtype) else v
        vals[i] = v
    outs = [encode(np.ascontiguousarray(vals[o]), graph.nodes[o].dtype) for o in graph.outputs]
    if return_all:
        return outs, vals
    return outs


# ---- permutation ------------------------------------------------------------------------------------
def output_strides_reference(swaps: Sequence[Sequence[int]], in_shape: Sequence[int]) -> List[int]:
    """compute_output_strides exactly as written in helium/src/cuda/instr/permute_dims.rs:158-172.

    For a chain of swaps whose composition is not an involution this yields the layout of the
    INVERSE permutation; the reference's unit test (permute_dims.rs:183-187) pins that behaviour.
    """
    rank = len(in_shape)
    perm = list(range(rank))
    for a, b in swaps:
        perm[a], perm[b] = perm[b], perm[a]
    strides = [1] * rank
    stride = 1
    for i in reversed(range(rank)):
        j = perm.index(i)
        strides[j] = stride
        stride *= in_shape[j]
    return strides


def output_strides_semantic(swaps: Sequence[Sequence[int]], in_shape: Sequence[int]) -> List[int]:
    """Strides (per input axis) of the tensor the IR describes after applying the swaps in order
    (helium-ir/src/opgraph/op.rs:102-110): what `x.swap_dims(..).swap_dims(..)` means."""
    rank = len(in_shape)
    perm = list(range(rank))  # perm[k] = input axis at output position k
    for a, b in swaps:
        perm[a], perm[b] = perm[b], perm[a]
    strides = [0] * rank
    stride = 1
    for k in reversed(range(rank)):
        strides[perm[k]] = stride
        stride *= in_shape[perm[k]]
    return strides


def permute(x: np.ndarray, out_strides: Sequence[int]) -> np.ndarray:
    """out[sum_i out_strides[i] * c_i] = x[c] (permute_dims/jit.rs:75-79); returns the flat output."""
    x = np.asarray(x)
    order = sorted(range(x.ndim), key=lambda i: -out_strides[i])
    # sanity: the strides must describe a dense layout
    expect = 1
    for i in reversed(order):
        if x.shape[i] != 1 and out_strides[i] != expect:
            raise ValueError("out_strides do not form a dense permutation")
        expect *= x.shape[i]
    return np.ascontiguousarray(np.transpose(x, order)).reshape(-1)


# ---- convolution -------------------------------------------------------------------------------------
PAD_SAME, PAD_VALID, PAD_FULL = 0, 1, 2


def conv_geometry(in_hw, kernel, stride, padding_mode=PAD_SAME):
    """(output size, padding) of Conv2dParams (helium-ir/src/opgraph/op/conv.rs:51-74, 86-94): the input size is
    adjusted by the padding mode (Full: + k/2, Valid: - k/2, Same: unchanged) and divided by the stride
    (integer division); the zero padding on both sides is k/2 (Same), 0 (Valid) or k-1 (Full)."""
    size = list(in_hw)
    for i in range(2):
        if padding_mode == PAD_FULL:
            size[i] += kernel[i] // 2
        elif padding_mode == PAD_VALID:
            size[i] = max(0, size[i] - kernel[i] // 2)
        size[i] //= stride[i]
    pad = {PAD_SAME: [kernel[0] // 2, kernel[1] // 2], PAD_VALID: [0, 0], PAD_FULL: [kernel[0] - 1, kernel[1] - 1]}[padding_mode]
    return size, pad


def _padded(x, pad, P, Q, R, S, stride):
    """x [N,H,W,C] zero-padded so that every tap of every output pixel is addressable."""
    n, h, w, c = x.shape
    hh = max(h + 2 * pad[0], (P - 1) * stride[0] + R)
    ww = max(w + 2 * pad[1], (Q - 1) * stride[1] + S)
    xp = np.zeros((n, hh, ww, c), dtype=np.float64)
    xp[:, pad[0]:pad[0] + h, pad[1]:pad[1] + w, :] = x
    return xp


def conv2d(x, w, stride=(1, 1), padding_mode=PAD_SAME):
    """Op::Conv (helium/src/raw_tensor.rs:232-287; cuDNN cross-correlation, cudnn_graph.rs:196-207):
    y[n,p,q,k] = sum_{r,s,c} x[n, p*sh + r - pad_h, q*sw + s - pad_w, c] * w[k,r,s,c], zeros outside the image.
    x NHWC, w KRSC, float64."""
    x = np.asarray(x, dtype=np.float64); w = np.asarray(w, dtype=np.float64)
    K, R, S, C = w.shape
    (P, Q), pad = conv_geometry(x.shape[1:3], (R, S), stride, padding_mode)
    xp = _padded(x, pad, P, Q, R, S, stride)
    y = np.zeros((x.shape[0], P, Q, K))
    for r in range(R):
        for s in range(S):
            patch = xp[:, r:r + (P - 1) * stride[0] + 1:stride[0], s:s + (Q - 1) * stride[1] + 1:stride[1], :]
            y += patch @ w[:, r, s, :].T
    return y


def conv2d_backward_data(dy, w, in_hw, stride=(1, 1), padding_mode=PAD_SAME):
    """Op::ConvBackwardData: the gradient of conv2d with respect to the image, shape [N, in_h, in_w, C]."""
    dy = np.asarray(dy, dtype=np.float64); w = np.asarray(w, dtype=np.float64)
    K, R, S, C = w.shape
    (P, Q), pad = conv_geometry(in_hw, (R, S), stride, padding_mode)
    n = dy.shape[0]
    hh = max(in_hw[0] + 2 * pad[0], (P - 1) * stride[0] + R)
    ww = max(in_hw[1] + 2 * pad[1], (Q - 1) * stride[1] + S)
    dxp = np.zeros((n, hh, ww, C))
    for r in range(R):
        for s in range(S):
            dxp[:, r:r + (P - 1) * stride[0] + 1:stride[0], s:s + (Q - 1) * stride[1] + 1:stride[1], :] += dy @ w[:, r, s, :]
    return dxp[:, pad[0]:pad[0] + in_hw[0], pad[1]:pad[1] + in_hw[1], :]


def conv2d_backward_filter(dy, x, kernel, stride=(1, 1), padding_mode=PAD_SAME):
    """Op::ConvBackwardFilter: the gradient of conv2d with respect to the filter, shape [K, R, S, C]."""
    dy = np.asarray(dy, dtype=np.float64); x = np.asarray(x, dtype=np.float64)
    R, S = kernel
    (P, Q), pad = conv_geometry(x.shape[1:3], (R, S), stride, padding_mode)
    xp = _padded(x, pad, P, Q, R, S, stride)
    K, C = dy.shape[3], x.shape[3]
    dw = np.zeros((K, R, S, C))
    flow = dy.reshape(-1, K)
    for r in range(R):
        for s in range(S):
            patch = xp[:, r:r + (P - 1) * stride[0] + 1:stride[0], s:s + (Q - 1) * stride[1] + 1:stride[1], :]
            dw[:, r, s, :] = flow.T @ patch.reshape(-1, C)
    return dw


# ---- config-level helpers ---------------------------------------------------------------------------
def affine_relu_nchw_to_nhwc(x_bits: np.ndarray, scale: np.ndarray, bias: np.ndarray) -> np.ndarray:
    """Fused affine + relu + NCHW -> NHWC benchmark case: y = relu(x * s_c + b_c) on bf16 [N,C,H,W], written as [N,H,W,C] bf16 bits.

    One fused multiply-add in f32 (f64 product and sum are exact enough to round identically except
    for double-rounding ties), then max with 0, then one rounding to bf16.
    """
    x = bf16_bits_to_f32(x_bits).astype(np.float64)
    s = np.asarray(scale, dtype=np.float32).astype(np.float64).reshape(1, -1, 1, 1)
    b = np.asarray(bias, dtype=np.float32).astype(np.float64).reshape(1, -1, 1, 1)
    y = np.maximum((x * s + b).astype(np.float32), np.float32(0))
    return f32_to_bf16_bits(np.ascontiguousarray(np.transpose(y, (0, 2, 3, 1))))


def rel_l2(a: np.ndarray, b: np.ndarray) -> float:
    a = np.asarray(a, dtype=np.float64).reshape(-1)
    b = np.asarray(b, dtype=np.float64).reshape(-1)
    den = float(np.linalg.norm(b))
    return float(np.linalg.norm(a - b)) / (den if den > 0 else 1.0)
