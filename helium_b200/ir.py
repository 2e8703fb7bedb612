"""Host-side mirror of the helium-ir op graph (helium-ir/src/opgraph.rs, opgraph/op.rs) and of the
playground op vocabulary (helium-playground/src/opgraph.rs), flattened to the `he_node` records
the C ABI takes.

Shape / dtype inference follows `Op::output_descriptor` (helium-ir/src/opgraph/op.rs:52-179).
"""
from __future__ import annotations

import ctypes as C
import struct
from dataclasses import dataclass, field
from typing import List, Sequence, Tuple

from ._abi import HE_MAX_RANK, HeGraphDesc, HeNode

# ---- enums (values = include/helium_b200.h) ------------------------------------------------------
F16, BF16, F32, U32, BOOL = 0, 1, 2, 3, 4
DTYPE_NAMES = {F16: "f16", BF16: "bf16", F32: "f32", U32: "u32", BOOL: "bool"}

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


def prec_f8(kind: int, mode_a: int = F8_E4M3, mode_b: int = F8_E4M3) -> int:
    """MulF8Accum* { mode_a, mode_b } (helium-ir/src/opgraph/op/precision.rs:60-81) packed the way the
    C ABI's `sub_op` carries it."""
    assert kind in (PREC_F8_F32, PREC_F8_F16)
    return kind | (mode_a << 8) | (mode_b << 12)


def _is_float(dt: int) -> bool:
    return dt in (F16, BF16, F32)


def f32_bits(v: float) -> int:
    return struct.unpack("<I", struct.pack("<f", float(v)))[0]


def scalar_bits(v, dtype: int) -> int:
    """Bit pattern of a constant of `dtype` (Scalar in helium-ir/src/data_type.rs)."""
    if dtype == F32:
        return f32_bits(v)
    if dtype == BF16:
        b = f32_bits(v)
        # round to nearest even like half::bf16::from_f32
        return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16) & 0xFFFF
    if dtype == F16:
        return struct.unpack("<H", struct.pack("<e", float(v)))[0]
    if dtype == U32:
        return int(v) & 0xFFFFFFFF
    return 1 if v else 0


@dataclass
class Node:
    kind: int
    dtype: int
    shape: Tuple[int, ...]
    sub_op: int = 0
    inputs: Tuple[int, ...] = ()
    const_bits: int = 0
    axis_a: int = 0
    axis_b: int = 0
    axes: int = 0

    @property
    def num_elements(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n


@dataclass
class Graph:
    """An `OpSubgraph`: nodes in topological order, inputs = OP_INPUT nodes in order, outputs = leafs."""

    nodes: List[Node] = field(default_factory=list)
    outputs: List[int] = field(default_factory=list)

    # -- construction ----------------------------------------------------------------------------
    def _add(self, node: Node) -> int:
        if len(node.shape) > HE_MAX_RANK:
            raise ValueError(f"rank {len(node.shape)} exceeds {HE_MAX_RANK}")
        self.nodes.append(node)
        return len(self.nodes) - 1

    def new_input(self, shape: Sequence[int], dtype: int) -> int:
        return self._add(Node(OP_INPUT, dtype, tuple(int(d) for d in shape)))

    def new_output(self, node: int) -> None:
        self.outputs.append(node)

    def constant(self, value, shape: Sequence[int], dtype: int = F32) -> int:
        return self._add(Node(OP_CONSTANT, dtype, tuple(shape), const_bits=scalar_bits(value, dtype)))

    def unary(self, op: int, x: int, const: float = 0.0) -> int:
        n = self.nodes[x]
        return self._add(Node(OP_UNARY, n.dtype, n.shape, sub_op=op, inputs=(x,), const_bits=f32_bits(const)))

    def binary(self, op: int, lhs: int, rhs: int) -> int:
        n = self.nodes[lhs]  # result takes the lhs descriptor (op.rs:74-77)
        return self._add(Node(OP_BINARY, n.dtype, n.shape, sub_op=op, inputs=(lhs, rhs)))

    def cast(self, x: int, dtype: int) -> int:
        return self._add(Node(OP_CAST, dtype, self.nodes[x].shape, inputs=(x,)))

    def reduce(self, op: int, x: int, depth: int) -> int:
        """helium-ir Reduce: the last `depth` dims collapse into one dim of size 1 (op.rs:78-89)."""
        n = self.nodes[x]
        r = len(n.shape)
        if not 1 <= depth <= r:
            raise ValueError("bad reduce depth")
        axes = ((1 << depth) - 1) << (r - depth)
        shape = tuple(n.shape[: r - depth]) + (1,)
        return self._add(Node(OP_REDUCE, F32, shape, sub_op=op, inputs=(x,), axes=axes))

    def reduce_axes(self, op: int, x: int, axes: Sequence[int]) -> int:
        """Playground Reduction: rank kept, reduced dims become 1 (helium-playground/src/opgraph.rs:397-413)."""
        n = self.nodes[x]
        mask = 0
        shape = list(n.shape)
        for a in axes:
            mask |= 1 << a
            shape[a] = 1
        return self._add(Node(OP_REDUCE, F32, tuple(shape), sub_op=op, inputs=(x,), axes=mask))

    def broadcast(self, x: int, new_dim_count: int, axes: Sequence[Tuple[int, int]]) -> int:
        """helium-ir Broadcast{new_dim_count, broadcast_axes[(axis, new_size)]} (op.rs:369-395)."""
        n = self.nodes[x]
        shape = list(n.shape)
        while len(shape) < new_dim_count:
            shape.insert(0, 1)
        for axis, size in axes:
            shape[axis] = size
        return self._add(Node(OP_BROADCAST, n.dtype, tuple(shape), inputs=(x,)))

    def broadcast_to(self, x: int, shape: Sequence[int]) -> int:
        """Right-aligned broadcast like RawTensor::broadcast_to (helium/src/raw_tensor.rs:371-425)."""
        n = self.nodes[x]
        pad = len(shape) - len(n.shape)
        axes = []
        for k, size in enumerate(shape):
            in_dim = 1 if k < pad else n.shape[k - pad]
            if in_dim != size:
                axes.append((k, size))
        return self.broadcast(x, len(shape), axes)

    def reshape(self, x: int, shape: Sequence[int]) -> int:
        n = self.nodes[x]
        return self._add(Node(OP_RESHAPE, n.dtype, tuple(shape), inputs=(x,)))

    def swap_dims(self, x: int, a: int, b: int) -> int:
        n = self.nodes[x]
        shape = list(n.shape)
        shape[a], shape[b] = shape[b], shape[a]
        return self._add(Node(OP_SWAP_DIMS, n.dtype, tuple(shape), inputs=(x,), axis_a=a, axis_b=b))

    def transpose(self, x: int) -> int:
        r = len(self.nodes[x].shape)
        return self.swap_dims(x, r - 2, r - 1)

    def compare(self, op: int, lhs: int, rhs: int) -> int:
        return self._add(Node(OP_COMPARE, BOOL, self.nodes[lhs].shape, sub_op=op, inputs=(lhs, rhs)))

    def select(self, lhs: int, rhs: int, selector: int) -> int:
        n = self.nodes[lhs]
        return self._add(Node(OP_SELECT, n.dtype, n.shape, inputs=(lhs, rhs, selector)))

    def matmul(self, a: int, b: int, precision: int = PREC_BF16_F32) -> int:
        na, nb = self.nodes[a], self.nodes[b]
        shape = tuple(na.shape[:-1]) + (nb.shape[-1],)
        # the node's dtype is the accumulator type (precision.rs:84-96)
        acc = F16 if (precision & 0xff) in (PREC_F16_F16, PREC_F8_F16) else F32
        return self._add(Node(OP_MATMUL, acc, shape, sub_op=precision, inputs=(a, b)))

    # -- queries ---------------------------------------------------------------------------------
    @property
    def inputs(self) -> List[int]:
        return [i for i, n in enumerate(self.nodes) if n.kind == OP_INPUT]

    def to_desc(self):
        """Returns (he_graph_desc, keepalive) for the C ABI."""
        arr = (HeNode * len(self.nodes))()
        for i, n in enumerate(self.nodes):
            c = arr[i]
            c.kind, c.sub_op, c.dtype, c.rank = n.kind, n.sub_op, n.dtype, len(n.shape)
            for k in range(3):
                c.inp[k] = n.inputs[k] if k < len(n.inputs) else -1
            for k, d in enumerate(n.shape):
                c.shape[k] = d
            c.const_bits, c.axis_a, c.axis_b, c.axes = n.const_bits, n.axis_a, n.axis_b, n.axes
        outs = (C.c_int32 * len(self.outputs))(*self.outputs)
        desc = HeGraphDesc(len(self.nodes), arr, len(self.outputs), outs)
        return desc, (arr, outs)
