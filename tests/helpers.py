"""Shared test tooling: seeded inputs, graphs of the benchmark configs, and a numpy emulator of the
pointwise interpreter program (validates the host-side compiler without a GPU)."""
from __future__ import annotations

import ctypes as C
import math
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from helium_b200 import ir  # noqa: E402
from helium_b200._lib import check, lib  # noqa: E402
from oracle import oracle as O  # noqa: E402


def storage_to_torch(arr: np.ndarray, dtype: int, device="cuda"):
    import torch

    if dtype == ir.BF16:
        return torch.from_numpy(np.ascontiguousarray(arr).view(np.int16)).view(torch.bfloat16).to(device)
    if dtype == ir.F16:
        return torch.from_numpy(np.ascontiguousarray(arr).view(np.float16)).to(device)
    if dtype == ir.F32:
        return torch.from_numpy(np.ascontiguousarray(arr, dtype=np.float32)).to(device)
    return torch.from_numpy(np.ascontiguousarray(arr).view(np.int32)).to(device)


def torch_to_storage(t, dtype: int) -> np.ndarray:
    import torch

    t = t.detach().cpu().contiguous()
    if dtype == ir.BF16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if dtype == ir.F16:
        return t.numpy()
    if dtype == ir.F32:
        return t.numpy()
    return t.numpy().view(np.uint32)


def values(storage: np.ndarray, dtype: int, shape) -> np.ndarray:
    return O.decode(storage, dtype, shape)


# ---- benchmark-config graphs (defined in the package; re-exported for the tests) ---------------------
from helium_b200.configs import (bf16_bernoulli, bf16_normal, c2_inputs, c3_inputs, graph_affine_relu_permute,  # noqa: E402,F401
                                 graph_c3, graph_linear, rng)


# ---- pointwise program emulator -----------------------------------------------------------------------
class _FastDiv(C.Structure):
    _fields_ = [("d", C.c_uint32), ("m", C.c_uint32), ("s", C.c_uint32)]


class _PwInstr(C.Structure):
    _fields_ = [(n, C.c_uint8) for n in ("op", "sub", "dst", "a", "b", "c", "dt", "slot")] + [
        ("imm", C.c_uint32), ("view0", C.c_uint8), ("nviews", C.c_uint8), ("slot2", C.c_uint8), ("pad", C.c_uint8)]


class _PwView(C.Structure):
    _fields_ = [("nd", C.c_int32), ("fd", _FastDiv * 8), ("stride", C.c_uint32 * 8)]


class _PwProgram(C.Structure):
    _fields_ = [("n_instr", C.c_int32), ("n_inputs", C.c_int32), ("n_outputs", C.c_int32), ("n_elems", C.c_uint32),
                ("group_size", C.c_uint32), ("n_reductions", C.c_int32), ("mean_scale", C.c_double),
                ("inp", C.c_void_p * 16), ("out", C.c_void_p * 8), ("instr", _PwInstr * 160), ("views", _PwView * 24)]


(PW_LOAD, PW_CONST, PW_UNARY, PW_BIN_F, PW_BIN_U, PW_BIN_B, PW_FMA, PW_CMP_F, PW_CMP_U, PW_SELECT, PW_CVT,
 PW_MEAN_SCALE, PW_STORE, PW_REDUCE, PW_ACC) = range(15)


def dump_program(graph: ir.Graph, epilogue: bool = False) -> _PwProgram:
    desc, keep = graph.to_desc()
    size = C.c_size_t()
    check(lib.he_debug_dump_program(C.byref(desc), int(epilogue), None, 0, C.byref(size)))
    assert size.value == C.sizeof(_PwProgram), (size.value, C.sizeof(_PwProgram))
    prog = _PwProgram()
    check(lib.he_debug_dump_program(C.byref(desc), int(epilogue), C.byref(prog), C.sizeof(prog), C.byref(size)))
    del keep
    return prog


def canonical_text(graph: ir.Graph) -> str:
    desc, keep = graph.to_desc()
    buf = C.create_string_buffer(1 << 20)
    check(lib.he_debug_canonical_text(C.byref(desc), buf, len(buf)))
    del keep
    return buf.value.decode()


def _fastdiv(n: np.ndarray, fd: _FastDiv):
    """q, r exactly as FastDiv::divmod computes them on the device (umulhi + shift)."""
    n = n.astype(np.uint64)
    if fd.m == 0:
        q = n
    else:
        q = ((n * np.uint64(fd.m)) >> np.uint64(32)) >> np.uint64(fd.s)
    r = n - q * np.uint64(fd.d)
    return q.astype(np.uint32), r.astype(np.uint32)


def _apply_views(prog: _PwProgram, v0: int, nv: int, idx: np.ndarray) -> np.ndarray:
    for v in range(v0, v0 + nv):
        vw = prog.views[v]
        rem = idx
        off = np.zeros_like(idx, dtype=np.uint64)
        for k in range(vw.nd):
            rem, c = _fastdiv(rem, vw.fd[k])
            off += c.astype(np.uint64) * np.uint64(vw.stride[k])
        idx = off.astype(np.uint32)
    return idx


def emulate_program(graph: ir.Graph, inputs, epilogue_acc: np.ndarray | None = None):
    """Runs the dumped program over the whole iteration space with f32 arithmetic; returns storage
    arrays of the outputs (reductions: float32 per group for trailing-dim reductions)."""
    prog = dump_program(graph, epilogue=epilogue_acc is not None)
    n = prog.n_elems
    idx = np.arange(n, dtype=np.uint32)
    regs = {}
    outs = {}
    f32 = np.float32
    in_nodes = [graph.nodes[i] for i in graph.inputs]
    for pc in range(prog.n_instr):
        i = prog.instr[pc]
        op = i.op
        if op == PW_LOAD:
            node = in_nodes[i.slot]
            src = O.decode(inputs[i.slot], node.dtype, (node.num_elements,))
            at = _apply_views(prog, i.view0, i.nviews, idx) if i.nviews else idx
            v = src[at]
            regs[i.dst] = v.astype(f32) if node.dtype in (ir.F16, ir.BF16, ir.F32) else v
        elif op == PW_CONST:
            regs[i.dst] = np.full(n, i.imm, dtype=np.uint32)  # reinterpreted by the consumer
            regs[i.dst] = _ConstBits(regs[i.dst])
        elif op == PW_ACC:
            regs[i.dst] = np.asarray(epilogue_acc, dtype=f32).reshape(-1)
        elif op == PW_UNARY:
            a = _as_f32(regs[i.a]).astype(np.float64)
            c = float(np.array([i.imm], dtype=np.uint32).view(np.float32)[0])
            regs[i.dst] = O._unary(i.sub, a, c).astype(f32)
        elif op == PW_BIN_F:
            a, b = _as_f32(regs[i.a]), _as_f32(regs[i.b])
            if i.sub in (ir.BIN_POW,):
                regs[i.dst] = O._binary(i.sub, a.astype(np.float64), b.astype(np.float64), True).astype(f32)
            else:
                regs[i.dst] = np.asarray(O._binary(i.sub, a, b, True), dtype=f32)
        elif op == PW_FMA:
            a, b, c = (_as_f32(regs[r]).astype(np.float64) for r in (i.a, i.b, i.c))
            regs[i.dst] = (a * b + c).astype(f32)
        elif op == PW_BIN_U:
            regs[i.dst] = O._binary(i.sub, _as_u32(regs[i.a]), _as_u32(regs[i.b]), False).astype(np.uint32)
        elif op == PW_BIN_B:
            regs[i.dst] = O._binary(i.sub, _as_bool(regs[i.a]), _as_bool(regs[i.b]), False)
        elif op == PW_CMP_F:
            regs[i.dst] = O._CMP[i.sub](_as_f32(regs[i.a]), _as_f32(regs[i.b]))
        elif op == PW_CMP_U:
            regs[i.dst] = O._CMP[i.sub](_as_u32(regs[i.a]), _as_u32(regs[i.b]))
        elif op == PW_SELECT:
            sel = _as_bool(regs[i.c])
            a, b = regs[i.a], regs[i.b]
            if isinstance(a, _ConstBits) and isinstance(b, _ConstBits):
                regs[i.dst] = _ConstBits(np.where(sel, b.bits, a.bits))
                continue
            if isinstance(a, _ConstBits) or isinstance(b, _ConstBits):
                like = b if isinstance(a, _ConstBits) else a
                a = _coerce(a, like)
                b = _coerce(b, like)
            regs[i.dst] = np.where(sel, b, a)
        elif op == PW_CVT:
            frm, to = i.sub >> 2, i.sub & 3
            a = regs[i.a]
            if (frm, to) == (0, 2): regs[i.dst] = _as_f32(a) != 0
            elif (frm, to) == (2, 0): regs[i.dst] = _as_bool(a).astype(f32)
            elif (frm, to) == (0, 1): regs[i.dst] = np.clip(np.trunc(np.nan_to_num(_as_f32(a).astype(np.float64))), 0, 4294967295).astype(np.uint32)
            elif (frm, to) == (1, 0): regs[i.dst] = _as_u32(a).astype(f32)
            elif (frm, to) == (2, 1): regs[i.dst] = _as_bool(a).astype(np.uint32)
            else: regs[i.dst] = _as_u32(a) != 0
        elif op == PW_MEAN_SCALE:
            regs[i.dst] = (_as_f32(regs[i.a]).astype(np.float64) * prog.mean_scale).astype(f32)
        elif op == PW_STORE:
            v = regs[i.a]
            if i.dt == ir.BOOL:
                outs[i.slot] = O.pack_bools(_as_bool(v))
            elif i.dt == ir.U32:
                outs[i.slot] = _as_u32(v)
            else:
                outs[i.slot] = O.encode(_as_f32(v).astype(np.float64), i.dt)
        elif op == PW_REDUCE:
            v = _as_f32(regs[i.a]).astype(np.float64).reshape(-1, prog.group_size)
            r = {ir.RED_SUM: v.sum(1), ir.RED_MEAN: v.sum(1), ir.RED_MAX: v.max(1), ir.RED_MIN: v.min(1)}[i.sub]
            outs[i.slot] = r.astype(f32)
        else:
            raise AssertionError(f"unknown instruction {op}")
    return [outs[k] for k in range(prog.n_outputs)], prog


class _ConstBits:
    """A PW_CONST register: 32 raw bits whose class is decided by the consumer."""

    def __init__(self, bits):
        self.bits = bits


def _as_f32(v):
    if isinstance(v, _ConstBits):
        return v.bits.view(np.float32)
    return np.asarray(v, dtype=np.float32)


def _as_u32(v):
    if isinstance(v, _ConstBits):
        return v.bits
    return np.asarray(v).astype(np.uint32)


def _as_bool(v):
    if isinstance(v, _ConstBits):
        return v.bits != 0
    return np.asarray(v).astype(bool)


def _coerce(v, like):
    if not isinstance(v, _ConstBits):
        return v
    if like.dtype == np.float32:
        return _as_f32(v)
    if like.dtype == bool:
        return _as_bool(v)
    return _as_u32(v)
