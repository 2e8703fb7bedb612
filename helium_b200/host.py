"""Python handle on the C++ host runtime (heh_* entry points): whole-graph planning and execution.

The C++ side restates helium's `plan_generation.rs` and `execute_graph` (see
helium_b200/csrc/host_graph.cu); this module only feeds it an `ir.Graph` and device buffers.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

from . import ir
from ._lib import HeNode, check, lib
from .runtime import Context, _stream_ptr


class HostGraph:
    """heh_graph built from an ir.Graph (node ids are preserved)."""

    def __init__(self, graph: ir.Graph):
        self.ir = graph
        h = C.c_void_p()
        check(lib.heh_graph_create(C.byref(h)))
        self._h = h
        for n in graph.nodes:
            out = C.c_int32()
            if n.kind == ir.OP_INPUT:
                shp = (C.c_int64 * max(1, len(n.shape)))(*n.shape)
                check(lib.heh_graph_new_input(h, n.dtype, len(n.shape), shp, C.byref(out)))
            else:
                c = HeNode()
                c.kind, c.sub_op, c.dtype, c.rank = n.kind, n.sub_op, n.dtype, len(n.shape)
                for k in range(3):
                    c.inp[k] = n.inputs[k] if k < len(n.inputs) else -1
                for k, d in enumerate(n.shape):
                    c.shape[k] = d
                c.const_bits, c.axis_a, c.axis_b, c.axes = n.const_bits, n.axis_a, n.axis_b, n.axes
                check(lib.heh_graph_new_op(h, C.byref(c), C.byref(out)))
        for o in graph.outputs:
            check(lib.heh_graph_new_output(h, o))

    def plan_text(self, ctx: Optional[Context] = None) -> str:
        buf = C.create_string_buffer(1 << 20)
        check(lib.heh_graph_plan_text(ctx._h if ctx else None, self._h, buf, len(buf)))
        return buf.value.decode()

    def set_planner(self, mode: str = "search", depth: int = 0, max_states: int = 0) -> None:
        """"pairwise": the reference's greedy merging (default); "search": the fusion search."""
        check(lib.heh_graph_set_planner(self._h, {"pairwise": 0, "search": 1}[mode], depth, max_states))

    def search_text(self, ctx: Optional[Context] = None) -> str:
        buf = C.create_string_buffer(1 << 20)
        check(lib.heh_graph_search_text(ctx._h if ctx else None, self._h, buf, len(buf)))
        return buf.value.decode()

    def subdivisions(self):
        """[(node, portion)] per subdivision; portion "m" / "e" for the two sides of a matmul, "" otherwise."""
        buf = C.create_string_buffer(1 << 20)
        check(lib.heh_graph_subdivisions_text(self._h, buf, len(buf)))
        out = []
        for line in buf.value.decode().splitlines():
            out.append([(int(t.rstrip("me")), t[len(t.rstrip("me")):]) for t in line.split()])
        return out

    def close(self):
        if self._h:
            lib.heh_graph_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Executor:
    """heh_exec: a planned graph bound to fixed device buffers, optionally captured as a CUDA graph."""

    def __init__(self, ctx: Context, graph: HostGraph, inputs: Sequence, outputs: Sequence, capture: bool = False):
        self.graph = graph
        self._keep = (list(inputs), list(outputs))
        ins = (C.c_void_p * max(1, len(inputs)))(*[t.data_ptr() for t in inputs])
        outs = (C.c_void_p * max(1, len(outputs)))(*[t.data_ptr() for t in outputs])
        h = C.c_void_p()
        check(lib.heh_exec_create(ctx._h, graph._h, ins, outs, 1 if capture else 0, C.byref(h)))
        self._h = h

    def run(self, stream=None) -> None:
        check(lib.heh_exec_run(self._h, C.c_void_p(_stream_ptr(stream))))

    def stats(self):
        a, b, c = C.c_int32(), C.c_int32(), C.c_int32()
        check(lib.heh_exec_stats(self._h, C.byref(a), C.byref(b), C.byref(c)))
        return {"launches": a.value, "steps": b.value, "instrs": c.value}

    def close(self):
        if self._h:
            lib.heh_exec_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
