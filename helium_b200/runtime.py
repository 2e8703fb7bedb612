"""Thin object layer over the C ABI: Context and Plan.

PyTorch is used only as the device-memory and stream provider (what helium's allocator and
CudaContext do in the reference, helium/src/cuda/context.rs, allocator/*).  Every compute call
goes through `he_launch`; nothing here computes on the host.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import numpy as np

from . import ir
from ._abi import HeConv2dFusion, HeConv2dParams
from ._lib import HeliumError, check, lib

_TORCH_DTYPES = None


def _torch():
    import torch

    global _TORCH_DTYPES
    if _TORCH_DTYPES is None:
        _TORCH_DTYPES = {ir.F16: torch.float16, ir.BF16: torch.bfloat16, ir.F32: torch.float32,
                         ir.U32: torch.int32, ir.BOOL: torch.int32}
    return torch


def storage_elems(dtype: int, n: int) -> int:
    """Elements of the backing torch tensor (bool tensors are bit-packed u32 words)."""
    return (n + 31) // 32 if dtype == ir.BOOL else n


class Context:
    """he_ctx: one per device."""

    def __init__(self, device: int = 0):
        h = C.c_void_p()
        check(lib.he_ctx_create(device, C.byref(h)))
        self._h = h
        self.device = device

    def reserve_sms(self, sms: int) -> None:
        """he_ctx_reserve_sms: plans created afterwards leave `sms` SMs to concurrent work."""
        check(lib.he_ctx_reserve_sms(self._h, sms))

    def poll(self, stream=None) -> None:
        check(lib.he_ctx_poll_device_status(self._h, C.c_void_p(_stream_ptr(stream))))

    def close(self) -> None:
        if self._h:
            lib.he_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _stream_ptr(stream) -> int:
    if stream is None:
        torch = _torch()
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


class Plan:
    """he_plan plus the descriptors needed to allocate outputs."""

    def __init__(self, handle: C.c_void_p, out_shapes: List[tuple], out_dtypes: List[int], n_inputs: int,
                 ctx: Optional[Context]):
        self._h = handle
        self.out_shapes = out_shapes
        self.out_dtypes = out_dtypes
        self.n_inputs = n_inputs
        self.ctx = ctx
        self._workspace = None

    # -- constructors ------------------------------------------------------------------------------
    @staticmethod
    def pointwise(ctx: Optional[Context], graph: ir.Graph) -> "Plan":
        return Plan._from_graph(lib.he_plan_pointwise, ctx, graph)

    @staticmethod
    def fused_matmul(ctx: Optional[Context], graph: ir.Graph) -> "Plan":
        return Plan._from_graph(lib.he_plan_fused_matmul, ctx, graph)

    @staticmethod
    def _from_graph(fn, ctx, graph: ir.Graph) -> "Plan":
        desc, keep = graph.to_desc()
        h = C.c_void_p()
        check(fn(ctx._h if ctx else None, C.byref(desc), C.byref(h)))
        del keep
        shapes = [graph.nodes[o].shape for o in graph.outputs]
        dtypes = [graph.nodes[o].dtype for o in graph.outputs]
        return Plan(h, shapes, dtypes, len(graph.inputs), ctx)

    @staticmethod
    def permute(ctx: Optional[Context], in_shape: Sequence[int], out_strides: Sequence[int], dtype: int,
                out_shape: Optional[Sequence[int]] = None) -> "Plan":
        rank = len(in_shape)
        shp = (C.c_int64 * rank)(*in_shape)
        st = (C.c_int64 * rank)(*out_strides)
        h = C.c_void_p()
        check(lib.he_plan_permute(ctx._h if ctx else None, rank, shp, st, dtype, C.byref(h)))
        if out_shape is None:
            order = sorted(range(rank), key=lambda i: -out_strides[i])
            out_shape = [in_shape[i] for i in order]
        return Plan(h, [tuple(out_shape)], [dtype], 1, ctx)

    @staticmethod
    def conv2d(ctx: Optional[Context], kind: str, batch: int, in_hw, in_channels: int, out_channels: int, kernel, stride: int = 1,
               dilation: int = 1, padding_mode: int = 0, dtype: int = ir.BF16, out_dtype: Optional[int] = None, bias: bool = False,
               bias_dtype: int = ir.F32, resid: bool = False, gate: bool = False, stats: bool = False) -> "Plan":
        """he_plan_conv2d.  kind: "fwd" (inputs image, filter[, bias][, resid]), "bwd_data" (flow, filter[, resid]
        [, gate_x, gate_scale, gate_shift]) or "bwd_filter" (flow, image).  `in_hw` is the image's size."""
        k = {"fwd": 0, "bwd_data": 1, "bwd_filter": 2}[kind]
        prm = HeConv2dParams(in_channels, out_channels, kernel[0], kernel[1], stride, stride, dilation, dilation, padding_mode)
        od = dtype if out_dtype is None else out_dtype
        fus = HeConv2dFusion(od, int(bias), bias_dtype, int(resid), int(gate), int(stats))
        h = C.c_void_p()
        check(lib.he_plan_conv2d(ctx._h if ctx else None, k, C.byref(prm), batch, in_hw[0], in_hw[1], dtype, C.byref(fus), C.byref(h)))
        size = list(in_hw)
        for i in range(2):
            if padding_mode == 2:
                size[i] += kernel[i] // 2
            elif padding_mode == 1:
                size[i] = max(0, size[i] - kernel[i] // 2)
            size[i] //= stride
        if k == 0:
            shapes, n_in = [(batch, size[0], size[1], out_channels)], 2 + int(bias) + int(resid)
        elif k == 1:
            shapes, n_in = [(batch, in_hw[0], in_hw[1], in_channels)], 2 + int(resid) + 3 * int(gate)
        else:
            shapes, n_in = [(out_channels, kernel[0], kernel[1], in_channels)], 2
        dtypes = [od]
        if stats:
            shapes.append((2, shapes[0][3]))
            dtypes.append(ir.F32)
        return Plan(h, shapes, dtypes, n_in, ctx)

    # -- queries -----------------------------------------------------------------------------------
    @property
    def workspace_bytes(self) -> int:
        n = C.c_size_t()
        check(lib.he_plan_workspace_bytes(self._h, C.byref(n)))
        return n.value

    @property
    def description(self) -> str:
        return lib.he_plan_describe(self._h).decode()

    @property
    def last_launch_count(self) -> int:
        return lib.he_plan_last_launch_count(self._h)

    def fault_injection(self, wait_limit_us: int = 0, withhold_loads: bool = False) -> None:
        """he_debug_plan_fault_injection: bound of the kernels' device-side waits (0 = default 2 s) and
        whether the TMA producers stay silent, which makes the first operand wait run out."""
        check(lib.he_debug_plan_fault_injection(self._h, wait_limit_us, 1 if withhold_loads else 0))

    # -- launching ---------------------------------------------------------------------------------
    def alloc_outputs(self, device: str = "cuda"):
        torch = _torch()
        outs = []
        for shape, dt in zip(self.out_shapes, self.out_dtypes):
            n = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
            if dt == ir.BOOL:
                outs.append(torch.empty(storage_elems(dt, n), dtype=torch.int32, device=device))
            else:
                outs.append(torch.empty(tuple(shape), dtype=_TORCH_DTYPES[dt], device=device))
        return outs

    def launch_ptrs(self, in_ptrs: Sequence[int], out_ptrs: Sequence[int], workspace_ptr: int = 0, stream=None) -> None:
        """Direct call of he_launch with raw device addresses."""
        ins = (C.c_void_p * max(1, len(in_ptrs)))(*in_ptrs)
        outs = (C.c_void_p * max(1, len(out_ptrs)))(*out_ptrs)
        check(lib.he_launch(self._h, ins, outs, C.c_void_p(workspace_ptr), C.c_void_p(_stream_ptr(stream))))

    def launch(self, inputs: Sequence, outputs: Optional[Sequence] = None, stream=None):
        """Runs the plan on torch CUDA tensors; allocates outputs (and the workspace once) if needed."""
        torch = _torch()
        if len(inputs) != self.n_inputs:
            raise ValueError(f"plan takes {self.n_inputs} inputs, got {len(inputs)}")
        for t in inputs:
            if not t.is_cuda or not t.is_contiguous():
                raise ValueError("inputs must be contiguous CUDA tensors")
        if outputs is None:
            outputs = self.alloc_outputs(inputs[0].device if inputs else "cuda")
        ws = self.workspace_bytes
        if ws and (self._workspace is None or self._workspace.numel() < ws):
            self._workspace = torch.empty(ws + 256, dtype=torch.uint8, device=outputs[0].device)
        wptr = 0
        if ws:
            wptr = (self._workspace.data_ptr() + 255) // 256 * 256
        self.launch_ptrs([t.data_ptr() for t in inputs], [t.data_ptr() for t in outputs], wptr, stream)
        return outputs

    def close(self) -> None:
        if self._h:
            lib.he_plan_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Comm:
    """he_comm: NCCL communicator behind the C ABI (one per process / GPU).  The 128-byte unique id is made
    on rank 0 and handed out through `exchange`, a callable bytes -> bytes that broadcasts rank 0's value
    (a torch.distributed broadcast in bench.py and the tests; any other channel works)."""

    def __init__(self, ctx: Optional[Context], rank: int, world: int, exchange, max_ctas: int = 0, timeout_ms: int = 60000):
        uid = C.create_string_buffer(128)
        if rank == 0:
            check(lib.he_comm_unique_id(uid))
        uid = C.create_string_buffer(exchange(bytes(uid.raw)), 128)
        h = C.c_void_p()
        check(lib.he_comm_create(ctx._h if ctx else None, rank, world, uid, max_ctas, timeout_ms, C.byref(h)))
        self._h = h
        self.rank, self.world, self.max_ctas = rank, world, max_ctas

    def allreduce(self, tensors: Sequence, mean: bool = True, stream=None) -> None:
        """In-place sum / mean over ranks of same-dtype CUDA tensors, one NCCL group on `stream`."""
        torch = _torch()
        if not tensors:
            return
        dt = {torch.float16: ir.F16, torch.bfloat16: ir.BF16, torch.float32: ir.F32}[tensors[0].dtype]
        n = len(tensors)
        bufs = (C.c_void_p * n)(*[t.data_ptr() for t in tensors])
        counts = (C.c_size_t * n)(*[t.numel() for t in tensors])
        check(lib.he_allreduce_grads(self._h, bufs, counts, n, dt, 1 if mean else 0, C.c_void_p(_stream_ptr(stream))))

    def poll(self) -> None:
        check(lib.he_comm_poll(self._h))

    def abort(self) -> None:
        check(lib.he_comm_abort(self._h))

    def close(self) -> None:
        if self._h:
            lib.he_comm_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def plan_supported(graph: ir.Graph, kind: int, ctx: Optional[Context] = None) -> int:
    """he_plan_supported: 0 unsupported, 1 interpreter tier, 2 hand-written kernel."""
    desc, keep = graph.to_desc()
    r = lib.he_plan_supported(ctx._h if ctx else None, C.byref(desc), kind)
    del keep
    return r


def permute_output_strides(in_shape: Sequence[int], swaps: Sequence[tuple], reference_compat: bool = False) -> List[int]:
    rank = len(in_shape)
    shp = (C.c_int64 * rank)(*in_shape)
    flat = [a for s in swaps for a in s]
    sw = (C.c_int32 * max(1, len(flat)))(*flat)
    out = (C.c_int64 * rank)()
    check(lib.he_permute_output_strides(rank, shp, len(swaps), sw, 1 if reference_compat else 0, out))
    return list(out)


__all__ = ["Context", "Plan", "Comm", "HeliumError", "plan_supported", "permute_output_strides", "storage_elems"]
