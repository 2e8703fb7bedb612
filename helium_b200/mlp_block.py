"""Transformer MLP block, forward + backward, as six fused matmul plans (the token-sharded benchmark workload:
d -> ff with bias + GELU, ff -> d with bias + residual, and their backward GEMMs).

    forward :  Z = X W1 + b1,  H = gelu(Z)            one GEMM, bias + GELU epilogue, Z kept for backward
               O = H W2 + b2 + X                      one GEMM, bias + residual epilogue
    backward:  dZ = (dO W2^T) * gelu'(Z), db1 = colsum(dZ)    one GEMM (B read K-major), gate + Columns sum
               dW1 = X^T dZ                           one GEMM (A read M-major)
               dW2 = H^T dO                           one GEMM (A read M-major)
               dX = dZ W1^T + dO,     db2 = colsum(dO)        one GEMM (B K-major), residual + Columns sum

The graphs are what helium's front end records for `Linear::forward` and its backward
(helium/src/modules/linear.rs:44-57; matmul gradient dA = flow B^T, dB = A^T flow with explicit
transposes, helium/src/tensor.rs:437-450; bias gradient = sum over the broadcast axis,
tensor.rs:83-142), each fused into the GEMM that produces or consumes it instead of running as
separate cast / bias / activation / transpose / reduction kernels.  GELU is the exact erf form (the
only definition the reference gives: helium-playground/src/torch_synthesizer.rs:48).

Weight gradients land in one flat bf16 buffer so the data-parallel exchange is two large
all-reduces (dW1 then dW2), each started while the next GEMM runs; bias gradients are f32 and go in
one small bucket at the end.
"""
from __future__ import annotations

from typing import Optional

import numpy as np

from . import ir
from .configs import bf16_normal, graph_linear, rng
from .grad_sync import GradReducer
from .runtime import Context, Plan


def mlp_block_graphs(tokens: int, d: int, ff: int):
    """The six subgraphs, keyed by the tensor they produce."""
    return {
        "H": graph_linear(tokens, ff, d, bias=True, act=ir.UN_GELU, store_z=True),          # X, W1, b1 -> H, Z
        "O": graph_linear(tokens, d, ff, bias=True, resid=True),                             # H, W2, b2, X -> O
        "dZ": graph_linear(tokens, ff, d, bias=False, b_t=True, gate="dgelu", colsum="y"),   # dO, W2, Z -> dZ, db1
        "dW1": graph_linear(d, ff, tokens, bias=False, a_t=True),                            # X, dZ -> dW1
        "dW2": graph_linear(ff, d, tokens, bias=False, a_t=True),                            # H, dO -> dW2
        "dX": graph_linear(tokens, d, ff, bias=False, b_t=True, resid=True, colsum="resid"),  # dZ, W1, dO -> dX, db2
    }


def mlp_block_inputs(tokens: int, d: int, ff: int, seed: int = 3, shard: int = 0):
    """Seeded host operands (bf16 bit patterns): W1, W2, b1, b2 ~ N(0,0.02) from `seed` (identical on
    every rank), X and dO ~ N(0,1) from a stream derived from (seed, shard) so that each rank's token
    shard is different data."""
    rw = rng(seed)
    rd = rng(seed + 104729 * (shard + 1))
    return {
        "W1": bf16_normal(rw, (d, ff), 0.02), "W2": bf16_normal(rw, (ff, d), 0.02),
        "b1": bf16_normal(rw, (ff,), 0.02), "b2": bf16_normal(rw, (d,), 0.02),
        "X": bf16_normal(rd, (tokens, d)), "dO": bf16_normal(rd, (tokens, d)),
    }


def flops_per_token(d: int, ff: int) -> int:
    """Six GEMMs of 2*d*ff flop per token (pointwise work is not counted)."""
    return 6 * 2 * d * ff


class MlpBlock:
    """Plans + device buffers for one rank's shard of tokens."""

    def __init__(self, ctx: Context, tokens: int, d: int, ff: int, device=None, overlap_sms: int = 0):
        """`overlap_sms` > 0: the two GEMMs that run while a weight-gradient all-reduce is in flight (dW2
        and dX) are planned for that many fewer SMs, so their persistent grids and the collective's CTAs
        do not queue behind each other."""
        import torch

        self.tokens, self.d, self.ff = tokens, d, ff
        self.graphs = mlp_block_graphs(tokens, d, ff)
        self.plans = {}
        for k, g in self.graphs.items():
            if overlap_sms and k in ("dW2", "dX"):
                ctx.reserve_sms(overlap_sms)
            try:
                self.plans[k] = Plan.fused_matmul(ctx, g)
            finally:
                if overlap_sms:
                    ctx.reserve_sms(0)
        dev = device if device is not None else torch.device("cuda", ctx.device)
        bf = torch.bfloat16
        e = lambda *s: torch.empty(s, dtype=bf, device=dev)
        self.X, self.dO = e(tokens, d), e(tokens, d)
        self.W1, self.W2, self.b1, self.b2 = e(d, ff), e(ff, d), e(ff), e(d)
        self.H, self.Z, self.O = e(tokens, ff), e(tokens, ff), e(tokens, d)
        self.dZ, self.dX = e(tokens, ff), e(tokens, d)
        # weight gradients: one flat buffer, dW1 first (it is produced first)
        self.dW_flat = torch.empty(2 * d * ff, dtype=bf, device=dev)
        self.dW1 = self.dW_flat[: d * ff].view(d, ff)
        self.dW2 = self.dW_flat[d * ff:].view(ff, d)
        # bias gradients: f32 (reductions produce f32, helium-ir/src/opgraph/op.rs:78-89)
        self.db_flat = torch.empty(ff + d, dtype=torch.float32, device=dev)
        self.db1 = self.db_flat[:ff].view(1, ff)
        self.db2 = self.db_flat[ff:].view(1, d)
        self.launches_per_step = 0

    def load(self, host: dict) -> None:
        import torch

        for k, v in host.items():
            getattr(self, k).view(torch.int16).copy_(torch.from_numpy(np.ascontiguousarray(v).view(np.int16)).reshape(getattr(self, k).shape))

    def forward(self) -> None:
        p = self.plans
        p["H"].launch([self.X, self.W1, self.b1], [self.H, self.Z])
        p["O"].launch([self.H, self.W2, self.b2, self.X], [self.O])

    def backward(self, reducer: Optional[GradReducer] = None) -> None:
        p = self.plans
        p["dZ"].launch([self.dO, self.W2, self.Z], [self.dZ, self.db1])
        p["dW1"].launch([self.X, self.dZ], [self.dW1])
        if reducer is not None:
            reducer.reduce_bucket([self.dW1])        # overlaps the dW2 GEMM
        p["dW2"].launch([self.H, self.dO], [self.dW2])
        if reducer is not None:
            reducer.reduce_bucket([self.dW2])        # overlaps the dX GEMM
        p["dX"].launch([self.dZ, self.W1, self.dO], [self.dX, self.db2])
        if reducer is not None:
            reducer.reduce_bucket([self.db_flat])
            reducer.finish()

    def step(self, reducer: Optional[GradReducer] = None) -> None:
        self.forward()
        self.backward(reducer)

    def launch_count(self) -> int:
        return sum(pl.last_launch_count for pl in self.plans.values())


__all__ = ["MlpBlock", "mlp_block_graphs", "mlp_block_inputs", "flops_per_token"]
