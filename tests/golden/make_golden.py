#!/usr/bin/env python
"""Writes tests/golden/golden_v1.npz: outputs of the CPU oracle on small seeded cases of every
benchmark configuration.

Provenance: the reference cannot be run in the build image (Rust, run-time generated CUDA), so these
vectors are NOT reference outputs.  They pin the oracle -- whose op semantics are themselves pinned on
the reference's own known-answer tests in tests/test_oracle_golden.py -- and the kernels against
drift: tests/test_oracle_golden.py::test_golden_fixtures re-evaluates the oracle against this file and
tests/test_kat_gpu.py::test_golden_fixtures_on_device runs the same cases through the C ABI.

Inputs are not stored: they are regenerated from the Philox seeds below (helium_b200/configs.py).

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from helium_b200 import configs, ir  # noqa: E402
from helium_b200.mlp_block import mlp_block_graphs, mlp_block_inputs  # noqa: E402
from oracle import oracle as O  # noqa: E402


def cases():
    """name -> (graph, inputs); shared by the generator and by the tests."""
    out = {}
    # configs[1]a at a small size: relu(x * s_c + b_c), NCHW -> NHWC
    g = configs.graph_affine_relu_permute(2, 16, 6, 8)
    r = configs.rng(101)
    out["affine_relu_nhwc"] = (g, [configs.bf16_normal(r, (2, 16, 6, 8)), r.random(16, dtype=np.float32) + np.float32(0.5),
                                   r.standard_normal(16, dtype=np.float32) * np.float32(0.1)])
    # configs[1]b: a three-cycle permutation of an f32 tensor
    g = ir.Graph()
    x = g.new_input([12, 10, 8], ir.F32)
    g.new_output(g.swap_dims(g.swap_dims(x, 1, 2), 0, 1))
    out["permute_201"] = (g, [configs.rng(102).standard_normal((12, 10, 8), dtype=np.float32)])
    # configs[2]: the README fused matmul graph
    out["readme_fused_matmul"] = (configs.graph_c3(128, 256, 64, False), configs.c3_inputs(128, 256, 64, False, seed=103))
    # configs[0]: MLP training step
    out["mlp_train_step"] = (configs.graph_mlp_train_step(16, 40, 24, 10, 0.01), configs.mlp_inputs(16, 40, 24, 10, seed=104))
    # configs[3]: the two forward GEMMs of the transformer MLP block (the backward graphs take the
    # forward results as inputs and are covered by tests/test_matmul_gpu.py)
    graphs = mlp_block_graphs(64, 64, 128)
    host = mlp_block_inputs(64, 64, 128, seed=105)
    out["mlp_block_H"] = (graphs["H"], [host["X"], host["W1"], host["b1"]])
    out["mlp_block_dW"] = (graphs["dW1"], [host["X"], configs.bf16_normal(configs.rng(106), (64, 128))])
    return out


def main():
    arrays = {}
    for name, (g, ins) in cases().items():
        for k, o in enumerate(O.evaluate(g, ins)):
            arrays[f"{name}/{k}"] = np.asarray(o)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden_v1.npz")
    np.savez_compressed(path, **arrays)
    print(path, os.path.getsize(path), "bytes,", len(arrays), "arrays")


if __name__ == "__main__":
    main()
