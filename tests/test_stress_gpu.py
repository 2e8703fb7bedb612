"""Determinism under concurrency, after helium/tests/stress_test.rs: four host threads, each with its
own stream and buffers, run the same two-matmul / sigmoid / cos / reduce chain over and over; every
result must equal the first one bit for bit, in every thread."""
import threading

import numpy as np
import pytest

import helium_b200 as hb
from helium_b200 import ir
from helpers import O, rng

pytestmark = pytest.mark.gpu


def _chain(d):
    g = ir.Graph()
    a1 = g.new_input([d, d], ir.F32)
    a2 = g.new_input([d, d], ir.F32)
    x = g.new_input([d], ir.F32)
    y = g.unary(ir.UN_SIGMOID, g.matmul(a1, g.reshape(x, [d, 1]), ir.PREC_TF32_F32))            # [d, 1]
    y = g.broadcast_to(g.reduce(ir.RED_SUM, y, 1), [d, d])
    z = g.unary(ir.UN_ADD_CONST, g.unary(ir.UN_COS, g.matmul(a2, y, ir.PREC_TF32_F32)), 1.0)
    g.new_output(g.reshape(g.reduce(ir.RED_MEAN, z, 1), [d]))
    return g


def test_four_threads_bit_identical(ctx):
    import torch
    d, iters, n_threads = 256, 60, 4
    g = _chain(d)
    r = rng(783542)
    host = [r.standard_normal((d, d), dtype=np.float32) / np.float32(16), r.standard_normal((d, d), dtype=np.float32) / np.float32(16),
            r.standard_normal(d, dtype=np.float32)]
    want = O.evaluate(g, host)[0]
    results, errors = [None] * n_threads, []

    def worker(t):
        try:
            torch.cuda.set_device(0)
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                ins = [torch.from_numpy(a).cuda() for a in host]
                out = torch.zeros(d, dtype=torch.float32, device="cuda")
                stream.synchronize()
                ex = hb.Executor(ctx, hb.HostGraph(g), ins, [out], capture=(t % 2 == 1))   # eager and graph replay side by side
                first = None
                for _ in range(iters):
                    ex.run(stream)
                    stream.synchronize()
                    got = out.cpu().numpy().copy()
                    if first is None:
                        first = got
                    elif not np.array_equal(first, got):
                        raise AssertionError(f"thread {t}: result changed between iterations")
                results[t] = first
        except Exception as e:  # surfaced in the main thread
            errors.append(e)

    threads = [threading.Thread(target=worker, args=(t,)) for t in range(n_threads)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not errors, errors
    ctx.poll()
    for t in range(1, n_threads):
        assert np.array_equal(results[0], results[t]), f"thread {t} differs from thread 0"
    assert O.rel_l2(results[0], want) <= 1e-5
