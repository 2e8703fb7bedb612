"""Plan-time specialised pointwise kernels, the part that needs no GPU: every program family of jit_cases.py is
printed and accepted by NVRTC for sm_100a at plan time (reductions over a prologue included); the switch, bit-packed
bool tensors and a missing NVRTC library leave the program on the interpreter without an error."""
import os
import subprocess
import sys

import pytest

import helium_b200 as hb
from helium_b200 import ir
from jit_cases import cases

SPECIALISED = "specialised at plan time with NVRTC"


@pytest.mark.parametrize("name,graph,_pos", cases(), ids=[c[0] for c in cases()])
def test_program_families_compile(name, graph, _pos):
    d = hb.Plan.pointwise(None, graph).description
    assert SPECIALISED in d, d
    assert hb.plan_supported(graph, 0) == 1


def test_switch_and_out_of_range_programs_stay_on_the_interpreter(monkeypatch):
    g = ir.Graph()
    x = g.new_input([16, 40], ir.F32)
    g.new_output(g.unary(ir.UN_TANH, g.unary(ir.UN_EXP, x)))
    monkeypatch.setenv("HE_PW_JIT", "0")
    assert "interpreter, " in hb.Plan.pointwise(None, g).description
    monkeypatch.delenv("HE_PW_JIT")
    assert SPECIALISED in hb.Plan.pointwise(None, g).description
    # a bool tensor in memory (bit-packed, one word per warp): interpreter
    gb = ir.Graph()
    a = gb.new_input([16, 40], ir.F32); b = gb.new_input([16, 40], ir.F32)
    gb.new_output(gb.compare(ir.CMP_LT, a, b))
    assert "interpreter, " in hb.Plan.pointwise(None, gb).description
    # a reduction over a prologue is specialised too (its own kernel); with the switch off it is interpreted
    gr = ir.Graph()
    a = gr.new_input([16, 40], ir.F32)
    gr.new_output(gr.reduce(ir.RED_SUM, gr.unary(ir.UN_EXP, a), 1))
    d = hb.Plan.pointwise(None, gr).description
    assert SPECIALISED in d and "reduce: 16 groups of 40" in d
    monkeypatch.setenv("HE_PW_JIT", "0")
    assert "interpreter" in hb.Plan.pointwise(None, gr).description
    monkeypatch.delenv("HE_PW_JIT")
    # the plain column sum keeps its hand-written kernel
    gs = ir.Graph()
    y = gs.new_input([4096, 512], ir.BF16)
    gs.new_output(gs.reduce(ir.RED_SUM, gs.swap_dims(y, 0, 1), 1))
    assert "dense column-sum kernel" in hb.Plan.pointwise(None, gs).description
    # catalogue programs keep their hand-written kernels
    gc = ir.Graph()
    a = gc.new_input([16, 40], ir.BF16)
    gc.new_output(gc.unary(ir.UN_RELU, a))
    assert "tier 2" in hb.Plan.pointwise(None, gc).description


def test_missing_nvrtc_falls_back_to_the_interpreter():
    code = (
        "import helium_b200 as hb\n"
        "from helium_b200 import ir\n"
        "g = ir.Graph(); x = g.new_input([16, 40], ir.F32); g.new_output(g.unary(ir.UN_TANH, g.unary(ir.UN_EXP, x)))\n"
        "print(hb.Plan.pointwise(None, g).description)\n")
    env = dict(os.environ, HE_NVRTC_LIBRARY="/nonexistent/libnvrtc.so")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd=os.path.dirname(os.path.dirname(__file__)))
    assert r.returncode == 0, r.stderr
    assert "interpreter, " in r.stdout and SPECIALISED not in r.stdout
