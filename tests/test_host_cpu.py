"""The C++ host runtime's planning half (instruction selection, fusion, steps, lifetimes) needs no
GPU: he_plan_supported answers without a device."""
import re

import helium_b200 as hb
from helium_b200 import configs, ir


def _instrs(text):
    out = []
    for line in text.splitlines():
        m = re.match(r"step (\d+) (\w+) tier=(\d) nodes=\[([\d,]*)\] in=\[([\d,]*)\] out=\[([\d,]*)\]", line)
        if m:
            f = lambda s: [int(v) for v in s.split(",") if v]
            out.append(dict(step=int(m.group(1)), kind=m.group(2), tier=int(m.group(3)), nodes=f(m.group(4)),
                            inputs=f(m.group(5)), outputs=f(m.group(6))))
    return out


def test_config_2a_becomes_one_single_pass_kernel():
    # the reference plans this as PointwiseGraph + PermuteDims (two passes over HBM)
    g = configs.graph_affine_relu_permute(64, 256, 56, 56)
    ins = _instrs(hb.HostGraph(g).plan_text())
    assert len(ins) == 1 and ins[0]["kind"] == "PointwiseGraph" and ins[0]["tier"] == 2


def test_large_swap_chain_fuses_into_one_permute():
    g = ir.Graph()
    x = g.new_input([4096, 4096, 8], ir.F32)
    g.new_output(g.swap_dims(g.swap_dims(x, 1, 2), 0, 1))
    ins = _instrs(hb.HostGraph(g).plan_text())
    assert len(ins) == 1 and ins[0]["kind"] == "PermuteDims" and len(ins[0]["nodes"]) == 2


def test_small_swaps_stay_pointwise():
    # helium/src/cuda.rs:38: only swaps above 1e6 elements become PermuteDims
    g = ir.Graph()
    x = g.new_input([8, 16, 32], ir.F32)
    g.new_output(g.swap_dims(x, 0, 2))
    ins = _instrs(hb.HostGraph(g).plan_text())
    assert len(ins) == 1 and ins[0]["kind"] == "PointwiseGraph"


def test_mlp_step_plan_structure():
    g = configs.graph_mlp_train_step()
    text = hb.HostGraph(g).plan_text()
    ins = _instrs(text)
    mm = [i for i in ins if i["kind"] == "FusedMatmul"]
    assert len(mm) == 5
    # explicit transposes of the backward matmuls fold into the matmul instructions, and both weight
    # gradients carry their SGD update (const, mul, neg, add) in the epilogue
    assert sum(1 for i in mm if len(i["nodes"]) >= 2) >= 3
    assert sum(1 for i in mm if len(i["nodes"]) >= 5) == 2
    assert len(ins) == 14
    # every node is planned exactly once and in dependency order
    seen = set(g.inputs)
    for i in ins:
        assert set(i["inputs"]) <= seen, text
        seen |= set(i["nodes"])
    planned = [n for i in ins for n in i["nodes"]]
    assert len(planned) == len(set(planned))
    # steps with several instructions exist (they run on different streams)
    steps = {}
    for i in ins:
        steps.setdefault(i["step"], []).append(i)
    assert max(len(v) for v in steps.values()) >= 2
    # tensors are released only after their last use
    last_use = {}
    for i in ins:
        for t in i["inputs"]:
            last_use[t] = i["step"]
    for line in text.splitlines():
        m = re.match(r"step (\d+) release=\[([\d,]*)\]", line)
        if m:
            for t in [int(v) for v in m.group(2).split(",") if v]:
                assert last_use[t] < int(m.group(1))
                assert t not in g.outputs


def test_dead_nodes_are_pruned():
    g = ir.Graph()
    x = g.new_input([64, 64], ir.F32)
    g.unary(ir.UN_EXP, x)  # never used
    g.new_output(g.unary(ir.UN_TANH, x))
    ins = _instrs(hb.HostGraph(g).plan_text())
    assert len(ins) == 1 and ins[0]["nodes"] == [2]


def test_dead_consumers_do_not_make_outputs():
    """A value that only a dead node reads besides its live consumers is not written to memory."""
    g = ir.Graph()
    x = g.new_input([64, 64], ir.F32)
    t = g.unary(ir.UN_TANH, x)
    g.unary(ir.UN_EXP, t)  # dead consumer of t
    g.new_output(g.unary(ir.UN_RELU, t))
    ins = _instrs(hb.HostGraph(g).plan_text())
    assert len(ins) == 1 and ins[0]["nodes"] == [1, 3] and ins[0]["outputs"] == [3]


def test_a_graph_can_grow_after_it_was_planned():
    """Planning remembers which nodes are live; nodes and outputs added afterwards must not be judged by that."""
    g = ir.Graph()
    x = g.new_input([64, 64], ir.F32)
    t = g.unary(ir.UN_TANH, x)
    e = g.unary(ir.UN_EXP, t)          # dead for now
    g.new_output(g.unary(ir.UN_RELU, t))
    h = hb.HostGraph(g)
    assert len(_instrs(h.plan_text())) == 1
    # grow the C++ graph behind the handle: one more op on the dead branch, which becomes an output
    from helium_b200._lib import HeNode, check, lib
    import ctypes as C
    c = HeNode()
    c.kind, c.sub_op, c.dtype, c.rank = ir.OP_UNARY, ir.UN_NEG, ir.F32, 2
    c.inp[0], c.inp[1], c.inp[2] = e, -1, -1
    c.shape[0], c.shape[1] = 64, 64
    out = C.c_int32()
    check(lib.heh_graph_new_op(h._h, C.byref(c), C.byref(out)))
    check(lib.heh_graph_new_output(h._h, out.value))
    ins = _instrs(h.plan_text())
    assert sorted(n for i in ins for n in i["nodes"]) == [1, 2, 3, out.value]
    assert sorted(o for i in ins for o in i["outputs"]) == [3, out.value]
    h.set_planner("search")
    ins = _instrs(h.plan_text())
    assert sorted(o for i in ins for o in i["outputs"]) == [3, out.value]


def test_matmul_epilogue_and_mainloop_fuse_through_the_planner():
    g = ir.Graph()
    a = g.new_input([512, 256], ir.BF16); mk = g.new_input([512, 256], ir.BF16); b = g.new_input([256, 512], ir.BF16)
    bias = g.new_input([512], ir.BF16)
    t = g.matmul(g.binary(ir.BIN_MUL, g.unary(ir.UN_RELU, a), mk), b)
    t = g.unary(ir.UN_GELU, g.binary(ir.BIN_ADD, t, g.broadcast_to(bias, [512, 512])))
    g.new_output(g.cast(t, ir.BF16))
    ins = _instrs(hb.HostGraph(g).plan_text())
    assert len(ins) == 1 and ins[0]["kind"] == "FusedMatmul" and ins[0]["tier"] == 2


def test_readme_graph_fuses_into_one_matmul_instruction():
    """Greedy pairwise fusion (plan_generation.rs:243-256) folds the README graph, op by op, into a
    single FusedMatmul instruction that the kernel catalogue serves at tier 2; the intermediate
    merges are legal because the interpreted epilogue accepts Sum reductions."""
    import helium_b200 as hb
    from helium_b200.configs import graph_c3
    text = hb.HostGraph(graph_c3(1024, 1024, 1024)).plan_text()
    steps = [ln for ln in text.splitlines() if "FusedMatmul" in ln or "Pointwise" in ln or "Permute" in ln]
    assert len(steps) == 1 and "FusedMatmul tier=2" in steps[0], text
