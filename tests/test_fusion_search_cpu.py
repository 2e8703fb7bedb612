"""The fusion search of the C++ host runtime (helium_b200/csrc/fusion_search.cu), the counterpart of the
playground's search: helium-playground/src/fused_graph.rs (states, moves), subdivision.rs, cost_model.rs.

Planning needs no GPU.  The reference pins one expected value for this component (subdivision.rs:117-171,
`example_subdivision`); its other tests (`simple_graph_actions`, `complex_graph`, `merge_from_subdivisions`,
fused_graph.rs:1296-1446) build a graph, run the search and assert only that its invariants hold.  The same
graphs are searched here and the invariants are checked from the outside, on the text the C ABI returns."""
import re

import pytest

import helium_b200 as hb
from helium_b200 import configs, ir


def _parse(text):
    head = dict((k, float(v)) for k, v in re.findall(r"(\w+)=([-+.\de]+)", text.splitlines()[0]))
    groups = []
    for line in text.splitlines()[1:]:
        m = re.match(r"group (\d+) (\w+) anchor=(-?\d+) pre=\[([\d,]*)\] post=\[([\d,]*)\] in=\[([\d,]*)\] out=\[([\d,]*)\] seconds=(\S+)", line)
        assert m, line
        f = lambda s: [int(v) for v in s.split(",") if v]
        groups.append(dict(kind=m.group(2), anchor=int(m.group(3)), pre=f(m.group(4)), post=f(m.group(5)),
                           reads=f(m.group(6)), exports=f(m.group(7)), seconds=float(m.group(8))))
    return head, groups


def _live(g):
    live, stack = set(), list(g.outputs)
    while stack:
        n = stack.pop()
        if n in live:
            continue
        live.add(n)
        stack.extend(i for i in g.nodes[n].inputs if i >= 0)
    return live


def _check_invariants(g, head, groups):
    """What fused_graph.rs:838-883 (`assert_invariants`) asserts, restated for this result format."""
    live = _live(g)
    inputs = set(g.inputs)
    written = set(inputs)
    covered = set()
    for grp in groups:
        nodes = set(grp["pre"]) | set(grp["post"]) | ({grp["anchor"]} if grp["anchor"] >= 0 else set())
        assert nodes and nodes <= live - inputs
        assert (grp["anchor"] >= 0) == (grp["kind"] == "FusedMatmul")
        if grp["anchor"] >= 0:
            assert g.nodes[grp["anchor"]].kind == ir.OP_MATMUL
        assert not any(g.nodes[n].kind == ir.OP_MATMUL for n in grp["pre"] + grp["post"])   # a matmul is never recomputed
        # every value a node needs is computed in the group or read from memory, where an earlier group put it
        need = set()
        for n in nodes:
            need |= {i for i in g.nodes[n].inputs if i >= 0 and i not in nodes}
        assert need == set(grp["reads"]), (grp, need)
        assert need <= written, (grp, need - written)
        # operand-side values live in the mainloop only
        assert set(grp["exports"]) <= (set(grp["post"]) | {grp["anchor"]})
        assert grp["exports"], grp
        assert not (set(grp["exports"]) & written), "a node is written to memory by one kernel only"
        written |= set(grp["exports"])
        covered |= nodes
    assert covered == live - inputs
    assert set(g.outputs) - inputs <= written
    # the greedy start merges without looking at the cost, so it may be dearer than one kernel per node
    assert head["best"] <= min(head["maximal"], head["identity"]) * (1 + 1e-9)
    # the pairwise planner's plan seeds a descent of its own: never dearer than the reference's planner, by the model
    if head["pairwise"] >= 0:
        assert head["best"] <= head["pairwise"] * (1 + 1e-9)
    assert abs(sum(grp["seconds"] for grp in groups) - head["best"]) <= 1e-6 * head["best"] + 1e-12
    count = {}
    for grp in groups:
        for n in grp["pre"] + grp["post"]:
            count[n] = count.get(n, 0) + 1
    assert sum(1 for c in count.values() if c > 1) == int(head["recomputed"])
    # at most three copies of a node that costs instructions (fused_graph.rs:413)
    free = (ir.OP_CONSTANT, ir.OP_BROADCAST, ir.OP_RESHAPE, ir.OP_SWAP_DIMS)
    assert all(c <= 3 for n, c in count.items() if g.nodes[n].kind not in free)


def _search(g, depth=0, max_states=0):
    h = hb.HostGraph(g)
    h.set_planner("search", depth, max_states)
    text = h.search_text()
    head, groups = _parse(text)
    _check_invariants(g, head, groups)
    return h, head, groups


def _reference_subdivision_graph():
    g = ir.Graph()
    x = g.new_input([1, 256, 256], ir.F32)
    mm1 = g.matmul(x, x, ir.PREC_F32_F32)
    relu1 = g.unary(ir.UN_RELU, mm1)
    add1 = g.binary(ir.BIN_ADD, relu1, x)
    mm2 = g.matmul(mm1, x, ir.PREC_F32_F32)
    relu2 = g.unary(ir.UN_RELU, mm2)
    add2 = g.binary(ir.BIN_ADD, relu2, x)
    g.new_output(add1)
    g.new_output(add2)
    return g, (mm1, relu1, add1, mm2, relu2, add2)


def test_subdivision_golden_of_the_reference():
    """subdivision.rs:117-171: the one pinned expectation the reference holds for this component."""
    g, (mm1, relu1, add1, mm2, relu2, add2) = _reference_subdivision_graph()
    got = sorted(sorted(s) for s in hb.HostGraph(g).subdivisions())
    want = sorted([
        sorted([(mm1, "m")]),
        sorted([(mm1, "e"), (relu1, ""), (add1, ""), (mm2, "m")]),
        sorted([(mm2, "e"), (relu2, ""), (add2, "")]),
    ])
    assert got == want


def test_every_whole_node_is_in_exactly_one_subdivision_and_every_matmul_in_two():
    for g in (configs.graph_mlp_train_step(), configs.graph_mlp_block_train(256, 128, 256), configs.graph_c3(256, 256, 256)):
        seen = {}
        for s in hb.HostGraph(g).subdivisions():
            for n, portion in s:
                seen.setdefault(n, []).append(portion)
        for i, n in enumerate(g.nodes):
            if n.kind == ir.OP_INPUT:
                assert i not in seen
            elif n.kind == ir.OP_MATMUL:
                assert sorted(seen[i]) == ["e", "m"]
            else:
                assert seen[i] == [""]


def test_search_on_the_reference_subdivision_graph():
    g, _ = _reference_subdivision_graph()
    _, head, groups = _search(g)
    assert head["subdivisions"] == 3
    assert len(groups) <= 4   # six nodes in at most four kernels


def test_simple_graph_of_the_reference_tests():
    """fused_graph.rs:1296-1327: c = a + b; d = c x b; e = exp(d); f = d x e."""
    g = ir.Graph()
    a = g.new_input([1, 256, 256], ir.BF16)
    b = g.new_input([1, 256, 256], ir.BF16)
    c = g.binary(ir.BIN_ADD, a, b)
    d = g.cast(g.matmul(c, b), ir.BF16)
    e = g.unary(ir.UN_EXP, d)
    f = g.matmul(d, e)
    g.new_output(f)
    _, head, groups = _search(g)
    # two matmuls, two kernels: the sum moves to the first one's operand side, exp to either matmul
    assert [grp["kind"] for grp in groups] == ["FusedMatmul", "FusedMatmul"]
    assert groups[0]["pre"] == [c]
    assert head["best"] < head["identity"]


def test_complex_graph_of_the_reference_tests():
    """fused_graph.rs:1376-1410: forward and backward of a two-layer net with shared operands."""
    g = ir.Graph()
    n0 = g.new_input([1, 1024, 1024], ir.BF16)
    n1 = g.new_input([1, 1024, 1024], ir.BF16)
    mm = lambda x, y: g.cast(g.matmul(x, y), ir.BF16)
    n2 = mm(n0, n1)
    n3 = g.unary(ir.UN_EXP, n2)
    n4 = g.binary(ir.BIN_ADD, n3, n1)
    n5 = mm(n0, n4)
    n6 = mm(n5, n4)
    n7 = mm(n5, n0)
    n8 = g.binary(ir.BIN_ADD, n3, n7)
    n9 = mm(n8, n2)
    g.new_output(n6)
    g.new_output(n9)
    _, head, groups = _search(g)
    assert sum(grp["kind"] == "FusedMatmul" for grp in groups) == 5
    assert head["best"] < head["maximal"] or len(groups) == 5


def test_merge_graph_of_the_reference_tests():
    """fused_graph.rs:1413-1445: relu(x x x) + x ends up in the matmul's kernel or next to it, never in three kernels."""
    g = ir.Graph()
    a = g.new_input([1, 256, 256], ir.BF16)
    b = g.new_input([1, 256, 256], ir.BF16)
    r = g.binary(ir.BIN_ADD, g.unary(ir.UN_RELU, g.matmul(a, b)), g.cast(a, ir.F32))
    g.new_output(r)
    _, head, groups = _search(g)
    assert len(groups) == 1 and groups[0]["kind"] == "FusedMatmul"


def test_a_shared_cheap_producer_is_recomputed_instead_of_written():
    """The bias row broadcast to [M, N] feeds the epilogues of two matmuls.  Pairwise merging cannot fold a node
    with two consumers into either; the search recomputes it in both kernels (fused_graph.rs:19-31) and no
    kernel writes the broadcast tensor."""
    M, N, K = 512, 512, 256
    g = ir.Graph()
    x = g.new_input([M, K], ir.BF16); w1 = g.new_input([K, N], ir.BF16); w2 = g.new_input([K, N], ir.BF16)
    b = g.new_input([N], ir.F32)
    bb = g.broadcast_to(b, [M, N])
    g.new_output(g.cast(g.binary(ir.BIN_ADD, g.matmul(x, w1), bb), ir.BF16))
    g.new_output(g.cast(g.binary(ir.BIN_ADD, g.matmul(x, w2), bb), ir.BF16))
    h, head, groups = _search(g)
    assert len(groups) == 2 and all(grp["kind"] == "FusedMatmul" for grp in groups)
    assert all(bb in grp["post"] and bb not in grp["exports"] for grp in groups)
    assert head["recomputed"] == 1
    # the plan built from it runs both kernels in one step and never materialises the broadcast
    lines = [ln for ln in h.plan_text().splitlines() if "tier=" in ln]
    assert len(lines) == 2 and all(ln.startswith("step 0 FusedMatmul") for ln in lines)
    # pairwise merging folds the broadcast into the first matmul, which then has to write it to memory for the
    # second one: two steps and M x N x 4 bytes more traffic each way
    pairwise = [ln for ln in hb.HostGraph(g).plan_text().splitlines() if "tier=" in ln]
    assert len(pairwise) == 2 and pairwise[0].startswith("step 0") and pairwise[1].startswith("step 1")
    assert f"out=[{bb}," in pairwise[0]


@pytest.mark.parametrize("name", ["mlp_step", "mlp_block", "readme"])
def test_search_plans_are_executable_plans(name):
    g = {"mlp_step": lambda: configs.graph_mlp_train_step(),
         "mlp_block": lambda: configs.graph_mlp_block_train(256, 128, 256),
         "readme": lambda: configs.graph_c3(1024, 1024, 1024)}[name]()
    h, head, groups = _search(g, max_states=3000)
    text = h.plan_text()
    seen = set(g.inputs)
    n_instr = 0
    for line in text.splitlines():
        m = re.match(r"step (\d+) (\w+) tier=(\d) nodes=\[([\d,]*)\] in=\[([\d,]*)\] out=\[([\d,]*)\]", line)
        if not m:
            continue
        n_instr += 1
        f = lambda s: [int(v) for v in s.split(",") if v]
        assert int(m.group(3)) > 0, line                       # every kernel of the result exists
        assert set(f(m.group(5))) <= seen, line               # and reads only what earlier steps wrote
        seen |= set(f(m.group(6)))
    assert n_instr == len(groups)
    assert set(g.outputs) <= seen
    if name == "readme":
        assert n_instr == 1   # the whole README graph is one fused matmul, as with the pairwise planner
    # the default planner is untouched by all of this
    assert hb.HostGraph(g).plan_text() != ""


def test_search_is_deterministic_and_bounded():
    g = configs.graph_mlp_train_step()
    h1, head1, groups1 = _search(g, depth=2, max_states=500)
    h2, head2, groups2 = _search(g, depth=2, max_states=500)
    assert groups1 == groups2 and head1 == head2
    # two descents (from the greedy start and from single nodes) over four subdivisions, 500 states each at most,
    # plus the greedy start itself
    assert head1["states"] <= 2 * 4 * 500 + 2000
    # a larger budget never gives a costlier plan
    _, head3, _ = _search(g, depth=3, max_states=4000)
    assert head3["best"] <= head1["best"] * (1 + 1e-9)


def test_planner_arguments_are_checked():
    g = configs.graph_c3(256, 256, 256)
    h = hb.HostGraph(g)
    with pytest.raises(hb.HeliumError):
        h.set_planner("search", depth=99)
    with pytest.raises(KeyError):
        h.set_planner("annealing")


@pytest.mark.parametrize("flavour", ["bf16", "f32", "batched", "f16_select"])
@pytest.mark.parametrize("seed", range(30))
def test_invariants_on_random_graphs(seed, flavour):
    """Shared operands, transposes, broadcast rows and column sums around up to three matmuls (tests/graph_fuzz.py):
    every result of the search is a consistent set of kernels, each of which exists."""
    from graph_fuzz import random_graph
    g, _ = random_graph(seed, flavour=flavour)
    h, head, groups = _search(g, max_states=2000)
    text = h.plan_text()
    assert "tier=0" not in text, text
    assert text.count("tier=") == len(groups)
    assert "tier=0" not in hb.HostGraph(g).plan_text()


@pytest.mark.parametrize("shape,axes", [([128, 128], [0]), ([4, 64, 32], [1]), ([4, 64, 32], [0]), ([4, 64, 32], [0, 2]), ([8, 1, 16], [0])])
def test_rank_kept_reductions_over_leading_axes_have_a_kernel(shape, axes):
    """The playground's Reduction over any axes (opgraph.rs:397-413) as a kernel of its own, not only inside a
    matmul epilogue: he_plan_supported accepts it (it is planned as swaps to a trailing reduction)."""
    g = ir.Graph()
    x = g.new_input(shape, ir.BF16)
    g.new_output(g.reduce_axes(ir.RED_SUM, g.unary(ir.UN_RELU, x), axes))
    assert hb.plan_supported(g, 0) == 1
