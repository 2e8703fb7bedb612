// Graph types shared by the whole-graph planner (host_graph.cu) and the fusion search (fusion_search.cu):
//   OpGraph / OpSubgraph          helium-ir/src/opgraph.rs:12-191, helium-ir/src/opgraph/subgraph.rs:12-120
//   make_instr_for_op             helium/src/cuda.rs:33-60
//   Instr::{can_fuse_with,fuse_with}   helium/src/cuda/instr.rs:54-99
#pragma once
#include <algorithm>
#include <map>
#include <set>
#include <vector>

#include "he_internal.h"

namespace he {
namespace host {

using NodeId = int;

struct OpGraph {
  std::vector<he_node> nodes;           // in[] = NodeIds; topological by construction
  std::vector<NodeId> inputs;           // HE_OP_INPUT nodes in creation order
  std::vector<NodeId> outputs;          // nodes marked as outputs, in marking order
  std::vector<std::vector<NodeId>> outbound;
  std::vector<bool> live_mask;          // set by the planner: consumers that no output needs do not make a node a leaf

  NodeId add(const he_node& n) {
    nodes.push_back(n);
    outbound.emplace_back();
    live_mask.clear();   // belongs to the graph as it was when a planner last ran
    const NodeId id = (NodeId)nodes.size() - 1;
    for (int k = 0; k < 3; ++k)
      if (n.in[k] >= 0) outbound[n.in[k]].push_back(id);
    if (n.kind == HE_OP_INPUT) inputs.push_back(id);
    return id;
  }
  bool is_output(NodeId id) const { return std::find(outputs.begin(), outputs.end(), id) != outputs.end(); }
  std::vector<NodeId> inbound(NodeId id) const {
    std::vector<NodeId> r;
    for (int k = 0; k < 3; ++k)
      if (nodes[id].in[k] >= 0) r.push_back(nodes[id].in[k]);
    return r;
  }
  // OpGraph::optimize (opgraph.rs:165-191): which intermediates are needed for the outputs
  std::vector<bool> live() const {
    std::vector<bool> l(nodes.size(), false);
    std::vector<NodeId> stack(outputs.begin(), outputs.end());
    while (!stack.empty()) {
      NodeId n = stack.back();
      stack.pop_back();
      if (l[n]) continue;
      l[n] = true;
      for (NodeId p : inbound(n)) stack.push_back(p);
    }
    return l;
  }
};

// Subset of intermediate nodes (subgraph.rs:12-79).
struct OpSubgraph {
  const OpGraph* graph = nullptr;
  std::vector<NodeId> nodes, inputs, leafs;  // all sorted

  static OpSubgraph from_nodes(const OpGraph* g, std::vector<NodeId> ns) {
    OpSubgraph s;
    s.graph = g;
    std::sort(ns.begin(), ns.end());
    ns.erase(std::unique(ns.begin(), ns.end()), ns.end());
    s.nodes = ns;
    std::set<NodeId> in_set(ns.begin(), ns.end()), inputs;
    for (NodeId n : ns)
      for (NodeId p : g->inbound(n))
        if (!in_set.count(p)) inputs.insert(p);
    s.inputs.assign(inputs.begin(), inputs.end());
    for (NodeId n : ns) {
      bool leaf = g->is_output(n);
      for (NodeId c : g->outbound[n])
        if (!in_set.count(c) && (g->live_mask.empty() || g->live_mask[c])) leaf = true;
      if (leaf) s.leafs.push_back(n);
    }
    return s;
  }
  // A subgraph whose outputs are chosen by the caller: with recomputation a node may sit in several
  // instructions and only one of them writes it to memory.
  static OpSubgraph from_nodes_with_leafs(const OpGraph* g, std::vector<NodeId> ns, std::vector<NodeId> leafs) {
    OpSubgraph s = from_nodes(g, std::move(ns));
    std::sort(leafs.begin(), leafs.end());
    leafs.erase(std::unique(leafs.begin(), leafs.end()), leafs.end());
    s.leafs = std::move(leafs);
    return s;
  }
  OpSubgraph merge_with(const OpSubgraph& o) const {
    std::vector<NodeId> ns = nodes;
    ns.insert(ns.end(), o.nodes.begin(), o.nodes.end());
    return from_nodes(graph, ns);
  }
  bool contains(NodeId n) const { return std::binary_search(nodes.begin(), nodes.end(), n); }

  // Flat descriptor for the C ABI: inputs first (as HE_OP_INPUT), then the nodes.
  struct Flat {
    std::vector<he_node> nodes;
    std::vector<int32_t> outputs;
    he_graph_desc desc() const { return he_graph_desc{(int32_t)nodes.size(), nodes.data(), (int32_t)outputs.size(), outputs.data()}; }
  };
  Flat flatten() const {
    Flat f;
    std::map<NodeId, int> index;
    for (NodeId i : inputs) {
      he_node n = graph->nodes[i];
      n.kind = HE_OP_INPUT;
      n.in[0] = n.in[1] = n.in[2] = -1;
      index[i] = (int)f.nodes.size();
      f.nodes.push_back(n);
    }
    for (NodeId i : nodes) {
      he_node n = graph->nodes[i];
      for (int k = 0; k < 3; ++k)
        if (n.in[k] >= 0) n.in[k] = index.at(n.in[k]);
      index[i] = (int)f.nodes.size();
      f.nodes.push_back(n);
    }
    for (NodeId l : leafs) f.outputs.push_back(index.at(l));
    return f;
  }
};

enum class InstrKind { PointwiseGraph = 0, PermuteDims = 1, FusedMatmul = 2 };
inline const char* kind_name(InstrKind k) {
  return k == InstrKind::PointwiseGraph ? "PointwiseGraph" : k == InstrKind::PermuteDims ? "PermuteDims" : "FusedMatmul";
}

struct Instr {
  InstrKind kind;
  OpSubgraph sub;
  const std::vector<NodeId>& inputs() const { return sub.inputs; }
  const std::vector<NodeId>& outputs() const { return sub.leafs; }

  int tier(he_ctx* ctx) const {
    OpSubgraph::Flat f = sub.flatten();
    he_graph_desc d = f.desc();
    return he_plan_supported(ctx, &d, (int)kind);
  }

  // Kind of the instruction that results from fusing `this` with `next`, or nothing.
  bool fused_kind(const Instr& next, InstrKind* out) const {
    if (kind == InstrKind::FusedMatmul && next.kind == InstrKind::FusedMatmul) return false;
    if (kind == InstrKind::FusedMatmul || next.kind == InstrKind::FusedMatmul) {
      *out = InstrKind::FusedMatmul;
      return true;
    }
    if (kind == next.kind) {
      *out = kind;
      return true;
    }
    *out = InstrKind::PointwiseGraph;  // PermuteDims x PointwiseGraph: only via a single-pass kernel
    return true;
  }

  bool can_fuse_with(const Instr& next, he_ctx* ctx) const {
    InstrKind k;
    if (!fused_kind(next, &k)) return false;
    Instr merged{k, sub.merge_with(next.sub)};
    const int t = merged.tier(ctx);
    if (kind != next.kind && k == InstrKind::PointwiseGraph) {
      // a permutation folds into a pointwise kernel when a single-pass kernel exists for the pair
      // (tier 2), or when it only feeds reductions: those read through the swapped view in column
      // mode, coalesced, and no permuted copy is ever written
      bool only_reductions = true;
      for (NodeId l : merged.sub.leafs) only_reductions = only_reductions && sub.graph->nodes[l].kind == HE_OP_REDUCE;
      return t == 2 || (t > 0 && only_reductions);
    }
    // Greedy pairwise fusion passes through partial subgraphs that only the interpreter tier
    // serves on the way to one that a hand-written kernel serves, so tier 1 is accepted here.
    return t > 0;
  }
  Instr fuse_with(const Instr& next) const {
    InstrKind k = kind;
    fused_kind(next, &k);
    return Instr{k, sub.merge_with(next.sub)};
  }
};

// cuda.rs:33-60
inline Instr make_instr_for_op(const OpGraph* g, NodeId id) {
  const he_node& n = g->nodes[id];
  OpSubgraph s = OpSubgraph::from_nodes(g, {id});
  if (n.kind == HE_OP_MATMUL) return Instr{InstrKind::FusedMatmul, s};
  if (n.kind == HE_OP_SWAP_DIMS && num_elements(n) > 1000000 && n.dtype != HE_BOOL) return Instr{InstrKind::PermuteDims, s};
  return Instr{InstrKind::PointwiseGraph, s};
}

}  // namespace host
}  // namespace he
