// Fusion search (see fusion_search.h).  Host code only.
//
// State.  A state is a set of groups, one kernel each.  A group is a matmul with operand-side ("pre") and
// result-side ("post") nodes, or a pointwise kernel (all nodes in "post").  A node may sit in several groups: it is
// then recomputed in each of them (fused_graph.rs:19-31).  For every node that some group reads from memory, or that
// is an output of the graph, exactly one group is its exporter: the one kernel that writes it.  Everything else --
// what a group reads, which group depends on which -- is derived from these two facts, so a state cannot be
// inconsistent in the ways the playground's assert_invariants (fused_graph.rs:838-883) has to look for.
//
// Moves (fused_graph.rs:1225-1262 has four kinds):
//   absorb a consumer of a group's result side into that side, the group becoming its exporter;
//   absorb a producer of a result-side node into the result side (recomputation: the group stops reading it);
//   absorb a producer of a matmul operand into the operand side;
//   hand the export of a node to another group that also computes it (the playground's edge transition, for all
//   readers at once);
//   take a whole pointwise group into the result side or the operand side of a group it exchanges a value with
//   (the pairwise merge of plan_generation.rs:243-256 as a move: some kernels exist for a chain -- a transposed
//   view, its reduction and the reshape of that -- and for no proper prefix of it).
// After a move, nodes a group computes for nobody are dropped and groups left empty disappear.  A move is legal only
// if the group graph stays acyclic and he_plan_supported accepts every group: the search ranges over what the
// kernels of this library run, not over an abstract op vocabulary.
//
// Search (cost_model.rs:241-343): three starting states -- the greedy one (merge while a merge removes a kernel:
// produce_maximal_fusions, fused_graph.rs:113-223), one kernel per node, and the plan of the pairwise planner when
// the caller hands it over -- are each improved by steepest descent, one move at a time; where that is stuck a
// look-ahead of a few moves follows the cheapest moves of each level; the cheapest end state wins.  The number of
// states costed per descent is capped, so planning time is bounded; the playground's descent is exhaustive to
// depth 7.
// Subdivisions restrict which nodes may move in one descent instead of cutting the graph into subgraphs that have to
// be merged afterwards (fused_graph.rs:925-1079): the state is always the whole graph.
#include "fusion_search.h"

#include <cmath>
#include <cstring>
#include <functional>
#include <numeric>
#include <sstream>
#include <unordered_map>
#include <unordered_set>

namespace he {
namespace host {

namespace {

bool in_sorted(const std::vector<NodeId>& v, NodeId n) { return std::binary_search(v.begin(), v.end(), n); }
void insert_sorted(std::vector<NodeId>& v, NodeId n) {
  auto it = std::lower_bound(v.begin(), v.end(), n);
  if (it == v.end() || *it != n) v.insert(it, n);
}

struct Group {
  NodeId anchor = -1;
  std::vector<NodeId> pre, post;
  bool has(NodeId n) const { return n == anchor || in_sorted(pre, n) || in_sorted(post, n); }
  bool exportable(NodeId n) const { return n == anchor || in_sorted(post, n); }
  bool empty() const { return anchor < 0 && post.empty(); }
  std::vector<NodeId> all() const {
    std::vector<NodeId> v = pre;
    v.insert(v.end(), post.begin(), post.end());
    if (anchor >= 0) v.push_back(anchor);
    std::sort(v.begin(), v.end());
    return v;
  }
};

struct State {
  std::map<int, Group> groups;
  int next_id = 0;
  std::vector<int> exporter;   // per node: id of the group that writes it to memory, or -1
};

enum class MoveKind { AbsorbConsumer, AbsorbProducer, AbsorbOperand, MoveExport, MergeConsumerGroup, MergeOperandGroup };
struct Move {
  MoveKind kind;
  int group;
  NodeId node;   // for the two merges: id of the pointwise group that is taken in whole
};

// ---- cost model ------------------------------------------------------------------------------------
// Constants are measurements of this library's kernels on one B200, not the playground's Ampere fit
// (cost_model.rs:206-213):
//   kLaunch        a kernel replayed from a CUDA graph next to its neighbours: ~2 us of device time
//   kHbm           6.55e12 B/s copy bandwidth; elementwise kernels specialised at plan time reach 0.84 of it,
//                  reductions 0.76, GEMM operand / result traffic ~0.8
//   kTensor        1.40e15 flop/s sustained bf16; a GEMM with a light epilogue reaches 0.86 of it
//   kEpilogueOp    8192 x 16384 x 4096 with bias + exact GELU + a second output runs at 0.73 instead of 0.86 of
//                  sustained: 0.16 ms for 1.34e8 outputs x 21 weight units (add 1, GELU 20) = 5.7e-14 s per unit and
//                  output element; the gelu' gate with its column sum (0.78 of sustained) then puts DGELU at ~12 units
//   kMainloopOp    4096^3 with relu(A) * mask rewritten in the mainloop: 0.278 ms against 0.170 ms planned with a
//                  pre-pass: 0.1 ms for 1.7e7 elements x 16 column tiles x 2 units = 2e-13 s per unit, element and tile
//   kAluOp         pointwise kernels stay HBM-bound up to ~40 units per element: 148 SMs x 128 lanes x 1.9 GHz
constexpr double kLaunch = 2.0e-6;
constexpr double kHbm = 6.55e12;
constexpr double kTensor = 1.40e15 * 0.86;
constexpr double kEpilogueOp = 5.7e-14;
constexpr double kMainloopOp = 2.0e-13;
constexpr double kAluOp = 1.0 / (148.0 * 128.0 * 1.9e9);

// Relative instruction cost of one node per element (cost_model.rs:150-186 has the playground's table).
double op_weight(const he_node& n) {
  switch (n.kind) {
    case HE_OP_UNARY:
      switch (n.sub_op) {
        case HE_UN_NEG: case HE_UN_RELU: case HE_UN_ADD_CONST: case HE_UN_MUL_CONST: return 1;
        case HE_UN_RECIP: case HE_UN_SQRT: return 4;
        case HE_UN_EXP: case HE_UN_LOG: case HE_UN_SIGMOID: return 6;
        case HE_UN_SIN: case HE_UN_COS: case HE_UN_TAN: case HE_UN_TANH: return 8;
        case HE_UN_GELU: return 20;
        case HE_UN_DGELU: return 12;
        case HE_UN_POW_CONST: return 12;
        default: return 4;
      }
    case HE_OP_BINARY:
      return n.sub_op == HE_BIN_DIV ? 5 : n.sub_op == HE_BIN_POW ? 24 : n.sub_op == HE_BIN_DRELU ? 2 : 1;
    case HE_OP_CAST: case HE_OP_COMPARE: case HE_OP_SELECT: return 1;
    case HE_OP_REDUCE: return 3;
    default: return 0;   // constants, broadcasts, reshapes and swaps only change how elements are addressed
  }
}

double node_bytes(const he_node& n) { return (double)storage_bytes(n.dtype, num_elements(n)); }

struct Searcher {
  const OpGraph& g;
  he_ctx* ctx;
  SearchOptions opt;
  int N;
  std::vector<bool> live;
  std::vector<char> is_output;
  mutable std::unordered_map<std::string, int> support_cache;
  int states = 0;

  Searcher(const OpGraph& graph, he_ctx* c, const SearchOptions& o) : g(graph), ctx(c), opt(o), N((int)graph.nodes.size()) {
    live = g.live();
    is_output.assign(N, 0);
    for (NodeId o2 : g.outputs) is_output[o2] = 1;
  }

  const he_node& node(NodeId n) const { return g.nodes[n]; }
  bool is_input(NodeId n) const { return node(n).kind == HE_OP_INPUT; }
  bool is_anchor(NodeId n) const { return node(n).kind == HE_OP_MATMUL; }
  bool is_reduce(NodeId n) const { return node(n).kind == HE_OP_REDUCE; }

  // Nodes the group reads from memory.  *bad: a result-side node would need a value that exists only in the
  // mainloop's registers, or the other way round.
  std::vector<NodeId> reads(const Group& G, bool* bad) const {
    std::set<NodeId> r;
    for (NodeId n : G.pre)
      for (NodeId p : g.inbound(n))
        if (!in_sorted(G.pre, p)) {
          if (G.exportable(p) && bad) *bad = true;
          r.insert(p);
        }
    if (G.anchor >= 0)
      for (NodeId p : g.inbound(G.anchor))
        if (!in_sorted(G.pre, p)) {
          if (in_sorted(G.post, p) && bad) *bad = true;
          r.insert(p);
        }
    for (NodeId n : G.post)
      for (NodeId p : g.inbound(n))
        if (!G.exportable(p)) {
          if (in_sorted(G.pre, p) && bad) *bad = true;
          r.insert(p);
        }
    return std::vector<NodeId>(r.begin(), r.end());
  }

  std::vector<NodeId> exports(const State& s, int id, const Group& G) const {
    std::vector<NodeId> e;
    for (NodeId n : G.post)
      if (s.exporter[n] == id) e.push_back(n);
    if (G.anchor >= 0 && s.exporter[G.anchor] == id) e.push_back(G.anchor);
    std::sort(e.begin(), e.end());
    return e;
  }

  State identity() const {
    State s;
    s.exporter.assign(N, -1);
    for (NodeId n = 0; n < N; ++n) {
      if (is_input(n) || !live[n]) continue;
      Group G;
      if (is_anchor(n)) G.anchor = n;
      else G.post.push_back(n);
      s.groups.emplace(s.next_id++, std::move(G));
    }
    return s;
  }

  // Brings the derived facts back in line after a change: exporters for what is read, nothing computed for
  // nobody.  false when the state cannot be completed.
  bool fix(State& s) const {
    for (int iter = 0; iter < 64; ++iter) {
      bool changed = false;
      std::vector<char> read_ext(N, 0);
      for (auto& kv : s.groups) {
        bool bad = false;
        for (NodeId p : reads(kv.second, &bad)) read_ext[p] = 1;
        if (bad) return false;
      }
      for (NodeId n = 0; n < N; ++n) {
        if (is_input(n)) continue;
        const bool need = live[n] && (is_output[n] || read_ext[n]);
        if (s.exporter[n] >= 0) {
          auto it = s.groups.find(s.exporter[n]);
          if (!need || it == s.groups.end() || !it->second.exportable(n)) {
            s.exporter[n] = -1;
            changed = true;
          }
        }
        if (need && s.exporter[n] < 0) {
          for (auto& kv : s.groups)
            if (kv.second.exportable(n)) {
              s.exporter[n] = kv.first;
              break;
            }
          if (s.exporter[n] < 0) return false;
          changed = true;
        }
      }
      std::vector<int> ids;
      for (auto& kv : s.groups) ids.push_back(kv.first);
      for (int id : ids) {
        Group& G = s.groups.at(id);
        std::set<NodeId> needed_pre, needed_post;
        std::vector<std::pair<NodeId, int>> stack;   // (node, side: 0 operand, 1 result, 2 anchor)
        for (NodeId n : G.post)
          if (s.exporter[n] == id) stack.push_back({n, 1});
        if (G.anchor >= 0) stack.push_back({G.anchor, 2});
        std::set<std::pair<NodeId, int>> seen(stack.begin(), stack.end());
        while (!stack.empty()) {
          auto [cur, side] = stack.back();
          stack.pop_back();
          if (side == 0) needed_pre.insert(cur);
          if (side == 1) needed_post.insert(cur);
          for (NodeId p : g.inbound(cur)) {
            std::pair<NodeId, int> nx{-1, 0};
            if (side == 1) {
              if (p == G.anchor) continue;
              if (in_sorted(G.post, p)) nx = {p, 1};
            } else if (in_sorted(G.pre, p)) {
              nx = {p, 0};
            }
            if (nx.first >= 0 && seen.insert(nx).second) stack.push_back(nx);
          }
        }
        if (needed_pre.size() != G.pre.size() || needed_post.size() != G.post.size()) {
          G.pre.assign(needed_pre.begin(), needed_pre.end());
          G.post.assign(needed_post.begin(), needed_post.end());
          changed = true;
        }
        if (G.empty()) {
          s.groups.erase(id);
          changed = true;
        }
      }
      if (!changed) return true;
    }
    return false;
  }

  bool acyclic(const State& s, std::vector<int>* order = nullptr) const {
    std::map<int, std::set<int>> out;
    std::map<int, int> indeg;
    for (auto& kv : s.groups) indeg[kv.first] = 0;
    for (auto& kv : s.groups)
      for (NodeId p : reads(kv.second, nullptr)) {
        if (is_input(p)) continue;
        const int src = s.exporter[p];
        if (src < 0 || src == kv.first) return false;
        if (out[src].insert(kv.first).second) ++indeg[kv.first];
      }
    std::vector<int> ready;
    for (auto& kv : indeg)
      if (kv.second == 0) ready.push_back(kv.first);
    size_t done = 0;
    while (!ready.empty()) {
      // smallest id first: a stable order for the report
      auto it = std::min_element(ready.begin(), ready.end());
      const int cur = *it;
      ready.erase(it);
      ++done;
      if (order) order->push_back(cur);
      for (int nx : out[cur])
        if (--indeg[nx] == 0) ready.push_back(nx);
    }
    return done == s.groups.size();
  }

  InstrKind kind_of(const Group& G) const {
    if (G.anchor >= 0) return InstrKind::FusedMatmul;
    bool all_swaps = true;
    for (NodeId n : G.post) all_swaps = all_swaps && node(n).kind == HE_OP_SWAP_DIMS;
    if (all_swaps && !G.post.empty()) {
      const he_node& last = node(G.post.back());
      if (num_elements(last) > 1000000 && last.dtype != HE_BOOL) return InstrKind::PermuteDims;
    }
    return InstrKind::PointwiseGraph;
  }

  // Tier he_plan_supported gives the group as one kernel (0: no kernel).
  int tier_of(const Group& G, const std::vector<NodeId>& exp) const {
    std::ostringstream key;
    key << G.anchor << '|';
    for (NodeId n : G.pre) key << n << ',';
    key << '|';
    for (NodeId n : G.post) key << n << ',';
    key << '|';
    for (NodeId n : exp) key << n << ',';
    auto it = support_cache.find(key.str());
    if (it != support_cache.end()) return it->second;
    OpSubgraph sub = OpSubgraph::from_nodes_with_leafs(&g, G.all(), exp);
    InstrKind k = kind_of(G);
    OpSubgraph::Flat f = sub.flatten();
    he_graph_desc d = f.desc();
    int tier = exp.empty() ? 0 : he_plan_supported(ctx, &d, (int)k);
    if (k == InstrKind::PermuteDims && tier == 0) tier = he_plan_supported(ctx, &d, (int)InstrKind::PointwiseGraph);
    if (k == InstrKind::PointwiseGraph && tier > 0 && G.post.size() > 1) {
      // a large permutation joins a pointwise kernel only where host_graph.cu's pairwise rule lets it: a single-pass
      // kernel exists, or the permuted view only feeds reductions
      bool big_swap = false, only_reductions = true;
      for (NodeId n : G.post) {
        if (!(node(n).kind == HE_OP_SWAP_DIMS && num_elements(node(n)) > 1000000 && node(n).dtype != HE_BOOL)) continue;
        big_swap = true;
        only_reductions = only_reductions && !std::binary_search(exp.begin(), exp.end(), n);
        for (NodeId c : g.outbound[n])
          if (G.has(c)) only_reductions = only_reductions && (is_reduce(c) || node(c).kind == HE_OP_SWAP_DIMS);
      }
      if (big_swap && tier != 2 && !only_reductions) tier = 0;
    }
    support_cache.emplace(key.str(), tier);
    return tier;
  }

  static bool single(const Group& G) { return G.pre.empty() && G.post.size() + (G.anchor >= 0 ? 1 : 0) == 1; }

  // A node without a kernel of its own (the pairwise planner starts from such instructions too) stays in the
  // state at a prohibitive cost, so that the search fuses it away if it can.
  bool legal(const State& s) const {
    for (auto& kv : s.groups)
      if (!single(kv.second) && tier_of(kv.second, exports(s, kv.first, kv.second)) == 0) return false;
    return true;
  }

  int copies(const State& s, NodeId n) const {
    int c = 0;
    for (auto& kv : s.groups) c += kv.second.has(n) ? 1 : 0;
    return c;
  }

  std::vector<Move> moves(const State& s, const std::vector<char>* allowed) const {
    constexpr int kMaxCopies = 3;   // fused_graph.rs:413: HEURISTIC_MAX_NODE_RECOMPUTATIONS
    std::vector<Move> mv;
    auto movable = [&](NodeId n) {
      if (!live[n] || is_input(n) || is_anchor(n)) return false;
      if (allowed && !(*allowed)[n]) return false;
      return !(op_weight(node(n)) > 0 && copies(s, n) >= kMaxCopies);
    };
    for (auto& kv : s.groups) {
      const Group& G = kv.second;
      std::set<NodeId> seen_c, seen_p;
      std::vector<NodeId> bases = G.post;
      if (G.anchor >= 0) bases.push_back(G.anchor);
      for (NodeId x : bases) {
        // The playground ends a fusion at every reduction and transpose (opgraph.rs:456-458).  Here the kernels
        // answer: a reshape of a reduced value, say, still belongs to the kernel that reduces.
        for (NodeId c : g.outbound[x])
          if (!G.has(c) && movable(c) && seen_c.insert(c).second) mv.push_back({MoveKind::AbsorbConsumer, kv.first, c});
        if (x != G.anchor)
          for (NodeId p : g.inbound(x))
            if (!G.has(p) && movable(p) && !is_reduce(p) && seen_p.insert(p).second) mv.push_back({MoveKind::AbsorbProducer, kv.first, p});
      }
      if (G.anchor >= 0) {
        std::set<NodeId> seen_o;
        std::vector<NodeId> ob = G.pre;
        ob.push_back(G.anchor);
        for (NodeId x : ob)
          for (NodeId p : g.inbound(x))
            if (!G.has(p) && movable(p) && !is_reduce(p) && seen_o.insert(p).second) mv.push_back({MoveKind::AbsorbOperand, kv.first, p});
      }
    }
    for (NodeId n = 0; n < N; ++n) {
      if (s.exporter[n] < 0 || (allowed && !(*allowed)[n])) continue;
      for (auto& kv : s.groups)
        if (kv.first != s.exporter[n] && kv.second.exportable(n)) mv.push_back({MoveKind::MoveExport, kv.first, n});
    }
    // whole pointwise groups into a group they read from (result side) or feed an operand of (operand side)
    for (auto& hv : s.groups) {
      const Group& H = hv.second;
      if (H.anchor >= 0) continue;
      bool ok = true;
      for (NodeId n : H.post) ok = ok && movable(n);
      if (!ok) continue;
      std::set<int> producers, consumers;
      for (NodeId p : reads(H, nullptr))
        if (!is_input(p) && s.exporter[p] >= 0 && s.exporter[p] != hv.first) producers.insert(s.exporter[p]);
      for (int gid : producers) mv.push_back({MoveKind::MergeConsumerGroup, gid, hv.first});
      for (auto& gv : s.groups) {
        const Group& G = gv.second;
        if (G.anchor < 0 || gv.first == hv.first) continue;
        bool feeds = false;
        std::vector<NodeId> ob = G.pre;
        ob.push_back(G.anchor);
        for (NodeId x : ob)
          for (NodeId p : g.inbound(x)) feeds = feeds || (s.exporter[p] == hv.first && in_sorted(H.post, p));
        if (feeds) mv.push_back({MoveKind::MergeOperandGroup, gv.first, hv.first});
      }
    }
    return mv;
  }

  bool apply(const State& cur, const Move& m, State* out) {
    State s = cur;
    auto it = s.groups.find(m.group);
    if (it == s.groups.end()) return false;
    switch (m.kind) {
      case MoveKind::AbsorbConsumer:
        insert_sorted(it->second.post, m.node);
        s.exporter[m.node] = m.group;
        break;
      case MoveKind::AbsorbProducer: insert_sorted(it->second.post, m.node); break;
      case MoveKind::AbsorbOperand: insert_sorted(it->second.pre, m.node); break;
      case MoveKind::MoveExport: s.exporter[m.node] = m.group; break;
      case MoveKind::MergeConsumerGroup:
      case MoveKind::MergeOperandGroup: {
        auto ht = s.groups.find((int)m.node);
        if (ht == s.groups.end() || ht == it || ht->second.anchor >= 0) return false;
        const std::vector<NodeId> taken = ht->second.post;
        for (NodeId n : taken) {
          if (it->second.has(n)) continue;
          insert_sorted(m.kind == MoveKind::MergeConsumerGroup ? it->second.post : it->second.pre, n);
          if (m.kind == MoveKind::MergeConsumerGroup && s.exporter[n] == ht->first) s.exporter[n] = m.group;
        }
        if (m.kind == MoveKind::MergeConsumerGroup) s.groups.erase(ht);
        break;
      }
    }
    ++states;
    if (!fix(s) || !acyclic(s) || !legal(s)) return false;
    *out = std::move(s);
    return true;
  }

  double group_cost(const State& s, int id, const Group& G) const {
    if (single(G) && tier_of(G, exports(s, id, G)) == 0) return 1.0;
    double rd = 0, wr = 0;
    for (NodeId p : reads(G, nullptr)) rd += node_bytes(node(p));
    for (NodeId e : exports(s, id, G)) wr += node_bytes(node(e));
    if (G.anchor < 0) {
      double units = 0;
      bool reduces = false;
      for (NodeId n : G.post) {
        const he_node& nd = node(n);
        const he_node& src = nd.kind == HE_OP_REDUCE ? node(nd.in[0]) : nd;
        units += op_weight(nd) * (double)num_elements(src);
        reduces = reduces || nd.kind == HE_OP_REDUCE;
      }
      if (kind_of(G) == InstrKind::PermuteDims) return kLaunch + (rd + wr) / (kHbm * 0.98);
      const bool hand_written = tier_of(G, exports(s, id, G)) == 2;
      return kLaunch + std::max((rd + wr) / (kHbm * (hand_written ? 0.95 : reduces ? 0.76 : 0.84)), units * kAluOp);
    }
    const he_node& mm = node(G.anchor);
    const he_node& a = node(mm.in[0]);
    const double M = (double)mm.shape[mm.rank - 2], Nn = (double)mm.shape[mm.rank - 1];
    const double K = (double)a.shape[a.rank - 1];
    const double batch = (double)num_elements(mm) / (M * Nn);
    const double t_mma = 2.0 * M * Nn * K * batch / kTensor;
    double epi_units = 0;
    for (NodeId n : G.post) {
      const he_node& nd = node(n);
      const he_node& src = nd.kind == HE_OP_REDUCE ? node(nd.in[0]) : nd;
      epi_units += op_weight(nd) * (double)num_elements(src);
    }
    // operand side: the plan evaluates it in the mainloop or with a pre-pass, whichever it has; the model takes
    // the cheaper of the two per operand
    double t_pre = 0;
    for (int side = 0; side < 2; ++side) {
      const NodeId root = mm.in[side];
      if (!in_sorted(G.pre, root)) continue;
      std::vector<NodeId> stack{root};
      std::set<NodeId> mine{root};
      while (!stack.empty()) {
        NodeId c = stack.back();
        stack.pop_back();
        for (NodeId p : g.inbound(c))
          if (in_sorted(G.pre, p) && mine.insert(p).second) stack.push_back(p);
      }
      double units = 0, side_reads = 0;
      std::set<NodeId> ext;
      for (NodeId n : mine) {
        units += op_weight(node(n)) * (double)num_elements(node(n));
        for (NodeId p : g.inbound(n))
          if (!mine.count(p)) ext.insert(p);
      }
      for (NodeId p : ext) side_reads += node_bytes(node(p));
      const double tiles = std::ceil((side == 0 ? Nn : M) / 256.0);
      const double in_kernel = units * tiles * kMainloopOp;
      // the pre-pass is a pointwise kernel of its own in front of the GEMM, which then reads the operand copy
      const double pre_pass = 0.8 * kLaunch + (side_reads + node_bytes(node(root))) / (kHbm * 0.84);
      t_pre += std::min(in_kernel, pre_pass);
    }
    // an epilogue outside the hand-written catalogue runs as a register program: about twice the instructions
    const double epi_rate = kEpilogueOp * (tier_of(G, exports(s, id, G)) == 2 ? 1.0 : 2.0);
    return kLaunch + std::max(t_mma + epi_units * epi_rate, (rd + wr) / (kHbm * 0.8)) + t_pre;
  }

  double cost(const State& s) const {
    double c = 0;
    for (auto& kv : s.groups) c += group_cost(s, kv.first, kv.second);
    return c;
  }

  uint64_t hash(const State& s) const {
    std::vector<std::string> parts;
    for (auto& kv : s.groups) {
      std::ostringstream os;
      os << kv.second.anchor << '|';
      for (NodeId n : kv.second.pre) os << n << ',';
      os << '|';
      for (NodeId n : kv.second.post) os << n << ',';
      os << '|';
      for (NodeId n : exports(s, kv.first, kv.second)) os << n << ',';
      parts.push_back(os.str());
    }
    std::sort(parts.begin(), parts.end());
    uint64_t h = 1469598103934665603ull;
    for (const std::string& p : parts) {
      for (unsigned char ch : p) h = (h ^ ch) * 1099511628211ull;
      h = (h ^ 0xffu) * 1099511628211ull;
    }
    return h;
  }

  // Greedy start: absorb a consumer whenever that removes a kernel.
  void maximal(State& s) {
    for (bool again = true; again;) {
      again = false;
      for (const Move& m : moves(s, nullptr)) {
        if (m.kind != MoveKind::AbsorbConsumer && m.kind != MoveKind::MergeConsumerGroup) continue;
        State t;
        if (apply(s, m, &t) && t.groups.size() < s.groups.size()) {
          s = std::move(t);
          again = true;
          break;
        }
      }
    }
  }

  struct Best {
    State state;
    double cost;
    bool improved = false;
  };

  void look_ahead(const State& cur, int depth, int max_depth, const std::vector<char>* allowed,
                  std::unordered_set<uint64_t>& visited, Best& best, int budget_end) {
    if (depth == max_depth || states >= budget_end) return;
    std::vector<std::pair<double, State>> next;
    for (const Move& m : moves(cur, allowed)) {
      if (states >= budget_end) break;
      State t;
      if (!apply(cur, m, &t)) continue;
      if (!visited.insert(hash(t)).second) continue;
      const double c = cost(t);
      next.emplace_back(c, std::move(t));
    }
    std::stable_sort(next.begin(), next.end(), [](const auto& x, const auto& y) { return x.first < y.first; });
    if ((int)next.size() > opt.beam) next.resize(opt.beam);
    for (auto& cs : next) {
      if (cs.first < best.cost * (1.0 - 1e-9)) {
        best.state = cs.second;
        best.cost = cs.first;
        best.improved = true;
      }
      look_ahead(cs.second, depth + 1, max_depth, allowed, visited, best, budget_end);
    }
  }

  void descend(Best& best, const std::vector<char>* allowed) {
    const int budget_end = states + opt.max_states;
    // steepest descent one move at a time while that helps; the deeper look-ahead only where it is stuck
    for (int max_depth = 1; states < budget_end;) {
      best.improved = false;
      std::unordered_set<uint64_t> visited;
      visited.insert(hash(best.state));
      const State from = best.state;
      look_ahead(from, 0, max_depth, allowed, visited, best, budget_end);
      if (best.improved) {
        max_depth = 1;
      } else if (max_depth < opt.depth) {
        max_depth = opt.depth;
      } else {
        break;
      }
    }
  }
};

}  // namespace

std::vector<Subdivision> subdivide(const OpGraph& g) {
  const int N = (int)g.nodes.size();
  // vertex 2n: operand side of n (or all of n when n is no matmul); vertex 2n+1: result side of a matmul
  std::vector<int> parent(2 * N);
  std::iota(parent.begin(), parent.end(), 0);
  std::function<int(int)> find = [&](int x) { return parent[x] == x ? x : parent[x] = find(parent[x]); };
  auto anchor = [&](NodeId n) { return g.nodes[n].kind == HE_OP_MATMUL; };
  auto input = [&](NodeId n) { return g.nodes[n].kind == HE_OP_INPUT; };
  for (NodeId v = 0; v < N; ++v) {
    if (input(v)) continue;
    for (NodeId u : g.inbound(v)) {
      if (input(u)) continue;
      parent[find(anchor(u) ? 2 * u + 1 : 2 * u)] = find(2 * v);
    }
  }
  std::map<int, Subdivision> comps;
  for (NodeId n = 0; n < N; ++n) {
    if (input(n)) continue;
    if (anchor(n)) {
      comps[find(2 * n)].push_back({n, Portion::OperandSide});
      comps[find(2 * n + 1)].push_back({n, Portion::ResultSide});
    } else {
      comps[find(2 * n)].push_back({n, Portion::Whole});
    }
  }
  std::vector<Subdivision> out;
  for (auto& kv : comps) {
    std::sort(kv.second.begin(), kv.second.end());
    out.push_back(kv.second);
  }
  std::sort(out.begin(), out.end());
  return out;
}

SearchResult search_fusions(const OpGraph& g, he_ctx* ctx, const SearchOptions& opt, const std::vector<Instr>* seed) {
  SearchResult r;
  Searcher S(g, ctx, opt);
  State s = S.identity();
  if (!S.fix(s) || !S.acyclic(s)) {
    r.error = "the graph has no consistent one-kernel-per-node state";
    return r;
  }
  r.cost_identity = S.cost(s);
  const State singletons = s;
  S.maximal(s);
  r.cost_maximal = S.cost(s);
  // Moves only grow groups, so a descent cannot undo a merge of the greedy start.  It therefore runs twice, from
  // the greedy start and from the singletons, and the cheaper end state wins.
  const std::vector<Subdivision> subs = subdivide(g);
  r.subdivisions = opt.use_subdivision ? (int)subs.size() : 1;
  auto descend_all = [&](Searcher::Best& b) {
    if (!opt.use_subdivision) {
      S.descend(b, nullptr);
      return;
    }
    for (const Subdivision& sub : subs) {
      std::vector<char> allowed(S.N, 0);
      bool any = false;
      for (auto& np : sub)
        if (np.second == Portion::Whole && S.live[np.first]) {
          allowed[np.first] = 1;
          any = true;
        }
      if (any) S.descend(b, &allowed);
    }
  };
  Searcher::Best best{s, r.cost_maximal, false};
  descend_all(best);
  Searcher::Best from_singletons{singletons, r.cost_identity, false};
  descend_all(from_singletons);
  if (from_singletons.cost < best.cost) best = from_singletons;
  if (seed) {
    // the other planner's instructions as a state: operand side = the matmul's ancestors inside the instruction
    State t;
    t.exporter.assign(S.N, -1);
    bool usable = true;
    for (const Instr& in : *seed) {
      Group G;
      for (NodeId n : in.sub.nodes)
        if (S.is_anchor(n)) {
          usable = usable && G.anchor < 0;
          G.anchor = n;
        }
      std::set<NodeId> pre;
      if (G.anchor >= 0) {
        std::vector<NodeId> stack{G.anchor};
        while (!stack.empty()) {
          NodeId c = stack.back();
          stack.pop_back();
          for (NodeId p : g.inbound(c))
            if (in.sub.contains(p) && pre.insert(p).second) stack.push_back(p);
        }
      }
      for (NodeId n : in.sub.nodes) {
        if (n == G.anchor) continue;
        if (pre.count(n)) G.pre.push_back(n);
        else G.post.push_back(n);
      }
      const int id = t.next_id++;
      for (NodeId o : in.sub.leafs) {
        usable = usable && G.exportable(o) && t.exporter[o] < 0;
        t.exporter[o] = id;
      }
      t.groups.emplace(id, std::move(G));
    }
    if (usable && S.fix(t) && S.acyclic(t) && S.legal(t)) {
      r.cost_seed = S.cost(t);
      Searcher::Best from_seed{t, r.cost_seed, false};
      descend_all(from_seed);
      if (from_seed.cost < best.cost) best = from_seed;
    }
  }
  r.cost_best = best.cost;
  r.states = S.states;
  std::vector<int> order;
  if (!S.acyclic(best.state, &order)) {
    r.error = "internal: the best state is cyclic";
    return r;
  }
  std::vector<int> count(S.N, 0);
  for (int id : order) {
    const Group& G = best.state.groups.at(id);
    SearchGroup sg;
    sg.anchor = G.anchor;
    sg.pre = G.pre;
    sg.post = G.post;
    sg.reads = S.reads(G, nullptr);
    sg.exports = S.exports(best.state, id, G);
    sg.seconds = S.group_cost(best.state, id, G);
    for (NodeId n : G.all()) ++count[n];
    r.groups.push_back(std::move(sg));
  }
  for (NodeId n = 0; n < S.N; ++n) {
    if (count[n] > 1) ++r.recomputed_nodes;
    if (S.live[n] && g.nodes[n].kind != HE_OP_INPUT && count[n] == 0) {
      r.error = "internal: a live node is in no group";
      return r;
    }
  }
  r.valid = true;
  return r;
}

std::vector<Instr> instrs_from_search(const OpGraph& g, const SearchResult& r) {
  std::vector<Instr> out;
  for (const SearchGroup& sg : r.groups) {
    std::vector<NodeId> all = sg.pre;
    all.insert(all.end(), sg.post.begin(), sg.post.end());
    if (sg.anchor >= 0) all.push_back(sg.anchor);
    OpSubgraph sub = OpSubgraph::from_nodes_with_leafs(&g, all, sg.exports);
    InstrKind k = InstrKind::PointwiseGraph;
    if (sg.anchor >= 0) {
      k = InstrKind::FusedMatmul;
    } else {
      bool all_swaps = true;
      for (NodeId n : sg.post) all_swaps = all_swaps && g.nodes[n].kind == HE_OP_SWAP_DIMS;
      const he_node& last = g.nodes[sg.post.back()];
      if (all_swaps && num_elements(last) > 1000000 && last.dtype != HE_BOOL) {
        OpSubgraph::Flat f = sub.flatten();
        he_graph_desc d = f.desc();
        if (he_plan_supported(nullptr, &d, (int)InstrKind::PermuteDims) > 0) k = InstrKind::PermuteDims;
      }
    }
    out.push_back(Instr{k, std::move(sub)});
  }
  return out;
}

}  // namespace host
}  // namespace he
