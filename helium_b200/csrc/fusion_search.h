// Fusion search over an op graph: which nodes go into which kernel, on which side of a matmul (operand side =
// mainloop, result side = epilogue), and which nodes are recomputed in several kernels instead of being written
// to memory once.  The counterpart of the playground's search (helium-playground/src/fused_graph.rs:113-223,
// 285-593 states and moves; subdivision.rs:24-113 problem-size reduction; cost_model.rs:90-343 cost functions and
// the depth-limited descent), rebuilt around this library's kernels: a state is legal only if he_plan_supported
// accepts every group, and the cost model is fitted to measurements of these kernels on a B200.
#pragma once
#include <string>
#include <utility>
#include <vector>

#include "host_graph.h"

namespace he {
namespace host {

// Side of a matmul node a subdivision holds (subdivision.rs:9-14); every other node is held whole.
enum class Portion : int { OperandSide = 0, ResultSide = 1, Whole = 2 };
using Subdivision = std::vector<std::pair<NodeId, Portion>>;   // sorted

// Weakly connected components of the graph in which every matmul is split into an operand-side vertex and a
// result-side vertex and graph inputs are left out: fusions never cross from one component to another, so each is
// searched on its own.
std::vector<Subdivision> subdivide(const OpGraph& g);

struct SearchOptions {
  int depth = 3;           // moves looked ahead where single moves no longer help (the playground looks 7 ahead, exhaustively)
  int beam = 6;            // cheapest moves followed at each level of the look-ahead
  int max_states = 12000;  // states costed per subdivision and descent; the search keeps the best found when it runs out
  bool use_subdivision = true;
};

struct SearchGroup {        // one kernel of the result
  NodeId anchor = -1;       // matmul node, or -1 for a pointwise kernel
  std::vector<NodeId> pre;  // operand-side nodes (evaluated in the mainloop or by the plan's pre-pass)
  std::vector<NodeId> post; // result-side nodes, or all nodes of a pointwise kernel
  std::vector<NodeId> reads, exports;
  double seconds = 0;       // cost model's estimate
};

struct SearchResult {
  std::vector<SearchGroup> groups;   // in a topological order
  double cost_identity = 0, cost_maximal = 0, cost_best = 0;
  double cost_seed = -1;             // estimate for the seed plan (the pairwise planner's), -1 if none was usable
  int states = 0, subdivisions = 0, recomputed_nodes = 0;
  bool valid = false;
  std::string error;
};

// `seed`: instructions of another planner for the same graph (each node in exactly one of them).  When they form a
// state of the search (no operand-side node of a matmul is written to memory) a third descent starts there, so the
// result is never dearer, by the cost model, than the seed plan.
SearchResult search_fusions(const OpGraph& g, he_ctx* ctx, const SearchOptions& opt, const std::vector<Instr>* seed = nullptr);

// Instructions for generate_plan from a search result.
std::vector<Instr> instrs_from_search(const OpGraph& g, const SearchResult& r);

}  // namespace host
}  // namespace he
