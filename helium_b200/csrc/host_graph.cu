// Host runtime above the C ABI: op graph, instruction selection, fusion, plan generation and a
// multi-stream / CUDA-graph executor.
//
// This restates, in C++, the parts of helium that sit between a recorded op graph and the kernel
// calls (the reference's are Rust):
//   OpGraph / OpSubgraph          helium-ir/src/opgraph.rs:12-191, helium-ir/src/opgraph/subgraph.rs:12-120
//   make_instr_for_op             helium/src/cuda.rs:33-60
//   Instr::{can_fuse_with,fuse_with}   helium/src/cuda/instr.rs:54-99
//   InstrGraph, do_fusions, generate_plan_from_graph, delay_computations, analyze_tensor_lifetimes
//                                 helium/src/backend/plan_generation.rs:86-446
//   execute_graph / CudaExecutor  helium/src/backend.rs:40-80, helium/src/cuda.rs:98-230
// Differences, all deliberate: Op::Matmul becomes a FusedMatmul instruction whose can_fuse_with is
// answered by he_plan_supported (the reference's cuDNN instruction refuses every fusion,
// cudnn_graph.rs:319-321); a PermuteDims and a PointwiseGraph may merge when the merged subgraph has
// a single-pass kernel; instructions of one step are spread over several streams; the whole plan
// can be captured into a CUDA graph.
#include <algorithm>
#include <map>
#include <memory>
#include <set>
#include <sstream>

#include "he_internal.h"

#include "host_graph.h"
#include "fusion_search.h"

namespace he {
namespace host {

// ---- InstrGraph (plan_generation.rs:86-249) -------------------------------------------------------
struct InstrGraph {
  std::map<int, Instr> instrs;
  int next_id = 0;
  std::map<NodeId, int> producers;
  std::map<NodeId, std::set<int>> consumers;

  int insert(Instr in) {
    const int id = next_id++;
    for (NodeId i : in.inputs()) consumers[i].insert(id);
    for (NodeId o : in.outputs()) producers[o] = id;
    instrs.emplace(id, std::move(in));
    return id;
  }
  Instr remove(int id) {
    Instr in = instrs.at(id);
    for (NodeId i : in.inputs()) consumers[i].erase(id);
    for (NodeId o : in.outputs()) producers.erase(o);
    instrs.erase(id);
    return in;
  }
  std::set<int> dependents(int id) const {
    std::set<int> r;
    for (NodeId o : instrs.at(id).outputs()) {
      auto it = consumers.find(o);
      if (it != consumers.end()) r.insert(it->second.begin(), it->second.end());
    }
    return r;
  }
  std::set<int> dependencies(int id) const {
    std::set<int> r;
    for (NodeId i : instrs.at(id).inputs()) {
      auto it = producers.find(i);
      if (it != producers.end()) r.insert(it->second);
    }
    return r;
  }
  // plan_generation.rs:198-216: a second path a -> .. -> b would make the merged node cyclic
  bool exist_multiple_paths(int a, int b) const {
    std::vector<int> stack;
    std::set<int> visited;
    for (int d : dependents(a))
      if (d != b) {
        stack.push_back(d);
        visited.insert(d);
      }
    while (!stack.empty()) {
      int cur = stack.back();
      stack.pop_back();
      if (cur == b) return true;
      for (int nx : dependents(cur))
        if (visited.insert(nx).second) stack.push_back(nx);
    }
    return false;
  }
};

struct Step {
  std::vector<Instr> instrs;
  std::vector<NodeId> tensors_to_release;
};
struct Plan {
  std::vector<Step> steps;
};

static bool has_intersection(const std::vector<NodeId>& a, const std::vector<NodeId>& b) {
  for (NodeId x : a)
    if (std::find(b.begin(), b.end(), x) != b.end()) return true;
  return false;
}

// How instructions are formed from nodes: the reference's greedy pairwise merging, or the fusion search.
struct PlannerChoice {
  int mode = 0;   // 0 pairwise (plan_generation.rs:243-256), 1 search (fusion_search.h)
  SearchOptions search;
};

// The reference's instruction selection: one instruction per live node, merged pairwise and greedily.
static InstrGraph pairwise_instr_graph(const OpGraph& g, he_ctx* ctx) {
  InstrGraph ig;
  // make_instr_graph (plan_generation.rs:259-270), dead nodes pruned first (backend.rs:46)
  const std::vector<bool> live = g.live();
  for (NodeId id = 0; id < (NodeId)g.nodes.size(); ++id)
    if (g.nodes[id].kind != HE_OP_INPUT && live[id]) ig.insert(make_instr_for_op(&g, id));

  // do_fusions (plan_generation.rs:243-256)
  std::set<int> working;
  for (auto& kv : ig.instrs) working.insert(kv.first);
  while (!working.empty()) {
    const int current = *working.begin();
    working.erase(working.begin());
    for (int next : ig.dependents(current)) {
      if (ig.instrs.at(current).can_fuse_with(ig.instrs.at(next), ctx) && !ig.exist_multiple_paths(current, next)) {
        Instr a = ig.remove(current), b = ig.remove(next);
        const int nid = ig.insert(a.fuse_with(b));
        working.erase(next);
        working.insert(nid);
        break;
      }
    }
  }
  return ig;
}

// The fusion search, seeded with the pairwise plan so that its result is never dearer than that plan by the model.
static SearchResult run_search(const OpGraph& g, he_ctx* ctx, const SearchOptions& opt) {
  std::vector<Instr> seed;
  for (auto& kv : pairwise_instr_graph(g, ctx).instrs) seed.push_back(kv.second);
  return search_fusions(g, ctx, opt, &seed);
}

static Plan generate_plan(const OpGraph& g, he_ctx* ctx, const PlannerChoice& choice, std::string* error) {
  InstrGraph ig;
  if (choice.mode == 1) {
    // every instruction comes out of the search with its outputs chosen: a node that several instructions
    // recompute is written to memory by one of them only
    SearchResult r = run_search(g, ctx, choice.search);
    if (!r.valid) {
      if (error) *error = r.error;
      return Plan{};
    }
    for (Instr& in : instrs_from_search(g, r)) ig.insert(std::move(in));
  } else {
    ig = pairwise_instr_graph(g, ctx);
  }

  // generate_plan_from_graph (plan_generation.rs:275-321): Kahn layers
  std::map<int, int> indegree;
  std::vector<int> stack;
  for (auto& kv : ig.instrs) {
    indegree[kv.first] = (int)ig.dependencies(kv.first).size();
    if (indegree[kv.first] == 0) stack.push_back(kv.first);
  }
  Plan plan;
  std::vector<std::vector<int>> layers;
  while (!stack.empty()) {
    std::vector<int> step;
    step.swap(stack);
    for (int id : step)
      for (int nx : ig.dependents(id))
        if (--indegree[nx] == 0) stack.push_back(nx);
    layers.push_back(step);
  }
  for (auto& layer : layers) {
    Step s;
    for (int id : layer) s.instrs.push_back(ig.instrs.at(id));
    plan.steps.push_back(std::move(s));
  }

  // delay_computations (plan_generation.rs:325-353)
  for (int i = (int)plan.steps.size() - 1; i >= 0; --i) {
    std::vector<Instr> keep;
    std::vector<Instr> instrs;
    instrs.swap(plan.steps[i].instrs);
    for (Instr& in : instrs) {
      int target = -1;
      for (int j = i + 1; j < (int)plan.steps.size(); ++j) {
        bool used = false;
        for (const Instr& in2 : plan.steps[j].instrs) used = used || has_intersection(in2.inputs(), in.outputs());
        if (used) {
          target = j - 1;
          break;
        }
      }
      if (target >= 0 && target != i) plan.steps[target].instrs.push_back(in);
      else keep.push_back(in);
    }
    plan.steps[i].instrs = keep;
  }

  // analyze_tensor_lifetimes (plan_generation.rs:360-416)
  std::vector<std::vector<NodeId>> release(1);
  for (size_t i = 0; i < plan.steps.size(); ++i) {
    std::set<NodeId> used;
    for (const Instr& in : plan.steps[i].instrs) used.insert(in.inputs().begin(), in.inputs().end());
    std::vector<NodeId> rel;
    for (NodeId t : used) {
      if (g.is_output(t)) continue;
      bool later = false;
      for (size_t j = i + 1; j < plan.steps.size() && !later; ++j)
        for (const Instr& in : plan.steps[j].instrs)
          if (std::find(in.inputs().begin(), in.inputs().end(), t) != in.inputs().end()) later = true;
      if (!later) rel.push_back(t);
    }
    release.push_back(rel);
  }
  plan.steps.emplace_back();
  for (size_t i = 0; i < plan.steps.size(); ++i) plan.steps[i].tensors_to_release = release[i];
  return plan;
}

}  // namespace host
}  // namespace he

using namespace he;
using namespace he::host;

struct heh_graph {
  OpGraph g;
  PlannerChoice planner;
};

// One prepared evaluation of a graph with fixed buffers.
struct heh_exec {
  he_ctx* ctx = nullptr;
  Plan plan;
  struct Bound {
    he_plan* plan = nullptr;
    std::vector<const void*> ins;
    std::vector<void*> outs;
    void* workspace = nullptr;
    int step = 0;
  };
  std::vector<Bound> launches;
  std::vector<void*> owned;        // intermediates and workspaces
  std::vector<cudaStream_t> streams;
  std::vector<cudaEvent_t> events; // one per worker stream + fork
  cudaEvent_t fork_event = nullptr;
  cudaGraphExec_t graph_exec = nullptr;
  int n_steps = 0, n_instrs = 0, n_launches = 0;

  ~heh_exec() {
    for (Bound& b : launches) he_plan_destroy(b.plan);
    for (void* p : owned) cudaFree(p);
    if (graph_exec) cudaGraphExecDestroy(graph_exec);
    for (cudaEvent_t e : events) cudaEventDestroy(e);
    if (fork_event) cudaEventDestroy(fork_event);
    for (cudaStream_t s : streams) cudaStreamDestroy(s);
  }

  // Issues every launch: instructions of a step round-robin over the worker streams, a step starts
  // only when the previous one has finished on all of them (plan_generation.rs:52-58).
  int32_t issue(cudaStream_t main) {
    const int ns = (int)streams.size();
    n_launches = 0;
    HE_CUDA(cudaEventRecord(fork_event, main));
    for (int s = 0; s < ns; ++s) HE_CUDA(cudaStreamWaitEvent(streams[s], fork_event, 0));
    int cur_step = -1, slot = 0;
    std::vector<bool> used(ns, false);
    auto join_step = [&]() -> int32_t {
      // every stream that worked in this step is joined by all others
      for (int s = 0; s < ns; ++s)
        if (used[s]) HE_CUDA(cudaEventRecord(events[s], streams[s]));
      for (int s = 0; s < ns; ++s)
        for (int t = 0; t < ns; ++t)
          if (used[t] && t != s) HE_CUDA(cudaStreamWaitEvent(streams[s], events[t], 0));
      std::fill(used.begin(), used.end(), false);
      return HE_OK;
    };
    for (Bound& b : launches) {
      if (b.step != cur_step) {
        if (cur_step >= 0) HE_TRY(join_step());
        cur_step = b.step;
        slot = 0;
      }
      const int s = slot++ % ns;
      used[s] = true;
      HE_TRY(he_launch(b.plan, b.ins.data(), b.outs.data(), b.workspace, streams[s]));
      n_launches += he_plan_last_launch_count(b.plan);
    }
    HE_TRY(join_step());
    // join back into the caller's stream
    for (int s = 0; s < ns; ++s) {
      HE_CUDA(cudaEventRecord(events[s], streams[s]));
      HE_CUDA(cudaStreamWaitEvent(main, events[s], 0));
    }
    return HE_OK;
  }
};

extern "C" {

int32_t heh_graph_create(heh_graph** out) {
  if (!out) HE_FAIL(HE_ERR_INVALID, "heh_graph_create: null argument");
  *out = new heh_graph();
  // HE_PLANNER=search makes the fusion search the default planner of new graphs (heh_graph_set_planner overrides)
  const char* env = getenv("HE_PLANNER");
  if (env && strcmp(env, "search") == 0) (*out)->planner.mode = 1;
  return HE_OK;
}
void heh_graph_destroy(heh_graph* g) { delete g; }

int32_t heh_graph_new_input(heh_graph* g, int32_t dtype, int32_t rank, const int64_t* shape, int32_t* node_out) {
  if (!g || !node_out || (rank > 0 && !shape)) HE_FAIL(HE_ERR_INVALID, "heh_graph_new_input: null argument");
  if (rank < 0 || rank > HE_MAX_RANK || !dtype_valid(dtype)) HE_FAIL(HE_ERR_INVALID, "heh_graph_new_input: bad descriptor");
  he_node n{};
  n.kind = HE_OP_INPUT;
  n.dtype = dtype;
  n.rank = rank;
  for (int i = 0; i < rank; ++i) n.shape[i] = shape[i];
  n.in[0] = n.in[1] = n.in[2] = -1;
  *node_out = g->g.add(n);
  return HE_OK;
}

int32_t heh_graph_new_op(heh_graph* g, const he_node* op, int32_t* node_out) {
  if (!g || !op || !node_out) HE_FAIL(HE_ERR_INVALID, "heh_graph_new_op: null argument");
  if (op->kind == HE_OP_INPUT) HE_FAIL(HE_ERR_INVALID, "heh_graph_new_op: use heh_graph_new_input for inputs");
  // validate the new node against its operands with the same rules the kernels' planner uses
  std::vector<he_node> tmp = g->g.nodes;
  tmp.push_back(*op);
  int32_t last = (int32_t)tmp.size() - 1;
  he_graph_desc d{(int32_t)tmp.size(), tmp.data(), 1, &last};
  Graph parsed;
  HE_TRY(parse_graph(&d, &parsed));
  *node_out = g->g.add(parsed.nodes.back());
  return HE_OK;
}

int32_t heh_graph_new_output(heh_graph* g, int32_t node) {
  if (!g || node < 0 || node >= (int32_t)g->g.nodes.size()) HE_FAIL(HE_ERR_INVALID, "heh_graph_new_output: bad node");
  g->g.outputs.push_back(node);
  g->g.live_mask.clear();
  return HE_OK;
}

int32_t heh_graph_plan_text(he_ctx* ctx, heh_graph* g, char* buf, size_t cap) {
  if (!g || !buf) HE_FAIL(HE_ERR_INVALID, "heh_graph_plan_text: null argument");
  if (g->g.outputs.empty()) HE_FAIL(HE_ERR_INVALID, "graph has no outputs");
  std::string plan_error;
  g->g.live_mask = g->g.live();
  Plan plan = generate_plan(g->g, ctx, g->planner, &plan_error);
  if (!plan_error.empty()) HE_FAIL(HE_ERR_UNSUPPORTED, "fusion search: %s", plan_error.c_str());
  std::ostringstream os;
  for (size_t i = 0; i < plan.steps.size(); ++i) {
    for (const Instr& in : plan.steps[i].instrs) {
      os << "step " << i << " " << kind_name(in.kind) << " tier=" << in.tier(ctx) << " nodes=[";
      for (size_t k = 0; k < in.sub.nodes.size(); ++k) os << (k ? "," : "") << in.sub.nodes[k];
      os << "] in=[";
      for (size_t k = 0; k < in.inputs().size(); ++k) os << (k ? "," : "") << in.inputs()[k];
      os << "] out=[";
      for (size_t k = 0; k < in.outputs().size(); ++k) os << (k ? "," : "") << in.outputs()[k];
      os << "]\n";
    }
    if (!plan.steps[i].tensors_to_release.empty()) {
      os << "step " << i << " release=[";
      for (size_t k = 0; k < plan.steps[i].tensors_to_release.size(); ++k) os << (k ? "," : "") << plan.steps[i].tensors_to_release[k];
      os << "]\n";
    }
  }
  const std::string s = os.str();
  if (s.size() + 1 > cap) HE_FAIL(HE_ERR_INVALID, "heh_graph_plan_text: buffer too small (need %zu)", s.size() + 1);
  memcpy(buf, s.c_str(), s.size() + 1);
  return HE_OK;
}

int32_t heh_graph_set_planner(heh_graph* g, int32_t mode, int32_t depth, int32_t max_states) {
  if (!g) HE_FAIL(HE_ERR_INVALID, "heh_graph_set_planner: null argument");
  if (mode != 0 && mode != 1) HE_FAIL(HE_ERR_INVALID, "heh_graph_set_planner: mode %d (0 pairwise, 1 search)", mode);
  if (depth < 0 || depth > 12 || max_states < 0) HE_FAIL(HE_ERR_INVALID, "heh_graph_set_planner: depth %d, max_states %d", depth, max_states);
  g->planner.mode = mode;
  if (depth > 0) g->planner.search.depth = depth;
  if (max_states > 0) g->planner.search.max_states = max_states;
  return HE_OK;
}

static void print_nodes(std::ostringstream& os, const char* name, const std::vector<NodeId>& v) {
  os << ' ' << name << "=[";
  for (size_t k = 0; k < v.size(); ++k) os << (k ? "," : "") << v[k];
  os << ']';
}

int32_t heh_graph_search_text(he_ctx* ctx, heh_graph* g, char* buf, size_t cap) {
  if (!g || !buf) HE_FAIL(HE_ERR_INVALID, "heh_graph_search_text: null argument");
  if (g->g.outputs.empty()) HE_FAIL(HE_ERR_INVALID, "graph has no outputs");
  g->g.live_mask = g->g.live();
  SearchResult r = run_search(g->g, ctx, g->planner.search);
  if (!r.valid) HE_FAIL(HE_ERR_UNSUPPORTED, "fusion search: %s", r.error.c_str());
  std::ostringstream os;
  os.precision(9);
  os << "cost identity=" << r.cost_identity << " maximal=" << r.cost_maximal << " pairwise=" << r.cost_seed << " best=" << r.cost_best
     << " states=" << r.states
     << " subdivisions=" << r.subdivisions << " recomputed=" << r.recomputed_nodes << "\n";
  for (size_t i = 0; i < r.groups.size(); ++i) {
    const SearchGroup& sg = r.groups[i];
    os << "group " << i << (sg.anchor >= 0 ? " FusedMatmul" : " Pointwise") << " anchor=" << sg.anchor;
    print_nodes(os, "pre", sg.pre);
    print_nodes(os, "post", sg.post);
    print_nodes(os, "in", sg.reads);
    print_nodes(os, "out", sg.exports);
    os << " seconds=" << sg.seconds << "\n";
  }
  const std::string s = os.str();
  if (s.size() + 1 > cap) HE_FAIL(HE_ERR_INVALID, "heh_graph_search_text: buffer too small (need %zu)", s.size() + 1);
  memcpy(buf, s.c_str(), s.size() + 1);
  return HE_OK;
}

int32_t heh_graph_subdivisions_text(heh_graph* g, char* buf, size_t cap) {
  if (!g || !buf) HE_FAIL(HE_ERR_INVALID, "heh_graph_subdivisions_text: null argument");
  std::ostringstream os;
  for (const Subdivision& sub : subdivide(g->g)) {
    for (size_t k = 0; k < sub.size(); ++k)
      os << (k ? " " : "") << sub[k].first << (sub[k].second == Portion::OperandSide ? "m" : sub[k].second == Portion::ResultSide ? "e" : "");
    os << "\n";
  }
  const std::string s = os.str();
  if (s.size() + 1 > cap) HE_FAIL(HE_ERR_INVALID, "heh_graph_subdivisions_text: buffer too small (need %zu)", s.size() + 1);
  memcpy(buf, s.c_str(), s.size() + 1);
  return HE_OK;
}

int32_t heh_exec_create(he_ctx* ctx, heh_graph* g, const void* const* inputs, void* const* outputs,
                        int32_t capture_cuda_graph, heh_exec** out) {
  if (!ctx || !g || !out) HE_FAIL(HE_ERR_INVALID, "heh_exec_create: null argument");
  *out = nullptr;
  const OpGraph& G = g->g;
  if (G.outputs.empty()) HE_FAIL(HE_ERR_INVALID, "graph has no outputs");
  std::unique_ptr<heh_exec> e(new heh_exec());
  e->ctx = ctx;
  std::string plan_error;
  g->g.live_mask = g->g.live();
  e->plan = generate_plan(G, ctx, g->planner, &plan_error);
  if (!plan_error.empty()) HE_FAIL(HE_ERR_UNSUPPORTED, "fusion search: %s", plan_error.c_str());
  DeviceGuard device_guard(ctx->device);   // the caller's current device is restored on return
  HE_TRY(device_guard.status());

  // tensor table: caller buffers for inputs / outputs, owned buffers for the rest
  std::map<NodeId, void*> tensors;
  for (size_t i = 0; i < G.inputs.size(); ++i) {
    if (!inputs || !inputs[i]) HE_FAIL(HE_ERR_INVALID, "heh_exec_create: input %zu is null", i);
    tensors[G.inputs[i]] = const_cast<void*>(inputs[i]);
  }
  for (size_t j = 0; j < G.outputs.size(); ++j) {
    if (!outputs || !outputs[j]) HE_FAIL(HE_ERR_INVALID, "heh_exec_create: output %zu is null", j);
    if (G.nodes[G.outputs[j]].kind == HE_OP_INPUT) HE_FAIL(HE_ERR_UNSUPPORTED, "an input marked as output needs no execution");
    // one node bound to two caller buffers would need a device copy appended to the plan
    if (tensors.count(G.outputs[j]))
      HE_FAIL(HE_ERR_UNSUPPORTED, "heh_exec_create: node %d is listed as an output more than once (output %zu)", (int)G.outputs[j], j);
    tensors[G.outputs[j]] = outputs[j];
  }
  int step_idx = 0;
  for (const Step& st : e->plan.steps) {
    for (const Instr& in : st.instrs) {
      ++e->n_instrs;
      // owned by the executor from here on, so that every error return below releases the plan
      e->launches.emplace_back();
      heh_exec::Bound& b = e->launches.back();
      b.step = step_idx;
      OpSubgraph::Flat f = in.sub.flatten();
      he_graph_desc d = f.desc();
      int32_t rc;
      if (in.kind == InstrKind::PermuteDims) {
        // swap chain -> strides (permute_dims.rs:112-172, semantic form)
        std::vector<int32_t> swaps;
        for (NodeId n : in.sub.nodes) {
          swaps.push_back(G.nodes[n].axis_a);
          swaps.push_back(G.nodes[n].axis_b);
        }
        const he_node& src = G.nodes[in.inputs()[0]];
        int64_t strides[HE_MAX_RANK];
        HE_TRY(he_permute_output_strides(src.rank, src.shape, (int32_t)swaps.size() / 2, swaps.data(), 0, strides));
        rc = he_plan_permute(ctx, src.rank, src.shape, strides, src.dtype, &b.plan);
      } else if (in.kind == InstrKind::FusedMatmul) {
        rc = he_plan_fused_matmul(ctx, &d, &b.plan);
      } else {
        rc = he_plan_pointwise(ctx, &d, &b.plan);
      }
      if (rc != HE_OK) return rc;
      for (NodeId o : in.outputs()) {
        if (!tensors.count(o)) {
          void* p = nullptr;
          const he_node& n = G.nodes[o];
          HE_CUDA(cudaMalloc(&p, std::max<size_t>(256, storage_bytes(n.dtype, num_elements(n)))));
          e->owned.push_back(p);
          tensors[o] = p;
        }
      }
      for (NodeId i : in.inputs()) {
        if (!tensors.count(i)) HE_FAIL(HE_ERR_INVALID, "plan order error: tensor %d used before it is produced", i);
        b.ins.push_back(tensors[i]);
      }
      for (NodeId o : in.outputs()) b.outs.push_back(tensors[o]);
      size_t ws = 0;
      HE_TRY(he_plan_workspace_bytes(b.plan, &ws));
      if (ws) {
        HE_CUDA(cudaMalloc(&b.workspace, ws));
        e->owned.push_back(b.workspace);
      }
    }
    ++step_idx;
  }
  e->n_steps = step_idx;
  // an output that is also consumed internally was bound to the caller's buffer above
  size_t widest = 1;
  for (const Step& st : e->plan.steps) widest = std::max(widest, st.instrs.size());
  const int ns = (int)std::min<size_t>(4, widest);
  for (int s = 0; s < ns; ++s) {
    cudaStream_t st;
    HE_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    e->streams.push_back(st);
    cudaEvent_t ev;
    HE_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    e->events.push_back(ev);
  }
  HE_CUDA(cudaEventCreateWithFlags(&e->fork_event, cudaEventDisableTiming));

  if (capture_cuda_graph) {
    // One eager pass first: lazy one-time initialisation (module loading, function attributes,
    // driver entry points) must not happen inside a capture.  The pass writes to scratch copies
    // of the caller's output buffers, never to the buffers themselves: an output may alias live
    // state (a weight updated in place), and creating an executor must not advance it.
    cudaStream_t cap;
    HE_CUDA(cudaStreamCreateWithFlags(&cap, cudaStreamNonBlocking));
    std::vector<void*> scratch(G.outputs.size(), nullptr);
    auto free_scratch = [&]() {
      for (void* p : scratch)
        if (p) cudaFree(p);
    };
    int32_t rc = HE_OK;
    for (size_t j = 0; j < G.outputs.size() && rc == HE_OK; ++j) {
      const he_node& n = G.nodes[G.outputs[j]];
      if (cudaMalloc(&scratch[j], std::max<size_t>(256, storage_bytes(n.dtype, num_elements(n)))) != cudaSuccess) {
        cudaGetLastError();
        set_error("heh_exec_create: no memory for the warm-up copies of the outputs");
        rc = HE_ERR_CUDA;
      }
    }
    auto swap_outputs = [&](bool to_scratch) {
      for (heh_exec::Bound& b : e->launches)
        for (void*& o : b.outs)
          for (size_t j = 0; j < G.outputs.size(); ++j)
            if (o == (to_scratch ? outputs[j] : scratch[j])) { o = to_scratch ? scratch[j] : outputs[j]; break; }
    };
    if (rc == HE_OK) {
      swap_outputs(true);
      rc = e->issue(cap);
      if (rc == HE_OK && cudaStreamSynchronize(cap) != cudaSuccess) rc = HE_ERR_CUDA;
      swap_outputs(false);
    }
    free_scratch();
    if (rc != HE_OK) {
      cudaStreamDestroy(cap);
      return rc;
    }
    cudaGraph_t graph = nullptr;
    HE_CUDA(cudaStreamBeginCapture(cap, cudaStreamCaptureModeThreadLocal));
    rc = e->issue(cap);
    cudaError_t ce = cudaStreamEndCapture(cap, &graph);
    if (rc != HE_OK || ce != cudaSuccess) {
      if (graph) cudaGraphDestroy(graph);
      cudaStreamDestroy(cap);
      if (rc != HE_OK) return rc;
      HE_FAIL(HE_ERR_CUDA, "cudaStreamEndCapture failed: %s", cudaGetErrorString(ce));
    }
    ce = cudaGraphInstantiate(&e->graph_exec, graph, 0);
    cudaGraphDestroy(graph);
    cudaStreamDestroy(cap);
    if (ce != cudaSuccess) HE_FAIL(HE_ERR_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(ce));
  }
  *out = e.release();
  return HE_OK;
}

int32_t heh_exec_run(heh_exec* e, void* cu_stream) {
  if (!e) HE_FAIL(HE_ERR_INVALID, "heh_exec_run: null argument");
  TraceRange range("heh_exec_run");
  if (e->graph_exec) {
    HE_CUDA(cudaGraphLaunch(e->graph_exec, (cudaStream_t)cu_stream));
    return HE_OK;
  }
  return e->issue((cudaStream_t)cu_stream);
}

int32_t heh_exec_stats(const heh_exec* e, int32_t* launches, int32_t* steps, int32_t* instrs) {
  if (!e) HE_FAIL(HE_ERR_INVALID, "heh_exec_stats: null argument");
  if (launches) *launches = e->n_launches;
  if (steps) *steps = e->n_steps;
  if (instrs) *instrs = e->n_instrs;
  return HE_OK;
}

void heh_exec_destroy(heh_exec* e) { delete e; }

}  // extern "C"
