// Host-side lowering of a pointwise-family subgraph to the interpreter program.
//
// Follows the structure of the reference's code generator -- a memoised recursive walk from each
// leaf towards the inputs that carries an index mapping (helium/src/cuda/instr/pointwise/jit.rs:
// 196-509, 590-729) -- but emits a register program instead of CUDA source, and composes
// broadcast / swap_dims mappings symbolically into a single strided view where that is possible
// (the reference chains `/` and `%` per mapping, jit.rs:616-729).
#include <algorithm>
#include <map>

#include "pointwise_program.h"

namespace he {
namespace {

// Where the current node's axes come from.  `src[j]` = iteration-space dim that axis j of the
// current node walks, or -1 when the coordinate is pinned to 0 (broadcast).  `linear` means the
// element index passes through unchanged (robust to reshapes).  `chain` holds views that were
// materialised earlier (outermost first) when a reshape could not be expressed symbolically.
struct Mapping {
  std::vector<int> chain;
  bool linear = true;
  int root_rank = 0;
  int64_t root_shape[HE_MAX_RANK] = {0};
  int rank = 0;
  int src[HE_MAX_RANK] = {0};

  std::string key() const {
    std::string k;
    for (int v : chain) k += "v" + std::to_string(v);
    if (linear) return k + "L";
    k += "R";
    for (int i = 0; i < root_rank; ++i) k += std::to_string(root_shape[i]) + ",";
    k += "|";
    for (int i = 0; i < rank; ++i) k += std::to_string(src[i]) + ",";
    return k;
  }
};

struct VInstr {  // virtual-register instruction
  PwInstr i;
  int vdst = -1, va = -1, vb = -1, vc = -1;
};

struct Compiler {
  const Graph& g;
  int acc_node;
  PwCompiled* out;
  std::vector<VInstr> code;
  std::map<std::pair<int, std::string>, int> memo;
  int next_vreg = 0;
  int n_views = 0;
  int32_t status = HE_OK;

  Compiler(const Graph& g_, int acc, PwCompiled* o) : g(g_), acc_node(acc), out(o) {}

  int class_id(int dt) { return dclass(dt) == DClass::Float ? 0 : dclass(dt) == DClass::Int ? 1 : 2; }

  int fail(int32_t code, const char* msg) {
    if (status == HE_OK) {
      status = code;
      set_error("pointwise: %s", msg);
    }
    return -1;
  }

  int emit(PwInstr pi, int va = -1, int vb = -1, int vc = -1, bool has_dst = true) {
    VInstr v;
    v.i = pi;
    v.va = va; v.vb = vb; v.vc = vc;
    v.vdst = has_dst ? next_vreg++ : -1;
    code.push_back(v);
    return v.vdst;
  }

  // Adds a strided view given per-dim (ext, stride), OUTERMOST first; returns view id, -1 for an
  // identity view, -2 on overflow.
  int add_view(int nd, const int64_t* ext, const int64_t* stride) {
    // innermost first, drop ext-1 dims, merge dims that are contiguous in the target
    std::vector<std::pair<int64_t, int64_t>> d;
    for (int k = nd - 1; k >= 0; --k) {
      if (ext[k] == 1) continue;
      if (!d.empty() && stride[k] == d.back().second * d.back().first) d.back().first *= ext[k];
      else d.push_back({ext[k], stride[k]});
    }
    // zero-stride dims at the outer end never contribute
    bool dropped = false;
    while (!d.empty() && d.back().second == 0) {
      d.pop_back();
      dropped = true;
    }
    if (d.size() == 1 && d[0].second == 1 && !dropped) return -1;  // identity over the whole space
    if (d.empty()) d.push_back({1, 0});                // constant index 0
    if ((int)d.size() > kPwMaxViewDims || n_views >= kPwMaxViews) return -2;
    PwView& v = out->prog.views[n_views];
    v.nd = (int)d.size();
    for (int k = 0; k < v.nd; ++k) {
      v.fd[k] = FastDiv((uint32_t)d[k].first);
      v.stride[k] = (uint32_t)d[k].second;
    }
    return n_views++;
  }

  static void packed_strides(const he_node& n, int64_t* st) {
    int64_t s = 1;
    for (int i = n.rank - 1; i >= 0; --i) {
      st[i] = s;
      s *= n.shape[i];
    }
  }

  // Turns the symbolic part of `m` into a view over m.root_shape that yields the linear index
  // into `n` (the node the mapping currently points at) and appends it to the chain.
  bool materialise(Mapping& m, const he_node& n) {
    if (m.linear) return true;
    int64_t st[HE_MAX_RANK], nst[HE_MAX_RANK];
    packed_strides(n, nst);
    for (int k = 0; k < m.root_rank; ++k) st[k] = 0;
    for (int j = 0; j < m.rank; ++j)
      if (m.src[j] >= 0) st[m.src[j]] += nst[j];
    int v = add_view(m.root_rank, m.root_shape, st);
    if (v == -2) { fail(HE_ERR_UNSUPPORTED, "too many index views"); return false; }
    if (v >= 0) m.chain.push_back(v);
    m.linear = true;
    return true;
  }

  // Start of a symbolic mapping at node `n` from a linear one.
  static void open_symbolic(Mapping& m, const he_node& n) {
    m.linear = false;
    m.root_rank = n.rank;
    m.rank = n.rank;
    for (int i = 0; i < n.rank; ++i) {
      m.root_shape[i] = n.shape[i];
      m.src[i] = i;
    }
  }

  int eval(int node, const Mapping& m) {
    if (status != HE_OK) return -1;
    auto key = std::make_pair(node, m.key());
    auto it = memo.find(key);
    if (it != memo.end()) return it->second;
    int r = eval_uncached(node, m);
    memo[key] = r;
    return r;
  }

  // The mapping to use for an operand whose shape may differ from the consumer's shape while the
  // element count is equal (binary ops only require matching element counts, op.rs:306-307).
  Mapping for_operand(const Mapping& m, const he_node& consumer, const he_node& operand) {
    if (m.linear) return m;
    bool same = consumer.rank == operand.rank;
    for (int i = 0; same && i < consumer.rank; ++i) same = consumer.shape[i] == operand.shape[i];
    if (same) return m;
    Mapping mm = m;
    materialise(mm, consumer);
    return mm;
  }

  int eval_uncached(int node, const Mapping& m) {
    const he_node& n = g.nodes[node];
    PwInstr pi{};
    if (node == acc_node) {
      if (!m.linear || !m.chain.empty()) return fail(HE_ERR_UNSUPPORTED, "matmul result is used through a broadcast/swap");
      pi.op = PW_ACC;
      return emit(pi);
    }
    switch (n.kind) {
      case HE_OP_INPUT: {
        Mapping mm = m;
        PwLoadInfo li{};
        li.single_view = mm.chain.empty();
        li.identity = mm.linear && mm.chain.empty();
        if (!mm.linear) {
          int64_t nst[HE_MAX_RANK];
          packed_strides(n, nst);
          for (int k = 0; k < mm.root_rank; ++k) li.iter_stride[k] = 0;
          for (int j = 0; j < mm.rank; ++j)
            if (mm.src[j] >= 0) li.iter_stride[mm.src[j]] += nst[j];
        }
        if (!materialise(mm, n)) return -1;
        if (mm.chain.size() > 4) return fail(HE_ERR_UNSUPPORTED, "index mapping chain too deep");
        // chain views must be consecutive in the view table: copy them if they are not
        int v0 = 0;
        if (!mm.chain.empty()) {
          bool consecutive = true;
          for (size_t k = 1; k < mm.chain.size(); ++k) consecutive = consecutive && mm.chain[k] == mm.chain[k - 1] + 1;
          if (!consecutive) {
            if (n_views + (int)mm.chain.size() > kPwMaxViews) return fail(HE_ERR_UNSUPPORTED, "too many index views");
            int base = n_views;
            for (int v : mm.chain) out->prog.views[n_views++] = out->prog.views[v];
            v0 = base;
          } else {
            v0 = mm.chain[0];
          }
        }
        int slot = -1;
        for (size_t k = 0; k < g.inputs.size(); ++k)
          if (g.inputs[k] == node) slot = (int)k;
        pi.op = PW_LOAD;
        pi.dt = (uint8_t)n.dtype;
        pi.slot = (uint8_t)slot;
        pi.view0 = (uint8_t)v0;
        pi.nviews = (uint8_t)mm.chain.size();
        if (n.dtype == HE_BOOL) out->has_bool_io = true;
        int r = emit(pi);
        li.instr = (int)code.size() - 1;
        li.input_slot = slot;
        li.node = node;
        li.identity = pi.nviews == 0;
        out->loads.push_back(li);
        return r;
      }
      case HE_OP_CONSTANT: {
        pi.op = PW_CONST;
        uint32_t bits = n.const_bits;
        if (n.dtype == HE_BF16) bits = bits << 16;  // widen to the f32 the interpreter computes in
        else if (n.dtype == HE_F16) {
          // exact f16 -> f32 widening
          uint32_t h = bits & 0xffffu, sign = (h >> 15) << 31, exp = (h >> 10) & 0x1f, man = h & 0x3ff;
          if (exp == 0) {
            if (man == 0) bits = sign;
            else {
              int e = -1;
              do { ++e; man <<= 1; } while (!(man & 0x400));
              bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ff) << 13);
            }
          } else if (exp == 31) bits = sign | 0x7f800000u | (man << 13);
          else bits = sign | ((exp + 112) << 23) | (man << 13);
        } else if (n.dtype == HE_BOOL) bits = bits ? 1u : 0u;
        pi.imm = bits;
        return emit(pi);
      }
      case HE_OP_UNARY: {
        int a = eval(n.in[0], m);
        pi.op = PW_UNARY;
        pi.sub = (uint8_t)n.sub_op;
        pi.imm = n.const_bits;
        bool known = (n.sub_op >= HE_UN_RECIP && n.sub_op <= HE_UN_LOG) || (n.sub_op >= HE_UN_GELU && n.sub_op <= HE_UN_DGELU);
        if (!known) return fail(HE_ERR_INVALID, "unknown unary op");
        return emit(pi, a);
      }
      case HE_OP_BINARY: {
        const he_node& L = g.nodes[n.in[0]];
        const he_node& R = g.nodes[n.in[1]];
        int a = eval(n.in[0], m);
        int b = eval(n.in[1], for_operand(m, L, R));
        DClass c = dclass(n.dtype);
        pi.sub = (uint8_t)n.sub_op;
        if (c == DClass::Float) {
          pi.op = PW_BIN_F;
          bool ok = (n.sub_op >= HE_BIN_ADD && n.sub_op <= HE_BIN_MAX) || (n.sub_op >= HE_BIN_SUB && n.sub_op <= HE_BIN_DRELU);
          if (!ok) return fail(HE_ERR_INVALID, "binary op not valid for float tensors");
        } else if (c == DClass::Int) {
          pi.op = PW_BIN_U;
          bool ok = n.sub_op == HE_BIN_ADD || n.sub_op == HE_BIN_MUL || (n.sub_op >= HE_BIN_MIN && n.sub_op <= HE_BIN_XOR) || n.sub_op == HE_BIN_SUB;
          if (!ok) return fail(HE_ERR_UNSUPPORTED, "binary op not supported for u32 tensors");
        } else {
          pi.op = PW_BIN_B;
        }
        return emit(pi, a, b);
      }
      case HE_OP_COMPARE: {
        const he_node& L = g.nodes[n.in[0]];
        const he_node& R = g.nodes[n.in[1]];
        int a = eval(n.in[0], m);
        int b = eval(n.in[1], for_operand(m, L, R));
        pi.op = dclass(L.dtype) == DClass::Float ? PW_CMP_F : PW_CMP_U;
        pi.sub = (uint8_t)n.sub_op;
        return emit(pi, a, b);
      }
      case HE_OP_SELECT: {
        const he_node& L = g.nodes[n.in[0]];
        int a = eval(n.in[0], m);
        int b = eval(n.in[1], for_operand(m, L, g.nodes[n.in[1]]));
        int c = eval(n.in[2], for_operand(m, L, g.nodes[n.in[2]]));
        pi.op = PW_SELECT;
        return emit(pi, a, b, c);
      }
      case HE_OP_CAST: {
        const he_node& A = g.nodes[n.in[0]];
        int a = eval(n.in[0], m);
        int from = class_id(A.dtype), to = class_id(n.dtype);
        if (from == to) return a;  // only affects loads / stores (jit.rs:488-504)
        pi.op = PW_CVT;
        pi.sub = (uint8_t)(from << 2 | to);
        return emit(pi, a);
      }
      case HE_OP_RESHAPE: {
        const he_node& A = g.nodes[n.in[0]];
        Mapping mm = m;
        if (!mm.linear) {
          // a reshape that only inserts/removes size-1 dims keeps the symbolic form
          std::vector<int> keep_out, keep_in;
          for (int i = 0; i < n.rank; ++i) if (n.shape[i] != 1) keep_out.push_back(i);
          for (int i = 0; i < A.rank; ++i) if (A.shape[i] != 1) keep_in.push_back(i);
          bool trivial = keep_out.size() == keep_in.size();
          for (size_t k = 0; trivial && k < keep_out.size(); ++k) trivial = n.shape[keep_out[k]] == A.shape[keep_in[k]];
          if (trivial) {
            Mapping t = mm;
            t.rank = A.rank;
            for (int i = 0; i < A.rank; ++i) t.src[i] = -1;
            for (size_t k = 0; k < keep_out.size(); ++k) t.src[keep_in[k]] = mm.src[keep_out[k]];
            mm = t;
          } else if (!materialise(mm, n)) {
            return -1;
          }
        }
        return eval(n.in[0], mm);
      }
      case HE_OP_SWAP_DIMS: {
        Mapping mm = m;
        if (mm.linear) open_symbolic(mm, n);
        int t = mm.src[n.axis_a];
        mm.src[n.axis_a] = mm.src[n.axis_b];
        mm.src[n.axis_b] = t;
        return eval(n.in[0], mm);
      }
      case HE_OP_BROADCAST: {
        const he_node& A = g.nodes[n.in[0]];
        Mapping mm = m;
        if (mm.linear) open_symbolic(mm, n);
        Mapping t = mm;
        int pad = n.rank - A.rank;
        t.rank = A.rank;
        for (int j = 0; j < A.rank; ++j) {
          bool widened = A.shape[j] != n.shape[j + pad];  // coordinate pinned to 0 (jit.rs:689-704)
          t.src[j] = widened ? -1 : mm.src[j + pad];
        }
        return eval(n.in[0], t);
      }
      case HE_OP_REDUCE:
        return fail(HE_ERR_UNSUPPORTED, "a reduction must be a leaf of the subgraph (pointwise.rs:159-163)");
      default:
        return fail(HE_ERR_UNSUPPORTED, "op kind is not part of the pointwise family");
    }
  }
};

}  // namespace

int32_t compile_pointwise(const Graph& g, const PwCompileOptions& opt, PwCompiled* out) {
  const int acc_node = opt.acc_node;
  memset(&out->prog, 0, sizeof out->prog);
  out->loads.clear();
  out->out_dtypes.clear();
  out->out_is_reduce.clear();
  out->has_bool_io = false;
  if ((int)g.inputs.size() > kPwMaxInputs) HE_FAIL(HE_ERR_UNSUPPORTED, "pointwise: more than %d inputs", kPwMaxInputs);
  if ((int)g.outputs.size() > kPwMaxOutputs) HE_FAIL(HE_ERR_UNSUPPORTED, "pointwise: more than %d outputs", kPwMaxOutputs);

  // iteration space = shape of the first leaf, or of its input for a reduction leaf
  // (compute_output_shape, jit.rs:164-176); all leaves must agree on the element count
  // (supports_subgraph, pointwise.rs:135-147).
  auto iter_node = [&](int leaf) { return g.nodes[leaf].kind == HE_OP_REDUCE ? g.nodes[leaf].in[0] : leaf; };
  const he_node& it0 = g.nodes[iter_node(g.outputs[0])];
  const int64_t n_elems = num_elements(it0);
  if (n_elems >= (1ll << 31)) HE_FAIL(HE_ERR_UNSUPPORTED, "pointwise: %lld elements exceed the 32-bit index range", (long long)n_elems);
  out->iter_rank = it0.rank;
  for (int i = 0; i < it0.rank; ++i) out->iter_shape[i] = it0.shape[i];
  int64_t group_size = n_elems;
  int n_red = 0;
  const he_node* first_red_in = nullptr;
  uint32_t first_axes = 0;
  for (int leaf : g.outputs) {
    const he_node& itn = g.nodes[iter_node(leaf)];
    if (num_elements(itn) != n_elems) HE_FAIL(HE_ERR_UNSUPPORTED, "pointwise: all outputs must cover the same number of elements");
    const he_node& L = g.nodes[leaf];
    if (L.kind == HE_OP_REDUCE) {
      const he_node& A = g.nodes[L.in[0]];
      int d = __builtin_popcount(L.axes);
      if (opt.epilogue) { ++n_red; continue; }
      if (L.axes != (((1u << d) - 1u) << (A.rank - d)))
        HE_FAIL(HE_ERR_UNSUPPORTED, "pointwise: only reductions over trailing dims (helium-ir Reduce.depth) are supported");
      if (first_red_in) {
        bool same = first_red_in->rank == A.rank && first_axes == L.axes;
        for (int i = 0; same && i < A.rank; ++i) same = first_red_in->shape[i] == A.shape[i];
        if (!same) HE_FAIL(HE_ERR_UNSUPPORTED, "pointwise: all reductions must share input shape and depth (pointwise.rs:166-175)");
      } else {
        first_red_in = &A;
        first_axes = L.axes;
        group_size = 1;
        for (int i = A.rank - d; i < A.rank; ++i) group_size *= A.shape[i];
      }
      ++n_red;
    }
  }
  if (n_red > 4 && !opt.epilogue) HE_FAIL(HE_ERR_UNSUPPORTED, "pointwise: more than 4 reductions in one kernel");

  Compiler c(g, acc_node, out);
  Mapping ident;
  int red_slot = 0;
  for (size_t o = 0; o < g.outputs.size(); ++o) {
    const int leaf = g.outputs[o];
    const he_node& L = g.nodes[leaf];
    PwInstr pi{};
    if (L.kind == HE_OP_REDUCE) {
      int v = c.eval(L.in[0], ident);
      if (c.status != HE_OK) return c.status;
      if (L.sub_op == HE_RED_MEAN && !opt.epilogue) {   // a fused-matmul epilogue scales when it folds its partials
        PwInstr ms{};
        ms.op = PW_MEAN_SCALE;
        v = c.emit(ms, v);
      }
      pi.op = PW_REDUCE;
      pi.sub = (uint8_t)L.sub_op;
      pi.slot = (uint8_t)o;
      pi.slot2 = (uint8_t)red_slot++;
      if (opt.epilogue) {
        // axes relative to the end of the shape: bit 0 = last dim (columns), bit 1 = rows, bit 2 = any batch dim
        const he_node& A = g.nodes[L.in[0]];
        uint32_t m = 0;
        for (int k = 0; k < A.rank; ++k)
          if ((L.axes >> k) & 1u) m |= (k == A.rank - 1) ? 1u : (k == A.rank - 2) ? 2u : (A.shape[k] != 1 ? 4u : 0u);
        // a batch of one is "reduced" for free in both forms
        pi.imm = m;
      }
      c.emit(pi, v, -1, -1, false);
      out->out_dtypes.push_back(HE_F32);
      out->out_is_reduce.push_back(L.sub_op);
    } else {
      int v = c.eval(leaf, ident);
      if (c.status != HE_OK) return c.status;
      pi.op = PW_STORE;
      pi.dt = (uint8_t)L.dtype;
      pi.slot = (uint8_t)o;
      c.emit(pi, v, -1, -1, false);
      out->out_dtypes.push_back(L.dtype);
      out->out_is_reduce.push_back(-1);
      if (L.dtype == HE_BOOL) out->has_bool_io = true;
    }
  }
  if (c.status != HE_OK) return c.status;

  // ---- peephole: a multiply whose only consumer is an add becomes one fused multiply-add.
  // The reference's NVRTC build leaves fmad at its default (kernel_jit.rs:155-168), so `x * s + b`
  // is contracted there as well.
  std::vector<VInstr>& code = c.code;
  if (opt.fuse_fma) {
    std::vector<int> uses(c.next_vreg, 0), def(c.next_vreg, -1);
    for (size_t i = 0; i < code.size(); ++i) {
      if (code[i].va >= 0) ++uses[code[i].va];
      if (code[i].vb >= 0) ++uses[code[i].vb];
      if (code[i].vc >= 0) ++uses[code[i].vc];
      if (code[i].vdst >= 0) def[code[i].vdst] = (int)i;
    }
    for (size_t i = 0; i < code.size(); ++i) {
      VInstr& add = code[i];
      if (add.i.op != PW_BIN_F || add.i.sub != HE_BIN_ADD) continue;
      for (int side = 0; side < 2; ++side) {
        int mv = side == 0 ? add.va : add.vb, other = side == 0 ? add.vb : add.va;
        if (mv < 0 || uses[mv] != 1 || mv == other) continue;
        VInstr& mul = code[def[mv]];
        if (mul.i.op != PW_BIN_F || mul.i.sub != HE_BIN_MUL) continue;
        add.i.op = PW_FMA;
        add.va = mul.va; add.vb = mul.vb; add.vc = other;
        mul.i.op = 255;  // dead
        break;
      }
    }
    std::vector<VInstr> live;
    std::vector<int> remap(code.size(), -1);
    for (size_t i = 0; i < code.size(); ++i)
      if (code[i].i.op != 255) {
        remap[i] = (int)live.size();
        live.push_back(code[i]);
      }
    for (auto& li : out->loads) li.instr = remap[li.instr];
    code.swap(live);
  }
  if ((int)code.size() > kPwMaxInstr) HE_FAIL(HE_ERR_UNSUPPORTED, "pointwise: program has %zu instructions (max %d)", code.size(), kPwMaxInstr);

  // ---- register allocation: linear scan over last uses
  std::vector<int> last_use(c.next_vreg, -1);
  for (size_t i = 0; i < code.size(); ++i) {
    if (code[i].va >= 0) last_use[code[i].va] = (int)i;
    if (code[i].vb >= 0) last_use[code[i].vb] = (int)i;
    if (code[i].vc >= 0) last_use[code[i].vc] = (int)i;
  }
  std::vector<int> phys(c.next_vreg, -1);
  std::vector<int> free_regs;
  for (int r = kPwMaxRegs - 1; r >= 0; --r) free_regs.push_back(r);
  int max_reg = 0;
  for (size_t i = 0; i < code.size(); ++i) {
    VInstr& v = code[i];
    PwInstr& pi = v.i;
    pi.a = v.va >= 0 ? (uint8_t)phys[v.va] : 0;
    pi.b = v.vb >= 0 ? (uint8_t)phys[v.vb] : 0;
    pi.c = v.vc >= 0 ? (uint8_t)phys[v.vc] : 0;
    // operands whose last use is here are released before the destination is assigned
    int ops[3] = {v.va, v.vb, v.vc};
    for (int k = 0; k < 3; ++k) {
      int o = ops[k];
      if (o < 0 || last_use[o] != (int)i || phys[o] < 0) continue;
      bool dup = false;
      for (int q = 0; q < k; ++q) dup = dup || ops[q] == o;
      if (!dup) free_regs.push_back(phys[o]);
    }
    if (v.vdst >= 0) {
      if (free_regs.empty()) HE_FAIL(HE_ERR_UNSUPPORTED, "pointwise: more than %d live values", kPwMaxRegs);
      // lowest-numbered free register keeps the footprint small
      size_t best = 0;
      for (size_t k = 1; k < free_regs.size(); ++k)
        if (free_regs[k] < free_regs[best]) best = k;
      phys[v.vdst] = free_regs[best];
      free_regs.erase(free_regs.begin() + best);
      pi.dst = (uint8_t)phys[v.vdst];
      if (phys[v.vdst] + 1 > max_reg) max_reg = phys[v.vdst] + 1;
      if (last_use[v.vdst] < 0) free_regs.push_back(phys[v.vdst]);  // never read
    }
    out->prog.instr[i] = pi;
  }
  out->n_regs = max_reg;
  out->prog.n_instr = (int)code.size();
  out->prog.n_inputs = (int)g.inputs.size();
  out->prog.n_outputs = (int)g.outputs.size();
  out->prog.n_elems = (uint32_t)n_elems;
  out->prog.group_size = (uint32_t)group_size;
  out->prog.n_reductions = n_red;
  out->prog.mean_scale = group_size > 0 ? 1.0 / (double)group_size : 0.0;
  return HE_OK;
}


// ------------------------------------------------------------------------------------------------
// canonical text
// ------------------------------------------------------------------------------------------------
namespace {
std::string blank_slots(const std::string& t) {
  std::string o;
  for (size_t i = 0; i < t.size(); ++i) {
    if (t[i] == 'I' && i + 1 < t.size() && isdigit((unsigned char)t[i + 1])) {
      o += "I#";
      ++i;
      while (i + 1 < t.size() && isdigit((unsigned char)t[i + 1])) ++i;
    } else {
      o += t[i];
    }
  }
  return o;
}
bool canon_less(const std::string& a, const std::string& b) {
  const std::string ba = blank_slots(a), bb = blank_slots(b);
  if (ba != bb) return ba < bb;
  return a < b;
}
}  // namespace

int32_t canonicalize_program(const Graph& g, const PwCompiled& c, int m_dim, int n_dim, PwCanon* out) {
  const PwProgram& P = c.prog;
  std::vector<std::string> reg(kPwMaxRegs);
  // add / mul chains are flattened into sorted term lists so that (a + b) + c and a + (c + b)
  // read the same; chain[r] is '+', '*' or 0 and terms[r] the operands of the chain in reg r
  std::vector<char> chain(kPwMaxRegs, 0);
  std::vector<std::vector<std::string>> terms(kPwMaxRegs);
  std::vector<std::pair<std::string, int>> outs;  // (text, caller output index)
  auto load_class = [&](const PwLoadInfo& li) -> char {
    const he_node& n = g.nodes[li.node];
    if (!li.single_view) return 'X';
    if (li.identity) return num_elements(n) == (int64_t)P.n_elems ? 'F' : 'X';
    int64_t sM = m_dim >= 0 ? li.iter_stride[m_dim] : 0, sN = n_dim >= 0 ? li.iter_stride[n_dim] : 0;
    bool batch_zero = true, batch_packed = true;
    int64_t expect = (m_dim >= 0 ? c.iter_shape[m_dim] : 1) * (n_dim >= 0 ? c.iter_shape[n_dim] : 1);
    for (int k = c.iter_rank - 1; k >= 0; --k) {
      if (k == m_dim || k == n_dim || c.iter_shape[k] == 1) continue;
      if (li.iter_stride[k] != 0) batch_zero = false;
      if (li.iter_stride[k] != expect) batch_packed = false;
      expect *= c.iter_shape[k];
    }
    const int64_t N = n_dim >= 0 ? c.iter_shape[n_dim] : 1, M = m_dim >= 0 ? c.iter_shape[m_dim] : 1;
    const bool n1 = sN == 1 || N == 1, n0 = sN == 0 || N == 1;
    if (n1 && (sM == N || M == 1) && batch_packed) return 'F';
    if (n1 && (sM == 0 || M == 1) && batch_zero) return 'R';   // varies with the column only
    if (n0 && (sM == 1 || M == 1) && batch_zero) return 'C';   // varies with the row only
    if (n0 && (sM == 0 || M == 1) && batch_zero) return 'S';
    return 'X';
  };
  char buf[64];
  for (int i = 0; i < P.n_instr; ++i) {
    const PwInstr& in = P.instr[i];
    std::string t;
    switch (in.op) {
      case PW_LOAD: {
        const PwLoadInfo* li = nullptr;
        for (const PwLoadInfo& l : c.loads)
          if (l.instr == i) li = &l;
        if (!li) HE_FAIL(HE_ERR_INVALID, "canonicalize: load without info");
        snprintf(buf, sizeof buf, "I%d:%c", li->input_slot, load_class(*li));
        t = buf;
        break;
      }
      case PW_CONST: snprintf(buf, sizeof buf, "K%08x", in.imm); t = buf; break;
      case PW_ACC: t = "A"; break;
      case PW_UNARY: {
        const bool has_imm = in.sub >= HE_UN_ADD_CONST && in.sub <= HE_UN_POW_CONST;
        if (has_imm) snprintf(buf, sizeof buf, "u%d[%08x](", in.sub, in.imm);
        else snprintf(buf, sizeof buf, "u%d(", in.sub);
        t = buf + reg[in.a] + ")";
        break;
      }
      case PW_BIN_F: case PW_BIN_U: case PW_BIN_B: {
        if (in.op == PW_BIN_F && (in.sub == HE_BIN_ADD || in.sub == HE_BIN_MUL)) {
          const char kind = in.sub == HE_BIN_ADD ? '+' : '*';
          std::vector<std::string> ts;
          const int ops[2] = {in.a, in.b};
          for (int o : ops) {
            if (chain[o] == kind) ts.insert(ts.end(), terms[o].begin(), terms[o].end());
            else ts.push_back(reg[o]);
          }
          std::sort(ts.begin(), ts.end(), canon_less);
          t = kind == '+' ? "sum(" : "prod(";
          for (size_t k = 0; k < ts.size(); ++k) t += (k ? "," : "") + ts[k];
          t += ")";
          reg[in.dst] = t;
          chain[in.dst] = kind;
          terms[in.dst] = ts;
          continue;
        }
        std::string a = reg[in.a], b = reg[in.b];
        const bool comm = in.sub == HE_BIN_ADD || in.sub == HE_BIN_MUL || in.sub == HE_BIN_MIN || in.sub == HE_BIN_MAX ||
                          (in.sub >= HE_BIN_AND && in.sub <= HE_BIN_XOR);
        if (comm && canon_less(b, a)) std::swap(a, b);
        snprintf(buf, sizeof buf, "b%d%c(", in.sub, in.op == PW_BIN_F ? 'f' : in.op == PW_BIN_U ? 'u' : 'b');
        t = buf + a + "," + b + ")";
        break;
      }
      case PW_FMA: t = "fma(" + reg[in.a] + "," + reg[in.b] + "," + reg[in.c] + ")"; break;
      case PW_CMP_F: case PW_CMP_U:
        snprintf(buf, sizeof buf, "c%d%c(", in.sub, in.op == PW_CMP_F ? 'f' : 'u');
        t = buf + reg[in.a] + "," + reg[in.b] + ")";
        break;
      case PW_SELECT: t = "sel(" + reg[in.a] + "," + reg[in.b] + "," + reg[in.c] + ")"; break;
      case PW_CVT: snprintf(buf, sizeof buf, "cvt%d(", in.sub); t = buf + reg[in.a] + ")"; break;
      case PW_MEAN_SCALE: t = "mean(" + reg[in.a] + ")"; break;
      case PW_STORE: outs.push_back({"store(" + reg[in.a] + ")", in.slot}); continue;
      case PW_REDUCE:
        snprintf(buf, sizeof buf, "red%d@%u(", in.sub, in.imm);
        outs.push_back({buf + reg[in.a] + ")", in.slot});
        continue;
      default: HE_FAIL(HE_ERR_INVALID, "canonicalize: unknown instruction");
    }
    if (t.size() > (1u << 20)) HE_FAIL(HE_ERR_UNSUPPORTED, "canonicalize: expression too large");
    reg[in.dst] = t;
    chain[in.dst] = 0;
    terms[in.dst].clear();
  }
  std::stable_sort(outs.begin(), outs.end(), [](const std::pair<std::string, int>& a, const std::pair<std::string, int>& b) {
    return canon_less(a.first, b.first);
  });
  std::string all;
  out->out_order.clear();
  for (auto& o : outs) {
    all += o.first + ";";
    out->out_order.push_back(o.second);
  }
  // rename input slots in order of first appearance
  out->slot_order.clear();
  std::string text;
  for (size_t i = 0; i < all.size(); ++i) {
    if (all[i] == 'I' && i + 1 < all.size() && isdigit((unsigned char)all[i + 1])) {
      size_t j = i + 1;
      int slot = 0;
      while (j < all.size() && isdigit((unsigned char)all[j])) slot = slot * 10 + (all[j++] - '0');
      int k = -1;
      for (size_t q = 0; q < out->slot_order.size(); ++q)
        if (out->slot_order[q] == slot) k = (int)q;
      if (k < 0) {
        k = (int)out->slot_order.size();
        out->slot_order.push_back(slot);
      }
      text += "I" + std::to_string(k);
      i = j - 1;
    } else {
      text += all[i];
    }
  }
  out->text = text;
  return HE_OK;
}

}  // namespace he
