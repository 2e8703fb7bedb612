// Planner for fused matmul subgraphs (hot-path rows G0-G3, F1-F2).
//
// Replaces, on the host side, MatmulGenerator::new / find_root / find_and_verify_leafs
// (helium-kernel-generator/src/generators/matmul.rs:88-130, 234-318) and the playground's
// KernelGenerator::generate (helium-playground/src/kernel_generator.rs:51-117): it splits the
// subgraph into operand side (mainloop) and result side (epilogue), decides operand majors from
// swap_dims nodes, and maps the epilogue onto either a hand-written functor (catalogue match on a
// canonical text of the epilogue program) or the interpreted tier.
#include <cuda.h>

#include <algorithm>
#include <memory>
#include <mutex>

#include "gemm_plan.cuh"
#include "pointwise_dense.cuh"

namespace he {
namespace {

// ------------------------------------------------------------------------------------------------
// TMA descriptor encoding through the driver entry point (no link-time dependency on libcuda)
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Operand tensor [batch, R, K] (K-major) or [batch, K, R] (MN-major), 2-byte elements.
// `pitch` = elements between consecutive rows of the stored matrix (0: dense, i.e. K or R).
int32_t make_operand_tmap(CUtensorMap* out, const void* ptr, int ab_format, bool mn_major, int64_t R, int64_t K,
                          int64_t batch, int box_rows, int64_t pitch = 0) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) HE_FAIL(HE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if ((uintptr_t)ptr % 16 != 0) HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: operand pointer is not 16-byte aligned");
  cuuint64_t dims[3], strides[2];
  cuuint32_t box[3], estr[3] = {1, 1, 1};
  if (!mn_major) {
    const cuuint64_t ld = (cuuint64_t)(pitch ? pitch : K);
    dims[0] = (cuuint64_t)K; dims[1] = (cuuint64_t)R; dims[2] = (cuuint64_t)batch;
    strides[0] = ld * 2; strides[1] = (cuuint64_t)R * ld * 2;
    box[0] = kBK; box[1] = (cuuint32_t)box_rows; box[2] = 1;
  } else {
    const cuuint64_t ld = (cuuint64_t)(pitch ? pitch : R);
    dims[0] = (cuuint64_t)R; dims[1] = (cuuint64_t)K; dims[2] = (cuuint64_t)batch;
    strides[0] = ld * 2; strides[1] = (cuuint64_t)K * ld * 2;
    box[0] = 64; box[1] = kBK; box[2] = 1;
  }
  if (strides[0] % 16 != 0) HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: operand row pitch %llu B is not a multiple of 16", (unsigned long long)strides[0]);
  CUresult r = fn(out, ab_format == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                  const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) HE_FAIL(HE_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return HE_OK;
}

// 8-bit operand copy [batch, R, k_pitch] bytes, K-major: box = 128 bytes of K x box_rows rows.
int32_t make_f8_tmap(CUtensorMap* out, const void* ptr, int64_t R, int64_t K, int64_t k_pitch, int64_t batch, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) HE_FAIL(HE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)R, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)k_pitch, (cuuint64_t)R * k_pitch};
  cuuint32_t box[3] = {128u, (cuuint32_t)box_rows, 1u}, estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) HE_FAIL(HE_ERR_CUDA, "cuTensorMapEncodeTiled (8-bit operand) failed with CUresult %d", (int)r);
  return HE_OK;
}

// ------------------------------------------------------------------------------------------------
// operand (mainloop) side
// ------------------------------------------------------------------------------------------------
struct OperandInfo {
  int root = -1;      // graph node of the tensor that feeds the MMA
  int mask = -1;      // second tensor combined elementwise (relu(A) * M, A + E, ...)
  bool relu = false;  // the chain is exactly relu(root) (* mask): the hand-written rewrite applies
  bool transposed = false;  // root is stored with its last two dims swapped w.r.t. what matmul sees
  bool ok = true;
  std::vector<MlStep> steps;   // the chain in evaluation order (unary steps, at most one multiply / add by `mask`)
  bool pure() const { return ok && steps.empty(); }
  bool relu_mask() const { return ok && relu && mask >= 0 && steps.size() == 2; }
};

MlStep ml_unary(int op, uint32_t imm) {
  MlStep s{};
  s.kind = 0;
  s.op = (unsigned char)op;
  s.imm = imm;
  return s;
}

// Value of a node that is a constant broadcast to any shape (Constant, or Broadcast / Reshape / same-class Cast of one).
bool constant_value(const Graph& g, int node, float* out) {
  const he_node& n = g.nodes[node];
  if (n.kind == HE_OP_CONSTANT && dclass(n.dtype) == DClass::Float) {
    if (n.dtype == HE_F32) memcpy(out, &n.const_bits, 4);
    else if (n.dtype == HE_BF16) { const uint32_t b = n.const_bits << 16; memcpy(out, &b, 4); }
    else return false;
    return true;
  }
  if ((n.kind == HE_OP_BROADCAST || n.kind == HE_OP_RESHAPE || (n.kind == HE_OP_CAST && dclass(n.dtype) == DClass::Float)) && n.in[0] >= 0)
    return constant_value(g, n.in[0], out);
  return false;
}

OperandInfo trace_operand(const Graph& g, int node, bool transposed) {
  const he_node& n = g.nodes[node];
  OperandInfo r;
  switch (n.kind) {
    case HE_OP_INPUT:
      r.root = node;
      r.transposed = transposed;
      return r;
    case HE_OP_CAST:
      // a cast between float types only changes where the value is rounded; the chain is evaluated in f32 and
      // rounded once to the operand type
      if (dclass(n.dtype) == DClass::Float && dclass(g.nodes[n.in[0]].dtype) == DClass::Float) {
        r = trace_operand(g, n.in[0], transposed);
        if (r.ok && (n.dtype == g.nodes[n.in[0]].dtype || !r.steps.empty() || g.nodes[r.root].dtype == n.dtype)) return r;
      }
      break;
    case HE_OP_RESHAPE: {
      const he_node& a = g.nodes[n.in[0]];
      // only leading size-1 dims may come and go
      if (n.rank >= 2 && a.rank >= 2 && n.shape[n.rank - 1] == a.shape[a.rank - 1] && n.shape[n.rank - 2] == a.shape[a.rank - 2])
        return trace_operand(g, n.in[0], transposed);
      break;
    }
    case HE_OP_SWAP_DIMS: {
      const int lo = std::min(n.axis_a, n.axis_b), hi = std::max(n.axis_a, n.axis_b);
      if (lo == hi) return trace_operand(g, n.in[0], transposed);
      if (lo == n.rank - 2 && hi == n.rank - 1) return trace_operand(g, n.in[0], !transposed);
      break;
    }
    case HE_OP_UNARY: {
      r = trace_operand(g, n.in[0], transposed);
      if (!r.ok) break;
      if (n.sub_op == HE_UN_RELU && r.pure()) r.relu = true;
      else if (!r.steps.empty()) r.relu = false;
      r.steps.push_back(ml_unary(n.sub_op, n.const_bits));
      return r;
    }
    case HE_OP_BINARY:
      if (n.sub_op == HE_BIN_MUL || n.sub_op == HE_BIN_ADD) {
        // x (op) constant becomes a unary step
        for (int side = 0; side < 2; ++side) {
          float cv;
          if (constant_value(g, n.in[1 - side], &cv)) {
            r = trace_operand(g, n.in[side], transposed);
            if (!r.ok) break;
            uint32_t bits;
            memcpy(&bits, &cv, 4);
            r.relu = false;
            r.steps.push_back(ml_unary(n.sub_op == HE_BIN_MUL ? HE_UN_MUL_CONST : HE_UN_ADD_CONST, bits));
            return r;
          }
        }
        OperandInfo l = trace_operand(g, n.in[0], transposed), rr = trace_operand(g, n.in[1], transposed);
        if (l.ok && rr.ok) {
          if (!rr.pure() && l.pure()) std::swap(l, rr);
          if (rr.pure() && l.mask < 0 && l.transposed == rr.transposed &&
              num_elements(g.nodes[rr.root]) == num_elements(g.nodes[l.root])) {
            l.mask = rr.root;
            MlStep st{};
            st.kind = n.sub_op == HE_BIN_MUL ? 1 : 2;
            l.steps.push_back(st);
            if (!(l.relu && l.steps.size() == 2 && st.kind == 1)) l.relu = false;
            return l;
          }
        }
      }
      break;
    default: break;
  }
  r.ok = false;
  return r;
}

// ------------------------------------------------------------------------------------------------
// small graph builder for the catalogue patterns
// ------------------------------------------------------------------------------------------------
struct GB {
  std::vector<he_node> nodes;
  std::vector<int> outputs;
  int add(he_node n) {
    nodes.push_back(n);
    return (int)nodes.size() - 1;
  }
  static he_node base(int kind, int dtype, std::initializer_list<int64_t> shape) {
    he_node n{};
    n.kind = kind;
    n.dtype = dtype;
    n.rank = (int)shape.size();
    int i = 0;
    for (int64_t d : shape) n.shape[i++] = d;
    n.in[0] = n.in[1] = n.in[2] = -1;
    return n;
  }
  int input(int dtype, std::initializer_list<int64_t> shape) { return add(base(HE_OP_INPUT, dtype, shape)); }
  int like(int kind, int src) {
    he_node n = nodes[src];
    n.kind = kind;
    n.in[0] = n.in[1] = n.in[2] = -1;
    n.sub_op = 0;
    n.const_bits = 0;
    return add(n);
  }
  int unary(int op, int a, float c = 0.0f) {
    int i = like(HE_OP_UNARY, a);
    nodes[i].sub_op = op;
    nodes[i].in[0] = a;
    memcpy(&nodes[i].const_bits, &c, 4);
    return i;
  }
  int binary(int op, int a, int b) {
    int i = like(HE_OP_BINARY, a);
    nodes[i].sub_op = op;
    nodes[i].in[0] = a;
    nodes[i].in[1] = b;
    return i;
  }
  int constant(float v, std::initializer_list<int64_t> shape) {
    he_node n = base(HE_OP_CONSTANT, HE_F32, shape);
    memcpy(&n.const_bits, &v, 4);
    return add(n);
  }
  int broadcast(int a, int axis, int64_t amount) {
    int i = like(HE_OP_BROADCAST, a);
    nodes[i].in[0] = a;
    nodes[i].shape[axis] = amount;
    return i;
  }
  int reduce_sum(int a, uint32_t axes) {
    int i = like(HE_OP_REDUCE, a);
    nodes[i].in[0] = a;
    nodes[i].sub_op = HE_RED_SUM;
    nodes[i].axes = axes;
    nodes[i].dtype = HE_F32;
    for (int k = 0; k < nodes[i].rank; ++k)
      if ((axes >> k) & 1u) nodes[i].shape[k] = 1;
    return i;
  }
  int matmul(int a, int b) {
    he_node n = base(HE_OP_MATMUL, HE_F32, {nodes[a].shape[0], nodes[a].shape[1], nodes[b].shape[2]});
    n.in[0] = a;
    n.in[1] = b;
    n.sub_op = HE_PREC_BF16_F32;
    return add(n);
  }
  Graph graph() const {
    Graph g;
    he_graph_desc d{(int32_t)nodes.size(), nodes.data(), (int32_t)outputs.size(), outputs.data()};
    parse_graph(&d, &g);
    return g;
  }
};

constexpr int64_t kPM = 8, kPN = 16, kPK = 8;  // pattern graphs only need distinct M and N

struct FlexCombo {
  bool bias, resid, store_z;
  int act, gate, colsum;
};

struct FlexPattern {
  FlexCombo combo;
  PwCanon canon;
  int bias_slot = -1, resid_slot = -1, gate_slot = -1;  // pattern-graph epilogue input slots
  int y_out = -1, z_out = -1, colsum_out = -1;
};

struct C3Roles {
  int b1 = -1, b2 = -1, mask = -1, y = -1, e1 = -1, e2 = -1;               // input slots
  int loss = -1, db2 = -1, db1 = -1, gt = -1, gz1 = -1;                      // output indices
};

int32_t canon_of(const Graph& g, int matmul_node, PwCompiled* c, PwCanon* canon) {
  PwCompileOptions opt;
  opt.acc_node = matmul_node;
  opt.fuse_fma = false;
  opt.epilogue = true;
  HE_TRY(compile_pointwise(g, opt, c));
  const int r = c->iter_rank;
  return canonicalize_program(g, *c, r - 2, r - 1, canon);
}

// Pattern graphs put the two matmul operands first, so graph input slot s >= 2 is epilogue input.
bool build_flex_pattern(const FlexCombo& fc, FlexPattern* out) {
  GB b;
  int a = b.input(HE_BF16, {1, kPM, kPK}), w = b.input(HE_BF16, {1, kPK, kPN});
  int acc = b.matmul(a, w);
  int next_slot = 2;
  int t = acc;
  out->combo = fc;
  if (fc.bias) {
    int bias = b.input(HE_BF16, {1, 1, kPN});
    out->bias_slot = next_slot++;
    t = b.binary(HE_BIN_ADD, t, b.broadcast(bias, 1, kPM));
  }
  int resid = -1;
  if (fc.resid) {
    resid = b.input(HE_BF16, {1, kPM, kPN});
    out->resid_slot = next_slot++;
    t = b.binary(HE_BIN_ADD, t, resid);
  }
  int nout = 0;
  int z = t;
  int y = t;
  if (fc.act == ACT_RELU) y = b.unary(HE_UN_RELU, y);
  else if (fc.act == ACT_GELU) y = b.unary(HE_UN_GELU, y);
  else if (fc.act == ACT_TANH) y = b.unary(HE_UN_TANH, y);
  if (fc.gate != GATE_NONE) {
    int gi = b.input(HE_BF16, {1, kPM, kPN});
    out->gate_slot = next_slot++;
    if (fc.gate == GATE_MUL) y = b.binary(HE_BIN_MUL, y, gi);
    else if (fc.gate == GATE_DGELU) y = b.binary(HE_BIN_MUL, y, b.unary(HE_UN_DGELU, gi));
    else if (fc.gate == GATE_DRELU) y = b.binary(HE_BIN_DRELU, y, gi);
    else return false;
  }
  b.outputs.push_back(y);
  out->y_out = nout++;
  if (fc.store_z) {
    if (z == y) return false;
    b.outputs.push_back(z);
    out->z_out = nout++;
  }
  if (fc.colsum == 1) {
    if (!fc.resid) return false;
    b.outputs.push_back(b.reduce_sum(resid, 1u << 1));
    out->colsum_out = nout++;
  } else if (fc.colsum == 2) {
    b.outputs.push_back(b.reduce_sum(y, 1u << 1));
    out->colsum_out = nout++;
  }
  Graph g = b.graph();
  PwCompiled c;
  return canon_of(g, acc, &c, &out->canon) == HE_OK;
}

const std::vector<FlexPattern>& flex_catalogue() {
  static std::vector<FlexPattern> cat;
  static std::once_flag once;
  std::call_once(once, [] {
    for (int bias = 0; bias < 2; ++bias)
      for (int resid = 0; resid < 2; ++resid)
        for (int sz = 0; sz < 2; ++sz)
          for (int act = ACT_NONE; act <= ACT_TANH; ++act)
            for (int gate = GATE_NONE; gate <= GATE_DRELU; ++gate)
              for (int cs = 0; cs < 3; ++cs) {
                FlexPattern p;
                if (build_flex_pattern(FlexCombo{bias != 0, resid != 0, sz != 0, act, gate, cs}, &p)) cat.push_back(p);
              }
  });
  return cat;
}

// README.md:33-79, node numbers in comments.
bool build_c3_pattern(bool with_e, float inv_n, PwCanon* canon, C3Roles* roles) {
  GB b;
  int a = b.input(HE_BF16, {1, kPM, kPK}), w = b.input(HE_BF16, {1, kPK, kPN});
  int acc = b.matmul(a, w);
  int slot = 2;
  int b1 = b.input(HE_BF16, {1, 1, kPN}); roles->b1 = slot++;      // 6
  int b2 = b.input(HE_BF16, {1, 1, kPN}); roles->b2 = slot++;      // 8
  int mk = b.input(HE_BF16, {1, kPM, kPN}); roles->mask = slot++;  // 9
  int yy = b.input(HE_BF16, {1, kPM, kPN}); roles->y = slot++;     // 11
  int n14 = acc, n27 = acc;
  if (with_e) {
    int e1 = b.input(HE_BF16, {1, kPM, kPN}); roles->e1 = slot++;  // 13
    int e2 = b.input(HE_BF16, {1, kPM, kPN}); roles->e2 = slot++;  // 26
    n14 = b.binary(HE_BIN_ADD, acc, e1);                           // 14
    n27 = b.binary(HE_BIN_ADD, acc, e2);                           // 27
  }
  int n16 = b.binary(HE_BIN_ADD, n14, b.broadcast(b1, 1, kPM));    // 15, 16
  int n17 = b.unary(HE_UN_RELU, n16);                              // 17
  int n29 = b.binary(HE_BIN_ADD, n27, b.broadcast(b2, 1, kPM));    // 28, 29
  int n30 = b.unary(HE_UN_TANH, n29);                              // 30
  int n32 = b.unary(HE_UN_ADD_CONST, b.unary(HE_UN_NEG, n17), 1.0f);  // 31, 32
  int n33 = b.binary(HE_BIN_MUL, n32, mk);                         // 33
  int n34 = b.binary(HE_BIN_MUL, n17, n30);                        // 34
  int n35 = b.binary(HE_BIN_ADD, n33, n34);                        // 35
  int n36 = b.binary(HE_BIN_SUB, n35, yy);                         // 36
  int n37 = b.unary(HE_UN_POW_CONST, n36, 2.0f);                   // 37
  int n38 = b.unary(HE_UN_MUL_CONST, n37, inv_n);                  // 38
  int n39 = b.reduce_sum(n38, 7u);                                 // 39 Batch
  int n41 = b.constant(1.0f, {1, 1, 1});                           // 41
  int n44 = b.broadcast(b.broadcast(b.broadcast(n41, 1, kPM), 2, kPN), 0, 1);  // 42-44
  int n45 = b.unary(HE_UN_MUL_CONST, n44, inv_n);                  // 45
  int n46 = b.constant(2.0f, {1, kPM, kPN});                       // 46
  int n47 = b.constant(1.0f, {1, kPM, kPN});                       // 47
  int n48 = b.binary(HE_BIN_POW, n36, n47);                        // 48
  int n49 = b.binary(HE_BIN_MUL, n48, n46);                        // 49
  int n50 = b.binary(HE_BIN_MUL, n49, n45);                        // 50
  int n52 = b.binary(HE_BIN_MUL, n50, n30);                        // 52
  int n53 = b.binary(HE_BIN_MUL, n17, n50);                        // 53
  int n56 = b.unary(HE_UN_ADD_CONST, b.unary(HE_UN_NEG, b.unary(HE_UN_POW_CONST, n30, 2.0f)), 1.0f);  // 54-56
  int n57 = b.binary(HE_BIN_MUL, n53, n56);                        // 57
  int n58 = b.reduce_sum(n57, 1u << 1);                            // 58 Columns
  int n81 = b.binary(HE_BIN_MUL, n50, mk);                         // 81
  int n85 = b.binary(HE_BIN_ADD, n52, b.unary(HE_UN_NEG, n81));    // 84, 85
  int n86 = b.binary(HE_BIN_DRELU, n85, n16);                      // 86
  int n87 = b.reduce_sum(n86, 1u << 1);                            // 87 Columns
  b.outputs = {n39, n58, n87, n57, n86};
  roles->loss = 0; roles->db2 = 1; roles->db1 = 2; roles->gt = 3; roles->gz1 = 4;
  Graph g = b.graph();
  PwCompiled c;
  return canon_of(g, acc, &c, canon) == HE_OK;
}

// ------------------------------------------------------------------------------------------------
// the plan
// ------------------------------------------------------------------------------------------------
enum class EpiKind { Flex, C3, Program, Sgemm };

struct MatmulPlan : he_plan {
  GemmCore core{};
  GemmLaunchCfg cfg{};
  EpiKind kind = EpiKind::Flex;
  int a_slot = -1, b_slot = -1, mask_slot = -1;  // he_launch input slots
  // Flex
  EpiFlexParams flex{};
  int f_bias = -1, f_resid = -1, f_gate = -1, f_y = -1, f_z = -1, f_colsum = -1;
  // C3
  EpiC3Params c3{};
  C3Roles r3;
  // Program (interpreted epilogue) and its reductions: kind 0 columns, 1 rows, 2 scalar
  PwCompiled prog;
  int pr_n_red = 0, pr_kind[4] = {0, 0, 0, 0}, pr_out[4] = {-1, -1, -1, -1}, pr_fold_batch[4] = {0, 0, 0, 0};
  int pr_op[4] = {0, 0, 0, 0};               // 0 sum, 1 max, 2 min
  float pr_scale[4] = {1.f, 1.f, 1.f, 1.f};  // 1 / count for a mean
  size_t pr_off[4] = {0, 0, 0, 0};   // workspace offsets in floats
  int pr_n_col = 0, pr_col_slot[2] = {0, 0}, pr_row_slots = 0;
  int n_inputs = 0, n_outputs = 0;
  // Sgemm
  int s_bias = -1, s_act = 0, s_in_dt = HE_F32, s_out_dt = HE_F32, s_bias_dt = HE_F32;
  // SIMT scale/accumulate epilogue: out = [resid +] [-] (acc * (s_alpha | mul input))
  bool s_axpy = false;
  int s_resid = -1, s_resid_dt = HE_F32, s_mul = -1, s_mul_dt = HE_F32, s_negate = 0;
  float s_alpha = 1.0f;
  // workspace layout (floats)
  size_t ws_col_off[2] = {0, 0}, ws_scalar_off = 0;
  // Mainloop fusion by materialisation: relu(A) * mask is written once to the workspace by the dense
  // elementwise kernel and the GEMM runs its plain mainloop on it.  Chosen at plan time when the
  // in-kernel rewrite (repeated for every N tile, at about half the plain mainloop's rate) would
  // cost more than one extra pass over A and the mask.
  bool materialise_a = false;
  bool ml_b = false;          // generic mainloop program on the B operand (single-CTA kernel only)
  size_t ws_aprime_off = 0;   // bytes
  // Operands whose row pitch is not a multiple of 16 bytes cannot be described to TMA.  They are copied
  // once per launch into the workspace with the pitch rounded up to 8 elements (`pad_pitch`), and the
  // tensor map reads that copy with the true extent, so the ragged edge is zero-filled by TMA as usual.
  // The reference's generator serves such shapes with predicated mma.sync tiles
  // (helium-kernel-generator/src/generators/matmul/sm80.rs:470-526); here they stay on tcgen05.
  int64_t pad_pitch[2] = {0, 0};   // A, B
  size_t ws_pad_off[2] = {0, 0};   // bytes
  // 8-bit multiplication (MulF8Accum*): both operands are rounded once per launch into K-major 8-bit copies in the
  // workspace (the reference converts fragments in registers, sm80.rs:317-333) and the kernels run
  // tcgen05.mma kind::f8f6f4 on them: twice the math per byte staged in shared memory.
  int f8 = 0;                      // GemmCore::f8
  bool f8_src_mn[2] = {false, false};
  int f8_src_dt[2] = {HE_BF16, HE_BF16};
  size_t ws_f8_off[2] = {0, 0};    // bytes

  int32_t set_fault_injection(uint32_t wait_limit_us, int32_t withhold_loads) override {
    if (kind == EpiKind::Sgemm) HE_FAIL(HE_ERR_UNSUPPORTED, "the SIMT matmul has no device-side waits to bound");
    core.wait_limit_us = wait_limit_us ? wait_limit_us : ptx::kDefaultWaitLimitUs;
    core.withhold_loads = withhold_loads ? 1 : 0;
    return HE_OK;
  }

  int32_t launch(const void* const* inputs, void* const* outputs, void* workspace, cudaStream_t stream) override {
    for (int i = 0; i < n_inputs; ++i)
      if (!inputs || !inputs[i]) HE_FAIL(HE_ERR_INVALID, "fused matmul launch: input %d is null", i);
    for (int i = 0; i < n_outputs; ++i)
      if (!outputs || !outputs[i]) HE_FAIL(HE_ERR_INVALID, "fused matmul launch: output %d is null", i);
    if (core.M == 0 || core.N == 0 || core.batch == 0) return HE_OK;
    if (kind == EpiKind::Sgemm) {
      SgemmAxpy axpy;
      if (s_axpy) {
        axpy.enabled = 1; axpy.alpha = s_alpha; axpy.negate = s_negate;
        if (s_resid >= 0) { axpy.resid = inputs[s_resid]; axpy.resid_dt = s_resid_dt; }
        if (s_mul >= 0) { axpy.mul = inputs[s_mul]; axpy.mul_dt = s_mul_dt; }
      }
      HE_TRY(launch_sgemm(inputs[a_slot], inputs[b_slot], outputs[0], s_in_dt, s_out_dt, core.batch, core.M, core.N, core.K,
                          cfg.a_mn, cfg.b_mn, s_bias >= 0 ? inputs[s_bias] : nullptr, s_bias_dt, s_act, axpy, stream));
      last_launches = 1;
      return HE_OK;
    }
    float* ws = reinterpret_cast<float*>(workspace);
    if (workspace_bytes > 0 && !workspace) HE_FAIL(HE_ERR_WORKSPACE, "fused matmul launch: this plan needs a %zu-byte workspace", workspace_bytes);
    CUtensorMap ta, tb, tm;
    memset(&tm, 0, sizeof tm);
    const void* a_ptr = inputs[a_slot];
    GemmLaunchCfg cfg = this->cfg;
    int extra_launches = 0;
    if (materialise_a) {
      void* a_prime = reinterpret_cast<char*>(workspace) + ws_aprime_off;
      const void* ew_in[3] = {inputs[mask_slot], inputs[a_slot], nullptr};   // a * relu(b): mask * relu(A)
      if ((reinterpret_cast<uintptr_t>(ew_in[0]) | reinterpret_cast<uintptr_t>(ew_in[1])) & 15)
        HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: operand pointer is not 16-byte aligned");
      HE_TRY(launch_dense_elementwise(EW_MUL_RELU, core.ab_format == 1 ? HE_BF16 : HE_F16, ew_in, a_prime,
                                      (unsigned long long)core.batch * core.M * core.K, 0.0f, ctx_sm_count(ctx), stream));
      a_ptr = a_prime;
      cfg.ml = ML_NONE;
      extra_launches = 1;
    }
    const void* b_ptr = inputs[b_slot];
    for (int side = 0; side < 2; ++side) {
      if (!pad_pitch[side]) continue;
      // stored matrix: rows x cols with cols contiguous
      const bool mn = side == 0 ? cfg.a_mn : cfg.b_mn;
      const int64_t R = side == 0 ? core.M : core.N;
      const int64_t rows = (mn ? core.K : R) * core.batch, cols = mn ? R : core.K;
      void* dst = reinterpret_cast<char*>(workspace) + ws_pad_off[side];
      HE_TRY(launch_pad_rows(side == 0 ? a_ptr : b_ptr, dst, rows, cols, pad_pitch[side], stream));
      (side == 0 ? a_ptr : b_ptr) = dst;
      ++extra_launches;
    }
    if (f8) {
      const int64_t kp = (core.K + 15) / 16 * 16;
      void* a8 = reinterpret_cast<char*>(workspace) + ws_f8_off[0];
      void* b8 = reinterpret_cast<char*>(workspace) + ws_f8_off[1];
      HE_TRY(launch_to_f8(a_ptr, f8_src_dt[0], f8_src_mn[0], a8, core.batch, core.M, core.K, kp, f8 & 2, stream));
      HE_TRY(launch_to_f8(b_ptr, f8_src_dt[1], f8_src_mn[1], b8, core.batch, core.N, core.K, kp, f8 & 4, stream));
      extra_launches += 2;
      HE_TRY(make_f8_tmap(&ta, a8, core.M, core.K, kp, core.batch, kBM));
      HE_TRY(make_f8_tmap(&tb, b8, core.N, core.K, kp, core.batch, cfg.two_cta ? 128 : cfg.bn));
    } else {
    HE_TRY(make_operand_tmap(&ta, a_ptr, core.ab_format, cfg.a_mn, core.M, core.K, core.batch, kBM, pad_pitch[0]));
    HE_TRY(make_operand_tmap(&tb, b_ptr, core.ab_format, cfg.b_mn, core.N, core.K, core.batch, cfg.two_cta ? 128 : cfg.bn, pad_pitch[1]));
    }
    if (mask_slot >= 0 && !materialise_a) HE_TRY(make_operand_tmap(&tm, inputs[mask_slot], core.ab_format, cfg.a_mn, core.M, core.K, core.batch, kBM));
    GemmCore c = core;
    c.status = ctx ? ctx->d_status : nullptr;
    if (kind == EpiKind::Flex) {
      GemmParams<EpiFlexParams> p;
      p.tma_a = ta; p.tma_b = tb; p.tma_mask = tm;
      p.core = c;
      p.epi = flex;
      p.epi.out = outputs[f_y];
      p.epi.out_z = f_z >= 0 ? outputs[f_z] : nullptr;
      p.epi.bias = f_bias >= 0 ? inputs[f_bias] : nullptr;
      p.epi.resid = f_resid >= 0 ? inputs[f_resid] : nullptr;
      p.epi.gate_in = f_gate >= 0 ? inputs[f_gate] : nullptr;
      p.epi.colsum_partials = ws ? ws + ws_col_off[0] : nullptr;
      bool vec = c.N % 8 == 0;
      const void* ptrs[] = {p.epi.out, p.epi.out_z, p.epi.resid, p.epi.gate_in};
      bool vec32 = c.N % 16 == 0;
      for (const void* q : ptrs) {
        vec = vec && ((uintptr_t)q % 16 == 0);
        vec32 = vec32 && ((uintptr_t)q % 32 == 0);
      }
      p.epi.vec_ok = vec ? (vec32 ? 2 : 1) : 0;
      p.epi.bias_vec = (c.N % 8 == 0 && (uintptr_t)p.epi.bias % 16 == 0) ? 1 : 0;
      HE_TRY(launch_gemm_flex(cfg, p, stream));
      last_launches = 1 + extra_launches;
      if (flex.colsum_src != 0) {
        HE_TRY(launch_colsum_finalize(ws + ws_col_off[0], (float*)outputs[f_colsum], c.batch, c.tiles_m, c.N, stream));
        ++last_launches;
      }
      return HE_OK;
    }
    if (kind == EpiKind::C3) {
      GemmParams<EpiC3Params> p;
      p.tma_a = ta; p.tma_b = tb; p.tma_mask = tm;
      p.core = c;
      p.epi = c3;
      p.epi.mask = inputs[r3.mask];
      p.epi.y = inputs[r3.y];
      p.epi.b1 = inputs[r3.b1];
      p.epi.b2 = inputs[r3.b2];
      p.epi.e1 = r3.e1 >= 0 ? inputs[r3.e1] : nullptr;
      p.epi.e2 = r3.e2 >= 0 ? inputs[r3.e2] : nullptr;
      p.epi.out_gt = outputs[r3.gt];
      p.epi.out_gz1 = outputs[r3.gz1];
      p.epi.db2_partials = ws + ws_col_off[0];
      p.epi.db1_partials = ws + ws_col_off[1];
      p.epi.loss_partials = ws + ws_scalar_off;
      bool vec = c.N % 8 == 0;
      const void* ptrs[] = {p.epi.mask, p.epi.y, p.epi.e1, p.epi.e2, p.epi.out_gt, p.epi.out_gz1};
      bool vec32 = c.N % 16 == 0;
      for (const void* q : ptrs) {
        vec = vec && ((uintptr_t)q % 16 == 0);
        vec32 = vec32 && ((uintptr_t)q % 32 == 0);
      }
      p.epi.vec_ok = vec ? (vec32 ? 2 : 1) : 0;
      p.epi.bias_vec = (c.N % 8 == 0 && (uintptr_t)p.epi.b1 % 16 == 0 && (uintptr_t)p.epi.b2 % 16 == 0) ? 1 : 0;
      HE_TRY(launch_gemm_c3(cfg, p, stream));
      HE_TRY(launch_readme_finalize(ws + ws_col_off[0], (float*)outputs[r3.db2], ws + ws_col_off[1], (float*)outputs[r3.db1], c.batch, c.tiles_m,
                                    c.N, ws + ws_scalar_off, (float*)outputs[r3.loss], c.num_tiles, stream));
      last_launches = 2 + extra_launches;
      return HE_OK;
    }
    GemmParams<EpiProgramParams> p;
    p.tma_a = ta; p.tma_b = tb; p.tma_mask = tm;
    p.core = c;
    p.epi.prog = prog.prog;
    for (int i = 0; i < n_inputs; ++i) p.epi.prog.in[i] = inputs[i];
    for (int i = 0; i < n_outputs; ++i) p.epi.prog.out[i] = outputs[i];
    p.epi.n_red = pr_n_red;
    p.epi.n_col = pr_n_col;
    p.epi.col_slot[0] = pr_col_slot[0];
    p.epi.col_slot[1] = pr_col_slot[1];
    p.epi.rows_total = c.batch * c.M;
    for (int s = 0; s < 4; ++s) {
      p.epi.red_kind[s] = pr_kind[s];
      p.epi.red_op[s] = pr_op[s];
      p.epi.red_partials[s] = s < pr_n_red ? ws + pr_off[s] : nullptr;
    }
    HE_TRY(launch_gemm_program(cfg, p, stream));
    last_launches = 1 + extra_launches;
    for (int s = 0; s < pr_n_red; ++s) {
      float* dst = reinterpret_cast<float*>(outputs[pr_out[s]]);
      if (pr_kind[s] == 0) {
        // [batch][tile_m][N] partials; folding the batch in just lengthens the tile axis
        if (pr_fold_batch[s]) HE_TRY(launch_colsum_finalize(ws + pr_off[s], dst, 1, c.batch * c.tiles_m, c.N, stream, pr_op[s], pr_scale[s]));
        else HE_TRY(launch_colsum_finalize(ws + pr_off[s], dst, c.batch, c.tiles_m, c.N, stream, pr_op[s], pr_scale[s]));
      } else if (pr_kind[s] == 1) {
        HE_TRY(launch_colsum_finalize(ws + pr_off[s], dst, 1, pr_row_slots, c.batch * c.M, stream, pr_op[s], pr_scale[s]));   // [slot][batch * M]
      } else {
        HE_TRY(launch_scalar_finalize(ws + pr_off[s], dst, c.num_tiles, stream, pr_op[s], pr_scale[s]));
      }
      ++last_launches;
    }
    return HE_OK;
  }
};

}  // namespace

namespace {
int32_t plan_fused_matmul_core(he_ctx* ctx, const Graph& g, he_plan** out, int* tier_only);

// Pointwise sub-DAG that computes `node`, as a graph of its own: ancestors keep their order, input
// slots are the caller's slots that the sub-DAG reads (`slots`), the single output is `node`.
int32_t extract_operand_graph(const Graph& g, int node, Graph* sub, std::vector<int>* slots) {
  std::vector<char> used(g.nodes.size(), 0);
  std::vector<int> stack{node};
  while (!stack.empty()) {
    const int i = stack.back();
    stack.pop_back();
    if (used[i]) continue;
    used[i] = 1;
    const he_node& n = g.nodes[i];
    if (n.kind == HE_OP_MATMUL) HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: a matmul operand depends on another matmul");
    if (n.kind == HE_OP_REDUCE) HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: a reduction on the operand side cannot be fused");
    for (int k = 0; k < 3; ++k)
      if (n.in[k] >= 0) stack.push_back(n.in[k]);
  }
  std::vector<int> remap(g.nodes.size(), -1);
  for (size_t i = 0; i < g.nodes.size(); ++i) {
    if (!used[i]) continue;
    he_node n = g.nodes[i];
    for (int k = 0; k < 3; ++k)
      if (n.in[k] >= 0) n.in[k] = remap[n.in[k]];
    remap[i] = (int)sub->nodes.size();
    sub->nodes.push_back(n);
  }
  for (size_t k = 0; k < g.inputs.size(); ++k)
    if (used[g.inputs[k]]) {
      sub->inputs.push_back(remap[g.inputs[k]]);
      slots->push_back((int)k);
    }
  sub->outputs.push_back(remap[node]);
  return HE_OK;
}

// A fused matmul whose A and / or B operand is a pointwise expression beyond what the kernels apply
// in their mainloop (helium-kernel-generator accepts Constant / Unary / Binary / ChangeDataType /
// Reshape / SwapDims chains there, generators/matmul.rs:234-264).  The expression is evaluated once
// by a pointwise plan into the workspace and the inner plan sees it as one more input.
struct PrologueMatmulPlan : he_plan {
  std::unique_ptr<he_plan> inner;
  int n_caller_inputs = 0;
  struct Pro {
    std::unique_ptr<he_plan> plan;
    std::vector<int> slots;   // caller input slots, in the pointwise plan's input order
    size_t off = 0;           // bytes into the workspace
  };
  std::vector<Pro> pros;      // in the order their results were appended to the inner plan's inputs

  int32_t set_fault_injection(uint32_t wait_limit_us, int32_t withhold_loads) override {
    return inner->set_fault_injection(wait_limit_us, withhold_loads);
  }

  int32_t launch(const void* const* inputs, void* const* outputs, void* workspace, cudaStream_t stream) override {
    if (!workspace) HE_FAIL(HE_ERR_WORKSPACE, "fused matmul launch: this plan needs a %zu-byte workspace", workspace_bytes);
    std::vector<const void*> ext(inputs, inputs + n_caller_inputs);
    last_launches = 0;
    for (Pro& pr : pros) {
      std::vector<const void*> pin;
      for (int sl : pr.slots) {
        if (!inputs[sl]) HE_FAIL(HE_ERR_INVALID, "fused matmul launch: input %d is null", sl);
        pin.push_back(inputs[sl]);
      }
      void* dst = reinterpret_cast<char*>(workspace) + pr.off;
      void* pout[1] = {dst};
      HE_TRY(pr.plan->launch(pin.data(), pout, nullptr, stream));
      last_launches += pr.plan->last_launches;
      ext.push_back(dst);
    }
    HE_TRY(inner->launch(ext.data(), outputs, inner->workspace_bytes ? workspace : nullptr, stream));
    last_launches += inner->last_launches;
    return HE_OK;
  }
};
}  // namespace

// helium's front end spells a reduction over the rows of y as swap_dims(y) -> Reduce{depth 1}
// (-> reshape): "move the axis last, reduce trailing dims" (helium/src/tensor.rs:83-142).  The GEMM
// epilogue walks y in its own layout, so those leaves are rewritten to the equivalent reduction
// over y's row axis; the output bytes are the same ([.., N, 1] and [.., 1, N] are both N contiguous
// values per batch).
Graph normalise_reduction_leaves(const Graph& g) {
  Graph o = g;
  for (int& leaf : o.outputs) {
    if (o.nodes[leaf].kind == HE_OP_RESHAPE) {
      const int src = o.nodes[leaf].in[0];
      if (src >= 0 && o.nodes[src].kind == HE_OP_REDUCE && num_elements(o.nodes[src]) == num_elements(o.nodes[leaf])) leaf = src;
    }
    he_node& R = o.nodes[leaf];
    if (R.kind != HE_OP_REDUCE || R.in[0] < 0) continue;
    const he_node& S = o.nodes[R.in[0]];
    if (S.kind != HE_OP_SWAP_DIMS || S.rank < 2) continue;
    const int lo = std::min(S.axis_a, S.axis_b), hi = std::max(S.axis_a, S.axis_b);
    if (lo != S.rank - 2 || hi != S.rank - 1) continue;
    const he_node& V = o.nodes[S.in[0]];
    const uint32_t b_lo = 1u << lo, b_hi = 1u << hi;
    uint32_t axes = R.axes & ~(b_lo | b_hi);
    if (R.axes & b_lo) axes |= b_hi;
    if (R.axes & b_hi) axes |= b_lo;
    R.in[0] = S.in[0];
    R.axes = axes;
    R.rank = V.rank;
    for (int k = 0; k < V.rank; ++k) R.shape[k] = ((axes >> k) & 1u) ? 1 : V.shape[k];
  }
  return o;
}

int32_t plan_fused_matmul(he_ctx* ctx, const Graph& g_in, he_plan** out, int* tier_only) {
  const Graph g = normalise_reduction_leaves(g_in);
  int mm = -1;
  for (int i = 0; i < (int)g.nodes.size(); ++i)
    if (g.nodes[i].kind == HE_OP_MATMUL && mm < 0) mm = i;
  if (mm < 0) return plan_fused_matmul_core(ctx, g, out, tier_only);   // reports the error
  const OperandInfo A = trace_operand(g, g.nodes[mm].in[0], false), B = trace_operand(g, g.nodes[mm].in[1], false);
  // Operand-side expressions run either inside the kernel's mainloop (transform warps rewrite the tile in
  // shared memory: the hand-written relu(A) * mask rewrite, or a generic program of unary steps with at most
  // one elementwise multiply / add by a second tensor) or as a pointwise pre-pass that writes the operand once.
  // The in-kernel rewrite is repeated for every tile across the other dimension and slows the mainloop, so
  // it is chosen when that repetition is short (same cost rule as for relu * mask, see choose_mainloop), when
  // HE_GEMM_MAINLOOP=fused forces it, and never for shapes / dtypes the tensor-core path does not take.
  const he_node& M0 = g.nodes[mm];
  const int64_t Md = M0.shape[M0.rank - 2], Kd = g.nodes[M0.in[0]].shape[M0.rank - 1], Nd = M0.shape[M0.rank - 1];
  int64_t batch0 = 1;
  for (int k = 0; k < M0.rank - 2; ++k) batch0 *= M0.shape[k];
  const char* ml_env = getenv("HE_GEMM_MAINLOOP");
  auto in_kernel_ok = [&](const OperandInfo& X, bool is_a) {
    if (!X.ok || X.pure()) return false;
    const int dt = g.nodes[X.root].dtype;
    // both MMA operands must have the stored tensor's 2-byte type (the other one may come out of a pre-pass)
    if ((dt != HE_BF16 && dt != HE_F16) || g.nodes[M0.in[0]].dtype != dt || g.nodes[M0.in[1]].dtype != dt) return false;
    if (X.mask >= 0 && (g.nodes[X.mask].dtype != dt || !is_a)) return false;
    if ((int)X.steps.size() > kMlMaxSteps) return false;
    if ((A.transposed ? Md : Kd) % 8 != 0 || (B.transposed ? Kd : Nd) % 8 != 0) return false;
    return true;
  };
  auto prefers_kernel = [&](bool is_a) {
    if (ml_env) return ml_env[0] == 'f';
    // repetition count of the rewrite = tiles across the other dimension; the pre-pass costs one more pass over the operand
    const double gemm_us = 2.0 * batch0 * Md * (double)Nd * Kd / 1.3e9;
    const double bytes = 3.0 * batch0 * (is_a ? Md : Nd) * (double)Kd * 2.0;
    return 0.7 * gemm_us <= bytes / 4.5e6 + 5.0;
  };
  bool fusable_a = A.ok;
  if (A.ok && !A.pure()) {
    if (A.relu_mask()) fusable_a = in_kernel_ok(A, true) && g.nodes[A.root].dtype == HE_BF16 && B.pure();   // materialise-or-fuse is decided in the core planner
    else fusable_a = in_kernel_ok(A, true) && prefers_kernel(true);
  }
  bool fusable_b = B.ok;
  if (B.ok && !B.pure()) fusable_b = in_kernel_ok(B, false) && prefers_kernel(false) && !(A.ok && A.relu_mask());
  bool pro_a = !fusable_a, pro_b = !fusable_b;
  if (!pro_a && !pro_b) {
    const int32_t st = plan_fused_matmul_core(ctx, g, out, tier_only);
    const bool generic = (A.ok && !A.pure() && !A.relu_mask()) || (B.ok && !B.pure());
    if (st == HE_OK || !generic) return st;
    // the generic in-kernel rewrite is not compiled for this epilogue family: evaluate the operands by a pre-pass
    set_error("");
    pro_a = !A.pure();
    pro_b = !B.pure();
  }

  // replace each such operand by a virtual input (same node index, so the list stays topological)
  Graph g2 = g;
  auto plan = std::make_unique<PrologueMatmulPlan>();
  plan->ctx = ctx;
  plan->n_caller_inputs = (int)g.inputs.size();
  std::string note;
  size_t extra = 0;
  for (int side = 0; side < 2; ++side) {
    if (!(side == 0 ? pro_a : pro_b)) continue;
    const int node = g.nodes[mm].in[side];
    const he_node& on = g.nodes[node];
    PrologueMatmulPlan::Pro pr;
    Graph sub;
    HE_TRY(extract_operand_graph(g, node, &sub, &pr.slots));
    he_plan* pp = nullptr;
    int tier = 0;
    HE_TRY(plan_pointwise(ctx, sub, tier_only ? nullptr : &pp, tier_only ? &tier : nullptr));
    pr.plan.reset(pp);
    pr.off = extra;   // relative to the end of the inner workspace, fixed up below
    extra += ((size_t)num_elements(on) * (on.dtype == HE_F32 ? 4 : 2) + 255) / 256 * 256;
    he_node in{};
    in.kind = HE_OP_INPUT;
    in.dtype = on.dtype;
    in.rank = on.rank;
    for (int k = 0; k < on.rank; ++k) in.shape[k] = on.shape[k];
    in.in[0] = in.in[1] = in.in[2] = -1;
    g2.nodes[node] = in;
    g2.inputs.push_back(node);
    if (pp) note += std::string(", operand ") + (side == 0 ? "A" : "B") + " evaluated by a pre-pass (" + pp->description + ")";
    plan->pros.push_back(std::move(pr));
  }
  he_plan* inner = nullptr;
  int inner_tier = 0;
  HE_TRY(plan_fused_matmul_core(ctx, g2, tier_only ? nullptr : &inner, tier_only ? &inner_tier : nullptr));
  if (tier_only) {
    *tier_only = inner_tier > 0 ? 1 : 0;   // runs, but the operand side is not fused into the mainloop
    return HE_OK;
  }
  plan->inner.reset(inner);
  const size_t base = (inner->workspace_bytes + 255) / 256 * 256;
  for (auto& pr : plan->pros) pr.off += base;
  plan->workspace_bytes = base + extra;
  plan->description = inner->description + note;
  *out = plan.release();
  return HE_OK;
}

namespace {
int32_t plan_fused_matmul_core(he_ctx* ctx, const Graph& g, he_plan** out, int* tier_only) {
  int mm = -1;
  for (int i = 0; i < (int)g.nodes.size(); ++i)
    if (g.nodes[i].kind == HE_OP_MATMUL) {
      if (mm >= 0) HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: more than one matmul in the subgraph");
      mm = i;
    }
  if (mm < 0) HE_FAIL(HE_ERR_INVALID, "fused matmul: subgraph has no matmul (matmul.rs:222-232)");
  const he_node& M = g.nodes[mm];
  const int r = M.rank;
  const OperandInfo A = trace_operand(g, M.in[0], false), B = trace_operand(g, M.in[1], false);
  if (!A.ok || !B.ok)
    HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: operand side uses ops outside {cast, reshape, transpose, unary, multiply / add by one tensor or a constant}");
  if (B.mask >= 0) HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: a second tensor on the B operand side is not implemented in the mainloop");
  const he_node& An = g.nodes[A.root];
  const he_node& Bn = g.nodes[B.root];

  MatmulPlan* plan = new MatmulPlan();
  std::unique_ptr<MatmulPlan> guard(plan);
  plan->ctx = ctx;
  GemmCore& c = plan->core;
  c.M = (int)M.shape[r - 2];
  c.N = (int)M.shape[r - 1];
  c.K = (int)g.nodes[M.in[0]].shape[r - 1];
  int64_t batch = 1;
  for (int k = 0; k < r - 2; ++k) batch *= M.shape[k];
  c.batch = (int)batch;
  if (num_elements(M) >= (1ll << 31)) HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: output exceeds the 32-bit index range");
  auto slot_of = [&](int node) {
    for (size_t k = 0; k < g.inputs.size(); ++k)
      if (g.inputs[k] == node) return (int)k;
    return -1;
  };
  plan->a_slot = slot_of(A.root);
  plan->b_slot = slot_of(B.root);
  plan->mask_slot = A.mask >= 0 ? slot_of(A.mask) : -1;
  plan->n_inputs = (int)g.inputs.size();
  plan->n_outputs = (int)g.outputs.size();
  plan->cfg.a_mn = A.transposed;
  plan->cfg.b_mn = !B.transposed;  // helium stores B as [K, N] row-major = N-major
  if (A.pure() && B.pure()) plan->cfg.ml = ML_NONE;
  else if (A.relu_mask() && B.pure()) plan->cfg.ml = ML_RELU_MASK;
  else plan->cfg.ml = ML_GENERIC | (A.mask >= 0 ? ML_MASK : 0);
  auto fill_prog = [](const OperandInfo& X, MlProg* P) -> bool {
    memset(P, 0, sizeof *P);
    if ((int)X.steps.size() > kMlMaxSteps) return false;
    P->n = (int)X.steps.size();
    for (int i = 0; i < P->n; ++i) P->s[i] = X.steps[i];
    return true;
  };
  if (!fill_prog(A, &c.ml_a) || !fill_prog(B, &c.ml_b))
    HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: operand-side chains of more than %d steps are not fused into the mainloop", kMlMaxSteps);
  plan->ml_b = !B.pure();

  // ---- SIMT path: f32 operands (exact f32 products; the precision setting is a minimum,
  // precision.rs:3-9) and 2-byte operands that break the TMA pitch rules
  auto try_simt = [&](const char* why) -> int32_t {
    if (plan->cfg.ml != ML_NONE) HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: mainloop fusion needs the tensor-core path (%s)", why);
    PwCompiled pc;
    PwCanon canon;
    HE_TRY(canon_of(g, mm, &pc, &canon));
    int bias_slot = -1, act = 0, axpy_slot = -1, mul_slot = -1, axpy_neg = 0;
    float axpy_alpha = 1.0f;
    bool has_axpy = false;
    bool ok = false;
    if (canon.text == "store(A);") ok = true;
    else if (canon.text == "store(sum(A,I0:R));") { ok = true; bias_slot = canon.slot_order[0]; }
    else if (canon.text == "store(u8(sum(A,I0:R)));") { ok = true; bias_slot = canon.slot_order[0]; act = 1; }
    else if (canon.text == "store(u8(A));") { ok = true; act = 1; }
    else {
      // scaled / negated / accumulated forms: [I:F +] [-] (A * (K | I:F)) -- the SGD update of a weight
      // gradient, w + (-(g * lr)) (helium/src/optimizer/sgd.rs), and every partial subgraph that greedy
      // pairwise fusion passes through on the way there.  A constant is spelled K<8 hex digits>.
      std::string t = canon.text;
      auto eat = [&](const char* lit) {
        const size_t n = strlen(lit);
        if (t.compare(0, n, lit) != 0) return false;
        t.erase(0, n);
        return true;
      };
      auto eat_full_input = [&](int* slot) {   // I<k>:F
        if (t.size() < 4 || t[0] != 'I') return false;
        size_t q = 1;
        int k = 0;
        while (q < t.size() && t[q] >= '0' && t[q] <= '9') k = k * 10 + (t[q++] - '0');
        if (q == 1 || t.compare(q, 2, ":F") != 0 || k >= (int)canon.slot_order.size()) return false;
        *slot = canon.slot_order[k];
        t.erase(0, q + 2);
        return true;
      };
      bool good = eat("store(");
      const bool has_sum = good && eat("sum(");
      if (has_sum) good = eat_full_input(&axpy_slot) && eat(",");
      const bool neg = good && eat("u1(");
      good = good && eat("prod(A,");
      if (good) {
        if (t.size() >= 9 && t[0] == 'K') {
          char* end = nullptr;
          const std::string hex = t.substr(1, 8);
          const uint32_t b32 = (uint32_t)strtoul(hex.c_str(), &end, 16);
          good = end == hex.c_str() + 8;
          memcpy(&axpy_alpha, &b32, 4);
          t.erase(0, 9);
        } else {
          good = eat_full_input(&mul_slot);
        }
      }
      good = good && eat(")") && (!neg || eat(")")) && (!has_sum || eat(")")) && eat(");") && t.empty();
      if (good) { ok = true; axpy_neg = neg; has_axpy = true; }
      else { axpy_slot = mul_slot = -1; }
    }
    const int odt = g.nodes[g.outputs[0]].dtype;
    for (int sl : {axpy_slot, mul_slot})
      if (ok && sl >= 0 && dclass(g.nodes[g.inputs[sl]].dtype) != DClass::Float) ok = false;
    if (!ok || dclass(odt) != DClass::Float || (bias_slot >= 0 && dclass(g.nodes[g.inputs[bias_slot]].dtype) != DClass::Float))
      HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: the SIMT path (%s) supports only store / +bias / relu / axpy epilogues", why);
    if (tier_only) { *tier_only = 2; return HE_OK; }
    plan->kind = EpiKind::Sgemm;
    plan->s_bias = bias_slot;
    plan->s_act = act;
    plan->s_in_dt = An.dtype;
    plan->s_out_dt = odt;
    plan->s_bias_dt = bias_slot >= 0 ? g.nodes[g.inputs[bias_slot]].dtype : HE_F32;
    plan->s_axpy = has_axpy;
    plan->s_resid = axpy_slot;
    plan->s_resid_dt = axpy_slot >= 0 ? g.nodes[g.inputs[axpy_slot]].dtype : HE_F32;
    plan->s_mul = mul_slot;
    plan->s_mul_dt = mul_slot >= 0 ? g.nodes[g.inputs[mul_slot]].dtype : HE_F32;
    plan->s_alpha = axpy_alpha;
    plan->s_negate = axpy_neg;
    plan->description = std::string("fused matmul: SIMT FFMA kernel, 64x64 tiles (") + why + (has_axpy ? ", scale/accumulate epilogue)" : ")");
    *out = guard.release();
    return HE_OK;
  };
  // 8-bit multiplication: the setting is a minimum (precision.rs:3-9), so small products stay at the operand
  // precision; from ~4 GFLOP on the two conversion passes are cheap against a mainloop that does twice the math
  // per byte.  HE_GEMM_F8=native|operand forces either.
  {
    const int pk = HE_PREC_KIND(M.sub_op);
    const bool same = An.dtype == Bn.dtype && (An.dtype == HE_BF16 || An.dtype == HE_F16 || An.dtype == HE_F32);
    bool native = (pk == HE_PREC_F8_F32 || pk == HE_PREC_F8_F16) && same && plan->cfg.ml == ML_NONE &&
                  2.0 * c.batch * c.M * (double)c.N * c.K >= 4294967296.0;
    if (const char* e = getenv("HE_GEMM_F8"))
      native = (pk == HE_PREC_F8_F32 || pk == HE_PREC_F8_F16) && same && plan->cfg.ml == ML_NONE && (e[0] == 'n' ? true : e[0] == 'o' ? false : native);
    if (native) {
      plan->f8 = 1 | (((M.sub_op >> 8) & 1) << 1) | (((M.sub_op >> 12) & 1) << 2);
      plan->f8_src_mn[0] = plan->cfg.a_mn; plan->f8_src_mn[1] = plan->cfg.b_mn;
      plan->f8_src_dt[0] = An.dtype; plan->f8_src_dt[1] = Bn.dtype;
      plan->cfg.a_mn = plan->cfg.b_mn = false;   // the copies are K-major
      plan->cfg.ml = ML_F8;                      // kernels instantiated for 8-bit tiles
      c.f8 = plan->f8;
    }
  }
  if (!plan->f8 && An.dtype == HE_F32 && Bn.dtype == HE_F32) return try_simt("f32 operands");
  if (!plan->f8 && !((An.dtype == HE_BF16 && Bn.dtype == HE_BF16) || (An.dtype == HE_F16 && Bn.dtype == HE_F16)))
    HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: operands must both be bf16, both f16 or both f32 (got %s x %s)", dtype_name(An.dtype), dtype_name(Bn.dtype));
  c.ab_format = An.dtype == HE_BF16 ? 1 : 0;
  c.group_m = 1;
  c.wait_limit_us = ptx::kDefaultWaitLimitUs;
  c.withhold_loads = 0;
  {
    const char* e = getenv("HE_GEMM_K_SERPENTINE");
    c.k_serpentine = e ? (e[0] == '1') : 1;
  }
  if (plan->cfg.ml == ML_RELU_MASK && (An.dtype != HE_BF16 || g.nodes[A.mask].dtype != HE_BF16))
    HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: the relu * mask mainloop rewrite needs bf16 A and mask");
  if (A.mask >= 0 && g.nodes[A.mask].dtype != An.dtype)
    HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: the second tensor of a mainloop fusion must have the operand's dtype");
  // TMA pitch rules (16-byte multiples).  Small problems off the rules run on the SIMT kernel when its
  // epilogues cover the graph; everything else gets a pitch-padded copy of the offending operand.
  const int64_t a_cols = plan->cfg.a_mn ? c.M : c.K, b_cols = plan->cfg.b_mn ? c.N : c.K;
  std::string pad_note;
  if (!plan->f8 && (a_cols % 8 != 0 || b_cols % 8 != 0)) {
    const double flop = 2.0 * c.batch * c.M * (double)c.N * c.K;
    if (flop < 268435456.0 && plan->cfg.ml == ML_NONE) {
      set_error("");
      const int32_t st = try_simt("operand rows are not multiples of 8 elements, TMA needs 16-byte pitches");
      if (st == HE_OK) return st;
    }
    if (plan->cfg.ml != ML_NONE)
      HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: in-kernel mainloop fusion needs operand rows that are multiples of 8 elements (M=%d N=%d K=%d)", c.M, c.N, c.K);
    if (a_cols % 8 != 0) { plan->pad_pitch[0] = (a_cols + 7) / 8 * 8; pad_note += ", A copied to a 16-byte pitch"; }
    if (b_cols % 8 != 0) { plan->pad_pitch[1] = (b_cols + 7) / 8 * 8; pad_note += ", B copied to a 16-byte pitch"; }
  }

  // ---- epilogue
  PwCompiled pc;
  PwCanon canon;
  HE_TRY(canon_of(g, mm, &pc, &canon));
  if ((int64_t)pc.prog.n_elems != num_elements(M))
    HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: epilogue outputs must have the matmul's element count");

  plan->cfg.bn = 256;
  plan->cfg.two_cta = false;
  auto finish_tiles = [&]() {
    c.tiles_m = (c.M + kBM - 1) / kBM;
    c.tiles_n = (c.N + plan->cfg.bn - 1) / plan->cfg.bn;
    c.k_blocks = plan->f8 ? (c.K + 2 * kBK - 1) / (2 * kBK) : (c.K + kBK - 1) / kBK;   // 128 bytes of K per block
    // Two SMs per 256 x 256 tile whenever there are at least two row tiles to pair up; the
    // environment switch keeps the single-CTA kernel reachable for comparisons.
    const char* force1 = getenv("HE_GEMM_ONE_CTA");
    plan->cfg.two_cta = plan->cfg.bn == 256 && c.tiles_m >= 2 && !(force1 && force1[0] == '1') && !plan->ml_b;   // the B rewrite lives in the single-CTA kernel
    if (plan->cfg.two_cta) {
      const int tiles_m2 = (c.M + 255) / 256;
      c.tiles_m = 2 * tiles_m2;                       // partial-sum rows: the odd CTA of the last pair may be empty
      const int pair_tiles = tiles_m2 * c.tiles_n * c.batch;
      const int pairs = std::max(1, std::min(pair_tiles, ctx_sm_count(ctx) / 2));
      plan->cfg.grid = 2 * pairs;
      // Tail balancing: when the last round of the static schedule would leave more than half of
      // the pairs idle, its tiles are issued as two half-width tiles each (the tile list grows by
      // `rest` entries and the last round keeps 2 * rest pairs busy for about half a tile time).
      const int rest = pair_tiles % pairs;
      const char* no_split = getenv("HE_GEMM_NO_SPLIT");
      if (pair_tiles > pairs && rest > 0 && 2 * rest <= pairs && !(no_split && no_split[0] == '1')) {
        c.split_from = pair_tiles - rest;
        c.split_count = rest;
      } else {
        c.split_from = pair_tiles;
        c.split_count = 0;
      }
      c.num_tiles = 2 * (pair_tiles + c.split_count);  // one scalar partial per CTA tile of the list
      c.group_m = 8;    // 2048 rows of A per group
    } else {
      c.group_m = 16;
      c.split_from = 0;
      c.split_count = 0;
      c.num_tiles = c.tiles_m * c.tiles_n * c.batch;
      plan->cfg.grid = std::max(1, std::min(c.num_tiles, ctx_sm_count(ctx)));
    }
    if (const char* gm = getenv("HE_GEMM_GROUP_M")) c.group_m = std::max(1, atoi(gm));
  };
  // Decide how a mainloop fusion is executed (after the epilogue's own workspace is laid out).
  // Cost model from measurements on B200: the in-kernel rewrite runs the mainloop at about half the
  // plain rate (1316 -> 680-770 TFLOP/s at 4096^3), i.e. it adds ~0.7 x the plain GEMM time; the
  // pre-pass reads A and the mask and writes A' once at ~4.5 TB/s plus a launch.
  auto choose_mainloop = [&]() -> std::string {
    // pitch-padded operand copies live behind the epilogue's own workspace
    for (int side = 0; side < 2; ++side) {
      if (!plan->pad_pitch[side]) continue;
      const bool mn = side == 0 ? plan->cfg.a_mn : plan->cfg.b_mn;
      const int64_t rows = (mn ? c.K : (side == 0 ? c.M : c.N)) * (int64_t)c.batch;
      plan->ws_pad_off[side] = (plan->workspace_bytes + 255) / 256 * 256;
      plan->workspace_bytes = plan->ws_pad_off[side] + (size_t)rows * plan->pad_pitch[side] * 2;
    }
    if (plan->f8) {
      const size_t kp = (size_t)(c.K + 15) / 16 * 16;
      plan->ws_f8_off[0] = (plan->workspace_bytes + 255) / 256 * 256;
      plan->ws_f8_off[1] = (plan->ws_f8_off[0] + (size_t)c.batch * c.M * kp + 255) / 256 * 256;
      plan->workspace_bytes = plan->ws_f8_off[1] + (size_t)c.batch * c.N * kp;
      return std::string(", 8-bit multiplication (A ") + (plan->f8 & 2 ? "E5M2" : "E4M3") + ", B " + (plan->f8 & 4 ? "E5M2" : "E4M3") +
             ": operands rounded once per launch into K-major copies, tcgen05 kind::f8f6f4)";
    }
    if (plan->cfg.ml == ML_NONE) return pad_note;
    if (plan->cfg.ml & ML_GENERIC) return ", generic mainloop rewrite in shared memory";
    const double gemm_us = 2.0 * c.batch * c.M * (double)c.N * c.K / 1.3e9;
    const double bytes = 3.0 * c.batch * c.M * (double)c.K * 2.0;
    const double prepass_us = bytes / 4.5e6 + 5.0;
    bool mat = 0.7 * gemm_us > prepass_us;
    if (const char* e = getenv("HE_GEMM_MAINLOOP")) mat = e[0] == 'm' ? true : e[0] == 'f' ? false : mat;   // "materialise" / "fused"
    if (!mat) return ", mainloop rewrite in shared memory";
    plan->materialise_a = true;
    plan->ws_aprime_off = (plan->workspace_bytes + 255) / 256 * 256;
    plan->workspace_bytes = plan->ws_aprime_off + (size_t)c.batch * c.M * c.K * 2;
    return ", mainloop operand materialised by a pre-pass";
  };
  auto out_dt = [&](int out_idx) { return g.nodes[g.outputs[out_idx]].dtype; };
  auto in_dt = [&](int slot) { return g.nodes[g.inputs[slot]].dtype; };
  char desc[320];

  // (1) Flex catalogue
  for (const FlexPattern& fp : flex_catalogue()) {
    if (fp.canon.text != canon.text) continue;
    auto cand_slot = [&](int pattern_slot) {
      for (size_t k = 0; k < fp.canon.slot_order.size(); ++k)
        if (fp.canon.slot_order[k] == pattern_slot) return canon.slot_order[k];
      return -1;
    };
    auto cand_out = [&](int pattern_out) {
      for (size_t k = 0; k < fp.canon.out_order.size(); ++k)
        if (fp.canon.out_order[k] == pattern_out) return canon.out_order[k];
      return -1;
    };
    if (tier_only) { *tier_only = 2; return HE_OK; }
    plan->kind = EpiKind::Flex;
    plan->f_bias = fp.bias_slot >= 0 ? cand_slot(fp.bias_slot) : -1;
    plan->f_resid = fp.resid_slot >= 0 ? cand_slot(fp.resid_slot) : -1;
    plan->f_gate = fp.gate_slot >= 0 ? cand_slot(fp.gate_slot) : -1;
    plan->f_y = cand_out(fp.y_out);
    plan->f_z = fp.z_out >= 0 ? cand_out(fp.z_out) : -1;
    plan->f_colsum = fp.colsum_out >= 0 ? cand_out(fp.colsum_out) : -1;
    EpiFlexParams& f = plan->flex;
    f.act = fp.combo.act;
    f.gate = fp.combo.gate;
    f.colsum_src = fp.combo.colsum;
    f.out_dt = out_dt(plan->f_y);
    f.z_dt = plan->f_z >= 0 ? out_dt(plan->f_z) : HE_F32;
    f.bias_dt = plan->f_bias >= 0 ? in_dt(plan->f_bias) : HE_F32;
    f.resid_dt = plan->f_resid >= 0 ? in_dt(plan->f_resid) : HE_F32;
    f.gate_dt = plan->f_gate >= 0 ? in_dt(plan->f_gate) : HE_F32;
    const int dts[] = {f.out_dt, f.z_dt, f.bias_dt, f.resid_dt, f.gate_dt};
    for (int dt : dts)
      if (dclass(dt) != DClass::Float) HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: epilogue tensors must be float");
    // a narrow N wastes half of a 256-wide tile
    if (c.N <= 128 && plan->cfg.ml == ML_NONE) plan->cfg.bn = 128;
    finish_tiles();
    if (f.colsum_src != 0) {
      plan->ws_col_off[0] = 0;
      plan->workspace_bytes = (size_t)c.batch * c.tiles_m * c.N * sizeof(float);
    }
    snprintf(desc, sizeof desc,
             "fused matmul tier 2: tcgen05 %sx%dx64, %s-major A, %s-major B, mainloop %d, epilogue flex(bias=%d resid=%d act=%d gate=%d z=%d colsum=%d), grid %d",
             plan->cfg.two_cta ? "2-CTA 256" : "128", plan->cfg.bn, plan->cfg.a_mn ? "M" : "K", plan->cfg.b_mn ? "N" : "K", plan->cfg.ml, plan->f_bias >= 0, plan->f_resid >= 0,
             f.act, f.gate, plan->f_z >= 0, f.colsum_src, plan->cfg.grid);
    plan->description = std::string(desc) + choose_mainloop();
    *out = guard.release();
    return HE_OK;
  }

  // (2) the README graph: find the MulConstant operand, rebuild the pattern with it, compare
  {
    float inv_n = 0.0f;
    bool have = false;
    for (const he_node& n : g.nodes)
      if (n.kind == HE_OP_UNARY && n.sub_op == HE_UN_MUL_CONST && !have) {
        memcpy(&inv_n, &n.const_bits, 4);
        have = true;
      }
    for (int with_e = 0; have && with_e < 2; ++with_e) {
      PwCanon pat;
      C3Roles roles;
      if (!build_c3_pattern(with_e != 0, inv_n, &pat, &roles) || pat.text != canon.text) continue;
      auto cand_slot = [&](int pattern_slot) {
        for (size_t k = 0; k < pat.slot_order.size(); ++k)
          if (pat.slot_order[k] == pattern_slot) return canon.slot_order[k];
        return -1;
      };
      auto cand_out = [&](int pattern_out) {
        for (size_t k = 0; k < pat.out_order.size(); ++k)
          if (pat.out_order[k] == pattern_out) return canon.out_order[k];
        return -1;
      };
      C3Roles rr;
      rr.b1 = cand_slot(roles.b1); rr.b2 = cand_slot(roles.b2); rr.mask = cand_slot(roles.mask); rr.y = cand_slot(roles.y);
      rr.e1 = roles.e1 >= 0 ? cand_slot(roles.e1) : -1;
      rr.e2 = roles.e2 >= 0 ? cand_slot(roles.e2) : -1;
      rr.loss = cand_out(roles.loss); rr.db2 = cand_out(roles.db2); rr.db1 = cand_out(roles.db1);
      rr.gt = cand_out(roles.gt); rr.gz1 = cand_out(roles.gz1);
      const int full_dt = in_dt(rr.mask);
      bool dt_ok = in_dt(rr.y) == full_dt && out_dt(rr.gt) == full_dt && out_dt(rr.gz1) == full_dt &&
                   in_dt(rr.b1) == in_dt(rr.b2) && dclass(full_dt) == DClass::Float && dclass(in_dt(rr.b1)) == DClass::Float;
      if (rr.e1 >= 0) dt_ok = dt_ok && in_dt(rr.e1) == full_dt && in_dt(rr.e2) == full_dt;
      if (!dt_ok) continue;  // falls through to the interpreter tier
      if (plan->cfg.ml & ML_GENERIC) HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: the README epilogue is compiled with the relu * mask mainloop only");
      if (tier_only) { *tier_only = 2; return HE_OK; }
      plan->kind = EpiKind::C3;
      plan->r3 = rr;
      plan->c3.inv_n = inv_n;
      plan->c3.full_dt = full_dt;
      plan->c3.vec_dt = in_dt(rr.b1);
      finish_tiles();
      const size_t col = ((size_t)c.batch * c.tiles_m * c.N + 63) / 64 * 64;
      plan->ws_col_off[0] = 0;
      plan->ws_col_off[1] = col;
      plan->ws_scalar_off = 2 * col;
      plan->workspace_bytes = (2 * col + (size_t)c.num_tiles) * sizeof(float);
      snprintf(desc, sizeof desc,
               "fused matmul tier 2: tcgen05 %sx256x64, %s-major A, %s-major B, mainloop %d, epilogue README graph (loss + 2 column sums + 2 tiles%s), grid %d",
               plan->cfg.two_cta ? "2-CTA 256" : "128", plan->cfg.a_mn ? "M" : "K", plan->cfg.b_mn ? "N" : "K", plan->cfg.ml, with_e ? ", E1/E2" : "", plan->cfg.grid);
      plan->description = std::string(desc) + choose_mainloop();
      *out = guard.release();
      return HE_OK;
    }
  }

  // (3) interpreter tier: any pointwise epilogue without reductions
  {
    PwCompileOptions opt;
    opt.acc_node = mm;
    opt.fuse_fma = true;
    opt.epilogue = true;
    HE_TRY(compile_pointwise(g, opt, &plan->prog));
    if (plan->prog.has_bool_io) HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: bool tensors in the epilogue are not supported");
    // reductions of the interpreted epilogue: Sum over rows, over columns, or over the whole tile
    const PwProgram& EP = plan->prog.prog;
    if (EP.n_reductions > 4) HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: more than 4 reductions in one epilogue");
    for (int i = 0; i < EP.n_instr; ++i) {
      const PwInstr& in = EP.instr[i];
      if (in.op != PW_REDUCE) continue;
      const int s = in.slot2;
      const uint32_t m = in.imm;
      int kind;
      if ((m & 3u) == 3u) {
        if (!(m & 4u) && c.batch != 1)
          HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: a per-item scalar reduction needs batch 1 in the generic epilogue");
        kind = 2;
      } else if ((m & 3u) == 2u) {
        kind = 0;
        plan->pr_fold_batch[s] = (m & 4u) ? 1 : 0;
      } else if (m == 1u) {
        kind = 1;
      } else {
        HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: reduction axes mask %u is not one of rows / columns / item / batch", m);
      }
      plan->pr_kind[s] = kind;
      plan->pr_out[s] = in.slot;
      plan->pr_op[s] = in.sub == HE_RED_MAX ? 1 : in.sub == HE_RED_MIN ? 2 : 0;
      if (in.sub == HE_RED_MEAN) {
        double count = 1.0;
        if (m & 1u) count *= c.N;
        if (m & 2u) count *= c.M;
        if (m & 4u) count *= c.batch;
        plan->pr_scale[s] = (float)(1.0 / count);
      }
      if (kind == 0) {
        if (plan->pr_n_col == 2) HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: at most two column reductions in the generic epilogue");
        plan->pr_col_slot[plan->pr_n_col++] = s;
      }
      plan->pr_n_red = std::max(plan->pr_n_red, s + 1);
    }
    if (tier_only) { *tier_only = 1; return HE_OK; }
    plan->kind = EpiKind::Program;
    finish_tiles();
    {
      size_t off = 0;
      plan->pr_row_slots = c.tiles_n * (plan->cfg.bn / 64);
      for (int s = 0; s < plan->pr_n_red; ++s) {
        plan->pr_off[s] = off;
        const size_t n = plan->pr_kind[s] == 0 ? (size_t)c.batch * c.tiles_m * c.N
                         : plan->pr_kind[s] == 1 ? (size_t)plan->pr_row_slots * c.batch * c.M
                                                 : (size_t)c.num_tiles;
        off += (n + 63) / 64 * 64;
      }
      plan->workspace_bytes = off * sizeof(float);
    }
    snprintf(desc, sizeof desc,
             "fused matmul tier 1: tcgen05 %sx256x64, %s-major A, %s-major B, mainloop %d, interpreted epilogue (%d instr, %d reductions), grid %d",
             plan->cfg.two_cta ? "2-CTA 256" : "128", plan->cfg.a_mn ? "M" : "K", plan->cfg.b_mn ? "N" : "K", plan->cfg.ml, plan->prog.prog.n_instr,
             plan->pr_n_red, plan->cfg.grid);
    plan->description = std::string(desc) + choose_mainloop();
    *out = guard.release();
    return HE_OK;
  }
}

}  // namespace

}  // namespace he
