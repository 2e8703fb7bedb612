// C ABI entry points: context, descriptor validation, plan dispatch, launch.
#include <nvtx3/nvToolsExt.h>
#include "he_internal.h"
#include "pointwise_program.h"

#include <mutex>

namespace he {
namespace {
bool nvtx_enabled() {
  static const bool on = [] {
    const char* e = getenv("HE_NVTX");
    return !(e && e[0] == '0');
  }();
  return on;
}
}  // namespace
TraceRange::TraceRange(const char* name) : on_(nvtx_enabled()) {
  if (on_) nvtxRangePushA(name ? name : "helium_b200");
}
TraceRange::~TraceRange() {
  if (on_) nvtxRangePop();
}
}  // namespace he

namespace he {

static thread_local std::string g_last_error;

void set_error(const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_last_error = buf;
}

const char* dtype_name(int32_t dt) {
  switch (dt) {
    case HE_F16: return "f16";
    case HE_BF16: return "bf16";
    case HE_F32: return "f32";
    case HE_U32: return "u32";
    case HE_BOOL: return "bool";
    default: return "?";
  }
}

static bool same_shape(const he_node& a, const he_node& b) {
  if (a.rank != b.rank) return false;
  for (int i = 0; i < a.rank; ++i)
    if (a.shape[i] != b.shape[i]) return false;
  return true;
}

// Shape / dtype rules of helium_ir::Op::output_descriptor (helium-ir/src/opgraph/op.rs:52-179),
// checked here instead of trusted because the descriptor crosses an FFI boundary.
int32_t parse_graph(const he_graph_desc* desc, Graph* out) {
  if (!desc || !desc->nodes || desc->num_nodes <= 0) HE_FAIL(HE_ERR_INVALID, "empty graph descriptor");
  if (desc->num_nodes > 4096) HE_FAIL(HE_ERR_INVALID, "graph has %d nodes (max 4096)", desc->num_nodes);
  if (!desc->outputs || desc->num_outputs <= 0) HE_FAIL(HE_ERR_INVALID, "graph has no outputs");
  out->nodes.assign(desc->nodes, desc->nodes + desc->num_nodes);
  out->inputs.clear();
  out->outputs.assign(desc->outputs, desc->outputs + desc->num_outputs);
  auto& N = out->nodes;
  for (int i = 0; i < (int)N.size(); ++i) {
    he_node& n = N[i];
    if (n.rank < 0 || n.rank > HE_MAX_RANK) HE_FAIL(HE_ERR_INVALID, "node %d: rank %d out of range", i, n.rank);
    if (!dtype_valid(n.dtype)) HE_FAIL(HE_ERR_INVALID, "node %d: bad dtype %d", i, n.dtype);
    for (int d = 0; d < n.rank; ++d)
      if (n.shape[d] < 0) HE_FAIL(HE_ERR_INVALID, "node %d: negative dim", i);
    int arity = 0;
    switch (n.kind) {
      case HE_OP_INPUT: case HE_OP_CONSTANT: arity = 0; break;
      case HE_OP_UNARY: case HE_OP_CAST: case HE_OP_REDUCE: case HE_OP_BROADCAST:
      case HE_OP_RESHAPE: case HE_OP_SWAP_DIMS: arity = 1; break;
      case HE_OP_BINARY: case HE_OP_COMPARE: case HE_OP_MATMUL: arity = 2; break;
      case HE_OP_SELECT: arity = 3; break;
      default: HE_FAIL(HE_ERR_INVALID, "node %d: unknown op kind %d", i, n.kind);
    }
    for (int k = 0; k < 3; ++k) {
      if (k < arity) {
        if (n.in[k] < 0 || n.in[k] >= i)
          HE_FAIL(HE_ERR_INVALID, "node %d: operand %d = %d is not an earlier node", i, k, n.in[k]);
      } else {
        n.in[k] = -1;
      }
    }
    const he_node* a = arity > 0 ? &N[n.in[0]] : nullptr;
    const he_node* b = arity > 1 ? &N[n.in[1]] : nullptr;
    switch (n.kind) {
      case HE_OP_INPUT: out->inputs.push_back(i); break;
      case HE_OP_CONSTANT: break;
      case HE_OP_UNARY:
        if (!same_shape(n, *a) || n.dtype != a->dtype)
          HE_FAIL(HE_ERR_INVALID, "node %d: unary output descriptor must equal its input's", i);
        if (dclass(n.dtype) != DClass::Float)
          HE_FAIL(HE_ERR_INVALID, "node %d: unary ops need a float tensor", i);
        break;
      case HE_OP_BINARY:
        if (!same_shape(n, *a) || n.dtype != a->dtype)
          HE_FAIL(HE_ERR_INVALID, "node %d: binary output descriptor must equal lhs's", i);
        if (num_elements(*a) != num_elements(*b))
          HE_FAIL(HE_ERR_INVALID, "node %d: binary operands differ in element count", i);
        if (dclass(a->dtype) != dclass(b->dtype))
          HE_FAIL(HE_ERR_INVALID, "node %d: binary operands differ in data class", i);
        if (n.sub_op >= HE_BIN_AND && n.sub_op <= HE_BIN_XOR) {
          if (dclass(n.dtype) == DClass::Float)
            HE_FAIL(HE_ERR_INVALID, "node %d: and/or/xor need bool or u32 operands", i);
        } else if (dclass(n.dtype) == DClass::Bool) {
          HE_FAIL(HE_ERR_INVALID, "node %d: arithmetic on bool tensors", i);
        }
        break;
      case HE_OP_CAST:
        if (!same_shape(n, *a)) HE_FAIL(HE_ERR_INVALID, "node %d: cast changes shape", i);
        break;
      case HE_OP_REDUCE: {
        if (n.dtype != HE_F32) HE_FAIL(HE_ERR_INVALID, "node %d: reduce output must be f32", i);
        if (dclass(a->dtype) != DClass::Float) HE_FAIL(HE_ERR_INVALID, "node %d: reduce of non-float", i);
        if (n.axes == 0 || (a->rank < 32 && (n.axes >> a->rank) != 0))
          HE_FAIL(HE_ERR_INVALID, "node %d: reduce axes mask 0x%x invalid for rank %d", i, n.axes, a->rank);
        // Form A (helium-ir): last d dims collapsed into one dim of size 1.
        int d = __builtin_popcount(n.axes);
        bool trailing = n.axes == (((1u << d) - 1u) << (a->rank - d));
        bool form_a = trailing && n.rank == a->rank - d + 1 && n.shape[n.rank - 1] == 1;
        for (int k = 0; form_a && k < n.rank - 1; ++k) form_a = n.shape[k] == a->shape[k];
        // Form B (playground): rank kept, reduced dims become 1.
        bool form_b = n.rank == a->rank;
        for (int k = 0; form_b && k < n.rank; ++k)
          form_b = n.shape[k] == ((n.axes >> k) & 1u ? 1 : a->shape[k]);
        if (!form_a && !form_b) HE_FAIL(HE_ERR_INVALID, "node %d: reduce output shape inconsistent with axes", i);
        break;
      }
      case HE_OP_BROADCAST: {
        if (n.dtype != a->dtype) HE_FAIL(HE_ERR_INVALID, "node %d: broadcast changes dtype", i);
        if (n.rank < a->rank) HE_FAIL(HE_ERR_INVALID, "node %d: broadcast lowers rank", i);
        int pad = n.rank - a->rank;
        for (int k = 0; k < n.rank; ++k) {
          int64_t in_dim = k < pad ? 1 : a->shape[k - pad];
          if (in_dim != n.shape[k] && in_dim != 1)
            HE_FAIL(HE_ERR_INVALID, "node %d: broadcast of a dim of size %lld", i, (long long)in_dim);
        }
        break;
      }
      case HE_OP_RESHAPE:
        if (n.dtype != a->dtype || num_elements(n) != num_elements(*a))
          HE_FAIL(HE_ERR_INVALID, "node %d: reshape changes element count or dtype", i);
        break;
      case HE_OP_SWAP_DIMS: {
        if (n.dtype != a->dtype || n.rank != a->rank) HE_FAIL(HE_ERR_INVALID, "node %d: bad swap_dims descriptor", i);
        if (n.axis_a < 0 || n.axis_a >= n.rank || n.axis_b < 0 || n.axis_b >= n.rank)
          HE_FAIL(HE_ERR_INVALID, "node %d: swap axes out of range", i);
        for (int k = 0; k < n.rank; ++k) {
          int src = k == n.axis_a ? n.axis_b : k == n.axis_b ? n.axis_a : k;
          if (n.shape[k] != a->shape[src]) HE_FAIL(HE_ERR_INVALID, "node %d: swap_dims output shape wrong", i);
        }
        break;
      }
      case HE_OP_COMPARE:
        if (n.dtype != HE_BOOL || !same_shape(n, *a)) HE_FAIL(HE_ERR_INVALID, "node %d: compare must output bool of lhs shape", i);
        if (num_elements(*a) != num_elements(*b) || dclass(a->dtype) != dclass(b->dtype))
          HE_FAIL(HE_ERR_INVALID, "node %d: compare operands mismatch", i);
        if (n.sub_op < HE_CMP_EQ || n.sub_op > HE_CMP_GE) HE_FAIL(HE_ERR_INVALID, "node %d: bad compare op", i);
        break;
      case HE_OP_SELECT: {
        const he_node& sel = N[n.in[2]];
        if (!same_shape(n, *a) || n.dtype != a->dtype) HE_FAIL(HE_ERR_INVALID, "node %d: select output must equal lhs", i);
        if (sel.dtype != HE_BOOL) HE_FAIL(HE_ERR_INVALID, "node %d: selector must be bool", i);
        if (num_elements(*b) != num_elements(*a) || num_elements(sel) != num_elements(*a) ||
            dclass(a->dtype) != dclass(b->dtype))
          HE_FAIL(HE_ERR_INVALID, "node %d: select operands mismatch", i);
        break;
      }
      case HE_OP_MATMUL: {
        if (a->rank < 2 || b->rank != a->rank || n.rank != a->rank)
          HE_FAIL(HE_ERR_INVALID, "node %d: matmul operands must have equal rank >= 2", i);
        int r = a->rank;
        if (a->shape[r - 1] != b->shape[r - 2]) HE_FAIL(HE_ERR_INVALID, "node %d: matmul K mismatch", i);
        for (int k = 0; k < r - 2; ++k)
          if (a->shape[k] != b->shape[k] || n.shape[k] != a->shape[k])
            HE_FAIL(HE_ERR_INVALID, "node %d: matmul batch dims mismatch", i);
        if (n.shape[r - 2] != a->shape[r - 2] || n.shape[r - 1] != b->shape[r - 1])
          HE_FAIL(HE_ERR_INVALID, "node %d: matmul output shape wrong", i);
        {
          // the node's dtype is the accumulator type of its precision (precision.rs:84-96)
          const int kind = HE_PREC_KIND(n.sub_op);
          if (kind < HE_PREC_F32_F32 || kind > HE_PREC_F8_F16) HE_FAIL(HE_ERR_INVALID, "node %d: unknown matmul precision %d", i, kind);
          const bool f8 = kind == HE_PREC_F8_F32 || kind == HE_PREC_F8_F16;
          if ((n.sub_op & ~0xff) != 0 && (!f8 || (n.sub_op & ~0x11ff) != 0))
            HE_FAIL(HE_ERR_INVALID, "node %d: malformed matmul precision 0x%x", i, n.sub_op);
          const int acc = (kind == HE_PREC_F16_F16 || kind == HE_PREC_F8_F16) ? HE_F16 : HE_F32;
          if (n.dtype != acc) HE_FAIL(HE_ERR_INVALID, "node %d: matmul output must be the accumulator type of its precision (%s)", i, dtype_name(acc));
        }
        if (dclass(a->dtype) != DClass::Float || dclass(b->dtype) != DClass::Float)
          HE_FAIL(HE_ERR_INVALID, "node %d: matmul of non-float", i);
        break;
      }
    }
  }
  for (int o : out->outputs)
    if (o < 0 || o >= (int)N.size()) HE_FAIL(HE_ERR_INVALID, "output index %d out of range", o);
  if (out->inputs.empty()) {
    // A graph of constants only is legal (Tensor::from_constant); nothing to check.
  }
  return HE_OK;
}

}  // namespace he

using namespace he;

extern "C" {

int32_t he_ctx_create(int32_t device_ordinal, he_ctx** out) {
  if (!out) HE_FAIL(HE_ERR_INVALID, "he_ctx_create: out is null");
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    HE_FAIL(HE_ERR_CUDA, "no CUDA device available (%s); this library has no CPU path",
            e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
  if (device_ordinal < 0 || device_ordinal >= count)
    HE_FAIL(HE_ERR_INVALID, "device ordinal %d out of range (0..%d)", device_ordinal, count - 1);
  DeviceGuard guard(device_ordinal);
  HE_TRY(guard.status());
  cudaDeviceProp prop;
  HE_CUDA(cudaGetDeviceProperties(&prop, device_ordinal));
  if (prop.major != 10)
    HE_FAIL(HE_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library only carries sm_100a code",
            device_ordinal, prop.major, prop.minor);
  he_ctx* c = new he_ctx();
  c->device = device_ordinal;
  c->sm_count = prop.multiProcessorCount;
  c->max_smem_optin = (int)prop.sharedMemPerBlockOptin;
  e = cudaMalloc(&c->d_status, 64);
  if (e != cudaSuccess) {
    delete c;
    HE_FAIL(HE_ERR_CUDA, "cudaMalloc(status block) failed: %s", cudaGetErrorString(e));
  }
  cudaMemset(c->d_status, 0, 64);
  *out = c;
  return HE_OK;
}

int32_t he_ctx_reserve_sms(he_ctx* ctx, int32_t sms) {
  if (!ctx) HE_FAIL(HE_ERR_INVALID, "he_ctx_reserve_sms: ctx is null");
  if (sms < 0 || sms > ctx->sm_count - 2) HE_FAIL(HE_ERR_INVALID, "he_ctx_reserve_sms: %d is not in [0, %d]", sms, ctx->sm_count - 2);
  ctx->sm_reserved = sms;
  return HE_OK;
}

void he_ctx_destroy(he_ctx* ctx) {
  if (!ctx) return;
  if (ctx->d_status) cudaFree(ctx->d_status);
  delete ctx;
}

int32_t he_ctx_poll_device_status(he_ctx* ctx, void* cu_stream) {
  if (!ctx) HE_FAIL(HE_ERR_INVALID, "ctx is null");
  HE_CUDA(cudaStreamSynchronize((cudaStream_t)cu_stream));
  DeviceStatus st;
  HE_CUDA(cudaMemcpy(&st, ctx->d_status, sizeof st, cudaMemcpyDeviceToHost));
  if (st.code != 0) {
    cudaMemset(ctx->d_status, 0, 64);
    HE_FAIL(HE_ERR_DEVICE_TIMEOUT,
            "device-side bounded wait gave up: site %u detail %u in block %u (aux %u %u)",
            st.code >> 16, st.code & 0xffffu, st.block, st.aux0, st.aux1);
  }
  return HE_OK;
}

int32_t he_plan_pointwise(he_ctx* ctx, const he_graph_desc* desc, he_plan** out) {
  if (!out) HE_FAIL(HE_ERR_INVALID, "he_plan_pointwise: null argument");
  *out = nullptr;
  Graph g;
  HE_TRY(parse_graph(desc, &g));
  return plan_pointwise(ctx, g, out, nullptr);
}

int32_t he_plan_permute(he_ctx* ctx, int32_t rank, const int64_t* in_shape,
                        const int64_t* out_strides, int32_t dtype, he_plan** out) {
  if (!out || !in_shape || !out_strides) HE_FAIL(HE_ERR_INVALID, "he_plan_permute: null argument");
  *out = nullptr;
  return plan_permute(ctx, rank, in_shape, out_strides, dtype, out);
}

int32_t he_permute_output_strides(int32_t rank, const int64_t* in_shape, int32_t num_swaps,
                                  const int32_t* swaps, int32_t reference_compat,
                                  int64_t* out_strides) {
  if (rank < 1 || rank > HE_MAX_RANK || !in_shape || !out_strides || (num_swaps > 0 && !swaps))
    HE_FAIL(HE_ERR_INVALID, "he_permute_output_strides: bad argument");
  int perm[HE_MAX_RANK];
  for (int i = 0; i < rank; ++i) perm[i] = i;
  for (int s = 0; s < num_swaps; ++s) {
    int a = swaps[2 * s], b = swaps[2 * s + 1];
    if (a < 0 || a >= rank || b < 0 || b >= rank) HE_FAIL(HE_ERR_INVALID, "swap %d axes out of range", s);
    int t = perm[a]; perm[a] = perm[b]; perm[b] = t;
  }
  // perm[k] = the input axis that sits at output position k once all swaps are applied.
  int64_t stride = 1;
  for (int i = rank - 1; i >= 0; --i) {
    if (reference_compat) {
      // permute_dims.rs:164-170: looks up the POSITION of i in perm and treats that position as
      // the input axis, i.e. applies the inverse permutation.
      int j = 0;
      while (perm[j] != i) ++j;
      out_strides[j] = stride;
      stride *= in_shape[j];
    } else {
      out_strides[perm[i]] = stride;
      stride *= in_shape[perm[i]];
    }
  }
  return HE_OK;
}

int32_t he_plan_fused_matmul(he_ctx* ctx, const he_graph_desc* desc, he_plan** out) {
  if (!out) HE_FAIL(HE_ERR_INVALID, "he_plan_fused_matmul: null argument");
  *out = nullptr;
  Graph g;
  HE_TRY(parse_graph(desc, &g));
  return plan_fused_matmul(ctx, g, out, nullptr);
}

int32_t he_plan_supported(he_ctx* ctx, const he_graph_desc* desc, int32_t kind) {
  Graph g;
  if (parse_graph(desc, &g) != HE_OK) return 0;
  int tier = 0;
  if (kind == 0) {
    if (plan_pointwise(ctx, g, nullptr, &tier) != HE_OK) return 0;
    return tier;
  } else if (kind == 1) {
    // PermuteDims::can_fuse_with -> enumerate_swaps (permute_dims.rs:112-142): one input and a
    // linear chain of swap_dims.
    if (g.inputs.size() != 1 || g.outputs.size() != 1) return 0;
    int cur = g.inputs[0];
    for (int i = 0; i < (int)g.nodes.size(); ++i) {
      if (i == g.inputs[0]) continue;
      if (g.nodes[i].kind != HE_OP_SWAP_DIMS || g.nodes[i].in[0] != cur) return 0;
      cur = i;
    }
    if (cur == g.inputs[0] || g.outputs[0] != cur) return 0;
    int dt = g.nodes[cur].dtype;
    return dt == HE_BOOL ? 0 : 2;
  } else if (kind == 2) {
    if (plan_fused_matmul(ctx, g, nullptr, &tier) != HE_OK) return 0;
    return tier;
  }
  return 0;
}

int32_t he_plan_workspace_bytes(const he_plan* plan, size_t* out) {
  if (!plan || !out) HE_FAIL(HE_ERR_INVALID, "he_plan_workspace_bytes: null argument");
  *out = plan->workspace_bytes;
  return HE_OK;
}

int32_t he_launch(he_plan* plan, const void* const* inputs, void* const* outputs, void* workspace,
                  void* cu_stream) {
  if (!plan) HE_FAIL(HE_ERR_INVALID, "he_launch: plan is null");
  if (!plan->ctx) HE_FAIL(HE_ERR_INVALID, "he_launch: the plan was created without a context (planning only); there is no CPU path");
  if (plan->workspace_bytes > 0) {
    if (!workspace) HE_FAIL(HE_ERR_WORKSPACE, "plan needs %zu workspace bytes but workspace is null", plan->workspace_bytes);
    if ((uintptr_t)workspace % 256 != 0) HE_FAIL(HE_ERR_WORKSPACE, "workspace must be 256-byte aligned");
  }
  DeviceGuard guard(plan->ctx->device);   // restores the caller's current device on return
  HE_TRY(guard.status());
  plan->last_launches = 0;
  TraceRange range(plan->description.c_str());
  return plan->launch(inputs, outputs, workspace, (cudaStream_t)cu_stream);
}

static int find_matmul(const Graph& g) {
  for (int i = 0; i < (int)g.nodes.size(); ++i)
    if (g.nodes[i].kind == HE_OP_MATMUL) return i;
  return -1;
}

int32_t he_debug_dump_program(const he_graph_desc* desc, int32_t epilogue, void* buf, size_t cap, size_t* size_out) {
  Graph g;
  HE_TRY(parse_graph(desc, &g));
  PwCompileOptions opt;
  if (epilogue) {
    opt.acc_node = find_matmul(g);
    opt.epilogue = true;
    if (opt.acc_node < 0) HE_FAIL(HE_ERR_INVALID, "he_debug_dump_program: epilogue mode needs a matmul node");
  }
  PwCompiled c;
  HE_TRY(compile_pointwise(g, opt, &c));
  if (size_out) *size_out = sizeof(PwProgram);
  if (buf) {
    if (cap < sizeof(PwProgram)) HE_FAIL(HE_ERR_INVALID, "he_debug_dump_program: buffer too small (%zu < %zu)", cap, sizeof(PwProgram));
    memcpy(buf, &c.prog, sizeof(PwProgram));
  }
  return HE_OK;
}

int32_t he_debug_canonical_text(const he_graph_desc* desc, char* buf, size_t cap) {
  Graph g;
  HE_TRY(parse_graph(desc, &g));
  PwCompileOptions opt;
  opt.acc_node = find_matmul(g);
  opt.fuse_fma = false;
  opt.epilogue = opt.acc_node >= 0;
  PwCompiled c;
  HE_TRY(compile_pointwise(g, opt, &c));
  PwCanon canon;
  HE_TRY(canonicalize_program(g, c, c.iter_rank - 2, c.iter_rank - 1, &canon));
  if (!buf || cap < canon.text.size() + 1) HE_FAIL(HE_ERR_INVALID, "he_debug_canonical_text: buffer too small (need %zu)", canon.text.size() + 1);
  memcpy(buf, canon.text.c_str(), canon.text.size() + 1);
  return HE_OK;
}

int32_t he_debug_plan_fault_injection(he_plan* plan, uint32_t wait_limit_us, int32_t withhold_loads) {
  if (!plan) HE_FAIL(HE_ERR_INVALID, "he_debug_plan_fault_injection: plan is null");
  return plan->set_fault_injection(wait_limit_us, withhold_loads);
}

int32_t he_plan_last_launch_count(const he_plan* plan) { return plan ? plan->last_launches : 0; }
const char* he_plan_describe(const he_plan* plan) { return plan ? plan->description.c_str() : ""; }
void he_plan_destroy(he_plan* plan) { delete plan; }
const char* he_last_error_string(void) { return he::g_last_error.c_str(); }
const char* he_version(void) { return "helium_b200 0.1 (sm_100a)"; }

}  // extern "C"
