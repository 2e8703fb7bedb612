// Stand-alone pointwise kernels (hot-path rows P1-P4).
//
// The reference JIT-compiles one kernel per subgraph: one element per thread, scalar loads and a
// `/`-`%` chain per broadcast or swap (helium/src/cuda/instr/pointwise/jit.rs:19-121, 616-729),
// reductions through a shared-memory tree, warp shuffles and float atomics (jit.rs:402-458).
// JIT is not available to this library, so a subgraph is served by one of two tiers:
//   tier 2  hand-written kernels for catalogued shapes of graph -- today the
//           "x * scale[c] + bias[c] (relu) + permutation" family, run by the tiled transpose kernel
//           of permute.cu in a single pass over HBM;
//   tier 1  a register-program interpreter (pointwise_interp.cuh): 4 consecutive elements per
//           thread with 16-byte loads/stores where the operand is contiguous, strided views with
//           precomputed magic-number division elsewhere.
// Reductions are deterministic: a CTA (or a warp, for short groups) reduces its slice in a fixed
// order; groups that span several CTAs write partials to the workspace and a second small kernel
// folds them in index order (the reference's float atomics are order-dependent).
#include "permute.cuh"
#include "pointwise_interp.cuh"
#include "pointwise_jit.h"
#include "pointwise_dense.cuh"

#include <algorithm>

namespace he {

constexpr int kPwThreads = 256;

template <int V>
__global__ void __launch_bounds__(kPwThreads) pw_elementwise_kernel(const __grid_constant__ PwProgram P) {
  const uint32_t idx0 = (blockIdx.x * (uint32_t)kPwThreads + threadIdx.x) * V;
  int nvalid = 0;
  if (idx0 < P.n_elems) nvalid = min((uint32_t)V, P.n_elems - idx0);
  if (V > 1 && nvalid == 0) return;  // V == 1 keeps whole warps alive for the bool ballot
  pw_run<V>(P, idx0, nvalid, nullptr, nullptr);
}

// Reduction kernel.  Iteration space = [num_groups][group_size] (the reduce input, row-major with
// the reduced dims trailing, jit.rs:137-162).
__global__ void __launch_bounds__(kPwThreads) pw_reduce_kernel(const __grid_constant__ PwProgram P,
                                                               const __grid_constant__ PwReduceLaunch L) {
  __shared__ float sred[4][kPwThreads / 32];
  float red[4];
#pragma unroll
  for (int s = 0; s < 4; ++s) red[s] = s < P.n_reductions ? pw_reduce_identity(L.red_ops[s]) : 0.0f;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (L.warp_mode == 1) {
    const uint32_t group = blockIdx.x * (kPwThreads / 32) + warp;
    if (group >= L.num_groups) return;  // whole warp leaves together
    const uint32_t base = group * P.group_size;
    const uint32_t iters = (P.group_size + 31) / 32;
    for (uint32_t it = 0; it < iters; ++it) {
      const uint32_t e = it * 32 + lane;
      pw_run<1>(P, base + e, e < P.group_size ? 1 : 0, nullptr, red);
    }
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      if (s >= P.n_reductions) break;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) red[s] = pw_reduce_combine(L.red_ops[s], red[s], __shfl_down_sync(0xffffffffu, red[s], off));
      if (lane == 0) reinterpret_cast<float*>(P.out[L.red_out_slot[s]])[group] = red[s];
    }
    return;
  }
  if (L.warp_mode == 2) {
    // Column mode, for reductions read through a transposing view (helium's bias gradients:
    // swap_dims -> reduce): consecutive GROUPS are contiguous in memory, consecutive elements of one
    // group are a row pitch apart.  Lanes therefore own 32 consecutive groups, so that every load of
    // the warp is one contiguous run, and the 8 warps of the CTA split this CTA's slice of the group.
    __shared__ float scol[4][kPwThreads / 32][32];
    const uint32_t gblocks = (L.num_groups + 31) / 32;
    const uint32_t blk = blockIdx.x / gblocks, gb = blockIdx.x - blk * gblocks;
    const uint32_t group = gb * 32 + lane;
    const bool gvalid = group < L.num_groups;
    const uint32_t start = blk * L.chunk, end = min(start + L.chunk, P.group_size);
    const uint32_t base = gvalid ? group * P.group_size : 0u;
    for (uint32_t e = start + warp; e < end; e += kPwThreads / 32) pw_run<1>(P, base + e, gvalid ? 1 : 0, nullptr, red);
#pragma unroll
    for (int s = 0; s < 4; ++s)
      if (s < P.n_reductions) scol[s][warp][lane] = red[s];
    __syncthreads();
    if (warp == 0 && gvalid) {
      for (int s = 0; s < P.n_reductions; ++s) {
        float v = scol[s][0][lane];
        for (int w = 1; w < kPwThreads / 32; ++w) v = pw_reduce_combine(L.red_ops[s], v, scol[s][w][lane]);
        if (L.blocks_per_group == 1) reinterpret_cast<float*>(P.out[L.red_out_slot[s]])[group] = v;
        else L.partials[((size_t)s * L.num_groups + group) * L.blocks_per_group + blk] = v;
      }
    }
    return;
  }
  const uint32_t group = blockIdx.x / L.blocks_per_group;
  const uint32_t blk = blockIdx.x - group * L.blocks_per_group;
  const uint32_t start = blk * L.chunk;
  const uint32_t end = min(start + L.chunk, P.group_size);
  const uint32_t base = group * P.group_size;
  const uint32_t iters = (end - start + kPwThreads - 1) / kPwThreads;
  for (uint32_t it = 0; it < iters; ++it) {
    const uint32_t e = start + it * kPwThreads + threadIdx.x;
    pw_run<1>(P, base + e, e < end ? 1 : 0, nullptr, red);
  }
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    if (s >= P.n_reductions) break;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) red[s] = pw_reduce_combine(L.red_ops[s], red[s], __shfl_down_sync(0xffffffffu, red[s], off));
    if (lane == 0) sred[s][warp] = red[s];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int s = 0; s < P.n_reductions; ++s) {
      float v = sred[s][0];
      for (int w = 1; w < kPwThreads / 32; ++w) v = pw_reduce_combine(L.red_ops[s], v, sred[s][w]);
      if (L.blocks_per_group == 1) reinterpret_cast<float*>(P.out[L.red_out_slot[s]])[group] = v;
      else L.partials[((size_t)s * L.num_groups + group) * L.blocks_per_group + blk] = v;
    }
  }
}

struct PwFinalize {
  uint32_t num_groups, blocks_per_group;
  int n_red;
  int red_ops[4];
  float* out[4];
  const float* partials;
};

__global__ void __launch_bounds__(kPwThreads) pw_reduce_finalize_kernel(const __grid_constant__ PwFinalize F) {
  const uint32_t i = blockIdx.x * kPwThreads + threadIdx.x;
  if (i >= F.num_groups * (uint32_t)F.n_red) return;
  const uint32_t s = i / F.num_groups, g = i - s * F.num_groups;
  const float* p = F.partials + ((size_t)s * F.num_groups + g) * F.blocks_per_group;
  float v = p[0];
  for (uint32_t b = 1; b < F.blocks_per_group; ++b) v = pw_reduce_combine(F.red_ops[s], v, p[b]);
  F.out[s][g] = v;
}

// Many partials per group (one huge group cut into thousands of CTA slices): a warp per (reduction, group).  Lane l
// combines partials l, l + 32, ... in order, then the 32 lane values meet in a shuffle tree -- a fixed function of
// the partials, so results stay bit-stable across launches; one thread walking 9000 partials took ~0.4 ms.
__global__ void __launch_bounds__(kPwThreads) pw_reduce_finalize_warp_kernel(const __grid_constant__ PwFinalize F) {
  const uint32_t w = (blockIdx.x * kPwThreads + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= F.num_groups * (uint32_t)F.n_red) return;   // whole warps leave together
  const uint32_t s = w / F.num_groups, g = w - s * F.num_groups;
  const float* p = F.partials + ((size_t)s * F.num_groups + g) * F.blocks_per_group;
  float v = pw_reduce_identity(F.red_ops[s]);
#pragma unroll 4
  for (uint32_t b = lane; b < F.blocks_per_group; b += 32) v = pw_reduce_combine(F.red_ops[s], v, p[b]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = pw_reduce_combine(F.red_ops[s], v, __shfl_down_sync(0xffffffffu, v, off));
  if (lane == 0) F.out[s][g] = v;
}

// Thousands of partials per group: a CTA per (reduction, group); thread t combines partials t, t + 256, ... in
// order, a shuffle tree per warp, then the eight warp values in warp order.
__global__ void __launch_bounds__(kPwThreads) pw_reduce_finalize_cta_kernel(const __grid_constant__ PwFinalize F) {
  __shared__ float sw[kPwThreads / 32];
  const uint32_t w = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t s = w / F.num_groups, g = w - s * F.num_groups;
  const float* p = F.partials + ((size_t)s * F.num_groups + g) * F.blocks_per_group;
  float v = pw_reduce_identity(F.red_ops[s]);
#pragma unroll 4
  for (uint32_t b = threadIdx.x; b < F.blocks_per_group; b += kPwThreads) v = pw_reduce_combine(F.red_ops[s], v, p[b]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = pw_reduce_combine(F.red_ops[s], v, __shfl_down_sync(0xffffffffu, v, off));
  if (lane == 0) sw[warp] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = sw[0];
    for (int k = 1; k < kPwThreads / 32; ++k) t = pw_reduce_combine(F.red_ops[s], t, sw[k]);
    F.out[s][g] = t;
  }
}

int32_t launch_finalize(const PwFinalize& F, cudaStream_t stream) {
  const uint32_t items = F.num_groups * (uint32_t)F.n_red;
  if (F.blocks_per_group >= 1024) pw_reduce_finalize_cta_kernel<<<items, kPwThreads, 0, stream>>>(F);
  else if (F.blocks_per_group >= 64) pw_reduce_finalize_warp_kernel<<<(items * 32 + kPwThreads - 1) / kPwThreads, kPwThreads, 0, stream>>>(F);
  else pw_reduce_finalize_kernel<<<(items + kPwThreads - 1) / kPwThreads, kPwThreads, 0, stream>>>(F);
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

namespace {
// HE_PW_JIT=0 keeps every program outside the catalogue on the interpreter (A/B measurements, parity tests)
bool jit_enabled() {
  const char* e = getenv("HE_PW_JIT");
  return !(e && e[0] == '0');
}
}  // namespace

namespace {

struct PointwisePlan : he_plan {
  PwCompiled c;
  // dense elementwise tier-2 kernel (when the program is in its catalogue); ew_slot[k] = caller input
  // slot of canonical input k.  The interpreter program stays as the fallback for pointers or sizes
  // off the 16-byte rules.
  // dense column sum (reduce over rows of a plain tensor read through a swap): hand-written kernel
  bool cs_dense = false;
  unsigned cs_batch = 1, cs_M = 0, cs_N = 0, cs_slices = 1;
  int cs_dtype = HE_F32, cs_slot = 0;
  EwMatch ew;
  int ew_slot[3] = {-1, -1, -1};
  int ew_dtype = HE_F32;
  bool reduce = false;
  PwReduceLaunch rl{};
  int n_inputs = 0, n_outputs = 0;
  // elementwise programs outside the catalogue: the program printed as CUDA C and compiled at plan time
  std::shared_ptr<PwJitModule> jit;

  int32_t launch(const void* const* inputs, void* const* outputs, void* workspace, cudaStream_t stream) override {
    PwProgram P = c.prog;
    if (P.n_elems == 0) return HE_OK;
    for (int i = 0; i < n_inputs; ++i) {
      if (!inputs || !inputs[i]) HE_FAIL(HE_ERR_INVALID, "pointwise launch: input %d is null", i);
      P.in[i] = inputs[i];
    }
    for (int i = 0; i < n_outputs; ++i) {
      if (!outputs || !outputs[i]) HE_FAIL(HE_ERR_INVALID, "pointwise launch: output %d is null", i);
      P.out[i] = outputs[i];
    }
    if (!reduce && ew.kind >= 0) {
      const unsigned ve = ew_dtype == HE_F32 ? 4 : 8;
      const void* in[3] = {nullptr, nullptr, nullptr};
      bool ok = P.n_elems % ve == 0 && (reinterpret_cast<uintptr_t>(outputs[0]) & 15) == 0;
      for (int k = 0; k < ew.n_in; ++k) {
        in[k] = inputs[ew_slot[k]];
        ok = ok && (reinterpret_cast<uintptr_t>(in[k]) & 15) == 0;
      }
      if (ok) {
        HE_TRY(launch_dense_elementwise(ew.kind, ew_dtype, in, outputs[0], P.n_elems, ew.k, ctx_sm_count(ctx), stream));
        last_launches = 1;
        return HE_OK;
      }
    }
    if (!reduce && jit && pw_jit_pointers_ok(c, P)) {
      HE_TRY(pw_jit_launch(*jit, P, ctx_sm_count(ctx), stream));
      last_launches = 1;
      return HE_OK;
    }
    if (!reduce) {
      if (c.has_bool_io) {
        unsigned grid = (P.n_elems + kPwThreads - 1) / kPwThreads;
        pw_elementwise_kernel<1><<<grid, kPwThreads, 0, stream>>>(P);
      } else {
        unsigned grid = (unsigned)(((uint64_t)P.n_elems + kPwThreads * 4 - 1) / (kPwThreads * 4));
        pw_elementwise_kernel<4><<<grid, kPwThreads, 0, stream>>>(P);
      }
      HE_CUDA(cudaGetLastError());
      last_launches = 1;
      return HE_OK;
    }
    PwReduceLaunch L = rl;
    L.partials = reinterpret_cast<float*>(workspace);
    if (cs_dense && (reinterpret_cast<uintptr_t>(inputs[cs_slot]) & 15) == 0) {
      if (cs_slices > 1 && !workspace) HE_FAIL(HE_ERR_WORKSPACE, "pointwise launch: this plan needs a %zu-byte workspace", workspace_bytes);
      float* dst = cs_slices > 1 ? L.partials : reinterpret_cast<float*>(outputs[L.red_out_slot[0]]);
      HE_TRY(launch_colsum_dense(cs_dtype, inputs[cs_slot], dst, cs_batch, cs_M, cs_N, cs_slices, 256, stream));
      last_launches = 1;
      if (cs_slices > 1) {
        PwFinalize F{};
        F.num_groups = cs_batch * cs_N;
        F.blocks_per_group = cs_slices;
        F.n_red = 1;
        F.red_ops[0] = HE_RED_SUM;
        F.out[0] = reinterpret_cast<float*>(outputs[L.red_out_slot[0]]);
        F.partials = L.partials;
        HE_TRY(launch_finalize(F, stream));
        last_launches = 2;
      }
      return HE_OK;
    }
    unsigned grid = L.warp_mode == 1 ? (L.num_groups + 7) / 8
                    : L.warp_mode == 2 ? (L.num_groups + 31) / 32 * L.blocks_per_group
                                       : L.num_groups * L.blocks_per_group;
    if (jit) {
      HE_TRY(pw_jit_launch_reduce(*jit, P, L, grid, stream));
    } else {
      pw_reduce_kernel<<<grid, kPwThreads, 0, stream>>>(P, L);
      HE_CUDA(cudaGetLastError());
    }
    last_launches = 1;
    if (L.warp_mode != 1 && L.blocks_per_group > 1) {
      PwFinalize F{};
      F.num_groups = L.num_groups;
      F.blocks_per_group = L.blocks_per_group;
      F.n_red = P.n_reductions;
      for (int s = 0; s < P.n_reductions; ++s) {
        F.red_ops[s] = L.red_ops[s];
        F.out[s] = reinterpret_cast<float*>(P.out[L.red_out_slot[s]]);
      }
      F.partials = L.partials;
      HE_TRY(launch_finalize(F, stream));
      last_launches = 2;
    }
    return HE_OK;
  }
};

// Tier-2 matcher: store(relu?(x * s + b)) where x is read through a pure axis permutation and
// s / b vary along exactly one axis of x.  Returns true and fills the permute arguments.
bool match_affine_permute(const Graph& g, const PwCompiled& c, AffineFunctor* f, int* rank,
                          int64_t* in_shape, int64_t* out_strides, int* dtype) {
  const PwProgram& P = c.prog;
  if (P.n_outputs != 1 || P.n_reductions != 0 || c.has_bool_io) return false;
  // instruction shapes accepted (after FMA fusion):
  //   LOAD x [LOAD s] [LOAD b] (MUL | FMA | ADD) [RELU] STORE   in compiler emission order
  int x_load = -1;
  std::vector<const PwLoadInfo*> params;
  for (const PwLoadInfo& li : c.loads) {
    const he_node& n = g.nodes[li.node];
    if (dclass(n.dtype) != DClass::Float) return false;
    if (!li.single_view) return false;
    if (num_elements(n) == (int64_t)P.n_elems && !li.identity) {
      if (x_load >= 0) return false;
      x_load = (int)(&li - &c.loads[0]);
    } else {
      params.push_back(&li);
    }
  }
  if (x_load < 0 || params.size() > 2) return false;
  const PwLoadInfo& X = c.loads[x_load];
  const he_node& xn = g.nodes[X.node];
  // x's view must be a bijection: every iteration dim walks a distinct axis of x with that axis' extent
  int64_t xst[HE_MAX_RANK];
  {
    int64_t s = 1;
    for (int i = xn.rank - 1; i >= 0; --i) { xst[i] = s; s *= xn.shape[i]; }
  }
  int64_t iter_packed[HE_MAX_RANK];
  {
    int64_t s = 1;
    for (int k = c.iter_rank - 1; k >= 0; --k) { iter_packed[k] = s; s *= c.iter_shape[k]; }
  }
  int axis_of_iter[HE_MAX_RANK];
  bool used[HE_MAX_RANK] = {false};
  for (int k = 0; k < c.iter_rank; ++k) {
    axis_of_iter[k] = -1;
    if (c.iter_shape[k] == 1) continue;
    for (int j = 0; j < xn.rank; ++j)
      if (!used[j] && xn.shape[j] == c.iter_shape[k] && xst[j] == X.iter_stride[k] && xn.shape[j] != 1) {
        axis_of_iter[k] = j;
        used[j] = true;
        break;
      }
    if (axis_of_iter[k] < 0) return false;
  }
  for (int j = 0; j < xn.rank; ++j)
    if (!used[j] && xn.shape[j] != 1) return false;
  *rank = xn.rank;
  for (int j = 0; j < xn.rank; ++j) { in_shape[j] = xn.shape[j]; out_strides[j] = 1; }
  for (int k = 0; k < c.iter_rank; ++k)
    if (axis_of_iter[k] >= 0) out_strides[axis_of_iter[k]] = iter_packed[k];
  // parameters: one non-zero stride (== 1 after collapsing), along an iteration dim that maps to an x axis
  int param_axis = -1;
  for (const PwLoadInfo* pl : params) {
    int dim = -1;
    for (int k = 0; k < c.iter_rank; ++k) {
      if (pl->identity) return false;
      if (pl->iter_stride[k] != 0 && c.iter_shape[k] != 1) {
        if (dim >= 0 || pl->iter_stride[k] != 1) return false;
        dim = k;
      }
    }
    int axis = dim >= 0 ? axis_of_iter[dim] : 0;
    if (dim >= 0 && num_elements(g.nodes[pl->node]) != c.iter_shape[dim]) return false;
    if (dim < 0 && num_elements(g.nodes[pl->node]) != 1) return false;
    if (param_axis >= 0 && axis != param_axis && dim >= 0) return false;
    if (dim >= 0) param_axis = axis;
  }
  if (param_axis < 0) param_axis = 0;
  // walk the instruction stream
  auto load_slot_of_reg_def = [&](int instr_idx) -> const PwLoadInfo* {
    for (const PwLoadInfo& li : c.loads)
      if (li.instr == instr_idx) return &li;
    return nullptr;
  };
  // symbolic evaluation: each register holds one of {x, s, b (raw loads), expr}
  struct Val { int kind; int scale_slot, bias_slot; bool relu; };  // kind: 0 none 1 x-expr 2 param
  Val regs[kPwMaxRegs];
  int param_slot[kPwMaxRegs];
  for (int r = 0; r < kPwMaxRegs; ++r) { regs[r] = {0, -1, -1, false}; param_slot[r] = -1; }
  Val result{0, -1, -1, false};
  for (int i = 0; i < P.n_instr; ++i) {
    const PwInstr& in = P.instr[i];
    switch (in.op) {
      case PW_LOAD: {
        const PwLoadInfo* li = load_slot_of_reg_def(i);
        if (!li) return false;
        if (li == &X) regs[in.dst] = {1, -1, -1, false};
        else { regs[in.dst] = {2, -1, -1, false}; param_slot[in.dst] = li->input_slot; }
        break;
      }
      case PW_BIN_F: {
        Val a = regs[in.a], b = regs[in.b];
        int pa = param_slot[in.a], pb = param_slot[in.b];
        if (a.kind == 2 && b.kind == 1) { std::swap(a, b); std::swap(pa, pb); }
        if (a.kind != 1 || b.kind != 2 || a.relu) return false;
        if (in.sub == HE_BIN_MUL) {
          if (a.scale_slot >= 0 || a.bias_slot >= 0) return false;
          a.scale_slot = pb;
        } else if (in.sub == HE_BIN_ADD) {
          if (a.bias_slot >= 0) return false;
          a.bias_slot = pb;
        } else return false;
        regs[in.dst] = a;
        param_slot[in.dst] = -1;
        break;
      }
      case PW_FMA: {
        Val a = regs[in.a], b = regs[in.b], cc = regs[in.c];
        int pa = param_slot[in.a], pb = param_slot[in.b], pc = param_slot[in.c];
        if (a.kind == 2 && b.kind == 1) { std::swap(a, b); std::swap(pa, pb); }
        if (a.kind != 1 || b.kind != 2 || cc.kind != 2 || a.relu || a.scale_slot >= 0 || a.bias_slot >= 0) return false;
        a.scale_slot = pb;
        a.bias_slot = pc;
        regs[in.dst] = a;
        param_slot[in.dst] = -1;
        break;
      }
      case PW_UNARY: {
        Val a = regs[in.a];
        if (in.sub != HE_UN_RELU || a.kind != 1 || a.relu) return false;
        a.relu = true;
        regs[in.dst] = a;
        param_slot[in.dst] = -1;
        break;
      }
      case PW_STORE:
        result = regs[in.a];
        if (result.kind != 1) return false;
        if (in.dt != xn.dtype) return false;
        break;
      default: return false;
    }
  }
  if (result.kind != 1) return false;
  if (result.scale_slot < 0 && result.bias_slot < 0 && !result.relu) return false;  // plain permute: not ours
  f->enabled = true;
  f->axis = param_axis;
  f->x_dtype = xn.dtype;
  f->x_input = X.input_slot;
  f->has_scale = result.scale_slot >= 0;
  f->has_bias = result.bias_slot >= 0;
  f->relu = result.relu;
  f->scale_input = result.scale_slot;
  f->bias_input = result.bias_slot;
  if (f->has_scale) f->scale_dtype = g.nodes[g.inputs[result.scale_slot]].dtype;
  if (f->has_bias) f->bias_dtype = g.nodes[g.inputs[result.bias_slot]].dtype;
  *dtype = xn.dtype;
  return true;
}

}  // namespace

// A reshape of a reduction result as a leaf (helium's bias gradient ends in `.reshape([n])`,
// tensor.rs:139) writes the same bytes as the reduction itself: the leaf becomes the reduction.
static Graph peel_reshaped_reduction_leaves(const Graph& g) {
  Graph o = g;
  for (int& leaf : o.outputs) {
    const he_node& L = o.nodes[leaf];
    if (L.kind != HE_OP_RESHAPE || L.in[0] < 0) continue;
    const he_node& R = o.nodes[L.in[0]];
    if (R.kind == HE_OP_REDUCE && num_elements(R) == num_elements(L)) leaf = L.in[0];
  }
  return o;
}

// A reduction leaf over dims that are not the trailing ones (the playground's rank-kept Reduction over any axes,
// helium-playground/src/opgraph.rs:397-413: a column sum is Reduction{axes = [rows]}) is rewritten to the helium-ir
// form the kernels take: swap_dims until the reduced dims are last, the kept ones in their old order, then a
// reduction over the trailing dims.  The result has the same elements in the same order, so the leaf's buffer is
// written exactly as before; the reduction kernel reads through the swapped view (column mode where a lane can
// own a group), and no permuted copy exists.
static Graph trail_reduction_leaves(const Graph& g) {
  Graph o = g;
  for (int& leaf : o.outputs) {
    const he_node L = o.nodes[leaf];
    if (L.kind != HE_OP_REDUCE || L.in[0] < 0) continue;
    const he_node A = o.nodes[L.in[0]];
    const int d = __builtin_popcount(L.axes);
    if (d == 0 || A.rank < 2 || L.axes == (((1u << d) - 1u) << (A.rank - d))) continue;
    std::vector<int> target, cur(A.rank);
    for (int k = 0; k < A.rank; ++k)
      if (!((L.axes >> k) & 1u)) target.push_back(k);
    for (int k = 0; k < A.rank; ++k)
      if ((L.axes >> k) & 1u) target.push_back(k);
    for (int k = 0; k < A.rank; ++k) cur[k] = k;
    int src = L.in[0];
    he_node view = A;
    for (int pos = 0; pos < A.rank; ++pos) {
      int j = pos;
      while (cur[j] != target[pos]) ++j;
      if (j == pos) continue;
      std::swap(cur[pos], cur[j]);
      std::swap(view.shape[pos], view.shape[j]);
      he_node sw = view;
      sw.kind = HE_OP_SWAP_DIMS;
      sw.sub_op = 0;
      sw.in[0] = src;
      sw.in[1] = sw.in[2] = -1;
      sw.axis_a = pos;
      sw.axis_b = j;
      sw.axes = 0;
      sw.const_bits = 0;
      o.nodes.push_back(sw);
      src = (int)o.nodes.size() - 1;
    }
    he_node red = L;
    red.in[0] = src;
    red.axes = ((1u << d) - 1u) << (A.rank - d);
    red.rank = A.rank - d + 1;
    for (int k = 0; k < A.rank - d; ++k) red.shape[k] = view.shape[k];
    red.shape[A.rank - d] = 1;
    o.nodes.push_back(red);
    leaf = (int)o.nodes.size() - 1;
  }
  return o;
}

int32_t plan_pointwise(he_ctx* ctx, const Graph& g_in, he_plan** out, int* tier_only) {
  const Graph g = trail_reduction_leaves(peel_reshaped_reduction_leaves(g_in));
  for (const he_node& n : g.nodes)
    if (n.kind == HE_OP_MATMUL) HE_FAIL(HE_ERR_UNSUPPORTED, "pointwise: subgraph contains a matmul");
  PointwisePlan* plan = new PointwisePlan();
  int32_t st = compile_pointwise(g, PwCompileOptions{}, &plan->c);
  if (st != HE_OK) {
    delete plan;
    return st;
  }
  // tier 2
  {
    AffineFunctor f;
    int rank, dtype;
    int64_t in_shape[HE_MAX_RANK], out_strides[HE_MAX_RANK];
    if (match_affine_permute(g, plan->c, &f, &rank, in_shape, out_strides, &dtype)) {
      he_plan* pp = nullptr;
      // the tile kernel needs the innermost axis to move; otherwise the interpreter is already coalesced
      std::string saved = he_last_error_string();
      if (make_permute_plan(ctx, rank, in_shape, out_strides, dtype, &f, &pp) == HE_OK) {
        delete plan;
        if (tier_only) {
          *tier_only = 2;
          delete pp;
          return HE_OK;
        }
        pp->description = "pointwise tier 2 (fused affine + " + pp->description + ")";
        *out = pp;
        return HE_OK;
      }
      set_error("%s", saved.c_str());
    }
  }
  // tier 2, dense elementwise: one output, every load a dense identity load, one dtype throughout
  {
    const PwProgram& P0 = plan->c.prog;
    bool dense = P0.n_outputs == 1 && P0.n_reductions == 0 && !plan->c.has_bool_io && !plan->c.loads.empty() &&
                 plan->c.loads.size() <= 3 && g.inputs.size() == plan->c.loads.size();
    const int dt = g.nodes[g.outputs[0]].dtype;
    dense = dense && (dt == HE_F32 || dt == HE_BF16 || dt == HE_F16);
    for (const PwLoadInfo& li : plan->c.loads)
      dense = dense && li.identity && g.nodes[li.node].dtype == dt && num_elements(g.nodes[li.node]) == (int64_t)P0.n_elems;
    if (dense) {
      PwCompileOptions opt;
      opt.fuse_fma = false;
      PwCompiled plain;
      PwCanon canon;
      std::string saved = he_last_error_string();
      if (compile_pointwise(g, opt, &plain) == HE_OK && canonicalize_program(g, plain, -1, -1, &canon) == HE_OK &&
          match_dense_elementwise(canon.text, &plan->ew) && (int)canon.slot_order.size() == plan->ew.n_in) {
        for (int k = 0; k < plan->ew.n_in; ++k) plan->ew_slot[k] = canon.slot_order[k];
        plan->ew_dtype = dt;
      } else {
        plan->ew.kind = -1;
        set_error("%s", saved.c_str());
      }
    }
  }
  if (tier_only) {
    *tier_only = plan->ew.kind >= 0 ? 2 : 1;
    delete plan;
    return HE_OK;
  }
  plan->ctx = ctx;
  plan->n_inputs = plan->c.prog.n_inputs;
  plan->n_outputs = plan->c.prog.n_outputs;
  const PwProgram& P = plan->c.prog;
  plan->reduce = P.n_reductions > 0;
  char desc[256];
  if (plan->reduce) {
    PwReduceLaunch& L = plan->rl;
    L.num_groups = P.group_size ? P.n_elems / P.group_size : 0;
    int s = 0;
    for (size_t o = 0; o < plan->c.out_is_reduce.size(); ++o)
      if (plan->c.out_is_reduce[o] >= 0) {
        L.red_ops[s] = plan->c.out_is_reduce[o];
        L.red_out_slot[s] = (int)o;
        ++s;
      }
    // Small problems (a few launches' worth of latency, not bandwidth) are spread as widely as they
    // go: a thread that walks 8-16 elements of a fused prologue serially pays a dependent memory
    // latency per element, which made 2560-element reductions take 30 us.
    const bool small = (uint64_t)L.num_groups * P.group_size <= (1u << 21);
    // Does the largest tensor walk memory contiguously along the GROUPS rather than along the
    // elements of a group?  (the reduce input is a transposing view of it)
    bool column = false;
    {
      const PwLoadInfo* big = nullptr;
      for (const PwLoadInfo& li : plan->c.loads)
        if (!big || num_elements(g.nodes[li.node]) > num_elements(g.nodes[big->node])) big = &li;
      int gdim = plan->c.iter_rank - 1;   // last dim that indexes groups
      int64_t prod = 1;
      while (gdim >= 0 && prod < (int64_t)P.group_size) prod *= plan->c.iter_shape[gdim--];
      while (gdim > 0 && plan->c.iter_shape[gdim] == 1) --gdim;
      if (big && big->single_view && !big->identity && gdim >= 0 && prod == (int64_t)P.group_size && P.group_size > 1 &&
          L.num_groups >= 32 && big->iter_stride[gdim] == 1 && big->iter_stride[plan->c.iter_rank - 1] > 1)
        column = true;
    }
    if (column) {
      L.warp_mode = 2;
      uint32_t chunk = small ? 64 : 256;   // elements of a group per CTA: 8 / 32 per lane
      chunk = std::min<uint32_t>(chunk, (P.group_size + 7) / 8 * 8);
      uint32_t bpg = (P.group_size + chunk - 1) / chunk;
      const uint64_t gblocks = (L.num_groups + 31) / 32, max_ctas = (uint64_t)ctx_sm_count(ctx) * 64;
      if (bpg * gblocks > max_ctas) {
        bpg = (uint32_t)std::max<uint64_t>(1, max_ctas / gblocks);
        chunk = (P.group_size + bpg - 1) / bpg;
        chunk = (chunk + 7) / 8 * 8;
        bpg = (P.group_size + chunk - 1) / chunk;
      }
      L.blocks_per_group = bpg;
      L.chunk = chunk;
      if (bpg > 1) plan->workspace_bytes = (size_t)P.n_reductions * L.num_groups * bpg * sizeof(float);
      // the plain case -- one tensor, no prologue, Sum over its rows -- has a kernel of its own
      const PwLoadInfo& li = plan->c.loads[0];
      const he_node& xn = g.nodes[li.node];
      const int rk = plan->c.iter_rank;
      if (plan->c.loads.size() == 1 && P.n_instr == 2 && P.n_reductions == 1 && L.red_ops[0] == HE_RED_SUM && rk >= 2 &&
          (xn.dtype == HE_F32 || xn.dtype == HE_BF16 || xn.dtype == HE_F16) && num_elements(xn) == (int64_t)P.n_elems) {
        const int64_t N = plan->c.iter_shape[rk - 2], M = plan->c.iter_shape[rk - 1];
        bool ok = (int64_t)P.group_size == M && li.iter_stride[rk - 1] == N && li.iter_stride[rk - 2] == 1 &&
                  N % (xn.dtype == HE_F32 ? 4 : 8) == 0;
        int64_t expect = M * N, batch = 1;
        for (int k = rk - 3; k >= 0; --k) {
          if (plan->c.iter_shape[k] != 1 && li.iter_stride[k] != expect) ok = false;
          expect *= plan->c.iter_shape[k];
          batch *= plan->c.iter_shape[k];
        }
        if (ok && batch <= 65535) {
          plan->cs_dense = true;
          plan->cs_batch = (unsigned)batch; plan->cs_M = (unsigned)M; plan->cs_N = (unsigned)N;
          plan->cs_slices = (unsigned)((M + 255) / 256);
          plan->cs_dtype = xn.dtype;
          plan->cs_slot = li.input_slot;
          if (plan->cs_slices > 1)
            plan->workspace_bytes = std::max(plan->workspace_bytes, (size_t)batch * N * plan->cs_slices * sizeof(float));
        }
      }
    } else if (P.group_size <= (small ? 32u : 2048u)) {
      L.warp_mode = 1;
      L.blocks_per_group = 1;
      L.chunk = P.group_size;
    } else {
      L.warp_mode = 0;
      // ~16 elements per thread per CTA (one for small problems), but never more CTAs than ~8 waves' worth of the GPU
      uint32_t chunk = kPwThreads * (small ? 1 : 16);
      uint32_t bpg = (P.group_size + chunk - 1) / chunk;
      uint64_t max_ctas = (uint64_t)ctx_sm_count(ctx) * 64;
      if ((uint64_t)bpg * L.num_groups > max_ctas) {
        bpg = (uint32_t)std::max<uint64_t>(1, max_ctas / std::max<uint32_t>(1, L.num_groups));
        chunk = (P.group_size + bpg - 1) / bpg;
        chunk = (chunk + kPwThreads - 1) / kPwThreads * kPwThreads;
        bpg = (P.group_size + chunk - 1) / chunk;
      }
      L.blocks_per_group = bpg;
      L.chunk = chunk;
      if (bpg > 1) plan->workspace_bytes = (size_t)P.n_reductions * L.num_groups * bpg * sizeof(float);
    }
    const bool red_jit = !plan->cs_dense && jit_enabled() && !plan->c.has_bool_io && [&] {
      const std::string saved = he_last_error_string();
      const bool ok = pw_jit_compile(plan->c, &plan->jit) == HE_OK;
      if (!ok) set_error("%s", saved.c_str());
      return ok;
    }();
    if (plan->cs_dense)
      snprintf(desc, sizeof desc, "pointwise tier 2 (dense column-sum kernel, [%u x %u x %u], %u row slices; column-mode interpreter for unaligned tensors)",
               plan->cs_batch, plan->cs_M, plan->cs_N, plan->cs_slices);
    else
    snprintf(desc, sizeof desc, "pointwise tier 1 (%s, %d instr, %d regs), reduce: %u groups of %u, %s, %u CTAs/group",
             red_jit ? "program specialised at plan time with NVRTC" : "interpreter", P.n_instr, plan->c.n_regs, L.num_groups, P.group_size, L.warp_mode == 1 ? "warp per group" : L.warp_mode == 2 ? "column mode (lane per group)" : "CTA slices", L.blocks_per_group);
  } else if (plan->ew.kind >= 0) {
    snprintf(desc, sizeof desc, "pointwise tier 2 (dense elementwise kernel %s, 16-byte vectors; interpreter fallback for unaligned tensors)",
             plan->ew.name);
  } else if (jit_enabled() && !plan->c.has_bool_io && [&] {
               const std::string saved = he_last_error_string();
               const bool ok = pw_jit_compile(plan->c, &plan->jit) == HE_OK;
               if (!ok) set_error("%s", saved.c_str());
               return ok;
             }()) {
    snprintf(desc, sizeof desc, "pointwise tier 1 (program of %d instr specialised at plan time with NVRTC, 8 elems/thread, 16-byte vectors; "
             "interpreter fallback for unaligned tensors)", P.n_instr);
  } else {
    snprintf(desc, sizeof desc, "pointwise tier 1 (interpreter, %d instr, %d regs, %d elems/thread)", P.n_instr,
             plan->c.n_regs, plan->c.has_bool_io ? 1 : 4);
  }
  plan->description = desc;
  *out = plan;
  return HE_OK;
}

}  // namespace he
