// Host side of the implicit-GEMM convolutions (conv_sm100.cuh): geometry, tensor maps, tap tables, plans.
//
// Replaces the cuDNN graphs of Op::Conv / Op::ConvBackwardData / Op::ConvBackwardFilter
// (helium/src/cuda/instr/cudnn_graph.rs:182-228, make_conv_descriptor :384-396) with the parameters of
// Conv2dParams (helium-ir/src/opgraph/op/conv.rs:5-95): output size = input size adjusted by the padding mode,
// divided by the stride (conv.rs:51-74); padding k/2 (Same), 0 (Valid), k-1 (Full) on both sides
// (conv.rs:86-94).  Images are NHWC, filters KRSC (helium/src/raw_tensor.rs:232-240).
#include <cuda.h>

#include <algorithm>
#include <memory>
#include <mutex>

#include "conv_sm100.cuh"
#include "gemm_plan.cuh"

namespace he {
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int32_t encode(CUtensorMap* out, int ab_format, int rank, const void* base, const cuuint64_t* dims, const cuuint64_t* strides,
               const cuuint32_t* box, const char* what) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) HE_FAIL(HE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if ((uintptr_t)base % 16 != 0) HE_FAIL(HE_ERR_UNSUPPORTED, "conv2d: %s pointer is not 16-byte aligned", what);
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(out, ab_format == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (cuuint32_t)rank,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) HE_FAIL(HE_ERR_CUDA, "cuTensorMapEncodeTiled (%s) failed with CUresult %d", what, (int)r);
  return HE_OK;
}

// NHWC activation [NB, H, W, C], parity class (ph, pw) of a stride-`s` sampling: pixels (ph + s i, pw + s j).
// Dimensions (C, W', H', NB); box 64 channels x tw x th x tn pixels.
int32_t make_activation_tmap(CUtensorMap* out, const void* ptr, int ab_format, int NB, int H, int W, int C, int s, int ph, int pw,
                             int tw, int th, int tn) {
  const int Wc = (W - pw + s - 1) / s, Hc = (H - ph + s - 1) / s;
  if (Wc <= 0 || Hc <= 0) {   // class does not exist (a 1-pixel-wide image); the map is never used
    memset(out, 0, sizeof *out);
    return HE_OK;
  }
  cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)Wc, (cuuint64_t)Hc, (cuuint64_t)NB};
  cuuint64_t strides[3] = {(cuuint64_t)s * C * 2, (cuuint64_t)s * W * C * 2, (cuuint64_t)H * W * C * 2};
  cuuint32_t box[4] = {(cuuint32_t)kBK, (cuuint32_t)tw, (cuuint32_t)th, (cuuint32_t)tn};
  const char* base = reinterpret_cast<const char*>(ptr) + ((size_t)ph * W + pw) * C * 2;
  return encode(out, ab_format, 4, base, dims, strides, box, "activation");
}

// KRSC filter as (C, R*S, K); box = (64 c, 1 tap, rows_k output channels).
int32_t make_filter_tmap(CUtensorMap* out, const void* ptr, int ab_format, int K, int RS, int C, int box_c, int box_k) {
  cuuint64_t dims[3] = {(cuuint64_t)C, (cuuint64_t)RS, (cuuint64_t)K};
  cuuint64_t strides[2] = {(cuuint64_t)C * 2, (cuuint64_t)RS * C * 2};
  cuuint32_t box[3] = {(cuuint32_t)box_c, 1u, (cuuint32_t)box_k};
  return encode(out, ab_format, 3, ptr, dims, strides, box, "filter");
}

// Patch of `total` pixels (a power of two) over a grid of GN images x GP rows x GQ columns: powers of two
// (tw, th, tn) with tw * th * tn = total that cover the grid with the least padding; ties prefer wide rows
// (longer contiguous runs in memory).
void choose_patch(int total, int GQ, int GP, int GN, int* tw, int* th, int* tn) {
  long long best = -1;
  for (int a = total; a >= 1; a >>= 1)          // tw
    for (int b = total / a; b >= 1; b >>= 1) {  // th
      const int cimg = total / a / b;           // tn
      const long long vol = (long long)((GQ + a - 1) / a) * a * ((GP + b - 1) / b) * b * ((GN + cimg - 1) / cimg) * cimg;
      if (best < 0 || vol < best) {
        best = vol;
        *tw = a; *th = b; *tn = cimg;
      }
    }
}

int floor_div(int a, int b) { return (a >= 0) ? a / b : -((-a + b - 1) / b); }

__global__ void conv_wgrad_fold(const float* __restrict__ partials, void* __restrict__ out, int out_dt, long long n, int splits) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = partials[i];
  for (int k = 1; k < splits; ++k) s += partials[(size_t)k * n + i];   // fixed order: bit-stable
  if (out_dt == HE_F32) reinterpret_cast<float*>(out)[i] = s;
  else reinterpret_cast<unsigned short*>(out)[i] = (unsigned short)(out_dt == HE_BF16 ? f32_to_bf16_bits(s) : f32_to_f16_bits(s));
}

// out[2][N] = column sums of the two statistics partial blocks [rows][N].  A CTA is 32 columns x 32 row lanes:
// lane y adds rows y, y + 32, ... in order (independent loads, so the L2 latency is paid once per few rows, not
// once per row), and the 32 lane sums meet in shared memory in lane order -- a fixed function of the
// partials, bit-stable across launches.
__global__ void __launch_bounds__(1024) conv_stats_fold(const float* __restrict__ p0, const float* __restrict__ p1, float* __restrict__ out,
                                                       int rows, int N) {
  __shared__ float sh[32][33];
  const int i = blockIdx.x * 32 + threadIdx.x;
  float s = 0.0f;
  if (i < 2 * N) {
    const float* p = (i < N ? p0 : p1) + (i < N ? i : i - N);
#pragma unroll 4
    for (int r = threadIdx.y; r < rows; r += 32) s += p[(size_t)r * N];
  }
  sh[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && i < 2 * N) {
    float t = sh[0][threadIdx.x];
#pragma unroll
    for (int y = 1; y < 32; ++y) t += sh[y][threadIdx.x];
    out[i] = t;
  }
}

template <int BN, bool B_MN>
int32_t launch_fprop(const ConvParams& p, int grid, cudaStream_t stream) {
  constexpr int STAGES = BN == 128 ? 6 : 8;
  using SM = ConvSmem<BN, STAGES>;
  static_assert(SM::dynamic_bytes <= 232448, "shared memory budget of sm_100 exceeded");
  auto kernel = conv_fprop_kernel<BN, STAGES, B_MN>;
  static bool configured = false;
  if (!configured) {
    HE_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::dynamic_bytes));
    configured = true;
  }
  kernel<<<grid, 352, SM::dynamic_bytes, stream>>>(p);   // producer, two MMA issuers, eight epilogue warps
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

template <int BN, int T>
int32_t launch_wgrad(const ConvWgradParams& p, int grid, cudaStream_t stream) {
  // stages: as many as fit beside 1 KB of alignment slack (16 KB flow tile + T image tiles per stage)
  constexpr int STAGES = T == 1 ? 6 : (BN == 64 ? 5 : 3);
  using SM = ConvWgradSmem<BN, STAGES, T>;
  static_assert(SM::dynamic_bytes <= 232448, "shared memory budget of sm_100 exceeded");
  auto kernel = conv_wgrad_kernel<BN, STAGES, T>;
  static bool configured = false;
  if (!configured) {
    HE_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::dynamic_bytes));
    configured = true;
  }
  kernel<<<grid, 256, SM::dynamic_bytes, stream>>>(p);   // producer, three MMA issuers (warps 1, 6, 7), four epilogue warps
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

struct ConvPlan : he_plan {
  int kind = 0;
  he_conv2d_params prm{};
  he_conv2d_fusion fus{};
  int NB = 0, H = 0, W = 0, P = 0, Q = 0, pad_h = 0, pad_w = 0;
  int ab_format = 1, dtype = HE_BF16;
  int bn = 128;
  GemmCore core{};
  // forward / data gradient: one launch per output parity class (one class unless data gradient with stride 2)
  struct Pass {
    ConvGeom geom{};
    int grid = 0, num_tiles = 0, tile_m_base = 0;
  };
  std::vector<Pass> passes;
  bool memset_out = false;
  int total_tiles_m = 0;
  // input slots
  int n_in = 0, s_bias = -1, s_resid = -1, s_gate_x = -1, s_gate_scale = -1, s_gate_shift = -1;
  size_t ws_stat_off[2] = {0, 0};
  // filter gradient
  ConvGeom wgeom{};
  int splits = 1, k_tiles = 0, wgrid = 0, taps_per_cta = 1;

  int32_t launch(const void* const* inputs, void* const* outputs, void* workspace, cudaStream_t stream) override {
    for (int i = 0; i < n_in; ++i)
      if (!inputs || !inputs[i]) HE_FAIL(HE_ERR_INVALID, "conv2d launch: input %d is null", i);
    if (!outputs || !outputs[0] || (fus.want_stats && !outputs[1])) HE_FAIL(HE_ERR_INVALID, "conv2d launch: an output is null");
    if (workspace_bytes > 0 && !workspace) HE_FAIL(HE_ERR_WORKSPACE, "conv2d launch: this plan needs a %zu-byte workspace", workspace_bytes);
    last_launches = 0;
    const int Cin = prm.in_channels, Kout = prm.out_channels, RS = prm.kernel_h * prm.kernel_w;
    GemmCore c = core;
    c.status = ctx ? ctx->d_status : nullptr;
    if (kind == HE_CONV_BWD_FILTER) {
      ConvWgradParams p;
      memset(&p, 0, sizeof p);
      // inputs: flow [NB, P, Q, K], image [NB, H, W, C]
      HE_TRY(make_activation_tmap(&p.tma_dy, inputs[0], ab_format, NB, P, Q, Kout, 1, 0, 0, wgeom.tw, wgeom.th, wgeom.tn));
      const int s = prm.stride_h;
      for (int ph = 0; ph < s; ++ph)
        for (int pw = 0; pw < s; ++pw)
          HE_TRY(make_activation_tmap(&p.tma_x[ph * 2 + pw], inputs[1], ab_format, NB, H, W, Cin, s, ph, pw, wgeom.tw, wgeom.th, wgeom.tn));
      p.core = c;
      p.geom = wgeom;
      p.partials = reinterpret_cast<float*>(workspace);
      p.splits = splits;
      p.k_tiles = k_tiles;
      p.rs = RS;
      p.tap_groups = (RS + taps_per_cta - 1) / taps_per_cta;
      if (taps_per_cta == 3) HE_TRY(bn == 64 ? (launch_wgrad<64, 3>(p, wgrid, stream)) : (launch_wgrad<128, 3>(p, wgrid, stream)));
      else HE_TRY(bn == 64 ? (launch_wgrad<64, 1>(p, wgrid, stream)) : (launch_wgrad<128, 1>(p, wgrid, stream)));
      const long long n = (long long)Kout * RS * Cin;
      conv_wgrad_fold<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(p.partials, outputs[0], fus.out_dtype, n, splits);
      HE_CUDA(cudaGetLastError());
      last_launches = 2;
      return HE_OK;
    }
    const bool fwd = kind == HE_CONV_FWD;
    const int Nout = fwd ? Kout : Cin;          // columns of the output
    const int Cred = fwd ? Cin : Kout;          // contraction channels per tap
    const int AH = fwd ? H : P, AW = fwd ? W : Q;   // grid of the activation operand (image / flow)
    const int OHt = fwd ? P : H, OWt = fwd ? Q : W; // output tensor grid
    if (memset_out) HE_CUDA(cudaMemsetAsync(outputs[0], 0, (size_t)NB * OHt * OWt * Nout * (fus.out_dtype == HE_F32 ? 4 : 2), stream));
    float* ws = reinterpret_cast<float*>(workspace);
    if (fus.want_stats) HE_CUDA(cudaMemsetAsync(workspace, 0, workspace_bytes, stream));   // CTAs add into their partial rows
    for (const Pass& ps : passes) {
      ConvParams p;
      memset(&p, 0, sizeof p);
      const int s = fwd ? prm.stride_h : 1;     // the data gradient reads the flow densely
      for (int ph = 0; ph < s; ++ph)
        for (int pw = 0; pw < s; ++pw)
          HE_TRY(make_activation_tmap(&p.tma_x[ph * 2 + pw], inputs[0], ab_format, NB, AH, AW, Cred, s, ph, pw, ps.geom.tw, ps.geom.th,
                                      ps.geom.tn));
      if (fwd) HE_TRY(make_filter_tmap(&p.tma_w, inputs[1], ab_format, Kout, RS, Cin, kBK, bn));
      else HE_TRY(make_filter_tmap(&p.tma_w, inputs[1], ab_format, Kout, RS, Cin, 64, kBK));
      p.core = c;
      p.core.num_tiles = ps.num_tiles;
      p.geom = ps.geom;
      EpiConvParams& e = p.epi;
      e.out = outputs[0];
      e.out_dt = fus.out_dtype;
      e.bias = s_bias >= 0 ? inputs[s_bias] : nullptr;
      e.bias_dt = fus.bias_dtype;
      e.resid = s_resid >= 0 ? inputs[s_resid] : nullptr;
      e.resid_dt = dtype;
      e.gate_x = s_gate_x >= 0 ? inputs[s_gate_x] : nullptr;
      e.gate_dt = dtype;
      e.gate_scale = s_gate_scale >= 0 ? reinterpret_cast<const float*>(inputs[s_gate_scale]) : nullptr;
      e.gate_shift = s_gate_shift >= 0 ? reinterpret_cast<const float*>(inputs[s_gate_shift]) : nullptr;
      e.stat0_partials = fus.want_stats ? ws + ws_stat_off[0] : nullptr;
      e.stat1_partials = fus.want_stats ? ws + ws_stat_off[1] : nullptr;
      bool vec = Nout % 8 == 0, vec32 = Nout % 16 == 0;
      const void* ptrs[] = {e.out, e.resid, e.gate_x};
      for (const void* q : ptrs) {
        vec = vec && ((uintptr_t)q % 16 == 0);
        vec32 = vec32 && ((uintptr_t)q % 32 == 0);
      }
      if (fus.out_dtype == HE_F32) vec32 = vec32 && Nout % 8 == 0;
      e.vec_ok = vec ? (vec32 ? 2 : 1) : 0;
      if (fwd) HE_TRY(bn == 64 ? (launch_fprop<64, false>(p, ps.grid, stream)) : (launch_fprop<128, false>(p, ps.grid, stream)));
      else HE_TRY(bn == 64 ? (launch_fprop<64, true>(p, ps.grid, stream)) : (launch_fprop<128, true>(p, ps.grid, stream)));
      ++last_launches;
    }
    if (fus.want_stats) {
      float* st = reinterpret_cast<float*>(outputs[1]);
      conv_stats_fold<<<(2 * Nout + 31) / 32, dim3(32, 32), 0, stream>>>(ws + ws_stat_off[0], ws + ws_stat_off[1], st, total_tiles_m, Nout);
      HE_CUDA(cudaGetLastError());
      ++last_launches;
    }
    return HE_OK;
  }
};

}  // namespace

int32_t plan_conv2d(he_ctx* ctx, int32_t kind, const he_conv2d_params* prm, int32_t batch, int32_t in_h, int32_t in_w, int32_t dtype,
                    const he_conv2d_fusion* fusion, he_plan** out) {
  if (!prm || !out) HE_FAIL(HE_ERR_INVALID, "he_plan_conv2d: null argument");
  *out = nullptr;
  if (kind < HE_CONV_FWD || kind > HE_CONV_BWD_FILTER) HE_FAIL(HE_ERR_INVALID, "he_plan_conv2d: unknown kind %d", kind);
  // Conv2dParams::validate (conv.rs:27-49)
  if (prm->in_channels <= 0 || prm->out_channels <= 0) HE_FAIL(HE_ERR_INVALID, "conv requires nonzero channel counts");
  if (prm->kernel_h <= 0 || prm->kernel_w <= 0) HE_FAIL(HE_ERR_INVALID, "conv filter must have nonzero size");
  if (prm->stride_h <= 0 || prm->stride_w <= 0) HE_FAIL(HE_ERR_INVALID, "stride cannot be zero");
  if (prm->dilation_h <= 0 || prm->dilation_w <= 0) HE_FAIL(HE_ERR_INVALID, "dilation cannot be zero");
  if (batch <= 0 || in_h <= 0 || in_w <= 0) HE_FAIL(HE_ERR_INVALID, "he_plan_conv2d: empty image");
  if (dtype != HE_BF16 && dtype != HE_F16) HE_FAIL(HE_ERR_UNSUPPORTED, "conv2d: images and filters must be bf16 or f16 (got %s)", dtype_name(dtype));
  if (prm->dilation_h != 1 || prm->dilation_w != 1) HE_FAIL(HE_ERR_UNSUPPORTED, "conv2d: dilation other than 1 is not implemented");
  if (prm->stride_h != prm->stride_w || prm->stride_h > 2) HE_FAIL(HE_ERR_UNSUPPORTED, "conv2d: strides other than 1x1 and 2x2 are not implemented");
  if (prm->kernel_h * prm->kernel_w > kConvMaxTaps) HE_FAIL(HE_ERR_UNSUPPORTED, "conv2d: filters above %d taps are not implemented", kConvMaxTaps);
  if (prm->in_channels % 8 != 0 || prm->out_channels % 8 != 0)
    HE_FAIL(HE_ERR_UNSUPPORTED, "conv2d: channel counts must be multiples of 8 (16-byte pixel pitch for TMA); pad %d / %d",
            prm->in_channels, prm->out_channels);
  const int R = prm->kernel_h, S = prm->kernel_w, s = prm->stride_h;
  // output size and padding, conv.rs:51-74, 86-94
  int oh = in_h, ow = in_w, pad_h = 0, pad_w = 0;
  switch (prm->padding_mode) {
    case HE_PAD_SAME: pad_h = R / 2; pad_w = S / 2; break;
    case HE_PAD_VALID: oh = std::max(0, oh - R / 2); ow = std::max(0, ow - S / 2); break;
    case HE_PAD_FULL: oh += R / 2; ow += S / 2; pad_h = R - 1; pad_w = S - 1; break;
    default: HE_FAIL(HE_ERR_INVALID, "he_plan_conv2d: unknown padding mode %d", prm->padding_mode);
  }
  const int P = oh / s, Q = ow / s;
  if (P <= 0 || Q <= 0) HE_FAIL(HE_ERR_INVALID, "he_plan_conv2d: the output is empty");

  auto plan = std::make_unique<ConvPlan>();
  plan->ctx = ctx;
  plan->kind = kind;
  plan->prm = *prm;
  if (fusion) plan->fus = *fusion;
  else { plan->fus = he_conv2d_fusion{}; plan->fus.out_dtype = dtype; plan->fus.bias_dtype = HE_F32; }
  he_conv2d_fusion& f = plan->fus;
  if (f.out_dtype != HE_BF16 && f.out_dtype != HE_F16 && f.out_dtype != HE_F32) HE_FAIL(HE_ERR_INVALID, "conv2d: output dtype must be a float type");
  plan->NB = batch; plan->H = in_h; plan->W = in_w; plan->P = P; plan->Q = Q; plan->pad_h = pad_h; plan->pad_w = pad_w;
  plan->dtype = dtype;
  plan->ab_format = dtype == HE_BF16 ? 1 : 0;
  GemmCore& c = plan->core;
  memset(&c, 0, sizeof c);
  c.ab_format = plan->ab_format;
  c.batch = 1;
  c.wait_limit_us = ptx::kDefaultWaitLimitUs;
  const int sms = ctx_sm_count(ctx);
  char desc[320];

  if (kind == HE_CONV_BWD_FILTER) {
    if (f.has_bias || f.has_resid || f.has_gate || f.want_stats) HE_FAIL(HE_ERR_UNSUPPORTED, "conv2d: the filter gradient takes no fused epilogue");
    plan->n_in = 2;
    c.M = prm->out_channels; c.N = prm->in_channels;
    plan->bn = c.N <= 64 ? 64 : 128;
    c.tiles_m = (c.M + kBM - 1) / kBM;
    c.tiles_n = (c.N + plan->bn - 1) / plan->bn;
    ConvGeom& g = plan->wgeom;
    memset(&g, 0, sizeof g);
    choose_patch(kBK, Q, P, batch, &g.tw, &g.th, &g.tn);
    g.GP = P; g.GQ = Q; g.GN = batch;
    g.tiles_q = (Q + g.tw - 1) / g.tw; g.tiles_p = (P + g.th - 1) / g.th; g.tiles_nb = (batch + g.tn - 1) / g.tn;
    g.n_taps = R * S;
    g.c_blocks = 1;
    for (int r = 0; r < R; ++r)
      for (int q = 0; q < S; ++q) {
        // input pixel of output (p, q') under tap (r, q): (s p + r - pad, s q' + q - pad)
        const int offh = r - pad_h, offw = q - pad_w;
        const int ph = ((offh % s) + s) % s, pw = ((offw % s) + s) % s;
        ConvTap& t = g.taps[r * S + q];
        t.dh = (short)floor_div(offh - ph, s); t.dw = (short)floor_div(offw - pw, s);
        t.map = (short)(ph * 2 + pw);
        t.tap = (short)(r * S + q);
      }
    plan->k_tiles = g.tiles_q * g.tiles_p * g.tiles_nb;
    // up to three taps share a CTA's flow tiles (three image tiles of 128 columns fill the 512 TMEM columns)
    plan->taps_per_cta = g.n_taps >= 3 ? 3 : 1;
    const int tap_groups = (g.n_taps + plan->taps_per_cta - 1) / plan->taps_per_cta;
    const int items = c.tiles_m * c.tiles_n * tap_groups;
    // one wave of CTAs (one per SM: a CTA's set-up, its f32 tile stores and the fold's reads grow with the
    // split count), at least 8 pixel tiles each
    int splits = std::max(1, sms / items);
    splits = std::min(splits, std::max(1, plan->k_tiles / 8));
    plan->splits = splits;
    plan->wgrid = items * splits;
    plan->workspace_bytes = (size_t)splits * c.M * R * S * c.N * sizeof(float);
    snprintf(desc, sizeof desc,
             "conv2d filter gradient: tcgen05 implicit GEMM 128x%dx64, K = %d x %d x %d pixels in patches %dx%dx%d, %d taps (%d per CTA) x %d splits, grid %d",
             plan->bn, batch, P, Q, g.tn, g.th, g.tw, g.n_taps, plan->taps_per_cta, splits, plan->wgrid);
    plan->description = desc;
    *out = plan.release();
    return HE_OK;
  }

  const bool fwd = kind == HE_CONV_FWD;
  // input slots after the two operands
  int slot = 2;
  if (f.has_bias) plan->s_bias = slot++;
  if (f.has_resid) plan->s_resid = slot++;
  if (f.has_gate) { plan->s_gate_x = slot++; plan->s_gate_scale = slot++; plan->s_gate_shift = slot++; }
  plan->n_in = slot;
  const int Nout = fwd ? prm->out_channels : prm->in_channels;
  const int Cred = fwd ? prm->in_channels : prm->out_channels;
  const int OH = fwd ? P : in_h, OW = fwd ? Q : in_w;
  c.M = batch * OH * OW;
  c.N = Nout;
  if ((long long)c.M * Nout >= (1ll << 31)) HE_FAIL(HE_ERR_UNSUPPORTED, "conv2d: output exceeds the 32-bit index range");
  plan->bn = Nout <= 64 ? 64 : 128;
  c.tiles_n = (Nout + plan->bn - 1) / plan->bn;
  const int os = fwd ? 1 : s;   // output parity classes of a strided data gradient
  int tile_m_base = 0;
  bool any_empty = false;
  for (int ch = 0; ch < os; ++ch)
    for (int cw = 0; cw < os; ++cw) {
      ConvPlan::Pass ps;
      ConvGeom& g = ps.geom;
      memset(&g, 0, sizeof g);
      g.GP = (OH - ch + os - 1) / os; g.GQ = (OW - cw + os - 1) / os; g.GN = batch;
      if (g.GP <= 0 || g.GQ <= 0) continue;
      g.OH = OH; g.OW = OW; g.os = os; g.oh0 = ch; g.ow0 = cw;
      g.c_blocks = (Cred + kBK - 1) / kBK;
      int nt = 0;
      for (int r = 0; r < R; ++r)
        for (int q = 0; q < S; ++q) {
          ConvTap t;
          t.tap = (short)(r * S + q);
          if (fwd) {
            const int offh = r - pad_h, offw = q - pad_w;
            const int ph = ((offh % s) + s) % s, pw = ((offw % s) + s) % s;
            t.dh = (short)floor_div(offh - ph, s); t.dw = (short)floor_div(offw - pw, s);
            t.map = (short)(ph * 2 + pw);
          } else {
            // dx[h] takes dy[(h + pad - r) / s] when divisible; h = s i + ch
            const int nh = ch + pad_h - r, nw = cw + pad_w - q;
            if (((nh % s) + s) % s != 0 || ((nw % s) + s) % s != 0) continue;
            t.dh = (short)floor_div(nh, s); t.dw = (short)floor_div(nw, s);
            t.map = 0;
          }
          g.taps[nt++] = t;
        }
      g.n_taps = nt;
      if (nt == 0) { any_empty = true; continue; }
      choose_patch(kBM, g.GQ, g.GP, batch, &g.tw, &g.th, &g.tn);
      g.tiles_q = (g.GQ + g.tw - 1) / g.tw; g.tiles_p = (g.GP + g.th - 1) / g.th; g.tiles_nb = (batch + g.tn - 1) / g.tn;
      const int tiles_m = g.tiles_q * g.tiles_p * g.tiles_nb;
      ps.num_tiles = tiles_m * c.tiles_n;
      ps.grid = std::max(1, std::min(ps.num_tiles, sms));
      ps.tile_m_base = tile_m_base;     // statistics partials: one row per CTA of every pass
      tile_m_base += ps.grid;
      plan->passes.push_back(ps);
    }
  if (plan->passes.empty()) HE_FAIL(HE_ERR_INVALID, "conv2d: nothing to compute");
  if (any_empty) {
    if (f.has_bias || f.has_resid || f.has_gate || f.want_stats)
      HE_FAIL(HE_ERR_UNSUPPORTED, "conv2d: this strided data gradient leaves output pixels no tap reaches; they are zero-filled, which "
                                  "a fused epilogue would have to see");
    plan->memset_out = true;
  }
  plan->total_tiles_m = tile_m_base;
  c.tiles_m = tile_m_base;
  for (ConvPlan::Pass& ps : plan->passes) ps.geom.tile_m_base = ps.tile_m_base;
  if (f.want_stats) {
    const size_t n = ((size_t)tile_m_base * Nout + 63) / 64 * 64;
    plan->ws_stat_off[0] = 0;
    plan->ws_stat_off[1] = n;
    plan->workspace_bytes = 2 * n * sizeof(float);
  }
  const ConvGeom& g0 = plan->passes[0].geom;
  snprintf(desc, sizeof desc,
           "conv2d %s: tcgen05 implicit GEMM 128x%dx64, %dx%d/%d pad %d,%d, [%d,%d,%d,%d] -> [%d,%d,%d,%d], patch %dx%dx%d, %d pass%s, "
           "epilogue(bias=%d resid=%d gate=%d stats=%d), grid %d",
           fwd ? "forward" : "data gradient", plan->bn, R, S, s, pad_h, pad_w, batch, fwd ? in_h : P, fwd ? in_w : Q, Cred, batch, OH, OW, Nout,
           g0.tn, g0.th, g0.tw, (int)plan->passes.size(), plan->passes.size() > 1 ? "es" : "", f.has_bias, f.has_resid, f.has_gate,
           f.want_stats, plan->passes[0].grid);
  plan->description = desc;
  *out = plan.release();
  return HE_OK;
}

}  // namespace he

extern "C" int32_t he_plan_conv2d(he_ctx* ctx, int32_t kind, const he_conv2d_params* params, int32_t batch, int32_t in_h, int32_t in_w,
                                  int32_t dtype, const he_conv2d_fusion* fusion, he_plan** out) {
  return he::plan_conv2d(ctx, kind, params, batch, in_h, in_w, dtype, fusion, out);
}
