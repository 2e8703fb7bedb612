// Implicit-GEMM 2-D convolution kernels for sm_100a on the tcgen05 / TMEM / TMA core.
//
// What they replace: the three cuDNN graphs the reference builds for Op::Conv, Op::ConvBackwardData and
// Op::ConvBackwardFilter (helium/src/cuda/instr/cudnn_graph.rs:182-228; geometry from
// helium-ir/src/opgraph/op/conv.rs:51-95; layouts NHWC for images and KRSC for filters,
// helium/src/raw_tensor.rs:232-240).  No im2col buffer exists anywhere: the "A" operand of the GEMM is
// fetched straight from the NHWC tensor, one filter tap and 64 channels at a time, by a 4-D TMA box whose
// pixel extent is a small patch of the output grid (tw x th pixels of tn images).  The tap's shift is an
// offset of the box's start coordinate, padding is the zero fill TMA gives out-of-range coordinates, and a
// stride of two is served by four tensor maps over the parity classes of the input (even / odd rows x
// even / odd columns), so that every load is a plain dense box.
//
//   conv_fprop_kernel   y[pix, ko]  = sum_{tap, c}  x[pix + tap, c] * w[ko, tap, c]           (forward)
//                       dx[pix, c]  = sum_{tap, ko} dy[pix - tap, ko] * w[ko, tap, c]          (data gradient:
//                       the same kernel with the filter read N-major and mirrored taps; a stride of two
//                       runs it once per parity class of the input grid)
//   conv_wgrad_kernel   dw[ko, tap, c] = sum_pix dy[pix, ko] * x[pix + tap, c]                 (filter gradient:
//                       both operands MN-major, the pixel axis is the contraction and is split over CTAs,
//                       a CTA multiplies one flow tile with the image tiles of up to three taps;
//                       f32 partial tiles go to the workspace and are folded in a fixed order)
//
// Roles, barriers, bounded waits and the abort path are those of gemm_tcgen05_kernel (gemm_sm100.cuh).
#pragma once
#include "gemm_sm100.cuh"

namespace he {

constexpr int kConvMaxTaps = 49;   // up to 7 x 7

struct ConvTap {
  short dh, dw;    // start-coordinate offset of the activation box for this tap, in the tensor map's pixel units
  short map;       // which of the (up to four) activation tensor maps
  short tap;       // filter tap index r * S + s (coordinate 1 of the filter map)
};

// Pixel patch of one M tile (forward / data gradient) or one K block (filter gradient): tn images x th rows
// x tw columns of the patch grid, all powers of two.  Patches may hang over the grid's edge; those pixels
// read zeros (TMA fill) and are never written.
struct ConvGeom {
  int tw, th, tn;
  int GP, GQ, GN;               // patch grid: rows, columns, images
  int tiles_q, tiles_p, tiles_nb;
  // where patch-grid pixel (n, p, q) lives in the OUTPUT tensor: ((n * OH + p * os + oh0) * OW + q * os + ow0)
  int OH, OW, os, oh0, ow0;
  int n_taps, c_blocks;         // k-blocks per tile = n_taps * c_blocks (64 channels each)
  int tile_m_base;              // first statistics-partial row of this pass; CTA b of the pass owns row tile_m_base + b
  ConvTap taps[kConvMaxTaps];
};

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// ---- epilogue of the forward / data-gradient kernel ------------------------------------------------
//   t = acc (+ bias[col]) (+ resid[pix, col]);
//   gate (backward through relu(x * s[col] + b[col])):  t = (gx[pix, col] * s[col] + b[col] > 0) ? t : 0;
//   out[pix, col] = t;   stats: S0[col] = sum_pix t,  S1[col] = sum_pix t * (gate ? gx : t)
// Forward use: bias, residual add, and the batch statistics (sum, sum of squares) of the tensor the next
// batch norm normalises (helium/src/modules/batch_norm.rs:38-65).  Backward use: the gradient arriving at a
// batch-normalised, rectified activation, masked by the rectifier, with the two sums batch norm's backward
// needs (sum g and sum g x).
struct EpiConvParams {
  void* out;
  const void* bias; const void* resid; const void* gate_x;
  const float* gate_scale; const float* gate_shift;
  float* stat0_partials; float* stat1_partials;
  int out_dt, bias_dt, resid_dt, gate_dt;
  int vec_ok;
};

struct EpiConv {
  using Params = EpiConvParams;
  // blocks 0, 1: the two column-sum scratch areas; block 2: bias / gate scale / gate shift slices of the tile
  static constexpr int kColReductions = 3;
  static constexpr int kChunk = 32;
  struct State {};
  __device__ static void tile_begin(const Params&, State&) {}
  __device__ static void tile_prepare(const Params& p, const EpiEnv& env, const TileInfo& t) {
    if (!p.bias && !p.gate_x) return;
    ptx::named_barrier_sync(1, env.n_epi_threads);   // the previous tile's chunks are done with the slices
    float* bs = env.scratch + 2 * 4 * env.bn;
    const int n = env.core->N;
    for (int i = env.epi_tid; i < env.bn; i += env.n_epi_threads) {
      const int gc = t.n0 + i;
      const bool ok = gc < n;
      bs[i] = (ok && p.bias) ? load_param_as_f32(p.bias, p.bias_dt, gc) : 0.0f;
      bs[env.bn + i] = (ok && p.gate_x) ? __ldg(p.gate_scale + gc) : 0.0f;
      bs[2 * env.bn + i] = (ok && p.gate_x) ? __ldg(p.gate_shift + gc) : 0.0f;
    }
    ptx::named_barrier_sync(1, env.n_epi_threads);
  }
  // `row` is the output pixel's linear index (or core->M for a patch pixel outside the grid)
  __device__ static void chunk(const Params& p, const EpiEnv& env, const TileInfo& t, State&, int row, int col, float (&v)[kChunk]) {
    const GemmCore& c = *env.core;
    const int gcol = t.n0 + col;
    const int nvalid = row < c.M ? max(0, min(kChunk, c.N - gcol)) : 0;
    const size_t off = (size_t)row * c.N + gcol;
    const int vec = p.vec_ok;
    const float* bs = env.scratch + 2 * 4 * env.bn;
    float aux[kChunk];
    if (p.bias) {
#pragma unroll
      for (int i = 0; i < kChunk; ++i) v[i] += bs[col + i];
    }
    if (p.resid) {
      load_row<kChunk>(p.resid, p.resid_dt, off, nvalid, vec, aux);
#pragma unroll
      for (int i = 0; i < kChunk; ++i) v[i] += aux[i];
    }
    if (p.gate_x) {
      load_row<kChunk>(p.gate_x, p.gate_dt, off, nvalid, vec, aux);
#pragma unroll
      for (int i = 0; i < kChunk; ++i) v[i] = fmaf(aux[i], bs[env.bn + col + i], bs[2 * env.bn + col + i]) > 0.0f ? v[i] : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < kChunk; ++i) v[i] = i < nvalid ? v[i] : 0.0f;
    if (nvalid > 0) store_row<kChunk>(p.out, p.out_dt, off, nvalid, vec, v);
    if (p.stat0_partials) {
      float s1[kChunk];
#pragma unroll
      for (int i = 0; i < kChunk; ++i) s1[i] = v[i] * (p.gate_x ? aux[i] : v[i]);   // aux is 0 where nvalid cuts
      warp_colsum_store<kChunk>(v, env.scratch + env.quadrant * env.bn + col);
      warp_colsum_store<kChunk>(s1, env.scratch + (4 + env.quadrant) * env.bn + col);
    }
  }
  // The two column sums go to ONE partial row per CTA (row = t.tile_m, which the kernel sets to the CTA's row):
  // a CTA adds every tile it processes into its own row, in its fixed tile order, so the fold that follows
  // reads at most one row per CTA instead of one per tile, and the result is still a fixed function of the
  // inputs.  The rows are zeroed by the host before the launch.
  __device__ static void tile_end(const Params& p, const EpiEnv& env, const TileInfo& t, State&) {
    if (!p.stat0_partials) return;
    ptx::named_barrier_sync(1, env.n_epi_threads);
    const GemmCore& c = *env.core;
    for (int col = env.epi_tid; col < t.bn; col += env.n_epi_threads) {
      const int gc = t.n0 + col;
      if (gc < c.N) {
        float* parts[2] = {p.stat0_partials, p.stat1_partials};
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const float* s = env.scratch + (size_t)r * 4 * env.bn;
          const float v = ((s[col] + s[env.bn + col]) + s[2 * env.bn + col]) + s[3 * env.bn + col];
          float* dst = parts[r] + (size_t)t.tile_m * c.N + gc;
          *dst += v;   // only this thread of this CTA ever touches this word
        }
      }
    }
    ptx::named_barrier_sync(1, env.n_epi_threads);
  }
};

struct alignas(64) ConvParams {
  CUtensorMap tma_x[4];   // activation (forward: image, data gradient: flow), one per input parity class
  CUtensorMap tma_w;      // filter as (C, R*S, K)
  GemmCore core;          // M = output pixels (all images), N = output columns, K unused, tiles_m = M tiles
  ConvGeom geom;
  EpiConvParams epi;
};

template <int BN, int STAGES>
struct ConvSmem {
  static constexpr int kBTileBytes = BN * kBK * 2;
  static constexpr int off_a = 0;
  static constexpr int off_b = off_a + STAGES * kATileBytes;
  static constexpr int off_scratch = off_b + STAGES * kBTileBytes;
  static constexpr int scratch_bytes = (EpiConv::kColReductions * 4 * BN + 64) * 4;
  static constexpr int off_bar = off_scratch + scratch_bytes;
  static constexpr int n_bars = 2 * STAGES + 4;
  static constexpr int off_misc = off_bar + n_bars * 8;
  static constexpr int total = off_misc + 16 + kConvMaxTaps * (int)sizeof(ConvTap);   // flags, then the tap table
  static constexpr int dynamic_bytes = total + 1024;
};

// B_MN = false: filter tiles are K-major ([ko rows][64 c], forward); true: N-major ([64 ko rows][c], data gradient).
template <int BN, int STAGES, bool B_MN>
__global__ void __launch_bounds__(32 * 11, 1) conv_fprop_kernel(const __grid_constant__ ConvParams p) {
  using SM = ConvSmem<BN, STAGES>;
  constexpr int NE_WARPS = 8;
  // TWO MMA-issuing threads (warps 1 and 10).  A tile's hand-over groups alternate between them and each
  // accumulates into its own TMEM half; the epilogue adds the halves.  The issuing thread was the bottleneck (~65
  // cycles per MMA statement against 32-64 cycles of tensor-pipe work at 64-128 columns); two accumulators keep
  // the order of every sum fixed, which two threads feeding one accumulator would not.
  constexpr int kIssuer1Warp = 2 + NE_WARPS;
  // shared memory is handed over two k-blocks at a time: the MMA-issuing thread spends ~65 cycles per MMA and
  // ~280 per hand-over (barrier wait, commit, bookkeeping), against 128-256 tensor-pipe cycles per k-block
  constexpr int KSUB = 2;
  constexpr int GROUPS = STAGES / KSUB;
  static_assert(STAGES % KSUB == 0, "stages are handed over in groups of KSUB");
  constexpr int kTmemCols = 4 * BN <= 256 ? 256 : 512;   // two tiles in flight x two halves
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = ptx::smem_u32(smem);
  const uint32_t bar0 = smem_base + SM::off_bar;
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto bar_tmem_full = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
  auto bar_tmem_empty = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem + SM::off_misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::off_misc + 4);
  float* scratch = reinterpret_cast<float*>(smem + SM::off_scratch);

  const GemmCore& c = p.core;
  const ConvGeom& g = p.geom;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_blocks = g.n_taps * g.c_blocks;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(bar_full(s), 1);
      ptx::mbar_init(bar_empty(s), 2);       // both issuing threads let go of a slot: see the MMA loop
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(bar_tmem_full(a), 2);   // one arrival per issuing thread
      ptx::mbar_init(bar_tmem_empty(a), NE_WARPS);
    }
    ptx::fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    for (int i = 0; i < 4; ++i) ptx::prefetch_tmap(&p.tma_x[i]);
    ptx::prefetch_tmap(&p.tma_w);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  // tile -> (column tile, patch origin); column tiles fastest so that neighbouring CTAs share the patch
  struct Origin { int n0, p0, q0, nb0, tile_m; };
  auto decode = [&](int tile) {
    Origin o;
    const int tn_ = tile % c.tiles_n;
    int m = tile / c.tiles_n;
    o.tile_m = g.tile_m_base + (int)blockIdx.x;
    o.n0 = tn_ * BN;
    const int qi = m % g.tiles_q; m /= g.tiles_q;
    const int pi = m % g.tiles_p; m /= g.tiles_p;
    o.q0 = qi * g.tw; o.p0 = pi * g.th; o.nb0 = m * g.tn;
    return o;
  };

  if (warp == 0) {
    if (lane == 0) {
      constexpr uint32_t kStageBytes = kATileBytes + SM::kBTileBytes;
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      // This thread's latency between "stage free" and "loads issued" is part of every stage's round trip, and the
      // round trip over the stages in flight is what paces the kernel.  An indexed read of the tap table in the
      // kernel-parameter block goes through a generic address (hundreds of cycles), and every inline-asm statement
      // makes the compiler reload parameter fields: the table goes to shared memory, the fields to registers,
      // and (tap, channel block) are counted instead of divided.  Measured: 7-8 % on every 3 x 3 layer.
      ConvTap* const s_taps = reinterpret_cast<ConvTap*>(smem + SM::off_misc + 16);
      for (int i = 0; i < g.n_taps; ++i) s_taps[i] = g.taps[i];
      const int c_blocks = g.c_blocks;
      DeviceStatus* const status = c.status;
      const uint32_t wait_us = c.wait_limit_us;
      for (int tile = blockIdx.x; alive && !c.withhold_loads && tile < c.num_tiles; tile += gridDim.x) {
        const Origin o = decode(tile);
        int ti = 0, cb_next = 0;
        for (int kb0 = 0; kb0 < k_blocks; kb0 += KSUB) {
          const int nsub = min(KSUB, k_blocks - kb0);
          if (!ptx::mbar_wait(bar_empty(stage), phase ^ 1u, abort_flag, status, 1, stage, wait_us)) { alive = false; break; }
          ptx::mbar_arrive_expect_tx(bar_full(stage), (uint32_t)nsub * kStageBytes);
#pragma unroll
          for (int u = 0; u < KSUB; ++u) {
          if (u >= nsub) break;
          const int slot = stage * KSUB + u;
          const ConvTap tp = s_taps[ti];
          const int cb = cb_next;
          if (++cb_next == c_blocks) { cb_next = 0; ++ti; }
          const uint32_t a_dst = smem_base + SM::off_a + slot * kATileBytes;
          const uint32_t b_dst = smem_base + SM::off_b + slot * SM::kBTileBytes;
          // activation: 64 channels x (tw x th x tn) pixels, shifted by the tap
          tma_load_4d(a_dst, &p.tma_x[tp.map], bar_full(stage), cb * kBK, o.q0 + tp.dw, o.p0 + tp.dh, o.nb0);
          if (B_MN) {
            // rows = 64 contraction channels (ko), columns = output channels c: boxes of 64 columns
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              ptx::tma_load_3d(b_dst + j * (kBK * 128), &p.tma_w, bar_full(stage), o.n0 + 64 * j, tp.tap, cb * kBK);
          } else {
            // rows = BN output channels (ko), columns = 64 contraction channels c
            ptx::tma_load_3d(b_dst, &p.tma_w, bar_full(stage), cb * kBK, tp.tap, o.n0);
          }
          }   // u
          if (++stage == GROUPS) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1 || warp == kIssuer1Warp) {
    if (lane == 0) {
      const int me = warp == 1 ? 0 : 1;
      const uint32_t idesc = ptx::make_idesc_f16(c.ab_format, 0, B_MN ? 1 : 0, kBM, BN);
      constexpr uint32_t b_lbo = B_MN ? kBK * 128 : 16;
      constexpr uint32_t b_kadv = B_MN ? 2048 : 32;
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool alive = true;
      DeviceStatus* const status = c.status;
      const uint32_t wait_us = c.wait_limit_us;
      for (int tile = blockIdx.x; alive && tile < c.num_tiles; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
        if (!ptx::mbar_wait(bar_tmem_empty(acc), acc_phase ^ 1u, abort_flag, status, 2, acc, wait_us)) { alive = false; break; }
        ptx::tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)((acc * 2 + me) * BN);
        bool first = true;
        int g_idx = 0;
        for (int kb0 = 0; kb0 < k_blocks; kb0 += KSUB, ++g_idx) {
          // every group advances the ring for both issuers; a group belongs to the issuer of its parity
          const int my_stage = stage;
          const uint32_t my_phase = phase;
          if (++stage == GROUPS) { stage = 0; phase ^= 1u; }
          // Both threads wait for EVERY group, also the other thread's.  A parity wait only tells "the latest phase
          // of this parity has completed": a thread that skipped the other's phase L of a slot and came back for
          // phase L + 1 while L was still loading (loads of different groups complete in any order) was let through
          // by phase L - 1, issued MMAs on stale tiles and released the slot a second time -- about once in 10^4
          // launches the ring then stopped.  Observing every phase in ring order rules that out, and because the
          // slot goes back to the producer only when BOTH threads have let go of it (the one that multiplies it
          // when its MMAs have retired, the other one here), neither can fall a lap behind a barrier it still has
          // to observe.  tests/test_pipeline_model_cpu.py runs the three protocols under random interleavings.
          if (!ptx::mbar_wait(bar_full(my_stage), my_phase, abort_flag, status, 3, my_stage, wait_us)) { alive = false; break; }
          if ((g_idx & 1) != me) {
            ptx::mbar_arrive(bar_empty(my_stage));
            continue;
          }
          const int nsub = min(KSUB, k_blocks - kb0);
          ptx::tcgen05_fence_after();
#pragma unroll
          for (int u = 0; u < KSUB; ++u) {
            if (u >= nsub) break;
            const int slot = my_stage * KSUB + u;
            const uint32_t a_addr = smem_base + SM::off_a + slot * kATileBytes;
            const uint32_t b_addr = smem_base + SM::off_b + slot * SM::kBTileBytes;
#pragma unroll
            for (int k = 0; k < kBK / kUmmaK; ++k) {
              const uint64_t adesc = ptx::make_smem_desc_sw128(a_addr + k * 32, 16, 1024);
              const uint64_t bdesc = ptx::make_smem_desc_sw128(b_addr + k * b_kadv, b_lbo, 1024);
              ptx::umma_f16(d_tmem, adesc, bdesc, idesc, (first && u == 0 && k == 0) ? 0u : 1u);
            }
          }
          first = false;
          ptx::umma_commit(bar_empty(my_stage));
        }
        if (alive) {
          if (!first) ptx::umma_commit(bar_tmem_full(acc));   // arrives when this thread's MMAs have retired
          else ptx::mbar_arrive(bar_tmem_full(acc));           // a tile of one group: nothing from this thread
        }
      }
    }
  } else if (warp >= 2 && warp < 2 + NE_WARPS) {
    EpiEnv env;
    env.core = &c;
    env.scratch = scratch;
    env.bn = BN;
    env.n_epi_threads = NE_WARPS * 32;
    env.epi_warp = warp - 2;
    env.epi_tid = env.epi_warp * 32 + lane;
    env.quadrant = warp & 3;
    constexpr int kColsPerWarp = BN / (NE_WARPS / 4);
    const int col_begin = (env.epi_warp / 4) * kColsPerWarp;
    // this thread's pixel within the patch: row = (in * th + ih) * tw + iw
    const int prow = env.quadrant * 32 + lane;
    const int iw = prow & (g.tw - 1);
    const int ih = (prow / g.tw) & (g.th - 1);
    const int in = prow / (g.tw * g.th);
    int it = 0;
    bool dead = false;
    for (int tile = blockIdx.x; tile < c.num_tiles; tile += gridDim.x, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
      const Origin o = decode(tile);
      TileInfo t;
      t.m0 = 0; t.n0 = o.n0; t.b = 0; t.tile_m = o.tile_m; t.tile_n = o.n0 / BN; t.tile_idx = tile; t.bn = BN;
      const int n = o.nb0 + in, pp = o.p0 + ih, qq = o.q0 + iw;
      const bool inside = n < g.GN && pp < g.GP && qq < g.GQ && in < g.tn;
      const int pix = inside ? ((n * g.OH + pp * g.os + g.oh0) * g.OW + qq * g.os + g.ow0) : c.M;
      EpiConv::tile_prepare(p.epi, env, t);
      if (!dead && !ptx::mbar_wait(bar_tmem_full(acc), acc_phase, abort_flag, c.status, 4, acc, c.wait_limit_us)) dead = true;
      dead = __any_sync(0xffffffffu, dead);
      EpiConv::State st;
      EpiConv::tile_begin(p.epi, st);
      if (!dead) {
        ptx::tcgen05_fence_after();
        const uint32_t taddr0 = tmem_base + ((uint32_t)(env.quadrant * 32) << 16) + (uint32_t)(acc * 2 * BN);
        const int col_end = min(col_begin + kColsPerWarp, ((c.N - t.n0 + 31) / 32) * 32);
        const bool two_halves = k_blocks > KSUB;   // the second issuer had at least one group
#pragma unroll 1
        for (int col = col_begin; col < col_end; col += EpiConv::kChunk) {
          float v[EpiConv::kChunk];
          tmem_ld_chunk<EpiConv::kChunk>(taddr0 + (uint32_t)col, v);
          if (two_halves) {
            float w[EpiConv::kChunk];
            tmem_ld_chunk<EpiConv::kChunk>(taddr0 + (uint32_t)(BN + col), w);
#pragma unroll
            for (int i = 0; i < EpiConv::kChunk; ++i) v[i] += w[i];
          }
          EpiConv::chunk(p.epi, env, t, st, pix, col, v);
        }
        ptx::tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(bar_tmem_empty(acc));
      }
      EpiConv::tile_end(p.epi, env, t, st);
    }
  }

  ptx::tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tcgen05_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- filter gradient -----------------------------------------------------------------------------------
struct alignas(64) ConvWgradParams {
  CUtensorMap tma_dy;     // flow as (K, Q, P, N), box 64 x patch
  CUtensorMap tma_x[4];   // image parity classes as (C, W', H', N), box 64 x patch
  GemmCore core;          // M = K (output channels), N = C (input channels); tiles_m / tiles_n over them
  ConvGeom geom;          // patch = one K block of 64 pixels; taps = all filter taps
  float* partials;        // [splits][K][R*S][C] f32
  int splits, k_tiles;    // pixel tiles in all, and how many CTAs share them
  int tap_groups;         // ceil(taps / T): a CTA owns the taps [g * T, g * T + T)
  int rs;                 // R * S
};

template <int BN, int STAGES, int T>
struct ConvWgradSmem {
  static constexpr int kBTapBytes = BN * kBK * 2;          // one tap's image tile
  static constexpr int kBTileBytes = T * kBTapBytes;
  static constexpr int off_a = 0;
  static constexpr int off_b = off_a + STAGES * kATileBytes;
  static constexpr int off_bar = off_b + STAGES * kBTileBytes;
  static constexpr int n_bars = 2 * STAGES + 1;
  static constexpr int off_misc = off_bar + n_bars * 8;
  static constexpr int total = off_misc + 16;
  static constexpr int dynamic_bytes = total + 1024;
};

// One CTA = one (output tile, group of T taps, split): it contracts its share of the pixel tiles and writes
// one f32 tile per tap.  The flow tile of a pixel block is fetched once and multiplied with the T shifted image
// tiles of the group, each tap into its own TMEM columns: what bounds these kernels is the rate at which TMA
// fills shared memory, and sharing the flow tile cuts the bytes per tap from (128 + BN) to (128 / T + BN) rows.
template <int BN, int STAGES, int T>
__global__ void __launch_bounds__(32 * 8, 1) conv_wgrad_kernel(const __grid_constant__ ConvWgradParams p) {
  using SM = ConvWgradSmem<BN, STAGES, T>;
  constexpr int kIssuers = 3;
  constexpr int kTmemCols = T * BN <= 64 ? 64 : T * BN <= 128 ? 128 : T * BN <= 256 ? 256 : 512;
  static_assert(T * BN <= 512, "the taps of a group share the 512 TMEM columns");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = ptx::smem_u32(smem);
  const uint32_t bar0 = smem_base + SM::off_bar;
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (STAGES + s); };
  const uint32_t bar_done = bar0 + 8u * (2 * STAGES);
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem + SM::off_misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::off_misc + 4);

  const GemmCore& c = p.core;
  const ConvGeom& g = p.geom;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // work item
  int item = blockIdx.x;
  const int split = item % p.splits; item /= p.splits;
  const int tg = item % p.tap_groups; item /= p.tap_groups;
  const int tile_n = item % c.tiles_n;
  const int tile_m = item / c.tiles_n;
  const int m0 = tile_m * kBM, n0 = tile_n * BN;
  const int kt_begin = (int)(((long long)p.k_tiles * split) / p.splits);
  const int kt_end = (int)(((long long)p.k_tiles * (split + 1)) / p.splits);
  const int tap0 = tg * T;
  const int nt = min(T, g.n_taps - tap0);   // taps of this group (the last group may be short)

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(bar_full(s), 1);
      ptx::mbar_init(bar_empty(s), kIssuers);   // a stage is free when both issuing threads' MMAs on it have retired
    }
    ptx::mbar_init(bar_done, kIssuers);
    ptx::fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tmap(&p.tma_dy);
    for (int t = 0; t < nt; ++t) ptx::prefetch_tmap(&p.tma_x[g.taps[tap0 + t].map]);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0 && !c.withhold_loads) {
      const uint32_t stage_bytes = kATileBytes + (uint32_t)nt * SM::kBTapBytes;
      int stage = 0;
      uint32_t phase = 0;
      // the group's taps and the geometry in registers, the pixel-tile coordinates counted instead of divided
      // (see the producer of conv_fprop_kernel)
      ConvTap taps[T];
#pragma unroll
      for (int t = 0; t < T; ++t) taps[t] = g.taps[min(tap0 + t, g.n_taps - 1)];
      const int tiles_q = g.tiles_q, tiles_p = g.tiles_p, tw = g.tw, th = g.th, tn = g.tn;
      DeviceStatus* const status = c.status;
      const uint32_t wait_us = c.wait_limit_us;
      int qi = kt_begin % tiles_q, pi = (kt_begin / tiles_q) % tiles_p, ni = kt_begin / (tiles_q * tiles_p);
      for (int kt = kt_begin; kt < kt_end; ++kt) {
        if (!ptx::mbar_wait(bar_empty(stage), phase ^ 1u, abort_flag, status, 1, stage, wait_us)) break;
        ptx::mbar_arrive_expect_tx(bar_full(stage), stage_bytes);
        const int q0 = qi * tw, p0 = pi * th, nb0 = ni * tn;
        if (++qi == tiles_q) { qi = 0; if (++pi == tiles_p) { pi = 0; ++ni; } }
        const uint32_t a_dst = smem_base + SM::off_a + stage * kATileBytes;
        const uint32_t b_dst = smem_base + SM::off_b + stage * SM::kBTileBytes;
        // A = flow^T: 64 pixels (contraction) x 128 output channels, as two boxes of 64 channels
#pragma unroll
        for (int j = 0; j < kBM / 64; ++j) tma_load_4d(a_dst + j * (kBK * 128), &p.tma_dy, bar_full(stage), m0 + 64 * j, q0, p0, nb0);
        // B = the image shifted by each tap of the group: 64 pixels x BN input channels per tap
#pragma unroll
        for (int t = 0; t < T; ++t) {
          if (t < nt) {
            const ConvTap tp = taps[t];
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_4d(b_dst + t * SM::kBTapBytes + j * (kBK * 128), &p.tma_x[tp.map], bar_full(stage), n0 + 64 * j, q0 + tp.dw,
                          p0 + tp.dh, nb0);
          }
        }
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1 || warp >= 6) {
    // Three MMA-issuing threads: the taps of the group are dealt out to them (each tap has its own TMEM columns, so
    // every sum keeps its order); one thread paid ~65 cycles per MMA statement against 32-64 of tensor-pipe work.
    if (lane == 0) {
      const int me = warp == 1 ? 0 : warp - 5;
      const uint32_t idesc = ptx::make_idesc_f16(c.ab_format, 1, 1, kBM, BN);
      DeviceStatus* const status = c.status;
      const uint32_t wait_us = c.wait_limit_us;
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int kt = kt_begin; kt < kt_end; ++kt) {
        if (!ptx::mbar_wait(bar_full(stage), phase, abort_flag, status, 3, stage, wait_us)) { alive = false; break; }
        ptx::tcgen05_fence_after();
        const uint32_t a_addr = smem_base + SM::off_a + stage * kATileBytes;
        const uint32_t b_addr = smem_base + SM::off_b + stage * SM::kBTileBytes;
#pragma unroll
        for (int t = 0; t < T; ++t) {
          if (t >= nt || (t % kIssuers) != me) continue;
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            const uint64_t adesc = ptx::make_smem_desc_sw128(a_addr + k * 2048, kBK * 128, 1024);
            const uint64_t bdesc = ptx::make_smem_desc_sw128(b_addr + t * SM::kBTapBytes + k * 2048, kBK * 128, 1024);
            ptx::umma_f16(tmem_base + (uint32_t)(t * BN), adesc, bdesc, idesc, (kt > kt_begin || k != 0) ? 1u : 0u);
          }
        }
        // with a single tap the second thread has no MMAs of its own: a commit with nothing outstanding arrives at once
        ptx::umma_commit(bar_empty(stage));
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
      if (alive) ptx::umma_commit(bar_done);
    }
  } else if (warp >= 2 && warp < 6) {
    // four epilogue warps: rows = output channels of the filter, columns = input channels of one tap
    const int quadrant = warp & 3;
    const int row = quadrant * 32 + lane;
    const int ko = m0 + row;
    bool ok = kt_end > kt_begin;
    if (ok) ok = ptx::mbar_wait(bar_done, 0, abort_flag, c.status, 4, 0, c.wait_limit_us);
    ok = __all_sync(0xffffffffu, ok);
    ptx::tcgen05_fence_after();
    const bool vec = (c.N & 3) == 0;   // a lane's 32 columns are then eight aligned 16-byte words
    for (int t = 0; t < nt; ++t) {
      float* dst = p.partials + (((size_t)split * c.M + ko) * p.rs + g.taps[tap0 + t].tap) * c.N + n0;
#pragma unroll 1
      for (int col = 0; col < BN; col += 32) {
        if (n0 + col >= c.N) break;
        float v[32];
        if (ok) {
          tmem_ld_chunk<32>(tmem_base + ((uint32_t)(quadrant * 32) << 16) + (uint32_t)(t * BN + col), v);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0.0f;   // an empty share of the pixel tiles contributes zeros
        }
        if (ko < c.M) {
          const int nvalid = min(32, c.N - (n0 + col));
          if (vec && nvalid == 32) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(dst + col + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < nvalid) dst[col + i] = v[i];
          }
        }
      }
    }
    ptx::tcgen05_fence_before();
  }

  ptx::tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tcgen05_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace he
