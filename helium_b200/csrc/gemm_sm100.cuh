// tcgen05 / TMEM / TMA GEMM core for sm_100a with mainloop and epilogue fusion (hot-path rows
// G0-G3, F1-F2).
//
// What it replaces: the sm_80 `mma.sync` + `cp.async` CuTe kernel the reference's generator emits
// (helium-kernel-generator/templates/matmul/sm80.cu:202-274, src/generators/matmul/sm80.rs:551-695)
// and the sm_90a WGMMA template of the playground (helium-playground/src/templates/matmul.cu).
// Nothing is shared with either: one persistent CTA per SM, warp-specialised --
//   warp 0        TMA producer: A / B (/ mask) tiles, 128-byte swizzle, STAGES-deep mbarrier ring
//   warp 1        single-thread tcgen05.mma issuer, 128 x BN x 16 per instruction, f32 accumulators
//                 in TMEM, two accumulator buffers so the epilogue of tile i overlaps tile i+1
//   warps 2..     epilogue: tcgen05.ld 32x32b -> registers -> fused functor -> global
//   last 4 warps  (mainloop fusion only) rewrite the A tile in shared memory between TMA arrival
//                 and MMA issue, then fence.proxy.async + mbarrier arrive
// Operands may be K-major or MN-major in global memory; the transposed case only changes the TMA
// box and the shared-memory descriptor, no data is moved.
#pragma once
#include "device_utils.cuh"
#include "pointwise_interp.cuh"
#include "sm100_ptx.cuh"

namespace he {

constexpr int kBM = 128;
constexpr int kBK = 64;                       // 64 bf16 = one 128-byte swizzle row
constexpr int kATileBytes = kBM * kBK * 2;    // 16 KiB
constexpr int kUmmaK = 16;

// ML_RELU | ML_MASK is the hand-written relu(A) * mask rewrite on packed bf16 pairs.  ML_GENERIC runs a short
// program of unary steps and at most one elementwise multiply / add with a second tensor (staged like the mask,
// ML_MASK then says that tensor exists) on the A tile, and a unary-only program on the B tile (single-CTA kernel).
enum MainloopKind : int { ML_NONE = 0, ML_RELU = 1, ML_MASK = 2, ML_RELU_MASK = 3, ML_GENERIC = 4, ML_GENERIC_MASK = 6,
                          ML_F8 = 8 };   // ML_F8: plain mainloop over 8-bit operand tiles (tcgen05 kind::f8f6f4), no rewrite
// true when transform warps rewrite the A (and B) tiles between TMA arrival and MMA issue
__host__ __device__ constexpr bool ml_transforms(int ml) { return (ml & 7) != 0; }
constexpr int kMlMaxSteps = 6;
struct MlStep {
  unsigned char kind;   // 0 unary (op = he_unary_op, imm = constant bits), 1 multiply by the second tensor, 2 add it
  unsigned char op;
  unsigned short pad;
  unsigned imm;
};
struct MlProg {
  int n;
  MlStep s[kMlMaxSteps];
};
enum ActKind : int { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU = 2, ACT_TANH = 3 };
enum GateKind : int { GATE_NONE = 0, GATE_MUL = 1, GATE_DGELU = 2, GATE_DRELU = 3, GATE_DTANH = 4 };

struct GemmCore {
  int M, N, K, batch;
  int tiles_m, tiles_n, num_tiles, k_blocks;
  int ab_format;  // 0 = f16, 1 = bf16
  // 8-bit multiplication (MulF8Accum*, helium-ir/src/opgraph/op/precision.rs:60-81): bit 0 set = the operand tiles
  // are 8-bit floats (K-major, 128 elements of K per 128-byte row), bit 1 = A is E5M2, bit 2 = B is E5M2 (else E4M3)
  int f8;
  int group_m;    // tile rasterisation: row tiles per group (see decode_tile)
  // Pair-tile kernel only: tiles [split_from, split_from + split_count) of the tile list are walked
  // as two half-width tiles each, by different CTA pairs (see finish_tiles in gemm_plan.cu).
  int split_from, split_count;
  // Bound of every device-side wait in microseconds (2 s by default).  `withhold_loads` is the host-side
  // fault injection of the tests: the TMA producers issue nothing, so the first wait on a full barrier
  // runs into the limit and the kernel leaves through its abort path (results are then undefined and
  // he_ctx_poll_device_status reports HE_ERR_DEVICE_TIMEOUT).  Set only by he_debug_plan_fault_injection.
  unsigned wait_limit_us;
  int withhold_loads;
  int k_serpentine;   // pair kernel: odd tiles of a CTA walk K from the end (L2 reuse between waves)
  MlProg ml_a, ml_b;  // ML_GENERIC: operand-side programs (ml_b: unary steps only)
  DeviceStatus* status;
};

struct TileInfo {
  int m0, n0, b, tile_m, tile_n, tile_idx;
  int bn;   // columns of this tile (the kernel's BN, or half of it for the split tiles of the last round)
};

// ---- row-segment load / store helpers (one thread owns CH consecutive columns of one row) -------
template <int CH>
__device__ __forceinline__ void load_row(const void* base, int dt, size_t elem_off, int nvalid, int vec, float (&o)[CH]) {
  // vec: 0 scalar accesses, 1 the segment is 16-byte aligned, 2 it is 32-byte aligned as well (256-bit
  // accesses: a warp whose lanes sit on 32 different rows then issues half as many load/store-unit
  // wavefronts for the same bytes)
  if (dt == HE_F32) {
    const float* p = reinterpret_cast<const float*>(base) + elem_off;
    if (vec == 2 && nvalid == CH && CH % 8 == 0) {
#pragma unroll
      for (int i = 0; i < CH / 8; ++i) {
        uint32_t r[8];
        ptx::ld_global_nc_256(p + 8 * i, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[8 * i + j] = __uint_as_float(r[j]);
      }
    } else if (vec && nvalid == CH) {
#pragma unroll
      for (int i = 0; i < CH / 4; ++i) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(p) + i);
        o[4 * i] = v.x; o[4 * i + 1] = v.y; o[4 * i + 2] = v.z; o[4 * i + 3] = v.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < CH; ++i) o[i] = i < nvalid ? __ldg(p + i) : 0.0f;
    }
  } else {
    const unsigned short* p = reinterpret_cast<const unsigned short*>(base) + elem_off;
    if (vec == 2 && nvalid == CH && dt == HE_BF16 && CH % 16 == 0) {
#pragma unroll
      for (int i = 0; i < CH / 16; ++i) {
        uint32_t r[8];
        ptx::ld_global_nc_256(p + 16 * i, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o[16 * i + 2 * j] = __uint_as_float(r[j] << 16);
          o[16 * i + 2 * j + 1] = __uint_as_float(r[j] & 0xffff0000u);
        }
      }
    } else if (vec && nvalid == CH && dt == HE_BF16) {
#pragma unroll
      for (int i = 0; i < CH / 8; ++i) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(p) + i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          o[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
          o[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const uint32_t h = i < nvalid ? (uint32_t)__ldg(p + i) : 0u;
        o[i] = dt == HE_BF16 ? bf16_bits_to_f32(h) : f16_bits_to_f32(h);
      }
    }
  }
}

template <int CH>
__device__ __forceinline__ void store_row(void* base, int dt, size_t elem_off, int nvalid, int vec, const float (&v)[CH]) {
  if (dt == HE_F32) {
    float* p = reinterpret_cast<float*>(base) + elem_off;
    if (vec == 2 && nvalid == CH && CH % 8 == 0) {
#pragma unroll
      for (int i = 0; i < CH / 8; ++i) {
        uint32_t r[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) r[j] = __float_as_uint(v[8 * i + j]);
        ptx::st_global_256(p + 8 * i, r);
      }
    } else if (vec && nvalid == CH) {
#pragma unroll
      for (int i = 0; i < CH / 4; ++i) reinterpret_cast<float4*>(p)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < CH; ++i)
        if (i < nvalid) p[i] = v[i];
    }
  } else {
    unsigned short* p = reinterpret_cast<unsigned short*>(base) + elem_off;
    if (vec == 2 && nvalid == CH && dt == HE_BF16 && CH % 16 == 0) {
#pragma unroll
      for (int i = 0; i < CH / 16; ++i) {
        uint32_t r[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) r[j] = f32x2_to_bf16x2(v[16 * i + 2 * j], v[16 * i + 2 * j + 1]);
        ptx::st_global_256(p + 16 * i, r);
      }
    } else if (vec && nvalid == CH && dt == HE_BF16) {
#pragma unroll
      for (int i = 0; i < CH / 8; ++i) {
        uint4 w;
        w.x = f32x2_to_bf16x2(v[8 * i], v[8 * i + 1]);
        w.y = f32x2_to_bf16x2(v[8 * i + 2], v[8 * i + 3]);
        w.z = f32x2_to_bf16x2(v[8 * i + 4], v[8 * i + 5]);
        w.w = f32x2_to_bf16x2(v[8 * i + 6], v[8 * i + 7]);
        reinterpret_cast<uint4*>(p)[i] = w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < CH; ++i)
        if (i < nvalid) p[i] = (unsigned short)(dt == HE_BF16 ? f32_to_bf16_bits(v[i]) : f32_to_f16_bits(v[i]));
    }
  }
}

// Column sums over the 32 lanes (= 32 rows) of a warp for CH per-lane values.  Recursive halving
// (CH - 1 shuffles) followed by 5 - log2(CH) all-reduce steps.  Afterwards the lanes whose low
// (5 - log2 CH) bits are zero hold the total of column (lane >> (5 - log2 CH)); this helper writes
// those totals to dst[0 .. CH).
template <int CH>
__device__ __forceinline__ void warp_colsum_store(float (&v)[CH], float* dst) {
  const int lane = threadIdx.x & 31;
  constexpr int kLog = CH == 32 ? 5 : CH == 16 ? 4 : 3;
  int bit = 16;
#pragma unroll
  for (int s = CH / 2; s >= 1; s >>= 1) {
    const bool upper = (lane & bit) != 0;
#pragma unroll
    for (int i = 0; i < s; ++i) {
      const float send = upper ? v[i] : v[i + s];
      const float keep = upper ? v[i + s] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
    }
    bit >>= 1;
  }
#pragma unroll
  for (int b = (1 << (5 - kLog)) >> 1; b >= 1; b >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], b);
  if ((lane & ((1 << (5 - kLog)) - 1)) == 0) dst[lane >> (5 - kLog)] = v[0];
}

// The same exchange pattern for Sum (0), Max (1) or Min (2), chosen at run time (interpreted epilogue).
__device__ __forceinline__ float red_combine(float a, float b, int op) { return op == 1 ? fmaxf(a, b) : op == 2 ? fminf(a, b) : a + b; }
__device__ __forceinline__ float red_identity(int op) { return op == 1 ? -INFINITY : op == 2 ? INFINITY : 0.0f; }
template <int CH>
__device__ __forceinline__ void warp_colreduce_store(float (&v)[CH], float* dst, int op) {
  const int lane = threadIdx.x & 31;
  constexpr int kLog = CH == 32 ? 5 : CH == 16 ? 4 : 3;
  int bit = 16;
#pragma unroll
  for (int s = CH / 2; s >= 1; s >>= 1) {
    const bool upper = (lane & bit) != 0;
#pragma unroll
    for (int i = 0; i < s; ++i) {
      const float send = upper ? v[i] : v[i + s];
      const float keep = upper ? v[i + s] : v[i];
      v[i] = red_combine(keep, __shfl_xor_sync(0xffffffffu, send, bit), op);
    }
    bit >>= 1;
  }
#pragma unroll
  for (int b = (1 << (5 - kLog)) >> 1; b >= 1; b >>= 1) v[0] = red_combine(v[0], __shfl_xor_sync(0xffffffffu, v[0], b), op);
  if ((lane & ((1 << (5 - kLog)) - 1)) == 0) dst[lane >> (5 - kLog)] = v[0];
}

// ---- generic mainloop rewrite of one 16-byte vector (8 operand elements) -----------------------------
// The reference's generator applies the operand-side pointwise chain to register fragments in f32 and casts
// to the MMA type (helium-kernel-generator/src/generators/matmul/sm80.rs:396-439); here the chain runs on the
// tile in shared memory between TMA arrival and MMA issue: unpack to f32, steps in order, one rounding back.
__device__ __forceinline__ void ml_unpack8(const uint4& v, int fmt, float (&x)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (fmt == 1) { x[2 * j] = __uint_as_float(w[j] << 16); x[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u); }
    else { x[2 * j] = f16_bits_to_f32(w[j] & 0xffffu); x[2 * j + 1] = f16_bits_to_f32(w[j] >> 16); }
  }
}
__device__ __forceinline__ uint4 ml_pack8(const float (&x)[8], int fmt) {
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
    w[j] = fmt == 1 ? f32x2_to_bf16x2(x[2 * j], x[2 * j + 1]) : (f32_to_f16_bits(x[2 * j]) | (f32_to_f16_bits(x[2 * j + 1]) << 16));
  return make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ void ml_apply8(const MlProg& P, int fmt, uint4& va, const uint4* second) {
  float x[8], m[8];
  ml_unpack8(va, fmt, x);
  if (second) ml_unpack8(*second, fmt, m);
#pragma unroll 1
  for (int i = 0; i < P.n; ++i) {
    const MlStep st = P.s[i];
    if (st.kind == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = pw_unary(st.op, x[j], st.imm);
    } else if (second) {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = st.kind == 1 ? x[j] * m[j] : x[j] + m[j];
    }
  }
  va = ml_pack8(x, fmt);
}

// =================================================================================================
// Epilogue functors.  Interface:
//   Params                      POD passed by value inside the kernel parameter block
//   kColReductions              number of per-column Sum reductions (shared scratch rows)
//   State                       per-thread state that lives across the chunks of one tile
//   chunk(...)                  called once per (row, 32-column chunk) with the f32 accumulators
//   tile_end(...)               called by every epilogue thread after the accumulator was released
// Column partial layout in the workspace: [reduction][batch][tile_m][N]; scalar partials: [tile].
// =================================================================================================
struct EpiEnv {
  const GemmCore* core;
  float* scratch;      // shared: [kColReductions][4 quadrants][BN] then [n_epi_warps] scalars
  int bn;
  int n_epi_threads;
  int epi_tid;         // 0 .. n_epi_threads-1
  int quadrant;        // TMEM lane quadrant of this warp (row block within the tile)
  int epi_warp;
};

__device__ __forceinline__ void col_partials_flush(const EpiEnv& env, const TileInfo& t, int nred, float* const* partials,
                                                   const int* ops = nullptr) {
  ptx::named_barrier_sync(1, env.n_epi_threads);
  const GemmCore& c = *env.core;
  for (int col = env.epi_tid; col < t.bn; col += env.n_epi_threads) {
    const int gc = t.n0 + col;
    if (gc < c.N) {
      for (int r = 0; r < nred; ++r) {
        const float* s = env.scratch + (size_t)r * 4 * env.bn;
        const int op = ops ? ops[r] : 0;
        const float v = red_combine(red_combine(red_combine(s[col], s[env.bn + col], op), s[2 * env.bn + col], op), s[3 * env.bn + col], op);
        partials[r][((size_t)t.b * c.tiles_m + t.tile_m) * c.N + gc] = v;
      }
    }
  }
  ptx::named_barrier_sync(1, env.n_epi_threads);
}

// ---- EpiFlex: bias / residual / activation / gate / column sum ----------------------------------
//   t = acc (+ bias[col]) (+ resid[row, col]);  Z = t (optional);  y = act(t);
//   y *= gate(G[row, col]) (optional);  Y = y;  colsum over {nothing, resid, y}
struct EpiFlexParams {
  void* out; void* out_z;
  const void* bias; const void* resid; const void* gate_in;
  float* colsum_partials;
  int out_dt, z_dt, bias_dt, resid_dt, gate_dt;
  int bias_vec;   // bias pointer and N allow 16-byte loads
  int act, gate, colsum_src;  // colsum_src: 0 none, 1 resid, 2 y
  int vec_ok;     // 1: 16-byte row segments are aligned; 2: 32-byte ones are too
};

// erf by Abramowitz & Stegun 7.1.26 (|error| <= 1.5e-7, below f32 rounding of the results it feeds):
// one reciprocal, one exp2 and a 5-term Horner chain instead of libm's branchy erff.  Used only in
// the GEMM epilogues, where the functor shares the SM with the tensor pipe.
__device__ __forceinline__ float fast_erf(float x) {
  const float ax = fabsf(x);
  const float t = __fdividef(1.0f, fmaf(0.3275911f, ax, 1.0f));
  float poly = fmaf(1.061405429f, t, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  const float y = 1.0f - poly * t * __expf(-ax * ax);
  return copysignf(y, x);
}
// tanh x = 1 - 2 / (1 + e^(2x)) on the exp2 / reciprocal units: absolute error ~2e-7 (libm's tanhf
// costs ~30 instructions per element, which made the README epilogue outlast its mainloop).
// Saturates correctly: e = inf gives 1, e = 0 gives -1.
__device__ __forceinline__ float exp2f_approx(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float fast_tanh(float x) { return 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * x)); }
__device__ __forceinline__ float fast_gelu(float x) { return 0.5f * x * (1.0f + fast_erf(x * 0.70710678118654752440f)); }
__device__ __forceinline__ float fast_dgelu(float x) {
  const float cdf = 0.5f * (1.0f + fast_erf(x * 0.70710678118654752440f));
  return fmaf(x * 0.39894228040143267794f, __expf(-0.5f * x * x), cdf);
}

// ---- GELU / GELU' on column pairs -----------------------------------------------------------------
// The same approximations as fast_erf / fast_gelu / fast_dgelu with the polynomial, the scalings and the
// final combinations as packed f32x2 operations (two IEEE-rounded f32 results per instruction); only the
// reciprocal and the exponential stay scalar.  1 + 0.3275911 |x| >= 1, so the bare reciprocal is safe.
__device__ __forceinline__ unsigned long long erf_pair(unsigned long long x2, unsigned long long* exp_neg_sq = nullptr) {
  using u64 = unsigned long long;
  const u64 ax = x2 & 0x7fffffff7fffffffull;
  float da, db;
  ptx::f2_unpack(ptx::f2_fma(ax, ptx::f2_pack(0.3275911f, 0.3275911f), ptx::f2_pack(1.0f, 1.0f)), da, db);
  const u64 t = ptx::f2_pack(rcp_approx(da), rcp_approx(db));
  u64 poly = ptx::f2_fma(ptx::f2_pack(1.061405429f, 1.061405429f), t, ptx::f2_pack(-1.453152027f, -1.453152027f));
  poly = ptx::f2_fma(poly, t, ptx::f2_pack(1.421413741f, 1.421413741f));
  poly = ptx::f2_fma(poly, t, ptx::f2_pack(-0.284496736f, -0.284496736f));
  poly = ptx::f2_fma(poly, t, ptx::f2_pack(0.254829592f, 0.254829592f));
  float ea, eb;
  ptx::f2_unpack(ptx::f2_mul(ptx::f2_mul(ax, ax), ptx::f2_pack(-1.4426950408889634f, -1.4426950408889634f)), ea, eb);
  const u64 e = ptx::f2_pack(exp2f_approx(ea), exp2f_approx(eb));
  if (exp_neg_sq) *exp_neg_sq = e;   // exp(-x^2) of the argument, for callers that need it as well
  const u64 y = ptx::f2_fma(ptx::f2_mul(ptx::f2_mul(poly, t), e), ptx::f2_pack(-1.0f, -1.0f), ptx::f2_pack(1.0f, 1.0f));
  return y | (x2 & 0x8000000080000000ull);   // y is in [0, 1]: or-ing the sign of x is copysign
}
__device__ __forceinline__ void gelu_pair(float& a, float& b) {
  const unsigned long long x2 = ptx::f2_pack(a, b);
  const unsigned long long e2 = erf_pair(ptx::f2_mul(x2, ptx::f2_pack(0.70710678118654752440f, 0.70710678118654752440f)));
  const unsigned long long hx = ptx::f2_mul(x2, ptx::f2_pack(0.5f, 0.5f));
  ptx::f2_unpack(ptx::f2_fma(hx, e2, hx), a, b);   // 0.5 x (1 + erf)
}
// (va, vb) *= gelu'(xa, xb)
__device__ __forceinline__ void dgelu_mul_pair(float& va, float& vb, float xa, float xb) {
  using u64 = unsigned long long;
  const u64 x2 = ptx::f2_pack(xa, xb);
  // erf is taken at x / sqrt 2, whose exp(-(.)^2) is the exp(-x^2 / 2) of the density term
  u64 pdf;
  const u64 e2 = erf_pair(ptx::f2_mul(x2, ptx::f2_pack(0.70710678118654752440f, 0.70710678118654752440f)), &pdf);
  const u64 cdf = ptx::f2_fma(e2, ptx::f2_pack(0.5f, 0.5f), ptx::f2_pack(0.5f, 0.5f));
  const u64 d = ptx::f2_fma(ptx::f2_mul(x2, ptx::f2_pack(0.39894228040143267794f, 0.39894228040143267794f)), pdf, cdf);
  ptx::f2_unpack(ptx::f2_mul(ptx::f2_pack(va, vb), d), va, vb);
}

struct EpiFlex {
  using Params = EpiFlexParams;
  // block 0: column-sum scratch; block 1: the tile's bias slice as f32 (tile_prepare)
  static constexpr int kColReductions = 2;
  static constexpr int kChunk = 32;
  struct State {};
  __device__ static void tile_begin(const Params&, State&) {}
  // Every epilogue thread, once per tile, before the accumulator is awaited: the tile's bias slice goes
  // to shared memory as f32, so that the chunks do not put an L2 round trip on their dependent chain.
  // The previous tile's readers are behind this barrier pair and the barriers of tile_end.
  __device__ static void tile_prepare(const Params& p, const EpiEnv& env, const TileInfo& t) {
    if (!p.bias) return;
    ptx::named_barrier_sync(1, env.n_epi_threads);   // the previous tile's chunks are done with the slice
    float* bs = env.scratch + 4 * env.bn;
    const int n = env.core->N;
    for (int i = env.epi_tid; i < env.bn; i += env.n_epi_threads) {
      const int gc = t.n0 + i;
      bs[i] = gc < n ? load_param_as_f32(p.bias, p.bias_dt, gc) : 0.0f;
    }
    ptx::named_barrier_sync(1, env.n_epi_threads);
  }
  // The op selectors are uniform per launch: switch once per chunk, not once per element.
  __device__ static void activate(int act, float (&v)[kChunk]) {
    switch (act) {
      case ACT_RELU:
#pragma unroll
        for (int i = 0; i < kChunk; ++i) v[i] = fmaxf(v[i], 0.0f);
        break;
      case ACT_GELU:
#pragma unroll
        for (int i = 0; i < kChunk; i += 2) gelu_pair(v[i], v[i + 1]);
        break;
      case ACT_TANH:
#pragma unroll
        for (int i = 0; i < kChunk; ++i) v[i] = fast_tanh(v[i]);
        break;
      default: break;
    }
  }
  __device__ static void apply_gate(int g, float (&v)[kChunk], const float (&x)[kChunk]) {
    switch (g) {
      case GATE_DGELU:
#pragma unroll
        for (int i = 0; i < kChunk; i += 2) dgelu_mul_pair(v[i], v[i + 1], x[i], x[i + 1]);
        break;
      case GATE_DRELU:
#pragma unroll
        for (int i = 0; i < kChunk; ++i) v[i] = x[i] > 0.0f ? v[i] : 0.0f;
        break;
      case GATE_DTANH:   // x is tanh(z)
#pragma unroll
        for (int i = 0; i < kChunk; ++i) v[i] *= 1.0f - x[i] * x[i];
        break;
      default:
#pragma unroll
        for (int i = 0; i < kChunk; ++i) v[i] *= x[i];
        break;
    }
  }
  __device__ static void chunk(const Params& p, const EpiEnv& env, const TileInfo& t, State&, int row, int col, float (&v)[kChunk]) {
    const GemmCore& c = *env.core;
    const int grow = t.m0 + row, gcol = t.n0 + col;
    const int nvalid = grow < c.M ? max(0, min(kChunk, c.N - gcol)) : 0;
    const size_t off = ((size_t)t.b * c.M + grow) * c.N + gcol;
    const int vec = p.vec_ok;
    float aux[kChunk];
    if (p.bias) {
      const float4* bs = reinterpret_cast<const float4*>(env.scratch + 4 * env.bn + col);   // staged by tile_prepare
#pragma unroll
      for (int i = 0; i < kChunk / 4; ++i) {
        const float4 b = bs[i];
        v[4 * i] += b.x; v[4 * i + 1] += b.y; v[4 * i + 2] += b.z; v[4 * i + 3] += b.w;
      }
    }
    if (p.resid) {
      load_row<kChunk>(p.resid, p.resid_dt, off, nvalid, vec, aux);
#pragma unroll
      for (int i = 0; i < kChunk; ++i) v[i] += aux[i];
      if (p.colsum_src == 1) warp_colsum_store<kChunk>(aux, env.scratch + env.quadrant * env.bn + col);
    }
    if (p.out_z && nvalid > 0) store_row<kChunk>(p.out_z, p.z_dt, off, nvalid, vec, v);
    if (p.act != ACT_NONE) activate(p.act, v);
    if (p.gate != GATE_NONE) {
      load_row<kChunk>(p.gate_in, p.gate_dt, off, nvalid, vec, aux);
      apply_gate(p.gate, v, aux);
    }
    if (nvalid > 0) store_row<kChunk>(p.out, p.out_dt, off, nvalid, vec, v);
    if (p.colsum_src == 2) {
#pragma unroll
      for (int i = 0; i < kChunk; ++i) v[i] = i < nvalid ? v[i] : 0.0f;
      warp_colsum_store<kChunk>(v, env.scratch + env.quadrant * env.bn + col);
    }
  }
  __device__ static void tile_end(const Params& p, const EpiEnv& env, const TileInfo& t, State&) {
    if (p.colsum_src != 0) {
      float* parts[1] = {p.colsum_partials};
      col_partials_flush(env, t, 1, parts);
    }
  }
};

// ---- EpiC3: the fused graph of the reference README (README.md:33-79) ---------------------------
//   z1 = C (+E1) + b1[col];  u = relu(z1);      z2 = C (+E2) + b2[col];  t = tanh(z2)
//   h  = (1 - u) * Mk + u * t;   d = h - Y;   l = d*d * inv_n;   LOSS = sum_all(l)
//   g  = d * 2 * inv_n;          gt = (u * g) * (1 - t*t);       DB2 = colsum(gt)
//   gu = g * t - g * Mk;         gz1 = z1 > 0 ? gu : 0;          DB1 = colsum(gz1)
struct EpiC3Params {
  const void* mask; const void* y; const void* b1; const void* b2; const void* e1; const void* e2;
  void* out_gt; void* out_gz1;
  float* db2_partials; float* db1_partials; float* loss_partials;
  float inv_n;       // MulConstant operand of README node 38 / 45
  int full_dt;       // dtype of mask / y / e1 / e2 / gt / gz1
  int vec_dt;        // dtype of b1 / b2
  int vec_ok;        // 1: 16-byte row segments are aligned; 2: 32-byte ones are too
  int bias_vec;      // b1 / b2 pointers and N allow 16-byte loads
};

struct EpiC3 {
  using Params = EpiC3Params;
  // two column-sum scratch blocks and a third block of the same size whose first 2 * BN floats hold the
  // tile's b1 and b2 values (see tile_prepare)
  static constexpr int kColReductions = 3;
  static constexpr int kChunk = 16;
  struct State { float loss; };
  __device__ static void tile_begin(const Params&, State& s) { s.loss = 0.0f; }
  // Called by every epilogue thread once per tile, before the accumulator is awaited (so it overlaps
  // the tile's mainloop): the tile's slice of both bias vectors goes to shared memory as f32.  Reading
  // them from global memory in every chunk put two L2 round trips on each chunk's dependent chain (L1
  // keeps next to nothing beside 200 KB of pipeline stages).  The previous tile's readers are behind
  // the barriers of its tile_end.
  __device__ static void tile_prepare(const Params& p, const EpiEnv& env, const TileInfo& t) {
    float* bs = env.scratch + 2 * 4 * env.bn;
    const int n = env.core->N;
    for (int i = env.epi_tid; i < 2 * env.bn; i += env.n_epi_threads) {
      const int which = i >= env.bn ? 1 : 0;
      const int gc = t.n0 + (i - which * env.bn);
      bs[i] = gc < n ? load_param_as_f32(which ? p.b2 : p.b1, p.vec_dt, gc) : 0.0f;
    }
    ptx::named_barrier_sync(1, env.n_epi_threads);
  }
  __device__ static void chunk(const Params& p, const EpiEnv& env, const TileInfo& t, State& st, int row, int col, float (&v)[kChunk]) {
    const GemmCore& c = *env.core;
    const int grow = t.m0 + row, gcol = t.n0 + col;
    const int nvalid = grow < c.M ? max(0, min(kChunk, c.N - gcol)) : 0;
    const size_t off = ((size_t)t.b * c.M + grow) * c.N + gcol;
    const int vec = p.vec_ok;
    float tnh[kChunk], a[kChunk];
    if (p.e2) {
      load_row<kChunk>(p.e2, p.full_dt, off, nvalid, vec, a);
#pragma unroll
      for (int i = 0; i < kChunk; ++i) tnh[i] = v[i] + a[i];
    } else {
#pragma unroll
      for (int i = 0; i < kChunk; ++i) tnh[i] = v[i];
    }
    if (p.e1) {
      load_row<kChunk>(p.e1, p.full_dt, off, nvalid, vec, a);
#pragma unroll
      for (int i = 0; i < kChunk; ++i) v[i] += a[i];
    }
    {
      const float4* s1 = reinterpret_cast<const float4*>(env.scratch + 2 * 4 * env.bn + col);
      const float4* s2 = reinterpret_cast<const float4*>(env.scratch + 2 * 4 * env.bn + env.bn + col);
      // z1 = c + b1 and t = tanh(c + b2) = 1 - 2 / (1 + e^(2 z2)) on column pairs: the adds, the scaling
      // of the exponent and the final 1 - q are packed f32x2 operations with the roundings of fast_tanh
      using u64 = unsigned long long;
      const u64 one2 = ptx::f2_pack(1.0f, 1.0f), neg2b = ptx::f2_pack(-2.0f, -2.0f);
      const u64 l2e2 = ptx::f2_pack(2.0f * 1.4426950408889634f, 2.0f * 1.4426950408889634f);
#pragma unroll
      for (int i = 0; i < kChunk / 4; ++i) {
        const float4 x = s1[i], y = s2[i];
        const float bx[4] = {x.x, x.y, x.z, x.w}, by[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int k = 4 * i + 2 * h;
          const u64 z1 = ptx::f2_fma(ptx::f2_pack(bx[2 * h], bx[2 * h + 1]), one2, ptx::f2_pack(v[k], v[k + 1]));
          ptx::f2_unpack(z1, v[k], v[k + 1]);
          const u64 z2 = ptx::f2_fma(ptx::f2_pack(by[2 * h], by[2 * h + 1]), one2, ptx::f2_pack(tnh[k], tnh[k + 1]));
          float ea, eb;
          ptx::f2_unpack(ptx::f2_mul(z2, l2e2), ea, eb);
          const u64 s = ptx::f2_fma(ptx::f2_pack(exp2f_approx(ea), exp2f_approx(eb)), one2, one2);
          float sa, sb;
          ptx::f2_unpack(s, sa, sb);
          // 1 + e >= 1, so the bare reciprocal needs none of the range handling of an approximate divide
          const u64 r = ptx::f2_pack(rcp_approx(sa), rcp_approx(sb));
          ptx::f2_unpack(ptx::f2_fma(r, neg2b, one2), tnh[k], tnh[k + 1]);
        }
      }
    }
    float mk[kChunk];
    // 16 bf16 columns are one 32-byte segment per lane.  Both 256-bit loads are issued before either is
    // unpacked, and both stores after both tiles are packed: measured 3.5 % faster on the 4096^3 README
    // graph than the same accesses made tensor by tensor through load_row / store_row.
    const bool wide = vec == 2 && nvalid == kChunk && kChunk == 16 && p.full_dt == HE_BF16;
    if (wide) {
      uint32_t qm[8], qy[8];
      ptx::ld_global_nc_256(reinterpret_cast<const unsigned short*>(p.mask) + off, qm);
      ptx::ld_global_nc_256(reinterpret_cast<const unsigned short*>(p.y) + off, qy);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        mk[2 * j] = __uint_as_float(qm[j] << 16); mk[2 * j + 1] = __uint_as_float(qm[j] & 0xffff0000u);
        a[2 * j] = __uint_as_float(qy[j] << 16); a[2 * j + 1] = __uint_as_float(qy[j] & 0xffff0000u);
      }
    } else {
      load_row<kChunk>(p.mask, p.full_dt, off, nvalid, vec, mk);
      load_row<kChunk>(p.y, p.full_dt, off, nvalid, vec, a);
    }
    // The graph's op order is relaxed where it only moves roundings (all intermediates are f32, the
    // outputs are bf16 tiles and f32 sums checked to 1e-2 / 1e-5): h = m + u (t - m) instead of
    // (1 - u) m + u t, g (t - m) instead of g t - g m, and the loss is summed as d^2 and scaled by
    // 1/n once per tile.  That is 19 instead of 30 instructions per element in an epilogue whose
    // issue slots, not its memory traffic, bound the kernel.
    float loss = 0.0f;
    const float g_scale = 2.0f * p.inv_n;
    auto element = [&](int i, float& gt, float& gz1, float& dd) {
      const float z1 = v[i], tt = tnh[i], m = mk[i];
      const float u = fmaxf(z1, 0.0f);
      const float tm = tt - m;
      const float d = fmaf(u, tm, m) - a[i];
      const float g = d * g_scale;
      gt = (u * g) * fmaf(-tt, tt, 1.0f);
      gz1 = z1 > 0.0f ? g * tm : 0.0f;
      dd = d;
    };
    if (nvalid == kChunk) {
      // interior chunk: no per-element predicates, and the arithmetic runs on pairs of columns with the
      // packed f32x2 instructions.  Every packed lane is the same IEEE operation as in `element`
      // (t - m as fma(m, -1, t); (u * -g) * (t^2 - 1) for (u * g) * (1 - t^2): negation commutes with
      // rounding), so both paths give the same bits; only the loss is summed as two interleaved chains.
      using u64 = unsigned long long;
      const u64 neg1 = ptx::f2_pack(-1.0f, -1.0f), gs2 = ptx::f2_pack(g_scale, g_scale), ngs2 = ptx::f2_pack(-g_scale, -g_scale);
      u64 loss2 = ptx::f2_pack(0.0f, 0.0f);
#pragma unroll
      for (int j = 0; j < kChunk / 2; ++j) {
        const float z1a = v[2 * j], z1b = v[2 * j + 1];
        const u64 u = ptx::f2_pack(fmaxf(z1a, 0.0f), fmaxf(z1b, 0.0f));
        const u64 tt = ptx::f2_pack(tnh[2 * j], tnh[2 * j + 1]);
        const u64 m = ptx::f2_pack(mk[2 * j], mk[2 * j + 1]);
        const u64 y = ptx::f2_pack(a[2 * j], a[2 * j + 1]);
        const u64 tm = ptx::f2_fma(m, neg1, tt);
        const u64 d = ptx::f2_fma(y, neg1, ptx::f2_fma(u, tm, m));
        const u64 g = ptx::f2_mul(d, gs2), ng = ptx::f2_mul(d, ngs2);
        const u64 gt = ptx::f2_mul(ptx::f2_mul(u, ng), ptx::f2_fma(tt, tt, neg1));
        const u64 gm = ptx::f2_mul(g, tm);
        loss2 = ptx::f2_fma(d, d, loss2);
        ptx::f2_unpack(gt, v[2 * j], v[2 * j + 1]);
        float ga, gb;
        ptx::f2_unpack(gm, ga, gb);
        tnh[2 * j] = z1a > 0.0f ? ga : 0.0f;
        tnh[2 * j + 1] = z1b > 0.0f ? gb : 0.0f;
      }
      float la, lb;
      ptx::f2_unpack(loss2, la, lb);
      loss = la + lb;
    } else {
#pragma unroll
      for (int i = 0; i < kChunk; ++i) {
        float gt, gz1, d;
        element(i, gt, gz1, d);
        const bool ok = i < nvalid;
        loss = ok ? fmaf(d, d, loss) : loss;
        v[i] = ok ? gt : 0.0f;
        tnh[i] = ok ? gz1 : 0.0f;
      }
    }
    st.loss += loss;
    if (wide) {
      uint32_t w0[8], w1[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        w0[j] = f32x2_to_bf16x2(v[2 * j], v[2 * j + 1]);
        w1[j] = f32x2_to_bf16x2(tnh[2 * j], tnh[2 * j + 1]);
      }
      ptx::st_global_256(reinterpret_cast<unsigned short*>(p.out_gt) + off, w0);
      ptx::st_global_256(reinterpret_cast<unsigned short*>(p.out_gz1) + off, w1);
    } else if (nvalid > 0) {
      store_row<kChunk>(p.out_gt, p.full_dt, off, nvalid, vec, v);
      store_row<kChunk>(p.out_gz1, p.full_dt, off, nvalid, vec, tnh);
    }
    warp_colsum_store<kChunk>(v, env.scratch + env.quadrant * env.bn + col);
    warp_colsum_store<kChunk>(tnh, env.scratch + (4 + env.quadrant) * env.bn + col);
  }
  __device__ static void tile_end(const Params& p, const EpiEnv& env, const TileInfo& t, State& st) {
    float l = st.loss * p.inv_n;   // chunk() sums d^2
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) l += __shfl_down_sync(0xffffffffu, l, off);
    float* scal = env.scratch + (size_t)kColReductions * 4 * env.bn;
    if ((threadIdx.x & 31) == 0) scal[env.epi_warp] = l;
    float* parts[2] = {p.db2_partials, p.db1_partials};
    col_partials_flush(env, t, 2, parts);   // its first barrier also publishes scal[]
    if (env.epi_tid == 0) {
      float tot = 0.0f;
      for (int w = 0; w < env.n_epi_threads / 32; ++w) tot += scal[w];
      p.loss_partials[t.tile_idx] = tot;
    }
    // scal[] is rewritten only after the next tile's flush barrier pair, which orders it after this read
  }
};

// ---- EpiProgram: generic tier, the pointwise interpreter fed with accumulator values -------------
// Any legal pointwise epilogue, plus up to four Sum reductions of pointwise expressions of the tile
// (the playground's Reduction{Sum, depth}, helium-playground/src/opgraph.rs:397-413):
//   kind 0  over rows (Columns, -> [b,1,N], or [1,1,N] when the batch is folded in): values are
//           summed over the warp's 32 rows, the four row quadrants meet in shared memory, one partial
//           per (M tile, column);
//   kind 1  over columns (Rows, -> [b,M,1]): a thread owns a row, so it keeps a running sum over
//           the chunks it walks and writes one partial per 64-column slot of the row;
//   kind 2  over the whole tile (Item with batch 1, Batch, -> one scalar): running sum per thread,
//           shuffle tree, one partial per CTA tile.
// Fixed-order folds of the partials (gemm_colsum_finalize / gemm_scalar_finalize) finish the job,
// so results repeat bit for bit.
struct EpiProgramParams {
  PwProgram prog;  // by value: lives in the kernel parameter block (constant bank)
  int n_red;             // reductions of the program (PwInstr::slot2 numbers them)
  int red_kind[4];       // per reduction slot: 0 columns, 1 rows, 2 scalar
  int red_op[4];         // 0 sum (also mean: scaled by the fold), 1 max, 2 min
  float* red_partials[4];
  int n_col;             // kind-0 reductions (at most kColReductions)
  int col_slot[2];       // their reduction slots
  int rows_total;        // batch * M
};
struct EpiProgram {
  using Params = EpiProgramParams;
  static constexpr int kColReductions = 2;
  static constexpr int kChunk = 32;
  struct State { float red[4]; };
  __device__ static void tile_begin(const Params& p, State& s) {
#pragma unroll
    for (int i = 0; i < 4; ++i) s.red[i] = p.red_op[i] == 1 ? -INFINITY : p.red_op[i] == 2 ? INFINITY : 0.0f;
  }
  __device__ static void tile_prepare(const Params&, const EpiEnv&, const TileInfo&) {}
  __device__ static void chunk(const Params& p, const EpiEnv& env, const TileInfo& t, State& st, int row, int col, float (&v)[kChunk]) {
    const GemmCore& c = *env.core;
    const int grow = t.m0 + row, gcol = t.n0 + col;
    float cbuf[kColReductions][kChunk];
    int col_op[kColReductions];
#pragma unroll
    for (int r = 0; r < kColReductions; ++r) col_op[r] = r < p.n_col ? p.red_op[p.col_slot[r]] : 0;
    if (p.n_col > 0) {
#pragma unroll
      for (int r = 0; r < kColReductions; ++r)
#pragma unroll
        for (int i = 0; i < kChunk; ++i) cbuf[r][i] = red_identity(col_op[r]);
    }
    if (grow < c.M) {
      const uint32_t base = (uint32_t)(((size_t)t.b * c.M + grow) * c.N + gcol);
      const bool row_aligned = (c.N & 3) == 0;
      // rolled on purpose: the interpreter body is large, eight inlined copies would not fit the
      // instruction cache (cbuf then lives in local memory, which only programs with column sums touch)
#pragma unroll 1
      for (int i = 0; i < kChunk; i += 4) {
        const int nv = max(0, min(4, c.N - (gcol + i)));
        if (nv > 0) {
          const float acc4[4] = {v[i], v[i + 1], v[i + 2], v[i + 3]};
          float cv[4][4];
          if (row_aligned) {
            pw_run<4>(p.prog, base + i, nv, acc4, st.red, p.n_col > 0 ? cv : nullptr);
          } else {
            for (int j = 0; j < nv; ++j) {
              float cv1[4][1];
              pw_run<1>(p.prog, base + i + j, 1, acc4 + j, st.red, p.n_col > 0 ? cv1 : nullptr);
#pragma unroll
              for (int s = 0; s < 4; ++s) cv[s][j] = cv1[s][0];
            }
            for (int j = nv; j < 4; ++j)
#pragma unroll
              for (int s = 0; s < 4; ++s) cv[s][j] = 0.0f;
          }
          if (p.n_col > 0) {
#pragma unroll
            for (int r = 0; r < kColReductions; ++r) {
              const int s = p.col_slot[r];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float x = s == 0 ? cv[0][j] : s == 1 ? cv[1][j] : s == 2 ? cv[2][j] : cv[3][j];
                if (r < p.n_col && j < nv) cbuf[r][i + j] = x;
              }
            }
          }
        }
      }
    }
    // every lane of the warp takes part in the shuffles, rows beyond M contribute the identity
#pragma unroll
    for (int r = 0; r < kColReductions; ++r)
      if (r < p.n_col) warp_colreduce_store<kChunk>(cbuf[r], env.scratch + (r * 4 + env.quadrant) * env.bn + col, col_op[r]);
  }
  __device__ static void tile_end(const Params& p, const EpiEnv& env, const TileInfo& t, State& st) {
    if (p.n_red == 0) return;
    const GemmCore& c = *env.core;
    const int lane = threadIdx.x & 31;
    float* scal = env.scratch + (size_t)kColReductions * 4 * env.bn;   // [reduction][epilogue warp]
    const int n_warps = env.n_epi_threads / 32;
    bool any_scalar = false;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      if (s >= p.n_red) break;
      if (p.red_kind[s] == 1) {
        // one partial per 64-column slot of the row; a warp that covers more than one slot puts its
        // sum into the first and zeros into the rest, so that the fold may read every slot
        const int cols_per_warp = t.bn / (n_warps / 4);
        const int col_begin = (env.epi_warp / 4) * cols_per_warp;
        const int grow = t.m0 + env.quadrant * 32 + lane;
        if (grow < c.M) {
          const int slot0 = (t.n0 + col_begin) / 64;
          const size_t r = (size_t)t.b * c.M + grow;
          for (int k = 0; k < cols_per_warp / 64; ++k)
            p.red_partials[s][(size_t)(slot0 + k) * p.rows_total + r] =
                k == 0 ? st.red[s] : (p.red_op[s] == 1 ? -INFINITY : p.red_op[s] == 2 ? INFINITY : 0.0f);
        }
      } else if (p.red_kind[s] == 2) {
        float l = st.red[s];
        const int op = p.red_op[s];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
          const float o = __shfl_down_sync(0xffffffffu, l, off);
          l = op == 1 ? fmaxf(l, o) : op == 2 ? fminf(l, o) : l + o;
        }
        if (lane == 0) scal[s * n_warps + env.epi_warp] = l;
        any_scalar = true;
      }
    }
    if (p.n_col > 0) {
      float* parts[kColReductions] = {p.red_partials[p.col_slot[0]], p.red_partials[p.col_slot[p.n_col > 1 ? 1 : 0]]};
      const int ops[kColReductions] = {p.red_op[p.col_slot[0]], p.red_op[p.col_slot[p.n_col > 1 ? 1 : 0]]};
      col_partials_flush(env, t, p.n_col, parts, ops);   // its first barrier also publishes scal[]
    } else if (any_scalar) {
      ptx::named_barrier_sync(1, env.n_epi_threads);
    }
    if (any_scalar) {
      if (env.epi_tid == 0) {
        for (int s = 0; s < p.n_red; ++s)
          if (p.red_kind[s] == 2) {
            const int op = p.red_op[s];
            float tot = scal[s * n_warps];
            for (int w = 1; w < n_warps; ++w) {
              const float o = scal[s * n_warps + w];
              tot = op == 1 ? fmaxf(tot, o) : op == 2 ? fminf(tot, o) : tot + o;
            }
            p.red_partials[s][t.tile_idx] = tot;
          }
      }
      ptx::named_barrier_sync(1, env.n_epi_threads);   // scal[] may be rewritten for the next tile
    }
  }
};

// =================================================================================================
// The kernel
// =================================================================================================
template <class EP>
struct alignas(64) GemmParams {
  CUtensorMap tma_a, tma_b, tma_mask;
  GemmCore core;
  EP epi;
};

template <int BN, int STAGES, int ML, int N_COLRED>
struct GemmSmem {
  static constexpr int kBTileBytes = BN * kBK * 2;
  static constexpr bool kHasMask = (ML & ML_MASK) != 0;
  static constexpr int off_a = 0;
  static constexpr int off_b = off_a + STAGES * kATileBytes;
  static constexpr int off_mask = off_b + STAGES * kBTileBytes;
  static constexpr int off_scratch = off_mask + (kHasMask ? STAGES * kATileBytes : 0);
  static constexpr int scratch_bytes = (N_COLRED * 4 * BN + 64) * 4;
  static constexpr int off_bar = off_scratch + scratch_bytes;
  static constexpr int n_bars = 3 * STAGES + 4;
  static constexpr int off_misc = off_bar + n_bars * 8;
  static constexpr int total = off_misc + 16;
  static constexpr int dynamic_bytes = total + 1024;  // slack for the manual 1024-byte alignment
};

template <int CH>
__device__ __forceinline__ void tmem_ld_chunk(uint32_t taddr, float (&v)[CH]) {
  if constexpr (CH == 32) {
    uint32_t r[32];
    ptx::tmem_ld_32x32(taddr, r);
    ptx::tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
  } else {
    static_assert(CH == 16, "chunk width");
    uint32_t r[16];
    ptx::tmem_ld_32x16(taddr, r);
    ptx::tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
  }
}

// Issue of a chunk load without its wait, and the walk over a warp's column chunks with the load of chunk
// i + 1 in flight while chunk i is computed: the TMEM read latency leaves the per-chunk dependent chain.
template <int CH>
__device__ __forceinline__ void tmem_ld_issue(uint32_t taddr, uint32_t (&r)[CH]) {
  if constexpr (CH == 32) ptx::tmem_ld_32x32(taddr, r);
  else ptx::tmem_ld_32x16(taddr, r);
}
template <class Epi, class State>
__device__ __forceinline__ void epilogue_walk_chunks(const typename Epi::Params& ep, const EpiEnv& env, const TileInfo& t, State& st,
                                                     uint32_t taddr0, int row, int col_begin, int col_end) {
  constexpr int CH = Epi::kChunk;
  uint32_t nxt[CH];
  if (col_begin < col_end) tmem_ld_issue<CH>(taddr0 + (uint32_t)col_begin, nxt);
#pragma unroll 1
  for (int col = col_begin; col < col_end; col += CH) {
    float v[CH];
    ptx::tmem_ld_wait_regs(nxt);
#pragma unroll
    for (int i = 0; i < CH; ++i) v[i] = __uint_as_float(nxt[i]);
    if (col + CH < col_end) tmem_ld_issue<CH>(taddr0 + (uint32_t)(col + CH), nxt);
    Epi::chunk(ep, env, t, st, row, col, v);
  }
  ptx::tmem_ld_wait();   // nothing of this warp is left in flight when the accumulator is handed back
}

template <int BN, int STAGES, bool A_MN, bool B_MN, int ML, int NE_WARPS, class Epi>
__global__ void __launch_bounds__(32 * (2 + NE_WARPS + (ml_transforms(ML) ? 4 : 0)), 1)
gemm_tcgen05_kernel(const __grid_constant__ GemmParams<typename Epi::Params> p) {
  using SM = GemmSmem<BN, STAGES, ML, Epi::kColReductions>;
  constexpr int kXformWarp0 = 2 + NE_WARPS;
  constexpr int kTmemCols = 2 * BN <= 32 ? 32 : 2 * BN <= 64 ? 64 : 2 * BN <= 128 ? 128 : 2 * BN <= 256 ? 256 : 512;
  constexpr int CH = Epi::kChunk;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = ptx::smem_u32(smem);
  const uint32_t bar0 = smem_base + SM::off_bar;
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto bar_xform = [&](int s) { return bar0 + 8u * (2 * STAGES + s); };
  auto bar_tmem_full = [&](int a) { return bar0 + 8u * (3 * STAGES + a); };
  auto bar_tmem_empty = [&](int a) { return bar0 + 8u * (3 * STAGES + 2 + a); };
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem + SM::off_misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::off_misc + 4);
  float* scratch = reinterpret_cast<float*>(smem + SM::off_scratch);

  const GemmCore& c = p.core;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(bar_full(s), 1);
      ptx::mbar_init(bar_empty(s), 1);
      ptx::mbar_init(bar_xform(s), 4);              // one arrival per transform warp
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(bar_tmem_full(a), 1);
      ptx::mbar_init(bar_tmem_empty(a), NE_WARPS);  // one arrival per epilogue warp
    }
    ptx::fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tmap(&p.tma_a);
    ptx::prefetch_tmap(&p.tma_b);
    if (SM::kHasMask) ptx::prefetch_tmap(&p.tma_mask);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  auto decode_tile = [&](int tile) {
    TileInfo t;
    t.tile_idx = tile;
    const int per_batch = c.tiles_m * c.tiles_n;
    t.b = tile / per_batch;
    const int r = tile - t.b * per_batch;
    // Grouped order: `group_m` row tiles x all column tiles at a time, rows fastest, so that the
    // CTAs running together share a small set of A row panels and B column panels in L2.
    const int gsz = c.group_m * c.tiles_n;
    const int g = r / gsz;
    const int first_m = g * c.group_m;
    const int gm = min(c.group_m, c.tiles_m - first_m);
    const int w = r - g * gsz;
    t.tile_n = w / gm;
    t.tile_m = first_m + (w - t.tile_n * gm);
    t.m0 = t.tile_m * kBM;
    t.n0 = t.tile_n * BN;
    t.bn = BN;
    return t;
  };

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      constexpr uint32_t kStageBytes = kATileBytes + SM::kBTileBytes + (SM::kHasMask ? kATileBytes : 0);
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int tile = blockIdx.x; alive && !c.withhold_loads && tile < c.num_tiles; tile += gridDim.x) {
        const TileInfo t = decode_tile(tile);
        for (int kb = 0; kb < c.k_blocks; ++kb) {
          if (!ptx::mbar_wait(bar_empty(stage), phase ^ 1u, abort_flag, c.status, 1, stage, c.wait_limit_us)) { alive = false; break; }
          ptx::mbar_arrive_expect_tx(bar_full(stage), kStageBytes);
          const int k0 = kb * ((ML & ML_F8) ? 2 * kBK : kBK);   // 128 bytes of K per block
          const uint32_t a_dst = smem_base + SM::off_a + stage * kATileBytes;
          const uint32_t b_dst = smem_base + SM::off_b + stage * SM::kBTileBytes;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < kBM / 64; ++j)
              ptx::tma_load_3d(a_dst + j * (kBK * 128), &p.tma_a, bar_full(stage), t.m0 + 64 * j, k0, t.b);
          } else {
            ptx::tma_load_3d(a_dst, &p.tma_a, bar_full(stage), k0, t.m0, t.b);
          }
          if (SM::kHasMask) {
            const uint32_t m_dst = smem_base + SM::off_mask + stage * kATileBytes;
            if (A_MN) {
#pragma unroll
              for (int j = 0; j < kBM / 64; ++j)
                ptx::tma_load_3d(m_dst + j * (kBK * 128), &p.tma_mask, bar_full(stage), t.m0 + 64 * j, k0, t.b);
            } else {
              ptx::tma_load_3d(m_dst, &p.tma_mask, bar_full(stage), k0, t.m0, t.b);
            }
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              ptx::tma_load_3d(b_dst + j * (kBK * 128), &p.tma_b, bar_full(stage), t.n0 + 64 * j, k0, t.b);
          } else {
            ptx::tma_load_3d(b_dst, &p.tma_b, bar_full(stage), k0, t.n0, t.b);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      const uint32_t idesc = (ML & ML_F8) ? ptx::make_idesc_f8(c.f8 & 2 ? 1 : 0, c.f8 & 4 ? 1 : 0, kBM, BN)
                                          : ptx::make_idesc_f16(c.ab_format, A_MN ? 1 : 0, B_MN ? 1 : 0, kBM, BN);
      // K-major: 8-row groups 1024 B apart (SBO), K advances 32 B inside the swizzle row.
      // MN-major: 64-element blocks kBK*128 B apart (LBO), 8-k groups 1024 B apart (SBO),
      //           K advances two k-groups = 2048 B per MMA.
      constexpr uint32_t a_lbo = A_MN ? kBK * 128 : 16, b_lbo = B_MN ? kBK * 128 : 16;
      constexpr uint32_t a_kadv = A_MN ? 2048 : 32, b_kadv = B_MN ? 2048 : 32;
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool alive = true;
      for (int tile = blockIdx.x; alive && tile < c.num_tiles; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
        if (!ptx::mbar_wait(bar_tmem_empty(acc), acc_phase ^ 1u, abort_flag, c.status, 2, acc, c.wait_limit_us)) { alive = false; break; }
        ptx::tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < c.k_blocks; ++kb) {
          const uint32_t ready = ml_transforms(ML) ? bar_xform(stage) : bar_full(stage);
          if (!ptx::mbar_wait(ready, phase, abort_flag, c.status, 3, stage, c.wait_limit_us)) { alive = false; break; }
          ptx::tcgen05_fence_after();
          const uint32_t a_addr = smem_base + SM::off_a + stage * kATileBytes;
          const uint32_t b_addr = smem_base + SM::off_b + stage * SM::kBTileBytes;
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            const uint64_t adesc = ptx::make_smem_desc_sw128(a_addr + k * a_kadv, a_lbo, 1024);
            const uint64_t bdesc = ptx::make_smem_desc_sw128(b_addr + k * b_kadv, b_lbo, 1024);
            if constexpr ((ML & ML_F8) != 0) ptx::umma_f8(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
            else ptx::umma_f16(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          ptx::umma_commit(bar_empty(stage));   // frees the smem stage when these MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (alive) ptx::umma_commit(bar_tmem_full(acc));
      }
    }
  } else if (warp < kXformWarp0) {
    // ===================== epilogue =====================
    EpiEnv env;
    env.core = &c;
    env.scratch = scratch;
    env.bn = BN;
    env.n_epi_threads = NE_WARPS * 32;
    env.epi_warp = warp - 2;
    env.epi_tid = env.epi_warp * 32 + lane;
    env.quadrant = warp & 3;  // a warp may only touch TMEM lanes 32*(warp%4) .. +31
    constexpr int kColsPerWarp = BN / (NE_WARPS / 4);
    const int col_begin = (env.epi_warp / 4) * kColsPerWarp;
    int it = 0;
    bool dead = false;
    for (int tile = blockIdx.x; tile < c.num_tiles; tile += gridDim.x, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
      const TileInfo t = decode_tile(tile);
      // After an abandoned wait the thread keeps walking the tile list without touching TMEM so
      // that the named barriers inside tile_end() still see every epilogue thread.
      Epi::tile_prepare(p.epi, env, t);   // per-tile staging that does not need the accumulator
      if (!dead && !ptx::mbar_wait(bar_tmem_full(acc), acc_phase, abort_flag, c.status, 4, acc, c.wait_limit_us)) dead = true;
      dead = __any_sync(0xffffffffu, dead);   // the warp decides together (it shares a __syncwarp below)
      typename Epi::State st;
      Epi::tile_begin(p.epi, st);
      if (!dead) {
        ptx::tcgen05_fence_after();
        const int row = env.quadrant * 32 + lane;
        const uint32_t taddr0 = tmem_base + ((uint32_t)(env.quadrant * 32) << 16) + (uint32_t)(acc * BN);
        // chunks that start at or beyond N are skipped (a ragged last chunk is handled inside the functor)
        const int col_end = min(col_begin + kColsPerWarp, ((c.N - t.n0 + CH - 1) / CH) * CH);
        epilogue_walk_chunks<Epi>(p.epi, env, t, st, taddr0, row, col_begin, col_end);
        ptx::tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(bar_tmem_empty(acc));   // 128+ arrivals on one word would serialise
      }
      Epi::tile_end(p.epi, env, t, st);
    }
  } else {
    // ===================== mainloop transform =====================
    if (ml_transforms(ML)) {
      const int tt = (warp - kXformWarp0) * 32 + lane;  // 0..127
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int tile = blockIdx.x; alive && tile < c.num_tiles; tile += gridDim.x) {
        for (int kb = 0; kb < c.k_blocks; ++kb) {
          const bool ok = ptx::mbar_wait(bar_full(stage), phase, abort_flag, c.status, 5, stage, c.wait_limit_us);
          if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
          uint4* a = reinterpret_cast<uint4*>(smem + SM::off_a + stage * kATileBytes);
          const uint4* mk = reinterpret_cast<const uint4*>(smem + SM::off_mask + stage * kATileBytes);
          // A and the mask were loaded with the same box and swizzle, so equal smem offsets hold
          // the same (row, k) element: the rewrite is position-wise.
          if constexpr ((ML & ML_GENERIC) != 0) {
#pragma unroll 1
            for (int i = 0; i < kATileBytes / 16 / 128; ++i) {
              const int idx = tt + i * 128;
              uint4 va = a[idx];
              uint4 vm;
              if (ML & ML_MASK) vm = mk[idx];
              ml_apply8(c.ml_a, c.ab_format, va, (ML & ML_MASK) ? &vm : nullptr);
              a[idx] = va;
            }
            if (c.ml_b.n > 0) {
              uint4* b = reinterpret_cast<uint4*>(smem + SM::off_b + stage * SM::kBTileBytes);
#pragma unroll 1
              for (int i = 0; i < SM::kBTileBytes / 16 / 128; ++i) {
                const int idx = tt + i * 128;
                uint4 vb = b[idx];
                ml_apply8(c.ml_b, c.ab_format, vb, nullptr);
                b[idx] = vb;
              }
            }
          } else
#pragma unroll
          for (int i = 0; i < kATileBytes / 16 / 128; ++i) {
            const int idx = tt + i * 128;
            uint4 va = a[idx];
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&va);
            if (ML & ML_RELU) {
              const __nv_bfloat162 z = __float2bfloat162_rn(0.0f);
#pragma unroll
              for (int j = 0; j < 4; ++j) h[j] = __hmax2(h[j], z);
            }
            if (ML & ML_MASK) {
              uint4 vm = mk[idx];
              const __nv_bfloat162* hm = reinterpret_cast<const __nv_bfloat162*>(&vm);
#pragma unroll
              for (int j = 0; j < 4; ++j) h[j] = __hmul2(h[j], hm[j]);
            }
            a[idx] = va;
          }
          ptx::fence_proxy_async_smem();   // every writer publishes its own stores to the async proxy
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(bar_xform(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  }

  // ---- teardown: every thread arrives here, also after an abandoned wait -----------------------
  ptx::tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tcgen05_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace he
