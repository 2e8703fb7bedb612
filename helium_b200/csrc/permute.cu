// permute_dims kernels (hot-path rows T1-T3) and the fused "affine (+relu) + permute" variant.
//
// The reference generates one 32x32 tile kernel per (shape, strides) with NVRTC, stages both the
// values and a u32 output index per element through 33-padded shared memory and moves one
// element per thread (helium/src/cuda/instr/permute_dims/jit.rs:15-117).  Here the kernels are
// precompiled and take the normalised problem as a parameter block:
//   * tile kernel  : input-innermost axis X differs from output-innermost axis Y.  A CTA moves a
//                    TX x TY tile with 16-byte global loads along X, 16-byte global stores along Y
//                    and a word-granular shared-memory transpose whose pitch (= 1 mod 8 words) makes
//                    the transposed reads bank-conflict free.  2-byte elements travel as packed
//                    pairs and are re-paired on the way out.
//   * row kernel   : X is also the output-innermost axis; 16-byte vectors are gathered row-wise.
//   * scalar kernels for shapes/pointers that do not meet the 16-byte rules.
#include "permute.cuh"
#include "device_utils.cuh"

#include <algorithm>
#include <cmath>

namespace he {

// ------------------------------------------------------------------------------------------------
// normalisation (host)
// ------------------------------------------------------------------------------------------------
int32_t normalize_permutation(int rank, const int64_t* in_shape, const int64_t* out_strides,
                              int elem_bytes, PermuteProblem* out, int keep_axis, int* axis_map) {
  if (rank < 1 || rank > HE_MAX_RANK) HE_FAIL(HE_ERR_INVALID, "permute: rank %d out of range", rank);
  int64_t total = 1;
  for (int i = 0; i < rank; ++i) {
    if (in_shape[i] < 0) HE_FAIL(HE_ERR_INVALID, "permute: negative dim");
    total *= in_shape[i];
  }
  out->elem_bytes = elem_bytes;
  out->total = total;
  out->r = 0;
  if (axis_map)
    for (int i = 0; i < rank; ++i) axis_map[i] = -1;
  if (total == 0) return HE_OK;
  // The strides must describe a dense layout of the same extents: sorted by stride, each stride
  // equals the product of the extents before it.
  std::vector<int> order;
  for (int i = 0; i < rank; ++i)
    if (in_shape[i] != 1) order.push_back(i);
  std::sort(order.begin(), order.end(), [&](int a, int b) { return out_strides[a] < out_strides[b]; });
  int64_t expect = 1;
  for (int a : order) {
    if (out_strides[a] != expect)
      HE_FAIL(HE_ERR_INVALID, "permute: out_strides do not form a dense permutation (axis %d has stride %lld, expected %lld)",
              a, (long long)out_strides[a], (long long)expect);
    expect *= in_shape[a];
  }
  // packed input strides
  int64_t in_stride[HE_MAX_RANK];
  int64_t s = 1;
  for (int i = rank - 1; i >= 0; --i) {
    in_stride[i] = s;
    s *= in_shape[i];
  }
  PermDim tmp[HE_MAX_RANK];
  int src_axis[HE_MAX_RANK];
  int n = 0;
  for (int i = 0; i < rank; ++i) {
    if (in_shape[i] == 1) continue;
    tmp[n] = {in_shape[i], in_stride[i], out_strides[i]};
    src_axis[n] = i;
    ++n;
  }
  // merge (i, i+1) when they are adjacent in the output too; `keep_axis` (the axis a fused
  // per-axis parameter varies along) is never merged with a neighbour.
  int m = 0;
  for (int i = 0; i < n; ++i) {
    const bool pinned = src_axis[i] == keep_axis || (i > 0 && src_axis[i - 1] == keep_axis);
    if (!pinned && m > 0 && out->d[m - 1].out_stride == tmp[i].out_stride * tmp[i].ext) {
      out->d[m - 1].ext *= tmp[i].ext;
      out->d[m - 1].in_stride = tmp[i].in_stride;
      out->d[m - 1].out_stride = tmp[i].out_stride;
    } else {
      out->d[m] = tmp[i];
      ++m;
    }
    if (axis_map) axis_map[src_axis[i]] = m - 1;
  }
  out->r = m;
  return HE_OK;
}

// ------------------------------------------------------------------------------------------------
// device code
// ------------------------------------------------------------------------------------------------
constexpr int kMaxBatchDims = HE_MAX_RANK;
constexpr int kThreads = 256;

enum FMode : int { F_NONE = 0, F_AXIS_Y = 1, F_AXIS_X = 2, F_BATCH = 3, F_CONST = 4 };

struct TileParams {
  const void* in;
  void* out;
  long long X, Y;        // extents of the two transposed axes (elements)
  long long in_sY;       // input stride of Y (elements); input stride of X is 1
  long long out_sX;      // output stride of X (elements); output stride of Y is 1
  int nb;
  long long b_ext[kMaxBatchDims], b_in[kMaxBatchDims], b_out[kMaxBatchDims];
  int TX, TY, P;         // tile extents in elements (powers of two), shared-memory pitch in 32-bit words
  int lg_chunks_x;       // log2 of 16-byte chunks per tile row
  int lg_y_blocks;       // log2(TY / 32)
  unsigned tiles_x, tiles_y;
  int xt;                // consecutive X tiles one CTA of the vector kernel walks (amortises its prologue)
  FastDiv fd_tiles_x, fd_tiles_y, fd_b[kMaxBatchDims];   // 32-bit magic division for the CTA prologue
                                                         // (fd_tiles_x divides by the number of X tile groups)
  // affine functor
  int f_mode, f_batch, relu, has_scale, has_bias, s_dt, b_dt;
  const void* scale;
  const void* bias;
};

struct RowParams {
  const void* in;
  void* out;
  int nd;                 // dims in OUTPUT order, innermost last (unit stride on both sides)
  long long ext[HE_MAX_RANK], in_stride[HE_MAX_RANK];
  FastDiv fd[HE_MAX_RANK];
  long long total_units;  // number of 16-byte vectors (or elements in the scalar kernel)
  int unit_elems;         // elements per unit
};

struct BatchOffsets {
  long long in_base, out_base, f_coord;
};

// Block index -> (tile x, tile y, batch offsets) with 32-bit magic-number divisions: the prologue
// runs in every thread of every CTA and a CTA only moves a few thousand elements, so 64-bit
// divisions here used to cost more instructions than the data movement itself.
__device__ __forceinline__ BatchOffsets decode_block(const TileParams& p, unsigned& tx, unsigned& ty) {
  unsigned blk = blockIdx.x, q;
  p.fd_tiles_x.divmod(blk, q, tx);
  blk = q;
  p.fd_tiles_y.divmod(blk, q, ty);
  blk = q;
  BatchOffsets o{0, 0, 0};
#pragma unroll 1
  for (int k = p.nb - 1; k >= 0; --k) {
    unsigned c;
    p.fd_b[k].divmod(blk, q, c);
    blk = q;
    o.in_base += (long long)c * p.b_in[k];
    o.out_base += (long long)c * p.b_out[k];
    if (p.f_mode == F_BATCH && k == p.f_batch) o.f_coord = (long long)c;
  }
  return o;
}

__device__ __forceinline__ BatchOffsets decode_batch(const TileParams& p, unsigned long long b) {
  BatchOffsets o{0, 0, 0};
#pragma unroll 1
  for (int k = p.nb - 1; k >= 0; --k) {
    unsigned long long e = (unsigned long long)p.b_ext[k];
    unsigned long long c = b % e;
    b /= e;
    o.in_base += (long long)c * p.b_in[k];
    o.out_base += (long long)c * p.b_out[k];
    if (p.f_mode == F_BATCH && k == p.f_batch) o.f_coord = (long long)c;
  }
  return o;
}

// y = x * s + b as one fused multiply-add (the reference's NVRTC build contracts `x * s + b`,
// helium/src/cuda/kernel_jit.rs:155-168 leaves fmad at its default), then optional relu
// (`fmaxf(v, 0.0)`, pointwise/jit.rs:542).
__device__ __forceinline__ float affine(float x, float s, float b, int relu) {
  float v = fmaf(x, s, b);
  return relu ? fmaxf(v, 0.0f) : v;
}
// Same with the relu folded into a floor value (0 or -inf): one FMNMX, no select.  fmaxf returns
// the non-NaN operand, so a NaN input becomes the floor exactly as fmaxf(v, 0.0) would make it 0.
__device__ __forceinline__ float affine_floor(float x, float s, float b, float floor_v) {
  return fmaxf(fmaf(x, s, b), floor_v);
}

// XDT: -1 = plain permutation, otherwise the he_dtype of the element for the affine functor.
// The host picks power-of-two tile extents, so every index decode below is a shift or a mask, and
// offsets inside a tile are 32-bit (the planner routes tensors of 2^32 elements or more elsewhere).
constexpr int ilog2_c(int v) { return v <= 1 ? 0 : 1 + ilog2_c(v / 2); }

// TXW_C / TY_C > 0 fix the tile shape at compile time (the common shapes), which unrolls both
// loops and folds every shift, mask and pitch; 0 keeps them as kernel parameters.
template <int EB, int XDT, int TXW_C = 0, int TY_C = 0>
__global__ void __launch_bounds__(kThreads, (EB == 2 && TXW_C > 0) ? 8 : 1) permute_tile_vec(const __grid_constant__ TileParams p) {
  extern __shared__ uint32_t sm[];
  constexpr int EPW = 4 / EB;            // elements per 32-bit word
  constexpr int VE = 16 / EB;            // elements per 16-byte vector
  constexpr bool kFixed = TXW_C > 0;
  unsigned tx, ty;
  const BatchOffsets bo = decode_block(p, tx, ty);
  const int TX = kFixed ? TXW_C * EPW : p.TX, TY = kFixed ? TY_C : p.TY;
  const int P = kFixed ? (TXW_C > 8 ? TXW_C : 8) + 1 : p.P;
  const long long y0 = (long long)ty * TY;
  const unsigned ny = (unsigned)min((long long)TY, p.Y - y0);   // rows of this tile that exist
  const unsigned in_sY = (unsigned)p.in_sY, out_sX = (unsigned)p.out_sX;
  const unsigned tx_first = tx * (unsigned)p.xt;
  long long x0 = (long long)tx_first * TX;

  // ---- fused-affine parameters: one (scale, bias) pair per row / column / CTA, staged in smem ----
  float* par = reinterpret_cast<float*>(sm + TY * P);
  if constexpr (XDT >= 0) {
    const int n_par = p.f_mode == F_AXIS_Y ? TY : p.f_mode == F_AXIS_X ? TX : 1;
    const long long c0 = p.f_mode == F_AXIS_Y ? y0 : p.f_mode == F_AXIS_X ? x0 : p.f_mode == F_BATCH ? bo.f_coord : 0;
    const long long c_end = p.f_mode == F_AXIS_Y ? p.Y : p.f_mode == F_AXIS_X ? p.X : c0 + 1;
    for (int i = threadIdx.x; i < n_par; i += kThreads) {
      const bool ok = c0 + i < c_end;
      par[2 * i] = (ok && p.has_scale) ? load_param_as_f32(p.scale, p.s_dt, c0 + i) : 1.0f;
      par[2 * i + 1] = (ok && p.has_bias) ? load_param_as_f32(p.bias, p.b_dt, c0 + i) : 0.0f;
    }
    __syncthreads();
  }

  // A CTA walks p.xt consecutive X tiles of the same (Y tile, batch): block decode and parameter
  // staging above are paid once (with parameters along X the host keeps p.xt at 1).
  // With a compile-time tile shape the input vectors of the NEXT X tile are fetched into registers
  // before the current tile's transposed stores start, so a CTA always has loads in flight.
  // (2-byte instantiations only: they carry 2-4 vectors per thread; the 4-byte ones would pay 16
  // more registers, which costs the streaming permutations more occupancy than the overlap returns)
  constexpr bool kPrefetch = kFixed && EB == 2;
  constexpr int NV = kPrefetch ? (TY_C * (TXW_C / 4)) / kThreads : 1;   // 16-byte vectors per thread per tile
  constexpr int kLgCx = kFixed ? ilog2_c(TXW_C / 4) : 0;
  uint4 pre[NV];
  auto fetch_tile = [&](long long xa) {
    const unsigned nxa = (unsigned)min((long long)TX, p.X - xa);
    const char* src = reinterpret_cast<const char*>(p.in) + (bo.in_base + y0 * p.in_sY + xa) * EB;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int q = threadIdx.x + i * kThreads;
      const unsigned cx = q & ((1u << kLgCx) - 1u), y = (unsigned)q >> kLgCx;
      if (cx * VE < nxa && y < ny) pre[i] = __ldcs(reinterpret_cast<const uint4*>(src + (size_t)(y * in_sY + cx * VE) * EB));
    }
  };
  if constexpr (kPrefetch) fetch_tile(x0);
#pragma unroll 1
  for (int xs = 0; xs < p.xt; ++xs, x0 += TX) {
  if (tx_first + xs >= p.tiles_x) break;
  if (xs > 0) __syncthreads();   // the previous tile's transposed reads are done
  const unsigned nx = (unsigned)min((long long)TX, p.X - x0);   // columns of this tile that exist
  const char* in_tile = reinterpret_cast<const char*>(p.in) + (bo.in_base + y0 * p.in_sY + x0) * EB;
  char* out_tile = reinterpret_cast<char*>(p.out) + (bo.out_base + x0 * p.out_sX + y0) * EB;
  // ---- phase 1: global (vector along X) -> shared [y][xw] -------------------------------------
  {
    const int lg_cx = kFixed ? ilog2_c(TXW_C / 4) : p.lg_chunks_x;   // chunks (16 B) per tile row = 1 << lg_cx
    const int total = TY << lg_cx;
    const float floor_v = p.relu ? 0.0f : -INFINITY;
#pragma unroll
    for (int q = threadIdx.x, qi = 0; q < total; q += kThreads, ++qi) {
      const unsigned cx = q & ((1u << lg_cx) - 1u), y = (unsigned)q >> lg_cx;
      const unsigned x = cx * VE;
      if (x < nx && y < ny) {
        uint4 v;
        if constexpr (kPrefetch) v = pre[qi < NV ? qi : 0];
        else v = __ldcs(reinterpret_cast<const uint4*>(in_tile + (size_t)(y * in_sY + x) * EB));
        if constexpr (XDT >= 0) {
          uint32_t w[4] = {v.x, v.y, v.z, v.w};
          if (p.f_mode == F_AXIS_X) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if constexpr (EB == 4) {
                const float2 sb = *reinterpret_cast<const float2*>(par + 2 * (x + j));
                w[j] = __float_as_uint(affine_floor(__uint_as_float(w[j]), sb.x, sb.y, floor_v));
              } else {
                const float4 sb = *reinterpret_cast<const float4*>(par + 2 * (x + 2 * j));
                if constexpr (XDT == HE_BF16) {
                  const float2 f = bf16x2_to_f32(w[j]);
                  w[j] = f32x2_to_bf16x2(affine_floor(f.x, sb.x, sb.y, floor_v), affine_floor(f.y, sb.z, sb.w, floor_v));
                } else {
                  w[j] = f32_to_f16_bits(affine_floor(f16_bits_to_f32(w[j] & 0xffffu), sb.x, sb.y, floor_v)) |
                         (f32_to_f16_bits(affine_floor(f16_bits_to_f32(w[j] >> 16), sb.z, sb.w, floor_v)) << 16);
                }
              }
            }
          } else {
            const float2 sb = *reinterpret_cast<const float2*>(par + 2 * (p.f_mode == F_AXIS_Y ? y : 0u));
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if constexpr (EB == 4) {
                w[j] = __float_as_uint(affine_floor(__uint_as_float(w[j]), sb.x, sb.y, floor_v));
              } else if constexpr (XDT == HE_BF16) {
                const float2 f = bf16x2_to_f32(w[j]);
                w[j] = f32x2_to_bf16x2(affine_floor(f.x, sb.x, sb.y, floor_v), affine_floor(f.y, sb.x, sb.y, floor_v));
              } else {
                w[j] = f32_to_f16_bits(affine_floor(f16_bits_to_f32(w[j] & 0xffffu), sb.x, sb.y, floor_v)) |
                       (f32_to_f16_bits(affine_floor(f16_bits_to_f32(w[j] >> 16), sb.x, sb.y, floor_v)) << 16);
              }
            }
          }
          v = make_uint4(w[0], w[1], w[2], w[3]);
        }
        uint32_t* dst = sm + y * P + cx * 4;
        dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
      }
    }
  }
  if constexpr (kPrefetch) {
    if (xs + 1 < p.xt && tx_first + xs + 1 < p.tiles_x) fetch_tile(x0 + TX);
  }
  __syncthreads();
  // ---- phase 2: shared (transposed read) -> global (vector along Y) ---------------------------
  const int lg_yb = kFixed ? ilog2_c(TY_C / 32) : p.lg_y_blocks;   // TY / 32 = 1 << lg_yb
  if constexpr (EB == 4) {
    // warp = 8 lanes along y-chunks (4 y each) x 4 lanes along x: banks (4*ly + x) distinct.
    const int total = TX * (TY / 4);
#pragma unroll
    for (int q = threadIdx.x; q < total; q += kThreads) {
      const unsigned yq_lo = q & 7, x_lo = (q >> 3) & 3, rest = (unsigned)q >> 5;
      const unsigned yq = ((rest & ((1u << lg_yb) - 1u)) << 3) + yq_lo, x = ((rest >> lg_yb) << 2) + x_lo;
      const unsigned y = yq * 4;
      if (x < nx && y < ny) {
        const uint32_t* src = sm + y * P + x;
        const uint4 v = make_uint4(src[0], src[P], src[2 * P], src[3 * P]);
        __stcs(reinterpret_cast<uint4*>(out_tile + (size_t)(x * out_sX + y) * 4), v);
      }
    }
  } else {
    // a thread owns one word column (2 x) and 8 consecutive y: two 16-byte output vectors.
    // warp = 4 lanes along y-chunks x 8 lanes along xw: banks (8*ly + xw) distinct.
    const int TXW = TX / EPW;
    const int total = TXW * (TY / 8);
#pragma unroll
    for (int q = threadIdx.x; q < total; q += kThreads) {
      const unsigned yq_lo = q & 3, xw_lo = (q >> 2) & 7, rest = (unsigned)q >> 5;
      const unsigned yq = ((rest & ((1u << lg_yb) - 1u)) << 2) + yq_lo, xw = ((rest >> lg_yb) << 3) + xw_lo;
      const unsigned x = 2 * xw, y = yq * 8;
      if (x < nx && y < ny) {
        const uint32_t* src = sm + y * P + xw;
        uint32_t w[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) w[k] = src[k * P];
        uint4 lo, hi;
        lo.x = __byte_perm(w[0], w[1], 0x5410); hi.x = __byte_perm(w[0], w[1], 0x7632);
        lo.y = __byte_perm(w[2], w[3], 0x5410); hi.y = __byte_perm(w[2], w[3], 0x7632);
        lo.z = __byte_perm(w[4], w[5], 0x5410); hi.z = __byte_perm(w[4], w[5], 0x7632);
        lo.w = __byte_perm(w[6], w[7], 0x5410); hi.w = __byte_perm(w[6], w[7], 0x7632);
        char* o = out_tile + (size_t)(x * out_sX + y) * 2;
        __stcs(reinterpret_cast<uint4*>(o), lo);
        // X is a multiple of 8 on this path, so x + 1 is in range whenever x is.
        __stcs(reinterpret_cast<uint4*>(o + (size_t)out_sX * 2), hi);
      }
    }
  }
  }  // X tiles of this CTA
}

// Scalar fallback: classic 32x32 tile, one element per thread per pass.
template <typename T, int XDT>
__global__ void __launch_bounds__(kThreads) permute_tile_scalar(const __grid_constant__ TileParams p) {
  __shared__ T tile[32][33];
  unsigned long long blk = blockIdx.x;
  const unsigned tx = (unsigned)(blk % p.tiles_x);
  blk /= p.tiles_x;
  const unsigned ty = (unsigned)(blk % p.tiles_y);
  blk /= p.tiles_y;
  const BatchOffsets bo = decode_batch(p, blk);
  const long long x0 = (long long)tx * 32, y0 = (long long)ty * 32;
  const int lx = threadIdx.x & 31, ly = threadIdx.x >> 5;
  const T* in = reinterpret_cast<const T*>(p.in);
  T* out = reinterpret_cast<T*>(p.out);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int y = ly + 8 * k;
    const long long gx = x0 + lx, gy = y0 + y;
    if (gx < p.X && gy < p.Y) {
      T v = in[bo.in_base + gy * p.in_sY + gx];
      if constexpr (XDT >= 0) {
        const long long c = p.f_mode == F_AXIS_Y ? gy : p.f_mode == F_AXIS_X ? gx : p.f_mode == F_BATCH ? bo.f_coord : 0;
        const float s = p.has_scale ? load_param_as_f32(p.scale, p.s_dt, c) : 1.0f;
        const float b = p.has_bias ? load_param_as_f32(p.bias, p.b_dt, c) : 0.0f;
        if constexpr (XDT == HE_F32) v = (T)__float_as_uint(affine(__uint_as_float((uint32_t)v), s, b, p.relu));
        else if constexpr (XDT == HE_BF16) v = (T)f32_to_bf16_bits(affine(bf16_bits_to_f32((uint32_t)v), s, b, p.relu));
        else v = (T)f32_to_f16_bits(affine(f16_bits_to_f32((uint32_t)v), s, b, p.relu));
      }
      tile[y][lx] = v;
    }
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int x = ly + 8 * k;
    const long long gx = x0 + x, gy = y0 + lx;
    if (gx < p.X && gy < p.Y) out[bo.out_base + gx * p.out_sX + gy] = tile[lx][x];
  }
}

// Row kernel: unit = 16 bytes (UNIT16) or one element; innermost dim shared by both layouts.
template <typename U>
__global__ void __launch_bounds__(kThreads) permute_rows(const __grid_constant__ RowParams p) {
  const long long stride = (long long)gridDim.x * kThreads;
  const U* in = reinterpret_cast<const U*>(p.in);
  U* out = reinterpret_cast<U*>(p.out);
  for (long long u = (long long)blockIdx.x * kThreads + threadIdx.x; u < p.total_units; u += stride) {
    long long rem = u, off = 0;
    if (p.total_units < (1ll << 31)) {
      uint32_t r32 = (uint32_t)u;
#pragma unroll 1
      for (int k = p.nd - 1; k >= 0; --k) {
        uint32_t q, c;
        p.fd[k].divmod(r32, q, c);
        r32 = q;
        off += (long long)c * p.in_stride[k];
      }
    } else {
#pragma unroll 1
      for (int k = p.nd - 1; k >= 0; --k) {
        long long c = rem % p.ext[k];
        rem /= p.ext[k];
        off += c * p.in_stride[k];
      }
    }
    out[u] = in[off];
  }
}

// ------------------------------------------------------------------------------------------------
// plan
// ------------------------------------------------------------------------------------------------
namespace {

enum class Mode { Empty, Copy, Rows, Tile };

struct PermutePlan : he_plan {
  Mode mode = Mode::Empty;
  int eb = 4;
  bool vec = false;
  AffineFunctor f;
  TileParams tp{};
  RowParams rp{};
  size_t bytes = 0;
  long long grid = 0;
  size_t smem = 0;
  int n_inputs = 1;

  int32_t launch(const void* const* inputs, void* const* outputs, void* /*workspace*/,
                 cudaStream_t stream) override {
    if (mode == Mode::Empty) return HE_OK;
    if (!inputs || !outputs || !inputs[f.enabled ? f.x_input : 0] || !outputs[0])
      HE_FAIL(HE_ERR_INVALID, "permute launch: null tensor pointer");
    const void* in = inputs[f.enabled ? f.x_input : 0];
    void* out = outputs[0];
    const bool aligned = ((uintptr_t)in % 16 == 0) && ((uintptr_t)out % 16 == 0);
    if (mode == Mode::Copy) {
      HE_CUDA(cudaMemcpyAsync(out, in, bytes, cudaMemcpyDeviceToDevice, stream));
      return HE_OK;
    }
    if (mode == Mode::Rows) {
      RowParams p = rp;
      p.in = in;
      p.out = out;
      bool use_vec = vec && aligned;
      if (!use_vec && vec) {
        // fall back to element units: innermost extent grows by the vector width
        p.unit_elems = 1;
        p.ext[p.nd - 1] *= 16 / eb;
        p.fd[p.nd - 1] = FastDiv((uint32_t)std::min<long long>(p.ext[p.nd - 1], 0x7fffffff));
        p.total_units *= 16 / eb;
        for (int k = 0; k < p.nd - 1; ++k) p.in_stride[k] *= 16 / eb;
      }
      long long blocks = (p.total_units + kThreads - 1) / kThreads;
      long long cap = (long long)ctx_sm_count(ctx) * 32;
      unsigned g = (unsigned)std::max<long long>(1, std::min(blocks, cap));
      if (use_vec) permute_rows<uint4><<<g, kThreads, 0, stream>>>(p);
      else if (eb == 4) permute_rows<uint32_t><<<g, kThreads, 0, stream>>>(p);
      else permute_rows<uint16_t><<<g, kThreads, 0, stream>>>(p);
      HE_CUDA(cudaGetLastError());
      last_launches = 1;
      return HE_OK;
    }
    TileParams p = tp;
    p.in = in;
    p.out = out;
    bool use_vec = vec && aligned;
    if (f.enabled) {
      p.scale = f.has_scale ? inputs[f.scale_input] : nullptr;
      p.bias = f.has_bias ? inputs[f.bias_input] : nullptr;
      if ((f.has_scale && !p.scale) || (f.has_bias && !p.bias)) HE_FAIL(HE_ERR_INVALID, "permute launch: null parameter pointer");
    }
    if (use_vec) {
      const int xdt = f.enabled ? f.x_dtype : -1;
      unsigned g = (unsigned)grid;
#define HE_LAUNCH_TILE(EB_, XDT_)                                                              \
  do {                                                                                         \
    const int txw_ = p.TX / (4 / EB_);                                                         \
    if (EB_ == 2 && txw_ == 32 && p.TY == 64) permute_tile_vec<EB_, XDT_, 32, 64><<<g, kThreads, smem, stream>>>(p);        \
    else if (EB_ == 2 && txw_ == 32 && p.TY == 128) permute_tile_vec<EB_, XDT_, 32, 128><<<g, kThreads, smem, stream>>>(p); \
    else if (EB_ == 4 && txw_ == 32 && p.TY == 128) permute_tile_vec<EB_, XDT_, 32, 128><<<g, kThreads, smem, stream>>>(p); \
    else if (EB_ == 4 && txw_ == 8 && p.TY == 512) permute_tile_vec<EB_, XDT_, 8, 512><<<g, kThreads, smem, stream>>>(p);   \
    else permute_tile_vec<EB_, XDT_><<<g, kThreads, smem, stream>>>(p);                         \
  } while (0)
      if (eb == 4) {
        if (xdt == HE_F32) HE_LAUNCH_TILE(4, HE_F32); else HE_LAUNCH_TILE(4, -1);
      } else {
        if (xdt == HE_BF16) HE_LAUNCH_TILE(2, HE_BF16);
        else if (xdt == HE_F16) HE_LAUNCH_TILE(2, HE_F16);
        else HE_LAUNCH_TILE(2, -1);
      }
#undef HE_LAUNCH_TILE
    } else {
      p.tiles_x = (unsigned)((p.X + 31) / 32);
      p.tiles_y = (unsigned)((p.Y + 31) / 32);
      long long batch = 1;
      for (int k = 0; k < p.nb; ++k) batch *= p.b_ext[k];
      long long g64 = (long long)p.tiles_x * p.tiles_y * batch;
      if (g64 > 0x7fffffffll) HE_FAIL(HE_ERR_UNSUPPORTED, "permute: too many tiles for the scalar path");
      unsigned g = (unsigned)g64;
      const int xdt = f.enabled ? f.x_dtype : -1;
      if (eb == 4) {
        if (xdt == HE_F32) permute_tile_scalar<uint32_t, HE_F32><<<g, kThreads, 0, stream>>>(p);
        else permute_tile_scalar<uint32_t, -1><<<g, kThreads, 0, stream>>>(p);
      } else {
        if (xdt == HE_BF16) permute_tile_scalar<uint16_t, HE_BF16><<<g, kThreads, 0, stream>>>(p);
        else if (xdt == HE_F16) permute_tile_scalar<uint16_t, HE_F16><<<g, kThreads, 0, stream>>>(p);
        else permute_tile_scalar<uint16_t, -1><<<g, kThreads, 0, stream>>>(p);
      }
    }
    HE_CUDA(cudaGetLastError());
    last_launches = 1;
    return HE_OK;
  }
};

int next_pow2(long long v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

}  // namespace

int32_t make_permute_plan(he_ctx* ctx, int rank, const int64_t* in_shape, const int64_t* out_strides,
                          int32_t dtype, const AffineFunctor* f, he_plan** out) {
  const int eb = dtype_bytes(dtype);
  if (eb == 0) HE_FAIL(HE_ERR_UNSUPPORTED, "permute: dtype %s is not supported (bit-packed)", dtype_name(dtype));
  PermuteProblem pr;
  int axis_map[HE_MAX_RANK];
  const bool fn = f && f->enabled;
  HE_TRY(normalize_permutation(rank, in_shape, out_strides, eb, &pr, fn ? f->axis : -1, axis_map));
  PermutePlan* plan = new PermutePlan();
  plan->ctx = ctx;
  plan->eb = eb;
  if (fn) plan->f = *f;
  plan->bytes = (size_t)pr.total * eb;
  char desc[256];
  if (pr.total == 0) {
    plan->mode = Mode::Empty;
    plan->description = "permute: empty";
    *out = plan;
    return HE_OK;
  }
  if (pr.total >= (1ll << 40)) {
    delete plan;
    HE_FAIL(HE_ERR_UNSUPPORTED, "permute: tensor too large");
  }
  // output-innermost dim
  int ydim = -1;
  for (int k = 0; k < pr.r; ++k)
    if (pr.d[k].out_stride == 1) ydim = k;
  const int xdim = pr.r - 1;
  if (!fn && (pr.r <= 1)) {
    plan->mode = Mode::Copy;
    plan->description = "permute: identity layout -> device memcpy";
    *out = plan;
    return HE_OK;
  }
  if (pr.r == 0 || ydim == xdim || pr.r == 1) {
    if (fn) {
      // pointwise planner handles inner-axis-preserving cases through its own kernels
      delete plan;
      HE_FAIL(HE_ERR_UNSUPPORTED, "permute+affine: innermost axis preserved; not a tile case");
    }
    // rows: dims in output order
    plan->mode = Mode::Rows;
    RowParams& rp = plan->rp;
    std::vector<int> order;
    for (int k = 0; k < pr.r; ++k) order.push_back(k);
    std::sort(order.begin(), order.end(), [&](int a, int b) { return pr.d[a].out_stride > pr.d[b].out_stride; });
    const int ve = 16 / eb;
    const bool vec = pr.d[xdim].ext % ve == 0;  // packed strides of outer dims are then multiples too
    plan->vec = vec;
    rp.nd = pr.r;
    for (int i = 0; i < pr.r; ++i) {
      const PermDim& d = pr.d[order[i]];
      long long ext = d.ext, st = d.in_stride;
      if (vec) {
        if (order[i] == xdim) ext /= ve; else st /= ve;
      }
      rp.ext[i] = ext;
      rp.in_stride[i] = st;
      rp.fd[i] = FastDiv((uint32_t)std::min<long long>(ext, 0x7fffffff));
    }
    rp.unit_elems = vec ? ve : 1;
    rp.total_units = pr.total / rp.unit_elems;
    snprintf(desc, sizeof desc, "permute: row gather, %d dims, %s units", pr.r, vec ? "16-byte" : "element");
    plan->description = desc;
    *out = plan;
    return HE_OK;
  }
  // ---- tile mode ----
  plan->mode = Mode::Tile;
  TileParams& tp = plan->tp;
  tp.X = pr.d[xdim].ext;
  tp.Y = pr.d[ydim].ext;
  tp.in_sY = pr.d[ydim].in_stride;
  tp.out_sX = pr.d[xdim].out_stride;
  tp.nb = 0;
  long long batch = 1;
  int norm_to_batch[HE_MAX_RANK];
  for (int k = 0; k < pr.r; ++k) {
    norm_to_batch[k] = -1;
    if (k == xdim || k == ydim) continue;
    norm_to_batch[k] = tp.nb;
    tp.b_ext[tp.nb] = pr.d[k].ext;
    tp.b_in[tp.nb] = pr.d[k].in_stride;
    tp.b_out[tp.nb] = pr.d[k].out_stride;
    batch *= pr.d[k].ext;
    ++tp.nb;
  }
  tp.f_mode = F_NONE;
  if (fn) {
    const int nd = axis_map[f->axis];
    tp.f_mode = nd < 0 ? F_CONST : nd == xdim ? F_AXIS_X : nd == ydim ? F_AXIS_Y : F_BATCH;
    tp.f_batch = nd >= 0 ? norm_to_batch[nd] : 0;
    tp.relu = f->relu;
    tp.has_scale = f->has_scale;
    tp.has_bias = f->has_bias;
    tp.s_dt = f->scale_dtype;
    tp.b_dt = f->bias_dtype;
  }
  const int ve = 16 / eb;
  bool vec = tp.X % ve == 0 && tp.Y % ve == 0 && tp.in_sY % ve == 0 && tp.out_sX % ve == 0;
  for (int k = 0; k < tp.nb; ++k) vec = vec && tp.b_in[k] % ve == 0 && tp.b_out[k] % ve == 0;
  plan->vec = vec;
  // tile shape: TX up to 32 words wide, ~16 KB of payload per CTA
  const int epw = 4 / eb;
  int txw = std::min(32, next_pow2((tp.X + epw - 1) / epw));
  txw = std::max(txw, eb == 4 ? 4 : 8);
  int ty = (4096 / txw);
  ty = std::min(ty, 512);
  while (ty > 32 && ty / 2 >= tp.Y) ty /= 2;   // stays a power of two
  ty = std::max(ty, 32);
  {
    // A CTA loads, synchronises, then stores, so the last partial wave of CTAs costs a full tile
    // time.  Among {ty, ty/2, ty/4} take the tile height with the best
    // (full waves / launched waves) x (output run length factor).
    const int sms = ctx_sm_count(ctx);
    double best = -1.0;
    int best_ty = ty;
    for (int cand = ty; cand >= 32 && cand >= ty / 4; cand /= 2) {
      const long long tiles = ((tp.X + txw * epw - 1) / (txw * epw)) * ((tp.Y + cand - 1) / cand) * batch;
      const size_t smem_c = (size_t)cand * (std::max(txw, 8) + 1) * 4 + 1024;
      const int per_sm = (int)std::max<size_t>(1, std::min<size_t>(2048 / kThreads, (size_t)(220 * 1024) / smem_c));
      const double waves = (double)tiles / ((double)sms * per_sm);
      const double quant = waves / std::ceil(waves);
      const long long run_bytes = (long long)std::min<long long>(cand, tp.Y) * eb;
      const double run = run_bytes >= 256 ? 1.0 : run_bytes >= 128 ? 0.96 : 0.85;
      const double score = quant * run;
      // smaller tiles carry fewer bytes in flight per thread: switch only for a clear gain
      if (score > best * 1.03) { best = score; best_ty = cand; }
    }
    ty = best_ty;
  }
  tp.TX = txw * epw;
  tp.TY = ty;
  tp.P = std::max(txw, 8) + 1;
  tp.lg_chunks_x = 0;
  while ((1 << tp.lg_chunks_x) < txw / 4) ++tp.lg_chunks_x;
  tp.lg_y_blocks = 0;
  while ((32 << tp.lg_y_blocks) < ty) ++tp.lg_y_blocks;
  // in-tile offsets are 32-bit in the vector kernel
  if (pr.total >= (1ll << 32)) vec = false;
  plan->vec = vec;
  tp.tiles_x = (unsigned)((tp.X + tp.TX - 1) / tp.TX);
  tp.tiles_y = (unsigned)((tp.Y + tp.TY - 1) / tp.TY);
  long long g64 = (long long)tp.tiles_x * tp.tiles_y * batch;
  if (g64 > 0x7fffffffll) {
    delete plan;
    HE_FAIL(HE_ERR_UNSUPPORTED, "permute: too many tiles");
  }
  // X tiles per CTA: as many (1, 2 or 4) as still leave at least two full waves of CTAs; beyond
  // the first tile a CTA's loads overlap its stores
  tp.xt = 1;
  if (vec && tp.f_mode != F_AXIS_X) {
    const size_t smem_c = (size_t)tp.TY * tp.P * 4 + 1024;
    const long long per_wave = (long long)ctx_sm_count(ctx) *
                               (long long)std::max<size_t>(1, std::min<size_t>(2048 / kThreads, (size_t)(220 * 1024) / smem_c));
    while (tp.xt < 4 && (long long)tp.tiles_x >= 2 * tp.xt && g64 / (2 * tp.xt) >= 2 * per_wave) tp.xt *= 2;
  }
  const unsigned tiles_xg = (tp.tiles_x + tp.xt - 1) / tp.xt;
  g64 = (long long)tiles_xg * tp.tiles_y * batch;
  tp.fd_tiles_x = FastDiv(tiles_xg);
  tp.fd_tiles_y = FastDiv(tp.tiles_y);
  for (int k = 0; k < tp.nb; ++k) tp.fd_b[k] = FastDiv((uint32_t)tp.b_ext[k]);
  plan->grid = g64;
  plan->smem = (size_t)tp.TY * tp.P * 4 + (fn ? (size_t)std::max(tp.TX, tp.TY) * 8 : 0);
  snprintf(desc, sizeof desc, "permute: tile %dx%d (%d-byte elems, pitch %d words, %s%s), %d X tile(s) per CTA, grid %lld",
           tp.TX, tp.TY, eb, tp.P, vec ? "16-byte vectors" : "scalar fallback", fn ? ", fused affine" : "", tp.xt, g64);
  plan->description = desc;
  *out = plan;
  return HE_OK;
}

int32_t plan_permute(he_ctx* ctx, int rank, const int64_t* in_shape, const int64_t* out_strides,
                     int32_t dtype, he_plan** out) {
  if (!dtype_valid(dtype)) HE_FAIL(HE_ERR_INVALID, "permute: bad dtype %d", dtype);
  return make_permute_plan(ctx, rank, in_shape, out_strides, dtype, nullptr, out);
}

}  // namespace he
