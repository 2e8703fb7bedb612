// Tier-2 pointwise kernels for dense, same-shape, same-dtype elementwise programs.
//
// The interpreter tier spends ~100 machine instructions per program instruction per 8 elements,
// which caps it at 1.8 (bf16) to 3.8 (f32) TB/s.  The short programs that dominate helium graphs
// once matmul epilogues are fused away -- relu, add, mul, relu(a) * m, relu(a + b), a * b + c, the
// SGD update w - lr * g (helium/src/optimizer/sgd.rs:48), gelu -- are compiled here as straight-line
// functors instead: 16-byte loads, two vectors per tensor in flight per thread, f32 arithmetic, one
// rounding at the store, exactly the operation order the interpreter uses (separately rounded mul
// and add unless the program's mul feeds only an add, which both tiers contract to one fma like
// the reference's NVRTC build does).
//
// A program qualifies when every load is a full-tensor identity load (canonical form `I<n>:F`), all
// tensors share one dtype of {bf16, f16, f32}, and its canonical text is in the table below.
#include "pointwise_dense.cuh"

#include <cstring>

namespace he {
namespace {

constexpr int kEwThreads = 256;
constexpr int kEwUnroll = 2;   // 16-byte vectors per tensor per thread per iteration

struct EwParams {
  const void* in[3];
  void* out;
  unsigned long long n_vec;   // 16-byte vectors per tensor
  float k;                    // the program's constant, when it has one
};

template <typename T> struct EwVec;
template <> struct EwVec<float> {
  static constexpr int kElems = 4;
  __device__ static void unpack(const uint4& q, float* o) {
    o[0] = __uint_as_float(q.x); o[1] = __uint_as_float(q.y); o[2] = __uint_as_float(q.z); o[3] = __uint_as_float(q.w);
  }
  __device__ static uint4 pack(const float* v) {
    return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
  }
};
template <> struct EwVec<__nv_bfloat16> {
  static constexpr int kElems = 8;
  __device__ static void unpack(const uint4& q, float* o) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) { o[2 * j] = __uint_as_float(w[j] << 16); o[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u); }
  }
  __device__ static uint4 pack(const float* v) {
    return make_uint4(f32x2_to_bf16x2(v[0], v[1]), f32x2_to_bf16x2(v[2], v[3]), f32x2_to_bf16x2(v[4], v[5]), f32x2_to_bf16x2(v[6], v[7]));
  }
};
template <> struct EwVec<__half> {
  static constexpr int kElems = 8;
  __device__ static void unpack(const uint4& q, float* o) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) { o[2 * j] = f16_bits_to_f32(w[j] & 0xffffu); o[2 * j + 1] = f16_bits_to_f32(w[j] >> 16); }
  }
  __device__ static uint4 pack(const float* v) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) w[j] = f32_to_f16_bits(v[2 * j]) | (f32_to_f16_bits(v[2 * j + 1]) << 16);
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// Functors: NIN inputs -> one value.  __fmul_rn / __fadd_rn keep separately rounded operations
// separate (the compiler would otherwise contract them, the interpreter cannot).
struct FRelu { static constexpr int kIn = 1; __device__ static float f(float a, float, float, float) { return fmaxf(a, 0.0f); } };
struct FGelu {
  static constexpr int kIn = 1;
  __device__ static float f(float a, float, float, float) { return 0.5f * a * (1.0f + erff(a * 0.70710678118654752440f)); }
};
struct FAdd { static constexpr int kIn = 2; __device__ static float f(float a, float b, float, float) { return __fadd_rn(a, b); } };
struct FMul { static constexpr int kIn = 2; __device__ static float f(float a, float b, float, float) { return __fmul_rn(a, b); } };
struct FAddRelu { static constexpr int kIn = 2; __device__ static float f(float a, float b, float, float) { return fmaxf(__fadd_rn(a, b), 0.0f); } };
// canonical `prod(I0, relu(I1))`
struct FMulRelu { static constexpr int kIn = 2; __device__ static float f(float a, float b, float, float) { return __fmul_rn(a, fmaxf(b, 0.0f)); } };
// canonical `sum(I0, prod(I1, I2))`: the mul feeds only the add, so it is one fma in both tiers
struct FFma { static constexpr int kIn = 3; __device__ static float f(float a, float b, float c, float) { return fmaf(b, c, a); } };
// canonical `sum(I0, neg(prod(I1, K)))`: mul, neg, add are three separately rounded steps
struct FAxmy { static constexpr int kIn = 2; __device__ static float f(float a, float b, float, float k) { return __fadd_rn(a, -__fmul_rn(b, k)); } };

template <class F, typename T>
__global__ void __launch_bounds__(kEwThreads) ew_dense_kernel(const __grid_constant__ EwParams p) {
  using V = EwVec<T>;
  const unsigned long long stride = (unsigned long long)gridDim.x * kEwThreads * kEwUnroll;
  for (unsigned long long base = (unsigned long long)blockIdx.x * kEwThreads * kEwUnroll + threadIdx.x; base < p.n_vec; base += stride) {
    uint4 q[3][kEwUnroll];
#pragma unroll
    for (int u = 0; u < kEwUnroll; ++u) {
      const unsigned long long i = base + (unsigned long long)u * kEwThreads;
      if (i < p.n_vec) {
#pragma unroll
        for (int t = 0; t < F::kIn; ++t) q[t][u] = __ldcs(reinterpret_cast<const uint4*>(p.in[t]) + i);
      }
    }
#pragma unroll
    for (int u = 0; u < kEwUnroll; ++u) {
      const unsigned long long i = base + (unsigned long long)u * kEwThreads;
      if (i >= p.n_vec) break;
      float a[V::kElems], b[V::kElems], c[V::kElems], r[V::kElems];
      V::unpack(q[0][u], a);
      if (F::kIn > 1) V::unpack(q[1][u], b);
      if (F::kIn > 2) V::unpack(q[2][u], c);
#pragma unroll
      for (int e = 0; e < V::kElems; ++e) r[e] = F::f(a[e], F::kIn > 1 ? b[e] : 0.0f, F::kIn > 2 ? c[e] : 0.0f, p.k);
      __stcs(reinterpret_cast<uint4*>(p.out) + i, V::pack(r));
    }
  }
}

template <class F>
int32_t launch_for_dtype(int dt, const EwParams& p, unsigned grid, cudaStream_t stream) {
  if (dt == HE_F32) ew_dense_kernel<F, float><<<grid, kEwThreads, 0, stream>>>(p);
  else if (dt == HE_BF16) ew_dense_kernel<F, __nv_bfloat16><<<grid, kEwThreads, 0, stream>>>(p);
  else ew_dense_kernel<F, __half><<<grid, kEwThreads, 0, stream>>>(p);
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

struct Entry {
  const char* text;   // canonical text with the constant blanked to K*
  int kind;
  int n_in;
  const char* name;
};
const Entry kTable[] = {
    {"store(u8(I0:F));", EW_RELU, 1, "relu(a)"},
    {"store(u16(I0:F));", EW_GELU, 1, "gelu(a)"},
    {"store(sum(I0:F,I1:F));", EW_ADD, 2, "a + b"},
    {"store(prod(I0:F,I1:F));", EW_MUL, 2, "a * b"},
    {"store(u8(sum(I0:F,I1:F)));", EW_ADD_RELU, 2, "relu(a + b)"},
    {"store(prod(I0:F,u8(I1:F)));", EW_MUL_RELU, 2, "a * relu(b)"},
    {"store(sum(I0:F,prod(I1:F,I2:F)));", EW_FMA, 3, "a + b * c"},
    {"store(sum(I0:F,u1(prod(I1:F,K*))));", EW_AXMY, 2, "a - k * b"},
};

}  // namespace

bool match_dense_elementwise(const std::string& canon_text, EwMatch* m) {
  // blank the (single) constant, remembering its bits
  std::string t = canon_text;
  uint32_t kbits = 0;
  int n_const = 0;
  for (size_t i = 0; i + 9 <= t.size(); ++i) {
    if (t[i] != 'K') continue;
    bool hex = true;
    for (int j = 1; j <= 8; ++j) hex = hex && isxdigit((unsigned char)t[i + j]);
    if (!hex) continue;
    kbits = (uint32_t)strtoul(t.substr(i + 1, 8).c_str(), nullptr, 16);
    t.replace(i + 1, 8, "*");
    ++n_const;
  }
  if (n_const > 1) return false;
  for (const Entry& e : kTable)
    if (t == e.text) {
      m->kind = e.kind;
      m->n_in = e.n_in;
      m->name = e.name;
      memcpy(&m->k, &kbits, 4);
      return true;
    }
  return false;
}

namespace {
// Column sums of a dense [batch, M, N] tensor: out[b, n] = sum_m x[b, m, n] -- what helium's bias
// gradient (swap_dims -> reduce_sum -> reshape, tensor.rs:83-142) computes when its operand is a
// plain tensor.  A thread owns 16 bytes of consecutive columns and walks rows ty, ty + 8, ... of its
// slice, so every warp load is one contiguous 512-byte run; the eight row lanes meet in shared
// memory; one partial per (column, slice), folded by the generic finalize kernel in slice order.
struct ColsumParams {
  const void* x;
  float* out;        // [batch * N] when slices == 1, else partials [(b * N + n) * slices + slice]
  unsigned M, N, batch, rows_per_slice, slices;
};

template <typename T>
__global__ void __launch_bounds__(256) colsum_dense_kernel(const __grid_constant__ ColsumParams p) {
  using V = EwVec<T>;
  constexpr int VE = V::kElems;
  __shared__ float part[8][32][VE + 1];
  const unsigned tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const unsigned col0 = (blockIdx.x * 32 + tx) * VE, slice = blockIdx.y, b = blockIdx.z;
  float acc[VE];
#pragma unroll
  for (int e = 0; e < VE; ++e) acc[e] = 0.0f;
  if (col0 < p.N) {
    const unsigned r_end = min(p.M, (slice + 1) * p.rows_per_slice);
    const T* base = reinterpret_cast<const T*>(p.x) + ((size_t)b * p.M) * p.N + col0;
    for (unsigned r = slice * p.rows_per_slice + ty; r < r_end; r += 8) {
      float v[VE];
      V::unpack(__ldcs(reinterpret_cast<const uint4*>(base + (size_t)r * p.N)), v);
#pragma unroll
      for (int e = 0; e < VE; ++e) acc[e] += v[e];
    }
  }
#pragma unroll
  for (int e = 0; e < VE; ++e) part[ty][tx][e] = acc[e];
  __syncthreads();
  if (ty == 0 && col0 < p.N) {
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      float v = part[0][tx][e];
#pragma unroll
      for (int w = 1; w < 8; ++w) v += part[w][tx][e];
      const size_t group = (size_t)b * p.N + col0 + e;
      if (p.slices == 1) p.out[group] = v;
      else p.out[group * p.slices + slice] = v;
    }
  }
}
}  // namespace

int32_t launch_colsum_dense(int dtype, const void* x, float* out_or_partials, unsigned batch, unsigned M, unsigned N,
                            unsigned slices, unsigned rows_per_slice, cudaStream_t stream) {
  const unsigned ve = dtype == HE_F32 ? 4 : 8;
  ColsumParams p{x, out_or_partials, M, N, batch, rows_per_slice, slices};
  dim3 grid((N / ve + 31) / 32, slices, batch);
  if (grid.y > 65535 || grid.z > 65535) HE_FAIL(HE_ERR_UNSUPPORTED, "dense column sum: shape too large");
  if (dtype == HE_F32) colsum_dense_kernel<float><<<grid, 256, 0, stream>>>(p);
  else if (dtype == HE_BF16) colsum_dense_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(p);
  else colsum_dense_kernel<__half><<<grid, 256, 0, stream>>>(p);
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

int32_t launch_dense_elementwise(int kind, int dtype, const void* const* in, void* out, unsigned long long n_elems, float k,
                                 int sm_count, cudaStream_t stream) {
  const int ve = dtype == HE_F32 ? 4 : 8;
  EwParams p{};
  for (int t = 0; t < 3; ++t) p.in[t] = in[t];
  p.out = out;
  p.n_vec = n_elems / ve;
  p.k = k;
  const unsigned long long per_cta = (unsigned long long)kEwThreads * kEwUnroll;
  // enough CTAs for every vector, capped at 32 per SM's worth (the loop strides over the rest)
  const unsigned grid = (unsigned)std::max<unsigned long long>(1, std::min<unsigned long long>((p.n_vec + per_cta - 1) / per_cta,
                                                                                             (unsigned long long)sm_count * 32));
  switch (kind) {
    case EW_RELU: return launch_for_dtype<FRelu>(dtype, p, grid, stream);
    case EW_GELU: return launch_for_dtype<FGelu>(dtype, p, grid, stream);
    case EW_ADD: return launch_for_dtype<FAdd>(dtype, p, grid, stream);
    case EW_MUL: return launch_for_dtype<FMul>(dtype, p, grid, stream);
    case EW_ADD_RELU: return launch_for_dtype<FAddRelu>(dtype, p, grid, stream);
    case EW_MUL_RELU: return launch_for_dtype<FMulRelu>(dtype, p, grid, stream);
    case EW_FMA: return launch_for_dtype<FFma>(dtype, p, grid, stream);
    case EW_AXMY: return launch_for_dtype<FAxmy>(dtype, p, grid, stream);
    default: HE_FAIL(HE_ERR_INVALID, "dense elementwise: unknown kernel %d", kind);
  }
}

// Row re-pitching copy for matmul operands whose row length breaks the 16-byte rule of TMA.  A warp walks a
// row in 64-byte steps of 2-byte loads (source rows of odd length start on odd 2-byte addresses) and
// writes the 16-byte-aligned destination row the same way; HBM-bound in spite of the narrow accesses
// because every byte of every sector that is touched is used.
__global__ void __launch_bounds__(256) pad_rows_kernel(const unsigned short* __restrict__ src, unsigned short* __restrict__ dst,
                                                       long long rows, long long cols, long long dst_pitch) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = warp; r < rows; r += n_warps) {
    const unsigned short* s = src + r * cols;
    unsigned short* d = dst + r * dst_pitch;
    for (long long c = lane; c < cols; c += 32) d[c] = __ldg(s + c);
  }
}

int32_t launch_pad_rows(const void* src, void* dst, long long rows, long long cols, long long dst_pitch, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return HE_OK;
  const long long warps = std::min<long long>(rows, 148ll * 64);
  const unsigned grid = (unsigned)((warps * 32 + 255) / 256);
  pad_rows_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const unsigned short*>(src), reinterpret_cast<unsigned short*>(dst), rows,
                                            cols, dst_pitch);
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}


// ---- 8-bit operand copies --------------------------------------------------------------------------------
namespace {
__device__ __forceinline__ unsigned f8x2(float lo, float hi, int e5m2) {
  unsigned short r;
  if (e5m2) asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  else asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float load_as_f32(const void* p, int dt, long long i) {
  if (dt == HE_F32) return __ldg(reinterpret_cast<const float*>(p) + i);
  const unsigned h = __ldg(reinterpret_cast<const unsigned short*>(p) + i);
  return dt == HE_BF16 ? bf16_bits_to_f32(h) : f16_bits_to_f32(h);
}

// rows of k elements, k contiguous: a thread converts 16 consecutive elements into one 16-byte store
__global__ void __launch_bounds__(256) to_f8_rows_kernel(const void* __restrict__ src, int dt, unsigned char* __restrict__ dst, long long rows,
                                                         long long k, long long k_pitch, int e5m2) {
  const long long vec_per_row = (k + 15) / 16;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < rows * vec_per_row; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row, c0 = (i - r * vec_per_row) * 16;
    const long long base = r * k + c0;
    float v[16];
    if (c0 + 16 <= k && dt != HE_F32 && ((base * 2 + reinterpret_cast<uintptr_t>(src)) & 15) == 0) {
      const uint4 a = __ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(src) + base));
      const uint4 b = __ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(src) + base) + 1);
      const unsigned w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[2 * j] = dt == HE_BF16 ? __uint_as_float(w[j] << 16) : f16_bits_to_f32(w[j] & 0xffffu);
        v[2 * j + 1] = dt == HE_BF16 ? __uint_as_float(w[j] & 0xffff0000u) : f16_bits_to_f32(w[j] >> 16);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = c0 + j < k ? load_as_f32(src, dt, base + j) : 0.0f;
    }
    unsigned o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = f8x2(v[4 * j], v[4 * j + 1], e5m2) | (f8x2(v[4 * j + 2], v[4 * j + 3], e5m2) << 16);
    unsigned char* d = dst + r * k_pitch + c0;
    if (c0 + 16 <= k_pitch) {
      *reinterpret_cast<uint4*>(d) = make_uint4(o[0], o[1], o[2], o[3]);   // k_pitch is a multiple of 16: the store stays inside the row
    }
  }
}

// [batch, k, rows] -> [batch, rows, k_pitch]: 64 x 64 tiles through shared memory (reads coalesced along rows,
// writes along k)
__global__ void __launch_bounds__(256) to_f8_transpose_kernel(const void* __restrict__ src, int dt, unsigned char* __restrict__ dst, long long rows,
                                                              long long k, long long k_pitch, int e5m2) {
  __shared__ float tile[64][65];
  const long long b = blockIdx.z;
  const long long r0 = (long long)blockIdx.x * 64, k0 = (long long)blockIdx.y * 64;
  // a thread reads 8 consecutive rows' worth of one k (one 16-byte load of 2-byte elements, two of f32), twice
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    const int kk = (threadIdx.x >> 3) + 32 * pass, ro = (threadIdx.x & 7) * 8;
    const long long kq = k0 + kk, r = r0 + ro;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.0f;
    if (kq < k && r < rows) {
      const long long e = (b * k + kq) * rows + r;
      const char* ptr = reinterpret_cast<const char*>(src) + e * (dt == HE_F32 ? 4 : 2);
      if (r + 8 <= rows && (reinterpret_cast<uintptr_t>(ptr) & 15) == 0) {
        if (dt == HE_F32) {
          const float4 a = __ldcs(reinterpret_cast<const float4*>(ptr)), c = __ldcs(reinterpret_cast<const float4*>(ptr) + 1);
          v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = c.x; v[5] = c.y; v[6] = c.z; v[7] = c.w;
        } else {
          const uint4 a = __ldcs(reinterpret_cast<const uint4*>(ptr));
          const unsigned w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            v[2 * j] = dt == HE_BF16 ? __uint_as_float(w[j] << 16) : f16_bits_to_f32(w[j] & 0xffffu);
            v[2 * j + 1] = dt == HE_BF16 ? __uint_as_float(w[j] & 0xffff0000u) : f16_bits_to_f32(w[j] >> 16);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (r + j < rows) v[j] = load_as_f32(src, dt, e + j);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) tile[kk][ro + j] = v[j];
  }
  __syncthreads();
  // a thread writes 16 consecutive k of one row: 4 threads per row, 64 rows
  const int row = threadIdx.x >> 2, seg = threadIdx.x & 3;
  const long long r = r0 + row, kq = k0 + seg * 16;
  if (r < rows && kq < k_pitch) {
    unsigned o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      o[j] = f8x2(tile[seg * 16 + 4 * j][row], tile[seg * 16 + 4 * j + 1][row], e5m2) |
             (f8x2(tile[seg * 16 + 4 * j + 2][row], tile[seg * 16 + 4 * j + 3][row], e5m2) << 16);
    *reinterpret_cast<uint4*>(dst + (b * rows + r) * k_pitch + kq) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}
}  // namespace

int32_t launch_to_f8(const void* src, int src_dtype, bool transposed, void* dst, long long batch, long long rows, long long k,
                     long long k_pitch, int e5m2, cudaStream_t stream) {
  if (!src || !dst || batch <= 0 || rows <= 0 || k <= 0) HE_FAIL(HE_ERR_INVALID, "8-bit operand copy: bad argument");
  if (k_pitch % 16 != 0 || k_pitch < k || (reinterpret_cast<uintptr_t>(dst) & 15)) HE_FAIL(HE_ERR_INVALID, "8-bit operand copy: pitch / alignment");
  if (!transposed) {
    const long long n = batch * rows * ((k + 15) / 16);
    const unsigned grid = (unsigned)std::max<long long>(1, std::min<long long>((n + 255) / 256, 148 * 16));
    to_f8_rows_kernel<<<grid, 256, 0, stream>>>(src, src_dtype, reinterpret_cast<unsigned char*>(dst), batch * rows, k, k_pitch, e5m2);
  } else {
    if (batch > 65535 || (k + 63) / 64 > 65535) HE_FAIL(HE_ERR_UNSUPPORTED, "8-bit operand copy: grid too large");
    dim3 grid((unsigned)((rows + 63) / 64), (unsigned)((k + 63) / 64), (unsigned)batch);
    to_f8_transpose_kernel<<<grid, 256, 0, stream>>>(src, src_dtype, reinterpret_cast<unsigned char*>(dst), rows, k, k_pitch, e5m2);
  }
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

}  // namespace he
