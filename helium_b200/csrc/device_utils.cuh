// Small device-side helpers shared by the kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

namespace he {

// Division by a runtime-constant divisor for n < 2^31: q = umulhi(n, m) >> s.
// m = ceil(2^(31+p) / d) with p = ceil(log2 d); the error term n*e/(d*2^(31+p)) stays below 1/d.
struct FastDiv {
  uint32_t d, m, s;  // s = p - 1; d == 1 is flagged by m == 0
#ifdef __CUDACC__
  __host__ __device__
#endif
  FastDiv() : d(1), m(0), s(0) {}
  explicit FastDiv(uint32_t div) : d(div), m(0), s(0) {
    if (div > 1) {
      uint32_t p = 0;
      while ((1ull << p) < div) ++p;
      m = (uint32_t)(((1ull << (31 + p)) + div - 1) / div);
      s = p - 1;
    }
  }
#ifdef __CUDACC__
  __device__ __forceinline__ uint32_t div(uint32_t n) const { return m == 0 ? n : (__umulhi(n, m) >> s); }
  __device__ __forceinline__ void divmod(uint32_t n, uint32_t& q, uint32_t& r) const {
    q = div(n);
    r = n - q * d;
  }
#endif
};

#ifdef __CUDACC__
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b) { return __uint_as_float(b << 16); }
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ float f16_bits_to_f32(uint32_t b) {
  return __half2float(__ushort_as_half((unsigned short)b));
}
__device__ __forceinline__ uint32_t f32_to_f16_bits(float f) {
  return (uint32_t)__half_as_ushort(__float2half_rn(f));
}
// Unpack two bf16 packed in one 32-bit word (low half = lower address).
__device__ __forceinline__ float2 bf16x2_to_f32(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
__device__ __forceinline__ uint32_t f32x2_to_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// Loads a scalar parameter stored as `dt` (HE_F16/HE_BF16/HE_F32 numbering) as float.
__device__ __forceinline__ float load_param_as_f32(const void* p, int dt, long long idx) {
  if (dt == 2) return __ldg(reinterpret_cast<const float*>(p) + idx);
  uint32_t h = __ldg(reinterpret_cast<const unsigned short*>(p) + idx);
  return dt == 1 ? bf16_bits_to_f32(h) : f16_bits_to_f32(h);
}
#endif

}  // namespace he
