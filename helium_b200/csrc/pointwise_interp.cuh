// Device-side interpreter for PwProgram.  One call evaluates the whole program for V consecutive
// elements of the iteration space; values live in a small per-thread register file.
//
// Arithmetic follows the reference's generated code: f32 intermediates, accurate libm functions
// (expf, tanhf, ... pointwise/jit.rs:532-546), `static_cast` rounding on store (jit.rs:99-106),
// bool tensors bit-packed LSB-first (jit.rs:107-114, 234-237).
#pragma once
#include "pointwise_program.h"

namespace he {

__device__ __forceinline__ uint32_t pw_apply_views(const PwProgram& P, int v0, int nv, uint32_t idx) {
#pragma unroll 1
  for (int v = 0; v < nv; ++v) {
    const PwView& vw = P.views[v0 + v];
    uint32_t rem = idx, off = 0;
#pragma unroll 1
    for (int k = 0; k < vw.nd; ++k) {
      uint32_t q, c;
      vw.fd[k].divmod(rem, q, c);
      rem = q;
      off += c * vw.stride[k];
    }
    idx = off;
  }
  return idx;
}

__device__ __forceinline__ uint32_t pw_load_elem(const void* base, int dt, uint32_t idx) {
  switch (dt) {
    case HE_F32: return __float_as_uint(__ldg(reinterpret_cast<const float*>(base) + idx));
    case HE_BF16: return (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(base) + idx) << 16;
    case HE_F16: return __float_as_uint(f16_bits_to_f32(__ldg(reinterpret_cast<const unsigned short*>(base) + idx)));
    case HE_U32: return __ldg(reinterpret_cast<const uint32_t*>(base) + idx);
    default: return (__ldg(reinterpret_cast<const uint32_t*>(base) + (idx >> 5)) >> (idx & 31)) & 1u;
  }
}

__device__ __forceinline__ float pw_gelu(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f)); }
__device__ __forceinline__ float pw_dgelu(float x) {
  const float cdf = 0.5f * (1.0f + erff(x * 0.70710678118654752440f));
  const float pdf = 0.39894228040143267794f * expf(-0.5f * x * x);
  return cdf + x * pdf;
}

__device__ __forceinline__ float pw_unary(int op, float x, uint32_t imm) {
  switch (op) {
    case HE_UN_RECIP: return 1.0f / x;
    case HE_UN_NEG: return -x;
    case HE_UN_EXP: return expf(x);
    case HE_UN_SIN: return sinf(x);
    case HE_UN_COS: return cosf(x);
    case HE_UN_TAN: return tanf(x);
    case HE_UN_SIGMOID: return 1.0f / (1.0f + expf(-x));
    case HE_UN_TANH: return tanhf(x);
    case HE_UN_RELU: return fmaxf(x, 0.0f);
    case HE_UN_SQRT: return sqrtf(x);
    case HE_UN_LOG: return logf(x);
    case HE_UN_GELU: return pw_gelu(x);
    case HE_UN_ADD_CONST: return x + __uint_as_float(imm);
    case HE_UN_MUL_CONST: return x * __uint_as_float(imm);
    case HE_UN_POW_CONST: {
      const float c = __uint_as_float(imm);
      return c == 2.0f ? x * x : powf(x, c);
    }
    case HE_UN_DGELU: return pw_dgelu(x);
    default: return x;
  }
}

__device__ __forceinline__ float pw_bin_f(int op, float a, float b) {
  switch (op) {
    case HE_BIN_ADD: return a + b;
    case HE_BIN_MUL: return a * b;
    case HE_BIN_POW: return powf(a, b);
    case HE_BIN_MIN: return fminf(a, b);
    case HE_BIN_MAX: return fmaxf(a, b);
    case HE_BIN_SUB: return a - b;
    case HE_BIN_DIV: return a / b;
    case HE_BIN_DRELU: return b > 0.0f ? a : 0.0f;
    default: return a;
  }
}

__device__ __forceinline__ uint32_t pw_bin_u(int op, uint32_t a, uint32_t b) {
  switch (op) {
    case HE_BIN_ADD: return a + b;
    case HE_BIN_MUL: return a * b;
    case HE_BIN_MIN: return min(a, b);
    case HE_BIN_MAX: return max(a, b);
    case HE_BIN_AND: return a & b;
    case HE_BIN_OR: return a | b;
    case HE_BIN_XOR: return a ^ b;
    case HE_BIN_SUB: return a - b;
    default: return a;
  }
}

template <typename T>
__device__ __forceinline__ bool pw_cmp(int op, T a, T b) {
  switch (op) {
    case HE_CMP_EQ: return a == b;
    case HE_CMP_NE: return a != b;
    case HE_CMP_LT: return a < b;
    case HE_CMP_LE: return a <= b;
    case HE_CMP_GT: return a > b;
    default: return a >= b;
  }
}

__device__ __forceinline__ float pw_reduce_combine(int op, float a, float b) {
  return op == HE_RED_MAX ? fmaxf(a, b) : op == HE_RED_MIN ? fminf(a, b) : a + b;
}
__device__ __forceinline__ float pw_reduce_identity(int op) {
  return op == HE_RED_MAX ? -INFINITY : op == HE_RED_MIN ? INFINITY : 0.0f;
}

// Evaluates the program for elements [idx0, idx0 + V) of which the first `nvalid` exist.
//   acc[j]      : matmul accumulator values (PW_ACC), ignored by stand-alone pointwise kernels
//   red[s]      : running reduction values, updated with every valid element
//   STORE_BOOL_BALLOT: bool outputs are written one word per warp with __ballot_sync (V == 1 and
//                      idx0 = 32 * k + lane); all lanes of the warp must call with the same program.
//   colv[s][j] : fused-matmul epilogues only.  A reduction over the rows of the output tile (axes mask
//                 2 or 6: "Columns" sums) cannot be folded into a per-thread scalar, because a thread
//                 owns one row; the values of its V elements are handed back per reduction slot and
//                 the caller sums them across the warp's rows.  Invalid elements yield 0.
template <int V>
__device__ __forceinline__ void pw_run(const PwProgram& P, uint32_t idx0, int nvalid, const float* acc,
                                       float* red, float (*colv)[V] = nullptr) {
  uint32_t R[kPwMaxRegs][V];
#pragma unroll 1
  for (int pc = 0; pc < P.n_instr; ++pc) {
    const PwInstr in = P.instr[pc];
    switch (in.op) {
      case PW_LOAD: {
        const void* base = P.in[in.slot];
        if (in.nviews == 0) {
          bool done = false;
          if (V == 4 && nvalid == 4) {
            if (in.dt == HE_F32 || in.dt == HE_U32) {
              if ((reinterpret_cast<uintptr_t>(base) & 15) == 0) {
                const uint4 v = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(base) + (size_t)idx0 * 4));
                R[in.dst][0] = v.x; R[in.dst][1 % V] = v.y; R[in.dst][2 % V] = v.z; R[in.dst][3 % V] = v.w;
                done = true;
              }
            } else if (in.dt == HE_BF16 || in.dt == HE_F16) {
              if ((reinterpret_cast<uintptr_t>(base) & 7) == 0) {
                const uint2 v = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const char*>(base) + (size_t)idx0 * 2));
                if (in.dt == HE_BF16) {
                  R[in.dst][0] = v.x << 16; R[in.dst][1 % V] = v.x & 0xffff0000u;
                  R[in.dst][2 % V] = v.y << 16; R[in.dst][3 % V] = v.y & 0xffff0000u;
                } else {
                  R[in.dst][0] = __float_as_uint(f16_bits_to_f32(v.x & 0xffffu));
                  R[in.dst][1 % V] = __float_as_uint(f16_bits_to_f32(v.x >> 16));
                  R[in.dst][2 % V] = __float_as_uint(f16_bits_to_f32(v.y & 0xffffu));
                  R[in.dst][3 % V] = __float_as_uint(f16_bits_to_f32(v.y >> 16));
                }
                done = true;
              }
            }
          }
          if (!done) {
#pragma unroll
            for (int j = 0; j < V; ++j) R[in.dst][j] = j < nvalid ? pw_load_elem(base, in.dt, idx0 + j) : 0u;
          }
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j)
            R[in.dst][j] = j < nvalid ? pw_load_elem(base, in.dt, pw_apply_views(P, in.view0, in.nviews, idx0 + j)) : 0u;
        }
        break;
      }
      case PW_CONST:
#pragma unroll
        for (int j = 0; j < V; ++j) R[in.dst][j] = in.imm;
        break;
      case PW_ACC:
#pragma unroll
        for (int j = 0; j < V; ++j) R[in.dst][j] = __float_as_uint(acc[j]);
        break;
      case PW_UNARY:
#pragma unroll
        for (int j = 0; j < V; ++j) R[in.dst][j] = __float_as_uint(pw_unary(in.sub, __uint_as_float(R[in.a][j]), in.imm));
        break;
      case PW_BIN_F:
#pragma unroll
        for (int j = 0; j < V; ++j)
          R[in.dst][j] = __float_as_uint(pw_bin_f(in.sub, __uint_as_float(R[in.a][j]), __uint_as_float(R[in.b][j])));
        break;
      case PW_FMA:
#pragma unroll
        for (int j = 0; j < V; ++j)
          R[in.dst][j] = __float_as_uint(fmaf(__uint_as_float(R[in.a][j]), __uint_as_float(R[in.b][j]), __uint_as_float(R[in.c][j])));
        break;
      case PW_BIN_U:
#pragma unroll
        for (int j = 0; j < V; ++j) R[in.dst][j] = pw_bin_u(in.sub, R[in.a][j], R[in.b][j]);
        break;
      case PW_BIN_B:
#pragma unroll
        for (int j = 0; j < V; ++j) R[in.dst][j] = pw_bin_u(in.sub, R[in.a][j], R[in.b][j]) & 1u;
        break;
      case PW_CMP_F:
#pragma unroll
        for (int j = 0; j < V; ++j) R[in.dst][j] = pw_cmp<float>(in.sub, __uint_as_float(R[in.a][j]), __uint_as_float(R[in.b][j])) ? 1u : 0u;
        break;
      case PW_CMP_U:
#pragma unroll
        for (int j = 0; j < V; ++j) R[in.dst][j] = pw_cmp<uint32_t>(in.sub, R[in.a][j], R[in.b][j]) ? 1u : 0u;
        break;
      case PW_SELECT:
#pragma unroll
        for (int j = 0; j < V; ++j) R[in.dst][j] = R[in.c][j] ? R[in.b][j] : R[in.a][j];
        break;
      case PW_CVT:
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const uint32_t x = R[in.a][j];
          uint32_t y;
          switch (in.sub) {
            case (0 << 2 | 2): y = __uint_as_float(x) != 0.0f ? 1u : 0u; break;          // float -> bool
            case (2 << 2 | 0): y = x ? __float_as_uint(1.0f) : 0u; break;                 // bool -> float
            case (0 << 2 | 1): y = __float2uint_rz(__uint_as_float(x)); break;             // float -> u32
            case (1 << 2 | 0): y = __float_as_uint((float)x); break;                       // u32 -> float
            case (2 << 2 | 1): y = x ? 1u : 0u; break;                                     // bool -> u32
            default: y = x != 0u ? 1u : 0u; break;                                         // u32 -> bool
          }
          R[in.dst][j] = y;
        }
        break;
      case PW_MEAN_SCALE:
#pragma unroll
        for (int j = 0; j < V; ++j) R[in.dst][j] = __float_as_uint((float)((double)__uint_as_float(R[in.a][j]) * P.mean_scale));
        break;
      case PW_STORE: {
        void* base = P.out[in.slot];
        if (in.dt == HE_BOOL) {
          // V == 1 by construction: one bit per lane, one word per warp
          const uint32_t word = __ballot_sync(0xffffffffu, nvalid > 0 && R[in.a][0] != 0u);
          if ((threadIdx.x & 31) == 0 && nvalid > 0) reinterpret_cast<uint32_t*>(base)[idx0 >> 5] = word;
        } else if (V == 4 && nvalid == 4 && (in.dt == HE_F32 || in.dt == HE_U32) && (reinterpret_cast<uintptr_t>(base) & 15) == 0) {
          *reinterpret_cast<uint4*>(reinterpret_cast<char*>(base) + (size_t)idx0 * 4) =
              make_uint4(R[in.a][0], R[in.a][1 % V], R[in.a][2 % V], R[in.a][3 % V]);
        } else if (V == 4 && nvalid == 4 && in.dt == HE_BF16 && (reinterpret_cast<uintptr_t>(base) & 7) == 0) {
          uint2 v;
          v.x = f32x2_to_bf16x2(__uint_as_float(R[in.a][0]), __uint_as_float(R[in.a][1 % V]));
          v.y = f32x2_to_bf16x2(__uint_as_float(R[in.a][2 % V]), __uint_as_float(R[in.a][3 % V]));
          *reinterpret_cast<uint2*>(reinterpret_cast<char*>(base) + (size_t)idx0 * 2) = v;
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j) {
            if (j >= nvalid) break;
            const uint32_t x = R[in.a][j];
            const size_t i = (size_t)idx0 + j;
            if (in.dt == HE_F32 || in.dt == HE_U32) reinterpret_cast<uint32_t*>(base)[i] = x;
            else if (in.dt == HE_BF16) reinterpret_cast<unsigned short*>(base)[i] = (unsigned short)f32_to_bf16_bits(__uint_as_float(x));
            else reinterpret_cast<unsigned short*>(base)[i] = (unsigned short)f32_to_f16_bits(__uint_as_float(x));
          }
        }
        break;
      }
      case PW_REDUCE:
        if (colv && (in.imm & 3u) == 2u) {
#pragma unroll
          for (int j = 0; j < V; ++j) colv[in.slot2 & 3][j] = j < nvalid ? __uint_as_float(R[in.a][j]) : 0.0f;
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j)
            if (j < nvalid) red[in.slot2] = pw_reduce_combine(in.sub, red[in.slot2], __uint_as_float(R[in.a][j]));
        }
        break;
      default: break;
    }
  }
}

}  // namespace he
