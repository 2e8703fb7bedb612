// Plan-time specialisation of pointwise programs with NVRTC (see pointwise_jit.h).
//
// Generated kernel: a thread owns 8 consecutive elements of the iteration space per trip of a grid-stride loop.
// Identity-mapped tensors move as 16-byte vectors (one for 2-byte types, two for 4-byte types), tensors read
// through a view chain (broadcasts, permutations) are gathered element by element with the chain's divisions
// printed as multiply-high constants.  Arithmetic is the interpreter's, statement for statement: f32
// intermediates in 32-bit registers, separately rounded adds and multiplies (`__fadd_rn` / `__fmul_rn`; only
// PW_FMA contracts), the accurate libm functions, the same store conversions -- so both tiers give the same bits
// and the parity tests hold for either.
#include "pointwise_jit.h"

#include <dlfcn.h>

#include <cstdarg>
#include <cstring>
#include <map>
#include <mutex>
#include <vector>

namespace he {

namespace {

// ---- NVRTC through dlopen (the library is part of the CUDA toolkit, not of the driver) --------------------
typedef struct _nvrtcProgram* nvrtcProgram;
struct Nvrtc {
  void* handle = nullptr;
  int (*CreateProgram)(nvrtcProgram*, const char*, const char*, int, const char* const*, const char* const*) = nullptr;
  int (*CompileProgram)(nvrtcProgram, int, const char* const*) = nullptr;
  int (*GetCUBINSize)(nvrtcProgram, size_t*) = nullptr;
  int (*GetCUBIN)(nvrtcProgram, char*) = nullptr;
  int (*GetProgramLogSize)(nvrtcProgram, size_t*) = nullptr;
  int (*GetProgramLog)(nvrtcProgram, char*) = nullptr;
  int (*DestroyProgram)(nvrtcProgram*) = nullptr;
  std::string why;
};

const Nvrtc& nvrtc() {
  static Nvrtc n;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* env = getenv("HE_NVRTC_LIBRARY");
    const char* names[] = {env, "libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12", "libnvrtc.so.13"};
    for (const char* nm : names) {
      if (!nm || !*nm) continue;
      n.handle = dlopen(nm, RTLD_NOW | RTLD_LOCAL);
      if (n.handle) break;
      if (nm == env) break;   // an explicit choice is not second-guessed
    }
    if (!n.handle) {
      n.why = "the NVRTC library could not be loaded (set HE_NVRTC_LIBRARY)";
      return;
    }
    auto sym = [&](const char* s) { return dlsym(n.handle, s); };
    n.CreateProgram = reinterpret_cast<decltype(n.CreateProgram)>(sym("nvrtcCreateProgram"));
    n.CompileProgram = reinterpret_cast<decltype(n.CompileProgram)>(sym("nvrtcCompileProgram"));
    n.GetCUBINSize = reinterpret_cast<decltype(n.GetCUBINSize)>(sym("nvrtcGetCUBINSize"));
    n.GetCUBIN = reinterpret_cast<decltype(n.GetCUBIN)>(sym("nvrtcGetCUBIN"));
    n.GetProgramLogSize = reinterpret_cast<decltype(n.GetProgramLogSize)>(sym("nvrtcGetProgramLogSize"));
    n.GetProgramLog = reinterpret_cast<decltype(n.GetProgramLog)>(sym("nvrtcGetProgramLog"));
    n.DestroyProgram = reinterpret_cast<decltype(n.DestroyProgram)>(sym("nvrtcDestroyProgram"));
    if (!n.CreateProgram || !n.CompileProgram || !n.GetCUBINSize || !n.GetCUBIN || !n.GetProgramLogSize || !n.GetProgramLog ||
        !n.DestroyProgram) {
      n.why = "the NVRTC library lacks an entry point this build needs";
      dlclose(n.handle);
      n.handle = nullptr;
    }
  });
  return n;
}

// ---- source printer ------------------------------------------------------------------------------------
struct Src {
  std::string s;
  void f(const char* fmt, ...) __attribute__((format(printf, 2, 3))) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    s += buf;
  }
};

const char* kPrelude = R"SRC(
typedef unsigned int u32;
struct JitParams { const void* in[16]; void* out[8]; };
__device__ __forceinline__ float pw_gelu(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f)); }
__device__ __forceinline__ float pw_dgelu(float x) {
  const float cdf = 0.5f * (1.0f + erff(x * 0.70710678118654752440f));
  const float pdf = 0.39894228040143267794f * expf(-0.5f * x * x);
  return cdf + x * pdf;
}
__device__ __forceinline__ float h2f(u32 b) { float f; asm("{ .reg .b16 h; cvt.u16.u32 h, %1; cvt.f32.f16 %0, h; }" : "=f"(f) : "r"(b)); return f; }
__device__ __forceinline__ u32 f2h(float f) { u32 b; asm("{ .reg .b16 h; cvt.rn.f16.f32 h, %1; cvt.u32.u16 %0, h; }" : "=r"(b) : "f"(f)); return b; }
__device__ __forceinline__ u32 f2bf(float f) { u32 b; asm("{ .reg .b16 h; cvt.rn.bf16.f32 h, %1; cvt.u32.u16 %0, h; }" : "=r"(b) : "f"(f)); return b; }
__device__ __forceinline__ u32 ldg_elem_f32(const void* p, u32 i) { return __ldg((const u32*)p + i); }
__device__ __forceinline__ u32 ldg_elem_bf16(const void* p, u32 i) { return (u32)__ldg((const unsigned short*)p + i) << 16; }
__device__ __forceinline__ u32 ldg_elem_f16(const void* p, u32 i) { return __float_as_uint(h2f(__ldg((const unsigned short*)p + i))); }
__device__ __forceinline__ uint4 ldv(const void* p, size_t byte) { return __ldcs((const uint4*)((const char*)p + byte)); }
__device__ __forceinline__ void stv(void* p, size_t byte, uint4 v) { __stcs((uint4*)((char*)p + byte), v); }
)SRC";

std::string fbits(uint32_t bits) {
  char b[48];
  snprintf(b, sizeof b, "__uint_as_float(0x%08xu)", bits);
  return b;
}

// value of register k as float / as bits, for element lane `j` of the vector body or the scalar body
struct Regs {
  bool vec;
  std::string u(int k) const {
    char b[32];
    if (vec) snprintf(b, sizeof b, "R%d[j]", k);
    else snprintf(b, sizeof b, "r%d", k);
    return b;
  }
  std::string fl(int k) const { return "__uint_as_float(" + u(k) + ")"; }
};

bool unary_expr(int sub, const std::string& x, uint32_t imm, std::string* e) {
  switch (sub) {
    case HE_UN_RECIP: *e = "(1.0f / " + x + ")"; return true;
    case HE_UN_NEG: *e = "(-" + x + ")"; return true;
    case HE_UN_EXP: *e = "expf(" + x + ")"; return true;
    case HE_UN_SIN: *e = "sinf(" + x + ")"; return true;
    case HE_UN_COS: *e = "cosf(" + x + ")"; return true;
    case HE_UN_TAN: *e = "tanf(" + x + ")"; return true;
    case HE_UN_SIGMOID: *e = "(1.0f / __fadd_rn(1.0f, expf(-" + x + ")))"; return true;
    case HE_UN_TANH: *e = "tanhf(" + x + ")"; return true;
    case HE_UN_RELU: *e = "fmaxf(" + x + ", 0.0f)"; return true;
    case HE_UN_SQRT: *e = "sqrtf(" + x + ")"; return true;
    case HE_UN_LOG: *e = "logf(" + x + ")"; return true;
    case HE_UN_GELU: *e = "pw_gelu(" + x + ")"; return true;
    case HE_UN_ADD_CONST: *e = "__fadd_rn(" + x + ", " + fbits(imm) + ")"; return true;
    case HE_UN_MUL_CONST: *e = "__fmul_rn(" + x + ", " + fbits(imm) + ")"; return true;
    case HE_UN_POW_CONST: {
      float c;
      memcpy(&c, &imm, 4);
      *e = c == 2.0f ? "__fmul_rn(" + x + ", " + x + ")" : "powf(" + x + ", " + fbits(imm) + ")";
      return true;
    }
    case HE_UN_DGELU: *e = "pw_dgelu(" + x + ")"; return true;
    default: return false;
  }
}

bool bin_f_expr(int sub, const std::string& a, const std::string& b, std::string* e) {
  switch (sub) {
    case HE_BIN_ADD: *e = "__fadd_rn(" + a + ", " + b + ")"; return true;
    case HE_BIN_MUL: *e = "__fmul_rn(" + a + ", " + b + ")"; return true;
    case HE_BIN_POW: *e = "powf(" + a + ", " + b + ")"; return true;
    case HE_BIN_MIN: *e = "fminf(" + a + ", " + b + ")"; return true;
    case HE_BIN_MAX: *e = "fmaxf(" + a + ", " + b + ")"; return true;
    case HE_BIN_SUB: *e = "__fsub_rn(" + a + ", " + b + ")"; return true;
    case HE_BIN_DIV: *e = "__fdiv_rn(" + a + ", " + b + ")"; return true;
    case HE_BIN_DRELU: *e = "(" + b + " > 0.0f ? " + a + " : 0.0f)"; return true;
    default: return false;
  }
}

bool bin_u_expr(int sub, const std::string& a, const std::string& b, std::string* e) {
  switch (sub) {
    case HE_BIN_ADD: *e = "(" + a + " + " + b + ")"; return true;
    case HE_BIN_MUL: *e = "(" + a + " * " + b + ")"; return true;
    case HE_BIN_MIN: *e = "min(" + a + ", " + b + ")"; return true;
    case HE_BIN_MAX: *e = "max(" + a + ", " + b + ")"; return true;
    case HE_BIN_AND: *e = "(" + a + " & " + b + ")"; return true;
    case HE_BIN_OR: *e = "(" + a + " | " + b + ")"; return true;
    case HE_BIN_XOR: *e = "(" + a + " ^ " + b + ")"; return true;
    case HE_BIN_SUB: *e = "(" + a + " - " + b + ")"; return true;
    default: return false;
  }
}

const char* cmp_token(int sub) {
  switch (sub) {
    case HE_CMP_EQ: return "==";
    case HE_CMP_NE: return "!=";
    case HE_CMP_LT: return "<";
    case HE_CMP_LE: return "<=";
    case HE_CMP_GT: return ">";
    default: return ">=";
  }
}

// idx -> element offset through the view chain [v0, v0 + nv), divisions as multiply-high literals
void emit_views(Src& o, const PwProgram& P, int v0, int nv, const char* idx_in, const char* idx_out) {
  o.f("      u32 %s = %s;\n", idx_out, idx_in);
  for (int v = 0; v < nv; ++v) {
    const PwView& vw = P.views[v0 + v];
    o.f("      { u32 rem = %s, off = 0u, q;\n", idx_out);
    for (int k = 0; k < vw.nd; ++k) {
      const FastDiv& fd = vw.fd[k];
      if (fd.m == 0) o.f("        q = rem;");
      else o.f("        q = __umulhi(rem, %uu) >> %u;", fd.m, fd.s);
      if (vw.stride[k] != 0) o.f(" off += (rem - q * %uu) * %uu;", fd.d, vw.stride[k]);
      o.f(" rem = q;\n");
    }
    o.f("        %s = off; }\n", idx_out);
  }
}

const char* elem_loader(int dt) { return dt == HE_BF16 ? "ldg_elem_bf16" : dt == HE_F16 ? "ldg_elem_f16" : "ldg_elem_f32"; }

// One program instruction as statements.  `vec`: the 8-lane body (identity tensors as 16-byte vectors); else
// the scalar tail body for element idx0 + j.
bool emit_instr(Src& o, const PwProgram& P, const PwInstr& in, bool vec, std::string* why) {
  const Regs R{vec};
  const char* loop = vec ? "#pragma unroll\n      for (int j = 0; j < 8; ++j) " : "";
  std::string e;
  switch (in.op) {
    case PW_LOAD: {
      if (in.dt == HE_BOOL) { *why = "bit-packed bool load"; return false; }
      if (in.nviews == 0) {
        if (!vec) {
          o.f("      r%d = %s(p.in[%d], idx0 + j);\n", in.dst, elem_loader(in.dt), in.slot);
        } else if (in.dt == HE_F32 || in.dt == HE_U32) {
          o.f("      { const uint4 a = ldv(p.in[%d], (size_t)idx0 * 4), b = ldv(p.in[%d], (size_t)idx0 * 4 + 16);\n", in.slot, in.slot);
          o.f("        R%d[0] = a.x; R%d[1] = a.y; R%d[2] = a.z; R%d[3] = a.w; R%d[4] = b.x; R%d[5] = b.y; R%d[6] = b.z; R%d[7] = b.w; }\n",
              in.dst, in.dst, in.dst, in.dst, in.dst, in.dst, in.dst, in.dst);
        } else {
          o.f("      { const uint4 a = ldv(p.in[%d], (size_t)idx0 * 2); const u32 w[4] = {a.x, a.y, a.z, a.w};\n", in.slot);
          if (in.dt == HE_BF16)
            o.f("#pragma unroll\n        for (int t = 0; t < 4; ++t) { R%d[2 * t] = w[t] << 16; R%d[2 * t + 1] = w[t] & 0xffff0000u; } }\n", in.dst, in.dst);
          else
            o.f("#pragma unroll\n        for (int t = 0; t < 4; ++t) { R%d[2 * t] = __float_as_uint(h2f(w[t] & 0xffffu)); R%d[2 * t + 1] = "
                "__float_as_uint(h2f(w[t] >> 16)); } }\n", in.dst, in.dst);
        }
      } else {
        // A single view whose innermost extent is a multiple of 8: the thread's 8 elements share every outer
        // coordinate, so the chain runs once for idx0.  Innermost stride 1 (a row vector along the last dim, a
        // sliced or permuted outer dim): 8 consecutive source elements, one or two 16-byte loads when every outer
        // stride keeps them aligned.  Innermost stride 0 (a column vector or a scalar): one load, replicated.
        const PwView& vw = P.views[in.view0];
        const bool run8 = vec && in.nviews == 1 && vw.nd >= 1 && vw.fd[0].d % 8 == 0 && (vw.stride[0] == 1 || vw.stride[0] == 0);
        if (run8) {
          const uint32_t per16 = (in.dt == HE_F32 || in.dt == HE_U32) ? 4 : 8;
          bool aligned = vw.stride[0] == 1;
          for (int k = 1; k < vw.nd; ++k) aligned = aligned && vw.stride[k] % per16 == 0;
          o.f("      {\n");
          emit_views(o, P, in.view0, 1, "idx0", "v0");
          if (vw.stride[0] == 0) {
            o.f("        const u32 x = %s(p.in[%d], v0);\n#pragma unroll\n        for (int j = 0; j < 8; ++j) R%d[j] = x; }\n", elem_loader(in.dt),
                in.slot, in.dst);
          } else if (!aligned) {
            o.f("#pragma unroll\n        for (int j = 0; j < 8; ++j) R%d[j] = %s(p.in[%d], v0 + j); }\n", in.dst, elem_loader(in.dt), in.slot);
          } else if (per16 == 4) {
            o.f("        const uint4 a = __ldg((const uint4*)((const char*)p.in[%d] + (size_t)v0 * 4)), b = __ldg((const uint4*)((const char*)p.in[%d] + "
                "(size_t)v0 * 4) + 1);\n", in.slot, in.slot);
            o.f("        R%d[0] = a.x; R%d[1] = a.y; R%d[2] = a.z; R%d[3] = a.w; R%d[4] = b.x; R%d[5] = b.y; R%d[6] = b.z; R%d[7] = b.w; }\n",
                in.dst, in.dst, in.dst, in.dst, in.dst, in.dst, in.dst, in.dst);
          } else {
            o.f("        const uint4 a = __ldg((const uint4*)((const char*)p.in[%d] + (size_t)v0 * 2)); const u32 w[4] = {a.x, a.y, a.z, a.w};\n", in.slot);
            if (in.dt == HE_BF16)
              o.f("#pragma unroll\n        for (int t = 0; t < 4; ++t) { R%d[2 * t] = w[t] << 16; R%d[2 * t + 1] = w[t] & 0xffff0000u; } }\n", in.dst, in.dst);
            else
              o.f("#pragma unroll\n        for (int t = 0; t < 4; ++t) { R%d[2 * t] = __float_as_uint(h2f(w[t] & 0xffffu)); R%d[2 * t + 1] = "
                  "__float_as_uint(h2f(w[t] >> 16)); } }\n", in.dst, in.dst);
          }
        } else {
          o.f("      %s{\n", loop);
          emit_views(o, P, in.view0, in.nviews, "(idx0 + j)", "vi");
          o.f("      %s = %s(p.in[%d], vi); }\n", R.u(in.dst).c_str(), elem_loader(in.dt), in.slot);
        }
      }
      return true;
    }
    case PW_CONST:
      o.f("      %s%s = 0x%08xu;\n", loop, R.u(in.dst).c_str(), in.imm);
      return true;
    case PW_UNARY:
      if (!unary_expr(in.sub, R.fl(in.a), in.imm, &e)) { *why = "unknown unary op"; return false; }
      o.f("      %s%s = __float_as_uint(%s);\n", loop, R.u(in.dst).c_str(), e.c_str());
      return true;
    case PW_BIN_F:
      if (!bin_f_expr(in.sub, R.fl(in.a), R.fl(in.b), &e)) { *why = "unknown float binary op"; return false; }
      o.f("      %s%s = __float_as_uint(%s);\n", loop, R.u(in.dst).c_str(), e.c_str());
      return true;
    case PW_FMA:
      o.f("      %s%s = __float_as_uint(fmaf(%s, %s, %s));\n", loop, R.u(in.dst).c_str(), R.fl(in.a).c_str(), R.fl(in.b).c_str(),
          R.fl(in.c).c_str());
      return true;
    case PW_BIN_U:
    case PW_BIN_B:
      if (!bin_u_expr(in.sub, R.u(in.a), R.u(in.b), &e)) { *why = "unknown integer binary op"; return false; }
      o.f("      %s%s = %s%s;\n", loop, R.u(in.dst).c_str(), e.c_str(), in.op == PW_BIN_B ? " & 1u" : "");
      return true;
    case PW_CMP_F:
      o.f("      %s%s = (%s %s %s) ? 1u : 0u;\n", loop, R.u(in.dst).c_str(), R.fl(in.a).c_str(), cmp_token(in.sub), R.fl(in.b).c_str());
      return true;
    case PW_CMP_U:
      o.f("      %s%s = (%s %s %s) ? 1u : 0u;\n", loop, R.u(in.dst).c_str(), R.u(in.a).c_str(), cmp_token(in.sub), R.u(in.b).c_str());
      return true;
    case PW_SELECT:
      o.f("      %s%s = %s ? %s : %s;\n", loop, R.u(in.dst).c_str(), R.u(in.c).c_str(), R.u(in.b).c_str(), R.u(in.a).c_str());
      return true;
    case PW_CVT: {
      const std::string x = R.u(in.a), xf = R.fl(in.a);
      switch (in.sub) {
        case (0 << 2 | 2): e = "(" + xf + " != 0.0f ? 1u : 0u)"; break;
        case (2 << 2 | 0): e = "(" + x + " ? 0x3f800000u : 0u)"; break;
        case (0 << 2 | 1): e = "__float2uint_rz(" + xf + ")"; break;
        case (1 << 2 | 0): e = "__float_as_uint((float)" + x + ")"; break;
        case (2 << 2 | 1): e = "(" + x + " ? 1u : 0u)"; break;
        default: e = "(" + x + " != 0u ? 1u : 0u)"; break;
      }
      o.f("      %s%s = %s;\n", loop, R.u(in.dst).c_str(), e.c_str());
      return true;
    }
    case PW_MEAN_SCALE: {
      unsigned long long bits;
      memcpy(&bits, &P.mean_scale, 8);
      o.f("      %s%s = __float_as_uint((float)((double)%s * __longlong_as_double(0x%016llxll)));\n", loop, R.u(in.dst).c_str(),
          R.fl(in.a).c_str(), bits);
      return true;
    }
    case PW_STORE: {
      if (in.dt == HE_BOOL) { *why = "bit-packed bool store"; return false; }
      if (!vec) {
        if (in.dt == HE_F32 || in.dt == HE_U32) o.f("      ((u32*)p.out[%d])[idx0 + j] = r%d;\n", in.slot, in.a);
        else o.f("      ((unsigned short*)p.out[%d])[idx0 + j] = (unsigned short)%s(__uint_as_float(r%d));\n", in.slot,
                 in.dt == HE_BF16 ? "f2bf" : "f2h", in.a);
      } else if (in.dt == HE_F32 || in.dt == HE_U32) {
        o.f("      stv(p.out[%d], (size_t)idx0 * 4, make_uint4(R%d[0], R%d[1], R%d[2], R%d[3]));\n", in.slot, in.a, in.a, in.a, in.a);
        o.f("      stv(p.out[%d], (size_t)idx0 * 4 + 16, make_uint4(R%d[4], R%d[5], R%d[6], R%d[7]));\n", in.slot, in.a, in.a, in.a, in.a);
      } else {
        const char* cv = in.dt == HE_BF16 ? "f2bf" : "f2h";
        o.f("      { u32 w[4];\n#pragma unroll\n        for (int t = 0; t < 4; ++t) w[t] = %s(__uint_as_float(R%d[2 * t])) | (%s(__uint_as_float(R%d[2 * t + 1])) << 16);\n",
            cv, in.a, cv, in.a);
        o.f("        stv(p.out[%d], (size_t)idx0 * 2, make_uint4(w[0], w[1], w[2], w[3])); }\n", in.slot);
      }
      return true;
    }
    case PW_REDUCE:
      if (vec) { *why = "reduction in the vector body"; return false; }
      o.f("      red[%d] = red_combine(%d, red[%d], __uint_as_float(r%d));\n", in.slot2, in.sub, in.slot2, in.a);
      return true;
    case PW_ACC: *why = "matmul accumulator"; return false;
    default: *why = "unknown instruction"; return false;
  }
}


// The reduction kernel: pw_reduce_kernel of pointwise.cu with the interpreter call replaced by the printed program.
// Thread-to-element mapping, shuffle trees, shared-memory folds and partial layout are the same text, so the
// two kernels combine the same values in the same order (tests/test_pointwise_jit_gpu.py compares their bits).
const char* kReduceSkeleton = R"SRC(
struct RedL { u32 num_groups, blocks_per_group, chunk; int warp_mode; int red_ops[4]; int red_out_slot[4]; float* partials; };
extern "C" __global__ void __launch_bounds__(256) pw_jit(const JitParams p, const RedL L) {
  __shared__ float sred[4][8];
  float red[4];
#pragma unroll
  for (int s = 0; s < 4; ++s) red[s] = s < NRED ? red_identity(L.red_ops[s]) : 0.0f;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (L.warp_mode == 1) {
    const u32 group = blockIdx.x * 8 + warp;
    if (group >= L.num_groups) return;
    const u32 base = group * GS;
    const u32 iters = (GS + 31) / 32;
    for (u32 it = 0; it < iters; ++it) {
      const u32 e = it * 32 + lane;
      pw_elem(p, base + e, e < GS, red);
    }
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      if (s >= NRED) break;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) red[s] = red_combine(L.red_ops[s], red[s], __shfl_down_sync(0xffffffffu, red[s], off));
      if (lane == 0) ((float*)p.out[L.red_out_slot[s]])[group] = red[s];
    }
    return;
  }
  if (L.warp_mode == 2) {
    __shared__ float scol[4][8][32];
    const u32 gblocks = (L.num_groups + 31) / 32;
    const u32 blk = blockIdx.x / gblocks, gb = blockIdx.x - blk * gblocks;
    const u32 group = gb * 32 + lane;
    const bool gvalid = group < L.num_groups;
    const u32 start = blk * L.chunk, end = min(start + L.chunk, (u32)GS);
    const u32 base = gvalid ? group * GS : 0u;
#pragma unroll 4
    for (u32 e = start + warp; e < end; e += 8) pw_elem(p, base + e, gvalid, red);
#pragma unroll
    for (int s = 0; s < 4; ++s)
      if (s < NRED) scol[s][warp][lane] = red[s];
    __syncthreads();
    if (warp == 0 && gvalid) {
      for (int s = 0; s < NRED; ++s) {
        float v = scol[s][0][lane];
        for (int w = 1; w < 8; ++w) v = red_combine(L.red_ops[s], v, scol[s][w][lane]);
        if (L.blocks_per_group == 1) ((float*)p.out[L.red_out_slot[s]])[group] = v;
        else L.partials[((size_t)s * L.num_groups + group) * L.blocks_per_group + blk] = v;
      }
    }
    return;
  }
  const u32 group = blockIdx.x / L.blocks_per_group;
  const u32 blk = blockIdx.x - group * L.blocks_per_group;
  const u32 start = blk * L.chunk;
  const u32 end = min(start + L.chunk, (u32)GS);
  const u32 base = group * GS;
  const u32 iters = (end - start + 255) / 256;
#pragma unroll 4
  for (u32 it = 0; it < iters; ++it) {
    const u32 e = start + it * 256 + threadIdx.x;
    pw_elem(p, base + e, e < end, red);
  }
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    if (s >= NRED) break;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) red[s] = red_combine(L.red_ops[s], red[s], __shfl_down_sync(0xffffffffu, red[s], off));
    if (lane == 0) sred[s][warp] = red[s];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int s = 0; s < NRED; ++s) {
      float v = sred[s][0];
      for (int w = 1; w < 8; ++w) v = red_combine(L.red_ops[s], v, sred[s][w]);
      if (L.blocks_per_group == 1) ((float*)p.out[L.red_out_slot[s]])[group] = v;
      else L.partials[((size_t)s * L.num_groups + group) * L.blocks_per_group + blk] = v;
    }
  }
}
)SRC";

bool generate_reduce(const PwCompiled& c, std::string* source, std::string* why) {
  const PwProgram& P = c.prog;
  if (P.n_reductions > 4) { *why = "more than four reductions"; return false; }
  int n_regs = 0;
  for (int i = 0; i < P.n_instr; ++i) {
    const PwInstr& in = P.instr[i];
    if (in.op == PW_STORE) { *why = "a stored tensor beside the reductions"; return false; }
    if (in.op != PW_REDUCE) n_regs = std::max(n_regs, in.dst + 1);
  }
  Src o;
  o.s = kPrelude;
  o.f("#define NRED %d\n#define GS %uu\n", P.n_reductions, P.group_size);
  o.f("__device__ __forceinline__ float red_combine(int op, float a, float b) { return op == %d ? fmaxf(a, b) : op == %d ? fminf(a, b) : a + b; }\n",
      HE_RED_MAX, HE_RED_MIN);
  o.f("__device__ __forceinline__ float red_identity(int op) { return op == %d ? -__int_as_float(0x7f800000) : op == %d ? __int_as_float(0x7f800000) : 0.0f; }\n",
      HE_RED_MAX, HE_RED_MIN);
  o.f("__device__ __forceinline__ void pw_elem(const JitParams& p, u32 idx0, bool valid, float* red) {\n");
  o.f("  if (!valid) return;\n  const u32 j = 0;\n");
  for (int k = 0; k < n_regs; ++k) o.f("      u32 r%d;\n", k);
  for (int i = 0; i < P.n_instr; ++i)
    if (!emit_instr(o, P, P.instr[i], false, why)) return false;
  o.f("}\n");
  o.s += kReduceSkeleton;
  *source = std::move(o.s);
  return true;
}

}  // namespace

bool pw_jit_generate(const PwCompiled& c, std::string* source, std::string* why) {
  const PwProgram& P = c.prog;
  if (c.has_bool_io) { *why = "bit-packed bool tensors run on the interpreter"; return false; }
  if (P.n_elems == 0 || P.n_elems > 0x7fffff00u) { *why = "iteration space outside 1 .. 2^31"; return false; }
  if (P.n_reductions != 0) return generate_reduce(c, source, why);
  if (c.has_bool_io) { *why = "bit-packed bool tensors run on the interpreter"; return false; }
  if (P.n_elems == 0 || P.n_elems > 0x7fffff00u) { *why = "iteration space outside 1 .. 2^31"; return false; }
  int n_regs = 0;
  for (int i = 0; i < P.n_instr; ++i) {
    const PwInstr& in = P.instr[i];
    if (in.op != PW_STORE && in.op != PW_REDUCE) n_regs = std::max(n_regs, in.dst + 1);
  }
  Src o;
  o.s = kPrelude;
  o.f("extern \"C\" __global__ void __launch_bounds__(256) pw_jit(const JitParams p) {\n");
  o.f("  const u32 n = %uu, nv = %uu;\n", P.n_elems, (P.n_elems + 7) / 8);
  o.f("  for (u32 iv = blockIdx.x * 256u + threadIdx.x; iv < nv; iv += gridDim.x * 256u) {\n");
  o.f("    const u32 idx0 = iv * 8u;\n");
  o.f("    if (idx0 + 8u <= n) {\n");
  for (int k = 0; k < n_regs; ++k) o.f("      u32 R%d[8];\n", k);
  for (int i = 0; i < P.n_instr; ++i)
    if (!emit_instr(o, P, P.instr[i], true, why)) return false;
  o.f("    } else {\n");
  o.f("      for (u32 j = 0; idx0 + j < n; ++j) {\n");
  for (int k = 0; k < n_regs; ++k) o.f("      u32 r%d;\n", k);
  for (int i = 0; i < P.n_instr; ++i)
    if (!emit_instr(o, P, P.instr[i], false, why)) return false;
  o.f("      }\n    }\n  }\n}\n");
  *source = std::move(o.s);
  return true;
}

struct PwJitModule {
  std::vector<char> cubin;
  std::mutex mu;
  std::map<int, std::pair<cudaLibrary_t, cudaKernel_t>> loaded;   // per device
  ~PwJitModule() {
    for (auto& kv : loaded) cudaLibraryUnload(kv.second.first);
  }
};

int32_t pw_jit_compile(const PwCompiled& c, std::shared_ptr<PwJitModule>* out) {
  std::string src, why;
  if (!pw_jit_generate(c, &src, &why)) HE_FAIL(HE_ERR_UNSUPPORTED, "pointwise specialisation: %s", why.c_str());
  const Nvrtc& n = nvrtc();
  if (!n.handle) HE_FAIL(HE_ERR_UNSUPPORTED, "pointwise specialisation: %s", n.why.c_str());
  // process-wide cache by source text; deliberately never destroyed, so that no module is unloaded from a static
  // destructor after the CUDA runtime has shut down
  static std::mutex cache_mu;
  static auto& cache = *new std::map<std::string, std::shared_ptr<PwJitModule>>();
  {
    std::lock_guard<std::mutex> lk(cache_mu);
    auto it = cache.find(src);
    if (it != cache.end()) { *out = it->second; return HE_OK; }
  }
  nvrtcProgram prog = nullptr;
  if (n.CreateProgram(&prog, src.c_str(), "pw_jit.cu", 0, nullptr, nullptr) != 0)
    HE_FAIL(HE_ERR_CUDA, "pointwise specialisation: nvrtcCreateProgram failed");
  const char* opts[] = {"--gpu-architecture=sm_100a", "--std=c++17"};
  const int rc = n.CompileProgram(prog, 2, opts);
  if (rc != 0) {
    size_t ls = 0;
    n.GetProgramLogSize(prog, &ls);
    std::string log(ls ? ls : 1, '\0');
    if (ls) n.GetProgramLog(prog, &log[0]);
    n.DestroyProgram(&prog);
    HE_FAIL(HE_ERR_CUDA, "pointwise specialisation: NVRTC rejected the generated kernel (code %d): %.600s", rc, log.c_str());
  }
  auto m = std::make_shared<PwJitModule>();
  size_t sz = 0;
  if (n.GetCUBINSize(prog, &sz) != 0 || sz == 0) {
    n.DestroyProgram(&prog);
    HE_FAIL(HE_ERR_CUDA, "pointwise specialisation: NVRTC produced no device image");
  }
  m->cubin.resize(sz);
  n.GetCUBIN(prog, m->cubin.data());
  n.DestroyProgram(&prog);
  {
    std::lock_guard<std::mutex> lk(cache_mu);
    auto ins = cache.emplace(src, m);
    *out = ins.first->second;
  }
  return HE_OK;
}

bool pw_jit_pointers_ok(const PwCompiled& c, const PwProgram& P) {
  // identity-mapped tensors and the contiguous runs of viewed ones move as 16-byte vectors
  for (int i = 0; i < P.n_inputs; ++i)
    if (reinterpret_cast<uintptr_t>(P.in[i]) & 15) return false;
  for (int i = 0; i < P.n_outputs; ++i)
    if (reinterpret_cast<uintptr_t>(P.out[i]) & 15) return false;
  (void)c;
  return true;
}

namespace {
int32_t load_kernel(PwJitModule& m, cudaKernel_t* out) {
  int dev = 0;
  HE_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(m.mu);
  auto it = m.loaded.find(dev);
  if (it == m.loaded.end()) {
    cudaLibrary_t lib = nullptr;
    HE_CUDA(cudaLibraryLoadData(&lib, m.cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0));
    cudaKernel_t k = nullptr;
    cudaError_t e = cudaLibraryGetKernel(&k, lib, "pw_jit");
    if (e != cudaSuccess) {
      cudaLibraryUnload(lib);
      HE_FAIL(HE_ERR_CUDA, "pointwise specialisation: kernel not found in its image: %s", cudaGetErrorString(e));
    }
    it = m.loaded.emplace(dev, std::make_pair(lib, k)).first;
  }
  *out = it->second.second;
  return HE_OK;
}
}  // namespace

int32_t pw_jit_launch(PwJitModule& m, const PwProgram& P, int sm_count, cudaStream_t stream) {
  cudaKernel_t fn = nullptr;
  HE_TRY(load_kernel(m, &fn));
  struct { const void* in[16]; void* out[8]; } prm;
  static_assert(kPwMaxInputs == 16 && kPwMaxOutputs == 8, "JitParams layout of the generated kernel");
  for (int i = 0; i < kPwMaxInputs; ++i) prm.in[i] = P.in[i];
  for (int i = 0; i < kPwMaxOutputs; ++i) prm.out[i] = P.out[i];
  const unsigned long long nv = ((unsigned long long)P.n_elems + 7) / 8;
  const unsigned grid = (unsigned)std::max<unsigned long long>(1, std::min<unsigned long long>((nv + 255) / 256, (unsigned long long)sm_count * 16));
  void* args[] = {&prm};
  HE_CUDA(cudaLaunchKernel(reinterpret_cast<const void*>(fn), dim3(grid), dim3(256), args, 0, stream));
  return HE_OK;
}

int32_t pw_jit_launch_reduce(PwJitModule& m, const PwProgram& P, const PwReduceLaunch& L, unsigned grid, cudaStream_t stream) {
  cudaKernel_t fn = nullptr;
  HE_TRY(load_kernel(m, &fn));
  struct { const void* in[16]; void* out[8]; } prm;
  for (int i = 0; i < kPwMaxInputs; ++i) prm.in[i] = P.in[i];
  for (int i = 0; i < kPwMaxOutputs; ++i) prm.out[i] = P.out[i];
  PwReduceLaunch l = L;
  void* args[] = {&prm, &l};
  HE_CUDA(cudaLaunchKernel(reinterpret_cast<const void*>(fn), dim3(grid), dim3(256), args, 0, stream));
  return HE_OK;
}

}  // namespace he
