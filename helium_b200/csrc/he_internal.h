// Internal declarations shared by the translation units of libhelium_b200.so.
#pragma once
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "helium_b200.h"

namespace he {

// ---- errors -----------------------------------------------------------------------------------
void set_error(const char* fmt, ...);
#define HE_FAIL(code, ...)        \
  do {                            \
    ::he::set_error(__VA_ARGS__); \
    return (code);                \
  } while (0)
#define HE_CUDA(expr)                                                                     \
  do {                                                                                    \
    cudaError_t e__ = (expr);                                                             \
    if (e__ != cudaSuccess)                                                               \
      HE_FAIL(HE_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, \
              __LINE__);                                                                  \
  } while (0)
#define HE_TRY(expr)           \
  do {                         \
    int32_t s__ = (expr);      \
    if (s__ != HE_OK) return s__; \
  } while (0)

// ---- dtype helpers ----------------------------------------------------------------------------
enum class DClass { Float, Int, Bool };
inline DClass dclass(int32_t dt) {
  return dt == HE_U32 ? DClass::Int : dt == HE_BOOL ? DClass::Bool : DClass::Float;
}
inline int dtype_bytes(int32_t dt) {  // bytes per element; 0 for bit-packed bool
  switch (dt) {
    case HE_F16: case HE_BF16: return 2;
    case HE_F32: case HE_U32: return 4;
    default: return 0;
  }
}
inline bool dtype_valid(int32_t dt) { return dt >= HE_F16 && dt <= HE_BOOL; }
const char* dtype_name(int32_t dt);

inline int64_t num_elements(const he_node& n) {
  int64_t c = 1;
  for (int i = 0; i < n.rank; ++i) c *= n.shape[i];
  return c;
}
inline size_t storage_bytes(int32_t dt, int64_t elems) {
  if (dt == HE_BOOL) return size_t((elems + 31) / 32) * 4;
  return size_t(elems) * dtype_bytes(dt);
}

// ---- device status block ----------------------------------------------------------------------
// Word 0: 0 = fine, otherwise (site << 16 | detail) of the first bounded wait that gave up.
struct DeviceStatus {
  unsigned int code;
  unsigned int block;
  unsigned int aux0;
  unsigned int aux1;
};

}  // namespace he

struct he_ctx {
  int device = 0;
  int sm_count = 0;
  int sm_reserved = 0;   // he_ctx_reserve_sms: SMs that plans created from now on leave to other work
  int max_smem_optin = 0;
  he::DeviceStatus* d_status = nullptr;  // device memory
};

// A plan may be created with a null context ("planning only": tier, tile shape and workspace can
// be inspected, launching is refused); such plans assume the SM count of a B200.
inline int ctx_sm_count(const he_ctx* c) { return c ? (c->sm_count - c->sm_reserved > 2 ? c->sm_count - c->sm_reserved : 2) : 148; }

// Base of every plan.  Immutable after creation except for the launch counter.
struct he_plan {
  he_ctx* ctx = nullptr;
  size_t workspace_bytes = 0;
  int last_launches = 0;
  std::string description;
  virtual ~he_plan() {}
  virtual int32_t launch(const void* const* inputs, void* const* outputs, void* workspace,
                         cudaStream_t stream) = 0;
  // he_debug_plan_fault_injection: only plans whose kernels contain bounded waits implement it
  virtual int32_t set_fault_injection(uint32_t /*wait_limit_us*/, int32_t /*withhold_loads*/) {
    he::set_error("this plan's kernels have no device-side waits to bound");
    return HE_ERR_UNSUPPORTED;
  }
};

namespace he {

// Makes `device` current for a scope and restores the caller's device afterwards, so that a host
// thread driving several GPUs does not find its current device changed by a library call.
class DeviceGuard {
 public:
  explicit DeviceGuard(int device) {
    if (cudaGetDevice(&prev_) != cudaSuccess) { prev_ = -1; failed_ = true; return; }
    if (prev_ != device) {
      if (cudaSetDevice(device) != cudaSuccess) failed_ = true;
      else switched_ = true;
    }
  }
  ~DeviceGuard() {
    if (switched_) cudaSetDevice(prev_);
  }
  int32_t status() const {
    if (!failed_) return HE_OK;
    set_error("could not make the plan's device current: %s", cudaGetErrorString(cudaGetLastError()));
    return HE_ERR_CUDA;
  }
 private:
  int prev_ = -1;
  bool switched_ = false, failed_ = false;
};

// NVTX range for the scope of a library call (visible in Nsight Systems / Compute timelines; the reference marks
// its planner, executor and instruction scopes with `#[profiling::function]`, helium/src/cuda.rs:178,190,225).
// The header-only NVTX v3 costs one indirect call when no tool is attached; HE_NVTX=0 removes even that.
class TraceRange {
 public:
  explicit TraceRange(const char* name);
  ~TraceRange();
 private:
  bool on_;
};

// ---- validated subgraph -----------------------------------------------------------------------
struct Graph {
  std::vector<he_node> nodes;
  std::vector<int> inputs;   // node indices of HE_OP_INPUT, in order
  std::vector<int> outputs;  // leaf node indices, in caller order
};
// Copies and validates a descriptor (operand indices, shapes, dtypes of every op).
int32_t parse_graph(const he_graph_desc* desc, Graph* out);

// planners (one per translation unit)
int32_t plan_pointwise(he_ctx* ctx, const Graph& g, he_plan** out, int* tier_only);
int32_t plan_permute(he_ctx* ctx, int rank, const int64_t* in_shape, const int64_t* out_strides,
                     int32_t dtype, he_plan** out);
int32_t plan_fused_matmul(he_ctx* ctx, const Graph& g, he_plan** out, int* tier_only);

}  // namespace he
