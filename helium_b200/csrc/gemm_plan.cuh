// Host-side interface between the fused-matmul planner and the kernel instantiations.
#pragma once
#include "gemm_sm100.cuh"

namespace he {

struct GemmLaunchCfg {
  int bn;        // 256 or 128
  bool a_mn;     // A operand is M-major in global memory ([K, M] row-major)
  bool b_mn;     // B operand is N-major in global memory ([K, N] row-major, the helium layout)
  int ml;        // MainloopKind
  int grid;      // CTAs
  bool two_cta;  // cluster-of-2 kernel (256 x 256 pair tiles); grid is then even
};

// One function per epilogue family; each switches over the instantiated (bn, majors, ml) set and
// returns HE_ERR_UNSUPPORTED for combinations that were not compiled in.
int32_t launch_gemm_flex(const GemmLaunchCfg& cfg, const GemmParams<EpiFlexParams>& p, cudaStream_t stream);
int32_t launch_gemm_c3(const GemmLaunchCfg& cfg, const GemmParams<EpiC3Params>& p, cudaStream_t stream);
int32_t launch_gemm_program(const GemmLaunchCfg& cfg, const GemmParams<EpiProgramParams>& p, cudaStream_t stream);
int32_t launch_colsum_finalize(const float* partials, float* out, int batch, int tiles_m, int N, cudaStream_t stream, int op = 0,
                               float scale = 1.0f);
int32_t launch_readme_finalize(const float* col_a, float* out_a, const float* col_b, float* out_b, int batch, int tiles_m, int N,
                               const float* scal, float* out_scal, int n_scal, cudaStream_t stream);
int32_t launch_scalar_finalize(const float* partials, float* out, int n, cudaStream_t stream, int op = 0, float scale = 1.0f);
// SIMT matmul: f32 operands, or 2-byte operands whose shapes break the TMA alignment rules
// `axpy`: optional epilogue out = [resid +] [-] (acc * (mul ? mul[i] : alpha)); resid and mul have the
// output's shape, every step rounds separately like the unfused graph
struct SgemmAxpy {
  int enabled = 0;
  const void* resid = nullptr;
  const void* mul = nullptr;
  int resid_dt = HE_F32, mul_dt = HE_F32;
  float alpha = 1.0f;
  int negate = 0;
};
int32_t launch_sgemm(const void* a, const void* b, void* c, int in_dt, int out_dt, int batch, int M, int N, int K,
                     bool a_mn, bool b_mn, const void* bias, int bias_dt, int act, const SgemmAxpy& axpy, cudaStream_t stream);

}  // namespace he
