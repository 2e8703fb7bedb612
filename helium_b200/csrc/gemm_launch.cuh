// Shared launcher template for the kernel instantiation files.
#pragma once
#include "gemm_plan.cuh"

namespace he {

template <int BN, int STAGES, bool A_MN, bool B_MN, int ML, int NE_WARPS, class Epi>
int32_t launch_one(const GemmLaunchCfg& cfg, const GemmParams<typename Epi::Params>& p, cudaStream_t stream) {
  using SM = GemmSmem<BN, STAGES, ML, Epi::kColReductions>;
  auto kernel = gemm_tcgen05_kernel<BN, STAGES, A_MN, B_MN, ML, NE_WARPS, Epi>;
  static_assert(SM::dynamic_bytes <= 232448, "shared memory budget of sm_100 exceeded");
  static bool configured = false;  // benign race: the attribute call is idempotent
  if (!configured) {
    HE_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::dynamic_bytes));
    configured = true;
  }
  constexpr int threads = 32 * (2 + NE_WARPS + (ML != ML_NONE ? 4 : 0));
  kernel<<<cfg.grid, threads, SM::dynamic_bytes, stream>>>(p);
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

// Dispatch over operand majors for one (BN, STAGES, ML) choice.
template <int BN, int STAGES, int ML, int NE_WARPS, class Epi>
int32_t launch_majors(const GemmLaunchCfg& cfg, const GemmParams<typename Epi::Params>& p, cudaStream_t stream) {
  if (!cfg.a_mn && cfg.b_mn) return launch_one<BN, STAGES, false, true, ML, NE_WARPS, Epi>(cfg, p, stream);
  if (!cfg.a_mn && !cfg.b_mn) return launch_one<BN, STAGES, false, false, ML, NE_WARPS, Epi>(cfg, p, stream);
  if (cfg.a_mn && cfg.b_mn) return launch_one<BN, STAGES, true, true, ML, NE_WARPS, Epi>(cfg, p, stream);
  return launch_one<BN, STAGES, true, false, ML, NE_WARPS, Epi>(cfg, p, stream);
}

}  // namespace he
