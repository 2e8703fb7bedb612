// Shared launcher template for the kernel instantiation files.
#pragma once
#include "gemm_plan.cuh"
#include "gemm_sm100_2cta.cuh"

#include <algorithm>

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
  constexpr int threads = 32 * (2 + NE_WARPS + (ml_transforms(ML) ? 4 : 0));
  kernel<<<cfg.grid, threads, SM::dynamic_bytes, stream>>>(p);
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

// Two-CTA (cluster of 2) variant; cfg.grid counts CTAs and is even.
template <int STAGES, bool A_MN, bool B_MN, int ML, int NE_WARPS, class Epi>
int32_t launch_one_2cta(const GemmLaunchCfg& cfg, const GemmParams<typename Epi::Params>& p, cudaStream_t stream) {
  using SM = GemmSmem2<STAGES, ML, Epi::kColReductions>;
  auto kernel = gemm_tcgen05_2cta_kernel<STAGES, A_MN, B_MN, ML, NE_WARPS, Epi>;
  static_assert(SM::dynamic_bytes <= 232448, "shared memory budget of sm_100 exceeded");
  constexpr int threads = 32 * (2 + NE_WARPS + (ml_transforms(ML) ? 4 : 0));
  static int max_pairs = 0;  // benign race: idempotent
  if (max_pairs == 0) {
    HE_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::dynamic_bytes));
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(2 * 74, 1, 1);
    lc.blockDim = dim3(threads, 1, 1);
    lc.dynamicSmemBytes = SM::dynamic_bytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    lc.attrs = &attr;
    lc.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &lc) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = 64;  // conservative: every cluster still gets scheduled, only later
    }
    max_pairs = n;
  }
  const int pairs = std::max(1, std::min(cfg.grid / 2, max_pairs));
  kernel<<<2 * pairs, threads, SM::dynamic_bytes, stream>>>(p);
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

template <int STAGES, int ML, int NE_WARPS, class Epi>
int32_t launch_majors_2cta(const GemmLaunchCfg& cfg, const GemmParams<typename Epi::Params>& p, cudaStream_t stream) {
  if (!cfg.a_mn && cfg.b_mn) return launch_one_2cta<STAGES, false, true, ML, NE_WARPS, Epi>(cfg, p, stream);
  if (!cfg.a_mn && !cfg.b_mn) return launch_one_2cta<STAGES, false, false, ML, NE_WARPS, Epi>(cfg, p, stream);
  if (cfg.a_mn && cfg.b_mn) return launch_one_2cta<STAGES, true, true, ML, NE_WARPS, Epi>(cfg, p, stream);
  return launch_one_2cta<STAGES, true, false, ML, NE_WARPS, Epi>(cfg, p, stream);
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
