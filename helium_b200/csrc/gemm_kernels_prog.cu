// Instantiations of the tcgen05 GEMM with the generic (interpreted) epilogue tier.
#include "gemm_launch.cuh"

namespace he {

int32_t launch_gemm_program(const GemmLaunchCfg& cfg, const GemmParams<EpiProgramParams>& p, cudaStream_t stream) {
  if (cfg.two_cta && cfg.bn == 256) {
    if (cfg.ml == ML_NONE) return launch_majors_2cta<6, ML_NONE, 8, EpiProgram>(cfg, p, stream);
    if (cfg.ml == ML_F8 && !cfg.a_mn && !cfg.b_mn) return launch_one_2cta<6, false, false, ML_F8, 8, EpiProgram>(cfg, p, stream);
    if (cfg.ml == ML_RELU_MASK) return launch_majors_2cta<4, ML_RELU_MASK, 8, EpiProgram>(cfg, p, stream);
    if (cfg.ml == ML_GENERIC) return launch_majors_2cta<6, ML_GENERIC, 8, EpiProgram>(cfg, p, stream);
    if (cfg.ml == ML_GENERIC_MASK) return launch_majors_2cta<4, ML_GENERIC_MASK, 8, EpiProgram>(cfg, p, stream);
  }
  if (cfg.bn == 256) {
    if (cfg.ml == ML_NONE) return launch_majors<256, 4, ML_NONE, 8, EpiProgram>(cfg, p, stream);
    if (cfg.ml == ML_F8 && !cfg.a_mn && !cfg.b_mn) return launch_one<256, 4, false, false, ML_F8, 8, EpiProgram>(cfg, p, stream);
    if (cfg.ml == ML_RELU_MASK) return launch_majors<256, 3, ML_RELU_MASK, 8, EpiProgram>(cfg, p, stream);
    if (cfg.ml == ML_GENERIC) return launch_majors<256, 4, ML_GENERIC, 8, EpiProgram>(cfg, p, stream);
    if (cfg.ml == ML_GENERIC_MASK) return launch_majors<256, 3, ML_GENERIC_MASK, 8, EpiProgram>(cfg, p, stream);
  }
  HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: no kernel compiled for bn=%d mainloop=%d with this epilogue", cfg.bn, cfg.ml);
}

}  // namespace he
