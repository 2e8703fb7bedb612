// Instantiations of the tcgen05 GEMM with the bias / residual / activation / gate epilogue.
#include "gemm_launch.cuh"

namespace he {

// ---- reduction finalisers (fixed summation order => bit-stable results) --------------------------
// out[b][n] = sum_{tm} partials[b][tm][n]
// op: 0 sum, 1 max, 2 min; the folded value is multiplied by `scale` (1 / count for a mean)
__device__ __forceinline__ float fold_op(int op, float a, float b) { return op == 1 ? fmaxf(a, b) : op == 2 ? fminf(a, b) : a + b; }
__global__ void gemm_colsum_finalize(const float* __restrict__ partials, float* __restrict__ out, int batch, int tiles_m, int N, int op,
                                     float scale) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= batch * N) return;
  const int b = i / N, n = i - b * N;
  const float* p = partials + (size_t)b * tiles_m * N + n;
  float s = p[0];
  for (int t = 1; t < tiles_m; ++t) s = fold_op(op, s, p[(size_t)t * N]);
  out[i] = s * scale;
}
// out[0] = sum_t partials[t], one CTA, tree in a fixed order
__global__ void gemm_scalar_finalize(const float* __restrict__ partials, float* __restrict__ out, int n, int op, float scale) {
  __shared__ float s[256];
  const float ident = op == 1 ? -INFINITY : op == 2 ? INFINITY : 0.0f;
  float v = ident;
  for (int i = threadIdx.x; i < n; i += 256) v = fold_op(op, v, partials[i]);
  s[threadIdx.x] = v;
  __syncthreads();
  for (int off = 128; off > 0; off >>= 1) {
    if ((int)threadIdx.x < off) s[threadIdx.x] = fold_op(op, s[threadIdx.x], s[threadIdx.x + off]);
    __syncthreads();
  }
  if (threadIdx.x == 0) out[0] = s[0] * scale;
}

// The three folds of the README graph in one launch: blocks [0, nb) fold the first column-sum
// partials, [nb, 2 nb) the second, the last block the scalar.  Same fixed orders as the kernels above.
__global__ void gemm_readme_finalize(const float* __restrict__ col_a, float* __restrict__ out_a, const float* __restrict__ col_b,
                                     float* __restrict__ out_b, int batch, int tiles_m, int N, const float* __restrict__ scal,
                                     float* __restrict__ out_scal, int n_scal) {
  const int nb = (batch * N + 255) / 256;
  if ((int)blockIdx.x < 2 * nb) {
    const bool second = (int)blockIdx.x >= nb;
    const int i = ((int)blockIdx.x - (second ? nb : 0)) * 256 + threadIdx.x;
    if (i >= batch * N) return;
    const int b = i / N, n = i - b * N;
    const float* p = (second ? col_b : col_a) + (size_t)b * tiles_m * N + n;
    float s = p[0];
    for (int t = 1; t < tiles_m; ++t) s += p[(size_t)t * N];
    (second ? out_b : out_a)[i] = s;
    return;
  }
  __shared__ float sh[256];
  float v = 0.0f;
  for (int i = threadIdx.x; i < n_scal; i += 256) v += scal[i];
  sh[threadIdx.x] = v;
  __syncthreads();
  for (int off = 128; off > 0; off >>= 1) {
    if ((int)threadIdx.x < off) sh[threadIdx.x] += sh[threadIdx.x + off];
    __syncthreads();
  }
  if (threadIdx.x == 0) out_scal[0] = sh[0];
}

int32_t launch_readme_finalize(const float* col_a, float* out_a, const float* col_b, float* out_b, int batch, int tiles_m, int N,
                               const float* scal, float* out_scal, int n_scal, cudaStream_t stream) {
  const int nb = (batch * N + 255) / 256;
  gemm_readme_finalize<<<2 * nb + 1, 256, 0, stream>>>(col_a, out_a, col_b, out_b, batch, tiles_m, N, scal, out_scal, n_scal);
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

int32_t launch_gemm_flex(const GemmLaunchCfg& cfg, const GemmParams<EpiFlexParams>& p, cudaStream_t stream) {
  if (cfg.two_cta && cfg.bn == 256) {
    if (cfg.ml == ML_NONE) return launch_majors_2cta<6, ML_NONE, 8, EpiFlex>(cfg, p, stream);
    if (cfg.ml == ML_F8 && !cfg.a_mn && !cfg.b_mn) return launch_one_2cta<6, false, false, ML_F8, 8, EpiFlex>(cfg, p, stream);
    if (cfg.ml == ML_RELU_MASK) return launch_majors_2cta<4, ML_RELU_MASK, 8, EpiFlex>(cfg, p, stream);
    if (cfg.ml == ML_GENERIC) return launch_majors_2cta<6, ML_GENERIC, 8, EpiFlex>(cfg, p, stream);
    if (cfg.ml == ML_GENERIC_MASK) return launch_majors_2cta<4, ML_GENERIC_MASK, 8, EpiFlex>(cfg, p, stream);
  }
  if (cfg.bn == 256) {
    if (cfg.ml == ML_NONE) return launch_majors<256, 4, ML_NONE, 8, EpiFlex>(cfg, p, stream);
    if (cfg.ml == ML_F8 && !cfg.a_mn && !cfg.b_mn) return launch_one<256, 4, false, false, ML_F8, 8, EpiFlex>(cfg, p, stream);
    if (cfg.ml == ML_RELU_MASK) return launch_majors<256, 3, ML_RELU_MASK, 8, EpiFlex>(cfg, p, stream);
    if (cfg.ml == ML_GENERIC) return launch_majors<256, 4, ML_GENERIC, 8, EpiFlex>(cfg, p, stream);
    if (cfg.ml == ML_GENERIC_MASK) return launch_majors<256, 3, ML_GENERIC_MASK, 8, EpiFlex>(cfg, p, stream);
  } else if (cfg.bn == 128) {
    if (cfg.ml == ML_NONE) return launch_majors<128, 6, ML_NONE, 4, EpiFlex>(cfg, p, stream);
  }
  HE_FAIL(HE_ERR_UNSUPPORTED, "fused matmul: no kernel compiled for bn=%d mainloop=%d with this epilogue", cfg.bn, cfg.ml);
}

int32_t launch_colsum_finalize(const float* partials, float* out, int batch, int tiles_m, int N, cudaStream_t stream, int op, float scale) {
  const int n = batch * N;
  gemm_colsum_finalize<<<(n + 255) / 256, 256, 0, stream>>>(partials, out, batch, tiles_m, N, op, scale);
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

int32_t launch_scalar_finalize(const float* partials, float* out, int n, cudaStream_t stream, int op, float scale) {
  gemm_scalar_finalize<<<1, 256, 0, stream>>>(partials, out, n, op, scale);
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

}  // namespace he
