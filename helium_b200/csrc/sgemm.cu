// SIMT matmul: f32 operands (MulF32AccumF32 / MulTf32AccumF32 requests) and 2-byte operands whose
// shapes break the 16-byte TMA rules of the tensor-core path (odd K or N, tiny matrices).
//
// The reference sends f32 matmuls to cuDNN with a TF32 request (helium/src/modules/linear.rs:45-50,
// helium/src/cuda/instr/cudnn_graph.rs:182-192) and documents the precision as a minimum
// (helium-ir/src/opgraph/op/precision.rs:3-9).  The f32 configurations here are small
// (256 x 784 x 512) and need f32-accurate products, so they run on FFMA with 64x64 tiles:
// 256 threads, a 4x4 micro-tile per thread, 16-deep K slices staged through shared memory.
#include "gemm_plan.cuh"

namespace he {

struct SgemmParams {
  const void* a; const void* b; void* c; const void* bias;
  int in_dt, out_dt, bias_dt;
  int M, N, K, batch;
  long long sam, sak, sbk, sbn;  // element strides of A(m, k) and B(k, n)
  int act;
};

__device__ __forceinline__ float sg_load(const void* base, int dt, long long idx) {
  if (dt == HE_F32) return __ldg(reinterpret_cast<const float*>(base) + idx);
  const uint32_t h = __ldg(reinterpret_cast<const unsigned short*>(base) + idx);
  return dt == HE_BF16 ? bf16_bits_to_f32(h) : f16_bits_to_f32(h);
}

__global__ void __launch_bounds__(256) sgemm_64x64_kernel(const __grid_constant__ SgemmParams p) {
  __shared__ float As[16][64 + 4];
  __shared__ float Bs[16][64 + 4];
  const int bz = blockIdx.z;
  const long long a_off = (long long)bz * p.M * p.K, b_off = (long long)bz * p.K * p.N;
  const size_t c_off = (size_t)bz * p.M * p.N;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < p.K; k0 += 16) {
    // 64 x 16 elements of A and 16 x 64 of B: 4 loads each per thread, indices chosen so that the
    // unit-stride global direction is walked by consecutive threads
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = threadIdx.x + i * 256;
      int m, k;
      if (p.sak == 1) { k = e & 15; m = e >> 4; } else { m = e & 63; k = e >> 6; }
      const int gm = m0 + m, gk = k0 + k;
      As[k][m] = (gm < p.M && gk < p.K) ? sg_load(p.a, p.in_dt, a_off + gm * p.sam + gk * p.sak) : 0.0f;
      int n, kk;
      if (p.sbn == 1) { n = e & 63; kk = e >> 6; } else { kk = e & 15; n = e >> 4; }
      const int gn = n0 + n, gk2 = k0 + kk;
      Bs[kk][n] = (gn < p.N && gk2 < p.K) ? sg_load(p.b, p.in_dt, b_off + gk2 * p.sbk + gn * p.sbn) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= p.N) continue;
      float v = acc[i][j];
      if (p.bias) v += sg_load(p.bias, p.bias_dt, gn);
      if (p.act == 1) v = fmaxf(v, 0.0f);
      const size_t o = c_off + (size_t)gm * p.N + gn;
      if (p.out_dt == HE_F32) reinterpret_cast<float*>(p.c)[o] = v;
      else reinterpret_cast<unsigned short*>(p.c)[o] = (unsigned short)(p.out_dt == HE_BF16 ? f32_to_bf16_bits(v) : f32_to_f16_bits(v));
    }
  }
}

int32_t launch_sgemm(const void* a, const void* b, void* c, int in_dt, int out_dt, int batch, int M, int N, int K,
                     bool a_mn, bool b_mn, const void* bias, int bias_dt, int act, cudaStream_t stream) {
  SgemmParams p{};
  p.a = a; p.b = b; p.c = c; p.bias = bias;
  p.in_dt = in_dt; p.out_dt = out_dt; p.bias_dt = bias_dt;
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  // a_mn: A stored [K, M]; b_mn: B stored [K, N] (the helium layout), else [N, K]
  p.sam = a_mn ? 1 : K; p.sak = a_mn ? M : 1;
  p.sbk = b_mn ? N : 1; p.sbn = b_mn ? 1 : K;
  p.act = act;
  dim3 grid((N + 63) / 64, (M + 63) / 64, batch);
  if (grid.y > 65535 || grid.z > 65535) HE_FAIL(HE_ERR_UNSUPPORTED, "sgemm: shape too large for the SIMT path");
  sgemm_64x64_kernel<<<grid, 256, 0, stream>>>(p);
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

}  // namespace he
