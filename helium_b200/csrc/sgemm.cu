// SIMT matmul: f32 operands (MulF32AccumF32 / MulTf32AccumF32 requests) and 2-byte operands whose
// shapes break the 16-byte TMA rules of the tensor-core path (odd K or N, tiny matrices).
//
// The reference sends f32 matmuls to cuDNN with a TF32 request (helium/src/modules/linear.rs:45-50,
// helium/src/cuda/instr/cudnn_graph.rs:182-192) and documents the precision as a minimum
// (helium-ir/src/opgraph/op/precision.rs:3-9).  The f32 configurations here are small
// (256 x 784 x 512) and need f32-accurate products, so they run on FFMA with 64x64 tiles:
// 256 threads, a 4x4 micro-tile per thread, 32-deep K slices staged through shared memory with the
// next slice prefetched into registers.
//
// Such shapes give 4-100 output tiles for 148 SMs and a long, latency-bound K loop, so K is split
// over a thread-block cluster of up to 8 CTAs: every CTA of a cluster accumulates the same output
// tile over its own K range, parks the partial tile in its shared memory, and after a cluster
// barrier each CTA sums one band of rows over all partials through distributed shared memory, in
// rank order (deterministic), applies the epilogue and stores.  One launch, no workspace.
#include <cooperative_groups.h>

#include "gemm_plan.cuh"

namespace he {

struct SgemmParams {
  const void* a; const void* b; void* c; const void* bias;
  // scale / accumulate epilogue (the SGD update of a weight gradient, w + (-(g * lr))):
  // out = [resid +] [-] (acc * (mul ? mul[i] : alpha)), resid and mul of the output's shape
  const void* resid; const void* mul;
  float alpha; int axpy, alpha_neg;
  int in_dt, out_dt, bias_dt, resid_dt, mul_dt;
  int M, N, K, batch;
  long long sam, sak, sbk, sbn;  // element strides of A(m, k) and B(k, n)
  int act;
  int split, k_chunk;            // CTAs per cluster along K (1, 2, 4 or 8) and the K range of each
};

__device__ __forceinline__ float sg_load(const void* base, int dt, long long idx) {
  if (dt == HE_F32) return __ldg(reinterpret_cast<const float*>(base) + idx);
  const uint32_t h = __ldg(reinterpret_cast<const unsigned short*>(base) + idx);
  return dt == HE_BF16 ? bf16_bits_to_f32(h) : f16_bits_to_f32(h);
}

constexpr int kSgBK = 32;
constexpr int kSgPitch = 64 + 4;

__device__ __forceinline__ void sg_store(const SgemmParams& p, size_t o, int gn, float v) {
  if (p.bias) v += sg_load(p.bias, p.bias_dt, gn);
  if (p.axpy) {
    // separately rounded product and sum, like the unfused graph
    float s = __fmul_rn(v, p.mul ? sg_load(p.mul, p.mul_dt, (long long)o) : p.alpha);
    if (p.alpha_neg) s = -s;
    v = p.resid ? __fadd_rn(sg_load(p.resid, p.resid_dt, (long long)o), s) : s;
  }
  if (p.act == 1) v = fmaxf(v, 0.0f);
  if (p.out_dt == HE_F32) reinterpret_cast<float*>(p.c)[o] = v;
  else reinterpret_cast<unsigned short*>(p.c)[o] = (unsigned short)(p.out_dt == HE_BF16 ? f32_to_bf16_bits(v) : f32_to_f16_bits(v));
}

__global__ void __launch_bounds__(256) sgemm_64x64_kernel(const __grid_constant__ SgemmParams p) {
  // K slices of A and B; after the K loop the same memory holds this CTA's 64x64 partial tile
  __shared__ __align__(16) float smem[2 * kSgBK * kSgPitch];
  float (*As)[kSgPitch] = reinterpret_cast<float (*)[kSgPitch]>(smem);
  float (*Bs)[kSgPitch] = reinterpret_cast<float (*)[kSgPitch]>(smem + kSgBK * kSgPitch);
  const int bz = blockIdx.z / p.split, ks = blockIdx.z - bz * p.split;
  const long long a_off = (long long)bz * p.M * p.K, b_off = (long long)bz * p.K * p.N;
  const size_t c_off = (size_t)bz * p.M * p.N;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int k_begin = ks * p.k_chunk, k_end = min(p.K, k_begin + p.k_chunk);
  float acc[4][4] = {};
  float ra[8], rb[8];
  // 64 x 32 elements of A and 32 x 64 of B per slice: 8 loads each per thread, indices chosen so
  // that the unit-stride global direction is walked by consecutive threads
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = threadIdx.x + i * 256;
      int m, k;
      if (p.sak == 1) { k = e & 31; m = e >> 5; } else { m = e & 63; k = e >> 6; }
      const int gm = m0 + m, gk = k0 + k;
      ra[i] = (gm < p.M && gk < k_end) ? sg_load(p.a, p.in_dt, a_off + gm * p.sam + gk * p.sak) : 0.0f;
      int n, kk;
      if (p.sbn == 1) { n = e & 63; kk = e >> 6; } else { kk = e & 31; n = e >> 5; }
      const int gn = n0 + n, gk2 = k0 + kk;
      rb[i] = (gn < p.N && gk2 < k_end) ? sg_load(p.b, p.in_dt, b_off + gk2 * p.sbk + gn * p.sbn) : 0.0f;
    }
  };
  auto park = [&]() {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = threadIdx.x + i * 256;
      if (p.sak == 1) As[e & 31][e >> 5] = ra[i]; else As[e >> 6][e & 63] = ra[i];
      if (p.sbn == 1) Bs[e >> 6][e & 63] = rb[i]; else Bs[e & 31][e >> 5] = rb[i];
    }
  };
  if (k_begin < k_end) fetch(k_begin);
  for (int k0 = k_begin; k0 < k_end; k0 += kSgBK) {
    park();
    __syncthreads();
    if (k0 + kSgBK < k_end) fetch(k0 + kSgBK);
#pragma unroll
    for (int k = 0; k < kSgBK; ++k) {
      const float4 a4 = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 b4 = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
      const float a[4] = {a4.x, a4.y, a4.z, a4.w}, b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  if (p.split == 1) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int gm = m0 + ty * 4 + i;
      if (gm >= p.M) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int gn = n0 + tx * 4 + j;
        if (gn < p.N) sg_store(p, c_off + (size_t)gm * p.N + gn, gn, acc[i][j]);
      }
    }
    return;
  }
  // split K: park the partial tile, then this CTA finishes rows [ks * band, (ks + 1) * band)
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
#pragma unroll
  for (int i = 0; i < 4; ++i)
    *reinterpret_cast<float4*>(&smem[(ty * 4 + i) * 64 + tx * 4]) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
  cluster.sync();
  const int band = 64 / p.split;
  for (int e = threadIdx.x; e < band * 64; e += 256) {
    const int r = ks * band + (e >> 6), cidx = e & 63;
    float v = 0.0f;
    for (int q = 0; q < p.split; ++q) v += cluster.map_shared_rank(smem, q)[r * 64 + cidx];
    const int gm = m0 + r, gn = n0 + cidx;
    if (gm < p.M && gn < p.N) sg_store(p, c_off + (size_t)gm * p.N + gn, gn, v);
  }
  cluster.sync();   // nobody leaves while a peer may still read its partial tile
}

int32_t launch_sgemm(const void* a, const void* b, void* c, int in_dt, int out_dt, int batch, int M, int N, int K,
                     bool a_mn, bool b_mn, const void* bias, int bias_dt, int act, const SgemmAxpy& axpy, cudaStream_t stream) {
  SgemmParams p{};
  p.a = a; p.b = b; p.c = c; p.bias = bias;
  p.axpy = axpy.enabled; p.resid = axpy.resid; p.resid_dt = axpy.resid_dt; p.mul = axpy.mul; p.mul_dt = axpy.mul_dt;
  p.alpha = axpy.alpha; p.alpha_neg = axpy.negate;
  p.in_dt = in_dt; p.out_dt = out_dt; p.bias_dt = bias_dt;
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  // a_mn: A stored [K, M]; b_mn: B stored [K, N] (the helium layout), else [N, K]
  p.sam = a_mn ? 1 : K; p.sak = a_mn ? M : 1;
  p.sbk = b_mn ? N : 1; p.sbn = b_mn ? 1 : K;
  p.act = act;
  dim3 grid((N + 63) / 64, (M + 63) / 64, batch);
  if (grid.y > 65535) HE_FAIL(HE_ERR_UNSUPPORTED, "sgemm: shape too large for the SIMT path");
  // enough CTAs for about two waves of a 148-SM part, at least one 32-deep slice each
  const long long tiles = (long long)grid.x * grid.y * batch;
  int split = 1;
  while (split < 8 && tiles * (split * 2) <= 296 && K / (split * 2) >= kSgBK) split *= 2;
  p.split = split;
  p.k_chunk = ((K + split - 1) / split + kSgBK - 1) / kSgBK * kSgBK;
  grid.z = batch * split;
  if (grid.z > 65535) HE_FAIL(HE_ERR_UNSUPPORTED, "sgemm: shape too large for the SIMT path");
  if (split == 1) {
    sgemm_64x64_kernel<<<grid, 256, 0, stream>>>(p);
  } else {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = 0; cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 1; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = split;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    HE_CUDA(cudaLaunchKernelEx(&cfg, sgemm_64x64_kernel, p));
  }
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

}  // namespace he
