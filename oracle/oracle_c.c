/*
 * CPU restatement (C + OpenMP) of the timed parts of the hot path.  TEST AND CPU-BASELINE INFRASTRUCTURE
 * ONLY: used by tests/ as a second opinion next to oracle/oracle.py and by bench.py's cpu_baseline
 * and `--impl reference` legs.  The product library never links or calls it.
 *
 * The reference has no CPU implementation of these paths (every Device::Cpu arm is todo!(),
 * helium/src/raw_tensor.rs:100,156,1073), so this file follows the semantics of its CUDA kernels:
 *   oc_permute                  helium/src/cuda/instr/permute_dims/jit.rs:15-117
 *   oc_affine_relu_nchw_nhwc    helium/src/cuda/instr/pointwise/jit.rs:300-340,532-561 fused with the
 *                               swap_dims chain of permute_dims.rs:112-172 (the bf16 [64,256,56,56] benchmark case)
 *   oc_gemm_bf16                helium-ir/src/opgraph/op.rs:272-282 (row-major [M,K] x [K,N], bf16
 *                               products, f32 accumulation) with the relu(A) * mask mainloop fusion of
 *                               README.md:36-39
 *   oc_c3_epilogue              README.md:40-79 (the fused epilogue graph)
 * Parity pin: checked against oracle/oracle.py, which is pinned on the reference's own test vectors.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fc0;
  return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}

int oc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* out[sum_i out_strides[i] * c_i] = in[c] for every coordinate c of the row-major input. */
void oc_permute(const void* in, void* out, int elem_bytes, int rank, const int64_t* shape, const int64_t* out_strides) {
  int64_t total = 1, inner = shape[rank - 1], outer;
  for (int i = 0; i < rank; ++i) total *= shape[i];
  if (total == 0) return;
  outer = total / inner;
  const int64_t inner_stride = out_strides[rank - 1];
#pragma omp parallel for schedule(static)
  for (int64_t o = 0; o < outer; ++o) {
    int64_t rem = o, base = 0;
    for (int d = rank - 2; d >= 0; --d) {
      base += (rem % shape[d]) * out_strides[d];
      rem /= shape[d];
    }
    if (elem_bytes == 4) {
      const uint32_t* src = (const uint32_t*)in + o * inner;
      uint32_t* dst = (uint32_t*)out + base;
      for (int64_t x = 0; x < inner; ++x) dst[x * inner_stride] = src[x];
    } else {
      const uint16_t* src = (const uint16_t*)in + o * inner;
      uint16_t* dst = (uint16_t*)out + base;
      for (int64_t x = 0; x < inner; ++x) dst[x * inner_stride] = src[x];
    }
  }
}

/* y[n,h,w,c] = bf16(relu(fma(x[n,c,h,w], s[c], b[c]))) */
void oc_affine_relu_nchw_nhwc(const uint16_t* x, const float* s, const float* b, uint16_t* y, int64_t N, int64_t C,
                              int64_t H, int64_t W) {
  const int64_t HW = H * W;
#pragma omp parallel for schedule(static) collapse(2)
  for (int64_t n = 0; n < N; ++n)
    for (int64_t p0 = 0; p0 < HW; p0 += 64) {
      const int64_t p1 = p0 + 64 < HW ? p0 + 64 : HW;
      for (int64_t c = 0; c < C; ++c) {
        const uint16_t* src = x + (n * C + c) * HW;
        const float sc = s[c], bc = b[c];
        for (int64_t p = p0; p < p1; ++p) {
          float v = fmaf(bf16_to_f32(src[p]), sc, bc);
          v = v > 0.0f ? v : 0.0f;
          y[(n * HW + p) * C + c] = f32_to_bf16(v);
        }
      }
    }
}

/* C[M,N] (f32) = A'[M,K] * B[K,N]; A' = A, or relu(A) * mask when mask != NULL; rows [m_begin, m_end). */
void oc_gemm_bf16(const uint16_t* A, const uint16_t* mask, const uint16_t* B, float* Cout, int64_t M, int64_t N,
                  int64_t K, int64_t m_begin, int64_t m_end) {
  (void)M;
  float* Bf = (float*)malloc(sizeof(float) * (size_t)K * (size_t)N);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < K * N; ++i) Bf[i] = bf16_to_f32(B[i]);
  const int64_t KB = 256;
#pragma omp parallel
  {
    float* arow = (float*)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(dynamic, 4)
    for (int64_t m = m_begin; m < m_end; ++m) {
      for (int64_t k = 0; k < K; ++k) {
        float a = bf16_to_f32(A[m * K + k]);
        if (mask) {
          a = a > 0.0f ? a : 0.0f;
          a = bf16_to_f32(f32_to_bf16(a * bf16_to_f32(mask[m * K + k])));
        }
        arow[k] = a;
      }
      float* c = Cout + (m - m_begin) * N;
      for (int64_t n = 0; n < N; ++n) c[n] = 0.0f;
      for (int64_t k0 = 0; k0 < K; k0 += KB) {
        const int64_t k1 = k0 + KB < K ? k0 + KB : K;
        for (int64_t k = k0; k < k1; ++k) {
          const float a = arow[k];
          if (a == 0.0f) continue;
          const float* brow = Bf + k * N;
          for (int64_t n = 0; n < N; ++n) c[n] += a * brow[n];
        }
      }
    }
    free(arow);
  }
  free(Bf);
}

/* Epilogue of README.md:40-79 on rows [m_begin, m_end) of an f32 accumulator block `acc` (row 0 = m_begin).
 * loss / db1 / db2 are accumulated in double so the result can serve as a check value. */
void oc_c3_epilogue(const float* acc, const uint16_t* mask, const uint16_t* y, const uint16_t* b1, const uint16_t* b2,
                    uint16_t* gt_out, uint16_t* gz1_out, double* loss, double* db2, double* db1, int64_t N,
                    int64_t m_begin, int64_t m_end, float inv_n) {
  double loss_total = 0.0;
#pragma omp parallel
  {
    double* l2 = (double*)calloc((size_t)N, sizeof(double));
    double* l1 = (double*)calloc((size_t)N, sizeof(double));
    double lloss = 0.0;
#pragma omp for schedule(static)
    for (int64_t m = m_begin; m < m_end; ++m) {
      const float* c = acc + (m - m_begin) * N;
      for (int64_t n = 0; n < N; ++n) {
        const float z1 = c[n] + bf16_to_f32(b1[n]);
        const float t = tanhf(c[n] + bf16_to_f32(b2[n]));
        const float mk = bf16_to_f32(mask[m * N + n]);
        const float u = z1 > 0.0f ? z1 : 0.0f;
        const float h = (1.0f - u) * mk + u * t;
        const float d = h - bf16_to_f32(y[m * N + n]);
        lloss += (double)((d * d) * inv_n);
        const float g = (d * 2.0f) * inv_n;
        const float gt = (u * g) * (1.0f - t * t);
        const float gu = g * t + (-(g * mk));
        const float gz1 = z1 > 0.0f ? gu : 0.0f;
        gt_out[m * N + n] = f32_to_bf16(gt);
        gz1_out[m * N + n] = f32_to_bf16(gz1);
        l2[n] += gt;
        l1[n] += gz1;
      }
    }
#pragma omp critical
    {
      loss_total += lloss;
      for (int64_t n = 0; n < N; ++n) {
        db2[n] += l2[n];
        db1[n] += l1[n];
      }
    }
    free(l2);
    free(l1);
  }
  *loss += loss_total;
}
