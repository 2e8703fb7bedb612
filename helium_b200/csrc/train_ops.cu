// Hand-written kernels for the pointwise / reduction chains a convolutional training step is made of, in the
// shapes helium's modules produce them (channels-last tensors, per-channel f32 parameters):
//   batch norm        helium/src/modules/batch_norm.rs:32-71 (train mode: mean and E[x^2] over N, H, W,
//                     biased variance E[x^2] - mean^2, eps 1e-3, running statistics 0.9 / 0.1)
//   relu              helium/src/tensor.rs:374-387 (forward and its mask in the backward)
//   SGD + momentum    helium/src/optimizer/sgd.rs:47-62 (an exponential average: avg = g (1 - m) + avg m,
//                     the first step takes avg = g; w -= lr avg)
//   cross entropy     helium/src/loss.rs:5-8 on logits that are a mean over the spatial positions
//                     (resnet-train/src/model.rs:77-82)
// In the reference each of these is a chain of generic pointwise / reduce instructions over broadcast views;
// here the statistics come out of the producing convolution's epilogue (conv_sm100.cuh) and every remaining
// pass over an activation tensor is one HBM-bound kernel with 16-byte accesses and per-channel coefficients.
#include <algorithm>

#include "device_utils.cuh"
#include "he_internal.h"

namespace he {
namespace {

constexpr float kBnEps = 1e-3f;

// stats = [2][C] (sum, sum of squares) over `count` values per channel.
__global__ void bn_finalize_kernel(const float* __restrict__ stats, float count, const float* __restrict__ gamma,
                                   const float* __restrict__ beta, float* __restrict__ running_mean, float* __restrict__ running_var,
                                   float* __restrict__ scale, float* __restrict__ shift, float* __restrict__ mean_out,
                                   float* __restrict__ rstd_out, int C) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const float mean = stats[c] / count;
  const float var = stats[C + c] / count - mean * mean;
  const float rstd = rsqrtf(fmaxf(var, 0.0f) + kBnEps);
  const float s = gamma[c] * rstd;
  scale[c] = s;
  shift[c] = beta[c] - mean * s;
  mean_out[c] = mean;
  rstd_out[c] = rstd;
  if (running_mean) running_mean[c] = running_mean[c] * 0.9f + mean * 0.1f;
  if (running_var) running_var[c] = running_var[c] * 0.9f + var * 0.1f;
}

// y = relu(x * scale[c] + shift[c]) on [pixels, C] bf16, C a multiple of 8.  Optionally the sums of y and
// y^2 per channel as per-CTA partials [grid][2][C] (folded by bn_fold_partials in CTA order).
// A thread owns one group of 8 channels and walks pixels; a CTA owns a contiguous range of pixels.
template <bool STATS, bool RELU>
__global__ void __launch_bounds__(256) bn_apply_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, const float* __restrict__ scale,
                                                       const float* __restrict__ shift, long long pixels, int C,
                                                       float* __restrict__ partials) {
  extern __shared__ float sh[];   // STATS: [256][16] staging for the block reduction
  const int groups = C >> 3;
  const int lanes = 256 / groups;           // pixel lanes per CTA (groups divides 256 or the tail threads idle)
  const int grp = threadIdx.x % groups, lane = threadIdx.x / groups;
  const bool active = lane < lanes;
  float sc[8], sf[8], s0[8], s1[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    sc[i] = scale[grp * 8 + i];
    sf[i] = shift[grp * 8 + i];
    s0[i] = 0.0f; s1[i] = 0.0f;
  }
  const long long per_cta = (pixels + gridDim.x - 1) / gridDim.x;
  const long long p_begin = per_cta * blockIdx.x, p_end = min(pixels, p_begin + per_cta);
  if (active) {
    for (long long p = p_begin + lane; p < p_end; p += lanes) {
      const uint4 v = __ldcs(x + p * groups + grp);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float a = fmaf(__uint_as_float(w[j] << 16), sc[2 * j], sf[2 * j]);
        float b = fmaf(__uint_as_float(w[j] & 0xffff0000u), sc[2 * j + 1], sf[2 * j + 1]);
        if (RELU) { a = fmaxf(a, 0.0f); b = fmaxf(b, 0.0f); }
        o[j] = f32x2_to_bf16x2(a, b);
        if (STATS) {
          // statistics of the values as stored (bf16): what the next normalisation will read
          const float ra = __uint_as_float(o[j] << 16), rb = __uint_as_float(o[j] & 0xffff0000u);
          s0[2 * j] += ra; s0[2 * j + 1] += rb;
          s1[2 * j] = fmaf(ra, ra, s1[2 * j]); s1[2 * j + 1] = fmaf(rb, rb, s1[2 * j + 1]);
        }
      }
      __stcs(y + p * groups + grp, make_uint4(o[0], o[1], o[2], o[3]));
    }
  }
  if (STATS) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      sh[threadIdx.x * 16 + i] = s0[i];
      sh[threadIdx.x * 16 + 8 + i] = s1[i];
    }
    __syncthreads();
    // thread (grp, 0) folds its group's pixel lanes in order
    if (lane == 0) {
      for (int i = 0; i < 8; ++i) {
        float a = 0.0f, b = 0.0f;
        for (int l = 0; l < lanes; ++l) {
          a += sh[(l * groups + grp) * 16 + i];
          b += sh[(l * groups + grp) * 16 + 8 + i];
        }
        partials[((size_t)blockIdx.x * 2 + 0) * C + grp * 8 + i] = a;
        partials[((size_t)blockIdx.x * 2 + 1) * C + grp * 8 + i] = b;
      }
    }
  }
}

// stats[i] = sum over the CTAs' partial rows, 32 columns x 32 row lanes per CTA: lane y adds rows y, y + 32, ...
// in order and the lane sums meet in shared memory in lane order (a fixed function of the partials).
__global__ void __launch_bounds__(1024) bn_fold_partials(const float* __restrict__ partials, float* __restrict__ stats, int n_parts, int C2) {
  __shared__ float sh[32][33];
  const int i = blockIdx.x * 32 + threadIdx.x;
  float s = 0.0f;
  if (i < C2) {
#pragma unroll 4
    for (int k = threadIdx.y; k < n_parts; k += 32) s += partials[(size_t)k * C2 + i];
  }
  sh[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && i < C2) {
    float t = sh[0][threadIdx.x];
#pragma unroll
    for (int y = 1; y < 32; ++y) t += sh[y][threadIdx.x];
    stats[i] = t;
  }
}

// Backward coefficients: with g the (rectifier-masked) gradient at the normalised output and x the
// normalised tensor, stats = [sum g, sum g x] per channel:
//   dbeta = sum g;  dgamma = rstd (sum g x - mean sum g);
//   dx = A g + B x + K,  A = gamma rstd,  B = -A rstd dgamma / m,  K = -A dbeta / m - B mean
__global__ void bn_backward_coeffs_kernel(const float* __restrict__ stats, float count, const float* __restrict__ gamma,
                                          const float* __restrict__ mean, const float* __restrict__ rstd, float* __restrict__ coef,
                                          float* __restrict__ dgamma, float* __restrict__ dbeta, int C) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const float sg = stats[c], sgx = stats[C + c];
  const float dg = rstd[c] * (sgx - mean[c] * sg);
  const float a = gamma[c] * rstd[c];
  const float b = -a * rstd[c] * dg / count;
  coef[c] = a;
  coef[C + c] = b;
  coef[2 * C + c] = -a * sg / count - b * mean[c];
  dgamma[c] = dg;
  dbeta[c] = sg;
}

// out = A[c] g + B[c] x + K[c] (+ e) on [pixels, C] bf16; with MASK the result is additionally zeroed where
// mx * ms[c] + mb[c] <= 0 (the rectifier in front of an enclosing normalisation) and the sums of out and
// out * mx per channel are produced like in bn_apply_kernel.
template <bool ADD, bool MASK, bool SUM = false>
__global__ void __launch_bounds__(256) bn_backward_apply_kernel(const uint4* __restrict__ g, const uint4* __restrict__ x,
                                                                const uint4* __restrict__ e, uint4* __restrict__ out,
                                                                const float* __restrict__ coef, const uint4* __restrict__ mx,
                                                                const float* __restrict__ ms, const float* __restrict__ mb,
                                                                long long pixels, int C, float* __restrict__ partials) {
  extern __shared__ float sh[];
  const int groups = C >> 3;
  const int lanes = 256 / groups;
  const int grp = threadIdx.x % groups, lane = threadIdx.x / groups;
  const bool active = lane < lanes;
  float ca[8], cb[8], ck[8], ksc[8], ksf[8], s0[8], s1[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    ca[i] = coef[grp * 8 + i]; cb[i] = coef[C + grp * 8 + i]; ck[i] = coef[2 * C + grp * 8 + i];
    ksc[i] = MASK ? ms[grp * 8 + i] : 0.0f; ksf[i] = MASK ? mb[grp * 8 + i] : 0.0f;
    s0[i] = 0.0f; s1[i] = 0.0f;
  }
  const long long per_cta = (pixels + gridDim.x - 1) / gridDim.x;
  const long long p_begin = per_cta * blockIdx.x, p_end = min(pixels, p_begin + per_cta);
  if (active) {
    for (long long p = p_begin + lane; p < p_end; p += lanes) {
      const size_t idx = (size_t)p * groups + grp;
      const uint4 vg = __ldcs(g + idx), vx = __ldcs(x + idx);
      uint4 ve = make_uint4(0, 0, 0, 0), vm = make_uint4(0, 0, 0, 0);
      if (ADD) ve = __ldcs(e + idx);
      if (MASK) vm = __ldcs(mx + idx);
      const uint32_t wg[4] = {vg.x, vg.y, vg.z, vg.w}, wx[4] = {vx.x, vx.y, vx.z, vx.w}, we[4] = {ve.x, ve.y, ve.z, ve.w},
                     wm[4] = {vm.x, vm.y, vm.z, vm.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float r[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int i = 2 * j + h;
          const float gv = h ? __uint_as_float(wg[j] & 0xffff0000u) : __uint_as_float(wg[j] << 16);
          const float xv = h ? __uint_as_float(wx[j] & 0xffff0000u) : __uint_as_float(wx[j] << 16);
          float t = fmaf(ca[i], gv, fmaf(cb[i], xv, ck[i]));
          if (ADD) t += h ? __uint_as_float(we[j] & 0xffff0000u) : __uint_as_float(we[j] << 16);
          if (MASK) {
            const float mv = h ? __uint_as_float(wm[j] & 0xffff0000u) : __uint_as_float(wm[j] << 16);
            t = fmaf(mv, ksc[i], ksf[i]) > 0.0f ? t : 0.0f;
            s0[i] += t;
            s1[i] = fmaf(t, mv, s1[i]);
          }
          r[h] = t;
        }
        o[j] = f32x2_to_bf16x2(r[0], r[1]);
        if (SUM) {   // column sums of the tensor as stored: what a reduction over the bf16 flow would add up
          s0[2 * j] += __uint_as_float(o[j] << 16);
          s0[2 * j + 1] += __uint_as_float(o[j] & 0xffff0000u);
        }
      }
      __stcs(out + idx, make_uint4(o[0], o[1], o[2], o[3]));
    }
  }
  if (MASK) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      sh[threadIdx.x * 16 + i] = s0[i];
      sh[threadIdx.x * 16 + 8 + i] = s1[i];
    }
    __syncthreads();
    if (lane == 0) {
      for (int i = 0; i < 8; ++i) {
        float a = 0.0f, b = 0.0f;
        for (int l = 0; l < lanes; ++l) {
          a += sh[(l * groups + grp) * 16 + i];
          b += sh[(l * groups + grp) * 16 + 8 + i];
        }
        partials[((size_t)blockIdx.x * 2 + 0) * C + grp * 8 + i] = a;
        partials[((size_t)blockIdx.x * 2 + 1) * C + grp * 8 + i] = b;
      }
    }
  }
  if (SUM && !MASK) {
#pragma unroll
    for (int i = 0; i < 8; ++i) sh[threadIdx.x * 8 + i] = s0[i];
    __syncthreads();
    if (lane == 0) {
      for (int i = 0; i < 8; ++i) {
        float a = 0.0f;
        for (int l = 0; l < lanes; ++l) a += sh[(l * groups + grp) * 8 + i];
        partials[(size_t)blockIdx.x * C + grp * 8 + i] = a;
      }
    }
  }
}

// out = a + b on bf16 tensors (gradient branches meeting at a fork), 16 bytes per thread per step
__global__ void __launch_bounds__(256) add_bf16_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b, uint4* __restrict__ out,
                                                       long long n_vec) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (long long)gridDim.x * blockDim.x) {
    const uint4 va = __ldcs(a + i), vb = __ldcs(b + i);
    const uint32_t wa[4] = {va.x, va.y, va.z, va.w}, wb[4] = {vb.x, vb.y, vb.z, vb.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      o[j] = f32x2_to_bf16x2(__uint_as_float(wa[j] << 16) + __uint_as_float(wb[j] << 16),
                             __uint_as_float(wa[j] & 0xffff0000u) + __uint_as_float(wb[j] & 0xffff0000u));
    __stcs(out + i, make_uint4(o[0], o[1], o[2], o[3]));
  }
}

// per-channel sum over pixels of a bf16 [pixels, C] tensor (the gradient of a convolution's bias), f32 out;
// one CTA per 8-channel group would starve the device on narrow layers, so CTAs split the pixels and a
// fold follows, like the statistics above
__global__ void __launch_bounds__(256) colsum_bf16_kernel(const uint4* __restrict__ x, long long pixels, int C, float* __restrict__ partials) {
  extern __shared__ float sh[];
  const int groups = C >> 3;
  const int lanes = 256 / groups;
  const int grp = threadIdx.x % groups, lane = threadIdx.x / groups;
  float s0[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) s0[i] = 0.0f;
  const long long per_cta = (pixels + gridDim.x - 1) / gridDim.x;
  const long long p_begin = per_cta * blockIdx.x, p_end = min(pixels, p_begin + per_cta);
  if (lane < lanes)
    for (long long p = p_begin + lane; p < p_end; p += lanes) {
      const uint4 v = __ldcs(x + p * groups + grp);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        s0[2 * j] += __uint_as_float(w[j] << 16);
        s0[2 * j + 1] += __uint_as_float(w[j] & 0xffff0000u);
      }
    }
#pragma unroll
  for (int i = 0; i < 8; ++i) sh[threadIdx.x * 8 + i] = s0[i];
  __syncthreads();
  if (lane == 0)
    for (int i = 0; i < 8; ++i) {
      float a = 0.0f;
      for (int l = 0; l < lanes; ++l) a += sh[(l * groups + grp) * 8 + i];
      partials[(size_t)blockIdx.x * C + grp * 8 + i] = a;
    }
}

// SGD with helium's momentum: avg = first ? g : g (1 - m) + avg m;  w -= lr avg;  w16 = bf16(w)
template <typename G>
__global__ void __launch_bounds__(256) sgd_momentum_kernel(float* __restrict__ w, float* __restrict__ avg, const G* __restrict__ g,
                                                           unsigned short* __restrict__ w16, long long n, float lr, float m, int first) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float gv;
    if (sizeof(G) == 4) gv = reinterpret_cast<const float*>(g)[i];
    else gv = bf16_bits_to_f32(reinterpret_cast<const unsigned short*>(g)[i]);
    const float a = first ? gv : gv * (1.0f - m) + avg[i] * m;
    if (avg) avg[i] = a;
    const float nw = w[i] - a * lr;
    w[i] = nw;
    if (w16) w16[i] = (unsigned short)f32_to_bf16_bits(nw);
  }
}

// One CTA per image: logits = mean over `positions` of y[n, pos, :] (bf16, rounded to bf16 like the reference's
// reduce_mean on a bf16 tensor), loss_n = -log_softmax(logits)[label] / batch, and the gradient at y:
// (softmax - onehot) / (batch * positions), the same value at every position, as bf16.
__global__ void __launch_bounds__(256) pool_softmax_ce_kernel(const unsigned short* __restrict__ y, const int* __restrict__ labels,
                                                              float* __restrict__ loss, unsigned short* __restrict__ dy, int positions,
                                                              int classes, int batch) {
  extern __shared__ float logit[];   // [classes]
  __shared__ float red[256];
  const int n = blockIdx.x;
  const unsigned short* src = y + (size_t)n * positions * classes;
  for (int c = threadIdx.x; c < classes; c += 256) {
    float s = 0.0f;
    for (int p = 0; p < positions; ++p) s += bf16_bits_to_f32(src[(size_t)p * classes + c]);
    logit[c] = bf16_bits_to_f32(f32_to_bf16_bits(s * (1.0f / positions)));
  }
  __syncthreads();
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < classes; c += 256) mx = fmaxf(mx, logit[c]);
  red[threadIdx.x] = mx;
  __syncthreads();
  for (int off = 128; off > 0; off >>= 1) {
    if ((int)threadIdx.x < off) red[threadIdx.x] = fmaxf(red[threadIdx.x], red[threadIdx.x + off]);
    __syncthreads();
  }
  mx = red[0];
  __syncthreads();
  float se = 0.0f;
  for (int c = threadIdx.x; c < classes; c += 256) se += expf(logit[c] - mx);
  red[threadIdx.x] = se;
  __syncthreads();
  for (int off = 128; off > 0; off >>= 1) {
    if ((int)threadIdx.x < off) red[threadIdx.x] += red[threadIdx.x + off];
    __syncthreads();
  }
  se = red[0];
  const float lse = mx + logf(se);
  const int label = labels[n];
  if (threadIdx.x == 0) loss[n] = -(logit[label] - lse) / batch;
  const float k = 1.0f / ((float)batch * positions);
  unsigned short* dst = dy + (size_t)n * positions * classes;
  for (int c = threadIdx.x; c < classes; c += 256) {
    const float gsm = (expf(logit[c] - lse) - (c == label ? 1.0f : 0.0f)) * k;
    const unsigned short b = (unsigned short)f32_to_bf16_bits(gsm);
    for (int p = 0; p < positions; ++p) dst[(size_t)p * classes + c] = b;
  }
}

// cols[n, p, q, k] = x[n, p * st + r - pad_h, q * st + s - pad_w, c] for k = (r * S + s) * C + c < R * S * C, zero
// elsewhere (outside the image, and the padding columns up to `pitch`).  One thread writes 8 consecutive k of
// one output pixel as a 16-byte store; the source elements are 2-byte loads that hit L1 / L2 (every input pixel
// is read by R * S / st^2 outputs).  Used for convolutions whose channel count is too small to feed the tensor
// core from the NHWC tensor directly (an RGB stem): the explicit patch matrix then goes through the same
// convolution kernels as a 1 x 1 convolution over `pitch` channels.
// A CTA produces the patch rows of `imq` consecutive output pixels of one output row: the R source rows they read
// are staged in shared memory with coalesced loads; then thread (group g, vector v) assembles vector v of pixels
// g, g + groups, ... from eight 2-byte shared-memory reads whose offsets inside the staged rows it computed once
// for the whole kernel (they depend on v only; a pixel step is a constant shift), and stores 16 bytes.  A warp's
// stores cover consecutive vectors of consecutive pixels, i.e. one contiguous stretch of the patch matrix.
__global__ void __launch_bounds__(256) im2col_kernel(const unsigned short* __restrict__ x, uint4* __restrict__ cols, int NB, int H, int W,
                                                     int C, int R, int S, int st, int pad_h, int pad_w, int P, int Q, int pitch, int imq) {
  extern __shared__ unsigned short srow[];   // [R][span * C], span = (imq - 1) * st + S source pixels
  const int span = (imq - 1) * st + S;
  const int row_pitch = span * C;
  const int q_tiles = (Q + imq - 1) / imq;
  const int vec_per_pix = pitch >> 3;
  const int groups = 256 / vec_per_pix;
  const int v = threadIdx.x % vec_per_pix, grp = threadIdx.x / vec_per_pix;
  const int rsc = R * S * C, sc = S * C;
  int off[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int k = v * 8 + j;
    const int r = k / sc;                         // k - r * sc = s * C + c: contiguous in the source row
    off[j] = k < rsc ? r * row_pitch + (k - r * sc) : -1;
  }
  const int pix_step = st * C;
  bool all_valid = true;
#pragma unroll
  for (int j = 0; j < 8; ++j) all_valid = all_valid && off[j] >= 0;
  // staging slots of this thread within a source row (the same for every row and tile): element index and the
  // source pixel it belongs to, so that the loop below does no division
  int slot_w[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) slot_w[q] = (threadIdx.x + 256 * q) / C;
  for (long long tile = blockIdx.x; tile < (long long)NB * P * q_tiles; tile += gridDim.x) {
    const int qt = (int)(tile % q_tiles);
    const long long np = tile / q_tiles;
    const int p = (int)(np % P), n = (int)(np / P);
    const int q0 = qt * imq, w0 = q0 * st - pad_w;
    __syncthreads();   // the previous tile's readers are done
    for (int r = 0; r < R; ++r) {
      const int h = p * st + r - pad_h;
      const bool row_ok = h >= 0 && h < H;
      const unsigned short* src = x + (((long long)n * H + h) * W + w0) * C;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int e = threadIdx.x + 256 * q;
        if (e < row_pitch) {
          const int w = w0 + slot_w[q];
          srow[r * row_pitch + e] = (row_ok && w >= 0 && w < W) ? __ldg(src + e) : (unsigned short)0;
        }
      }
      for (int e = threadIdx.x + 1024; e < row_pitch; e += 256) {   // rows longer than 1024 elements (wide tiles of many channels)
        const int w = w0 + e / C;
        srow[r * row_pitch + e] = (row_ok && w >= 0 && w < W) ? __ldg(src + e) : (unsigned short)0;
      }
    }
    __syncthreads();
    const int nq = min(imq, Q - q0);
    if (grp < groups) {
      uint4* dst = cols + (((size_t)n * P + p) * Q + q0) * vec_per_pix + v;
      if (all_valid) {
        for (int ql = grp; ql < nq; ql += groups) {
          const unsigned short* sp = srow + ql * pix_step;
          uint32_t e[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) e[j] = sp[off[j]];
          dst[(size_t)ql * vec_per_pix] = make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16), e[6] | (e[7] << 16));
        }
      } else {
        for (int ql = grp; ql < nq; ql += groups) {
          const unsigned short* sp = srow + ql * pix_step;
          uint32_t e[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) e[j] = off[j] >= 0 ? (uint32_t)sp[off[j]] : 0u;
          dst[(size_t)ql * vec_per_pix] = make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16), e[6] | (e[7] << 16));
        }
      }
    }
  }
}

int ctas_for(long long pixels, int C) {
  const int lanes = 256 / (C >> 3);
  const long long want = (pixels + (long long)lanes * 8 - 1) / ((long long)lanes * 8);
  return (int)std::max<long long>(1, std::min<long long>(want, 148 * 2));
}

int32_t check_channels(const char* who, long long pixels, int C) {
  if (pixels <= 0 || C <= 0) HE_FAIL(HE_ERR_INVALID, "%s: empty tensor", who);
  if (C % 8 != 0 || C > 2048) HE_FAIL(HE_ERR_UNSUPPORTED, "%s: channel count %d must be a multiple of 8 (at most 2048)", who, C);
  return HE_OK;
}

}  // namespace
}  // namespace he

using namespace he;

extern "C" {

int32_t he_bn_finalize(const float* stats, int64_t count, const float* gamma, const float* beta, float* running_mean, float* running_var,
                       float* scale, float* shift, float* mean, float* rstd, int32_t channels, void* cu_stream) {
  if (!stats || !gamma || !beta || !scale || !shift || !mean || !rstd || channels <= 0 || count <= 0)
    HE_FAIL(HE_ERR_INVALID, "he_bn_finalize: bad argument");
  bn_finalize_kernel<<<(channels + 127) / 128, 128, 0, (cudaStream_t)cu_stream>>>(stats, (float)count, gamma, beta, running_mean, running_var,
                                                                                 scale, shift, mean, rstd, channels);
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

size_t he_bn_workspace_bytes(int64_t pixels, int32_t channels) {
  if (pixels <= 0 || channels < 8) return 0;
  return (size_t)ctas_for(pixels, channels) * 2 * channels * sizeof(float);
}

int32_t he_bn_apply(const void* x, void* y, const float* scale, const float* shift, int64_t pixels, int32_t channels, int32_t relu,
                    float* stats_out, void* workspace, void* cu_stream) {
  if (!x || !y || !scale || !shift) HE_FAIL(HE_ERR_INVALID, "he_bn_apply: null argument");
  HE_TRY(check_channels("he_bn_apply", pixels, channels));
  if (((uintptr_t)x | (uintptr_t)y) & 15) HE_FAIL(HE_ERR_UNSUPPORTED, "he_bn_apply: tensors must be 16-byte aligned");
  if (stats_out && !workspace) HE_FAIL(HE_ERR_WORKSPACE, "he_bn_apply: statistics need he_bn_workspace_bytes() of workspace");
  cudaStream_t st = (cudaStream_t)cu_stream;
  const int grid = ctas_for(pixels, channels);
  const uint4* xi = reinterpret_cast<const uint4*>(x);
  uint4* yo = reinterpret_cast<uint4*>(y);
  float* parts = reinterpret_cast<float*>(workspace);
  if (stats_out) {
    if (relu) bn_apply_kernel<true, true><<<grid, 256, 256 * 16 * 4, st>>>(xi, yo, scale, shift, pixels, channels, parts);
    else bn_apply_kernel<true, false><<<grid, 256, 256 * 16 * 4, st>>>(xi, yo, scale, shift, pixels, channels, parts);
    HE_CUDA(cudaGetLastError());
    bn_fold_partials<<<(2 * channels + 31) / 32, dim3(32, 32), 0, st>>>(parts, stats_out, grid, 2 * channels);
  } else {
    if (relu) bn_apply_kernel<false, true><<<grid, 256, 0, st>>>(xi, yo, scale, shift, pixels, channels, nullptr);
    else bn_apply_kernel<false, false><<<grid, 256, 0, st>>>(xi, yo, scale, shift, pixels, channels, nullptr);
  }
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

int32_t he_bn_backward_coeffs(const float* stats, int64_t count, const float* gamma, const float* mean, const float* rstd, float* coef,
                              float* dgamma, float* dbeta, int32_t channels, void* cu_stream) {
  if (!stats || !gamma || !mean || !rstd || !coef || !dgamma || !dbeta || channels <= 0 || count <= 0)
    HE_FAIL(HE_ERR_INVALID, "he_bn_backward_coeffs: bad argument");
  bn_backward_coeffs_kernel<<<(channels + 127) / 128, 128, 0, (cudaStream_t)cu_stream>>>(stats, (float)count, gamma, mean, rstd, coef, dgamma,
                                                                                         dbeta, channels);
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

int32_t he_bn_backward_apply(const void* g, const void* x, const void* addend, void* out, const float* coef, const void* mask_x,
                             const float* mask_scale, const float* mask_shift, float* stats_out, void* workspace, int64_t pixels,
                             int32_t channels, void* cu_stream) {
  if (!g || !x || !out || !coef) HE_FAIL(HE_ERR_INVALID, "he_bn_backward_apply: null argument");
  HE_TRY(check_channels("he_bn_backward_apply", pixels, channels));
  if (((uintptr_t)g | (uintptr_t)x | (uintptr_t)out | (uintptr_t)addend | (uintptr_t)mask_x) & 15)
    HE_FAIL(HE_ERR_UNSUPPORTED, "he_bn_backward_apply: tensors must be 16-byte aligned");
  const bool mask = mask_x != nullptr;
  if (mask && (!mask_scale || !mask_shift || !stats_out || !workspace))
    HE_FAIL(HE_ERR_INVALID, "he_bn_backward_apply: a mask needs its scale, shift, a statistics output and a workspace");
  cudaStream_t st = (cudaStream_t)cu_stream;
  const int grid = ctas_for(pixels, channels);
  auto G = reinterpret_cast<const uint4*>(g); auto X = reinterpret_cast<const uint4*>(x); auto E = reinterpret_cast<const uint4*>(addend);
  auto O = reinterpret_cast<uint4*>(out); auto MX = reinterpret_cast<const uint4*>(mask_x);
  float* parts = reinterpret_cast<float*>(workspace);
  if (mask) {
    if (addend) bn_backward_apply_kernel<true, true><<<grid, 256, 256 * 16 * 4, st>>>(G, X, E, O, coef, MX, mask_scale, mask_shift, pixels, channels, parts);
    else bn_backward_apply_kernel<false, true><<<grid, 256, 256 * 16 * 4, st>>>(G, X, E, O, coef, MX, mask_scale, mask_shift, pixels, channels, parts);
    HE_CUDA(cudaGetLastError());
    bn_fold_partials<<<(2 * channels + 31) / 32, dim3(32, 32), 0, st>>>(parts, stats_out, grid, 2 * channels);
  } else if (stats_out) {
    // no mask: the statistics output is [C] column sums of `out` as stored (the bias gradient of the convolution
    // this flow enters next), folded from per-CTA partials in CTA order
    if (!workspace) HE_FAIL(HE_ERR_WORKSPACE, "he_bn_backward_apply: column sums need he_bn_workspace_bytes() of workspace");
    if (addend) bn_backward_apply_kernel<true, false, true><<<grid, 256, 256 * 8 * 4, st>>>(G, X, E, O, coef, nullptr, nullptr, nullptr, pixels, channels, parts);
    else bn_backward_apply_kernel<false, false, true><<<grid, 256, 256 * 8 * 4, st>>>(G, X, E, O, coef, nullptr, nullptr, nullptr, pixels, channels, parts);
    HE_CUDA(cudaGetLastError());
    bn_fold_partials<<<(channels + 31) / 32, dim3(32, 32), 0, st>>>(parts, stats_out, grid, channels);
  } else {
    if (addend) bn_backward_apply_kernel<true, false><<<grid, 256, 0, st>>>(G, X, E, O, coef, nullptr, nullptr, nullptr, pixels, channels, nullptr);
    else bn_backward_apply_kernel<false, false><<<grid, 256, 0, st>>>(G, X, E, O, coef, nullptr, nullptr, nullptr, pixels, channels, nullptr);
  }
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

int32_t he_add_bf16(const void* a, const void* b, void* out, int64_t n, void* cu_stream) {
  if (!a || !b || !out || n <= 0) HE_FAIL(HE_ERR_INVALID, "he_add_bf16: bad argument");
  if (n % 8 != 0 || (((uintptr_t)a | (uintptr_t)b | (uintptr_t)out) & 15)) HE_FAIL(HE_ERR_UNSUPPORTED, "he_add_bf16: needs 16-byte aligned tensors of a multiple of 8 elements");
  const long long nv = n / 8;
  const unsigned grid = (unsigned)std::min<long long>((nv + 255) / 256, 148 * 16);
  add_bf16_kernel<<<grid, 256, 0, (cudaStream_t)cu_stream>>>(reinterpret_cast<const uint4*>(a), reinterpret_cast<const uint4*>(b),
                                                             reinterpret_cast<uint4*>(out), nv);
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

int32_t he_colsum_bf16(const void* x, float* out, void* workspace, int64_t pixels, int32_t channels, void* cu_stream) {
  if (!x || !out || !workspace) HE_FAIL(HE_ERR_INVALID, "he_colsum_bf16: null argument");
  HE_TRY(check_channels("he_colsum_bf16", pixels, channels));
  cudaStream_t st = (cudaStream_t)cu_stream;
  const int grid = ctas_for(pixels, channels);
  float* parts = reinterpret_cast<float*>(workspace);
  colsum_bf16_kernel<<<grid, 256, 256 * 8 * 4, st>>>(reinterpret_cast<const uint4*>(x), pixels, channels, parts);
  HE_CUDA(cudaGetLastError());
  bn_fold_partials<<<(channels + 31) / 32, dim3(32, 32), 0, st>>>(parts, out, grid, channels);
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

int32_t he_sgd_momentum(float* w, float* avg, const void* grad, int32_t grad_dtype, void* w_bf16, int64_t n, float lr, float momentum,
                        int32_t first_step, void* cu_stream) {
  if (!w || !grad || n <= 0) HE_FAIL(HE_ERR_INVALID, "he_sgd_momentum: bad argument");
  if (grad_dtype != HE_F32 && grad_dtype != HE_BF16) HE_FAIL(HE_ERR_UNSUPPORTED, "he_sgd_momentum: gradients must be f32 or bf16");
  const unsigned grid = (unsigned)std::min<long long>((n + 255) / 256, 148 * 16);
  cudaStream_t st = (cudaStream_t)cu_stream;
  if (grad_dtype == HE_F32)
    sgd_momentum_kernel<float><<<grid, 256, 0, st>>>(w, avg, reinterpret_cast<const float*>(grad), reinterpret_cast<unsigned short*>(w_bf16), n, lr,
                                                     momentum, first_step);
  else
    sgd_momentum_kernel<unsigned short><<<grid, 256, 0, st>>>(w, avg, reinterpret_cast<const unsigned short*>(grad),
                                                              reinterpret_cast<unsigned short*>(w_bf16), n, lr, momentum, first_step);
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

int32_t he_im2col_nhwc(const void* x, void* cols, int32_t batch, int32_t in_h, int32_t in_w, int32_t channels, int32_t kernel_h,
                       int32_t kernel_w, int32_t stride, int32_t pitch, void* cu_stream) {
  if (!x || !cols || batch <= 0 || in_h <= 0 || in_w <= 0 || channels <= 0 || kernel_h <= 0 || kernel_w <= 0 || stride <= 0)
    HE_FAIL(HE_ERR_INVALID, "he_im2col_nhwc: bad argument");
  if (pitch % 8 != 0 || pitch < kernel_h * kernel_w * channels) HE_FAIL(HE_ERR_INVALID, "he_im2col_nhwc: pitch must be a multiple of 8 and at least R*S*C = %d", kernel_h * kernel_w * channels);
  if ((uintptr_t)cols & 15) HE_FAIL(HE_ERR_UNSUPPORTED, "he_im2col_nhwc: the patch matrix must be 16-byte aligned");
  const int P = in_h / stride, Q = in_w / stride;   // 'Same' geometry: helium-ir/src/opgraph/op/conv.rs:51-74
  if (pitch > 2048) HE_FAIL(HE_ERR_UNSUPPORTED, "he_im2col_nhwc: pitch above 2048 columns");
  // pixels per CTA tile: a whole output row if its source rows fit 48 KB of staging, else the largest power of two
  auto staging = [&](int q) { return (size_t)kernel_h * ((q - 1) * stride + kernel_w) * channels * sizeof(unsigned short); };
  int imq = 128;
  while (imq > 1 && (imq / 2 >= Q || staging(imq) > 48 * 1024)) imq >>= 1;
  const size_t smem = staging(imq);
  if (smem > 48 * 1024) HE_FAIL(HE_ERR_UNSUPPORTED, "he_im2col_nhwc: %zu bytes of staging exceed 48 KB (channel count too large for this route)", smem);
  const long long tiles = (long long)batch * P * ((Q + imq - 1) / imq);
  const unsigned grid = (unsigned)std::min<long long>(tiles, 148 * 8);
  im2col_kernel<<<grid, 256, smem, (cudaStream_t)cu_stream>>>(reinterpret_cast<const unsigned short*>(x), reinterpret_cast<uint4*>(cols), batch,
                                                          in_h, in_w, channels, kernel_h, kernel_w, stride, kernel_h / 2, kernel_w / 2, P, Q, pitch, imq);
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

int32_t he_pool_softmax_ce(const void* y, const int32_t* labels, float* loss, void* dy, int32_t batch, int32_t positions, int32_t classes,
                           void* cu_stream) {
  if (!y || !labels || !loss || !dy || batch <= 0 || positions <= 0 || classes <= 0) HE_FAIL(HE_ERR_INVALID, "he_pool_softmax_ce: bad argument");
  if (classes > 12000) HE_FAIL(HE_ERR_UNSUPPORTED, "he_pool_softmax_ce: more than 12000 classes");
  pool_softmax_ce_kernel<<<batch, 256, classes * sizeof(float), (cudaStream_t)cu_stream>>>(
      reinterpret_cast<const unsigned short*>(y), labels, loss, reinterpret_cast<unsigned short*>(dy), positions, classes, batch);
  HE_CUDA(cudaGetLastError());
  return HE_OK;
}

}  // extern "C"
