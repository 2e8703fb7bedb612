// Sum reduction over trailing dims that needs no device allocation from anybody.
//
// Why it exists: the reference's `PointwiseGraph::execute(tensors, stream, cx)`
// (helium/src/cuda/instr/pointwise.rs:57) receives no allocator handle -- only the cuDNN instruction
// is given `hold_allocations` / `allocation_stream` (helium/src/cuda/instr.rs:27-52).  A drop-in
// body for that call therefore has nowhere to obtain the partial-sum workspace that he_launch
// asks for when a reduction group spans several CTAs, and calling cudaMalloc from inside an
// instruction would serialise the device and break the executor's stream-ordered pool.  This
// entry point keeps its partial sums in a fixed array that lives in the library image instead.
//
// Same arithmetic as the workspace path of pointwise.cu: a CTA sums a 4096-element slice of a
// group (thread-strided adds, shuffle tree, warps folded in order), writes one partial, and a
// second kernel folds a group's partials the same way.  The order is fixed, so results repeat
// bit for bit; they agree with he_launch's to f32 rounding, not bitwise (it may slice differently).
#include <mutex>

#include "he_internal.h"

namespace he {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxDevices = 64;

// The scratch: one partial per (group, slice).  256 KiB in every GPU context that loads this
// library, held until the process exits.
static __device__ __align__(256) float g_noalloc_partials[HE_NOALLOC_MAX_PARTIALS];

// Device address of the array per device ordinal, looked up once (host code cannot use the symbol
// name as an address).
float* g_partials_addr[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;

__global__ void __launch_bounds__(kThreads) noalloc_sum_slices(const float* __restrict__ in, float* __restrict__ partials,
                                                               float* __restrict__ out, unsigned group_size,
                                                               unsigned slices_per_group, unsigned slice) {
  __shared__ float warp_sums[kThreads / 32];
  const unsigned group = blockIdx.x / slices_per_group;
  const unsigned s = blockIdx.x - group * slices_per_group;
  const unsigned start = s * slice;
  const unsigned end = min(start + slice, group_size);
  const float* src = in + (size_t)group * group_size;
  float acc = 0.0f;
  // A full slice on a 16-byte boundary is read as four float4 per thread (the slice is 256 threads x 16
  // elements); the per-thread order of additions is the same as in the scalar walk below, element e of the slice
  // goes to thread e % 256 in both, so the result does not depend on which walk ran.
  if (end - start == kThreads * 16 && ((reinterpret_cast<uintptr_t>(src + start) & 15) == 0)) {
    const float* base = src + start;
    // thread t owns elements t, t + 256, ...; the four elements of a 16-byte vector belong to four different threads,
    // so the CTA moves the slice to shared memory with 16-byte loads and every thread then reads its own elements
    __shared__ float stage[kThreads * 16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(base) + i * kThreads + threadIdx.x);
      reinterpret_cast<float4*>(stage)[i * kThreads + threadIdx.x] = v;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 16; ++i) acc += stage[i * kThreads + threadIdx.x];
  } else {
    for (unsigned e = start + threadIdx.x; e < end; e += kThreads) acc += __ldg(src + e);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, off);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float v = warp_sums[0];
    for (int w = 1; w < kThreads / 32; ++w) v += warp_sums[w];
    if (slices_per_group == 1) out[group] = v;
    else partials[(size_t)group * slices_per_group + s] = v;
  }
}

// One CTA per group folds that group's partials with the same thread-strided / tree order.
__global__ void __launch_bounds__(kThreads) noalloc_fold_partials(const float* __restrict__ partials, float* __restrict__ out,
                                                                  unsigned slices_per_group) {
  __shared__ float warp_sums[kThreads / 32];
  const float* p = partials + (size_t)blockIdx.x * slices_per_group;
  float acc = 0.0f;
  for (unsigned s = threadIdx.x; s < slices_per_group; s += kThreads) acc += p[s];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, off);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float v = warp_sums[0];
    for (int w = 1; w < kThreads / 32; ++w) v += warp_sums[w];
    out[blockIdx.x] = v;
  }
}

}  // namespace
}  // namespace he

using namespace he;

extern "C" int32_t he_reduce_sum_f32_noalloc(const float* in, float* out, int64_t num_groups, int64_t group_size,
                                             void* cu_stream) {
  if (!in || !out) HE_FAIL(HE_ERR_INVALID, "he_reduce_sum_f32_noalloc: null tensor pointer");
  if (num_groups < 0 || group_size < 0) HE_FAIL(HE_ERR_INVALID, "he_reduce_sum_f32_noalloc: negative extent");
  if (num_groups == 0) return HE_OK;
  // compared by division: the product of two hostile 64-bit extents can wrap past the bound
  if (group_size == 0 || group_size > ((1ll << 31) - 1) / num_groups)
    HE_FAIL(HE_ERR_UNSUPPORTED, "he_reduce_sum_f32_noalloc: needs 0 < num_groups * group_size < 2^31 (got %lld x %lld)",
            (long long)num_groups, (long long)group_size);
  int dev = -1;
  HE_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) HE_FAIL(HE_ERR_UNSUPPORTED, "he_reduce_sum_f32_noalloc: device ordinal %d out of range", dev);
  {
    // One-time set-up per device, with that device current: resolve the array's device address.
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_partials_addr[dev]) {
      float* addr = nullptr;
      cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&addr), g_noalloc_partials);
      if (e != cudaSuccess || !addr)
        HE_FAIL(HE_ERR_CUDA, "cudaGetSymbolAddress(partials) failed on device %d: %s", dev, cudaGetErrorString(e));
      g_partials_addr[dev] = addr;
    }
  }
  // One partial per 4096-element slice of a group (the slice he_launch's planner starts from,
  // pointwise.cu); a group that fits one slice is written straight to `out`.
  const unsigned slice = kThreads * 16;
  const unsigned spg = (unsigned)((group_size + slice - 1) / slice);
  const unsigned long long n_partials = spg > 1 ? (unsigned long long)spg * (unsigned long long)num_groups : 0;
  if (n_partials > HE_NOALLOC_MAX_PARTIALS)
    HE_FAIL(HE_ERR_WORKSPACE,
            "he_reduce_sum_f32_noalloc: %lld groups x %u slices need %llu partial sums, the built-in scratch holds %d; "
            "use he_plan_pointwise + he_launch with a caller workspace for this shape",
            (long long)num_groups, spg, n_partials, (int)HE_NOALLOC_MAX_PARTIALS);
  cudaStream_t stream = (cudaStream_t)cu_stream;
  float* partials = g_partials_addr[dev];
  // num_groups * group_size < 2^31 and spg <= ceil(group_size / 4096), so the grid fits 31 bits; checked anyway
  const unsigned long long grid = (unsigned long long)num_groups * spg;
  if (grid == 0 || grid > 0x7fffffffull)
    HE_FAIL(HE_ERR_UNSUPPORTED, "he_reduce_sum_f32_noalloc: grid of %llu CTAs is out of range", grid);
  noalloc_sum_slices<<<(unsigned)grid, kThreads, 0, stream>>>(in, partials, out, (unsigned)group_size, spg, slice);
  HE_CUDA(cudaGetLastError());
  if (spg > 1) {
    noalloc_fold_partials<<<(unsigned)num_groups, kThreads, 0, stream>>>(partials, out, spg);
    HE_CUDA(cudaGetLastError());
  }
  return HE_OK;
}
