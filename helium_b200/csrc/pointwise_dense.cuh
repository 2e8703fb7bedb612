// Dense elementwise tier-2 kernels (pointwise_dense.cu): catalogue lookup and launch.
#pragma once
#include <string>

#include "device_utils.cuh"
#include "he_internal.h"

namespace he {

enum EwKind : int { EW_RELU = 0, EW_GELU, EW_ADD, EW_MUL, EW_ADD_RELU, EW_MUL_RELU, EW_FMA, EW_AXMY };

struct EwMatch {
  int kind = -1;
  int n_in = 0;
  float k = 0.0f;          // the program's constant (EW_AXMY)
  const char* name = "";
};

// True when `canon_text` (canonicalize_program of a program compiled without FMA fusion) is one of
// the catalogued dense programs.  The caller still has to check that every tensor is dense, of one
// dtype, 16-byte aligned and a whole number of 16-byte vectors long.
bool match_dense_elementwise(const std::string& canon_text, EwMatch* m);

// in[0..n_in) follow the canonical input order (PwCanon::slot_order).
int32_t launch_dense_elementwise(int kind, int dtype, const void* const* in, void* out, unsigned long long n_elems, float k,
                                 int sm_count, cudaStream_t stream);

// out[b, n] = sum_m x[b, m, n] for a dense tensor (N a multiple of the 16-byte vector width, x
// 16-byte aligned).  With slices > 1 the kernel writes partials [(b * N + n) * slices + slice].
int32_t launch_colsum_dense(int dtype, const void* x, float* out_or_partials, unsigned batch, unsigned M, unsigned N,
                            unsigned slices, unsigned rows_per_slice, cudaStream_t stream);

// Copies a dense [rows, cols] matrix of 2-byte elements to a matrix with row pitch `dst_pitch` elements
// (dst_pitch >= cols); the padding columns are not written.  Source rows may start at any 2-byte
// address (cols odd), so reads are 2-byte accesses, coalesced along the row.
int32_t launch_pad_rows(const void* src, void* dst, long long rows, long long cols, long long dst_pitch, cudaStream_t stream);

// 8-bit copies of a matmul operand for MulF8Accum* (helium-ir/src/opgraph/op/precision.rs:60-81; the reference's
// generator converts the fragments in registers, helium-kernel-generator/src/generators/matmul/sm80.rs:317-333).
// src is [batch, rows, k] (`transposed` = false) or [batch, k, rows] (true) of f16 / bf16 / f32; dst is
// [batch, rows, k_pitch] bytes with k contiguous, each value rounded to nearest even and saturated to the
// format's largest finite value (`e5m2` != 0: E5M2, else E4M3).  The padding bytes k .. k_pitch are not written.
int32_t launch_to_f8(const void* src, int src_dtype, bool transposed, void* dst, long long batch, long long rows, long long k,
                     long long k_pitch, int e5m2, cudaStream_t stream);

}  // namespace he
