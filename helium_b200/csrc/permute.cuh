// Interface between the permute planner and the pointwise planner (which reuses the tiled
// transpose kernel for "pointwise + permutation" subgraphs).
#pragma once
#include "he_internal.h"

namespace he {

struct PermDim {
  int64_t ext, in_stride, out_stride;
};

// A permutation problem after normalisation: size-1 dims dropped, dims that stay adjacent in
// both layouts merged.  d[r-1] is the input's innermost dim (in_stride 1).
struct PermuteProblem {
  int r = 0;
  PermDim d[HE_MAX_RANK];
  int elem_bytes = 0;
  int64_t total = 0;
};

// Optional per-element function applied while the tile is loaded:
//   y = x * scale[c] + bias[c], optionally followed by max(y, 0),
// where c is the coordinate along ORIGINAL input axis `axis` (before normalisation).
struct AffineFunctor {
  bool enabled = false;
  int axis = 0;        // original input axis the parameters vary along
  int x_dtype = HE_BF16;
  int scale_dtype = HE_F32, bias_dtype = HE_F32;
  bool has_scale = true, has_bias = true, relu = true;
  int scale_input = -1, bias_input = -1;  // which he_launch input slots hold them
  int x_input = 0;
};

// Validates (shape, out_strides) as a dense permutation and normalises it.
int32_t normalize_permutation(int rank, const int64_t* in_shape, const int64_t* out_strides,
                              int elem_bytes, PermuteProblem* out, int keep_axis /*never merged, or -1*/,
                              int* axis_map /*orig axis -> norm dim or -1*/);

// Builds the plan object; `f` may be null.
int32_t make_permute_plan(he_ctx* ctx, int rank, const int64_t* in_shape, const int64_t* out_strides,
                          int32_t dtype, const AffineFunctor* f, he_plan** out);

}  // namespace he
