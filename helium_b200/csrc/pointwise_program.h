// The compact per-kernel program the pointwise interpreter executes, and the host-side compiler
// that lowers a validated subgraph to it.  Used by the stand-alone pointwise kernels and by the
// generic epilogue tier of the fused matmul.
#pragma once
#include "device_utils.cuh"
#include "he_internal.h"

namespace he {

constexpr int kPwMaxInstr = 160;
constexpr int kPwMaxViews = 24;
constexpr int kPwMaxViewDims = 8;
constexpr int kPwMaxInputs = 16;
constexpr int kPwMaxOutputs = 8;
constexpr int kPwMaxRegs = 32;

enum PwOp : uint8_t {
  PW_LOAD = 0,   // dst <- input[slot] at (view chain applied to the element index); dt = he_dtype
  PW_CONST,      // dst <- imm (f32 / u32 bits, or 0/1 for bool)
  PW_UNARY,      // dst <- f(a); sub = he_unary_op; imm = constant operand of *_CONST
  PW_BIN_F,      // float binary; sub = he_binary_op
  PW_BIN_U,      // u32 binary
  PW_BIN_B,      // bool binary (and/or/xor)
  PW_FMA,        // dst <- fmaf(a, b, c)
  PW_CMP_F,      // sub = he_compare_op
  PW_CMP_U,
  PW_SELECT,     // dst <- c ? b : a
  PW_CVT,        // class conversion; sub = (from_class << 2 | to_class), classes 0 float 1 int 2 bool
  PW_MEAN_SCALE, // dst <- (float)((double)a * scale); scale = reduce_mean_scale of the program
  PW_STORE,      // output[slot] <- a; dt = he_dtype
  PW_REDUCE,     // accumulate a into reduction `slot2`; sub = he_reduce_op; output slot = slot
  PW_ACC         // dst <- the matmul accumulator value (fused-matmul epilogue programs only)
};

struct PwInstr {
  uint8_t op, sub, dst, a, b, c, dt, slot;
  uint32_t imm;
  uint8_t view0;   // first view of the chain
  uint8_t nviews;  // 0 = element index used as is
  uint8_t slot2;
  uint8_t pad;
};
static_assert(sizeof(PwInstr) == 16, "PwInstr layout");

// offset = sum_k ((i / prod_{j<k} ext_j) % ext_k) * stride_k, dims listed innermost first.
struct PwView {
  int nd;
  FastDiv fd[kPwMaxViewDims];
  uint32_t stride[kPwMaxViewDims];
};

struct PwProgram {
  int n_instr;
  int n_inputs, n_outputs;
  uint32_t n_elems;       // size of the iteration space
  uint32_t group_size;    // reduction group (== n_elems when there is no reduction)
  int n_reductions;
  double mean_scale;      // 1 / group_size, computed in f64 like pointwise/jit.rs:414
  const void* in[kPwMaxInputs];
  void* out[kPwMaxOutputs];
  PwInstr instr[kPwMaxInstr];
  PwView views[kPwMaxViews];
};

struct PwReduceLaunch {
  uint32_t num_groups;
  uint32_t blocks_per_group;   // CTAs per group (block mode) -- 1 in warp mode
  uint32_t chunk;              // elements of a group handled by one CTA
  int warp_mode;               // 0: CTA slices of one group; 1: one warp per group, 8 groups per CTA;
                               // 2: column mode, a lane per group, 32 groups x one slice per CTA
  int red_ops[4];
  int red_out_slot[4];
  float* partials;             // [n_red][num_groups][blocks_per_group] when blocks_per_group > 1
};

// Host-side description produced by the compiler next to the program.
struct PwLoadInfo {
  int instr;              // index into program.instr
  int input_slot;
  int node;               // graph node of the input
  bool single_view;       // whole mapping collapsed into one view over the iteration space
  bool identity;          // element index used directly
  // per iteration-space dim (outermost first, rank = iter_rank): stride into the input tensor
  int64_t iter_stride[HE_MAX_RANK];
};

struct PwCompiled {
  PwProgram prog;
  int iter_rank = 0;
  int64_t iter_shape[HE_MAX_RANK] = {0};
  std::vector<PwLoadInfo> loads;
  std::vector<int> out_dtypes;     // per output slot
  std::vector<int> out_is_reduce;  // per output slot: -1 or he_reduce_op
  bool has_bool_io = false;        // any bool load or store (forces 1 element / thread)
  int n_regs = 0;
};

struct PwCompileOptions {
  int acc_node = -1;        // node whose value the caller supplies per element (PW_ACC): the matmul
  bool fuse_fma = true;     // contract mul+add (off when the program is only used for matching)
  bool epilogue = false;    // fused-matmul epilogue: reductions over any axes are accepted as leaves
                            // (PW_REDUCE.imm = axes bitmask: bit 0 columns dim, bit 1 rows dim, bit 2 batch)
};

// Lowers `g` (only pointwise-family ops) to a program.
int32_t compile_pointwise(const Graph& g, const PwCompileOptions& opt, PwCompiled* out);

// Canonical, input-order-independent text of a compiled program (fuse_fma = false), used to match
// subgraphs against the catalogue of hand-written kernels.  `slot_order[k]` = graph input slot of
// canonical input k; `out_order[k]` = caller output index of canonical output k.
struct PwCanon {
  std::string text;
  std::vector<int> slot_order;
  std::vector<int> out_order;
};
int32_t canonicalize_program(const Graph& g, const PwCompiled& c, int rows_dim_m, int cols_dim_n, PwCanon* out);

}  // namespace he
