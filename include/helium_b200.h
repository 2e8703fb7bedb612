/*
 * helium_b200 -- C ABI of the B200 (sm_100a) fused-kernel library that sits behind helium's
 * `Backend` / `Instruction` traits.
 *
 * Every entry point takes plain pointers and sizes.  Device pointers are raw CUdeviceptr values
 * of dense row-major tensors (helium aligns tensor storage to 64 bytes,
 * helium/src/cuda/tensor_storage.rs:53), `cu_stream` is a CUstream / cudaStream_t cast to void*.
 * Nothing here synchronises the device: work is enqueued on the caller's stream, exactly like
 * `Instr::execute` does in the reference (helium/src/cuda/instr.rs:27-52).
 *
 * All functions returning `int32_t` return HE_OK (0) on success or a negative he_status; the
 * message of the last failure on the calling thread is available from he_last_error_string().
 * The library never aborts, traps or falls back to a CPU path.
 */
#ifndef HELIUM_B200_H
#define HELIUM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HE_MAX_RANK 8

typedef enum he_status {
  HE_OK = 0,
  HE_ERR_INVALID = -1,      /* malformed descriptor / argument                               */
  HE_ERR_UNSUPPORTED = -2,  /* well-formed but outside what the kernels implement             */
  HE_ERR_CUDA = -3,         /* a CUDA runtime / driver call failed (message has the detail)    */
  HE_ERR_WORKSPACE = -4,    /* workspace pointer missing or too small                          */
  HE_ERR_DEVICE_TIMEOUT = -5, /* a bounded device-side wait gave up (see he_ctx_poll_device_status) */
  HE_ERR_COMM = -6,          /* NCCL is missing or reported an error; the communicator may have been aborted */
  HE_ERR_COMM_TIMEOUT = -7   /* a communicator call did not complete by its deadline; the communicator was aborted */
} he_status;

/* Mirrors helium_ir::data_type::DataType (helium-ir/src/data_type.rs:9-24).
 * HE_BOOL is bit-packed, 1 bit per element in little-endian u32 words, LSB first
 * (helium/src/cuda/instr/pointwise/jit.rs:107-114,234-237). */
typedef enum he_dtype { HE_F16 = 0, HE_BF16 = 1, HE_F32 = 2, HE_U32 = 3, HE_BOOL = 4 } he_dtype;

/* Node kinds: the helium-ir `Op` enum (helium-ir/src/opgraph/op.rs:15-30) minus the convolutions,
 * plus HE_OP_INPUT for tensors that enter the subgraph from outside. */
typedef enum he_op_kind {
  HE_OP_INPUT = 0,
  HE_OP_CONSTANT = 1,   /* op.rs:469-474   value in const_bits (bit pattern of `dtype`)          */
  HE_OP_UNARY = 2,      /* op.rs:285-304   sub_op = he_unary_op                                   */
  HE_OP_BINARY = 3,     /* op.rs:308-328   sub_op = he_binary_op; result dtype = lhs dtype         */
  HE_OP_CAST = 4,       /* op.rs:331-335   ChangeDataType                                          */
  HE_OP_REDUCE = 5,     /* op.rs:338-356   sub_op = he_reduce_op; axes = bitmask of reduced dims   */
  HE_OP_BROADCAST = 6,  /* op.rs:369-395   input left-padded with 1s to `rank`, then axes widened  */
  HE_OP_RESHAPE = 7,    /* op.rs:409-413                                                           */
  HE_OP_SWAP_DIMS = 8,  /* op.rs:415-420   axis_a, axis_b                                          */
  HE_OP_COMPARE = 9,    /* op.rs:422-437   sub_op = he_compare_op; output HE_BOOL                  */
  HE_OP_SELECT = 10,    /* op.rs:439-445   in = {lhs, rhs, selector}; selector ? rhs : lhs         */
  HE_OP_MATMUL = 11     /* op.rs:272-282   in = {a, b}; sub_op = he_precision                      */
} he_op_kind;

/* UnaryPointwiseOp (op.rs:291-304) followed by the playground-only unary ops
 * (helium-playground/src/opgraph.rs: UnaryPointwiseOp). The *_CONST ops take their constant
 * as an f32 bit pattern in const_bits. */
typedef enum he_unary_op {
  HE_UN_RECIP = 0, HE_UN_NEG, HE_UN_EXP, HE_UN_SIN, HE_UN_COS, HE_UN_TAN, HE_UN_SIGMOID,
  HE_UN_TANH, HE_UN_RELU, HE_UN_SQRT, HE_UN_LOG,
  HE_UN_GELU = 16,      /* exact erf form, the torch F.gelu default (torch_synthesizer.rs:48)     */
  HE_UN_ADD_CONST = 17, HE_UN_MUL_CONST = 18, HE_UN_POW_CONST = 19,
  HE_UN_DGELU = 20      /* d/dx gelu(x); used by backward graphs of HE_UN_GELU                     */
} he_unary_op;

/* BinaryPointwiseOp (op.rs:315-328) followed by the playground-only binary ops. */
typedef enum he_binary_op {
  HE_BIN_ADD = 0, HE_BIN_MUL, HE_BIN_POW, HE_BIN_MIN, HE_BIN_MAX, HE_BIN_AND, HE_BIN_OR, HE_BIN_XOR,
  HE_BIN_SUB = 16, HE_BIN_DIV = 17,
  HE_BIN_DRELU = 18     /* rhs > 0 ? lhs : 0  (helium-playground/src/kernel_generator.rs:409-411)  */
} he_binary_op;

typedef enum he_compare_op { HE_CMP_EQ = 0, HE_CMP_NE, HE_CMP_LT, HE_CMP_LE, HE_CMP_GT, HE_CMP_GE } he_compare_op;
typedef enum he_reduce_op { HE_RED_SUM = 0, HE_RED_MEAN, HE_RED_MAX, HE_RED_MIN } he_reduce_op;

/* helium_ir Precision (helium-ir/src/opgraph/op/precision.rs:36-81). */
typedef enum he_precision {
  HE_PREC_F32_F32 = 0,   /* MulF32AccumF32  */
  HE_PREC_TF32_F32 = 1,  /* MulTf32AccumF32 (a minimum: served with full f32 products here)        */
  HE_PREC_BF16_F32 = 2,  /* MulBf16AccumF32 */
  HE_PREC_F16_F32 = 3,   /* MulF16AccumF32  */
  HE_PREC_F16_F16 = 4,   /* MulF16AccumF16: the node's dtype is F16 (accumulator_type, precision.rs:84-96) */
  HE_PREC_F8_F32 = 5,    /* MulF8AccumF32 { mode_a, mode_b }: see HE_PREC_F8 */
  HE_PREC_F8_F16 = 6     /* MulF8AccumF16 { mode_a, mode_b }: node dtype F16 */
} he_precision;
/* F8Mode (precision.rs:100-108) of each operand rides in the upper bits of `sub_op`:
 * sub_op = HE_PREC_F8(HE_PREC_F8_F32, HE_F8_E4M3, HE_F8_E5M2).
 * The reference documents the setting as a MINIMUM (precision.rs:3-9).  This library multiplies at
 * the precision of the operand tensors (bf16 / f16 on tcgen05 with f32 accumulation, f32 on FFMA) and
 * never narrower, so the F8 and F16-accumulate requests are served above their minimum; the output
 * is rounded once to the node's dtype. */
typedef enum he_f8_mode { HE_F8_E4M3 = 0, HE_F8_E5M2 = 1 } he_f8_mode;
#define HE_PREC_KIND(sub_op) ((sub_op) & 0xff)
#define HE_PREC_F8(kind, mode_a, mode_b) ((kind) | ((mode_a) << 8) | ((mode_b) << 12))

/* One node of a subgraph, in topological order (every `in[i]` is a smaller index, or -1).
 * `shape`/`rank`/`dtype` describe the node's OUTPUT (the reference's `Descriptor`,
 * helium-ir/src/opgraph.rs:241-257).  For HE_OP_REDUCE the helium-ir form "collapse the last
 * `depth` dims into one dim of size 1" (op.rs:78-89) is axes = the last `depth` bits with
 * shape = [.., 1]; the playground forms Rows/Columns/Item/Batch
 * (helium-playground/src/opgraph.rs:397-413) keep rank 3 and set the reduced dims to 1. */
typedef struct he_node {
  int32_t kind;        /* he_op_kind */
  int32_t sub_op;      /* he_unary_op / he_binary_op / he_compare_op / he_reduce_op / he_precision */
  int32_t in[3];       /* operand node indices, -1 when unused */
  int32_t dtype;       /* he_dtype of the output */
  int32_t rank;
  int64_t shape[HE_MAX_RANK];
  uint32_t const_bits; /* HE_OP_CONSTANT value / *_CONST operand */
  int32_t axis_a;      /* HE_OP_SWAP_DIMS */
  int32_t axis_b;      /* HE_OP_SWAP_DIMS */
  uint32_t axes;       /* HE_OP_REDUCE: bitmask over the INPUT's dims */
} he_node;

/* Flat mirror of `OpSubgraph` (helium-ir/src/opgraph/subgraph.rs:12-18): nodes, and the leafs
 * that become kernel outputs.  Kernel inputs are the HE_OP_INPUT nodes in order of appearance;
 * he_launch's `inputs[i]` / `outputs[j]` follow those two orders. */
typedef struct he_graph_desc {
  int32_t num_nodes;
  const he_node* nodes;
  int32_t num_outputs;
  const int32_t* outputs;
} he_graph_desc;

typedef struct he_ctx he_ctx;
typedef struct he_plan he_plan;

/* Replaces CudaContext::global (helium/src/cuda/context.rs:50-69) for the purposes of this
 * library: binds to `device_ordinal`'s primary context, queries SM count / smem limits and
 * allocates one 64-byte device status block used by bounded device-side waits. */
int32_t he_ctx_create(int32_t device_ordinal, he_ctx** out);
void he_ctx_destroy(he_ctx* ctx);
/* Plans created after this call size their persistent grids for (SM count - sms) SMs.  For a kernel that
 * is meant to run beside other work on the same GPU -- the GEMM that overlaps a gradient all-reduce whose
 * communicator was created with `max_ctas` = sms: a persistent grid that claims every SM would have
 * some of its CTAs wait for the collective's to retire.  0 restores the full device.  Existing plans keep
 * the grid they were planned with.  No counterpart in the reference (one stream, one kernel at a time). */
int32_t he_ctx_reserve_sms(he_ctx* ctx, int32_t sms);
/* Reads (synchronously, after syncing `cu_stream`) and clears the device status word.
 * Returns HE_OK or HE_ERR_DEVICE_TIMEOUT; detail in he_last_error_string(). */
int32_t he_ctx_poll_device_status(he_ctx* ctx, void* cu_stream);

/* Replaces PointwiseGraph::{precompile,get_kernel} (helium/src/cuda/instr/pointwise.rs:40-54) and
 * pointwise::jit::generate_kernel (pointwise/jit.rs:19-121).  Accepts what `supports_subgraph`
 * accepts (pointwise.rs:121-186) and, beyond it, any number of swap_dims / broadcasts. */
int32_t he_plan_pointwise(he_ctx* ctx, const he_graph_desc* desc, he_plan** out);

/* Replaces PermuteDims::{precompile,build_kernel} (helium/src/cuda/instr/permute_dims.rs:55-83)
 * and permute_dims::jit::generate_kernel (permute_dims/jit.rs:15-117): out[sum_i out_strides[i] *
 * c[i]] = in[c] for every coordinate c of the row-major input of shape `in_shape`.
 * `out_strides[i]` is the stride, in elements, that INPUT axis i has in the output
 * (permute_dims.rs:158-172).  dtype may be F16/BF16/F32/U32. */
int32_t he_plan_permute(he_ctx* ctx, int32_t rank, const int64_t* in_shape,
                        const int64_t* out_strides, int32_t dtype, he_plan** out);

/* Host helper replacing compute_output_strides (permute_dims.rs:158-172).  `swaps` holds
 * num_swaps (axis_a, axis_b) pairs applied in order.  With reference_compat = 0 the strides
 * realise the composition of the swaps (what the IR's output shape describes, op.rs:102-110).
 * With reference_compat = 1 they reproduce the reference function verbatim, which yields the
 * INVERSE permutation for chains that are not their own inverse (its unit test
 * permute_dims.rs:183-187 pins exactly that). */
int32_t he_permute_output_strides(int32_t rank, const int64_t* in_shape, int32_t num_swaps,
                                  const int32_t* swaps, int32_t reference_compat,
                                  int64_t* out_strides);

/* Replaces MatmulGenerator::new + generate (helium-kernel-generator/src/generators/matmul.rs:
 * 88-153) and the playground's KernelGenerator (helium-playground/src/kernel_generator.rs:51-117):
 * one HE_OP_MATMUL node, mainloop pointwise ops on the operand side, epilogue pointwise /
 * broadcast / Sum-reduction ops on the result side.  Shapes are [.., M, K] x [.., K, N] row-major
 * (op.rs:272-282); a SWAP_DIMS of the last two dims feeding an operand selects the transposed
 * shared-memory descriptor instead of moving data. */
int32_t he_plan_fused_matmul(he_ctx* ctx, const he_graph_desc* desc, he_plan** out);
/* Environment switches read at plan time (benchmarks and comparisons only):
 *   HE_GEMM_ONE_CTA=1         one CTA per 128 x 256 tile instead of CTA pairs on 256 x 256 tiles
 *   HE_GEMM_GROUP_M=<n>       row tiles per rasterisation group
 *   HE_GEMM_NO_SPLIT=1        never run the tiles of an under-filled last round as half-width tiles
 *   HE_GEMM_MAINLOOP=fused|materialise   force how a mainloop fusion is executed
 *   HE_GEMM_K_SERPENTINE=0    every tile walks K forwards (default: every other tile of a CTA pair backwards)
 * None of them changes results.
 *   HE_GEMM_F8=native|operand  MulF8Accum* requests: always / never multiply 8-bit copies of the operands with
 *                             tcgen05 kind::f8f6f4 (default: from 4 GFLOP per launch).  This one does change results,
 *                             within what the precision contract allows (precision.rs:3-9). */

/* Backs Instruction::can_fuse_with (helium/src/backend.rs:85-95): 0 = cannot run as one kernel,
 * 1 = runs through a generic tier (pointwise: a kernel specialised at plan time with NVRTC when the program
 * has no bool tensor in memory and the NVRTC library can be loaded -- HE_NVRTC_LIBRARY names it, HE_PW_JIT=0 switches the tier off
 * -- else the register-program interpreter), 2 = matches a hand-written fast kernel.
 * kind: 0 pointwise, 1 permute (swap chain on one input), 2 fused matmul. */
int32_t he_plan_supported(he_ctx* ctx, const he_graph_desc* desc, int32_t kind);

/* Scratch the launch needs (caller-allocated from its stream allocator with 256-byte alignment,
 * like the cuDNN workspace in helium/src/cuda/instr/cudnn_graph.rs:75-92).  It holds the per-tile
 * partials of fused reductions and, when a mainloop fusion is executed by a pre-pass, the
 * materialised A operand (batch * M * K elements); contents are undefined between launches. */
int32_t he_plan_workspace_bytes(const he_plan* plan, size_t* out);

/* Replaces {PointwiseGraph,PermuteDims,CudnnGraph}::execute (pointwise.rs:57-86,
 * permute_dims.rs:33-53, cudnn_graph.rs:64-105).  Pre-filling of reduction / bool outputs
 * (pointwise.rs:62-74) happens inside, on the same stream. */
/* Every he_launch, heh_exec_run and he_allreduce_grads call is wrapped in an NVTX range named after the plan
 * (header-only NVTX v3: one indirect call when no tool is attached; HE_NVTX=0 switches the ranges off). */
int32_t he_launch(he_plan* plan, const void* const* inputs, void* const* outputs,
                  void* workspace, void* cu_stream);

/* Number of kernels (not memsets) the last he_launch of this plan enqueued. */
int32_t he_plan_last_launch_count(const he_plan* plan);
/* Short human-readable description of the kernel tier / tile configuration chosen. */
const char* he_plan_describe(const he_plan* plan);
void he_plan_destroy(he_plan* plan);

/* ------------------------------------------------------------------------------------------------
 * Host runtime: a C++ mirror of the pieces of helium that sit between a recorded op graph and the
 * three calls above, so that whole graphs can be driven without the Rust front end:
 *   OpGraph / OpSubgraph          helium-ir/src/opgraph.rs:12-191, opgraph/subgraph.rs:12-120
 *   Backend::make_instr_for_op    helium/src/cuda.rs:33-60 (Op::Matmul goes to the fused matmul)
 *   Instruction::can_fuse_with    helium/src/cuda/instr.rs:71-99, backed by he_plan_supported
 *   generate_plan                 helium/src/backend/plan_generation.rs:22-26,195-321,325-416
 *   BackendExt::execute_graph     helium/src/backend.rs:40-80, with the steps' instructions issued
 *                                 on several streams (the reference's executor uses one,
 *                                 helium/src/cuda.rs:117-118) and the plan optionally captured in a
 *                                 CUDA graph.
 * Node ids are the values returned by heh_graph_new_*; `op->in[]` holds node ids of this graph.
 * ------------------------------------------------------------------------------------------------ */
typedef struct heh_graph heh_graph;
typedef struct heh_exec heh_exec;

int32_t heh_graph_create(heh_graph** out);
void heh_graph_destroy(heh_graph* g);
/* OpGraph::new_input (opgraph.rs:73-85). */
int32_t heh_graph_new_input(heh_graph* g, int32_t dtype, int32_t rank, const int64_t* shape, int32_t* node_out);
/* OpGraph::new_op (opgraph.rs:87-110): `op` carries kind / sub_op / operands / attributes and the
 * output descriptor, which is validated against Op::output_descriptor's rules. */
int32_t heh_graph_new_op(heh_graph* g, const he_node* op, int32_t* node_out);
/* OpGraph::new_output (opgraph.rs:112-125): marks `node` as a value the caller wants back. */
int32_t heh_graph_new_output(heh_graph* g, int32_t node);

/* Plans the graph (instruction per op, greedy pairwise fusion, Kahn-layered steps, delayed
 * instructions, tensor release points) and writes a human-readable listing: one line per
 * instruction "step <i> <Kind> tier=<t> nodes=[..] in=[..] out=[..]". */
int32_t heh_graph_plan_text(he_ctx* ctx, heh_graph* g, char* buf, size_t cap);

/* Chooses how instructions are formed from nodes.  mode 0 (default): the greedy pairwise merging of
 * plan_generation.rs:243-256.  mode 1: the fusion search, the counterpart of the playground's
 * (helium-playground/src/fused_graph.rs:113-223,285-593 states and moves, subdivision.rs:24-113,
 * cost_model.rs:241-343): kernels are grown from single nodes by absorbing consumers into a kernel's
 * result side, producers into its result side (recomputation instead of a read) or into a matmul's
 * operand side, and by handing the export of a recomputed node from one kernel to another; a state is
 * legal only if he_plan_supported accepts every kernel, its cost is an estimate fitted to this
 * library's kernels on a B200, and the descent looks `depth` moves ahead (0 keeps 3) over at most
 * `max_states` states per subdivision (0 keeps 12000).  heh_graph_plan_text and heh_exec_create use
 * the chosen planner.  The environment variable HE_PLANNER=search makes mode 1 the default of graphs
 * created afterwards. */
int32_t heh_graph_set_planner(heh_graph* g, int32_t mode, int32_t depth, int32_t max_states);
/* Runs the fusion search and writes its result: a first line "cost identity=<s> maximal=<s>
 * pairwise=<s> best=<s> states=<n> subdivisions=<n> recomputed=<n>" (estimated seconds with one kernel
 * per node, after the greedy start, for the plan of the pairwise planner -- which seeds a descent of
 * its own, so best <= pairwise; -1 if that plan writes an operand-side value to memory and is no state
 * of the search -- and for the result), then one line per kernel in a topological order:
 * "group <i> FusedMatmul|Pointwise anchor=<node|-1> pre=[..] post=[..] in=[..] out=[..] seconds=<s>". */
int32_t heh_graph_search_text(he_ctx* ctx, heh_graph* g, char* buf, size_t cap);
/* subdivide (subdivision.rs:24-113): one line per subdivision, its nodes in ascending order; a matmul
 * node carries "m" where the subdivision holds its operand (mainloop) side and "e" for its result
 * (epilogue) side. */
int32_t heh_graph_subdivisions_text(heh_graph* g, char* buf, size_t cap);

/* Prepares an execution: plans, creates every he_plan, allocates intermediates and workspaces
 * once, binds the caller's device buffers (`inputs[i]` for the i-th new_input, `outputs[j]` for the
 * j-th new_output) and, if `capture_cuda_graph` != 0, records the whole plan into a CUDA graph.
 * Before recording, the plan runs once eagerly (one-time kernel set-up must not happen inside a
 * capture): that pass READS the caller's input buffers, which must therefore hold readable memory
 * already, and writes to temporary copies of the output buffers, so creating an executor never
 * changes the caller's outputs -- an output may alias live state such as a weight updated in place.
 * A node listed twice as an output is refused (HE_ERR_UNSUPPORTED).  The calling thread's current
 * device is left as it was.  heh_exec_run enqueues one evaluation on `cu_stream`. */
int32_t heh_exec_create(he_ctx* ctx, heh_graph* g, const void* const* inputs, void* const* outputs,
                        int32_t capture_cuda_graph, heh_exec** out);
int32_t heh_exec_run(heh_exec* e, void* cu_stream);
/* Kernels launched per run, number of steps, number of instructions after fusion. */
int32_t heh_exec_stats(const heh_exec* e, int32_t* launches, int32_t* steps, int32_t* instrs);
void heh_exec_destroy(heh_exec* e);

/* Introspection for tests (no counterpart in the reference, whose generated CUDA source is
 * inspected through insta snapshots instead, helium/src/cuda/instr/pointwise/jit.rs:752-803).
 * he_debug_dump_program lowers a subgraph to the interpreter program and copies the raw PwProgram
 * struct (layout: helium_b200/csrc/pointwise_program.h) into `buf`; `epilogue` != 0 treats the
 * graph's matmul node as the accumulator source, like the generic fused-matmul tier does.
 * he_debug_canonical_text returns the canonical text the kernel catalogue is matched on. */
int32_t he_debug_dump_program(const he_graph_desc* desc, int32_t epilogue, void* buf, size_t cap,
                              size_t* size_out);
int32_t he_debug_canonical_text(const he_graph_desc* desc, char* buf, size_t cap);

/* ------------------------------------------------------------------------------------------------
 * 2-D convolution as implicit GEMM on the tcgen05 core.  Replaces the cuDNN graphs the reference builds
 * for Op::Conv, Op::ConvBackwardData and Op::ConvBackwardFilter (helium/src/cuda/instr/cudnn_graph.rs:
 * 182-228).  Images are NHWC, filters KRSC (helium/src/raw_tensor.rs:232-240); geometry follows
 * Conv2dParams (helium-ir/src/opgraph/op/conv.rs:5-95): output size = input size adjusted by the padding
 * mode and divided by the stride, zero padding k/2 (Same), 0 (Valid), k-1 (Full) on both sides.
 * Implemented: bf16 / f16 tensors with f32 accumulation, dilation 1, strides 1x1 and 2x2, up to 49 taps,
 * channel counts that are multiples of 8 (a 16-byte pixel pitch; pad narrower images, e.g. RGB to 8).
 *
 * he_launch operands, in order:
 *   HE_CONV_FWD         inputs  image [N,H,W,C], filter [K,R,S,C] (, bias [K]) (, resid [N,P,Q,K])
 *                       outputs y [N,P,Q,K] (, stats f32 [2,K])
 *   HE_CONV_BWD_DATA    inputs  flow [N,P,Q,K], filter [K,R,S,C] (, resid [N,H,W,C])
 *                               (, gate_x [N,H,W,C], gate_scale f32 [C], gate_shift f32 [C])
 *                       outputs dx [N,H,W,C] (, stats f32 [2,C])
 *   HE_CONV_BWD_FILTER  inputs  flow [N,P,Q,K], image [N,H,W,C];  output dw [K,R,S,C]
 * Fused epilogue of the first two (he_conv2d_fusion): t = acc + bias[col] + resid[pix, col]; with a gate,
 * t = (gate_x[pix, col] * gate_scale[col] + gate_shift[col] > 0) ? t : 0 -- the backward of a rectified
 * batch-norm output; out = t; stats = per-column sums over all pixels of t and of t * t (or of
 * t * gate_x with a gate): the batch statistics of helium's BatchNorm2d (helium/src/modules/batch_norm.rs:
 * 38-65) in the forward direction, and the two sums its backward needs in the other.
 * ------------------------------------------------------------------------------------------------ */
typedef enum he_conv_kind { HE_CONV_FWD = 0, HE_CONV_BWD_DATA = 1, HE_CONV_BWD_FILTER = 2 } he_conv_kind;
typedef enum he_padding_mode { HE_PAD_SAME = 0, HE_PAD_VALID = 1, HE_PAD_FULL = 2 } he_padding_mode;   /* conv.rs:77-83 */
typedef struct he_conv2d_params {   /* Conv2dParams, conv.rs:5-12 */
  int32_t in_channels, out_channels;
  int32_t kernel_h, kernel_w;
  int32_t stride_h, stride_w;
  int32_t dilation_h, dilation_w;
  int32_t padding_mode;
} he_conv2d_params;
typedef struct he_conv2d_fusion {
  int32_t out_dtype;     /* dtype of the output tensor (F16 / BF16 / F32) */
  int32_t has_bias;      /* bias vector over output channels */
  int32_t bias_dtype;
  int32_t has_resid;     /* tensor of the output's shape and the operands' dtype, added */
  int32_t has_gate;      /* rectifier mask recomputed from gate_x, gate_scale, gate_shift */
  int32_t want_stats;    /* second output: f32 [2, columns] */
} he_conv2d_fusion;
/* `in_h`, `in_w`: spatial size of the IMAGE (for the gradients too); `fusion` may be NULL (plain store in
 * `dtype`).  A strided data gradient whose filter leaves some input pixels untouched (1x1 with stride 2)
 * zero-fills the output first and accepts no fusion. */
int32_t he_plan_conv2d(he_ctx* ctx, int32_t kind, const he_conv2d_params* params, int32_t batch, int32_t in_h,
                       int32_t in_w, int32_t dtype, const he_conv2d_fusion* fusion, he_plan** out);

/* ------------------------------------------------------------------------------------------------
 * Hand-written kernels for the pointwise / reduction chains of a convolutional training step.  In the
 * reference each is a chain of generic pointwise and reduce instructions over broadcast views of
 * channels-last tensors; here each remaining pass over an activation is one HBM-bound kernel.  All tensors
 * are bf16 [pixels, channels] (NHWC flattened) with channels a multiple of 8, 16-byte aligned; per-channel
 * vectors are f32.  Everything is enqueued on `cu_stream`; sums are folded in a fixed order.
 * ------------------------------------------------------------------------------------------------ */
/* BatchNorm2d::forward in train mode (helium/src/modules/batch_norm.rs:38-65) from the sums a convolution's
 * epilogue (or he_bn_apply) produced: stats = [sum x, sum x^2] per channel over `count` values.  Writes
 * scale = gamma * rstd, shift = beta - mean * scale, mean and rstd = 1 / sqrt(E[x^2] - mean^2 + 1e-3), and
 * updates the running statistics in place (x 0.9 + 0.1 x new; either may be NULL). */
int32_t he_bn_finalize(const float* stats, int64_t count, const float* gamma, const float* beta, float* running_mean,
                       float* running_var, float* scale, float* shift, float* mean, float* rstd, int32_t channels,
                       void* cu_stream);
/* y = x * scale[c] + shift[c], rectified when `relu` != 0 (batch_norm.rs:60-70 followed by tensor.rs:374-387).
 * With `stats_out` (f32 [2, channels]) the sums of y and y^2 as stored are produced as well, for a second
 * normalisation of the same tensor; that needs he_bn_workspace_bytes(pixels, channels) of workspace. */
size_t he_bn_workspace_bytes(int64_t pixels, int32_t channels);
int32_t he_bn_apply(const void* x, void* y, const float* scale, const float* shift, int64_t pixels, int32_t channels,
                    int32_t relu, float* stats_out, void* workspace, void* cu_stream);
/* Backward of the normalisation.  stats = [sum g, sum g x] per channel, with g the gradient at the normalised
 * (and rectifier-masked) output and x the normalised tensor -- the second output of an HE_CONV_BWD_DATA plan with
 * a gate.  Writes dgamma, dbeta and coef = [A, B, K] (f32 [3, channels]) such that dx = A g + B x + K. */
int32_t he_bn_backward_coeffs(const float* stats, int64_t count, const float* gamma, const float* mean, const float* rstd,
                              float* coef, float* dgamma, float* dbeta, int32_t channels, void* cu_stream);
/* out = coef.A[c] g + coef.B[c] x + coef.K[c] (+ addend).  With `mask_x` the result is zeroed where
 * mask_x * mask_scale[c] + mask_shift[c] <= 0 (a rectified normalisation in front of this one) and
 * stats_out = [sum out, sum out * mask_x] is produced (workspace as for he_bn_apply).  Without a mask, a non-null
 * stats_out receives f32 [channels] column sums of `out` as stored -- the bias gradient of the convolution that
 * `out` enters next, which the reference computes with a separate reduction -- and needs the same workspace. */
int32_t he_bn_backward_apply(const void* g, const void* x, const void* addend, void* out, const float* coef,
                             const void* mask_x, const float* mask_scale, const float* mask_shift, float* stats_out,
                             void* workspace, int64_t pixels, int32_t channels, void* cu_stream);
/* out = a + b on bf16 tensors of n elements (gradient branches meeting at a fork). */
int32_t he_add_bf16(const void* a, const void* b, void* out, int64_t n, void* cu_stream);
/* out[c] = sum over pixels of x[pixel, c]: the gradient of a convolution's bias (workspace as for he_bn_apply). */
int32_t he_colsum_bf16(const void* x, float* out, void* workspace, int64_t pixels, int32_t channels, void* cu_stream);
/* Sgd::step with momentum (helium/src/optimizer/sgd.rs:47-62): avg = first_step ? g : g (1 - m) + avg m;
 * w -= lr * avg; `w_bf16` (may be NULL) receives the updated weights rounded to bf16, the copy the next
 * step's convolutions read (helium/src/modules/conv.rs:63).  `avg` may be NULL for plain SGD (momentum 0). */
int32_t he_sgd_momentum(float* w, float* avg, const void* grad, int32_t grad_dtype, void* w_bf16, int64_t n, float lr,
                        float momentum, int32_t first_step, void* cu_stream);
/* Patch matrix of a 'Same'-padded convolution over a thin NHWC tensor (any channel count, e.g. RGB):
 * cols[n, p, q, (r * S + s) * C + c] = x[n, p * stride + r - R/2, q * stride + s - S/2, c], zero outside the image and
 * in the padding columns up to `pitch` (a multiple of 8).  The result, seen as an NHWC tensor with `pitch` channels,
 * goes through he_plan_conv2d as a 1 x 1 convolution whose filter is the original one reshaped to [K, 1, 1, pitch]:
 * the route for a stem whose 3 input channels cannot feed the tensor core from the image directly. */
int32_t he_im2col_nhwc(const void* x, void* cols, int32_t batch, int32_t in_h, int32_t in_w, int32_t channels, int32_t kernel_h,
                       int32_t kernel_w, int32_t stride, int32_t pitch, void* cu_stream);
/* Global average pooling + cross entropy (resnet-train/src/model.rs:77-82, helium/src/loss.rs:5-8): logits =
 * mean over `positions` of y[n, position, :], loss[n] = -log_softmax(logits)[labels[n]] / batch, and dy = the
 * gradient of sum(loss) at y (bf16, same shape). */
int32_t he_pool_softmax_ce(const void* y, const int32_t* labels, float* loss, void* dy, int32_t batch, int32_t positions,
                           int32_t classes, void* cu_stream);

/* ------------------------------------------------------------------------------------------------
 * Data-parallel gradient exchange.  No counterpart in the reference, which runs on one GPU: its
 * optimiser consumes whatever gradient tensors it is handed (helium/src/optimizer/sgd.rs:35-62).  A
 * data-parallel host calls he_allreduce_grads between `backward()` and `Optimizer::step`, once per
 * bucket of gradients, on a stream of its choice so that the exchange overlaps the remaining backward
 * kernels.  One process (or thread) per GPU; NCCL is loaded at run time (dlopen of the copy already in
 * the process, else libnccl.so.2; HE_NCCL_LIBRARY overrides the name).
 *
 * Failure handling is on the host: the communicator is non-blocking, every call below polls
 * ncclCommGetAsyncError against a deadline, and a call that misses its deadline (a peer that never
 * joined) or meets an NCCL error aborts the communicator (ncclCommAbort) and returns HE_ERR_COMM_TIMEOUT
 * / HE_ERR_COMM; afterwards only he_comm_destroy is valid.  Nothing here can wait for ever.
 * ------------------------------------------------------------------------------------------------ */
typedef struct he_comm he_comm;
#define HE_COMM_UNIQUE_ID_BYTES 128
/* Rank 0 calls this and hands the 128 bytes to every rank by any channel it has (a file, a socket, an
 * existing process group). */
int32_t he_comm_unique_id(void* id_out);
/* `ctx` selects the device (NULL: the calling thread's current device).  `max_ctas` > 0 caps the CTAs a
 * collective may occupy (ncclConfig_t::maxCTAs) so that a persistent GEMM launched next to it can be given
 * the remaining SMs; 0 leaves NCCL's default.  `timeout_ms` bounds this call and becomes the default
 * deadline of the later ones (0: 30 s). */
int32_t he_comm_create(he_ctx* ctx, int32_t rank, int32_t world, const void* unique_id, int32_t max_ctas,
                       int32_t timeout_ms, he_comm** out);
int32_t he_comm_info(const he_comm* comm, int32_t* rank, int32_t* world, int32_t* max_ctas);
/* In-place sum (mean != 0: mean) over ranks of n device buffers of `dtype` (F16 / BF16 / F32), enqueued on
 * `cu_stream` as one NCCL group.  The first call with a given layout (n, counts, dtype, mean) checks that
 * every rank passed the same layout -- a 16-byte collective whose result is read back before anything
 * else is enqueued; a mismatch returns HE_ERR_INVALID on the ranks that differ from the others and no
 * gradient is touched.  Later calls with that layout enqueue and return. */
int32_t he_allreduce_grads(he_comm* comm, void* const* bufs, const size_t* counts, int32_t n, int32_t dtype,
                           int32_t mean, void* cu_stream);
/* HE_OK while the communicator is healthy (idle or busy), HE_ERR_COMM once NCCL has reported an
 * asynchronous error or the communicator was aborted.  Cheap; meant to be called once per step. */
int32_t he_comm_poll(he_comm* comm);
int32_t he_comm_abort(he_comm* comm);
void he_comm_destroy(he_comm* comm);

/* Host-side fault injection for the bounded device waits of the tensor-core matmul kernels (no
 * counterpart in the reference, whose kernels have no such waits).  Every mbarrier wait in those
 * kernels gives up after `wait_limit_us` microseconds (0 restores the default of 2 s), records the wait
 * site in the context's status block and lets the kernel finish through its normal teardown; with
 * `withhold_loads` != 0 the kernel's TMA producers issue nothing, so the first wait for operands is
 * certain to run into the limit.  A launch of such a plan returns HE_OK (the failure happens on the
 * device), writes undefined results, and the next he_ctx_poll_device_status returns
 * HE_ERR_DEVICE_TIMEOUT; the context stays usable.  Plans without device-side waits (pointwise,
 * permute, SIMT matmul) return HE_ERR_UNSUPPORTED. */
int32_t he_debug_plan_fault_injection(he_plan* plan, uint32_t wait_limit_us, int32_t withhold_loads);

/* Sum over the trailing dims of an f32 tensor viewed as [num_groups, group_size], written to
 * out[num_groups], with no workspace argument and no device allocation by anyone.
 *
 * No counterpart in the reference.  It is here for callers that have no way to hand a kernel
 * scratch memory: a body for `PointwiseGraph::execute(tensors, stream, cx)`
 * (helium/src/cuda/instr/pointwise.rs:57) is given tensors and a stream but, unlike the cuDNN
 * instruction (helium/src/cuda/instr.rs:27-52), no allocator handle, and it must not call
 * cudaMalloc itself because that stalls the device and bypasses the executor's stream-ordered
 * pool.  he_launch needs a caller workspace once a reduction group is split over several CTAs;
 * this call keeps those partial sums in a fixed array inside the library instead.
 *
 * Limits and rules:
 *  - the array holds HE_NOALLOC_MAX_PARTIALS floats (256 KiB of device memory on every GPU the
 *    process uses this library on, for the life of the process).  A shape that needs more partial
 *    sums -- num_groups * ceil(group_size / 4096) when group_size > 4096 -- is refused with
 *    HE_ERR_WORKSPACE and a message naming both numbers; num_groups * group_size must be < 2^31;
 *  - the first call on each device looks the array's address up (a CUDA runtime query, no
 *    allocation).  Make that first call before starting any stream capture on that device;
 *  - all calls on a device share the one array, which keeps whatever the previous call left.
 *    Nothing in it has to start at zero: every partial is written by the call before the call reads
 *    it.  Two calls that can run at the same time (different streams, or different host threads
 *    on different streams) race on it; order them on one stream or with events;
 *  - the summation order is fixed, so results repeat bit for bit; they agree with he_launch's to
 *    f32 rounding (he_launch may slice a group differently).  `in` and `out` are device pointers
 *    on the current device. */
#define HE_NOALLOC_MAX_PARTIALS 65536
int32_t he_reduce_sum_f32_noalloc(const float* in, float* out, int64_t num_groups, int64_t group_size,
                                  void* cu_stream);

const char* he_last_error_string(void);
const char* he_version(void);

#ifdef __cplusplus
}
#endif
#endif /* HELIUM_B200_H */
