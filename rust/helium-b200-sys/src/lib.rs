//! NOT COMPILED in this repository's build image (no Rust toolchain); see ../../README.md.
//!
//! `#[repr(C)]` mirror of include/helium_b200.h.  Enum values are spelled as constants because the C
//! side takes plain `int32_t`s.
#![allow(non_camel_case_types)]
use std::os::raw::{c_char, c_void};

pub const HE_MAX_RANK: usize = 8;

// he_status
pub const HE_OK: i32 = 0;
pub const HE_ERR_INVALID: i32 = -1;
pub const HE_ERR_UNSUPPORTED: i32 = -2;
pub const HE_ERR_CUDA: i32 = -3;
pub const HE_ERR_WORKSPACE: i32 = -4;
pub const HE_ERR_DEVICE_TIMEOUT: i32 = -5;
pub const HE_ERR_COMM: i32 = -6;
pub const HE_ERR_COMM_TIMEOUT: i32 = -7;

// he_dtype (helium_ir::data_type::DataType)
pub const HE_F16: i32 = 0;
pub const HE_BF16: i32 = 1;
pub const HE_F32: i32 = 2;
pub const HE_U32: i32 = 3;
pub const HE_BOOL: i32 = 4;

// he_op_kind (helium_ir::opgraph::op::Op)
pub const HE_OP_INPUT: i32 = 0;
pub const HE_OP_CONSTANT: i32 = 1;
pub const HE_OP_UNARY: i32 = 2;
pub const HE_OP_BINARY: i32 = 3;
pub const HE_OP_CAST: i32 = 4;
pub const HE_OP_REDUCE: i32 = 5;
pub const HE_OP_BROADCAST: i32 = 6;
pub const HE_OP_RESHAPE: i32 = 7;
pub const HE_OP_SWAP_DIMS: i32 = 8;
pub const HE_OP_COMPARE: i32 = 9;
pub const HE_OP_SELECT: i32 = 10;
pub const HE_OP_MATMUL: i32 = 11;

// he_precision (helium_ir::opgraph::op::precision::Precision)
pub const HE_PREC_F32_F32: i32 = 0;
pub const HE_PREC_TF32_F32: i32 = 1;
pub const HE_PREC_BF16_F32: i32 = 2;
pub const HE_PREC_F16_F32: i32 = 3;
pub const HE_PREC_F16_F16: i32 = 4;
pub const HE_PREC_F8_F32: i32 = 5;
pub const HE_PREC_F8_F16: i32 = 6;
pub const fn he_prec_f8(kind: i32, mode_a: i32, mode_b: i32) -> i32 { kind | (mode_a << 8) | (mode_b << 12) }

#[repr(C)]
#[derive(Copy, Clone)]
pub struct he_node {
    pub kind: i32,
    pub sub_op: i32,
    pub r#in: [i32; 3],
    pub dtype: i32,
    pub rank: i32,
    pub shape: [i64; HE_MAX_RANK],
    pub const_bits: u32,
    pub axis_a: i32,
    pub axis_b: i32,
    pub axes: u32,
}

#[repr(C)]
#[derive(Copy, Clone)]
pub struct he_conv2d_params {
    pub in_channels: i32, pub out_channels: i32,
    pub kernel_h: i32, pub kernel_w: i32,
    pub stride_h: i32, pub stride_w: i32,
    pub dilation_h: i32, pub dilation_w: i32,
    pub padding_mode: i32,
}

#[repr(C)]
#[derive(Copy, Clone)]
pub struct he_conv2d_fusion {
    pub out_dtype: i32, pub has_bias: i32, pub bias_dtype: i32, pub has_resid: i32, pub has_gate: i32, pub want_stats: i32,
}

pub const HE_CONV_FWD: i32 = 0;
pub const HE_CONV_BWD_DATA: i32 = 1;
pub const HE_CONV_BWD_FILTER: i32 = 2;

#[repr(C)]
pub struct he_graph_desc {
    pub num_nodes: i32,
    pub nodes: *const he_node,
    pub num_outputs: i32,
    pub outputs: *const i32,
}

#[repr(C)] pub struct he_ctx { _p: [u8; 0] }
#[repr(C)] pub struct he_plan { _p: [u8; 0] }
#[repr(C)] pub struct he_comm { _p: [u8; 0] }
#[repr(C)] pub struct heh_graph { _p: [u8; 0] }
#[repr(C)] pub struct heh_exec { _p: [u8; 0] }

pub const HE_COMM_UNIQUE_ID_BYTES: usize = 128;
pub const HE_NOALLOC_MAX_PARTIALS: usize = 65536;

extern "C" {
    pub fn he_ctx_create(device_ordinal: i32, out: *mut *mut he_ctx) -> i32;
    pub fn he_ctx_destroy(ctx: *mut he_ctx);
    pub fn he_ctx_reserve_sms(ctx: *mut he_ctx, sms: i32) -> i32;
    pub fn he_ctx_poll_device_status(ctx: *mut he_ctx, cu_stream: *mut c_void) -> i32;

    pub fn he_plan_pointwise(ctx: *mut he_ctx, desc: *const he_graph_desc, out: *mut *mut he_plan) -> i32;
    pub fn he_plan_permute(ctx: *mut he_ctx, rank: i32, in_shape: *const i64, out_strides: *const i64,
                           dtype: i32, out: *mut *mut he_plan) -> i32;
    pub fn he_permute_output_strides(rank: i32, in_shape: *const i64, num_swaps: i32, swaps: *const i32,
                                     reference_compat: i32, out_strides: *mut i64) -> i32;
    pub fn he_plan_fused_matmul(ctx: *mut he_ctx, desc: *const he_graph_desc, out: *mut *mut he_plan) -> i32;
    pub fn he_plan_supported(ctx: *mut he_ctx, desc: *const he_graph_desc, kind: i32) -> i32;
    pub fn he_plan_workspace_bytes(plan: *const he_plan, out: *mut usize) -> i32;
    pub fn he_launch(plan: *mut he_plan, inputs: *const *const c_void, outputs: *const *mut c_void,
                     workspace: *mut c_void, cu_stream: *mut c_void) -> i32;
    pub fn he_plan_last_launch_count(plan: *const he_plan) -> i32;
    pub fn he_plan_describe(plan: *const he_plan) -> *const c_char;
    pub fn he_plan_destroy(plan: *mut he_plan);

    pub fn he_plan_conv2d(ctx: *mut he_ctx, kind: i32, params: *const he_conv2d_params, batch: i32, in_h: i32, in_w: i32,
                          dtype: i32, fusion: *const he_conv2d_fusion, out: *mut *mut he_plan) -> i32;
    pub fn he_bn_finalize(stats: *const f32, count: i64, gamma: *const f32, beta: *const f32, running_mean: *mut f32,
                          running_var: *mut f32, scale: *mut f32, shift: *mut f32, mean: *mut f32, rstd: *mut f32, channels: i32,
                          cu_stream: *mut c_void) -> i32;
    pub fn he_bn_workspace_bytes(pixels: i64, channels: i32) -> usize;
    pub fn he_bn_apply(x: *const c_void, y: *mut c_void, scale: *const f32, shift: *const f32, pixels: i64, channels: i32,
                       relu: i32, stats_out: *mut f32, workspace: *mut c_void, cu_stream: *mut c_void) -> i32;
    pub fn he_bn_backward_coeffs(stats: *const f32, count: i64, gamma: *const f32, mean: *const f32, rstd: *const f32,
                                 coef: *mut f32, dgamma: *mut f32, dbeta: *mut f32, channels: i32, cu_stream: *mut c_void) -> i32;
    pub fn he_bn_backward_apply(g: *const c_void, x: *const c_void, addend: *const c_void, out: *mut c_void, coef: *const f32,
                                mask_x: *const c_void, mask_scale: *const f32, mask_shift: *const f32, stats_out: *mut f32,
                                workspace: *mut c_void, pixels: i64, channels: i32, cu_stream: *mut c_void) -> i32;
    pub fn he_add_bf16(a: *const c_void, b: *const c_void, out: *mut c_void, n: i64, cu_stream: *mut c_void) -> i32;
    pub fn he_colsum_bf16(x: *const c_void, out: *mut f32, workspace: *mut c_void, pixels: i64, channels: i32,
                          cu_stream: *mut c_void) -> i32;
    pub fn he_sgd_momentum(w: *mut f32, avg: *mut f32, grad: *const c_void, grad_dtype: i32, w_bf16: *mut c_void, n: i64, lr: f32,
                           momentum: f32, first_step: i32, cu_stream: *mut c_void) -> i32;
    pub fn he_im2col_nhwc(x: *const c_void, cols: *mut c_void, batch: i32, in_h: i32, in_w: i32, channels: i32, kernel_h: i32,
                          kernel_w: i32, stride: i32, pitch: i32, cu_stream: *mut c_void) -> i32;
    pub fn he_pool_softmax_ce(y: *const c_void, labels: *const i32, loss: *mut f32, dy: *mut c_void, batch: i32, positions: i32,
                              classes: i32, cu_stream: *mut c_void) -> i32;

    pub fn he_comm_unique_id(id_out: *mut c_void) -> i32;
    pub fn he_comm_create(ctx: *mut he_ctx, rank: i32, world: i32, unique_id: *const c_void, max_ctas: i32,
                          timeout_ms: i32, out: *mut *mut he_comm) -> i32;
    pub fn he_comm_info(comm: *const he_comm, rank: *mut i32, world: *mut i32, max_ctas: *mut i32) -> i32;
    pub fn he_allreduce_grads(comm: *mut he_comm, bufs: *const *mut c_void, counts: *const usize, n: i32,
                              dtype: i32, mean: i32, cu_stream: *mut c_void) -> i32;
    pub fn he_comm_poll(comm: *mut he_comm) -> i32;
    pub fn he_comm_abort(comm: *mut he_comm) -> i32;
    pub fn he_comm_destroy(comm: *mut he_comm);

    pub fn heh_graph_create(out: *mut *mut heh_graph) -> i32;
    pub fn heh_graph_destroy(g: *mut heh_graph);
    pub fn heh_graph_new_input(g: *mut heh_graph, dtype: i32, rank: i32, shape: *const i64, node_out: *mut i32) -> i32;
    pub fn heh_graph_new_op(g: *mut heh_graph, op: *const he_node, node_out: *mut i32) -> i32;
    pub fn heh_graph_new_output(g: *mut heh_graph, node: i32) -> i32;
    pub fn heh_graph_plan_text(ctx: *mut he_ctx, g: *mut heh_graph, buf: *mut c_char, cap: usize) -> i32;
    /// mode 0: pairwise merging (plan_generation.rs:243-256); mode 1: fusion search (helium-playground).
    pub fn heh_graph_set_planner(g: *mut heh_graph, mode: i32, depth: i32, max_states: i32) -> i32;
    pub fn heh_graph_search_text(ctx: *mut he_ctx, g: *mut heh_graph, buf: *mut c_char, cap: usize) -> i32;
    pub fn heh_graph_subdivisions_text(g: *mut heh_graph, buf: *mut c_char, cap: usize) -> i32;
    pub fn heh_exec_create(ctx: *mut he_ctx, g: *mut heh_graph, inputs: *const *const c_void,
                           outputs: *const *mut c_void, capture_cuda_graph: i32, out: *mut *mut heh_exec) -> i32;
    pub fn heh_exec_run(e: *mut heh_exec, cu_stream: *mut c_void) -> i32;
    pub fn heh_exec_stats(e: *const heh_exec, launches: *mut i32, steps: *mut i32, instrs: *mut i32) -> i32;
    pub fn heh_exec_destroy(e: *mut heh_exec);

    pub fn he_debug_plan_fault_injection(plan: *mut he_plan, wait_limit_us: u32, withhold_loads: i32) -> i32;
    pub fn he_reduce_sum_f32_noalloc(input: *const f32, out: *mut f32, num_groups: i64, group_size: i64,
                                     cu_stream: *mut c_void) -> i32;
    pub fn he_last_error_string() -> *const c_char;
    pub fn he_version() -> *const c_char;
}

/// The thread-local message of the last failed call.
pub fn last_error() -> String {
    unsafe { std::ffi::CStr::from_ptr(he_last_error_string()).to_string_lossy().into_owned() }
}
