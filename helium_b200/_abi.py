"""ctypes mirror of the declarations of include/helium_b200.h: structures and the signature of every
exported symbol.  Pure declarations -- importing this module does not load the shared library, so the
host-side graph builders (ir.py, configs.py) can be used where the library is not wanted."""
from __future__ import annotations

import ctypes as C

HE_MAX_RANK = 8

class HeNode(C.Structure):
    """struct he_node of include/helium_b200.h."""

    _fields_ = [
        ("kind", C.c_int32),
        ("sub_op", C.c_int32),
        ("inp", C.c_int32 * 3),
        ("dtype", C.c_int32),
        ("rank", C.c_int32),
        ("shape", C.c_int64 * HE_MAX_RANK),
        ("const_bits", C.c_uint32),
        ("axis_a", C.c_int32),
        ("axis_b", C.c_int32),
        ("axes", C.c_uint32),
    ]


class HeGraphDesc(C.Structure):
    """struct he_graph_desc of include/helium_b200.h."""

    _fields_ = [
        ("num_nodes", C.c_int32),
        ("nodes", C.POINTER(HeNode)),
        ("num_outputs", C.c_int32),
        ("outputs", C.POINTER(C.c_int32)),
    ]


class HeConv2dParams(C.Structure):
    """struct he_conv2d_params of include/helium_b200.h."""

    _fields_ = [(n, C.c_int32) for n in ("in_channels", "out_channels", "kernel_h", "kernel_w", "stride_h", "stride_w",
                                         "dilation_h", "dilation_w", "padding_mode")]


class HeConv2dFusion(C.Structure):
    """struct he_conv2d_fusion of include/helium_b200.h."""

    _fields_ = [(n, C.c_int32) for n in ("out_dtype", "has_bias", "bias_dtype", "has_resid", "has_gate", "want_stats")]


#: every symbol include/helium_b200.h declares: name -> (restype, argtypes)
SIGNATURES = {
    "he_ctx_create": (C.c_int32, [C.c_int32, C.POINTER(C.c_void_p)]),
    "he_ctx_destroy": (None, [C.c_void_p]),
    "he_ctx_reserve_sms": (C.c_int32, [C.c_void_p, C.c_int32]),
    "he_ctx_poll_device_status": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "he_plan_pointwise": (C.c_int32, [C.c_void_p, C.POINTER(HeGraphDesc), C.POINTER(C.c_void_p)]),
    "he_plan_permute": (C.c_int32, [C.c_void_p, C.c_int32, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.c_int32,
                                    C.POINTER(C.c_void_p)]),
    "he_permute_output_strides": (C.c_int32, [C.c_int32, C.POINTER(C.c_int64), C.c_int32, C.POINTER(C.c_int32),
                                              C.c_int32, C.POINTER(C.c_int64)]),
    "he_plan_fused_matmul": (C.c_int32, [C.c_void_p, C.POINTER(HeGraphDesc), C.POINTER(C.c_void_p)]),
    "he_plan_conv2d": (C.c_int32, [C.c_void_p, C.c_int32, C.POINTER(HeConv2dParams), C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                   C.POINTER(HeConv2dFusion), C.POINTER(C.c_void_p)]),
    "he_bn_finalize": (C.c_int32, [C.c_void_p, C.c_int64] + [C.c_void_p] * 8 + [C.c_int32, C.c_void_p]),
    "he_bn_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int32]),
    "he_bn_apply": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                C.c_void_p]),
    "he_bn_backward_coeffs": (C.c_int32, [C.c_void_p, C.c_int64] + [C.c_void_p] * 6 + [C.c_int32, C.c_void_p]),
    "he_bn_backward_apply": (C.c_int32, [C.c_void_p] * 10 + [C.c_int64, C.c_int32, C.c_void_p]),
    "he_add_bf16": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "he_colsum_bf16": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_void_p]),
    "he_sgd_momentum": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int64, C.c_float, C.c_float, C.c_int32,
                                    C.c_void_p]),
    "he_im2col_nhwc": (C.c_int32, [C.c_void_p, C.c_void_p] + [C.c_int32] * 8 + [C.c_void_p]),
    "he_pool_softmax_ce": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "he_plan_supported": (C.c_int32, [C.c_void_p, C.POINTER(HeGraphDesc), C.c_int32]),
    "he_plan_workspace_bytes": (C.c_int32, [C.c_void_p, C.POINTER(C.c_size_t)]),
    "he_launch": (C.c_int32, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_void_p, C.c_void_p]),
    "he_plan_last_launch_count": (C.c_int32, [C.c_void_p]),
    "he_plan_describe": (C.c_char_p, [C.c_void_p]),
    "he_plan_destroy": (None, [C.c_void_p]),
    "heh_graph_create": (C.c_int32, [C.POINTER(C.c_void_p)]),
    "heh_graph_destroy": (None, [C.c_void_p]),
    "heh_graph_new_input": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_int64), C.POINTER(C.c_int32)]),
    "heh_graph_new_op": (C.c_int32, [C.c_void_p, C.POINTER(HeNode), C.POINTER(C.c_int32)]),
    "heh_graph_new_output": (C.c_int32, [C.c_void_p, C.c_int32]),
    "heh_graph_plan_text": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_char_p, C.c_size_t]),
    "heh_graph_set_planner": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32]),
    "heh_graph_search_text": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_char_p, C.c_size_t]),
    "heh_graph_subdivisions_text": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_size_t]),
    "heh_exec_create": (C.c_int32, [C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int32,
                                    C.POINTER(C.c_void_p)]),
    "heh_exec_run": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "heh_exec_stats": (C.c_int32, [C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "heh_exec_destroy": (None, [C.c_void_p]),
    "he_debug_dump_program": (C.c_int32, [C.POINTER(HeGraphDesc), C.c_int32, C.c_void_p, C.c_size_t, C.POINTER(C.c_size_t)]),
    "he_debug_canonical_text": (C.c_int32, [C.POINTER(HeGraphDesc), C.c_char_p, C.c_size_t]),
    "he_comm_unique_id": (C.c_int32, [C.c_void_p]),
    "he_comm_create": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_void_p)]),
    "he_comm_info": (C.c_int32, [C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "he_allreduce_grads": (C.c_int32, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_size_t), C.c_int32, C.c_int32, C.c_int32,
                                       C.c_void_p]),
    "he_comm_poll": (C.c_int32, [C.c_void_p]),
    "he_comm_abort": (C.c_int32, [C.c_void_p]),
    "he_comm_destroy": (None, [C.c_void_p]),
    "he_debug_plan_fault_injection": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_int32]),
    "he_last_error_string": (C.c_char_p, []),
    "he_reduce_sum_f32_noalloc": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    "he_version": (C.c_char_p, []),
}


