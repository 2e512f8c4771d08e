"""ctypes binding of libfuse_b200.so (the C ABI declared in include/fuse_b200.h).

Importing this module never falls back to another implementation: if the CUDA library has
not been built, `lib()` raises with the build command."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfuse_b200.so")

MAX_WORLD_SIZE = 8
READY_FLAG_STRIDE = 32

RASTER_HEURISTIC, RASTER_ALONG_M, RASTER_ALONG_N = 0, 1, 2
DTYPE_BF16, DTYPE_E4M3 = 0, 1
ROUTE_HEAD_TO_SEQUENCE, ROUTE_QKV_GQA_PACK = 0, 2
ROUTE_FORWARD, ROUTE_INVERSE = 0, 1
STATIC_SCRATCH_BYTES = 8 << 20
SKIP_PEER_WAIT = 1
QKV_ROUTE_COMM_CTAS = 2
QKV_ROUTE_DIRECT = 4
VECTOR_PULL = 8
VECTOR_EPILOGUE = 16
COMM_ONLY = 32
COMPUTE_ONLY = 64

CUDA_SUCCESS = 0
CUDA_ERROR_INVALID_VALUE = 1
CUDA_ERROR_NOT_SUPPORTED = 801


class MatrixStride(C.Structure):
    _fields_ = [("row", C.c_int64), ("column", C.c_int64), ("batch", C.c_int64)]

    def __init__(self, row=-1, column=-1, batch=-1):
        super().__init__(row, column, batch)


class GemmProblem(C.Structure):
    """include/fuse/layout/gemm.h:27-42 of the reference (GemmProblem)."""
    _fields_ = [("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("l", C.c_int32),
                ("stride_a", MatrixStride), ("stride_b", MatrixStride), ("stride_d", MatrixStride),
                ("input_dtype", C.c_int32), ("weight_dtype", C.c_int32),
                ("output_dtype", C.c_int32), ("transpose_a", C.c_uint8),
                ("transpose_b", C.c_uint8), ("raster", C.c_int32), ("max_swizzle_size", C.c_int32)]

    def __init__(self, m=0, n=0, k=0, raster=RASTER_HEURISTIC, max_swizzle_size=1, **kw):
        super().__init__()
        self.m, self.n, self.k, self.l = m, n, k, 1
        self.stride_a, self.stride_b, self.stride_d = MatrixStride(), MatrixStride(), MatrixStride()
        self.raster, self.max_swizzle_size = raster, max_swizzle_size
        for key, value in kw.items():
            setattr(self, key, value)


class UlyssesRoute(C.Structure):
    """include/fuse/layout/ulysses.h:24-63 of the reference (UlyssesRoute)."""
    _fields_ = [("world_size", C.c_int32), ("rank", C.c_int32), ("batch", C.c_int32),
                ("global_seq", C.c_int32), ("seq_local", C.c_int32), ("q_heads", C.c_int32),
                ("kv_heads", C.c_int32), ("local_heads", C.c_int32), ("head_dim", C.c_int32),
                ("channel_count", C.c_int32), ("qkv_peer_interleaved", C.c_uint8),
                ("defer_v_a2a", C.c_uint8), ("causal_load_balanced", C.c_uint8),
                ("cyclic_peer_order", C.c_uint8), ("packed_source_row", C.c_void_p),
                ("packed_row_granularity", C.c_int32), ("kind", C.c_int32),
                ("direction", C.c_int32)]

    def __init__(self, **kw):
        super().__init__()
        self.world_size, self.batch, self.channel_count = 1, 1, 1
        self.kind, self.direction = ROUTE_HEAD_TO_SEQUENCE, ROUTE_FORWARD
        for key, value in kw.items():
            setattr(self, key, value)


class KernelTraits(C.Structure):
    _fields_ = [("block_m", C.c_int32), ("block_n", C.c_int32), ("block_k", C.c_int32),
                ("threads", C.c_int32), ("dynamic_smem_bytes", C.c_int32)]


class GemmA2AParams(C.Structure):
    """include/fuse/operators/primitives/gemm_a2a.h:17-30 of the reference."""
    _fields_ = [("lhs", C.c_void_p), ("rhs_nt", C.c_void_p), ("local_output", C.c_void_p),
                ("peer_output", C.c_void_p * MAX_WORLD_SIZE),
                ("peer_route_done_epoch", C.c_void_p * MAX_WORLD_SIZE), ("ready", C.c_void_p),
                ("completion_epoch", C.c_void_p), ("gemm", GemmProblem), ("route", UlyssesRoute),
                ("num_comm_ctas", C.c_int32), ("epoch", C.c_uint32), ("alpha", C.c_float)]

    def __init__(self, **kw):
        super().__init__()
        self.alpha = 1.0
        for key, value in kw.items():
            setattr(self, key, value)


class A2AGemmParams(C.Structure):
    """include/fuse/operators/primitives/a2a_gemm.h:47-61 of the reference."""
    _fields_ = [("peer_input", C.c_void_p * MAX_WORLD_SIZE), ("input_staging", C.c_void_p),
                ("peer_input_ready", C.c_void_p * MAX_WORLD_SIZE), ("rhs_nt", C.c_void_p),
                ("output", C.c_void_p), ("ready", C.c_void_p), ("gemm", GemmProblem),
                ("route", UlyssesRoute), ("num_comm_ctas", C.c_int32), ("lhs_policy", C.c_int32),
                ("epoch", C.c_uint32), ("input_epoch", C.c_uint32), ("alpha", C.c_float)]

    def __init__(self, **kw):
        super().__init__()
        self.alpha = 1.0
        for key, value in kw.items():
            setattr(self, key, value)


class Options(C.Structure):
    _fields_ = [("wait_budget_ns", C.c_uint64), ("flags", C.c_uint32), ("block_n", C.c_int32),
                ("trace", C.c_void_p), ("trace_capacity", C.c_uint32), ("trace_cta", C.c_int32)]


class _Record(C.Structure):
    def __init__(self, **kw):
        super().__init__()
        for key, value in getattr(self, "_defaults_", {}).items():
            setattr(self, key, value)
        for key, value in kw.items():
            setattr(self, key, value)


class BackwardGemmTuning(C.Structure):
    _fields_ = [("epilogue_n", C.c_int32), ("max_swizzle_size", C.c_int32), ("along_m", C.c_uint8)]


class QkvBackwardDataParams(_Record):
    """include/fuse/operators/ulysses/qkv_backward.h:24-49 of the reference."""
    _fields_ = [("grad_q", C.c_void_p), ("grad_k", C.c_void_p), ("grad_v", C.c_void_p),
                ("peer_dqkv_staging", C.c_void_p * MAX_WORLD_SIZE), ("peer_ready", C.c_void_p * MAX_WORLD_SIZE),
                ("peer_done_epoch", C.c_void_p * MAX_WORLD_SIZE), ("weight", C.c_void_p),
                ("grad_input", C.c_void_p), ("local_tokens", C.c_int32), ("hidden", C.c_int32),
                ("batch", C.c_int32), ("q_heads", C.c_int32), ("kv_heads", C.c_int32), ("head_dim", C.c_int32),
                ("world_size", C.c_int32), ("rank", C.c_int32), ("num_comm_ctas", C.c_int32),
                ("gemm_policy", C.c_int32), ("gemm_tuning", BackwardGemmTuning), ("epoch", C.c_uint32),
                ("causal_load_balanced", C.c_uint8), ("alpha", C.c_float)]
    _defaults_ = {"batch": 1, "world_size": 1, "alpha": 1.0}


class QkvBackwardWeightParams(_Record):
    """include/fuse/operators/ulysses/qkv_backward.h:62-73 of the reference."""
    _fields_ = [("dqkv_staging", C.c_void_p), ("saved_input", C.c_void_p), ("grad_weight", C.c_void_p),
                ("local_tokens", C.c_int32), ("hidden", C.c_int32), ("q_heads", C.c_int32),
                ("kv_heads", C.c_int32), ("head_dim", C.c_int32), ("alpha", C.c_float), ("beta", C.c_float)]
    _defaults_ = {"alpha": 1.0}


class QkvBackwardParams(_Record):
    _fields_ = [("data", QkvBackwardDataParams), ("weight", QkvBackwardWeightParams),
                ("weight_mode", C.c_int32)]


class OprojBackwardDataParams(_Record):
    """include/fuse/operators/ulysses/oproj_backward.h:21-43 of the reference."""
    _fields_ = [("grad_output", C.c_void_p), ("weight", C.c_void_p), ("local_grad_attention", C.c_void_p),
                ("peer_grad_attention", C.c_void_p * MAX_WORLD_SIZE),
                ("peer_done_epoch", C.c_void_p * MAX_WORLD_SIZE), ("ready", C.c_void_p),
                ("local_tokens", C.c_int32), ("hidden", C.c_int32), ("batch", C.c_int32),
                ("q_heads", C.c_int32), ("head_dim", C.c_int32), ("world_size", C.c_int32),
                ("rank", C.c_int32), ("num_comm_ctas", C.c_int32), ("gemm_policy", C.c_int32),
                ("gemm_tuning", BackwardGemmTuning), ("epoch", C.c_uint32),
                ("causal_load_balanced", C.c_uint8), ("alpha", C.c_float)]
    _defaults_ = {"batch": 1, "world_size": 1, "alpha": 1.0}


class OprojBackwardWeightParams(_Record):
    """include/fuse/operators/ulysses/oproj_backward.h:54-64 of the reference."""
    _fields_ = [("grad_output", C.c_void_p), ("saved_attention", C.c_void_p), ("grad_weight", C.c_void_p),
                ("local_tokens", C.c_int32), ("hidden", C.c_int32), ("q_heads", C.c_int32),
                ("head_dim", C.c_int32), ("alpha", C.c_float), ("beta", C.c_float)]
    _defaults_ = {"alpha": 1.0}


class OprojBackwardParams(_Record):
    _fields_ = [("data", OprojBackwardDataParams), ("weight", OprojBackwardWeightParams),
                ("weight_mode", C.c_int32)]


class Mxfp8Activation(_Record):
    """include/fuse/types.h:31-35 of the reference."""
    _fields_ = [("data", C.c_void_p), ("scales", C.c_void_p), ("data_bytes", C.c_size_t),
                ("scale_bytes", C.c_size_t)]


class QkvPostprocess(_Record):
    _fields_ = [("q_gamma", C.c_void_p), ("k_gamma", C.c_void_p), ("cos", C.c_void_p), ("sin", C.c_void_p),
                ("epsilon", C.c_float)]
    _defaults_ = {"epsilon": 1e-6}


class Mxfp8GemmA2AParams(_Record):
    """include/fuse/operators/primitives/gemm_a2a_mxfp8.h:23-39 of the reference."""
    _fields_ = [("projection", GemmA2AParams), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
                ("activation", Mxfp8Activation), ("weight_preparation", C.c_int32), ("epilogue_n", C.c_int32),
                ("postprocess", QkvPostprocess)]
    _defaults_ = {"epilogue_n": 64}


class ResidualRmsNorm(_Record):
    _fields_ = [("residual", C.c_void_p), ("gamma", C.c_void_p), ("residual_output", C.c_void_p),
                ("epsilon", C.c_float)]
    _defaults_ = {"epsilon": 1e-6}


class Mxfp8A2AGemmParams(_Record):
    """include/fuse/operators/primitives/a2a_gemm_mxfp8.h:25-46 of the reference."""
    _fields_ = [("projection", A2AGemmParams), ("activation", Mxfp8Activation * MAX_WORLD_SIZE),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("epilogue_n", C.c_int32),
                ("m_window_tiles", C.c_int32), ("n_group_tiles", C.c_int32), ("postprocess", ResidualRmsNorm),
                ("overlap_postnorm", C.c_uint8), ("weight_preparation", C.c_int32)]
    _defaults_ = {"epilogue_n": 32}


class GroupedGemmPolicy(_Record):
    """include/fuse/operators/primitives/grouped_gemm.h:17-53 of the reference."""
    _fields_ = [("num_comm_ctas", C.c_int32), ("num_compute_ctas", C.c_int32), ("swizzle", C.c_int32),
                ("along_n", C.c_uint8), ("tile_n", C.c_int32), ("tile_k", C.c_int32),
                ("mma_sm_count", C.c_int32), ("dispatch_copy", C.c_int32),
                ("balance_dispatch_tail", C.c_uint8), ("swap_ab", C.c_uint8), ("trim_swap_tokens", C.c_uint8),
                ("scheduler", C.c_int32)]
    _defaults_ = {"num_comm_ctas": 20, "num_compute_ctas": 128, "swizzle": 1, "tile_n": 128, "tile_k": 64,
                  "mma_sm_count": 1, "trim_swap_tokens": 1}


class Bf16GroupedGemmParams(_Record):
    """include/fuse/operators/primitives/grouped_gemm.h:62-85 of the reference."""
    _fields_ = [("lhs", C.c_void_p), ("weight_nt", C.c_void_p), ("output", C.c_void_p),
                ("row_offsets", C.c_void_p), ("source", C.c_void_p),
                ("peer_input", C.c_void_p * MAX_WORLD_SIZE), ("peer_output", C.c_void_p * MAX_WORLD_SIZE),
                ("peer_started", C.c_void_p * MAX_WORLD_SIZE), ("peer_done", C.c_void_p * MAX_WORLD_SIZE),
                ("experts", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("expert_row_capacity", C.c_int32),
                ("rank", C.c_int32), ("world_size", C.c_int32), ("topk", C.c_int32),
                ("policy", GroupedGemmPolicy), ("dispatch_buffer_rows", C.c_int32)]


class Mxfp8QkvBackwardInput(_Record):
    _fields_ = [("grad_q", Mxfp8Activation), ("grad_k", Mxfp8Activation), ("grad_v", Mxfp8Activation),
                ("master_q", C.c_void_p), ("master_k", C.c_void_p), ("master_v", C.c_void_p)]


class Mxfp8QkvBackwardDataParams(_Record):
    """include/fuse/operators/ulysses/qkv_backward.h:219-224 of the reference."""
    _fields_ = [("projection", QkvBackwardDataParams), ("peer_input", Mxfp8QkvBackwardInput * MAX_WORLD_SIZE),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


class Mxfp8QkvBackwardWeightParams(_Record):
    _fields_ = [("projection", QkvBackwardWeightParams), ("gemm_tuning", BackwardGemmTuning),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


class Mxfp8QkvBackwardParams(_Record):
    _fields_ = [("data", Mxfp8QkvBackwardDataParams), ("weight", Mxfp8QkvBackwardWeightParams),
                ("weight_mode", C.c_int32)]


class Mxfp8OprojBackwardDataParams(_Record):
    """include/fuse/operators/ulysses/oproj_backward.h:191-196 of the reference."""
    _fields_ = [("projection", OprojBackwardDataParams), ("grad_output", Mxfp8Activation),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


class Mxfp8OprojBackwardWeightParams(_Record):
    _fields_ = [("projection", OprojBackwardWeightParams), ("gemm_tuning", BackwardGemmTuning),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


class Mxfp8OprojBackwardParams(_Record):
    _fields_ = [("data", Mxfp8OprojBackwardDataParams), ("weight", Mxfp8OprojBackwardWeightParams),
                ("weight_mode", C.c_int32)]


ABI_RECORDS = {0: GemmProblem, 1: UlyssesRoute, 2: GemmA2AParams, 3: A2AGemmParams,
               4: KernelTraits, 5: Options, 17: Mxfp8QkvBackwardDataParams, 18: Mxfp8QkvBackwardWeightParams,
               19: Mxfp8QkvBackwardParams, 20: Mxfp8OprojBackwardDataParams, 21: Mxfp8OprojBackwardWeightParams,
               22: Mxfp8OprojBackwardParams, 15: GroupedGemmPolicy, 16: Bf16GroupedGemmParams, 14: Mxfp8A2AGemmParams, 12: Mxfp8Activation, 13: Mxfp8GemmA2AParams, 6: QkvBackwardDataParams, 7: QkvBackwardWeightParams,
               8: QkvBackwardParams, 9: OprojBackwardDataParams, 10: OprojBackwardWeightParams,
               11: OprojBackwardParams}

# Every symbol include/fuse_b200.h declares: name -> (restype, argtypes).
_P = C.c_void_p
SYMBOLS = {
    "fuse_launch_gemm_a2a_cutlass": (C.c_int, [C.POINTER(GemmA2AParams), _P]),
    "fuse_launch_gemm_a2a_cutlass_ex": (C.c_int, [C.POINTER(GemmA2AParams), C.POINTER(Options), _P]),
    "fuse_launch_a2a_gemm_cutlass": (C.c_int, [C.POINTER(A2AGemmParams), _P]),
    "fuse_launch_a2a_gemm_cutlass_ex": (C.c_int, [C.POINTER(A2AGemmParams), C.POINTER(Options), _P]),
    "fuse_launch_batched_cutlass_reference": (C.c_int, [C.POINTER(GemmA2AParams), _P, C.c_int32]),
    "fuse_launch_a2a_gemm_cutlass_reference": (C.c_int, [C.POINTER(A2AGemmParams), _P, C.c_int32]),
    "fuse_launch_qkv_backward_data": (C.c_int, [C.POINTER(QkvBackwardDataParams), _P]),
    "fuse_launch_qkv_backward_data_ex": (C.c_int, [C.POINTER(QkvBackwardDataParams), C.POINTER(Options), _P]),
    "fuse_launch_qkv_backward_weight": (C.c_int, [C.POINTER(QkvBackwardWeightParams), _P]),
    "fuse_launch_qkv_backward": (C.c_int, [C.POINTER(QkvBackwardParams), _P]),
    "fuse_launch_oproj_backward_data": (C.c_int, [C.POINTER(OprojBackwardDataParams), _P]),
    "fuse_launch_oproj_backward_data_ex": (C.c_int, [C.POINTER(OprojBackwardDataParams), C.POINTER(Options), _P]),
    "fuse_launch_oproj_backward_weight": (C.c_int, [C.POINTER(OprojBackwardWeightParams), _P]),
    "fuse_launch_oproj_backward": (C.c_int, [C.POINTER(OprojBackwardParams), _P]),
    "fuse_qkv_backward_ready_elements": (C.c_int64, [C.POINTER(QkvBackwardDataParams)]),
    "fuse_oproj_backward_ready_elements": (C.c_int64, [C.POINTER(OprojBackwardDataParams)]),
    "fuse_recommended_qkv_backward_comm_ctas": (C.c_int32, [C.POINTER(QkvBackwardDataParams)]),
    "fuse_recommended_oproj_backward_comm_ctas": (C.c_int32, [C.POINTER(OprojBackwardDataParams)]),
    "fuse_gemm_a2a_mxfp8_activation_size": (C.c_int, [C.POINTER(GemmProblem), C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "fuse_quantize_gemm_a2a_mxfp8_activation": (C.c_int, [C.POINTER(GemmProblem), _P, C.POINTER(Mxfp8Activation), _P]),
    "fuse_gemm_a2a_mxfp8_workspace_size": (C.c_int, [C.POINTER(GemmProblem), C.POINTER(C.c_size_t)]),
    "fuse_launch_gemm_a2a_mxfp8_cutlass": (C.c_int, [C.POINTER(Mxfp8GemmA2AParams), _P]),
    "fuse_launch_gemm_a2a_mxfp8_cutlass_ex": (C.c_int, [C.POINTER(Mxfp8GemmA2AParams), C.POINTER(Options), _P]),
    "fuse_prepare_gemm_a2a_mxfp8": (C.c_int, [C.POINTER(Mxfp8GemmA2AParams), _P]),
    "fuse_launch_gemm_a2a_mxfp8_prequantized": (C.c_int, [C.POINTER(Mxfp8GemmA2AParams), _P]),
    "fuse_launch_gemm_a2a_mxfp8_prequantized_ex": (C.c_int, [C.POINTER(Mxfp8GemmA2AParams), C.POINTER(Options), _P]),
    "fuse_launch_gemm_a2a_mxfp8_compute_reference": (C.c_int, [C.POINTER(Mxfp8GemmA2AParams), _P]),
    "fuse_b200_launch_gemm_a2a_mxfp8_static": (C.c_int, [C.POINTER(Mxfp8GemmA2AParams), _P]),
    "fuse_b200_quantize_mxfp8": (C.c_int, [_P, C.c_int64, C.c_int32, C.c_int32, _P, _P, _P]),
    "fuse_b200_quantize_mxfp8_transposed": (C.c_int, [_P, C.c_int64, C.c_int32, C.c_int32, _P, _P, _P]),
    "fuse_b200_mxfp8_scale_bytes": (C.c_size_t, [C.c_int64, C.c_int64]),
    "fuse_a2a_gemm_mxfp8_activation_size": (C.c_int, [C.POINTER(GemmProblem), C.POINTER(UlyssesRoute), C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "fuse_a2a_gemm_mxfp8_workspace_size": (C.c_int, [C.POINTER(GemmProblem), C.POINTER(C.c_size_t)]),
    "fuse_a2a_gemm_mxfp8_staging_view": (C.c_int, [C.POINTER(Mxfp8A2AGemmParams), C.POINTER(Mxfp8Activation)]),
    "fuse_launch_a2a_gemm_mxfp8_cutlass": (C.c_int, [C.POINTER(Mxfp8A2AGemmParams), _P]),
    "fuse_launch_a2a_gemm_mxfp8_cutlass_ex": (C.c_int, [C.POINTER(Mxfp8A2AGemmParams), C.POINTER(Options), _P]),
    "fuse_create_bf16_a2a_grouped_gemm": (C.c_int, [C.POINTER(Bf16GroupedGemmParams), C.POINTER(C.c_void_p)]),
    "fuse_create_bf16_grouped_gemm_a2a": (C.c_int, [C.POINTER(Bf16GroupedGemmParams), C.POINTER(C.c_void_p)]),
    "fuse_launch_bf16_grouped_gemm": (C.c_int, [C.c_void_p, _P]),
    "fuse_launch_bf16_grouped_gemm_ex": (C.c_int, [C.c_void_p, C.POINTER(Options), _P]),
    "fuse_destroy_bf16_grouped_gemm": (C.c_int, [C.c_void_p]),
    "fuse_qkv_backward_mxfp8_data_workspace_size": (C.c_int, [C.POINTER(QkvBackwardDataParams), C.POINTER(C.c_size_t)]),
    "fuse_qkv_backward_mxfp8_weight_workspace_size": (C.c_int, [C.POINTER(QkvBackwardWeightParams), C.POINTER(C.c_size_t)]),
    "fuse_launch_qkv_backward_mxfp8_data": (C.c_int, [C.POINTER(Mxfp8QkvBackwardDataParams), _P]),
    "fuse_launch_qkv_backward_mxfp8_data_ex": (C.c_int, [C.POINTER(Mxfp8QkvBackwardDataParams), C.POINTER(Options), _P]),
    "fuse_launch_qkv_backward_mxfp8_weight": (C.c_int, [C.POINTER(Mxfp8QkvBackwardWeightParams), _P]),
    "fuse_launch_qkv_backward_mxfp8": (C.c_int, [C.POINTER(Mxfp8QkvBackwardParams), _P]),
    "fuse_oproj_backward_mxfp8_data_workspace_size": (C.c_int, [C.POINTER(OprojBackwardDataParams), C.POINTER(C.c_size_t)]),
    "fuse_oproj_backward_mxfp8_weight_workspace_size": (C.c_int, [C.POINTER(OprojBackwardWeightParams), C.POINTER(C.c_size_t)]),
    "fuse_launch_oproj_backward_mxfp8_data": (C.c_int, [C.POINTER(Mxfp8OprojBackwardDataParams), _P]),
    "fuse_launch_oproj_backward_mxfp8_data_ex": (C.c_int, [C.POINTER(Mxfp8OprojBackwardDataParams), C.POINTER(Options), _P]),
    "fuse_launch_oproj_backward_mxfp8_weight": (C.c_int, [C.POINTER(Mxfp8OprojBackwardWeightParams), _P]),
    "fuse_launch_oproj_backward_mxfp8": (C.c_int, [C.POINTER(Mxfp8OprojBackwardParams), _P]),
    "fuse_a2a_gemm_mxfp8_workspace_size_for_params": (C.c_int, [C.POINTER(Mxfp8A2AGemmParams), C.POINTER(C.c_size_t)]),
    "fuse_mxfp8_qkv_cutlass_kernel_traits": (None, [C.c_int32, C.POINTER(KernelTraits)]),
    "fuse_mxfp8_oproj_cutlass_kernel_traits": (None, [C.c_int32, C.c_uint8, C.POINTER(KernelTraits)]),
    "fuse_qkv_cutlass_kernel_traits": (None, [C.POINTER(GemmProblem), C.POINTER(KernelTraits)]),
    "fuse_cutlass_kernel_traits": (None, [C.POINTER(KernelTraits)]),
    "fuse_a2a_lhs_gemm_ready_elements": (C.c_int64, [C.POINTER(GemmProblem), C.POINTER(UlyssesRoute)]),
    "fuse_recommended_gemm_a2a_comm_ctas": (C.c_int32, [C.POINTER(GemmProblem), C.POINTER(UlyssesRoute)]),
    "fuse_recommended_a2a_lhs_gemm_comm_ctas": (C.c_int32, [C.POINTER(GemmProblem), C.POINTER(UlyssesRoute)]),
    "fuse_b200_plan": (C.c_int, [C.c_int32, C.c_double, C.c_double, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                 C.POINTER(C.c_double * 5)]),
    "fuse_b200_plan_remote": (C.c_int, [C.c_int32, C.c_double, C.c_double, C.c_int64, C.c_int32, C.c_int32, C.c_int32,
                                        C.c_int32, C.c_double, C.POINTER(C.c_double * 5)]),
    "fuse_b200_generate_bf16": (C.c_int, [_P, C.c_uint64, C.c_uint64, C.c_float, C.c_int, _P]),
    "fuse_b200_tile_order_decode": (C.c_int, [C.c_int32] * 4 + [C.c_int64, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "fuse_b200_select_swizzle": (C.c_int32, [C.c_int32] * 3),
    "fuse_b200_symmetric_alloc": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p), C.c_char_p]),
    "fuse_b200_symmetric_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "fuse_b200_symmetric_close": (C.c_int, [C.c_void_p]),
    "fuse_b200_symmetric_free": (C.c_int, [C.c_void_p]),
    "fuse_b200_read_status": (C.c_int, [C.POINTER(C.c_uint32 * 16), C.c_int]),
    "fuse_b200_abi_sizeof": (C.c_int, [C.c_int]),
    "fuse_b200_launch_count": (C.c_uint64, []),
}

_LIB = None


def lib():
    """The loaded CUDA library.  Raises when it has not been built: there is no CPU path."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m fuse_b200.build` (nvcc, sm_100a). "
                "fuse_b200 has no CPU or PyTorch fallback.")
        handle = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
        for name, (restype, argtypes) in SYMBOLS.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = restype, argtypes
        _LIB = handle
    return _LIB
