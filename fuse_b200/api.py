"""Host-side mirror of the reference's operator interface (namespace `fuse`), over the C ABI.

Function names, argument meaning and error behaviour follow the reference's free functions
(include/fuse/operators/primitives/gemm_a2a.h, a2a_gemm.h): each returns the cudaError_t value
as an int and never raises for a rejected launch.  Pointers are device addresses (ints);
`stream` is a cudaStream_t value (int, 0 = legacy default stream)."""
from __future__ import annotations

import ctypes as C

from . import _native as N
from ._native import (A2AGemmParams, GemmA2AParams, GemmProblem, KernelTraits, Options,  # noqa: F401
                      OprojBackwardDataParams, OprojBackwardParams, OprojBackwardWeightParams,
                      QkvBackwardDataParams, QkvBackwardParams, QkvBackwardWeightParams, UlyssesRoute)


def _opt(options):
    return C.byref(options) if options is not None else None


def launch_gemm_a2a_cutlass(params: GemmA2AParams, stream: int = 0, options: Options | None = None) -> int:
    """QKV projection + sequence->head all-to-all (fuse::launch_gemm_a2a_cutlass)."""
    if options is None:
        return N.lib().fuse_launch_gemm_a2a_cutlass(C.byref(params), stream)
    return N.lib().fuse_launch_gemm_a2a_cutlass_ex(C.byref(params), _opt(options), stream)


def launch_a2a_gemm_cutlass(params: A2AGemmParams, stream: int = 0, options: Options | None = None) -> int:
    """Head->sequence all-to-all + output projection (fuse::launch_a2a_gemm_cutlass)."""
    if options is None:
        return N.lib().fuse_launch_a2a_gemm_cutlass(C.byref(params), stream)
    return N.lib().fuse_launch_a2a_gemm_cutlass_ex(C.byref(params), _opt(options), stream)


def launch_batched_cutlass_reference(params: GemmA2AParams, stream: int = 0,
                                     reserved_comm_ctas: int = 0) -> int:
    """Projection GEMM alone on SMs - reserved_comm_ctas CTAs (the pure-GEMM denominator)."""
    return N.lib().fuse_launch_batched_cutlass_reference(C.byref(params), stream, reserved_comm_ctas)


def launch_a2a_gemm_cutlass_reference(params: A2AGemmParams, stream: int = 0,
                                      reserved_comm_ctas: int = 0) -> int:
    return N.lib().fuse_launch_a2a_gemm_cutlass_reference(C.byref(params), stream, reserved_comm_ctas)


def qkv_cutlass_kernel_traits(problem: GemmProblem) -> KernelTraits:
    out = KernelTraits()
    N.lib().fuse_qkv_cutlass_kernel_traits(C.byref(problem), C.byref(out))
    return out


def cutlass_kernel_traits() -> KernelTraits:
    out = KernelTraits()
    N.lib().fuse_cutlass_kernel_traits(C.byref(out))
    return out


def a2a_lhs_gemm_ready_elements(problem: GemmProblem, route: UlyssesRoute) -> int:
    return N.lib().fuse_a2a_lhs_gemm_ready_elements(C.byref(problem), C.byref(route))


def recommended_gemm_a2a_comm_ctas(problem: GemmProblem, route: UlyssesRoute) -> int:
    return N.lib().fuse_recommended_gemm_a2a_comm_ctas(C.byref(problem), C.byref(route))


def recommended_a2a_lhs_gemm_comm_ctas(problem: GemmProblem, route: UlyssesRoute) -> int:
    return N.lib().fuse_recommended_a2a_lhs_gemm_comm_ctas(C.byref(problem), C.byref(route))


def plan(kind: int, flops: float, nbytes: float, tiles: int, sm_count: int = 148, group: int = 2,
         explicit_comm_ctas: int = 0, embedded_allowed: bool = True, remote_share: float = 0.0) -> dict:
    """The host planner's choice for one launch (fuse_b200_plan_remote): communication CTAs or embedded
    copy warps.  remote_share: fraction of the bytes that crosses NVLink, (world - 1) / world."""
    out = (C.c_double * 5)()
    rc = N.lib().fuse_b200_plan_remote(kind, flops, nbytes, tiles, sm_count, group, explicit_comm_ctas,
                                       1 if embedded_allowed else 0, remote_share, C.byref(out))
    if rc != 0:
        raise ValueError(f"fuse_b200_plan -> cudaError {rc}")
    return {"comm_ctas": int(out[0]), "embedded": bool(out[1]), "makespan_us": out[2], "compute_us": out[3],
            "transfer_us": out[4]}


def read_status(clear: bool = True) -> list[int]:
    """The device status record of the current device (word 0 != 0: a device wait gave up)."""
    out = (C.c_uint32 * 16)()
    rc = N.lib().fuse_b200_read_status(C.byref(out), 1 if clear else 0)
    if rc != 0:
        raise RuntimeError(f"fuse_b200_read_status failed with cudaError {rc}")
    return list(out)


def launch_count() -> int:
    return int(N.lib().fuse_b200_launch_count())


def qkv_ready_elements(problem: GemmProblem) -> int:
    """u32 words the `ready` array of the QKV operator needs (finest publication tile)."""
    traits = qkv_cutlass_kernel_traits(problem)
    m_tiles = -(-problem.m // traits.block_m)
    n_tiles = -(-problem.n // traits.block_n)
    return m_tiles * n_tiles * N.READY_FLAG_STRIDE


def generate_bf16(ptr: int, count: int, seed: int, scale: float, normal: bool = False, stream: int = 0) -> int:
    """Seeded device-side fill (uniform, or N(0, scale^2) when `normal`)."""
    return N.lib().fuse_b200_generate_bf16(ptr, count, seed, scale, 1 if normal else 0, stream)


# ---- backward (include/fuse/operators/ulysses/{qkv,oproj}_backward.h of the reference) ----------

def launch_qkv_backward_data(params: QkvBackwardDataParams, stream: int = 0, options: Options | None = None) -> int:
    """Reverse all-to-all of planar dQ/dK/dV + dX = dQKV W (fuse::launch_qkv_backward_data)."""
    if options is None:
        return N.lib().fuse_launch_qkv_backward_data(C.byref(params), stream)
    return N.lib().fuse_launch_qkv_backward_data_ex(C.byref(params), _opt(options), stream)


def launch_qkv_backward_weight(params: QkvBackwardWeightParams, stream: int = 0) -> int:
    """dW = alpha dQKV^T X + beta dW (fuse::launch_qkv_backward_weight)."""
    return N.lib().fuse_launch_qkv_backward_weight(C.byref(params), stream)


def launch_qkv_backward(params: QkvBackwardParams, stream: int = 0) -> int:
    return N.lib().fuse_launch_qkv_backward(C.byref(params), stream)


def launch_oproj_backward_data(params: OprojBackwardDataParams, stream: int = 0,
                               options: Options | None = None) -> int:
    """dA = dY Wo + sequence->head all-to-all (fuse::launch_oproj_backward_data)."""
    if options is None:
        return N.lib().fuse_launch_oproj_backward_data(C.byref(params), stream)
    return N.lib().fuse_launch_oproj_backward_data_ex(C.byref(params), _opt(options), stream)


def launch_oproj_backward_weight(params: OprojBackwardWeightParams, stream: int = 0) -> int:
    return N.lib().fuse_launch_oproj_backward_weight(C.byref(params), stream)


def launch_oproj_backward(params: OprojBackwardParams, stream: int = 0) -> int:
    return N.lib().fuse_launch_oproj_backward(C.byref(params), stream)


def qkv_backward_ready_elements(params: QkvBackwardDataParams) -> int:
    return N.lib().fuse_qkv_backward_ready_elements(C.byref(params))


def oproj_backward_ready_elements(params: OprojBackwardDataParams) -> int:
    return N.lib().fuse_oproj_backward_ready_elements(C.byref(params))


# ---- MXFP8 (include/fuse/operators/primitives/gemm_a2a_mxfp8.h of the reference) ----------------
from ._native import Mxfp8Activation, Mxfp8GemmA2AParams  # noqa: E402,F401


def gemm_a2a_mxfp8_activation_size(problem: GemmProblem):
    data, scales = C.c_size_t(), C.c_size_t()
    rc = N.lib().fuse_gemm_a2a_mxfp8_activation_size(C.byref(problem), C.byref(data), C.byref(scales))
    return rc, data.value, scales.value


def gemm_a2a_mxfp8_workspace_size(problem: GemmProblem):
    size = C.c_size_t()
    rc = N.lib().fuse_gemm_a2a_mxfp8_workspace_size(C.byref(problem), C.byref(size))
    return rc, size.value


def quantize_gemm_a2a_mxfp8_activation(problem: GemmProblem, source: int, output: Mxfp8Activation, stream: int = 0) -> int:
    return N.lib().fuse_quantize_gemm_a2a_mxfp8_activation(C.byref(problem), source, C.byref(output), stream)


def launch_gemm_a2a_mxfp8_cutlass(params: Mxfp8GemmA2AParams, stream: int = 0, options: Options | None = None) -> int:
    """MXFP8 QKV projection (weight quantised in-kernel) + all-to-all, BF16 out."""
    if options is None:
        return N.lib().fuse_launch_gemm_a2a_mxfp8_cutlass(C.byref(params), stream)
    return N.lib().fuse_launch_gemm_a2a_mxfp8_cutlass_ex(C.byref(params), _opt(options), stream)


def prepare_gemm_a2a_mxfp8(params: Mxfp8GemmA2AParams, stream: int = 0) -> int:
    return N.lib().fuse_prepare_gemm_a2a_mxfp8(C.byref(params), stream)


def launch_gemm_a2a_mxfp8_prequantized(params: Mxfp8GemmA2AParams, stream: int = 0, options: Options | None = None) -> int:
    if options is None:
        return N.lib().fuse_launch_gemm_a2a_mxfp8_prequantized(C.byref(params), stream)
    return N.lib().fuse_launch_gemm_a2a_mxfp8_prequantized_ex(C.byref(params), _opt(options), stream)


def launch_gemm_a2a_mxfp8_compute_reference(params: Mxfp8GemmA2AParams, stream: int = 0) -> int:
    return N.lib().fuse_launch_gemm_a2a_mxfp8_compute_reference(C.byref(params), stream)


def quantize_mxfp8(source: int, row_stride: int, rows: int, k: int, data: int, scales: int, stream: int = 0) -> int:
    return N.lib().fuse_b200_quantize_mxfp8(source, row_stride, rows, k, data, scales, stream)


def quantize_mxfp8_transposed(source: int, row_stride: int, rows: int, cols: int, data: int, scales: int,
                              stream: int = 0) -> int:
    return N.lib().fuse_b200_quantize_mxfp8_transposed(source, row_stride, rows, cols, data, scales, stream)


def mxfp8_scale_bytes(rows: int, k: int) -> int:
    return int(N.lib().fuse_b200_mxfp8_scale_bytes(rows, k))


from ._native import Mxfp8A2AGemmParams  # noqa: E402,F401


def a2a_gemm_mxfp8_activation_size(problem: GemmProblem, route: UlyssesRoute):
    data, scales = C.c_size_t(), C.c_size_t()
    rc = N.lib().fuse_a2a_gemm_mxfp8_activation_size(C.byref(problem), C.byref(route), C.byref(data), C.byref(scales))
    return rc, data.value, scales.value


def a2a_gemm_mxfp8_workspace_size(problem):
    """Both reference overloads (include/fuse/operators/primitives/a2a_gemm_mxfp8.h:50-51): a
    GemmProblem or a whole Mxfp8A2AGemmParams record."""
    size = C.c_size_t()
    if isinstance(problem, Mxfp8A2AGemmParams):
        rc = N.lib().fuse_a2a_gemm_mxfp8_workspace_size_for_params(C.byref(problem), C.byref(size))
    else:
        rc = N.lib().fuse_a2a_gemm_mxfp8_workspace_size(C.byref(problem), C.byref(size))
    return rc, size.value


def mxfp8_qkv_cutlass_kernel_traits(epilogue_n: int = 64) -> KernelTraits:
    """include/fuse/operators/primitives/gemm_a2a_mxfp8.h:41."""
    out = KernelTraits()
    N.lib().fuse_mxfp8_qkv_cutlass_kernel_traits(epilogue_n, C.byref(out))
    return out


def mxfp8_oproj_cutlass_kernel_traits(epilogue_n: int = 32, overlap_postnorm: bool = False) -> KernelTraits:
    """include/fuse/operators/primitives/a2a_gemm_mxfp8.h:52."""
    out = KernelTraits()
    N.lib().fuse_mxfp8_oproj_cutlass_kernel_traits(epilogue_n, int(overlap_postnorm), C.byref(out))
    return out


def a2a_gemm_mxfp8_staging_view(params: Mxfp8A2AGemmParams) -> Mxfp8Activation:
    out = Mxfp8Activation()
    rc = N.lib().fuse_a2a_gemm_mxfp8_staging_view(C.byref(params), C.byref(out))
    if rc != 0:
        raise RuntimeError(f"a2a_gemm_mxfp8_staging_view -> cudaError {rc}")
    return out


def launch_a2a_gemm_mxfp8_cutlass(params: Mxfp8A2AGemmParams, stream: int = 0, options: Options | None = None) -> int:
    """MXFP8 head->sequence all-to-all (bytes + scale atoms) + output projection, BF16 out."""
    if options is None:
        return N.lib().fuse_launch_a2a_gemm_mxfp8_cutlass(C.byref(params), stream)
    return N.lib().fuse_launch_a2a_gemm_mxfp8_cutlass_ex(C.byref(params), _opt(options), stream)


# ---- MoE dispatch + grouped GEMM (include/fuse/operators/primitives/grouped_gemm.h) -------------
from ._native import Bf16GroupedGemmParams, GroupedGemmPolicy  # noqa: E402,F401


def create_bf16_a2a_grouped_gemm(params: Bf16GroupedGemmParams):
    """Returns (cudaError, plan handle).  Allocates private device metadata: call outside capture."""
    plan = C.c_void_p()
    rc = N.lib().fuse_create_bf16_a2a_grouped_gemm(C.byref(params), C.byref(plan))
    return rc, plan.value


def create_bf16_grouped_gemm_a2a(params: Bf16GroupedGemmParams):
    """The combine direction (expert FC2 -> rows scattered to the token owners): (cudaError, plan)."""
    plan = C.c_void_p()
    rc = N.lib().fuse_create_bf16_grouped_gemm_a2a(C.byref(params), C.byref(plan))
    return rc, plan.value


def launch_bf16_grouped_gemm(plan: int, stream: int = 0, options: Options | None = None) -> int:
    if options is None:
        return N.lib().fuse_launch_bf16_grouped_gemm(plan, stream)
    return N.lib().fuse_launch_bf16_grouped_gemm_ex(plan, _opt(options), stream)


def destroy_bf16_grouped_gemm(plan: int) -> int:
    return N.lib().fuse_destroy_bf16_grouped_gemm(plan)


# ---- MXFP8 backward (qkv_backward.h:196-283, oproj_backward.h:186-240 of the reference) ---------
from ._native import (Mxfp8OprojBackwardDataParams, Mxfp8OprojBackwardParams,  # noqa: E402,F401
                      Mxfp8OprojBackwardWeightParams, Mxfp8QkvBackwardDataParams, Mxfp8QkvBackwardInput,
                      Mxfp8QkvBackwardParams, Mxfp8QkvBackwardWeightParams)


def _size(fn, params):
    size = C.c_size_t()
    rc = fn(C.byref(params), C.byref(size))
    return rc, size.value


def qkv_backward_mxfp8_data_workspace_size(params: QkvBackwardDataParams):
    return _size(N.lib().fuse_qkv_backward_mxfp8_data_workspace_size, params)


def qkv_backward_mxfp8_weight_workspace_size(params: QkvBackwardWeightParams):
    return _size(N.lib().fuse_qkv_backward_mxfp8_weight_workspace_size, params)


def oproj_backward_mxfp8_data_workspace_size(params: OprojBackwardDataParams):
    return _size(N.lib().fuse_oproj_backward_mxfp8_data_workspace_size, params)


def oproj_backward_mxfp8_weight_workspace_size(params: OprojBackwardWeightParams):
    return _size(N.lib().fuse_oproj_backward_mxfp8_weight_workspace_size, params)


def launch_qkv_backward_mxfp8_data(params, stream: int = 0, options: Options | None = None) -> int:
    if options is None:
        return N.lib().fuse_launch_qkv_backward_mxfp8_data(C.byref(params), stream)
    return N.lib().fuse_launch_qkv_backward_mxfp8_data_ex(C.byref(params), _opt(options), stream)


def launch_qkv_backward_mxfp8_weight(params, stream: int = 0) -> int:
    return N.lib().fuse_launch_qkv_backward_mxfp8_weight(C.byref(params), stream)


def launch_qkv_backward_mxfp8(params, stream: int = 0) -> int:
    return N.lib().fuse_launch_qkv_backward_mxfp8(C.byref(params), stream)


def launch_oproj_backward_mxfp8_data(params, stream: int = 0, options: Options | None = None) -> int:
    if options is None:
        return N.lib().fuse_launch_oproj_backward_mxfp8_data(C.byref(params), stream)
    return N.lib().fuse_launch_oproj_backward_mxfp8_data_ex(C.byref(params), _opt(options), stream)


def launch_oproj_backward_mxfp8_weight(params, stream: int = 0) -> int:
    return N.lib().fuse_launch_oproj_backward_mxfp8_weight(C.byref(params), stream)


def launch_oproj_backward_mxfp8(params, stream: int = 0) -> int:
    return N.lib().fuse_launch_oproj_backward_mxfp8(C.byref(params), stream)


def launch_gemm_a2a_mxfp8_static(params: Mxfp8GemmA2AParams, stream: int = 0) -> int:
    """MXFP8 QKV operator with the library's built-in weight scratch (allocates nothing;
    weights whose scratch exceeds N.STATIC_SCRATCH_BYTES are rejected)."""
    return N.lib().fuse_b200_launch_gemm_a2a_mxfp8_static(C.byref(params), stream)
