"""CPU-side checks of the drop-in boundary: the library loads, exports every symbol that
include/fuse_b200.h declares, its records have the layout the binding assumes, the launch
entry points reject bad parameters with the reference's error codes before touching a device,
and the host-side tile order is a bijection."""
import ctypes as C
import os
import re

import numpy as np

from fuse_b200 import _native as N
from fuse_b200 import api, synthetic
from oracle import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "fuse_b200.h")).read()
    return sorted(set(re.findall(r"FUSE_API\s+[\w\s\*]+?\b(fuse_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = declared_symbols()
    assert len(names) >= 14
    handle = C.CDLL(N.LIB_PATH)
    for name in names:
        assert hasattr(handle, name), name
    assert set(names) == set(N.SYMBOLS), set(names) ^ set(N.SYMBOLS)


def test_record_layouts_match_the_compiled_library():
    lib = N.lib()
    for record, cls in N.ABI_RECORDS.items():
        assert lib.fuse_b200_abi_sizeof(record) == C.sizeof(cls), cls.__name__
    assert lib.fuse_b200_abi_sizeof(99) == -1
    # Offsets the reference's C++ records have (include/fuse/layout/gemm.h:27-42,
    # include/fuse/layout/ulysses.h:24-63 under the Itanium ABI).
    assert N.GemmProblem.raster.offset == 104 and N.GemmProblem.transpose_a.offset == 100
    assert N.UlyssesRoute.packed_source_row.offset == 48 and N.UlyssesRoute.kind.offset == 60
    assert N.GemmA2AParams.gemm.offset == 168 and N.GemmA2AParams.num_comm_ctas.offset == 352
    assert N.A2AGemmParams.gemm.offset == 160 and N.A2AGemmParams.alpha.offset == 360


def test_parameter_validation_without_a_device():
    # csrc/operators/sm103/detail/launch.cuh:508-511: epoch 0, no communication CTAs, a
    # non-finite alpha or an unsupported problem are cudaErrorInvalidValue.
    good = N.GemmProblem(256, 384, 64)
    p = N.GemmA2AParams(gemm=good, num_comm_ctas=4, epoch=0)
    assert api.launch_gemm_a2a_cutlass(p) == N.CUDA_ERROR_INVALID_VALUE
    p = N.GemmA2AParams(gemm=good, num_comm_ctas=0, epoch=1)
    assert api.launch_gemm_a2a_cutlass(p) == N.CUDA_ERROR_INVALID_VALUE
    # ... while the _ex entry point takes 0 as Auto: validation passes, the launch then needs a device
    assert api.launch_gemm_a2a_cutlass(p, 0, N.Options()) != N.CUDA_ERROR_INVALID_VALUE
    p = N.GemmA2AParams(gemm=good, num_comm_ctas=4, epoch=1, alpha=float("inf"))
    assert api.launch_gemm_a2a_cutlass(p) == N.CUDA_ERROR_INVALID_VALUE
    for bad in (N.GemmProblem(0, 384, 64), N.GemmProblem(256, 384, 60), N.GemmProblem(256, 384, 64, max_swizzle_size=3),
                N.GemmProblem(256, 384, 64, transpose_b=1), N.GemmProblem(256, 384, 64, input_dtype=N.DTYPE_E4M3)):
        p = N.GemmA2AParams(gemm=bad, num_comm_ctas=4, epoch=1)
        assert api.launch_gemm_a2a_cutlass(p) == N.CUDA_ERROR_INVALID_VALUE
        q = N.A2AGemmParams(gemm=bad, num_comm_ctas=4, epoch=1)
        assert api.launch_a2a_gemm_cutlass(q) == N.CUDA_ERROR_INVALID_VALUE
    q = N.A2AGemmParams(gemm=good, num_comm_ctas=4, epoch=1, lhs_policy=2)
    assert api.launch_a2a_gemm_cutlass(q) == N.CUDA_ERROR_INVALID_VALUE
    assert N.lib().fuse_launch_gemm_a2a_cutlass(None, None) == N.CUDA_ERROR_INVALID_VALUE


def test_ready_sizes():
    prob = N.GemmProblem(16384, 6144, 4096)
    traits = api.qkv_cutlass_kernel_traits(prob)
    assert (traits.block_m, traits.threads) == (128, 256) and traits.block_n in (64, 128)
    assert api.qkv_ready_elements(prob) == 128 * (6144 // traits.block_n) * 32
    route = N.UlyssesRoute(world_size=8)
    assert api.a2a_lhs_gemm_ready_elements(N.GemmProblem(16384, 4096, 4096), route) == 128 * 8 * 32
    assert api.a2a_lhs_gemm_ready_elements(N.GemmProblem(130, 4096, 4096), route) == 2 * 8 * 32


def test_auto_budget_of_the_output_projection_pull():
    route = N.UlyssesRoute(world_size=8)
    for shape in ((16384, 4096, 4096), (32768, 8192, 8192), (256, 512, 512), (65536, 1024, 16384)):
        ctas = api.recommended_a2a_lhs_gemm_comm_ctas(N.GemmProblem(*shape), route)
        assert 4 <= ctas <= 48 and ctas % 2 == 0
    assert 4 <= api.recommended_gemm_a2a_comm_ctas(N.GemmProblem(16384, 6144, 4096), route) <= 48


def test_planner_follows_the_scorer_rules_of_the_reference():
    # csrc/operators/sm103/detail/autotune.cuh:25-75,109-203: minimise max(compute, transfer) over the
    # measured candidates; an explicit budget is used exactly and never changed; ties go to fewer
    # communication CTAs; the model is monotone in the bytes to move.
    c2 = dict(flops=2.0 * 16384 * 4096 * 4096, nbytes=16384 * 4096 * 2.0, tiles=64 * 16)
    auto = api.plan(0, **c2)
    assert auto["embedded"] and auto["comm_ctas"] == 0             # B200: no SM given up when the copy warp can be embedded
    for budget in (8, 20, 32):
        explicit = api.plan(0, explicit_comm_ctas=budget, **c2)
        assert explicit["comm_ctas"] == budget and not explicit["embedded"]
        # Auto is the minimum over the candidates (a communication budget must beat the embedded warps by 10 %)
        assert explicit["makespan_us"] >= auto["makespan_us"] * 0.90 * (1 - 1e-9)
    ctas_only = api.plan(0, embedded_allowed=False, **c2)
    assert not ctas_only["embedded"] and ctas_only["comm_ctas"] in (4, 8, 12, 16, 20, 24, 32, 40, 48)
    candidates = [api.plan(0, explicit_comm_ctas=b, **c2)["makespan_us"] for b in (4, 8, 12, 16, 20, 24, 32, 40, 48)]
    assert abs(ctas_only["makespan_us"] - min(candidates)) <= 1e-9 * min(candidates)
    # the makespan covers the transfer and at least the GEMM on every SM (compute_us is the GEMM on
    # the compute CTAs alone; communication CTAs that join it afterwards can only shorten that)
    assert ctas_only["makespan_us"] >= ctas_only["transfer_us"]
    assert ctas_only["compute_us"] * (148 - ctas_only["comm_ctas"]) / 148 * 0.9 <= ctas_only["makespan_us"] <= ctas_only["compute_us"] * 1.001
    # more bytes to move never lowers the budget of the communication-CTA plan, nor the makespan
    last_budget, last_span = 0, 0.0
    for scale in (0.25, 1.0, 4.0, 16.0):
        plan = api.plan(0, c2["flops"], c2["nbytes"] * scale, c2["tiles"], embedded_allowed=False)
        assert plan["comm_ctas"] >= last_budget and plan["makespan_us"] >= last_span * (1 - 1e-9)
        last_budget, last_span = plan["comm_ctas"], plan["makespan_us"]
    # over NVLink (share of remote bytes = (world - 1) / world): pulls stay on the embedded copy warps, the
    # gradient push moves to communication CTAs (at least 16) beyond the calibrated share, and the
    # MoE dispatch on one-CTA tiles gets a larger budget the more of its rows are remote
    bwd = dict(flops=2.0 * 16384 * 4096 * 6144, nbytes=16384 * 6144 * 2.0, tiles=64 * 16)
    assert api.plan(0, remote_share=7 / 8, **c2)["embedded"]
    assert api.plan(2, remote_share=0.5, **bwd)["embedded"]
    far = api.plan(2, remote_share=0.75, **bwd)
    assert not far["embedded"] and far["comm_ctas"] >= 16
    c5 = dict(flops=2.0 * 65536 * 4096 * 7168, nbytes=65536 * 7168 * 2.0, tiles=512 * 16, group=1, embedded_allowed=False)
    budgets = [api.plan(6, remote_share=share, **c5)["comm_ctas"] for share in (0.0, 0.5, 0.75, 0.875)]
    assert budgets == sorted(budgets) and budgets[-1] > budgets[0]
    # budgets of CTA-pair kernels come in pairs; every kind answers; bad requests are rejected
    for kind in range(7):
        plan = api.plan(kind, 1.0e12, 5.0e8, 2048, group=2)
        assert plan["comm_ctas"] % 2 == 0 and plan["comm_ctas"] < 148 and plan["makespan_us"] > 0
    import pytest
    for bad in (dict(kind=7), dict(kind=0, explicit_comm_ctas=148), dict(kind=0, tiles=0)):
        args = dict(kind=0, flops=1e12, nbytes=1e8, tiles=100)
        args.update(bad)
        with pytest.raises(ValueError):
            api.plan(**args)


def test_mxfp8_traits_and_workspace_overloads():
    for traits in (api.mxfp8_qkv_cutlass_kernel_traits(64), api.mxfp8_qkv_cutlass_kernel_traits(32),
                   api.mxfp8_oproj_cutlass_kernel_traits(32, False), api.mxfp8_oproj_cutlass_kernel_traits(64, True)):
        assert (traits.block_m, traits.block_n, traits.block_k, traits.threads) == (128, 256, 128, 256)
        assert 114 * 1024 < traits.dynamic_smem_bytes <= 227 * 1024
    # the reference returns an empty record for an epilogue width it has no kernel for
    assert api.mxfp8_qkv_cutlass_kernel_traits(48).block_m == 0
    prob = N.GemmProblem(4096, 8192, 8192)
    params = N.Mxfp8A2AGemmParams()
    params.projection.gemm = prob
    by_problem = api.a2a_gemm_mxfp8_workspace_size(prob)
    assert by_problem[0] == 0 and by_problem[1] > 0
    assert api.a2a_gemm_mxfp8_workspace_size(params) == by_problem


def test_tile_order_is_a_bijection_and_bands_are_compact():
    lib = N.lib()
    for (mt, nt) in [(1, 1), (7, 5), (128, 24), (16, 3), (3, 16), (9, 9)]:
        for swizzle in (1, 2, 4, 8):
            for along_n in (0, 1):
                seen = set()
                prev = None
                for linear in range(mt * nt):
                    m, n = C.c_int32(), C.c_int32()
                    assert lib.fuse_b200_tile_order_decode(mt, nt, swizzle, along_n, linear, C.byref(m), C.byref(n)) == 0
                    assert 0 <= m.value < mt and 0 <= n.value < nt
                    seen.add((m.value, n.value))
                    minor = m.value if along_n else n.value
                    if prev is not None:  # the banded axis never moves backwards by more than a band
                        assert minor // swizzle >= prev // swizzle
                    prev = minor
                assert len(seen) == mt * nt
    m, n = C.c_int32(), C.c_int32()
    assert lib.fuse_b200_tile_order_decode(4, 4, 3, 0, 0, C.byref(m), C.byref(n)) == 1
    assert lib.fuse_b200_tile_order_decode(4, 4, 2, 0, 16, C.byref(m), C.byref(n)) == 1


def test_swizzle_selection_matches_oracle():
    for cap in (1, 2, 4, 8):
        for mt in (1, 2, 3, 5, 6, 40):
            for nt in (1, 2, 3, 5, 6, 40):
                assert N.lib().fuse_b200_select_swizzle(cap, mt, nt) == O.lib().fo_swizzle_size(cap, mt, nt)


def test_philox_known_answers_and_value_map():
    kat = [((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
           ((0xffffffff,) * 4, (0xffffffff,) * 2, (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
           ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0),
            (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1))]
    for counter, key, want in kat:
        got = synthetic.philox4x32_10(np.array([counter], dtype=np.uint32), np.array(key, dtype=np.uint32))[0]
        assert tuple(int(x) for x in got) == want
    words = synthetic.random_words(70000, 1234)
    assert np.array_equal(words[:100], synthetic.random_words(100, 1234))  # prefix stable
    vals = synthetic.uniform_bf16((70000,), 1234, 0.125)
    expect = np.array([O.lib().fo_f32_to_bf16(O.lib().fo_uniform_value(int(w), 0.125)) for w in words[:2000]],
                      dtype=np.uint16)
    assert np.array_equal(vals[:2000], expect)
    z = synthetic.bf16_bits_to_f32(synthetic.normal_bf16((1 << 16,), 5, 0.02))
    assert abs(z.mean()) < 5e-4 and abs(z.std() - 0.02) < 5e-4


def test_header_compiles_as_plain_c():
    # the boundary is a C ABI: the header must be usable from C (cgo, ctypes generators, other FFIs)
    import shutil
    import subprocess
    import tempfile

    import pytest
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    with tempfile.TemporaryDirectory() as tmp:
        source = os.path.join(tmp, "abi.c")
        with open(source, "w") as f:
            f.write('#include "fuse_b200.h"\nint main(void) { fuse_gemm_problem p; (void)p; return (int)sizeof(fuse_ulysses_route) == 0; }\n')
        result = subprocess.run([gcc, "-std=c11", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only", "-I",
                                 os.path.join(ROOT, "include"), source], capture_output=True, text=True)
        assert result.returncode == 0, result.stderr
