"""Record layouts against the reference's OWN headers: one translation unit includes
include/fuse/** of the reference and include/fuse_b200.h and static_asserts sizeof and the offset of
every member of every parameter record (g++ -fsyntax-only; host only).  Runs where the reference
tree is mounted ($FUSE_REF_ROOT, or a directory `reference` beside this repository); skipped elsewhere."""
import os
import re
import shutil
import subprocess

import pytest

from oracle import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# this library's C record -> the reference's C++ record
RECORDS = {
    "fuse_matrix_stride": "fuse::MatrixStride", "fuse_gemm_problem": "fuse::GemmProblem",
    "fuse_ulysses_route": "fuse::UlyssesRoute", "fuse_kernel_traits": "fuse::KernelTraits",
    "fuse_gemm_a2a_params": "fuse::GemmA2AParams", "fuse_a2a_gemm_params": "fuse::A2AGemmParams",
    "fuse_backward_gemm_tuning": "fuse::BackwardGemmTuning",
    "fuse_qkv_backward_data_params": "fuse::QkvBackwardDataParams",
    "fuse_qkv_backward_weight_params": "fuse::QkvBackwardWeightParams", "fuse_qkv_backward_params": "fuse::QkvBackwardParams",
    "fuse_oproj_backward_data_params": "fuse::OprojBackwardDataParams",
    "fuse_oproj_backward_weight_params": "fuse::OprojBackwardWeightParams",
    "fuse_oproj_backward_params": "fuse::OprojBackwardParams", "fuse_mxfp8_activation": "fuse::Mxfp8Activation",
    "fuse_mxfp8_gemm_a2a_params": "fuse::Mxfp8GemmA2AParams", "fuse_mxfp8_a2a_gemm_params": "fuse::Mxfp8A2AGemmParams",
    "fuse_grouped_token_source": "fuse::GroupedTokenSource", "fuse_grouped_gemm_policy": "fuse::GroupedGemmPolicy",
    "fuse_bf16_grouped_gemm_params": "fuse::Bf16GroupedGemmParams",
    "fuse_mxfp8_qkv_backward_input": "fuse::Mxfp8QkvBackwardInput",
    "fuse_mxfp8_qkv_backward_data_params": "fuse::Mxfp8QkvBackwardDataParams",
    "fuse_mxfp8_qkv_backward_weight_params": "fuse::Mxfp8QkvBackwardWeightParams",
    "fuse_mxfp8_qkv_backward_params": "fuse::Mxfp8QkvBackwardParams",
    "fuse_mxfp8_oproj_backward_data_params": "fuse::Mxfp8OprojBackwardDataParams",
    "fuse_mxfp8_oproj_backward_weight_params": "fuse::Mxfp8OprojBackwardWeightParams",
    "fuse_mxfp8_oproj_backward_params": "fuse::Mxfp8OprojBackwardParams",
}
REFERENCE_HEADERS = ["fuse/types.h", "fuse/layout/gemm.h", "fuse/layout/ulysses.h", "fuse/operators/primitives/gemm_a2a.h",
                     "fuse/operators/primitives/a2a_gemm.h", "fuse/operators/primitives/gemm_a2a_mxfp8.h",
                     "fuse/operators/primitives/a2a_gemm_mxfp8.h", "fuse/operators/primitives/grouped_gemm.h",
                     "fuse/operators/ulysses/backward_common.h", "fuse/operators/ulysses/qkv_backward.h",
                     "fuse/operators/ulysses/oproj_backward.h"]


def _members(body: str):
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = []
    for declaration in body.split(";"):
        for part in declaration.split(","):
            found = re.findall(r"(\w+)\s*$", re.sub(r"\[[^\]]*\]", "", part).strip())
            if found and declaration.strip():
                names.append(found[0])
    return names


def translation_unit() -> str:
    text = open(os.path.join(ROOT, "include", "fuse_b200.h")).read()
    lines = ["#include <cstddef>"] + [f'#include "{h}"' for h in REFERENCE_HEADERS] + ['#include "fuse_b200.h"']
    seen = set()
    for match in re.finditer(r"typedef struct (\w+) \{(.*?)\} (\w+);", text, re.S):
        name = match.group(1)
        if name not in RECORDS:
            continue
        seen.add(name)
        ref = RECORDS[name]
        lines.append(f'static_assert(sizeof({ref}) == sizeof({name}), "{name}: size");')
        for member in _members(match.group(2)):
            lines.append(f'static_assert(offsetof({ref}, {member}) == offsetof({name}, {member}), "{name}.{member}: offset");')
    assert seen == set(RECORDS), set(RECORDS) - seen
    lines.append("int main() { return 0; }")
    return "\n".join(lines) + "\n"


def test_translation_unit_covers_every_record_and_member():
    unit = translation_unit()
    assert unit.count("static_assert(sizeof(") == len(RECORDS)
    assert unit.count("offsetof(fuse::") >= 200  # every member of every record


def test_record_layouts_match_the_reference_headers(tmp_path):
    reference = O.reference_root()
    if not os.path.isdir(os.path.join(reference, "include", "fuse")):
        pytest.skip("the reference tree is not mounted here")
    compiler = shutil.which("g++", path="/usr/bin") or shutil.which("g++")
    if compiler is None:
        pytest.skip("no host C++ compiler")
    cutlass = subprocess.run(["python3", "-c", "import flashinfer, os; print(os.path.join(os.path.dirname(flashinfer.__file__), "
                              "'data', 'cutlass', 'include'))"], capture_output=True, text=True).stdout.strip()
    if not os.path.isdir(cutlass):
        pytest.skip("no CUTLASS headers for the reference's scalar types")
    source = tmp_path / "abi_layout.cpp"
    source.write_text(translation_unit())
    cmd = [compiler, "-std=c++17", "-fsyntax-only", "-Wno-invalid-offsetof", "-DFUSE_ARCH_SM103=1",
           f"-I{reference}/include", f"-I{ROOT}/include", "-I/usr/local/cuda/include", f"-I{cutlass}", str(source)]
    result = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert result.returncode == 0, result.stderr[-4000:]
