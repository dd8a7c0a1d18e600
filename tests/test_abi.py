"""CPU-side checks of the boundary: the library loads without a GPU and exports every symbol
the header declares; the Python mirror of the reference's operator wrappers exists."""
import ctypes
import os
import re

import pytest

import __graft_entry__ as entry


@pytest.fixture(scope="module")
def qi():
    module = entry.load_package()
    if not os.path.exists(module.LIB_PATH):
        module.build()
    return module


def declared_symbols():
    header = open(os.path.join(entry.ROOT, "include", "qipack_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    return sorted(set(re.findall(r"\b(qi_[a-z0-9_]+)\s*\(", header)))


def test_library_loads_and_exports_every_declared_symbol(qi):
    names = declared_symbols()
    assert {"qi_w4a4_quantize_activations", "qi_w4a4_gemm", "qi_w4a16_gemm", "qi_f32_to_f16"} <= set(names)
    library = ctypes.CDLL(qi.LIB_PATH)
    for name in names:
        assert hasattr(library, name), f"{name} is declared in include/qipack_b200.h but not exported"
    assert qi.version().startswith("qipack_b200")


def test_python_mirror_covers_every_entry_point(qi):
    for name in declared_symbols():
        if name in ("qi_b200_version",):
            continue
        assert name in qi.SIGNATURES, f"{name} has no ctypes signature"
    # the reference's wrapper names (cuda.cplus:128-130) and its dispatcher (transformer.cplus:673)
    for wrapper in ("w4a4_quantize_activations", "w4a4_gemm", "w4a16_gemm", "f32_to_f16", "linear"):
        assert callable(getattr(qi, wrapper))


def test_shape_checks_need_no_device(qi):
    # gemm.cu:185,264: shape violations return cudaErrorInvalidValue before anything is launched
    assert qi.w4a4_gemm(0, 0, 0, 0, 0, 100, 128, 256) == qi.CUDA_ERROR_INVALID_VALUE
    assert qi.w4a4_gemm(0, 0, 0, 0, 0, 128, 128, 128) == qi.CUDA_ERROR_INVALID_VALUE
    assert qi.w4a16_gemm(0, 0, 0, 0, 0, 128, 100, 64) == qi.CUDA_ERROR_INVALID_VALUE
    assert qi.w4a16_gemm(0, 0, 0, 0, 0, 128, 128, 32) == qi.CUDA_ERROR_INVALID_VALUE
    assert qi.w4a4_quantize_activations(0, 0, 0, 4, 100) == qi.CUDA_ERROR_INVALID_VALUE
    assert qi.w4a16_gemv_ex(0, 0, 0, 0, 0, 0, 0, 128, 9, 128, 64) == qi.CUDA_ERROR_INVALID_VALUE
