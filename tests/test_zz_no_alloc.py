"""The packed W4A4 GEMM that takes no memory from anywhere (its widened operands live in a fixed device array),
through the C ABI, against the entry point that takes them from the stream's pool. Collected last: the array is a
per-device resource of the library, and the test must pass on its own as well as after everything else has run."""
import os

import numpy as np
import pytest

import __graft_entry__ as entry
from tests import qi_testing as qt

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def qi():
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    module = entry.load_package()
    if not os.path.exists(module.LIB_PATH):
        module.build()
    module.lib()
    return module


def up(array):
    return torch.from_numpy(np.ascontiguousarray(array)).cuda()


def operands(rng, m, n, k):
    w_codes, w_scales = qt.random_w4a4_pack(rng, n, k, 1e-3, 6e-3)
    a_codes, a_scales = qt.random_w4a4_pack(rng, m, k, 0.05, 0.6)
    return up(a_codes), up(a_scales), up(w_codes), up(w_scales), up(qt.make_bias(rng, n))


def test_two_calls_in_a_row_match_the_pooled_entry_point(qi):
    rng = np.random.default_rng(7001)
    # two shapes, the second larger than the first: what the first call left in the array must not matter
    for m, n, k, dtype in ((384, 512, 1024, qi.DTYPE_F32), (1024, 768, 3072, qi.DTYPE_F16)):
        args = operands(rng, m, n, k)
        torch_dtype = torch.float32 if dtype == qi.DTYPE_F32 else torch.float16
        expected = torch.full((m, n), float("nan"), dtype=torch_dtype, device="cuda")
        assert qi.w4a4_gemm_ex(*args, expected, dtype, n, m, n, k) == 0
        for call in range(2):
            got = torch.full((m, n), float("nan"), dtype=torch_dtype, device="cuda")
            assert qi.w4a4_gemm_noalloc_ex(*args, got, dtype, n, m, n, k) == 0
            torch.cuda.synchronize()
            assert qi.kernel_status() == 0
            assert torch.equal(got, expected), (m, n, k, call)


def test_too_large_and_unfit_shapes_are_refused_before_anything_runs(qi):
    small = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    y = torch.zeros(1 << 16, dtype=torch.float32, device="cuda")
    # (m + n) k beyond the array: the sizes are checked before any pointer is used
    m = n = k = 8192
    assert (m + n) * k > qi.NOALLOC_SCRATCH_BYTES
    assert qi.w4a4_gemm_noalloc_ex(small, small, small, small, None, y, qi.DTYPE_F32, n, m, n, k) == qi.NOALLOC_TOO_LARGE
    # k must hold whole pipeline stages of the CTA-pair kernel; the scale arrays must be 8-byte aligned; no null operands
    assert qi.w4a4_gemm_noalloc_ex(small, small, small, small, None, y, qi.DTYPE_F32, 128, 128, 128, 128) == qi.CUDA_ERROR_INVALID_VALUE
    assert qi.w4a4_gemm_noalloc_ex(small, small[4:], small, small, None, y, qi.DTYPE_F32, 128, 128, 128, 256) == qi.CUDA_ERROR_INVALID_VALUE
    assert qi.w4a4_gemm_noalloc_ex(None, small, small, small, None, y, qi.DTYPE_F32, 128, 128, 128, 256) == qi.CUDA_ERROR_INVALID_VALUE
    torch.cuda.synchronize()
    assert qi.kernel_status() == 0
