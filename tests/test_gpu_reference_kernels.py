"""The reference's own kernels (qwen_image_cuda/cuda/gemm.cu, compiled unmodified for sm_100a
into oracle/_ref/ by `make -C oracle ref`) run beside the new ones on the same device buffers.
Skipped where that build is absent."""
import ctypes
import os

import numpy as np
import pytest

import __graft_entry__ as entry
from oracle import qipack_oracle as qo
from tests import qi_testing as qt

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

REF_PATH = os.path.join(entry.ROOT, "oracle", "_ref", "libqi_ref_gemm.so")


@pytest.fixture(scope="module")
def libs():
    if not os.path.exists(REF_PATH):
        pytest.skip("oracle/_ref/libqi_ref_gemm.so was not built (needs the reference tree)")
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    torch.cuda.set_device(0)
    ref = ctypes.CDLL(REF_PATH)
    P, I = ctypes.c_void_p, ctypes.c_int
    ref.qi_w4a4_quantize_activations.argtypes = [P, P, P, I, I]
    ref.qi_w4a4_gemm.argtypes = [P, P, P, P, P, I, I, I]
    ref.qi_w4a16_gemm.argtypes = [P, P, P, P, P, I, I, I]
    return entry.load_package(), ref


def up(array):
    return torch.from_numpy(np.ascontiguousarray(array)).cuda()


def ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def test_reference_kernels_agree_with_the_new_ones(libs):
    qi, ref = libs
    rng = np.random.default_rng(81)
    m, n, k = 256, 384, 1024
    x32 = qt.make_activations(rng, m, k).astype(np.float32) + rng.standard_normal((m, k), dtype=np.float32) * 1e-3
    xd = up(x32)
    w16 = qt.make_weights(rng, n, k)

    # activation quantiser: same bytes
    ours_c, ref_c = (torch.zeros(m, k // 2, dtype=torch.uint8, device="cuda") for _ in range(2))
    ours_s, ref_s = (torch.zeros(m, k // 64, dtype=torch.float16, device="cuda") for _ in range(2))
    assert ref.qi_w4a4_quantize_activations(ptr(xd), ptr(ref_c), ptr(ref_s), m, k) == 0
    assert qi.w4a4_quantize_activations(xd, ours_c, ours_s, m, k) == 0
    torch.cuda.synchronize()
    assert torch.equal(ours_c, ref_c) and torch.equal(ours_s.view(torch.int16), ref_s.view(torch.int16))
    oracle_c, oracle_s = qo.quantize_activations(x32)
    assert np.array_equal(ref_c.cpu().numpy(), oracle_c)  # and the oracle agrees with the reference itself

    # W4A4 GEMM: the same fused multiply-adds in the same order, so the same bits
    w_codes, w_scales = qt.pack_w4a4(w16)
    wc, ws = up(w_codes), up(w_scales)
    ours_y, ref_y = (torch.zeros(m, n, dtype=torch.float32, device="cuda") for _ in range(2))
    assert ref.qi_w4a4_gemm(ptr(ref_c), ptr(ref_s), ptr(wc), ptr(ws), ptr(ref_y), m, n, k) == 0
    assert qi.w4a4_gemm(ours_c, ours_s, wc, ws, ours_y, m, n, k) == 0
    torch.cuda.synchronize()
    assert qi.kernel_status() == 0
    assert torch.equal(ours_y, ref_y)
    assert np.array_equal(ref_y.cpu().numpy(), qo.w4a4_gemm(oracle_c, oracle_s, w_codes, w_scales))

    # W4A16 GEMM: same operands, different fp32 summation order inside the tensor cores
    codes, scales, minimums = qt.pack_w4a16(w16)
    x_half = torch.zeros(m, k, dtype=torch.float16, device="cuda")
    assert qi.f32_to_f16(xd, x_half, m * k) == 0
    c, s, z = up(codes), up(scales), up(minimums)
    assert ref.qi_w4a16_gemm(ptr(x_half), ptr(c), ptr(s), ptr(z), ptr(ref_y), m, n, k) == 0
    assert qi.w4a16_gemm(x_half, c, s, z, ours_y, m, n, k) == 0
    torch.cuda.synchronize()
    assert qi.kernel_status() == 0
    assert qt.max_relative_error(ours_y.cpu().numpy(), ref_y.cpu().numpy()) <= 1e-3
    expected = qo.w4a16_gemm(x_half.cpu().numpy(), codes, scales, minimums)
    assert qt.max_relative_error(ref_y.cpu().numpy(), expected) <= 1e-3
