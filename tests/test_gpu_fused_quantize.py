"""The activation function fused into the quantiser gives the bytes of the two-kernel sequence it replaces:
the reference's element-wise kernel (qwen_image_cuda/cuda/ops.cu: qi_swiglu :133-145, qi_gelu_tanh :155-166,
compiled unmodified into oracle/_ref where the reference tree was present at build time) writing an [m, k]
float32 matrix, then the activation quantiser on that matrix. Without that build the element-wise step is
evaluated by torch with the same expression."""
import ctypes
import os

import numpy as np
import pytest

import __graft_entry__ as entry
from oracle import qipack_oracle as qo

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

REF_OPS = os.path.join(entry.ROOT, "oracle", "_ref", "libqi_ref_ops.so")


@pytest.fixture(scope="module")
def qi():
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    module = entry.load_package()
    module.lib()
    torch.cuda.set_device(0)
    return module


@pytest.fixture(scope="module")
def reference_ops():
    if not os.path.exists(REF_OPS):
        return None
    ref = ctypes.CDLL(REF_OPS)
    P = ctypes.c_void_p
    ref.qi_swiglu.argtypes = [P, P, P, ctypes.c_ulonglong]
    ref.qi_gelu_tanh.argtypes = [P, P, ctypes.c_ulonglong]
    return ref


def ptr(tensor):
    return ctypes.c_void_p(tensor.data_ptr())


@pytest.mark.parametrize("producer", ["swiglu", "gelu"])
@pytest.mark.parametrize("m,k", [(5, 256), (300, 1024), (512, 12288)])
def test_fused_producer_gives_the_unfused_bytes(qi, reference_ops, producer, m, k):
    generator = torch.Generator(device="cuda").manual_seed(1000 + m + k)
    first = torch.randn(m, k, device="cuda", generator=generator) * 2.0
    second = torch.randn(m, k, device="cuda", generator=generator)
    first[:, ::97] *= 12.0  # outlier channels
    between = torch.empty(m, k, device="cuda")
    if reference_ops is not None:
        if producer == "swiglu":
            assert reference_ops.qi_swiglu(ptr(first), ptr(second), ptr(between), m * k) == 0
        else:
            assert reference_ops.qi_gelu_tanh(ptr(first), ptr(between), m * k) == 0
        torch.cuda.synchronize()
    elif producer == "swiglu":
        between = first / (1.0 + torch.exp(-first)) * second
    else:
        between = 0.5 * first * (1.0 + torch.tanh(0.7978845608028654 * (first + 0.044715 * first * first * first)))

    def outputs():
        return (torch.zeros(m, k // 2, dtype=torch.uint8, device="cuda"), torch.zeros(m, k // 64, dtype=torch.float16, device="cuda"),
                torch.zeros(m, k, dtype=torch.uint8, device="cuda"))

    codes, scales, wide = outputs()
    assert qi.w4a4_quantize_activations_wide_ex(between, qi.DTYPE_F32, codes, scales, wide, m, k) == 0
    fused_codes, fused_scales, fused_wide = outputs()
    if producer == "swiglu":
        assert qi.w4a4_swiglu_quantize_ex(first, second, fused_codes, fused_scales, fused_wide, m, k) == 0
    else:
        assert qi.w4a4_gelu_quantize_ex(first, fused_codes, fused_scales, fused_wide, m, k) == 0
    torch.cuda.synchronize()
    assert qi.kernel_status() == 0
    assert torch.equal(fused_scales.view(torch.int16), scales.view(torch.int16))
    assert torch.equal(fused_codes, codes)
    assert torch.equal(fused_wide, wide)
    # and the unfused pair is what the oracle says for that float32 matrix
    expected_codes, expected_scales = qo.quantize_activations(between[:64].cpu().numpy())
    assert np.array_equal(codes[:64].cpu().numpy(), expected_codes)
    assert np.array_equal(scales[:64].cpu().numpy().view(np.uint16), expected_scales)
    # only one of the two code formats
    only_codes, scales2, _ = outputs()
    if producer == "swiglu":
        assert qi.w4a4_swiglu_quantize_ex(first, second, only_codes, scales2, None, m, k) == 0
    else:
        assert qi.w4a4_gelu_quantize_ex(first, only_codes, scales2, None, m, k) == 0
    torch.cuda.synchronize()
    assert torch.equal(only_codes, codes)


def test_fused_quantisers_reject_bad_arguments(qi):
    t = torch.zeros(1 << 16, device="cuda")
    out = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    assert qi.w4a4_swiglu_quantize_ex(t, None, out, out, out, 4, 256) == qi.CUDA_ERROR_INVALID_VALUE
    assert qi.w4a4_swiglu_quantize_ex(t, t, None, out, None, 4, 256) == qi.CUDA_ERROR_INVALID_VALUE
    assert qi.w4a4_gelu_quantize_ex(t, out, out, out, 4, 320) == qi.CUDA_ERROR_INVALID_VALUE
    assert qi.w4a4_gelu_quantize_ex(t, out, out, out, 0, 256) == 0
