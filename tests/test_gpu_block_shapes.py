"""Parity at the sizes that are benchmarked, through the C ABI, against the CPU oracle on sampled rows.

The byte-operand W4A4 kernel on CTA pairs (qi_w4a4_gemm_wide_ex, the bench's timed path) on the three
wide block linears at M = 4096 and on one M = 16384 shape; the W4A16 kernel on the text stream's
M = 256 at the four block shapes; both operators on the reference engine's own shapes
(N, K in {4096, 12288}, qwen_image_cuda/cuda/bench/bench_w4a4.cu:405-410) at M = 1024, there also
against the reference's kernels where oracle/_ref was built.

Bars: activation codes and scales bit-equal; W4A4 fp32 outputs bit-equal (same fused multiply-adds in the
reference's order, qwen_image_cuda/cuda/gemm.cu:159-168); W4A16 within 1e-3 of max|y|; fp16 stores within
2 fp16 ulp on the elements at or above 2^-6 max|y|, whose share is asserted."""
import ctypes
import os

import numpy as np
import pytest

import __graft_entry__ as entry
from oracle import qipack_oracle as qo
from tests import qi_testing as qt

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

OUTPUT_TOLERANCE = 1e-3
FP16_STORE_ULPS = 2
SAMPLED_ROWS = 24
REF_PATH = os.path.join(entry.ROOT, "oracle", "_ref", "libqi_ref_gemm.so")


@pytest.fixture(scope="module")
def qi():
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    module = entry.load_package()
    module.lib()
    torch.cuda.set_device(0)
    return module


@pytest.fixture(scope="module")
def reference_kernels():
    """The reference's own gemm.cu built for sm_100a, or None where the reference tree was absent at build time."""
    if not os.path.exists(REF_PATH):
        return None
    ref = ctypes.CDLL(REF_PATH)
    P, I = ctypes.c_void_p, ctypes.c_int
    ref.qi_w4a4_gemm.argtypes = [P, P, P, P, P, I, I, I]
    ref.qi_w4a16_gemm.argtypes = [P, P, P, P, P, I, I, I]
    return ref


def up(array):
    return torch.from_numpy(np.ascontiguousarray(array)).cuda()


def ptr(tensor):
    return ctypes.c_void_p(tensor.data_ptr())


def check_status(qi):
    torch.cuda.synchronize()
    assert qi.kernel_status() == 0


def sample_rows(rng, m):
    """Rows from every part of the matrix: the first and last tile included."""
    picked = set(rng.choice(m, size=SAMPLED_ROWS - 4, replace=False).tolist()) | {0, 127, m - 128, m - 1}
    return np.array(sorted(picked))


def quantise_wide(qi, x16, m, k):
    """The activation quantiser at full size: packed codes, scales and byte-wide codes on the device."""
    codes = torch.zeros(m, k // 2, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(m, k // 64, dtype=torch.float16, device="cuda")
    wide = torch.zeros(m, k, dtype=torch.uint8, device="cuda")
    assert qi.w4a4_quantize_activations_wide_ex(up(x16), qi.DTYPE_F16, codes, scales, wide, m, k) == 0
    check_status(qi)
    return codes, scales, wide


def w4a4_case(qi, rng, m, n, k, kind):
    w_codes, w_scales = qt.random_w4a4_pack(rng, n, k, 1e-3, 6e-3)
    x16 = qt.make_activations(rng, m, k, kind)
    a_codes, a_scales, a_wide = quantise_wide(qi, x16, m, k)
    rows = sample_rows(rng, m)
    expected_codes, expected_scales = qo.quantize_activations(x16[rows])
    assert np.array_equal(a_codes.cpu().numpy()[rows], expected_codes)
    assert np.array_equal(a_scales.cpu().numpy().view(np.uint16)[rows], expected_scales)
    w_wide = torch.zeros(n, k, dtype=torch.uint8, device="cuda")
    wc, ws = up(w_codes), up(w_scales)
    assert qi.w4a4_widen_codes_ex(wc, w_wide, n, k) == 0
    expected = qo.w4a4_gemm(expected_codes, expected_scales, w_codes, w_scales)
    return dict(rows=rows, expected=expected, a_codes=a_codes, a_scales=a_scales, a_wide=a_wide, w_codes=wc,
                w_scales=ws, w_wide=w_wide)


@pytest.mark.parametrize("name,n,k,kind", [("qkv", 9216, 3072, "outliers"), ("fc1", 12288, 3072, "outliers"),
                                           ("fc2", 3072, 12288, "gelu")])
def test_w4a4_pair_kernel_block_linears_m4096_against_oracle(qi, name, n, k, kind):
    m = 4096
    rng = np.random.default_rng(6100 + n + k)
    case = w4a4_case(qi, rng, m, n, k, kind)
    y = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    assert qi.w4a4_gemm_wide_ex(case["a_wide"], case["a_scales"], case["w_wide"], case["w_scales"], None, y,
                                qi.DTYPE_F32, n, m, n, k) == 0
    check_status(qi)
    assert torch.isfinite(y).all()
    assert np.array_equal(y.cpu().numpy()[case["rows"]], case["expected"]), name
    y16 = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    assert qi.w4a4_gemm_wide_ex(case["a_wide"], case["a_scales"], case["w_wide"], case["w_scales"], None, y16,
                                qi.DTYPE_F16, n, m, n, k) == 0
    check_status(qi)
    distance, checked = qt.fp16_store_error(y16.cpu().numpy()[case["rows"]], case["expected"])
    assert distance <= FP16_STORE_ULPS
    assert checked > 0.25, f"only {checked:.2f} of the sampled outputs are large enough for the ulp check"
    # every fp16 output is the fp32 output rounded once: checks the whole matrix, not only the sampled rows
    assert torch.equal(y16, y.half())


def test_w4a4_pair_kernel_m16384_against_oracle(qi):
    # the 2048 x 2048 image: 16384 tokens through the attention-out linear, 64 row tiles per CTA pair column
    m, n, k = 16384, 3072, 3072
    rng = np.random.default_rng(6401)
    case = w4a4_case(qi, rng, m, n, k, "outliers")
    y16 = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    assert qi.w4a4_gemm_wide_ex(case["a_wide"], case["a_scales"], case["w_wide"], case["w_scales"], None, y16,
                                qi.DTYPE_F16, n, m, n, k) == 0
    check_status(qi)
    distance, checked = qt.fp16_store_error(y16.cpu().numpy()[case["rows"]], case["expected"])
    assert distance <= FP16_STORE_ULPS and checked > 0.25
    # the drop-in kernel on nibble-packed codes gives the same matrix
    y_packed = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    assert qi.w4a4_gemm_ex(case["a_codes"], case["a_scales"], case["w_codes"], case["w_scales"], None, y_packed,
                           qi.DTYPE_F16, n, m, n, k) == 0
    check_status(qi)
    assert torch.equal(y_packed, y16)


@pytest.mark.parametrize("n,k,kind", [(9216, 3072, "outliers"), (3072, 3072, "outliers"), (12288, 3072, "outliers"),
                                      (3072, 12288, "gelu")])
def test_w4a16_text_stream_m256_against_oracle(qi, n, k, kind):
    m = 256
    rng = np.random.default_rng(6500 + n + k)
    codes, scales, minimums = qt.random_w4a16_pack(rng, n, k)
    x16 = qt.make_activations(rng, m, k, kind)
    rows = sample_rows(rng, m)
    expected = qo.w4a16_gemm(x16[rows], codes, scales, minimums)
    y = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    args = (up(x16), up(codes), up(scales), up(minimums))
    assert qi.w4a16_gemm(*args, y, m, n, k) == 0
    check_status(qi)
    assert torch.isfinite(y).all()
    assert qt.max_relative_error(y.cpu().numpy()[rows], expected) <= OUTPUT_TOLERANCE
    y16 = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    assert qi.w4a16_gemm_ex(*args, None, y16, qi.DTYPE_F16, n, m, n, k) == 0
    check_status(qi)
    distance, checked = qt.fp16_store_error(y16.cpu().numpy()[rows], expected)
    assert distance <= FP16_STORE_ULPS and checked > 0.25


@pytest.mark.parametrize("n,k", [(4096, 4096), (12288, 4096), (4096, 12288)])
def test_reference_native_shapes_m1024(qi, reference_kernels, n, k):
    # the reference engine's own widths (transformer.cplus:32-39): WIDTH 4096, MLP 12288
    m = 1024
    rng = np.random.default_rng(6600 + n + k)
    rows = sample_rows(rng, m)

    # scheme 6
    case = w4a4_case(qi, rng, m, n, k, "outliers")
    y = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    assert qi.w4a4_gemm(case["a_codes"], case["a_scales"], case["w_codes"], case["w_scales"], y, m, n, k) == 0
    check_status(qi)
    assert np.array_equal(y.cpu().numpy()[case["rows"]], case["expected"])
    y_wide = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    assert qi.w4a4_gemm_wide_ex(case["a_wide"], case["a_scales"], case["w_wide"], case["w_scales"], None, y_wide,
                                qi.DTYPE_F32, n, m, n, k) == 0
    check_status(qi)
    assert torch.equal(y_wide, y)
    if reference_kernels is not None:
        y_ref = torch.zeros(m, n, dtype=torch.float32, device="cuda")
        assert reference_kernels.qi_w4a4_gemm(ptr(case["a_codes"]), ptr(case["a_scales"]), ptr(case["w_codes"]),
                                              ptr(case["w_scales"]), ptr(y_ref), m, n, k) == 0
        torch.cuda.synchronize()
        assert torch.equal(y_ref, y)

    # scheme 5
    codes, scales, minimums = qt.random_w4a16_pack(rng, n, k)
    x16 = qt.make_activations(rng, m, k)
    expected = qo.w4a16_gemm(x16[rows], codes, scales, minimums)
    args = (up(x16), up(codes), up(scales), up(minimums))
    y5 = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    assert qi.w4a16_gemm(*args, y5, m, n, k) == 0
    check_status(qi)
    assert qt.max_relative_error(y5.cpu().numpy()[rows], expected) <= OUTPUT_TOLERANCE
    if reference_kernels is not None:
        y_ref = torch.zeros(m, n, dtype=torch.float32, device="cuda")
        assert reference_kernels.qi_w4a16_gemm(*(ptr(t) for t in args), ptr(y_ref), m, n, k) == 0
        torch.cuda.synchronize()
        assert qt.max_relative_error(y5.cpu().numpy(), y_ref.cpu().numpy()) <= OUTPUT_TOLERANCE


# ---- stacks of blocks through the dispatcher: configs 3 and 5 in small -------------------------------------

def run_linear(qi, record, work, x, rows, n):
    y = torch.full((rows, n), float("nan"), dtype=torch.float16, device="cuda")
    assert qi.linear(record, work, x, y, rows, input_dtype=qi.DTYPE_F16, output_dtype=qi.DTYPE_F16) == 0
    check_status(qi)
    return y.cpu().numpy()


def make_work(qi, rows, k_max):
    return qi.LinearWork(torch.zeros(rows * k_max // 2, dtype=torch.uint8, device="cuda"),
                         torch.zeros(rows * k_max // 64, dtype=torch.float16, device="cuda"),
                         torch.zeros(rows * k_max, dtype=torch.float16, device="cuda"),
                         wide=torch.zeros(rows * k_max, dtype=torch.uint8, device="cuda"))


SMALL_BLOCK = [("qkv", 768, 256, "outliers"), ("attn_out", 256, 256, "outliers"), ("fc1", 1024, 256, "outliers"),
               ("fc2", 256, 1024, "gelu")]  # the block's four linears at hidden 256: every (N, K) relation of the real ones


def test_two_blocks_of_the_w4a16_stack_with_text_stream_and_modulation(qi):
    # config 3 in small: per block the four linears on an image stream and on a text stream with its own weights
    # (both through qi_linear, scheme 5) and two M = 1 modulation linears (the GEMV path)
    rng = np.random.default_rng(7300)
    for block in range(2):
        for stream_name, rows in (("image", 384), ("text", 40)):
            work = make_work(qi, rows, 1024)
            for name, n, k, kind in SMALL_BLOCK:
                codes, scales, minimums = qt.pack_w4a16(qt.make_weights(rng, n, k))
                x16 = qt.make_activations(rng, rows, k, kind)
                record = qi.PackedLinear(qi.SCHEME_W4A16, n, k, up(codes), up(scales), up(minimums))
                got = run_linear(qi, record, work, up(x16), rows, n)
                expected = qo.w4a16_gemm(x16, codes, scales, minimums)
                assert qt.max_relative_error(got.astype(np.float32), expected) <= OUTPUT_TOLERANCE, (block, stream_name, name)
                distance, checked = qt.fp16_store_error(got, expected)
                assert distance <= FP16_STORE_ULPS and checked > 0.25, (block, stream_name, name)
        for _ in range(2):
            n, k = 6 * 256, 256
            codes, scales, minimums = qt.pack_w4a16(qt.make_weights(rng, n, k))
            x16 = qt.make_activations(rng, 1, k, "silu")
            record = qi.PackedLinear(qi.SCHEME_W4A16, n, k, up(codes), up(scales), up(minimums))
            got = run_linear(qi, record, make_work(qi, 1, k), up(x16), 1, n)
            expected = qo.w4a16_gemm(x16, codes, scales, minimums)
            assert qt.max_relative_error(got.astype(np.float32), expected) <= OUTPUT_TOLERANCE


def test_two_blocks_of_the_mixed_policy_stack_with_a_stacked_batch(qi):
    # config 5 in small: each linear is scheme 6 with probability 0.7, else scheme 5 (seeded, every block draws
    # both here), and the batch of two is two requests' rows stacked: rows = 2 x (image + text tokens). A row's
    # result must not depend on what is stacked with it.
    rng = np.random.default_rng(7500)
    policy = np.random.default_rng(7501)
    tokens = 3 * 64 + 24  # three images' tokens and a text stream, per request
    rows = 2 * tokens
    work = make_work(qi, rows, 1024)
    single = make_work(qi, tokens, 1024)
    schemes_seen = set()
    for block in range(2):
        for name, n, k, kind in SMALL_BLOCK:
            scheme6 = policy.random() < 0.7
            if block == 1 and name == "fc2" and len(schemes_seen) < 2:
                scheme6 = qi.SCHEME_W4A4_H256 not in schemes_seen  # make sure both schemes occur
            w16 = qt.make_weights(rng, n, k)
            x16 = qt.make_activations(rng, rows, k, kind)
            if scheme6:
                schemes_seen.add(qi.SCHEME_W4A4_H256)
                codes, scales = qt.pack_w4a4(w16)
                wide = torch.zeros(n, k, dtype=torch.uint8, device="cuda")
                assert qi.w4a4_widen_codes_ex(up(codes), wide, n, k) == 0
                record = qi.PackedLinear(qi.SCHEME_W4A4_H256, n, k, up(codes), up(scales), weights_wide=wide)
                a_codes, a_scales = qo.quantize_activations(x16)
                expected = qo.w4a4_gemm(a_codes, a_scales, codes, scales)
            else:
                schemes_seen.add(qi.SCHEME_W4A16)
                codes, scales, minimums = qt.pack_w4a16(w16)
                record = qi.PackedLinear(qi.SCHEME_W4A16, n, k, up(codes), up(scales), up(minimums))
                expected = qo.w4a16_gemm(x16, codes, scales, minimums)
            got = run_linear(qi, record, work, up(x16), rows, n)
            assert qt.max_relative_error(got.astype(np.float32), expected) <= OUTPUT_TOLERANCE, (block, name, scheme6)
            distance, checked = qt.fp16_store_error(got, expected)
            assert distance <= FP16_STORE_ULPS and checked > 0.25, (block, name, scheme6)
            if scheme6:  # exact operator: the stacked batch gives each request the bits it gets alone
                alone = run_linear(qi, record, single, up(x16[tokens:]), tokens, n)
                assert np.array_equal(alone, got[tokens:]), (block, name)
    assert schemes_seen == {qi.SCHEME_W4A4_H256, qi.SCHEME_W4A16}
