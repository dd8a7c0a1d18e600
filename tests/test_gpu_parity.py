"""Parity of the CUDA kernels with the CPU oracle, through the C ABI, on a B200.

Bars (from the operator's definition): activation codes and scales, unpacked weights and
per-group integer dots bit-exact; fp32 outputs within 1e-3 of max|y|; fp16 stores within
2 fp16 ulp of the fp32 oracle rounded to fp16."""
import ctypes

import numpy as np
import pytest

import __graft_entry__ as entry
from oracle import qipack_oracle as qo
from tests import qi_testing as qt

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

OUTPUT_TOLERANCE = 1e-3  # max |y - oracle| / max |oracle|, fp32 accumulate
FP16_STORE_ULPS = 2


@pytest.fixture(scope="module")
def qi():
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    module = entry.load_package()
    module.lib()  # fails loudly if the CUDA library is missing: there is no fallback
    torch.cuda.set_device(0)
    return module


def up(array):
    return torch.from_numpy(np.ascontiguousarray(array)).cuda()


def half_bits(tensor):
    return tensor.cpu().numpy().view(np.uint16)


def check_status(qi):
    torch.cuda.synchronize()
    assert qi.kernel_status() == 0


# ---- activation quantiser -------------------------------------------------------------------

@pytest.mark.parametrize("m,k", [(1, 256), (3, 512), (128, 3072), (517, 1024), (256, 12288)])
@pytest.mark.parametrize("dtype", ["f32", "f16"])
def test_quantize_activations_bit_exact(qi, m, k, dtype):
    rng = np.random.default_rng(1000 + m + k)
    x16 = qt.make_activations(rng, m, k)
    x = x16 if dtype == "f16" else (x16.astype(np.float32) + rng.standard_normal((m, k), dtype=np.float32) * 1e-3)
    codes = torch.zeros(m, k // 2, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(m, k // 64, dtype=torch.float16, device="cuda")
    xd = up(x)
    if dtype == "f32":
        assert qi.w4a4_quantize_activations(xd, codes, scales, m, k) == 0
    else:
        assert qi.w4a4_quantize_activations_ex(xd, qi.DTYPE_F16, codes, scales, m, k) == 0
    check_status(qi)
    expected_codes, expected_scales = qo.quantize_activations(x)
    assert np.array_equal(half_bits(scales), expected_scales)
    assert np.array_equal(codes.cpu().numpy(), expected_codes)


def test_quantize_activations_rounding_ties(qi):
    # values that sit exactly on, and one fp32 step either side of, every rounding tie
    # (n + 0.5) * scale, so that the reciprocal shortcut must defer to the exact division
    rng = np.random.default_rng(77)
    m, k = 64, 1024
    # rotating H256(v) gives v back: build the wanted post-rotation values and rotate them
    target = np.zeros((m, k), dtype=np.float32)
    for row in range(m):
        for g in range(k // 64):
            scale = np.float16(rng.uniform(0.01, 2.0))
            peak = np.float32(scale) * np.float32(7.0)
            ties = (rng.integers(-7, 7, size=64).astype(np.float32) + np.float32(0.5)) * np.float32(scale)
            nudge = rng.integers(-2, 3, size=64)
            values = ties.copy()
            for _ in range(2):
                values = np.where(nudge > 0, np.nextafter(values, np.float32(np.inf)), values)
                values = np.where(nudge < 0, np.nextafter(values, np.float32(-np.inf)), values)
                nudge = nudge - np.sign(nudge)
            values[0] = peak
            target[row, g * 64:(g + 1) * 64] = values
    x = qo.hadamard_256(target)
    codes = torch.zeros(m, k // 2, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(m, k // 64, dtype=torch.float16, device="cuda")
    assert qi.w4a4_quantize_activations(up(x), codes, scales, m, k) == 0
    check_status(qi)
    expected_codes, expected_scales = qo.quantize_activations(x)
    assert np.array_equal(half_bits(scales), expected_scales)
    assert np.array_equal(codes.cpu().numpy(), expected_codes)


def test_quantize_activations_zero_and_tiny_rows(qi):
    m, k = 8, 512
    x = np.zeros((m, k), dtype=np.float32)
    x[1, :] = 1e-9
    x[2, 5] = 1e-7
    x[3, :] = -3e-8
    x[4, 0::2] = 65504.0
    codes = torch.full((m, k // 2), 0xAB, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(m, k // 64, dtype=torch.float16, device="cuda")
    assert qi.w4a4_quantize_activations(up(x), codes, scales, m, k) == 0
    check_status(qi)
    expected_codes, expected_scales = qo.quantize_activations(x)
    assert np.array_equal(half_bits(scales), expected_scales)
    assert np.array_equal(codes.cpu().numpy(), expected_codes)
    assert np.all(expected_scales[0] == 1)  # the 2^-24 floor (gemm.cu:45)


def test_quantize_rejects_bad_shapes(qi):
    x = torch.zeros(4, 320, device="cuda")
    out = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    assert qi.w4a4_quantize_activations(x, out, out, 4, 320) == qi.CUDA_ERROR_INVALID_VALUE
    assert qi.w4a4_quantize_activations(x, out, out, 0, 256) == 0  # empty input: nothing to do
    assert qi.w4a4_quantize_activations(None, out, out, 4, 256) == qi.CUDA_ERROR_INVALID_VALUE


def test_f32_to_f16_bit_exact(qi):
    rng = np.random.default_rng(3)
    for count in (1, 7, 8, 4099, 1 << 20):
        x = np.concatenate([rng.standard_normal(count).astype(np.float32) * np.float32(10.0 ** rng.integers(-8, 5)),
                            ])[:count]
        out = torch.zeros(count, dtype=torch.float16, device="cuda")
        assert qi.f32_to_f16(up(x), out, count) == 0
        torch.cuda.synchronize()
        assert np.array_equal(half_bits(out), qo.f32_to_f16(x))
        on_stream = torch.zeros(count, dtype=torch.float16, device="cuda")
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        assert qi.f32_to_f16_ex(up(x), on_stream, count, stream.cuda_stream) == 0
        stream.synchronize()
        assert np.array_equal(half_bits(on_stream), qo.f32_to_f16(x))


# ---- W4A16 ---------------------------------------------------------------------------------------

def test_w4a16_dequantize_bit_exact(qi):
    rng = np.random.default_rng(11)
    n, k = 384, 1024
    for source in ("packer", "packer_clip", "random", "wide"):
        if source.startswith("packer"):
            codes, scales, minimums = qt.pack_w4a16(qt.make_weights(rng, n, k), clip=source.endswith("clip"))
        elif source == "random":
            codes, scales, minimums = qt.random_w4a16_pack(rng, n, k)
        else:  # |w| up to 1: the edge of the range where a single rounding equals the reference's two
            codes = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
            scales = rng.uniform(0.01, 0.12, size=(n, k // 64)).astype(np.float16).view(np.uint16)
            minimums = rng.uniform(-0.95, -0.85, size=(n, k // 64)).astype(np.float16).view(np.uint16)
        out = torch.zeros(n, k, dtype=torch.float16, device="cuda")
        assert qi.w4a16_dequantize_ex(up(codes), up(scales), up(minimums), out, n, k) == 0
        torch.cuda.synchronize()
        expected = qo.w4a16_dequantize(codes, scales, minimums)
        assert np.abs(expected.astype(np.float32)).max() <= 1.0
        assert np.array_equal(half_bits(out), expected.view(np.uint16)), source


@pytest.mark.parametrize("tile", [1, 2, 3, 4, 5])
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (256, 256, 512), (384, 640, 1024), (128, 384, 3072)])
def test_w4a16_gemm_matches_oracle(qi, tile, m, n, k):
    rng = np.random.default_rng(2000 + m + n + k)
    codes, scales, minimums = qt.pack_w4a16(qt.make_weights(rng, n, k))
    x16 = qt.make_activations(rng, m, k)
    y = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    assert qi.w4a16_gemm_tile_ex(up(x16), up(codes), up(scales), up(minimums), None, y, qi.DTYPE_F32, n, m, n, k,
                                 tile) == 0
    check_status(qi)
    expected = qo.w4a16_gemm(x16, codes, scales, minimums)
    assert qt.max_relative_error(y.cpu().numpy(), expected) <= OUTPUT_TOLERANCE


def test_w4a16_gemm_default_tiles_large(qi):
    # the block shapes' to_q linear at 512x512 image size: m=1024, n=k=3072, checked on sampled rows
    rng = np.random.default_rng(31)
    m, n, k = 1024, 3072, 3072
    codes, scales, minimums = qt.pack_w4a16(qt.make_weights(rng, n, k))
    x16 = qt.make_activations(rng, m, k)
    y = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    assert qi.w4a16_gemm(up(x16), up(codes), up(scales), up(minimums), y, m, n, k) == 0
    check_status(qi)
    got = y.cpu().numpy()
    assert np.isfinite(got).all()
    rows = np.sort(rng.choice(m, size=48, replace=False))
    expected = qo.w4a16_gemm(x16[rows], codes, scales, minimums)
    assert qt.max_relative_error(got[rows], expected) <= OUTPUT_TOLERANCE


def test_w4a16_gemm_ex_bias_fp16_and_leading_dimension(qi):
    rng = np.random.default_rng(41)
    m, n, k, ldy = 200, 256, 512, 512  # m is not a multiple of 128: the _ex form takes any m > 8
    codes, scales, minimums = qt.pack_w4a16(qt.make_weights(rng, n, k))
    x16, bias = qt.make_activations(rng, m, k), qt.make_bias(rng, n)
    expected = qo.w4a16_gemm(x16, codes, scales, minimums, bias=bias)
    wide = torch.full((m, ldy), -7.0, dtype=torch.float32, device="cuda")
    assert qi.w4a16_gemm_ex(up(x16), up(codes), up(scales), up(minimums), up(bias), wide[:, 128:], qi.DTYPE_F32, ldy,
                            m, n, k) == 0
    check_status(qi)
    got = wide.cpu().numpy()
    assert qt.max_relative_error(got[:, 128:128 + n], expected) <= OUTPUT_TOLERANCE
    assert np.all(got[:, :128] == -7.0) and np.all(got[:, 128 + n:] == -7.0)  # nothing outside the slice
    y16 = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    assert qi.w4a16_gemm_ex(up(x16), up(codes), up(scales), up(minimums), up(bias), y16, qi.DTYPE_F16, n, m, n, k) == 0
    check_status(qi)
    distance, checked = qt.fp16_store_error(y16.cpu().numpy(), expected)
    assert distance <= FP16_STORE_ULPS and checked > 0.5
    assert qt.max_relative_error(y16.cpu().numpy().astype(np.float32), expected) <= OUTPUT_TOLERANCE


def test_w4a16_gemm_rejects_what_the_reference_rejects(qi):  # gemm.cu:264
    t = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    assert qi.w4a16_gemm(t, t, t, t, t, 100, 128, 64) == qi.CUDA_ERROR_INVALID_VALUE
    assert qi.w4a16_gemm(t, t, t, t, t, 128, 120, 64) == qi.CUDA_ERROR_INVALID_VALUE
    assert qi.w4a16_gemm(t, t, t, t, t, 128, 128, 96) == qi.CUDA_ERROR_INVALID_VALUE
    assert qi.w4a16_gemm(None, t, t, t, t, 128, 128, 64) == qi.CUDA_ERROR_INVALID_VALUE


@pytest.mark.parametrize("m", [1, 2, 8])
@pytest.mark.parametrize("n,k,kind", [(256, 64, "silu"), (1024, 1216, "silu"), (18432, 3072, "silu"),
                                      (3072, 12288, "outliers")])
def test_w4a16_gemv_matches_oracle(qi, m, n, k, kind):
    rng = np.random.default_rng(3000 + m + n + k)
    if n * k > (1 << 22):
        codes, scales, minimums = qt.random_w4a16_pack(rng, n, k)
    else:
        codes, scales, minimums = qt.pack_w4a16(qt.make_weights(rng, n, k))
    x16, bias = qt.make_activations(rng, m, k, kind), qt.make_bias(rng, n)
    expected = qo.w4a16_gemm(x16, codes, scales, minimums, bias=bias)
    y = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    assert qi.w4a16_gemv_ex(up(x16), up(codes), up(scales), up(minimums), up(bias), y, qi.DTYPE_F32, n, m, n, k) == 0
    torch.cuda.synchronize()
    assert qt.max_relative_error(y.cpu().numpy(), expected) <= OUTPUT_TOLERANCE
    y16 = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    assert qi.w4a16_gemm_ex(up(x16), up(codes), up(scales), up(minimums), up(bias), y16, qi.DTYPE_F16, n, m, n, k) == 0
    torch.cuda.synchronize()
    distance, _ = qt.fp16_store_error(y16.cpu().numpy(), expected)
    assert distance <= FP16_STORE_ULPS


@pytest.mark.parametrize("m", [1, 3])
def test_w4a16_gemv_scales_of_every_size(qi, m):
    # scales from fp16 denormals up to 4: the GEMV's unpack treats scale >= 1/16 (where scale * 2^20 leaves fp16)
    # and denormal scales on paths of their own; every one must give the reference's weights
    n, k = 512, 1024
    rng = np.random.default_rng(3100 + m)
    codes = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    exponents = rng.integers(-20, 3, size=(n, k // 64)).astype(np.float32)
    scales = (np.exp2(exponents) * rng.uniform(1.0, 2.0, size=exponents.shape)).astype(np.float16)
    scales[::7, ::3] = np.float16(0.0)
    minimums = (-7.5 * scales.astype(np.float32)).astype(np.float16)
    x16 = qt.make_activations(rng, m, k, "silu")
    expected = qo.w4a16_gemm(x16, codes, scales.view(np.uint16), minimums.view(np.uint16))
    y = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    assert qi.w4a16_gemv_ex(up(x16), up(codes), up(scales.view(np.uint16)), up(minimums.view(np.uint16)), None, y,
                            qi.DTYPE_F32, n, m, n, k) == 0
    torch.cuda.synchronize()
    assert qt.max_relative_error(y.cpu().numpy(), expected) <= OUTPUT_TOLERANCE


@pytest.mark.parametrize("m,count,n,k", [(1, 3, 1024, 1216), (1, 70, 256, 512), (2, 5, 18432, 3072)])
def test_w4a16_gemv_grouped_matches_oracle_and_the_single_launches(qi, m, count, n, k):
    """Several matrices of one shape against the same activations in one launch (two for more than 64 matrices): every
    output equals the oracle's within the tolerance and the single-matrix GEMV's bit for bit."""
    rng = np.random.default_rng(3200 + m + count + n + k)
    x16 = qt.make_activations(rng, m, k, "silu")
    x = up(x16)
    entries, singles, expected = [], [], []
    for index in range(count):
        codes, scales, minimums = qt.random_w4a16_pack(rng, n, k)
        bias = qt.make_bias(rng, n) if index % 2 == 0 else None
        device = (up(codes), up(scales), up(minimums), up(bias) if bias is not None else None,
                  torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda"))
        entries.append(device)
        single = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        assert qi.w4a16_gemv_ex(x, device[0], device[1], device[2], device[3], single, qi.DTYPE_F32, n, m, n, k) == 0
        singles.append(single)
        if index < 4 or index == count - 1:  # the oracle on a few of them; the single launches cover the rest
            expected.append((index, qo.w4a16_gemm(x16, codes, scales, minimums, bias=bias)))
    table, keep = qi.gemv_items(entries)
    assert qi.w4a16_gemv_grouped_ex(x, table, qi.DTYPE_F32, n, m, n, k) == 0
    torch.cuda.synchronize()
    check_status(qi)
    for index, (entry, single) in enumerate(zip(entries, singles)):
        assert torch.equal(entry[4], single), index
    for index, want in expected:
        assert qt.max_relative_error(entries[index][4].cpu().numpy(), want) <= OUTPUT_TOLERANCE
    # refused: no items, a misaligned region, rows too long for the streaming kernel
    assert qi.lib().qi_w4a16_gemv_grouped_ex(qi._p(x), table, 0, qi.DTYPE_F32, n, m, n, k, None) == qi.CUDA_ERROR_INVALID_VALUE
    bad, _ = qi.gemv_items([(entries[0][0].view(-1)[1:], entries[0][1], entries[0][2], None, entries[0][4])])
    assert qi.w4a16_gemv_grouped_ex(x, bad, qi.DTYPE_F32, n, m, n, k) == qi.CUDA_ERROR_INVALID_VALUE
    assert qi.w4a16_gemv_grouped_ex(x, table, qi.DTYPE_F32, n, m, n, 8192) == qi.CUDA_ERROR_INVALID_VALUE


# ---- W4A4 ----------------------------------------------------------------------------------------

@pytest.mark.parametrize("m,n,k", [(128, 128, 256), (256, 384, 512), (128, 256, 3072), (384, 128, 1280)])
def test_w4a4_gemm_matches_oracle_and_dots_are_exact(qi, m, n, k):
    rng = np.random.default_rng(4000 + m + n + k)
    w_codes, w_scales = qt.pack_w4a4(qt.make_weights(rng, n, k))
    a_codes, a_scales = qo.quantize_activations(qt.make_activations(rng, m, k))
    y = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    args = (up(a_codes), up(a_scales), up(w_codes), up(w_scales))
    assert qi.w4a4_gemm(*args, y, m, n, k) == 0
    check_status(qi)
    expected = qo.w4a4_gemm(a_codes, a_scales, w_codes, w_scales)
    got = y.cpu().numpy()
    assert qt.max_relative_error(got, expected) <= OUTPUT_TOLERANCE
    # same fused multiply-adds in the same order as the reference kernel: expect the very bits
    assert np.array_equal(got, expected)
    dots = torch.full((m, n, k // 64), 12345, dtype=torch.int32, device="cuda")
    y2 = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    assert qi.w4a4_group_dots_ex(*args, y2, dots, m, n, k) == 0
    check_status(qi)
    assert np.array_equal(dots.cpu().numpy(), qo.w4a4_group_dots(a_codes, w_codes))
    assert np.array_equal(y2.cpu().numpy(), got)


def test_w4a4_gemm_extreme_codes_and_scales(qi):
    # every code at +-7 (largest |dot| = 64*49) and scales from the 2^-24 floor to large
    m, n, k = 128, 128, 512
    a_codes = np.full((m, k // 2), 0x77, dtype=np.uint8)
    a_codes[1::2] = 0x99
    w_codes = np.full((n, k // 2), 0x77, dtype=np.uint8)
    w_codes[2::3] = 0x99
    w_codes[5::7] = 0x97
    rng = np.random.default_rng(9)
    a_scales = rng.choice(np.array([2.0 ** -24, 1e-3, 0.5, 30.0], dtype=np.float16), size=(m, k // 64)).view(np.uint16)
    w_scales = rng.choice(np.array([2.0 ** -24, 1e-4, 0.01, 2.0], dtype=np.float16), size=(n, k // 64)).view(np.uint16)
    y = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    dots = torch.zeros(m, n, k // 64, dtype=torch.int32, device="cuda")
    assert qi.w4a4_group_dots_ex(up(a_codes), up(a_scales), up(w_codes), up(w_scales), y, dots, m, n, k) == 0
    check_status(qi)
    assert np.array_equal(dots.cpu().numpy(), qo.w4a4_group_dots(a_codes, w_codes))
    assert np.array_equal(y.cpu().numpy(), qo.w4a4_gemm(a_codes, a_scales, w_codes, w_scales))


def test_w4a4_gemm_ex_bias_fp16_and_leading_dimension(qi):
    rng = np.random.default_rng(51)
    m, n, k, ldy = 256, 256, 768, 384
    w_codes, w_scales = qt.pack_w4a4(qt.make_weights(rng, n, k))
    a_codes, a_scales = qo.quantize_activations(qt.make_activations(rng, m, k, "gelu"))
    bias = qt.make_bias(rng, n)
    expected = qo.w4a4_gemm(a_codes, a_scales, w_codes, w_scales, bias=bias)
    args = (up(a_codes), up(a_scales), up(w_codes), up(w_scales), up(bias))
    wide = torch.full((m, ldy), 3.0, dtype=torch.float32, device="cuda")
    assert qi.w4a4_gemm_ex(*args, wide, qi.DTYPE_F32, ldy, m, n, k) == 0
    check_status(qi)
    got = wide.cpu().numpy()
    assert qt.max_relative_error(got[:, :n], expected) <= OUTPUT_TOLERANCE
    assert np.all(got[:, n:] == 3.0)
    y16 = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    assert qi.w4a4_gemm_ex(*args, y16, qi.DTYPE_F16, n, m, n, k) == 0
    check_status(qi)
    distance, checked = qt.fp16_store_error(y16.cpu().numpy(), expected)
    assert distance <= FP16_STORE_ULPS and checked > 0.5


def test_w4a4_gemm_block_shape_sampled(qi):
    # attention-out shape of the 1024x1024 block (m=4096, n=k=3072): full-size run, sampled rows
    rng = np.random.default_rng(61)
    m, n, k = 4096, 3072, 3072
    w_codes, w_scales = qt.random_w4a4_pack(rng, n, k, 1e-3, 6e-3)
    a_codes, a_scales = qt.random_w4a4_pack(rng, m, k, 0.05, 0.6)
    y = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    assert qi.w4a4_gemm(up(a_codes), up(a_scales), up(w_codes), up(w_scales), y, m, n, k) == 0
    check_status(qi)
    got = y.cpu().numpy()
    assert np.isfinite(got).all()
    rows = np.sort(rng.choice(m, size=32, replace=False))
    expected = qo.w4a4_gemm(a_codes[rows], a_scales[rows], w_codes, w_scales)
    assert np.array_equal(got[rows], expected)


@pytest.mark.parametrize("m,n,k", [(256, 384, 512), (512, 256, 3072), (200, 256, 768), (256, 256, 640)])
def test_w4a4_gemm_paths_give_the_same_bits(qi, m, n, k):
    """The packed-operand entry point on each of its kernels: the int8 kernel on nibbles, and both operands widened
    into scratch memory for the byte-operand kernel on CTA pairs (twice in a row: the scratch is taken and returned
    in stream order)."""
    rng = np.random.default_rng(4500 + m + n + k)
    if k % 256 == 0:
        w_codes, w_scales = qt.pack_w4a4(qt.make_weights(rng, n, k))
        a_codes, a_scales = qo.quantize_activations(qt.make_activations(rng, m, k))
    else:  # not a length the H256 format has, but one the int8 kernel takes (two groups per stage)
        w_codes, w_scales = qt.random_w4a4_pack(rng, n, k, 1e-3, 6e-3)
        a_codes, a_scales = qt.random_w4a4_pack(rng, m, k, 0.05, 0.6)
    bias = qt.make_bias(rng, n)
    expected = qo.w4a4_gemm(a_codes, a_scales, w_codes, w_scales, bias=bias)
    args = (up(a_codes), up(a_scales), up(w_codes), up(w_scales), up(bias))
    paths = [qi.W4A4_PATH_INT8, qi.W4A4_PATH_BY_SHAPE] + ([qi.W4A4_PATH_WIDENED] * 2 if k % 256 == 0 else [])
    for path in paths:
        y = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        assert qi.w4a4_gemm_path_ex(*args, y, qi.DTYPE_F32, n, m, n, k, path) == 0
        check_status(qi)
        assert np.array_equal(y.cpu().numpy(), expected), path
    torch.cuda.synchronize()
    assert qi.w4a4_scratch_trim() == 0  # the pool gives back what no call holds; the next call takes it again
    y = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    assert qi.w4a4_gemm_path_ex(*args, y, qi.DTYPE_F32, n, m, n, k, qi.W4A4_PATH_BY_SHAPE) == 0
    check_status(qi)
    assert np.array_equal(y.cpu().numpy(), expected)
    assert qi.w4a4_gemm_path_ex(*args, y, qi.DTYPE_F32, n, m, n, k, 3) == qi.CUDA_ERROR_INVALID_VALUE
    if k % 256 != 0:  # the pair kernel's stage is four groups
        assert qi.w4a4_gemm_path_ex(*args, y, qi.DTYPE_F32, n, m, n, k, qi.W4A4_PATH_WIDENED) == qi.CUDA_ERROR_INVALID_VALUE


def test_w4a4_gemm_rejects_what_the_reference_rejects(qi):  # gemm.cu:185
    t = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    assert qi.w4a4_gemm(t, t, t, t, t, 100, 128, 256) == qi.CUDA_ERROR_INVALID_VALUE
    assert qi.w4a4_gemm(t, t, t, t, t, 128, 100, 256) == qi.CUDA_ERROR_INVALID_VALUE
    assert qi.w4a4_gemm(t, t, t, t, t, 128, 128, 128) == qi.CUDA_ERROR_INVALID_VALUE
    assert qi.w4a4_gemm(t, None, t, t, t, 128, 128, 256) == qi.CUDA_ERROR_INVALID_VALUE


# ---- transformer::linear ---------------------------------------------------------------------------

def test_linear_dispatches_like_the_reference(qi):
    # transformer.cplus:673-713: q, k, v share one quantised / converted input (reuse_input)
    rng = np.random.default_rng(71)
    rows, n, k = 256, 384, 768
    x32 = qt.make_activations(rng, rows, k).astype(np.float32) + np.float32(1e-4)
    xd = up(x32)
    work = qi.LinearWork(torch.zeros(rows * k // 2, dtype=torch.uint8, device="cuda"),
                         torch.zeros(rows * k // 64, dtype=torch.float16, device="cuda"),
                         torch.zeros(rows * k, dtype=torch.float16, device="cuda"))
    a_codes, a_scales = qo.quantize_activations(x32)
    x_half = qo.f32_to_f16(x32).view(np.float16)
    for scheme in (qi.SCHEME_W4A4_H256, qi.SCHEME_W4A16):
        outputs = []
        for index in range(3):
            w16 = qt.make_weights(rng, n, k)
            if scheme == qi.SCHEME_W4A4_H256:
                codes, scales = qt.pack_w4a4(w16)
                record = qi.PackedLinear(scheme, n, k, up(codes), up(scales))
                expected = qo.w4a4_gemm(a_codes, a_scales, codes, scales)
            else:
                codes, scales, minimums = qt.pack_w4a16(w16)
                record = qi.PackedLinear(scheme, n, k, up(codes), up(scales), up(minimums))
                expected = qo.w4a16_gemm(x_half, codes, scales, minimums)
            y = torch.zeros(rows, n, dtype=torch.float32, device="cuda")
            assert qi.linear(record, work, xd, y, rows, reuse_input=index > 0) == 0
            check_status(qi)
            assert qt.max_relative_error(y.cpu().numpy(), expected) <= OUTPUT_TOLERANCE
            outputs.append(y)
    bad = qi.PackedLinear(3, n, k, xd, xd)
    assert qi.linear(bad, work, xd, outputs[0], rows) == qi.CUDA_ERROR_INVALID_VALUE


# ---- W4A4 on byte-wide (E4M3) operands ---------------------------------------------------------------

def e4m3_of_codes(codes):
    """Expected output of qi_w4a4_widen_codes_ex: the FP8 E4M3 encoding of each code in -8..7."""
    magnitude = np.array([0x00, 0x38, 0x40, 0x44, 0x48, 0x4A, 0x4C, 0x4E, 0x50], dtype=np.uint8)
    values = qo.unpack_codes(codes, True).astype(np.int32)
    return (magnitude[np.abs(values)] | np.where(values < 0, 0x80, 0)).astype(np.uint8)


def test_widen_codes_matches_e4m3_table(qi):
    rng = np.random.default_rng(91)
    rows, k = 96, 640
    codes = rng.integers(0, 256, size=(rows, k // 2), dtype=np.uint8)  # includes -8
    out = torch.zeros(rows, k, dtype=torch.uint8, device="cuda")
    assert qi.w4a4_widen_codes_ex(up(codes), out, rows, k) == 0
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), e4m3_of_codes(codes))


@pytest.mark.parametrize("dtype", ["f32", "f16"])
def test_quantize_wide_writes_the_same_codes_as_bytes(qi, dtype):
    rng = np.random.default_rng(93)
    m, k = 300, 1024
    x16 = qt.make_activations(rng, m, k)
    x = x16 if dtype == "f16" else x16.astype(np.float32)
    codes = torch.zeros(m, k // 2, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(m, k // 64, dtype=torch.float16, device="cuda")
    wide = torch.zeros(m, k, dtype=torch.uint8, device="cuda")
    x_dtype = qi.DTYPE_F16 if dtype == "f16" else qi.DTYPE_F32
    assert qi.w4a4_quantize_activations_wide_ex(up(x), x_dtype, codes, scales, wide, m, k) == 0
    torch.cuda.synchronize()
    expected_codes, expected_scales = qo.quantize_activations(x)
    assert np.array_equal(codes.cpu().numpy(), expected_codes)
    assert np.array_equal(half_bits(scales), expected_scales)
    assert np.array_equal(wide.cpu().numpy(), e4m3_of_codes(expected_codes))
    wide2 = torch.zeros(m, k, dtype=torch.uint8, device="cuda")
    assert qi.w4a4_quantize_activations_wide_ex(up(x), x_dtype, None, scales, wide2, m, k) == 0  # bytes only
    torch.cuda.synchronize()
    assert torch.equal(wide, wide2)


class WideKernel:
    """One of the two byte-operand kernels behind the same three calls."""

    def __init__(self, qi, single):
        self.qi, self.single = qi, single

    def gemm(self, a, sa, w, sw, bias, y, y_dtype, ldy, m, n, k):
        if self.single:
            return self.qi.w4a4_gemm_wide_single_ex(a, sa, w, sw, bias, y, y_dtype, ldy, None, m, n, k)
        return self.qi.w4a4_gemm_wide_ex(a, sa, w, sw, bias, y, y_dtype, ldy, m, n, k)

    def group_dots(self, a, sa, w, sw, y, dots, m, n, k):
        if self.single:
            return self.qi.w4a4_gemm_wide_single_ex(a, sa, w, sw, None, y, self.qi.DTYPE_F32, n, dots, m, n, k)
        return self.qi.w4a4_group_dots_wide_ex(a, sa, w, sw, y, dots, m, n, k)


@pytest.fixture(params=["pair", "single"])
def wide_kernel(request, qi):
    """Both byte-operand kernels: 256x128 tiles on CTA pairs (default) and 128x128 on single CTAs."""
    return WideKernel(qi, request.param == "single")


@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (256, 384, 512), (128, 256, 3072), (200, 160, 1280),
                                   (640, 768, 256)])
def test_w4a4_wide_gemm_bits_and_exact_dots(qi, wide_kernel, m, n, k):
    rng = np.random.default_rng(5000 + m + n + k)
    w_codes, w_scales = qt.random_w4a4_pack(rng, n, k, 1e-3, 6e-3)
    a_codes, a_scales = qt.random_w4a4_pack(rng, m, k, 0.05, 0.6)
    a_wide, w_wide = (torch.zeros(r, k, dtype=torch.uint8, device="cuda") for r in (m, n))
    assert qi.w4a4_widen_codes_ex(up(a_codes), a_wide, m, k) == 0
    assert qi.w4a4_widen_codes_ex(up(w_codes), w_wide, n, k) == 0
    y = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    dots = torch.full((m, n, k // 64), 12345, dtype=torch.int32, device="cuda")
    args = (a_wide, up(a_scales), w_wide, up(w_scales))
    assert wide_kernel.group_dots(*args, y, dots, m, n, k) == 0
    check_status(qi)
    assert np.array_equal(dots.cpu().numpy(), qo.w4a4_group_dots(a_codes, w_codes))
    expected = qo.w4a4_gemm(a_codes, a_scales, w_codes, w_scales)
    assert np.array_equal(y.cpu().numpy(), expected)
    bias = qt.make_bias(rng, n)
    y16 = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    assert wide_kernel.gemm(*args, up(bias), y16, qi.DTYPE_F16, n, m, n, k) == 0
    check_status(qi)
    distance, checked = qt.fp16_store_error(y16.cpu().numpy(), qo.w4a4_gemm(a_codes, a_scales, w_codes, w_scales, bias=bias))
    assert distance <= FP16_STORE_ULPS and checked > 0.25


@pytest.mark.parametrize("m,n,k", [(2304, 2048, 1024), (1000, 1280, 3072), (4096, 3072, 640), (333, 4224, 2048),
                                   (2048, 1152, 12288)])
def test_w4a4_wide_gemm_equals_packed_kernel_on_many_tiles(qi, wide_kernel, m, n, k):
    # Shapes with more tiles than CTA pairs, ragged row counts and long K: every CTA walks several tiles and the
    # pipelines wrap many times. The byte-operand kernels must give the packed kernel's bits, launch after launch.
    generator = torch.Generator(device="cuda").manual_seed(m + n + k)
    def signed_codes(rows):
        v = torch.randint(-7, 8, (rows, k), dtype=torch.int16, device="cuda", generator=generator) & 0xF
        return (v[:, 0::2] | (v[:, 1::2] << 4)).to(torch.uint8).contiguous()
    a_codes, w_codes = signed_codes(m), signed_codes(n)
    a_scales = (torch.rand(m, k // 64, device="cuda", generator=generator) * 0.5 + 0.05).half()
    w_scales = (torch.rand(n, k // 64, device="cuda", generator=generator) * 5e-3 + 1e-3).half()
    a_wide, w_wide = (torch.zeros(r, k, dtype=torch.uint8, device="cuda") for r in (m, n))
    assert qi.w4a4_widen_codes_ex(a_codes, a_wide, m, k) == 0
    assert qi.w4a4_widen_codes_ex(w_codes, w_wide, n, k) == 0
    expected = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    assert qi.w4a4_gemm_ex(a_codes, a_scales, w_codes, w_scales, None, expected, qi.DTYPE_F32, n, m, n, k) == 0
    check_status(qi)
    for _ in range(4):
        y = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        assert wide_kernel.gemm(a_wide, a_scales, w_wide, w_scales, None, y, qi.DTYPE_F32, n, m, n, k) == 0
        check_status(qi)
        assert torch.equal(y, expected)


def test_w4a4_wide_gemm_extreme_dots(qi, wide_kernel):
    # all codes +-7: every group dot is +-3136, the largest the format allows; fp32 accumulation must stay exact
    m, n, k = 128, 128, 512
    a_codes = np.full((m, k // 2), 0x77, dtype=np.uint8)
    a_codes[1::2] = 0x99
    w_codes = np.full((n, k // 2), 0x77, dtype=np.uint8)
    w_codes[2::3] = 0x99
    w_codes[5::7] = 0x97
    ones = np.full((m, k // 64), np.float16(1.0)).view(np.uint16)
    a_wide, w_wide = (torch.zeros(r, k, dtype=torch.uint8, device="cuda") for r in (m, n))
    assert qi.w4a4_widen_codes_ex(up(a_codes), a_wide, m, k) == 0
    assert qi.w4a4_widen_codes_ex(up(w_codes), w_wide, n, k) == 0
    y = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    dots = torch.zeros(m, n, k // 64, dtype=torch.int32, device="cuda")
    assert wide_kernel.group_dots(a_wide, up(ones), w_wide, up(ones[:n]), y, dots, m, n, k) == 0
    check_status(qi)
    expected = qo.w4a4_group_dots(a_codes, w_codes)
    assert np.abs(expected).max() == 3136
    assert np.array_equal(dots.cpu().numpy(), expected)


def test_linear_takes_the_wide_path_when_given_wide_operands(qi):
    rng = np.random.default_rng(95)
    rows, n, k = 256, 384, 768
    x32 = qt.make_activations(rng, rows, k).astype(np.float32)
    codes, scales = qt.pack_w4a4(qt.make_weights(rng, n, k))
    wide_w = torch.zeros(n, k, dtype=torch.uint8, device="cuda")
    assert qi.w4a4_widen_codes_ex(up(codes), wide_w, n, k) == 0
    work = qi.LinearWork(torch.zeros(rows * k // 2, dtype=torch.uint8, device="cuda"),
                         torch.zeros(rows * k // 64, dtype=torch.float16, device="cuda"),
                         torch.zeros(rows * k, dtype=torch.float16, device="cuda"),
                         wide=torch.zeros(rows * k, dtype=torch.uint8, device="cuda"))
    record = qi.PackedLinear(qi.SCHEME_W4A4_H256, n, k, up(codes), up(scales), weights_wide=wide_w)
    y = torch.zeros(rows, n, dtype=torch.float32, device="cuda")
    assert qi.linear(record, work, up(x32), y, rows) == 0
    check_status(qi)
    a_codes, a_scales = qo.quantize_activations(x32)
    assert np.array_equal(y.cpu().numpy(), qo.w4a4_gemm(a_codes, a_scales, codes, scales))
    assert work.wide.abs().sum().item() > 0  # the byte arena was really used


# ---- a wait that runs out ------------------------------------------------------------------------------

def test_a_wait_that_runs_out_reports_its_code_and_leaves_the_device_healthy(qi):
    # every device-side wait of the library is bounded; this makes one run out on purpose (a barrier nothing
    # arrives on, limit 1 ms) and follows the error path a caller would see: code set, cleared by reading it,
    # and the next launches unaffected
    assert qi.kernel_status() == 0
    assert qi.probe_wait_timeout(1_000_000) == 0
    torch.cuda.synchronize()
    code = qi.kernel_status()
    assert code == 0x0001A000, hex(code)
    assert qi.kernel_status() == 0  # reading clears it
    assert qi.probe_wait_timeout(0) == qi.CUDA_ERROR_INVALID_VALUE
    assert qi.probe_wait_timeout(10**9) == qi.CUDA_ERROR_INVALID_VALUE
    rng = np.random.default_rng(808)
    m, n, k = 256, 256, 512
    w_codes, w_scales = qt.random_w4a4_pack(rng, n, k, 1e-3, 6e-3)
    a_codes, a_scales = qt.random_w4a4_pack(rng, m, k, 0.05, 0.6)
    y = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    assert qi.w4a4_gemm(up(a_codes), up(a_scales), up(w_codes), up(w_scales), y, m, n, k) == 0
    check_status(qi)
    assert np.array_equal(y.cpu().numpy(), qo.w4a4_gemm(a_codes, a_scales, w_codes, w_scales))


@pytest.mark.parametrize("dtype_name", ["f16", "f32"])
def test_w4a4_scatter_epilogue_keeps_inside_a_slice_that_ends_within_a_tile(qi, dtype_name):
    """The GEMM that stores its slice into several copies of the whole output, on one GPU with two local buffers as the
    copies: n = 160 ends inside the kernel's 128-column tile, so the tile's last 96 columns must not be written. Canary
    values around the slice, in every copy, stay as they were."""
    import ctypes
    rng = np.random.default_rng(8100)
    m, n, k, ldy, column = 256, 160, 512, 512, 32
    w_codes, w_scales = qt.random_w4a4_pack(rng, n, k, 1e-3, 6e-3)
    a_codes, a_scales = qt.random_w4a4_pack(rng, m, k, 0.05, 0.6)
    expected = qo.w4a4_gemm(a_codes, a_scales, w_codes, w_scales)
    a_wide = torch.zeros(m, k, dtype=torch.uint8, device="cuda")
    w_wide = torch.zeros(n, k, dtype=torch.uint8, device="cuda")
    assert qi.w4a4_widen_codes_ex(up(a_codes), a_wide, m, k) == 0
    assert qi.w4a4_widen_codes_ex(up(w_codes), w_wide, n, k) == 0
    dtype, torch_dtype = (qi.DTYPE_F16, torch.float16) if dtype_name == "f16" else (qi.DTYPE_F32, torch.float32)
    outputs = [torch.full((m, ldy), -3.0, dtype=torch_dtype, device="cuda") for _ in range(2)]
    copies = (ctypes.c_void_p * 2)(*[t.data_ptr() for t in outputs])
    assert qi.w4a4_gemm_wide_scatter_ex(a_wide, up(a_scales), w_wide, up(w_scales), None, copies, 1, dtype, ldy, column,
                                        m, n, k) == 0
    torch.cuda.synchronize()
    check_status(qi)
    for output in outputs:
        got = output.float().cpu().numpy()
        assert np.all(got[:, :column] == -3.0) and np.all(got[:, column + n:] == -3.0)
        if dtype == qi.DTYPE_F32:
            assert np.array_equal(got[:, column:column + n], expected)
        else:
            distance, checked = qt.fp16_store_error(output[:, column:column + n].cpu().numpy(), expected)
            assert distance <= FP16_STORE_ULPS and checked > 0.5
