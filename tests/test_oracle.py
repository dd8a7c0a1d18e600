"""Pins the CPU oracle: the reference's in-source known-answer tests
(qwen_image_cuda/src/int4_pack.cplus:854-938, qwen_image_cuda/src/half.cplus:81-90) and
golden vectors produced by the reference's NumPy evaluator (tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest

from oracle import qipack_oracle as qo


@pytest.fixture(scope="module")
def known(golden_dir):
    return np.load(os.path.join(golden_dir, "known_answers.npz"))


def signed(codes):
    c = codes.astype(np.int32)
    return np.where(c > 7, c - 16, c)


# ---- the reference's own unit tests ---------------------------------------------------

def test_half_round_trip_is_exact_for_representable_values(known):  # half.cplus:81-90
    for value in known["half_exact"]:
        assert qo.half_to_f32(qo.half_from_f32(float(value))) == float(value)
    for value, bits in zip(known["half_inputs"], known["half_bits"]):
        assert qo.half_from_f32(float(value)) == int(bits)


def test_half_matches_ieee_everywhere():
    # every fp16 bit pattern converts to fp32 like IEEE, and back to itself (NaNs excepted)
    bits = np.arange(65536, dtype=np.uint16)
    as_f32 = bits.view(np.float16).astype(np.float32)
    back = qo.f32_to_f16(as_f32)
    finite = ~np.isnan(as_f32)
    assert np.array_equal(back[finite], bits[finite])
    rng = np.random.default_rng(1)
    values = np.concatenate([rng.normal(0, 1, 20000), rng.normal(0, 1e-6, 20000), rng.normal(0, 3e4, 20000),
                             [0.0, -0.0, 65519.9, 65520.0, 2.0 ** -25, 2.0 ** -24 * 1.5]]).astype(np.float32)
    with np.errstate(over="ignore"):
        expected = values.astype(np.float16).view(np.uint16)
    assert np.array_equal(qo.f32_to_f16(values), expected)


def test_hadamard_256_is_an_involution(known):  # int4_pack.cplus:856-870
    x = known["involution_in"]
    twice = qo.hadamard_256(qo.hadamard_256(x))
    assert np.max(np.abs(twice - x)) < float(known["involution_tolerance"])


def test_affine_group_reconstructs_within_half_a_step(known):  # int4_pack.cplus:872-892
    values = known["affine_in"]
    codes, scale_bits, minimum_bits = qo.quantize_affine_group(values, clip=False)
    scale, minimum = qo.half_to_f32(scale_bits), qo.half_to_f32(minimum_bits)
    assert codes.max() <= 15
    rebuilt = codes.astype(np.float32) * np.float32(scale) + np.float32(minimum)
    assert np.all(np.abs(rebuilt - values) <= scale * 0.5 + float(known["affine_slack"]))


def test_symmetric_group_uses_signed_nibbles(known):  # int4_pack.cplus:894-908
    codes, scale_bits = qo.quantize_symmetric_group(known["symmetric_in"], clip=False)
    assert abs(qo.half_to_f32(scale_bits) - float(known["symmetric_scale"])) < float(known["symmetric_scale_tolerance"])
    assert list(codes[:4]) == list(known["symmetric_codes"])


def test_clipping_never_increases_group_error(known):  # int4_pack.cplus:910-938
    values = known["clip_in"]
    plain, plain_scale = qo.quantize_symmetric_group(values, clip=False)
    clipped, clipped_scale = qo.quantize_symmetric_group(values, clip=True)
    def error(codes, scale_bits):
        e = np.float32(0)
        for c, v in zip(signed(codes), values):
            d = np.float32(c) * np.float32(qo.half_to_f32(scale_bits)) - np.float32(v)
            e = np.float32(e + d * d)
        return e
    assert error(clipped, clipped_scale) <= error(plain, plain_scale)


# ---- golden vectors from the reference's NumPy evaluator ---------------------------------

@pytest.mark.parametrize("clip", [0, 1])
def test_w4a16_packer_matches_reference_evaluator(golden_dir, clip):
    g = np.load(os.path.join(golden_dir, "weights_w4a16.npz"))
    codes, scales, minimums = qo.pack_matrix(g["weights_f16"], qo.SCHEME_W4A16, bool(clip))
    assert np.array_equal(codes, g[f"codes_clip{clip}"])
    assert np.array_equal(scales, g[f"scales_clip{clip}"])
    assert np.array_equal(minimums, g[f"minimums_clip{clip}"])


@pytest.mark.parametrize("clip", [0, 1])
def test_w4a4_packer_matches_reference_evaluator(golden_dir, clip):
    g = np.load(os.path.join(golden_dir, "weights_w4a4.npz"))
    w = g["weights_f16"].view(np.float16).astype(np.float32)
    rotated = qo.hadamard_256(w)
    assert np.array_equal(rotated, g["rotated_f32"])
    codes, scales, _ = qo.pack_matrix(g["weights_f16"], qo.SCHEME_W4A4_H256, bool(clip))
    assert np.array_equal(scales, g[f"scales_clip{clip}"])
    assert np.array_equal(codes, g[f"codes_clip{clip}"])


def test_activation_quantiser_matches_reference_evaluator(golden_dir):
    g = np.load(os.path.join(golden_dir, "activations_w4a4.npz"))
    x16 = g["x_f16"].view(np.float16)
    codes, scales = qo.quantize_activations(x16)
    codes32, scales32 = qo.quantize_activations(x16.astype(np.float32))
    assert np.array_equal(codes, codes32) and np.array_equal(scales, scales32)
    # on these inputs the evaluator's peak*(1/7) and the kernel's peak/7 round alike in every group
    assert g["scale_rules_agree"].all()
    assert np.array_equal(scales, g["scales"])
    assert np.array_equal(codes, g["codes"])
    dequantized = qo.unpack_codes(codes, True).astype(np.float32).reshape(codes.shape[0], -1, 64) * \
        scales.view(np.float16).astype(np.float32)[..., None]
    assert np.array_equal(dequantized.reshape(codes.shape[0], -1), g["dequantized_f32"])


def test_linear_outputs_match_reference_evaluator(golden_dir):
    g = np.load(os.path.join(golden_dir, "linear_outputs.npz"))
    x16, w16 = g["x_f16"].view(np.float16), g["weights_f16"]
    # W4A16 g64 (no clip): y = fp16(x) @ dequant(W).T
    codes, scales, minimums = qo.pack_matrix(w16, qo.SCHEME_W4A16, False)
    y = qo.w4a16_gemm(x16, codes, scales, minimums)
    expected = g["y_w4a16_g64"]
    # the evaluator keeps code*scale+minimum in fp32; the kernel rounds it to fp16 first
    assert np.max(np.abs(y - expected)) <= 2e-3 * np.max(np.abs(expected))
    # W4A4 H256 g64 clip
    w_codes, w_scales, _ = qo.pack_matrix(w16, qo.SCHEME_W4A4_H256, True)
    a_codes, a_scales = qo.quantize_activations(x16)
    y4 = qo.w4a4_gemm(a_codes, a_scales, w_codes, w_scales)
    y4d = qo.w4a4_gemm(a_codes, a_scales, w_codes, w_scales, double=True)
    expected4 = g["y_w4a4_h256_g64_clip"]
    assert np.max(np.abs(y4 - y4d)) <= 1e-5 * np.max(np.abs(y4d))
    # identical codes and scales; only the fp32 summation order of the evaluator's matmul differs
    assert np.max(np.abs(y4d - expected4)) <= 1e-5 * np.max(np.abs(expected4))


# ---- internal consistency ------------------------------------------------------------------

def test_group_dots_and_fold_agree():
    rng = np.random.default_rng(7)
    m, n, k = 8, 24, 512
    a = rng.integers(0, 256, size=(m, k // 2), dtype=np.uint8)
    w = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    sa = rng.uniform(0.01, 0.2, size=(m, k // 64)).astype(np.float16).view(np.uint16)
    sw = rng.uniform(0.001, 0.01, size=(n, k // 64)).astype(np.float16).view(np.uint16)
    dots = qo.w4a4_group_dots(a, w)
    av, wv = qo.unpack_codes(a, True).astype(np.int32), qo.unpack_codes(w, True).astype(np.int32)
    expected = np.einsum("mgk,ngk->mng", av.reshape(m, -1, 64), wv.reshape(n, -1, 64))
    assert np.array_equal(dots, expected)
    y = qo.w4a4_gemm(a, sa, w, sw, double=True)
    scale = sa.view(np.float16).astype(np.float64)[:, None, :] * sw.view(np.float16).astype(np.float64)[None, :, :]
    assert np.allclose(y, (dots * scale).sum(-1), rtol=1e-6, atol=1e-9)


def test_dequantize_rounds_once_to_fp16():
    rng = np.random.default_rng(9)
    n, k = 16, 256
    codes = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    scales = rng.uniform(1e-3, 1e-2, size=(n, k // 64)).astype(np.float16)
    minimums = rng.uniform(-0.08, -0.01, size=(n, k // 64)).astype(np.float16)
    w = qo.w4a16_dequantize(codes, scales.view(np.uint16), minimums.view(np.uint16))
    c = qo.unpack_codes(codes, False).astype(np.float64).reshape(n, -1, 64)
    exact = c * scales.astype(np.float64)[..., None] + minimums.astype(np.float64)[..., None]
    # fmaf is exact before its single rounding; fp64 holds code*scale+minimum exactly
    assert np.array_equal(w.reshape(n, -1, 64), exact.astype(np.float32).astype(np.float16))


def test_packer_rejects_what_the_reference_rejects():
    w = np.zeros((4, 128), dtype=np.float16)
    with pytest.raises(ValueError):
        qo.pack_matrix(w, qo.SCHEME_W4A4_H256, True)  # k % 256 != 0 (int4_pack.cplus:590-596)
    with pytest.raises(ValueError):
        qo.pack_matrix(w, qo.SCHEME_W4A16, False, group=48)  # group must divide 256 (:523-525)
    qo.pack_matrix(w, qo.SCHEME_W4A16, False)


def test_fast_baselines_match_oracle():
    rng = np.random.default_rng(11)
    m, n, k = 40, 48, 512
    w16 = rng.normal(0, 0.02, size=(n, k)).astype(np.float16)
    x16 = rng.normal(0, 1, size=(m, k)).astype(np.float16)
    c5, s5, m5 = qo.pack_matrix(w16, qo.SCHEME_W4A16, False)
    y = qo.w4a16_gemm(x16, c5, s5, m5)
    assert np.allclose(qo.w4a16_linear_fast(x16, c5, s5, m5), y, rtol=1e-4, atol=1e-5)
    c6, s6, _ = qo.pack_matrix(w16, qo.SCHEME_W4A4_H256, True)
    ac, asc = qo.quantize_activations(x16)
    assert np.array_equal(qo.w4a4_linear_fast(x16, c6, s6), qo.w4a4_gemm(ac, asc, c6, s6))
