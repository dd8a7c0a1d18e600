#!/usr/bin/env python3
"""Generate the golden vectors in this folder from the reference's own NumPy statement
of the QIPACK v6 quantisers and dequantise-and-matmul operator.

Run where the reference tree is mounted (it is imported, never copied):

    python tests/golden/make_golden.py [--reference /path/to/reference]

It imports ``tools/evaluate_int4_quantization.py`` from the reference and calls
``quantize_affine``, ``quantize_symmetric``, ``hadamard_256``, ``Mode.prepare`` and
``Mode.activations`` (tools/evaluate_int4_quantization.py:101-211) on seeded inputs
with the distributions the benchmark uses: W ~ N(0, 0.02) rounded to fp16,
X fp16 ~ N(0, 1) with a seeded 1 % of the input channels scaled by 20.

Outputs (small ``.npz`` files, committed):
  weights_w4a16.npz      codes/scales/minimums for clip in {0,1}
  weights_w4a4.npz       rotated symmetric codes/scales for clip in {0,1}
  activations_w4a4.npz   H256 + symmetric g64 codes/scales of X (NumPy rule) and the
                         dequantised activations
  linear_outputs.npz     y = act(x) @ prepare(W).T for w4a16-g64 and w4a4-h256-g64-clip
  known_answers.npz      inputs of the reference's in-source unit tests
                         (int4_pack.cplus:854-938, half.cplus:81-90) with the values
                         those tests assert

The activation rule differs between the two reference statements: the NumPy evaluator
computes ``fp16(peak * float32(1/7))`` (evaluate_int4_quantization.py:157) while the CUDA
kernel the engine runs computes ``fp16(peak / 7.0f)`` (gemm.cu:45). The kernel is the
operator being replaced, so activations_w4a4.npz also records, per group, whether the two
rules give the same fp16 scale; parity tests compare only those groups against this file
and all groups against the C oracle, which follows gemm.cu.
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(root: str):
    tools = os.path.join(root, "tools")
    sys.path.insert(0, tools)
    spec = importlib.util.spec_from_file_location(
        "evaluate_int4_quantization", os.path.join(tools, "evaluate_int4_quantization.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def make_weights(rng, n, k):
    return rng.normal(0.0, 0.02, size=(n, k)).astype(np.float32).astype(np.float16)


def make_activations(rng, m, k):
    x = rng.normal(0.0, 1.0, size=(m, k)).astype(np.float32)
    outliers = rng.choice(k, size=max(1, k // 100), replace=False)
    x[:, outliers] *= 20.0
    return x.astype(np.float16), np.sort(outliers)


def pack_nibbles(codes: np.ndarray) -> np.ndarray:
    """[rows,k] code values -> [rows,k/2] bytes, even column in the low nibble
    (int4_pack.cplus:414-419)."""
    c = codes.astype(np.int16) & 0xF
    return (c[:, 0::2] | (c[:, 1::2] << 4)).astype(np.uint8)


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", default=os.environ.get("QI_REFERENCE"), required="QI_REFERENCE" not in os.environ,
                        help="path of the netdur/qwen-image-cplus checkout (or set QI_REFERENCE)")
    args = parser.parse_args()
    ref = load_reference(args.reference)

    rng = np.random.default_rng(20240607)
    n, k, m = 96, 512, 48
    w16 = make_weights(rng, n, k)
    w = w16.astype(np.float32)
    x16, outliers = make_activations(rng, m, k)
    x = x16.astype(np.float32)

    # --- W4A16 weights (quantize_affine, :127-149)
    out = {"weights_f16": w16.view(np.uint16)}
    for clip in (0, 1):
        codes, scale, minimum = ref.quantize_affine(w, 64, bool(clip))
        out[f"codes_clip{clip}"] = pack_nibbles(codes)
        out[f"scales_clip{clip}"] = scale.astype(np.float16).view(np.uint16)
        out[f"minimums_clip{clip}"] = minimum.astype(np.float16).view(np.uint16)
    np.savez_compressed(os.path.join(HERE, "weights_w4a16.npz"), **out)

    # --- W4A4 weights (hadamard_256 :101-115, quantize_symmetric :152-171)
    rotated = ref.hadamard_256(w)
    out = {"weights_f16": w16.view(np.uint16), "rotated_f32": rotated.astype(np.float32)}
    for clip in (0, 1):
        codes, scale = ref.quantize_symmetric(rotated, 64, bool(clip))
        out[f"codes_clip{clip}"] = pack_nibbles(codes)
        out[f"scales_clip{clip}"] = scale.astype(np.float16).view(np.uint16)
    np.savez_compressed(os.path.join(HERE, "weights_w4a4.npz"), **out)

    # --- W4A4 activations (Mode.activations :206-211)
    rotated_x = ref.hadamard_256(x)
    codes, scale = ref.quantize_symmetric(rotated_x, 64, False)
    peak = np.abs(rotated_x.reshape(m, k // 64, 64)).max(axis=-1)
    kernel_scale = np.maximum(peak / np.float32(7.0), np.float32(2.0 ** -24)).astype(np.float16)
    same_rule = kernel_scale.view(np.uint16) == scale.astype(np.float16).view(np.uint16)
    mode = ref.Mode("w4a4-h256-g64-clip")
    np.savez_compressed(
        os.path.join(HERE, "activations_w4a4.npz"),
        x_f16=x16.view(np.uint16), outlier_channels=outliers, rotated_f32=rotated_x.astype(np.float32),
        codes=pack_nibbles(codes), scales=scale.astype(np.float16).view(np.uint16),
        scale_rules_agree=same_rule, dequantized_f32=mode.activations(x).astype(np.float32))

    # --- operator outputs (Model.block_linear :227-234)
    y_w4a16 = ref.Mode("w4a16-g64").activations(x) @ ref.Mode("w4a16-g64").prepare(w).T
    y_w4a4 = mode.activations(x) @ mode.prepare(w).T
    np.savez_compressed(os.path.join(HERE, "linear_outputs.npz"),
                        x_f16=x16.view(np.uint16), weights_f16=w16.view(np.uint16),
                        y_w4a16_g64=y_w4a16.astype(np.float32), y_w4a4_h256_g64_clip=y_w4a4.astype(np.float32))

    # --- the reference's in-source unit tests, as data
    involution_in = (np.arange(256, dtype=np.float32) * np.float32(0.01) - np.float32(1.0)).astype(np.float32)
    affine_in = (np.arange(64, dtype=np.float32) * np.float32(0.003) - np.float32(0.05)).astype(np.float32)
    symmetric_in = np.zeros(64, dtype=np.float32)
    symmetric_in[:3] = [-0.7, 0.7, 0.1]
    clip_in = ((np.arange(64) * 7) % 13).astype(np.float32) * np.float32(0.01)
    clip_in[5] = 2.0
    np.savez_compressed(
        os.path.join(HERE, "known_answers.npz"),
        involution_in=involution_in, involution_tolerance=np.float32(1e-5),       # int4_pack.cplus:856-870
        affine_in=affine_in, affine_slack=np.float32(1e-4),                       # :872-892
        symmetric_in=symmetric_in, symmetric_scale=np.float32(0.1),               # :894-908
        symmetric_scale_tolerance=np.float32(1e-4),
        symmetric_codes=np.array([9, 7, 1, 0], dtype=np.uint8),
        clip_in=clip_in,                                                          # :910-938
        half_exact=np.array([1.0, -2.5, 0.000061035156], dtype=np.float32),       # half.cplus:82-85
        half_inputs=np.array([0.000000059604645, 0.000000029802322, 65504.0], dtype=np.float32),
        half_bits=np.array([0x0001, 0x0000, 0x7BFF], dtype=np.uint16))            # :87-89
    agree = int(same_rule.sum())
    print(f"wrote golden vectors: n={n} k={k} m={m}; activation scale rules agree on "
          f"{agree}/{same_rule.size} groups")


if __name__ == "__main__":
    main()
