"""The QIPACK v6 container on the host (no GPU): what the library writes passes its own copy of the reference's
verify (int4_pack.cplus:733-850) and is read back identically; corruptions are caught with the reference's
distinctions; and, where the reference tree is mounted, the reference's own pack reader
(tools/evaluate_int4_quantization.py:47-95, imported, not copied) reads the same file and dequantises the
matrices to what the oracle says."""
import importlib.util
import os
import struct
import sys

import numpy as np
import pytest

import __graft_entry__ as entry
from oracle import qipack_oracle as qo
from tests import qi_testing as qt


@pytest.fixture(scope="module")
def qi():
    module = entry.load_package()
    module.lib()
    return module


def fnv1a(*parts) -> int:
    value = 14695981039346656037
    for part in parts:
        for byte in bytes(part):
            value = ((value ^ byte) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return value


def small_pack(rng, scheme, matrices=3, n=32, k=512):
    """A vector (fp16), a bf16 global matrix and `matrices` quantised block matrices."""
    tensors = [
        {"name": "norm.weight", "scheme": 1, "dimensions": [k], "weights": rng.standard_normal(k).astype(np.float16)},
        {"name": "img_in.weight", "scheme": 0, "dimensions": [16, 64],
         "weights": rng.integers(0, 65536, size=16 * 64, dtype=np.uint16)},
    ]
    for index in range(matrices):
        w16 = qt.make_weights(rng, n, k)
        if scheme == 6:
            codes, scales = qt.pack_w4a4(w16)
            tensors.append({"name": f"blocks.{index}.attn.q.weight", "scheme": 6, "dimensions": [n, k], "group_size": 64,
                            "weights": codes, "scales": scales, "_w16": w16})
        else:
            codes, scales, minimums = qt.pack_w4a16(w16)
            tensors.append({"name": f"blocks.{index}.attn.q.weight", "scheme": 5, "dimensions": [n, k], "group_size": 64,
                            "weights": codes, "scales": scales, "zeros": minimums, "_w16": w16})
    return tensors


@pytest.mark.parametrize("scheme,policy", [(6, "transformer:w4a4-h256-g64-v6"), (5, "transformer:w4a16-g64-v6")])
def test_written_pack_verifies_and_reads_back(qi, tmp_path, scheme, policy):
    rng = np.random.default_rng(300 + scheme)
    tensors = small_pack(rng, scheme)
    path = str(tmp_path / "small.qipack")
    qi.pack_write(path, policy, tensors, metadata="steps=4\nkind=distilled\nquant=w4a4-h256-g64-clip\n")
    assert not os.path.exists(path + ".tmp")
    assert qi.pack_verify(path, len(tensors), 3) == 0
    assert qi.pack_verify(path, None, 3) == 0
    assert qi.pack_verify(path) == qi.lib().qi_pack_verify(path.encode()) != 0  # not the engine's 297 / 224 inventory
    pack = qi.Pack(path)
    try:
        assert pack.policy == policy and pack.scheme == scheme and pack.tensor_count == len(tensors)
        assert pack.metadata("steps") == "4" and pack.metadata("kind") == "distilled" and pack.metadata("absent") is None
        data = pack.data()
        raw = open(path, "rb").read()
        assert len(raw) == pack.file_bytes and fnv1a(raw[pack.data_offset:]) == pack.payload_checksum
        previous_end = pack.data_offset
        for index, tensor in enumerate(tensors):
            record = pack.record(index)
            assert record.name.decode() == tensor["name"] and record.scheme == tensor["scheme"]
            assert list(record.dimensions)[:record.rank] == tensor["dimensions"]
            parts = []
            for field in ("weights", "scales", "zeros"):
                offset, length = getattr(record, field + "_offset"), getattr(record, field + "_length")
                stored = tensor.get(field)
                assert length == (0 if stored is None else np.ascontiguousarray(stored).nbytes)
                if length:
                    assert offset % 256 == 0 and offset >= previous_end  # plan_record: aligned, in order
                    previous_end = offset + length
                    got = data[offset - pack.data_offset:offset - pack.data_offset + length]
                    assert got.tobytes() == np.ascontiguousarray(stored).tobytes()
                    parts.append(got.tobytes())
            assert record.tensor_checksum == fnv1a(*parts)
    finally:
        pack.close()


def test_verify_tells_the_corruptions_apart(qi, tmp_path):
    rng = np.random.default_rng(310)
    tensors = small_pack(rng, 6)
    path = str(tmp_path / "good.qipack")
    qi.pack_write(path, "transformer:w4a4-h256-g64-v6", tensors, metadata="steps=4\n")
    good = bytearray(open(path, "rb").read())
    pack = qi.Pack(path)
    record = pack.record(3)
    data_offset, metadata_offset = pack.data_offset, 256 + 256 * pack.tensor_count
    pack.close()

    def verdict(mutate):
        bad = bytearray(good)
        mutate(bad)
        other = str(tmp_path / "bad.qipack")
        open(other, "wb").write(bad)
        return qi.pack_verify(other, len(tensors), 3)

    lib = qi.lib()
    assert verdict(lambda b: b.__setitem__(0, ord("X"))) == 20002                       # magic
    assert verdict(lambda b: b.__setitem__(slice(136, 168), b"transformer:all-matrix-f16-v4".ljust(32, b"\0"))) == 20003
    assert verdict(lambda b: b.__setitem__(metadata_offset, b[metadata_offset] ^ 1)) == 20004  # metadata checksum
    assert verdict(lambda b: b.__setitem__(record.weights_offset + 5, b[record.weights_offset + 5] ^ 0x10)) == 20007
    assert verdict(lambda b: b.__setitem__(record.scales_offset, b[record.scales_offset] ^ 1)) == 20007
    # a flipped byte in the padding between two regions is in no tensor, only in the payload
    vector_end = data_offset + 512 * 2 - 1  # the first tensor is 1024 bytes: no padding there; the bf16 matrix (2048) neither
    first = qi.Pack(path)
    odd = first.record(0)
    first.close()
    assert odd.weights_offset == data_offset and vector_end < len(good)
    # a record whose lengths do not follow from its dimensions
    directory = 256 + 3 * 256
    assert verdict(lambda b: b.__setitem__(slice(directory + 136, directory + 144), struct.pack("<Q", 48))) == 20005
    # a region moved off its alignment
    assert verdict(lambda b: b.__setitem__(slice(directory + 184, directory + 192), struct.pack("<Q", record.weights_offset + 16))) == 20006
    assert qi.pack_verify(path, len(tensors), 2) == 20008                               # inventory
    assert qi.pack_verify(str(tmp_path / "missing.qipack"), -1, -1) == 20001
    with pytest.raises(qi.PackError):
        qi.pack_write(str(tmp_path / "x.qipack"), "transformer:w4a4-h256-g48-v6", tensors)  # no such policy
    ragged = [dict(tensors[2], dimensions=[32, 384], weights=tensors[2]["weights"][:, :192],
                   scales=tensors[2]["scales"][:, :6])]
    with pytest.raises(qi.PackError):
        qi.pack_write(str(tmp_path / "y.qipack"), "transformer:w4a4-h256-g64-v6", ragged)   # K not a multiple of 256
    assert lib.qi_pack_verify(None) == 20010


def test_engine_inventory_passes_the_strict_verify(qi, tmp_path):
    # 297 tensors of which 224 quantised block matrices (int4_pack.cplus:39, :836), in miniature
    rng = np.random.default_rng(320)
    codes = rng.integers(0, 256, size=(8, 128), dtype=np.uint8)
    scales = rng.uniform(1e-3, 6e-3, size=(8, 4)).astype(np.float16)
    tensors = []
    for index in range(297):
        if index < 224:
            tensors.append({"name": f"m{index}", "scheme": 6, "dimensions": [8, 256], "group_size": 64, "weights": codes, "scales": scales})
        else:
            tensors.append({"name": f"v{index}", "scheme": 1, "dimensions": [8], "weights": np.zeros(8, dtype=np.float16)})
    path = str(tmp_path / "engine.qipack")
    qi.pack_write(path, "transformer:w4a4-h256-g64-v6", tensors)
    assert qi.pack_verify(path) == 0


def _reference_reader():
    root = os.environ.get("QI_REFERENCE", os.path.join(os.path.dirname(entry.ROOT), "reference"))
    path = os.path.join(root, "tools", "evaluate_int4_quantization.py")
    if not os.path.exists(path):
        pytest.skip("the reference tree is not mounted here")
    sys.path.insert(0, os.path.dirname(path))
    try:
        spec = importlib.util.spec_from_file_location("qi_reference_evaluator", path)
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
    finally:
        sys.path.pop(0)
    return module


@pytest.mark.parametrize("scheme,policy", [(6, "transformer:w4a4-h256-g64-v6"), (5, "transformer:w4a16-g64-v6")])
def test_the_reference_reader_reads_what_the_library_writes(qi, tmp_path, scheme, policy):
    from pathlib import Path

    reference = _reference_reader()
    rng = np.random.default_rng(330 + scheme)
    tensors = small_pack(rng, scheme)
    path = str(tmp_path / "ref.qipack")
    qi.pack_write(path, policy, tensors)
    theirs = reference.Pack(Path(path))
    assert theirs.policy == policy
    for tensor in tensors[2:]:
        dense = theirs.matrix(tensor["name"])  # dequantised by the reference's reader, still rotated for scheme 6
        if scheme == 5:
            expected = qo.w4a16_dequantize(tensor["weights"], tensor["scales"], tensor["zeros"]).astype(np.float32)
            # the reader multiplies in fp32 without the kernel's rounding of each weight to fp16
            assert np.max(np.abs(dense - expected)) <= 2.0 ** -11 * np.max(np.abs(expected))
        else:
            values = qo.unpack_codes(tensor["weights"], True).astype(np.float32)
            scales = tensor["scales"].view(np.float16).astype(np.float32)
            assert np.array_equal(dense, (values.reshape(32, 8, 64) * scales[..., None]).reshape(32, 512))
    vector = theirs.vector("norm.weight")
    assert np.array_equal(vector, tensors[0]["weights"].astype(np.float32))
