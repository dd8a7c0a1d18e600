"""Host-side binding of libqipack_b200.so (include/qipack_b200.h) for Python callers.

The product is the C-ABI shared library built from ``csrc/``; this module only loads it and
mirrors the reference's thin operator wrappers (qwen_image_cuda/src/cuda.cplus:128-130:
``w4a4_quantize_activations``, ``w4a4_gemm``, ``w4a16_gemm``, ``f32_to_f16``) and its
dispatcher ``linear`` (qwen_image_cuda/src/transformer.cplus:673-713) with the same argument
order and the same int status return (0 = success, 1 = cudaErrorInvalidValue).

Pointers may be given as integers or as anything with ``data_ptr()`` (torch tensors).
There is no CPU path: loading fails loudly when the library has not been built.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_HERE)
LIB_PATH = os.path.join(_HERE, "libqipack_b200.so")
SOURCES = ["qipack_b200.cu", "ptx.cuh", "quantize.cuh", "w4a16_gemm.cuh", "w4a16_gemv.cuh", "w4a16_gemv_stream.cuh", "w4a16_pair_gemm.cuh", "w4a4_gemm.cuh",
           "w4a4_wide_gemm.cuh", "w4a4_pair_gemm.cuh", "shard.cuh", "probe.cuh", "pack_file.cuh"]

DTYPE_F32 = 0
DTYPE_F16 = 1
SCHEME_W4A16 = 5
SCHEME_W4A4_H256 = 6
CUDA_ERROR_INVALID_VALUE = 1

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared"]


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile csrc/ for sm_100a into libqipack_b200.so next to this file (nvcc cross-compiles
    without a GPU)."""
    sources = [os.path.join(_HERE, "csrc", name) for name in SOURCES]
    sources = [s for s in sources if os.path.exists(s)] + [os.path.join(_ROOT, "include", "qipack_b200.h")]
    stale = force or not os.path.exists(LIB_PATH) or any(
        os.path.getmtime(s) > os.path.getmtime(LIB_PATH) for s in sources)
    if stale:
        nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
        command = [nvcc, *NVCC_FLAGS, "-o", LIB_PATH, os.path.join(_HERE, "csrc", "qipack_b200.cu")]
        if verbose:
            command.insert(1, "-Xptxas")
            command.insert(2, "-v")
        subprocess.run(command, check=True)
    return LIB_PATH


class qi_packed_linear(ctypes.Structure):
    _fields_ = [("scheme", ctypes.c_uint32), ("group_size", ctypes.c_uint32), ("n", ctypes.c_int),
                ("k", ctypes.c_int), ("weights", ctypes.c_void_p), ("scales", ctypes.c_void_p),
                ("zeros", ctypes.c_void_p), ("bias", ctypes.c_void_p), ("weights_wide", ctypes.c_void_p)]


class qi_gemv_item(ctypes.Structure):
    _fields_ = [("codes", ctypes.c_void_p), ("scales", ctypes.c_void_p), ("minimums", ctypes.c_void_p),
                ("bias", ctypes.c_void_p), ("y", ctypes.c_void_p)]


class qi_linear_work(ctypes.Structure):
    _fields_ = [("codes", ctypes.c_void_p), ("code_scales", ctypes.c_void_p), ("halves", ctypes.c_void_p),
                ("wide", ctypes.c_void_p)]


class qi_pack_header_info(ctypes.Structure):
    _fields_ = [("policy", ctypes.c_char * 33), ("scheme", ctypes.c_uint32), ("tensor_count", ctypes.c_uint32),
                ("data_offset", ctypes.c_uint64), ("file_bytes", ctypes.c_uint64), ("payload_checksum", ctypes.c_uint64)]


class qi_pack_record_info(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char * 129), ("scheme", ctypes.c_uint32), ("rank", ctypes.c_uint32),
                ("dimensions", ctypes.c_uint64 * 4), ("group_size", ctypes.c_uint32),
                ("weights_offset", ctypes.c_uint64), ("weights_length", ctypes.c_uint64),
                ("scales_offset", ctypes.c_uint64), ("scales_length", ctypes.c_uint64),
                ("zeros_offset", ctypes.c_uint64), ("zeros_length", ctypes.c_uint64), ("tensor_checksum", ctypes.c_uint64)]


class qi_pack_tensor(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("scheme", ctypes.c_uint32), ("rank", ctypes.c_uint32),
                ("dimensions", ctypes.c_uint64 * 4), ("group_size", ctypes.c_uint32),
                ("weights", ctypes.c_void_p), ("weights_length", ctypes.c_uint64),
                ("scales", ctypes.c_void_p), ("scales_length", ctypes.c_uint64),
                ("zeros", ctypes.c_void_p), ("zeros_length", ctypes.c_uint64)]


_P, _I, _LL, _ULL = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_ulonglong

# name -> argument types; every entry point of include/qipack_b200.h
SIGNATURES = {
    "qi_w4a4_quantize_activations": [_P, _P, _P, _I, _I],
    "qi_w4a4_gemm": [_P, _P, _P, _P, _P, _I, _I, _I],
    "qi_w4a16_gemm": [_P, _P, _P, _P, _P, _I, _I, _I],
    "qi_f32_to_f16": [_P, _P, _ULL],
    "qi_f32_to_f16_ex": [_P, _P, _ULL, _P],
    "qi_w4a4_quantize_activations_ex": [_P, _I, _P, _P, _I, _I, _P],
    "qi_w4a4_gemm_ex": [_P, _P, _P, _P, _P, _P, _I, _LL, _I, _I, _I, _P],
    "qi_w4a16_gemv_grouped_ex": [_P, ctypes.POINTER(qi_gemv_item), _I, _I, _LL, _I, _I, _I, _P],
    "qi_w4a4_gemm_path_ex": [_P, _P, _P, _P, _P, _P, _I, _LL, _I, _I, _I, _I, _P],
    "qi_w4a4_scratch_trim": [],
    "qi_w4a4_gemm_noalloc_ex": [_P, _P, _P, _P, _P, _P, _I, _LL, _I, _I, _I, _P],
    "qi_w4a16_gemm_ex": [_P, _P, _P, _P, _P, _P, _I, _LL, _I, _I, _I, _P],
    "qi_w4a16_gemv_ex": [_P, _P, _P, _P, _P, _P, _I, _LL, _I, _I, _I, _P],
    "qi_w4a16_dequantize_ex": [_P, _P, _P, _P, _I, _I, _P],
    "qi_w4a4_group_dots_ex": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _P],
    "qi_w4a4_widen_codes_ex": [_P, _P, _LL, _I, _P],
    "qi_w4a4_quantize_activations_wide_ex": [_P, _I, _P, _P, _P, _I, _I, _P],
    "qi_w4a4_gemm_wide_ex": [_P, _P, _P, _P, _P, _P, _I, _LL, _I, _I, _I, _P],
    "qi_w4a4_swiglu_quantize_ex": [_P, _P, _P, _P, _P, _I, _I, _P],
    "qi_w4a4_gelu_quantize_ex": [_P, _P, _P, _P, _I, _I, _P],
    "qi_w4a4_group_dots_wide_ex": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _P],
    "qi_linear": [ctypes.POINTER(qi_packed_linear), ctypes.POINTER(qi_linear_work), _P, _I, _P, _I, _LL, _I, _I, _P],
    "qi_shard_plan": [_I, _I, _I, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)],
    "qi_shard_plan_inputs": [_I, _I, _I, _I, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)],
    "qi_shard_linear_inputs": [_P, ctypes.POINTER(qi_packed_linear), ctypes.POINTER(qi_linear_work), _P, _I, _P, _I, _I, _P],
    "qi_shard_unique_id": [_P],
    "qi_shard_create": [ctypes.POINTER(ctypes.c_void_p), _I, _I, _P],
    "qi_shard_destroy": [_P],
    "qi_shard_rank": [_P, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)],
    "qi_shard_all_gather": [_P, _P, _P, _I, _I, _I, _P],
    "qi_shard_all_reduce_f32": [_P, _P, ctypes.c_ulonglong, _P],
    "qi_shard_reduce_scatter_f32": [_P, _P, _P, ctypes.c_ulonglong, _P],
    "qi_shard_barrier": [_P, _P],
    "qi_shard_put_slice": [_P, ctypes.POINTER(ctypes.c_void_p), _I, _I, _LL, _I, _I, _I, _P],
    "qi_shard_peer_export": [_P, _P, ctypes.POINTER(ctypes.c_size_t)],
    "qi_shard_peer_open": [_P, ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p)],
    "qi_shard_peer_close": [_P, ctypes.c_size_t],
    "qi_w4a4_gemm_wide_scatter_ex": [_P, _P, _P, _P, _P, ctypes.POINTER(ctypes.c_void_p), _I, _I, _I, _LL, _I, _I, _I,
                                     _I, _P],
    "qi_shard_linear": [_P, ctypes.POINTER(qi_packed_linear), ctypes.POINTER(qi_linear_work), _P, _I, _P, _P, _I, _I,
                        _I, _P],
    "qi_pack_open": [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)],
    "qi_pack_close": [_P],
    "qi_pack_info": [_P, ctypes.POINTER(qi_pack_header_info)],
    "qi_pack_record": [_P, _I, ctypes.POINTER(qi_pack_record_info)],
    "qi_pack_metadata": [_P, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_size_t],
    "qi_pack_read": [_P, ctypes.c_uint64, ctypes.c_uint64, _P],
    "qi_pack_linear": [_P, _I, _P, ctypes.POINTER(qi_packed_linear)],
    "qi_pack_verify": [ctypes.c_char_p],
    "qi_pack_verify_ex": [ctypes.c_char_p, _I, _I],
    "qi_pack_write": [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_char_p, ctypes.POINTER(qi_pack_tensor), _I],
    "qi_kernel_status": [ctypes.POINTER(ctypes.c_uint)],
    "qi_probe_tensor_rate": [_I, ctypes.c_double, ctypes.POINTER(ctypes.c_double)],
    "qi_probe_wait_timeout": [_ULL, _P],
    "qi_w4a16_gemm_tile_ex": [_P, _P, _P, _P, _P, _P, _I, _LL, _I, _I, _I, _I, _P],
    "qi_w4a4_gemm_wide_single_ex": [_P, _P, _P, _P, _P, _P, _I, _LL, _P, _I, _I, _I, _P],
}

_lib = None


def lib() -> ctypes.CDLL:
    """The loaded library. Raises if it was never built: there is no fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
                               "(the packed-linear operators exist only as CUDA kernels)")
        loaded = ctypes.CDLL(LIB_PATH)
        for name, argtypes in SIGNATURES.items():
            function = getattr(loaded, name)
            function.argtypes = argtypes
            function.restype = ctypes.c_int
        loaded.qi_b200_version.restype = ctypes.c_char_p
        loaded.qi_b200_version.argtypes = []
        _lib = loaded
    return _lib


def _p(pointer) -> ctypes.c_void_p:
    if pointer is None:
        return ctypes.c_void_p(0)
    if hasattr(pointer, "data_ptr"):
        return ctypes.c_void_p(pointer.data_ptr())
    return ctypes.c_void_p(int(pointer))


def version() -> str:
    return lib().qi_b200_version().decode()


# ---- the reference's operator wrappers (cuda.cplus:128-130), same argument order -------------

def w4a4_quantize_activations(x, codes, scales, m: int, k: int) -> int:
    return lib().qi_w4a4_quantize_activations(_p(x), _p(codes), _p(scales), m, k)


def w4a4_gemm(a_codes, a_scales, w_codes, w_scales, y, m: int, n: int, k: int) -> int:
    return lib().qi_w4a4_gemm(_p(a_codes), _p(a_scales), _p(w_codes), _p(w_scales), _p(y), m, n, k)


def w4a16_gemm(x_half, codes, scales, minimums, y, m: int, n: int, k: int) -> int:
    return lib().qi_w4a16_gemm(_p(x_half), _p(codes), _p(scales), _p(minimums), _p(y), m, n, k)


def f32_to_f16(source, out, count: int) -> int:
    return lib().qi_f32_to_f16(_p(source), _p(out), count)


def f32_to_f16_ex(source, out, count: int, stream=None) -> int:
    return lib().qi_f32_to_f16_ex(_p(source), _p(out), count, _p(stream))


# ---- extended forms ------------------------------------------------------------------------------

def w4a4_quantize_activations_ex(x, x_dtype: int, codes, scales, m: int, k: int, stream=None) -> int:
    return lib().qi_w4a4_quantize_activations_ex(_p(x), x_dtype, _p(codes), _p(scales), m, k, _p(stream))


def w4a4_gemm_ex(a_codes, a_scales, w_codes, w_scales, bias, y, y_dtype: int, ldy: int, m: int, n: int, k: int,
                 stream=None) -> int:
    return lib().qi_w4a4_gemm_ex(_p(a_codes), _p(a_scales), _p(w_codes), _p(w_scales), _p(bias), _p(y), y_dtype,
                                 ldy, m, n, k, _p(stream))


def gemv_items(entries):
    """A host table for w4a16_gemv_grouped_ex from (codes, scales, minimums, bias or None, y) tuples of device tensors.
    Returns (table, keep): `keep` holds the tensors so that they outlive the table."""
    table = (qi_gemv_item * len(entries))()
    for slot, (codes, scales, minimums, bias, y) in zip(table, entries):
        slot.codes, slot.scales, slot.minimums = _p(codes), _p(scales), _p(minimums)
        slot.bias, slot.y = (_p(bias) if bias is not None else None), _p(y)
    return table, list(entries)


def w4a16_gemv_grouped_ex(x_half, table, y_dtype: int, ldy: int, m: int, n: int, k: int, stream=None) -> int:
    """len(table) matrices [n, k] against the same x [m, k] in one launch per 64 (table from gemv_items)."""
    return lib().qi_w4a16_gemv_grouped_ex(_p(x_half), table, len(table), y_dtype, ldy, m, n, k, _p(stream))


W4A4_PATH_BY_SHAPE, W4A4_PATH_INT8, W4A4_PATH_WIDENED = 0, 1, 2
NOALLOC_SCRATCH_BYTES, NOALLOC_TOO_LARGE = 64 << 20, 30001


def w4a4_scratch_trim() -> int:
    """Returns the unused memory of the current device's scratch pool of the packed W4A4 entry points to the system."""
    return lib().qi_w4a4_scratch_trim()


def w4a4_gemm_noalloc_ex(a_codes, a_scales, w_codes, w_scales, bias, y, y_dtype: int, ldy: int, m: int, n: int, k: int,
                         stream=None) -> int:
    """qi_w4a4_gemm_ex on its widened path with the scratch in a fixed device array (no allocation of any kind)."""
    return lib().qi_w4a4_gemm_noalloc_ex(_p(a_codes), _p(a_scales), _p(w_codes), _p(w_scales), _p(bias), _p(y), y_dtype,
                                         ldy, m, n, k, _p(stream))


def w4a4_gemm_path_ex(a_codes, a_scales, w_codes, w_scales, bias, y, y_dtype: int, ldy: int, m: int, n: int, k: int,
                      path: int, stream=None) -> int:
    return lib().qi_w4a4_gemm_path_ex(_p(a_codes), _p(a_scales), _p(w_codes), _p(w_scales), _p(bias), _p(y), y_dtype,
                                      ldy, m, n, k, path, _p(stream))


def w4a16_gemm_ex(x_half, codes, scales, minimums, bias, y, y_dtype: int, ldy: int, m: int, n: int, k: int,
                  stream=None) -> int:
    return lib().qi_w4a16_gemm_ex(_p(x_half), _p(codes), _p(scales), _p(minimums), _p(bias), _p(y), y_dtype, ldy,
                                  m, n, k, _p(stream))


def w4a16_gemv_ex(x_half, codes, scales, minimums, bias, y, y_dtype: int, ldy: int, m: int, n: int, k: int,
                  stream=None) -> int:
    return lib().qi_w4a16_gemv_ex(_p(x_half), _p(codes), _p(scales), _p(minimums), _p(bias), _p(y), y_dtype, ldy,
                                  m, n, k, _p(stream))


def w4a16_dequantize_ex(codes, scales, minimums, w_half, n: int, k: int, stream=None) -> int:
    return lib().qi_w4a16_dequantize_ex(_p(codes), _p(scales), _p(minimums), _p(w_half), n, k, _p(stream))


def w4a4_group_dots_ex(a_codes, a_scales, w_codes, w_scales, y, dots, m: int, n: int, k: int, stream=None) -> int:
    return lib().qi_w4a4_group_dots_ex(_p(a_codes), _p(a_scales), _p(w_codes), _p(w_scales), _p(y), _p(dots), m, n,
                                       k, _p(stream))


def w4a4_widen_codes_ex(codes, out_bytes, rows: int, k: int, stream=None) -> int:
    return lib().qi_w4a4_widen_codes_ex(_p(codes), _p(out_bytes), rows, k, _p(stream))


def w4a4_quantize_activations_wide_ex(x, x_dtype: int, codes, scales, out_bytes, m: int, k: int, stream=None) -> int:
    return lib().qi_w4a4_quantize_activations_wide_ex(_p(x), x_dtype, _p(codes), _p(scales), _p(out_bytes), m, k,
                                                      _p(stream))


def w4a4_swiglu_quantize_ex(gate, up, codes, scales, out_bytes, m: int, k: int, stream=None) -> int:
    return lib().qi_w4a4_swiglu_quantize_ex(_p(gate), _p(up), _p(codes), _p(scales), _p(out_bytes), m, k, _p(stream))


def w4a4_gelu_quantize_ex(x, codes, scales, out_bytes, m: int, k: int, stream=None) -> int:
    return lib().qi_w4a4_gelu_quantize_ex(_p(x), _p(codes), _p(scales), _p(out_bytes), m, k, _p(stream))


def w4a4_gemm_wide_ex(a_bytes, a_scales, w_bytes, w_scales, bias, y, y_dtype: int, ldy: int, m: int, n: int, k: int,
                      stream=None) -> int:
    return lib().qi_w4a4_gemm_wide_ex(_p(a_bytes), _p(a_scales), _p(w_bytes), _p(w_scales), _p(bias), _p(y), y_dtype,
                                      ldy, m, n, k, _p(stream))


def w4a4_group_dots_wide_ex(a_bytes, a_scales, w_bytes, w_scales, y, dots, m: int, n: int, k: int, stream=None) -> int:
    return lib().qi_w4a4_group_dots_wide_ex(_p(a_bytes), _p(a_scales), _p(w_bytes), _p(w_scales), _p(y), _p(dots), m,
                                            n, k, _p(stream))


def kernel_status() -> int:
    """Code of the first wait that gave up on the current device since the last call (0 = none)."""
    value = ctypes.c_uint(0)
    error = lib().qi_kernel_status(ctypes.byref(value))
    if error != 0:
        raise RuntimeError(f"qi_kernel_status: cuda status {error}")
    return int(value.value)


def probe_tensor_rate(kind: int, seconds: float = 0.05) -> float:
    """Dense tcgen05.mma rate of the current device in TOP/s; kind 0 fp16, 1 FP8 E4M3, 2 int8."""
    value = ctypes.c_double(0.0)
    status = lib().qi_probe_tensor_rate(kind, seconds, ctypes.byref(value))
    if status != 0:
        raise RuntimeError(f"qi_probe_tensor_rate: cuda status {status}")
    return float(value.value)


def probe_wait_timeout(limit_ns: int, stream=None) -> int:
    """Launches a wait that runs out after `limit_ns`; kernel_status() then reports 0x0001A000."""
    return lib().qi_probe_wait_timeout(limit_ns, _p(stream))


def w4a16_gemm_tile_ex(x_half, codes, scales, minimums, bias, y, y_dtype: int, ldy: int, m: int, n: int, k: int,
                       tile: int, stream=None) -> int:
    """qi_w4a16_gemm_ex with the tile forced (1..5; 0 = by shape)."""
    return lib().qi_w4a16_gemm_tile_ex(_p(x_half), _p(codes), _p(scales), _p(minimums), _p(bias), _p(y), y_dtype,
                                       ldy, m, n, k, tile, _p(stream))


def w4a4_gemm_wide_single_ex(a_bytes, a_scales, w_bytes, w_scales, bias, y, y_dtype: int, ldy: int, dots, m: int,
                             n: int, k: int, stream=None) -> int:
    """The byte-operand W4A4 GEMM on single CTAs; `dots` [m, n, k/64] int32 or None."""
    return lib().qi_w4a4_gemm_wide_single_ex(_p(a_bytes), _p(a_scales), _p(w_bytes), _p(w_scales), _p(bias), _p(y),
                                             y_dtype, ldy, _p(dots), m, n, k, _p(stream))


# ---- transformer::linear (transformer.cplus:673-713) ------------------------------------------

class PackedLinear:
    """One packed record resident on the device: scheme, n, k and the three regions."""

    def __init__(self, scheme: int, n: int, k: int, weights, scales, zeros=None, bias=None, group_size: int = 64,
                 weights_wide=None):
        self.scheme, self.n, self.k, self.group_size = scheme, n, k, group_size
        self.weights, self.scales, self.zeros, self.bias = weights, scales, zeros, bias  # keep tensors alive
        self.weights_wide = weights_wide
        self.record = qi_packed_linear(scheme, group_size, n, k, _p(weights), _p(scales), _p(zeros), _p(bias),
                                       _p(weights_wide))


class LinearWork:
    """The activation arena of transformer.cplus:649-651 (codes, code_scales, halves)."""

    def __init__(self, codes, code_scales, halves, wide=None):
        self.codes, self.code_scales, self.halves, self.wide = codes, code_scales, halves, wide
        self.work = qi_linear_work(_p(codes), _p(code_scales), _p(halves), _p(wide))


def linear(model: PackedLinear, work: LinearWork, input, output, rows: int, reuse_input: bool = False, *,
           input_dtype: int = DTYPE_F32, output_dtype: int = DTYPE_F32, ld_output: int | None = None,
           stream=None) -> int:
    """output[rows, n] = input[rows, k] . W^T for one packed record; 0 on success."""
    return lib().qi_linear(ctypes.byref(model.record), ctypes.byref(work.work), _p(input), input_dtype, _p(output),
                           output_dtype, model.n if ld_output is None else ld_output, rows, int(reuse_input),
                           _p(stream))


# ---- the QIPACK v6 container (host side; int4_pack.cplus:36-95, 476-518, 733-850) ------------------------

class PackError(RuntimeError):
    def __init__(self, what: str, code: int):
        super().__init__(f"{what}: pack status {code}")
        self.code = code


def pack_write(path: str, policy: str, tensors, metadata: str = "") -> None:
    """Writes a pack. `tensors`: dicts with name, scheme, dimensions and the stored bytes as NumPy arrays:
    weights, and for a quantised matrix scales (and zeros for scheme 5) plus group_size."""
    import numpy as np

    keep, items = [], (qi_pack_tensor * len(tensors))()
    for item, tensor in zip(items, tensors):
        item.name = tensor["name"].encode()
        item.scheme, item.rank = tensor["scheme"], len(tensor["dimensions"])
        for index, size in enumerate(tensor["dimensions"]):
            item.dimensions[index] = size
        item.group_size = tensor.get("group_size", 0)
        for field in ("weights", "scales", "zeros"):
            array = tensor.get(field)
            if array is not None:
                array = np.ascontiguousarray(array)
                keep.append(array)
                setattr(item, field, array.ctypes.data)
                setattr(item, field + "_length", array.nbytes)
    status = lib().qi_pack_write(path.encode(), policy.encode(), metadata.encode(), items, len(tensors))
    if status != 0:
        raise PackError(f"qi_pack_write({path})", status)


def pack_verify(path: str, expected_tensors: int | None = None, expected_matrices: int | None = None) -> int:
    """0 when the pack passes every check of the reference's verify; with no counts given, the engine's own
    inventory (297 tensors, 224 quantised matrices) is expected."""
    if expected_tensors is None and expected_matrices is None:
        return lib().qi_pack_verify(path.encode())
    return lib().qi_pack_verify_ex(path.encode(), -1 if expected_tensors is None else expected_tensors,
                                   -1 if expected_matrices is None else expected_matrices)


class Pack:
    """An open pack: header, records, metadata; `linear(index, device_data)` gives the kernels' view of a record."""

    def __init__(self, path: str):
        self.handle = ctypes.c_void_p(0)
        status = lib().qi_pack_open(path.encode(), ctypes.byref(self.handle))
        if status != 0:
            raise PackError(f"qi_pack_open({path})", status)
        info = qi_pack_header_info()
        lib().qi_pack_info(self.handle, ctypes.byref(info))
        self.policy, self.scheme, self.tensor_count = info.policy.decode(), info.scheme, info.tensor_count
        self.data_offset, self.file_bytes, self.payload_checksum = info.data_offset, info.file_bytes, info.payload_checksum

    def record(self, index: int) -> qi_pack_record_info:
        info = qi_pack_record_info()
        status = lib().qi_pack_record(self.handle, index, ctypes.byref(info))
        if status != 0:
            raise PackError(f"qi_pack_record({index})", status)
        return info

    def metadata(self, key: str):
        value = ctypes.create_string_buffer(256)
        status = lib().qi_pack_metadata(self.handle, key.encode(), value, 256)
        return value.value.decode() if status == 0 else None

    def read(self, offset: int, count: int):
        import numpy as np

        out = np.empty(count, dtype=np.uint8)
        status = lib().qi_pack_read(self.handle, offset, count, out.ctypes.data)
        if status != 0:
            raise PackError(f"qi_pack_read({offset}, {count})", status)
        return out

    def data(self):
        """The whole data section, as the engine uploads it (transformer.cplus:120-123)."""
        return self.read(self.data_offset, self.file_bytes - self.data_offset)

    def linear(self, index: int, device_data) -> "PackedLinear":
        record = qi_packed_linear()
        status = lib().qi_pack_linear(self.handle, index, _p(device_data), ctypes.byref(record))
        if status != 0:
            raise PackError(f"qi_pack_linear({index})", status)
        view = PackedLinear.__new__(PackedLinear)
        view.scheme, view.n, view.k, view.group_size = record.scheme, record.n, record.k, record.group_size
        view.weights = view.scales = view.zeros = view.bias = view.weights_wide = device_data  # keeps the upload alive
        view.record = record
        return view

    def close(self) -> None:
        if self.handle:
            lib().qi_pack_close(self.handle)
            self.handle = ctypes.c_void_p(0)


# ---- column sharding over the GPUs of one box ------------------------------------------------------

SHARD_ID_BYTES = 128


def shard_plan(n: int, ranks: int, rank: int):
    """(first_row, row_count) of the weight rows `rank` owns; raises where no legal split exists."""
    first, count = ctypes.c_int(0), ctypes.c_int(0)
    status = lib().qi_shard_plan(n, ranks, rank, ctypes.byref(first), ctypes.byref(count))
    if status != 0:
        raise ValueError(f"n={n} cannot be split over {ranks} ranks in multiples of 128 rows (status {status})")
    return first.value, count.value


def shard_plan_inputs(k: int, scheme: int, ranks: int, rank: int):
    """(first_input, input_count) of the input columns `rank` owns in a row-parallel (K-sharded) linear."""
    first, count = ctypes.c_int(0), ctypes.c_int(0)
    status = lib().qi_shard_plan_inputs(k, scheme, ranks, rank, ctypes.byref(first), ctypes.byref(count))
    if status != 0:
        raise ValueError(f"k={k} cannot be split over {ranks} ranks in whole blocks of scheme {scheme} (status {status})")
    return first.value, count.value


def shard_unique_id() -> bytes:
    buffer = ctypes.create_string_buffer(SHARD_ID_BYTES)
    status = lib().qi_shard_unique_id(buffer)
    if status != 0:
        raise RuntimeError(f"qi_shard_unique_id: status {status}")
    return buffer.raw


class ShardContext:
    """One rank's handle on the NCCL communicator of a sharded linear stack."""

    def __init__(self, rank: int, ranks: int, unique_id: bytes):
        self.handle = ctypes.c_void_p(0)
        buffer = ctypes.create_string_buffer(unique_id, SHARD_ID_BYTES)
        status = lib().qi_shard_create(ctypes.byref(self.handle), rank, ranks, buffer)
        if status != 0:
            raise RuntimeError(f"qi_shard_create: status {status}")
        self.rank, self.ranks = rank, ranks

    def all_gather(self, y_local, y_slabs, output_dtype: int, rows: int, n_local: int, stream=None) -> int:
        return lib().qi_shard_all_gather(self.handle, _p(y_local), _p(y_slabs), output_dtype, rows, n_local, _p(stream))

    def all_reduce(self, y, count: int, stream=None) -> int:
        """y [count] float32 <- the sum over the ranks, in place."""
        return lib().qi_shard_all_reduce_f32(self.handle, _p(y), count, _p(stream))

    def reduce_scatter(self, y, y_share, count_per_rank: int, stream=None) -> int:
        """y_share [count_per_rank] float32 <- this rank's part of the sum over the ranks of y [ranks * count_per_rank]."""
        return lib().qi_shard_reduce_scatter_f32(self.handle, _p(y), _p(y_share), count_per_rank, _p(stream))

    def put_slice(self, copies, output_dtype: int, ldy: int, column: int, rows: int, n_local: int, stream=None) -> int:
        return lib().qi_shard_put_slice(self.handle, copies, len(copies), output_dtype, ldy, column, rows, n_local,
                                        _p(stream))

    def barrier(self, stream=None) -> int:
        return lib().qi_shard_barrier(self.handle, _p(stream))

    def linear(self, model: PackedLinear, work: LinearWork, input, y_local, y_slabs, rows: int,
               reuse_input: bool = False, *, input_dtype: int = DTYPE_F32, output_dtype: int = DTYPE_F32,
               stream=None) -> int:
        return lib().qi_shard_linear(self.handle, ctypes.byref(model.record), ctypes.byref(work.work), _p(input),
                                     input_dtype, _p(y_local), _p(y_slabs), output_dtype, rows, int(reuse_input),
                                     _p(stream))

    def linear_inputs(self, model: PackedLinear, work: LinearWork, input_local, y, rows: int, reuse_input: bool = False, *,
                      input_dtype: int = DTYPE_F32, stream=None) -> int:
        """Row-parallel linear: partial product over this rank's inputs, summed over the ranks into float32 y [rows, n]."""
        return lib().qi_shard_linear_inputs(self.handle, ctypes.byref(model.record), ctypes.byref(work.work), _p(input_local),
                                            input_dtype, _p(y), rows, int(reuse_input), _p(stream))

    def destroy(self) -> int:
        if self.handle:
            status = lib().qi_shard_destroy(self.handle)
            self.handle = ctypes.c_void_p(0)
            return status
        return 0


SHARD_PEER_HANDLE_BYTES = 64


class PeerMappingError(RuntimeError):
    """The ranks cannot map each other's device memory (qi_shard_peer_export / qi_shard_peer_open refused)."""


class PeerOutput:
    """The same device buffer on every rank of the box, each rank holding addresses of all copies.

    `local` is this rank's buffer (anything with data_ptr(), carved out of ONE cudaMalloc allocation
    that is exported once); `exchange(item) -> list` carries a picklable item to every rank and returns
    all ranks' items in rank order (torch.distributed.all_gather_object, for instance). Collective."""

    def __init__(self, context: ShardContext, local, exchange):
        """Raises PeerMappingError on EVERY rank when any rank could not export or map a buffer (a box whose
        processes may not share device memory): a rank never leaves the others waiting in `exchange`."""
        handle = ctypes.create_string_buffer(SHARD_PEER_HANDLE_BYTES)
        offset = ctypes.c_size_t(0)
        exported = lib().qi_shard_peer_export(_p(local), handle, ctypes.byref(offset))
        everyone = exchange((exported, handle.raw, offset.value))
        if len(everyone) != context.ranks:
            raise RuntimeError("exchange() must return one item per rank")
        self.rank, self.ranks = context.rank, context.ranks
        self.addresses, self._opened = [], []
        opened = 0
        if all(status == 0 for status, _, _ in everyone):
            for rank, (_, raw, peer_offset) in enumerate(everyone):
                if rank == context.rank:
                    self.addresses.append(_p(local).value)
                    continue
                pointer = ctypes.c_void_p(0)
                opened = lib().qi_shard_peer_open(ctypes.create_string_buffer(raw, SHARD_PEER_HANDLE_BYTES), peer_offset,
                                                  ctypes.byref(pointer))
                if opened != 0:
                    break
                self.addresses.append(pointer.value)
                self._opened.append((pointer.value, peer_offset))
        outcomes = exchange(opened)  # every rank learns whether every rank has every mapping
        failed = [status for status, _, _ in everyone if status != 0] + [status for status in outcomes if status != 0]
        if failed:
            self.close()
            raise PeerMappingError(f"a buffer could not be shared between the ranks (first status {failed[0]})")

    def copies(self, byte_offset: int = 0):
        """A C array of every rank's address of the byte `byte_offset` of the buffer."""
        return (ctypes.c_void_p * self.ranks)(*[address + byte_offset for address in self.addresses])

    def close(self) -> None:
        for address, offset in self._opened:
            lib().qi_shard_peer_close(ctypes.c_void_p(address), offset)
        self._opened = []


def w4a4_gemm_wide_scatter_ex(a_bytes, a_scales, w_bytes, w_scales, bias, copies, first_copy: int, y_dtype: int,
                              ldy: int, column: int, m: int, n: int, k: int, stream=None) -> int:
    """`copies`: what PeerOutput.copies() returns (keep it alive until the call returns)."""
    return lib().qi_w4a4_gemm_wide_scatter_ex(_p(a_bytes), _p(a_scales), _p(w_bytes), _p(w_scales), _p(bias), copies,
                                              len(copies), first_copy, y_dtype, ldy, column, m, n, k, _p(stream))
