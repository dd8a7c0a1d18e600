"""ctypes binding of the CPU oracle (oracle/qipack_oracle.c) over NumPy arrays.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the bench's
CPU-baseline legs. The shipped library never loads it.

Every wrapper takes and returns plain NumPy arrays in the reference's layouts:
codes ``[rows, k/2]`` uint8 (even column in the low nibble), scales and minimums
``[rows, k/64]`` as raw fp16 bits (uint16), y ``[m, n]`` float32.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libqipack_oracle.so")

SCHEME_W4A16 = 5
SCHEME_W4A4_H256 = 6
GROUP = 64


def build(force: bool = False) -> str:
    """Compile the C oracle (and, if the reference tree is mounted, its kernels)."""
    sources = [os.path.join(_HERE, "qipack_oracle.c"), os.path.join(_HERE, "qipack_oracle.h")]
    stale = force or not os.path.exists(_LIB_PATH) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in sources
    )
    if stale:
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s", "libqipack_oracle.so"], check=True)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.qio_half_to_f32.restype = ctypes.c_float
        _lib.qio_half_to_f32.argtypes = [ctypes.c_uint16]
        _lib.qio_half_from_f32.restype = ctypes.c_uint16
        _lib.qio_half_from_f32.argtypes = [ctypes.c_float]
        _lib.qio_half_round_f32.restype = ctypes.c_float
        _lib.qio_half_round_f32.argtypes = [ctypes.c_float]
        _lib.qio_pack_matrix.restype = ctypes.c_int
        _lib.qio_max_threads.restype = ctypes.c_int
    return _lib


def _ptr(array: np.ndarray | None):
    if array is None:
        return ctypes.c_void_p(0)
    assert array.flags["C_CONTIGUOUS"]
    return ctypes.c_void_p(array.ctypes.data)


def _c(array, dtype) -> np.ndarray:
    return np.ascontiguousarray(array, dtype=dtype)


def max_threads() -> int:
    """OpenMP's default team size (obeys OMP_NUM_THREADS)."""
    return int(lib().qio_max_threads())


def available_cores() -> int:
    """Host cores this process may run on, whatever OMP_NUM_THREADS says; pass it as `threads=`."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def half_from_f32(value: float) -> int:
    return int(lib().qio_half_from_f32(ctypes.c_float(value)))


def half_to_f32(bits: int) -> float:
    return float(lib().qio_half_to_f32(ctypes.c_uint16(bits)))


def f32_to_f16(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().qio_f32_to_f16(_ptr(x), _ptr(out), ctypes.c_size_t(x.size))
    return out


def hadamard_256(values: np.ndarray) -> np.ndarray:
    out = _c(values, np.float32).copy()
    assert out.size % 256 == 0
    flat = out.reshape(-1, 256)
    for row in flat:
        lib().qio_hadamard_256(_ptr(row))
    return out


def quantize_symmetric_group(values: np.ndarray, clip: bool):
    values = _c(values, np.float32)
    codes = np.zeros(values.size, dtype=np.uint8)
    scale = ctypes.c_uint16(0)
    lib().qio_quantize_symmetric_group(_ptr(values), ctypes.c_int(values.size), ctypes.c_int(int(clip)),
                                       _ptr(codes), ctypes.byref(scale))
    return codes, int(scale.value)


def quantize_affine_group(values: np.ndarray, clip: bool):
    values = _c(values, np.float32)
    codes = np.zeros(values.size, dtype=np.uint8)
    scale, minimum = ctypes.c_uint16(0), ctypes.c_uint16(0)
    lib().qio_quantize_affine_group(_ptr(values), ctypes.c_int(values.size), ctypes.c_int(int(clip)),
                                    _ptr(codes), ctypes.byref(scale), ctypes.byref(minimum))
    return codes, int(scale.value), int(minimum.value)


def pack_matrix(weights_f16: np.ndarray, scheme: int, clip: bool, group: int = GROUP, threads: int = 0):
    """fp16 weights [n,k] -> (codes [n,k/2] u8, scales [n,k/g] u16, minimums [n,k/g] u16 | None)."""
    w = _c(weights_f16.view(np.uint16) if weights_f16.dtype == np.float16 else weights_f16, np.uint16)
    n, k = w.shape
    codes = np.zeros((n, k // 2), dtype=np.uint8)
    scales = np.zeros((n, k // group), dtype=np.uint16)
    minimums = np.zeros((n, k // group), dtype=np.uint16) if scheme == SCHEME_W4A16 else None
    status = lib().qio_pack_matrix(_ptr(w), n, k, group, scheme, int(clip), _ptr(codes), _ptr(scales),
                                   _ptr(minimums), threads)
    if status != 0:
        raise ValueError(f"the packer rejects n={n} k={k} group={group} scheme={scheme}")
    return codes, scales, minimums


def quantize_activations(x: np.ndarray, threads: int = 0):
    """x [m,k] float32 or float16 -> (codes [m,k/2] u8, scales [m,k/64] u16)."""
    m, k = x.shape
    assert k % 256 == 0
    codes = np.zeros((m, k // 2), dtype=np.uint8)
    scales = np.zeros((m, k // GROUP), dtype=np.uint16)
    if x.dtype == np.float16:
        xx = _c(x.view(np.uint16), np.uint16)
        lib().qio_quantize_activations_f16(_ptr(xx), m, k, _ptr(codes), _ptr(scales), threads)
    else:
        xx = _c(x, np.float32)
        lib().qio_quantize_activations_f32(_ptr(xx), m, k, _ptr(codes), _ptr(scales), threads)
    return codes, scales


def w4a4_group_dots(a_codes, w_codes, threads: int = 0) -> np.ndarray:
    a_codes, w_codes = _c(a_codes, np.uint8), _c(w_codes, np.uint8)
    m, k = a_codes.shape[0], a_codes.shape[1] * 2
    n = w_codes.shape[0]
    dots = np.zeros((m, n, k // GROUP), dtype=np.int32)
    lib().qio_w4a4_group_dots(_ptr(a_codes), _ptr(w_codes), m, n, k, _ptr(dots), threads)
    return dots


def w4a4_gemm(a_codes, a_scales, w_codes, w_scales, bias=None, double: bool = False, threads: int = 0):
    a_codes, w_codes = _c(a_codes, np.uint8), _c(w_codes, np.uint8)
    a_scales, w_scales = _c(a_scales, np.uint16), _c(w_scales, np.uint16)
    bias = None if bias is None else _c(bias, np.float32)
    m, k = a_codes.shape[0], a_codes.shape[1] * 2
    n = w_codes.shape[0]
    y = np.zeros((m, n), dtype=np.float32)
    fn = lib().qio_w4a4_gemm_f64 if double else lib().qio_w4a4_gemm
    fn(_ptr(a_codes), _ptr(a_scales), _ptr(w_codes), _ptr(w_scales), _ptr(bias), _ptr(y), m, n, k, threads)
    return y


def w4a16_dequantize(codes, scales, minimums) -> np.ndarray:
    codes, scales, minimums = _c(codes, np.uint8), _c(scales, np.uint16), _c(minimums, np.uint16)
    n, k = codes.shape[0], codes.shape[1] * 2
    out = np.zeros((n, k), dtype=np.uint16)
    lib().qio_w4a16_dequantize(_ptr(codes), _ptr(scales), _ptr(minimums), n, k, _ptr(out))
    return out.view(np.float16)


def w4a16_gemm(x_f16, codes, scales, minimums, bias=None, threads: int = 0):
    x = _c(x_f16.view(np.uint16) if x_f16.dtype == np.float16 else x_f16, np.uint16)
    codes, scales, minimums = _c(codes, np.uint8), _c(scales, np.uint16), _c(minimums, np.uint16)
    bias = None if bias is None else _c(bias, np.float32)
    m, k = x.shape
    n = codes.shape[0]
    y = np.zeros((m, n), dtype=np.float32)
    lib().qio_w4a16_gemm(_ptr(x), _ptr(codes), _ptr(scales), _ptr(minimums), _ptr(bias), _ptr(y), m, n, k,
                         threads)
    return y


def w4a4_linear_fast(x_f16, w_codes, w_scales, threads: int = 0):
    x = _c(x_f16.view(np.uint16) if x_f16.dtype == np.float16 else x_f16, np.uint16)
    w_codes, w_scales = _c(w_codes, np.uint8), _c(w_scales, np.uint16)
    m, k = x.shape
    n = w_codes.shape[0]
    y = np.zeros((m, n), dtype=np.float32)
    lib().qio_w4a4_linear_fast(_ptr(x), _ptr(w_codes), _ptr(w_scales), _ptr(y), m, n, k, threads)
    return y


def w4a16_linear_fast(x_f16, codes, scales, minimums, threads: int = 0):
    x = _c(x_f16.view(np.uint16) if x_f16.dtype == np.float16 else x_f16, np.uint16)
    codes, scales, minimums = _c(codes, np.uint8), _c(scales, np.uint16), _c(minimums, np.uint16)
    m, k = x.shape
    n = codes.shape[0]
    y = np.zeros((m, n), dtype=np.float32)
    lib().qio_w4a16_linear_fast(_ptr(x), _ptr(codes), _ptr(scales), _ptr(minimums), _ptr(y), m, n, k, threads)
    return y


def unpack_codes(codes: np.ndarray, signed: bool) -> np.ndarray:
    """[rows, k/2] bytes -> [rows, k] int8 code values (even column = low nibble)."""
    codes = np.asarray(codes, dtype=np.uint8)
    out = np.empty((codes.shape[0], codes.shape[1] * 2), dtype=np.int8)
    out[:, 0::2] = codes & 0x0F
    out[:, 1::2] = codes >> 4
    if signed:
        out = np.where(out > 7, out - 16, out).astype(np.int8)
    return out
