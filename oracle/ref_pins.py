"""ctypes binding of oracle/_ref/libref_pins.so: pieces of the hot path compiled from the
reference tree itself (oracle/build_ref.py).  Test infrastructure only; available() is False
where neither the reference tree nor a library built earlier exists."""
import ctypes
import os

import numpy as np

from . import build_ref

_lib = None
_f32p = ctypes.POINTER(ctypes.c_float)


def lib():
    global _lib
    if _lib is None:
        path = build_ref.build()
        if not path or not os.path.exists(path):
            return None
        L = ctypes.CDLL(path)
        L.ref_fp32_to_bfloat16.restype = ctypes.c_uint16
        L.ref_fp32_to_bfloat16.argtypes = [ctypes.c_uint32]
        L.ref_bf16_sweep.restype = ctypes.c_uint64
        L.ref_bf16_sweep.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint64, ctypes.POINTER(ctypes.c_uint32)]
        L.ref_all_close.argtypes = [_f32p, _f32p, ctypes.c_size_t, ctypes.c_float, ctypes.c_float]
        L.ref_test_init_freq_cis.argtypes = [_f32p, ctypes.c_int, ctypes.c_int]
        L.ref_model_init_freq_cis.argtypes = [_f32p, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_int]
        L.ref_rope_golden.argtypes = [_f32p, _f32p, _f32p] + [ctypes.c_int] * 5
        L.ref_causal_mask.argtypes = [_f32p] + [ctypes.c_int] * 3
        _lib = L
    return _lib


def available():
    return lib() is not None


def _f32(a):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_f32p)


def fp32_to_bfloat16(bits):
    return int(lib().ref_fp32_to_bfloat16(int(bits)))


def bf16_sweep(other_fn_ptr, lo, hi):
    """(mismatches, first mismatching pattern) of a `uint16_t f(uint32_t)` against src/util.cpp's routine."""
    first = ctypes.c_uint32(0)
    n = int(lib().ref_bf16_sweep(other_fn_ptr, lo, hi, ctypes.byref(first)))
    return n, int(first.value)


def model_init_freq_cis(head_dim, max_seq_len, theta, dt):
    out = np.empty((max_seq_len, head_dim // 2, 2), dtype=np.float32)
    assert lib().ref_model_init_freq_cis(_f32(out), head_dim, max_seq_len, theta, dt) == 0
    return out


def test_init_freq_cis(head_dim, max_seq_len):
    out = np.empty((max_seq_len, head_dim // 2, 2), dtype=np.float32)
    lib().ref_test_init_freq_cis(_f32(out), head_dim, max_seq_len)
    return out


def rope_golden(x_f32, freq_cis, offset, head_num, head_dim, is_neox):
    """x_f32 [seq_len][head_num*head_dim] fp32 -> the reference loop's fp32 golden (unrounded)."""
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    out = np.zeros_like(x)
    lib().ref_rope_golden(_f32(out), _f32(x), _f32(np.ascontiguousarray(freq_cis, dtype=np.float32)), offset, x.shape[0],
                          head_num, head_dim, int(bool(is_neox)))
    return out


def causal_mask(m, n, offset):
    out = np.empty((m, n), dtype=np.float32)
    lib().ref_causal_mask(_f32(out), m, n, offset)
    return out


def all_close(out, golden, abs_err=1e-3, rel_err=1e-3):
    a = np.ascontiguousarray(out, dtype=np.float32).ravel()
    b = np.ascontiguousarray(golden, dtype=np.float32).ravel()
    # the reference's routine reports the first mismatch on stdout: keep the test output clean
    fd = os.dup(1)
    devnull = os.open(os.devnull, os.O_WRONLY)
    try:
        os.dup2(devnull, 1)
        return bool(lib().ref_all_close(_f32(a), _f32(b), a.size, abs_err, rel_err))
    finally:
        os.dup2(fd, 1)
        os.close(fd)
        os.close(devnull)
