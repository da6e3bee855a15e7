"""ctypes binding of the CPU checker (oracle/attn_oracle.cpp).

Test infrastructure only: imported by tests/, by the smoke check and by the
CPU-baseline leg of the benchmark.  The shipped package never imports it.
What pins it to reference code (tests/test_ref_pins.py) and what stays pinned
only by restatement (the attention contractions) is listed in attn_oracle.h.

All 16-bit tensors travel as numpy uint16 arrays holding the raw fp16 / bf16
bits; dtype codes are the reference's DataType values (prebuild/defs.hpp:8-18).
"""
import ctypes
import os
import subprocess

import numpy as np

DT_FLOAT16 = 4
DT_BFLOAT16 = 5
MODE_STRICT = 0  # rounding points of src/llama2_layer_cpu.cpp
MODE_GOLDEN = 1  # fp32 throughout, tests/flash_attn_test.cpp

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libattn_oracle.so")
_lib = None

_u16p = ctypes.POINTER(ctypes.c_uint16)
_f32p = ctypes.POINTER(ctypes.c_float)


def build(force=False):
    """Compile the checker with the Makefile beside it."""
    src = os.path.join(_HERE, "attn_oracle.cpp")
    if (not force and os.path.exists(_LIB_PATH)
            and os.path.getmtime(_LIB_PATH) >= os.path.getmtime(src)):
        return _LIB_PATH
    env = dict(os.environ)
    env.pop("CXX", None)
    subprocess.check_call(["make", "-C", _HERE, "-B", "libattn_oracle.so"], env=env,
                          stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = ctypes.CDLL(_LIB_PATH)
        L.cpu_fp32_to_bfloat16.restype = ctypes.c_uint16
        L.cpu_fp32_to_bfloat16.argtypes = [ctypes.c_uint32]
        L.cpu_oracle_max_threads.restype = ctypes.c_int
        _lib = L
    return _lib


def _u16(a):
    assert a.dtype == np.uint16 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_u16p)


def _f32(a):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_f32p)


def max_threads():
    return int(lib().cpu_oracle_max_threads())


def to_bits(x, dt):
    """fp32 array -> uint16 bit pattern of the dtype (round-to-nearest-even)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().cpu_f32_to_dt(_u16(out), _f32(x), ctypes.c_size_t(x.size), dt)
    return out


def to_f32(bits, dt):
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(bits.shape, dtype=np.float32)
    lib().cpu_dt_to_f32(_f32(out), _u16(bits), ctypes.c_size_t(bits.size), dt)
    return out


def init_freq_cis(head_dim, max_seq_len, theta, dt):
    """ModelBase::InitFreqCIS (src/model_base.cpp:27-83): [max_seq_len][D/2][2] fp32."""
    out = np.empty((max_seq_len, head_dim // 2, 2), dtype=np.float32)
    lib().cpu_init_freq_cis(_f32(out), head_dim, max_seq_len, ctypes.c_float(theta), dt)
    return out


def init_freq_cis_test(head_dim, max_seq_len):
    """tests/npu_op_test_util.cpp:109-142."""
    out = np.empty((max_seq_len, head_dim // 2, 2), dtype=np.float32)
    lib().cpu_init_freq_cis_test(_f32(out), head_dim, max_seq_len)
    return out


def rope_single_layer(x, freqs_cis, start_pos, n_heads, is_neox, dt):
    """x: uint16 [cur_size][n_heads*head_dim] -> rotated, same shape."""
    x = np.ascontiguousarray(x)
    cur_size = x.shape[0]
    hidden = int(np.prod(x.shape[1:]))
    out = np.empty_like(x)
    rc = lib().cpu_rope_single_layer(_u16(out), _f32(np.ascontiguousarray(freqs_cis)), _u16(x),
                                     start_pos, cur_size, n_heads, hidden, int(is_neox), dt)
    assert rc == 0
    return out


def rope_layer(q, k, freqs_cis, start_pos, n_heads, is_neox, dt):
    q = np.ascontiguousarray(q)
    k = np.ascontiguousarray(k)
    cur_size = q.shape[0]
    hidden = int(np.prod(q.shape[1:]))
    oq, ok = np.empty_like(q), np.empty_like(k)
    rc = lib().cpu_rope_layer(_u16(oq), _u16(ok), _f32(np.ascontiguousarray(freqs_cis)), _u16(q),
                              _u16(k), start_pos, cur_size, n_heads, hidden, int(is_neox), dt)
    assert rc == 0
    return oq, ok


def split_qkv(qkv, q_dim, k_dim, v_dim):
    """Row-wise split of a fused projection output [rows][q_dim + k_dim + v_dim] into
    three dense arrays: the definition of npu_split_qkv_layer (prebuild/npu_ops.h:27-30;
    the reference ships no CPU twin and no test of it)."""
    qkv = np.ascontiguousarray(qkv)
    assert qkv.shape[-1] == q_dim + k_dim + v_dim
    return (np.ascontiguousarray(qkv[..., :q_dim]), np.ascontiguousarray(qkv[..., q_dim:q_dim + k_dim]),
            np.ascontiguousarray(qkv[..., q_dim + k_dim:]))


def bias_add(x, bias, dt):
    """round_dt(float(x) + float(bias)), bias broadcast over rows: a projection whose
    epilogue adds the bias (npu_matmul_bias_nz_layer, prebuild/npu_ops.h:90-92, as the
    Qwen2 q/k/v projections use it, src/llama2_layer_npu.cpp:1174-1177) rounds once, here
    the projection output is already 16-bit, so this is the second rounding point."""
    return to_bits(to_f32(x, dt) + to_f32(bias, dt), dt)


def kv_append(k_cache, v_cache, k_emb, v, prev_pos, kv_heads, head_dim):
    """In place, token-major caches [max_pos][kv_heads][head_dim]."""
    cur_size = k_emb.shape[0]
    lib().cpu_kv_append(_u16(k_cache), _u16(v_cache), _u16(np.ascontiguousarray(k_emb)),
                        _u16(np.ascontiguousarray(v)), prev_pos, cur_size, kv_heads, head_dim)


def attn(q, k, v, m, n, offset, group_size, kv_heads, head_dim, dt, mode, layout="token",
         threads=1):
    """Attention of one sequence.

    q uint16 [m][kv_heads*group_size][D]; k, v uint16, token-major [>=n][kv_heads][D]
    or head-major [kv_heads][max_pos][D].  Returns uint16 [m][H*D] (STRICT) or
    float32 [m][H*D] (GOLDEN).
    """
    q = np.ascontiguousarray(q)
    H = group_size * kv_heads
    D = head_dim
    if layout == "token":
        pos_stride, head_stride = kv_heads * D, D
    else:
        max_pos = k.shape[1]
        pos_stride, head_stride = D, max_pos * D
    out16 = np.empty((m, H * D), dtype=np.uint16) if mode == MODE_STRICT else None
    out32 = np.empty((m, H * D), dtype=np.float32) if mode == MODE_GOLDEN else None
    L = lib()
    L.cpu_attn_strided.argtypes = [_u16p, _f32p, _u16p, _u16p, _u16p] + [ctypes.c_int] * 8 + \
        [ctypes.c_long] * 6 + [ctypes.c_int]
    rc = L.cpu_attn_strided(
        _u16(out16) if out16 is not None else None,
        _f32(out32) if out32 is not None else None,
        _u16(q), _u16(k), _u16(v), m, n, offset, group_size, kv_heads, D, dt, mode,
        H * D, pos_stride, head_stride, pos_stride, head_stride, H * D, threads)
    assert rc == 0
    return out16 if mode == MODE_STRICT else out32


def scores_one_head(q, k, m, n, offset, head_dim, dt, mode):
    """Scaled masked scores S and probabilities P of one head: two float32 [m][n]."""
    q = np.ascontiguousarray(q)
    k = np.ascontiguousarray(k)
    s = np.empty((m, n), dtype=np.float32)
    p = np.empty((m, n), dtype=np.float32)
    L = lib()
    L.cpu_scores_one_head.argtypes = [_f32p, _f32p, _u16p, _u16p] + [ctypes.c_int] * 6 + \
        [ctypes.c_long] * 2
    rc = L.cpu_scores_one_head(_f32(s), _f32(p), _u16(q), _u16(k), m, n, offset, head_dim, dt,
                               mode, head_dim, head_dim)
    assert rc == 0
    return s, p


def all_close(out, golden, abs_err=1e-3, rel_err=1e-3):
    """The reference tests' verdict (tests/npu_op_test_util.cpp:33-48)."""
    out = np.ascontiguousarray(out, dtype=np.float32).ravel()
    golden = np.ascontiguousarray(golden, dtype=np.float32).ravel()
    return bool(lib().cpu_all_close(_f32(out), _f32(golden), ctypes.c_size_t(out.size),
                                    ctypes.c_float(abs_err), ctypes.c_float(rel_err)))
