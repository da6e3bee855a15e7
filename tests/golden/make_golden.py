"""Generate the golden fixtures in this folder.

An independent numpy restatement of the golden math in the reference's own op
tests (not of the oracle, and sharing no code with it):

  * attention: tests/flash_attn_test.cpp:88-192 -- inputs rounded to the 16-bit
    dtype and widened again, mask col > row + offset -> -inf, S = (Q.K^T + mask)
    * 1/sqrt(D), row softmax, O = P.V, output [m][H*D], all in fp32;
  * RoPE: tests/rope_single_layer_test.cpp:78-97 (both pairings, result rounded
    to the dtype) with the table of tests/npu_op_test_util.cpp:109-142.

GQA cases expand K/V heads with the repeat convention q_head -> q_head // G
(call site src/llama2_layer_npu.cpp:866-869); the reference has no test for it.

The reference itself cannot be executed (closed Ascend binary; Eigen missing),
so these vectors are "restated", not "recorded".  Inputs are seeded N(0,1).

Run:  python tests/golden/make_golden.py      (needs numpy and ml_dtypes)
"""
import os

import ml_dtypes
import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
NPDT = {4: np.float16, 5: ml_dtypes.bfloat16}


def round_dt(x, dt):
    return x.astype(NPDT[dt]).astype(np.float32)


def bits(x, dt):
    return x.astype(NPDT[dt]).view(np.uint16)


def freq_table_test(head_dim, max_seq_len):
    theta = np.float32(10000.0)
    i = np.arange(head_dim // 2, dtype=np.float32)
    freq = (np.float32(1.0) / np.power(theta, (i * np.float32(2)) / np.float32(head_dim))).astype(np.float32)
    t = np.arange(max_seq_len, dtype=np.float32)
    ang = (t[:, None] * freq[None, :]).astype(np.float32)
    out = np.empty((max_seq_len, head_dim // 2, 2), np.float32)
    # cos/sin of the fp32 angle, evaluated in double and rounded once
    out[..., 0] = np.cos(ang.astype(np.float64)).astype(np.float32)
    out[..., 1] = np.sin(ang.astype(np.float64)).astype(np.float32)
    return out


def rope_golden(x, table, offset, n_heads, head_dim, neox, dt):
    s_len = x.shape[0]
    x = x.reshape(s_len, n_heads, head_dim)
    out = np.empty_like(x)
    fc = table[offset:offset + s_len, :, 0][:, None, :]
    fd = table[offset:offset + s_len, :, 1][:, None, :]
    half = head_dim // 2
    if neox:
        a, b = x[..., :half], x[..., half:]
        out[..., :half] = a * fc - b * fd
        out[..., half:] = a * fd + b * fc
    else:
        a, b = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = a * fc - b * fd
        out[..., 1::2] = a * fd + b * fc
    return round_dt(out, dt).reshape(s_len, n_heads * head_dim)


def attn_golden(q, k, v, m, n, offset, group, kv_heads, head_dim):
    H = group * kv_heads
    q = q.reshape(m, H, head_dim)
    k = np.repeat(k.reshape(n, kv_heads, head_dim), group, axis=1)
    v = np.repeat(v.reshape(n, kv_heads, head_dim), group, axis=1)
    scale = np.float32(1.0) / np.sqrt(np.float32(head_dim))
    s = np.einsum("mhd,nhd->hmn", q, k).astype(np.float32)
    rows = np.arange(m)[:, None]
    cols = np.arange(n)[None, :]
    mask = np.where(cols > rows + offset, -np.inf, 0.0).astype(np.float32)
    s = (s + mask[None]) * scale
    mx = s.max(axis=2, keepdims=True)
    e = np.exp(s - mx)
    p = e / e.sum(axis=2, keepdims=True)
    o = np.einsum("hmn,nhd->mhd", p.astype(np.float32), v).astype(np.float32)
    return o.reshape(m, H * head_dim), s, p


ATTN_CASES = [
    # name, dt, m, n, offset, group, kv_heads
    ("fa_fp16_m16_n16_o0_h2", 4, 16, 16, 0, 1, 2),
    ("fa_fp16_m7_n300_o293_h3", 4, 7, 300, 293, 1, 3),
    ("fa_fp16_m1_n65_o64_h4", 4, 1, 65, 64, 1, 4),
    ("fa_fp16_m1_n1_o0_h2", 4, 1, 1, 0, 1, 2),
    ("fa_fp16_m130_n130_o0_h1", 4, 130, 130, 0, 1, 1),
    ("fa_bf16_gqa_m5_n40_o35_g3_kv2", 5, 5, 40, 35, 3, 2),
    ("fa_bf16_gqa_m1_n129_o128_g6_kv2", 5, 1, 129, 128, 6, 2),
    ("fa_bf16_gqa_m33_n97_o64_g5_kv1", 5, 33, 97, 64, 5, 1),
]

ROPE_CASES = [
    # name, dt, seq_len, offset, heads, neox
    ("rope_fp16_inter_s5_o0_h3", 4, 5, 0, 3, False),
    ("rope_fp16_neox_s5_o17_h3", 4, 5, 17, 3, True),
    ("rope_bf16_inter_s1_o63_h2", 5, 1, 63, 2, False),
    ("rope_bf16_neox_s9_o40_h4", 5, 9, 40, 4, True),
]


def main():
    D = 128
    out = {}
    rng = np.random.default_rng(20250)
    for name, dt, m, n, offset, group, kvh in ATTN_CASES:
        H = group * kvh
        q = round_dt(rng.standard_normal((m, H * D), dtype=np.float32), dt)
        k = round_dt(rng.standard_normal((n, kvh * D), dtype=np.float32), dt)
        v = round_dt(rng.standard_normal((n, kvh * D), dtype=np.float32), dt)
        o, s, p = attn_golden(q, k, v, m, n, offset, group, kvh, D)
        out[name + "/q"] = bits(q, dt)
        out[name + "/k"] = bits(k, dt)
        out[name + "/v"] = bits(v, dt)
        out[name + "/o"] = o
        # scaled scores and probabilities of head 0, for the S / P known-answer checks
        if m * n <= 4096:
            out[name + "/s0"] = s[0]
            out[name + "/p0"] = p[0]
        out[name + "/meta"] = np.array([dt, m, n, offset, group, kvh, D], np.int32)
    table = freq_table_test(D, 64)
    out["rope_table_theta1e4_64"] = table
    for name, dt, s_len, offset, heads, neox in ROPE_CASES:
        x = round_dt(rng.standard_normal((s_len, heads * D), dtype=np.float32), dt)
        g = rope_golden(x, table, offset, heads, D, neox, dt)
        out[name + "/x"] = bits(x, dt)
        out[name + "/y"] = bits(g, dt)
        out[name + "/meta"] = np.array([dt, s_len, offset, heads, int(neox), D], np.int32)
    path = os.path.join(HERE, "attn_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
