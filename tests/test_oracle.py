"""CPU checks of the oracle itself: fixtures restated from the reference tests'
golden math, analytic known-answer cases, and the table / rounding helpers."""
import numpy as np
import pytest

from oracle import oracle as orc

D = 128
FP16, BF16 = orc.DT_FLOAT16, orc.DT_BFLOAT16

ATTN_CASES = [
    "fa_fp16_m16_n16_o0_h2", "fa_fp16_m7_n300_o293_h3", "fa_fp16_m1_n65_o64_h4",
    "fa_fp16_m1_n1_o0_h2", "fa_fp16_m130_n130_o0_h1", "fa_bf16_gqa_m5_n40_o35_g3_kv2",
    "fa_bf16_gqa_m1_n129_o128_g6_kv2", "fa_bf16_gqa_m33_n97_o64_g5_kv1",
]
ROPE_CASES = ["rope_fp16_inter_s5_o0_h3", "rope_fp16_neox_s5_o17_h3",
              "rope_bf16_inter_s1_o63_h2", "rope_bf16_neox_s9_o40_h4"]


def rnd(shape, dt, seed):
    rng = np.random.default_rng(seed)
    return orc.to_bits(rng.standard_normal(shape, dtype=np.float32), dt)


@pytest.mark.parametrize("name", ATTN_CASES)
def test_attention_golden_fixture(golden, name):
    dt, m, n, offset, g, kvh, d = [int(x) for x in golden[name + "/meta"]]
    out = orc.attn(golden[name + "/q"], golden[name + "/k"], golden[name + "/v"], m, n, offset,
                   g, kvh, d, dt, orc.MODE_GOLDEN)
    ref = golden[name + "/o"]
    # fp32 vs fp32: only summation order differs
    assert np.max(np.abs(out - ref)) < 2e-5
    assert orc.all_close(out, ref)


@pytest.mark.parametrize("name", [c for c in ATTN_CASES if "m130" not in c and "n300" not in c
                                  and "m33" not in c])
def test_scores_and_softmax_fixture(golden, name):
    """S and P of head 0 (the unfused triple the reference also tests:
    tests/npu_operator_test.cpp:553-715 and :93-189)."""
    dt, m, n, offset, g, kvh, d = [int(x) for x in golden[name + "/meta"]]
    q = golden[name + "/q"].reshape(m, g * kvh, d)[:, 0, :]
    k = golden[name + "/k"].reshape(n, kvh, d)[:, 0, :]
    s, p = orc.scores_one_head(q, k, m, n, offset, d, dt, orc.MODE_GOLDEN)
    s_ref, p_ref = golden[name + "/s0"], golden[name + "/p0"]
    assert np.array_equal(np.isneginf(s), np.isneginf(s_ref))
    fin = np.isfinite(s_ref)
    assert np.max(np.abs(s[fin] - s_ref[fin])) < 1e-5
    assert np.max(np.abs(p - p_ref)) < 1e-6


@pytest.mark.parametrize("name", ROPE_CASES)
def test_rope_golden_fixture(golden, name):
    dt, s_len, offset, heads, neox, d = [int(x) for x in golden[name + "/meta"]]
    table = golden["rope_table_theta1e4_64"]
    y = orc.rope_single_layer(golden[name + "/x"], table, offset, heads, neox, dt)
    assert np.array_equal(y, golden[name + "/y"])  # bit-exact: same table, same fp32 ops


def test_freq_cis_against_formula():
    for theta, rows in ((10000.0, 300), (1e6, 1200)):
        t = orc.init_freq_cis(D, rows, theta, FP16)
        i = np.arange(D // 2, dtype=np.float64)
        freq = (1.0 / np.power(np.float64(np.float32(theta)), 2 * i / D)).astype(np.float32)
        ang = (np.arange(rows, dtype=np.float32)[:, None] * freq[None, :]).astype(np.float32)
        assert np.max(np.abs(t[..., 0] - np.cos(ang.astype(np.float64)))) < 2e-7
        assert np.max(np.abs(t[..., 1] - np.sin(ang.astype(np.float64)))) < 2e-7
        assert np.all(t[0, :, 0] == 1.0) and np.all(t[0, :, 1] == 0.0)


def test_freq_cis_test_twin_matches_fixture_table(golden):
    # powf and numpy's float32 power may differ by one ulp in freq; at position p that
    # moves the angle by about p * 6e-8
    t = orc.init_freq_cis_test(D, 64)
    assert np.max(np.abs(t - golden["rope_table_theta1e4_64"])) < 5e-6


def test_freq_cis_bf16_variant_is_rne_of_fp32():
    t32 = orc.init_freq_cis(D, 128, 1e6, FP16)
    t16 = orc.init_freq_cis(D, 128, 1e6, BF16)
    assert np.all((t16.view(np.uint32) & 0xFFFF) == 0)
    assert np.array_equal(t16.view(np.uint32) >> 16, orc.to_bits(t32, BF16).astype(np.uint32))


def test_fp32_to_bfloat16_ties_to_even():
    L = orc.lib()
    rng = np.random.default_rng(1)
    xs = rng.standard_normal(2000).astype(np.float32)
    xs = np.concatenate([xs, np.array([1.0, 1.00390625, 1.01171875, 3.3895314e38, 0.5], np.float32)])
    for x in xs:
        u = int(np.float32(x).view(np.uint32))
        lsb = (u >> 16) & 1
        want = ((u + 0x7FFF + lsb) >> 16) & 0xFFFF
        assert L.cpu_fp32_to_bfloat16(u) == want
    # 1.00390625 = 1 + 2^-8 is an exact tie between 1.0 and 1 + 2^-7 -> even (1.0)
    assert L.cpu_fp32_to_bfloat16(int(np.float32(1.00390625).view(np.uint32))) == 0x3F80


@pytest.mark.parametrize("dt", [FP16, BF16])
def test_single_key_returns_v(dt):
    q, k, v = rnd((1, 4 * D), dt, 1), rnd((1, 2 * D), dt, 2), rnd((1, 2 * D), dt, 3)
    out = orc.attn(q, k, v, 1, 1, 0, 2, 2, D, dt, orc.MODE_STRICT)
    want = np.repeat(v.reshape(1, 2, D), 2, axis=1).reshape(1, 4 * D)
    assert np.array_equal(out, want)


def test_equal_keys_give_running_mean_of_v():
    m = n = 6
    q = rnd((m, D), FP16, 4)
    k = np.tile(rnd((1, D), FP16, 5), (n, 1))
    v = rnd((n, D), FP16, 6)
    out = orc.attn(q, k, v, m, n, 0, 1, 1, D, FP16, orc.MODE_GOLDEN)
    vf = orc.to_f32(v, FP16)
    for r in range(m):
        assert np.allclose(out[r], vf[: r + 1].mean(axis=0), atol=1e-6)


def test_one_hot_score_selects_value():
    n = 9
    q = orc.to_bits(np.full((1, D), 8.0, np.float32), FP16)
    kf = np.zeros((n, D), np.float32)
    kf[4] = 8.0  # score 8*8*128/sqrt(128) = 724 vs 0 elsewhere
    v = rnd((n, D), FP16, 7)
    out = orc.attn(q, orc.to_bits(kf, FP16), v, 1, n, n - 1, 1, 1, D, FP16, orc.MODE_STRICT)
    assert np.array_equal(out[0], v[4])


@pytest.mark.parametrize("mode", [orc.MODE_STRICT, orc.MODE_GOLDEN])
def test_decode_equals_last_prefill_row_and_chunks_equal_full(mode):
    n, H = 37, 3
    q, k, v = rnd((n, H * D), FP16, 8), rnd((n, H * D), FP16, 9), rnd((n, H * D), FP16, 10)
    full = orc.attn(q, k, v, n, n, 0, 1, H, D, FP16, mode)
    dec = orc.attn(q[n - 1:], k, v, 1, n, n - 1, 1, H, D, FP16, mode)
    assert np.array_equal(dec[0], full[n - 1])
    first = orc.attn(q[:20], k, v, 20, 20, 0, 1, H, D, FP16, mode)
    second = orc.attn(q[20:], k, v, n - 20, n, 20, 1, H, D, FP16, mode)
    assert np.array_equal(np.concatenate([first, second]), full)


def test_gqa_group_one_is_mha_and_mapping_is_h_div_g():
    m, n, kvh, g = 3, 11, 2, 3
    q, k, v = rnd((m, kvh * g * D), BF16, 11), rnd((n, kvh * D), BF16, 12), rnd((n, kvh * D), BF16, 13)
    gqa = orc.attn(q, k, v, m, n, n - m, g, kvh, D, BF16, orc.MODE_GOLDEN)
    k_rep = np.repeat(k.reshape(n, kvh, D), g, axis=1).reshape(n, -1)
    v_rep = np.repeat(v.reshape(n, kvh, D), g, axis=1).reshape(n, -1)
    mha = orc.attn(q, k_rep, v_rep, m, n, n - m, 1, kvh * g, D, BF16, orc.MODE_GOLDEN)
    assert np.array_equal(gqa, mha)


def test_head_major_layout_equals_token_major():
    m, n, kvh, g, max_pos = 2, 19, 2, 2, 32
    q, k, v = rnd((m, kvh * g * D), FP16, 14), rnd((n, kvh * D), FP16, 15), rnd((n, kvh * D), FP16, 16)
    tok = orc.attn(q, k, v, m, n, n - m, g, kvh, D, FP16, orc.MODE_STRICT)
    kh = np.zeros((kvh, max_pos, D), np.uint16)
    vh = np.zeros((kvh, max_pos, D), np.uint16)
    kh[:, :n] = k.reshape(n, kvh, D).transpose(1, 0, 2)
    vh[:, :n] = v.reshape(n, kvh, D).transpose(1, 0, 2)
    head = orc.attn(q, kh, vh, m, n, n - m, g, kvh, D, FP16, orc.MODE_STRICT, layout="head")
    assert np.array_equal(tok, head)


def test_strict_and_golden_agree_within_fp16_noise():
    m = n = 64
    H = 4
    q, k, v = rnd((m, H * D), FP16, 17), rnd((n, H * D), FP16, 18), rnd((n, H * D), FP16, 19)
    strict = orc.to_f32(orc.attn(q, k, v, m, n, 0, 1, H, D, FP16, orc.MODE_STRICT), FP16)
    gold = orc.attn(q, k, v, m, n, 0, 1, H, D, FP16, orc.MODE_GOLDEN)
    diff = np.abs(strict - gold)
    assert diff.max() < 1e-2 and diff.mean() < 1e-3


def test_threads_do_not_change_the_result():
    m, n, kvh, g = 4, 50, 4, 2
    q, k, v = rnd((m, kvh * g * D), BF16, 20), rnd((n, kvh * D), BF16, 21), rnd((n, kvh * D), BF16, 22)
    a = orc.attn(q, k, v, m, n, n - m, g, kvh, D, BF16, orc.MODE_GOLDEN, threads=1)
    b = orc.attn(q, k, v, m, n, n - m, g, kvh, D, BF16, orc.MODE_GOLDEN, threads=4)
    assert np.array_equal(a, b)


@pytest.mark.parametrize("dt", [FP16, BF16])
def test_rope_position_zero_is_identity_and_styles_agree_after_permutation(dt):
    table = orc.init_freq_cis(D, 64, 10000.0, dt)
    x = rnd((1, 2 * D), dt, 23)
    assert np.array_equal(orc.rope_single_layer(x, table, 0, 2, False, dt), x)
    assert np.array_equal(orc.rope_single_layer(x, table, 0, 2, True, dt), x)
    xs = rnd((5, 2 * D), dt, 24)
    inter = orc.rope_single_layer(xs, table, 9, 2, False, dt).reshape(5, 2, D)
    # neox on the lane-permuted input equals the interleaved result, permuted
    perm = np.concatenate([np.arange(0, D, 2), np.arange(1, D, 2)])
    neox = orc.rope_single_layer(xs.reshape(5, 2, D)[..., perm].reshape(5, -1), table, 9, 2, True,
                                 dt).reshape(5, 2, D)
    assert np.array_equal(inter[..., perm], neox)


def test_rope_layer_equals_two_single_calls_and_append_is_a_row_copy():
    table = orc.init_freq_cis(D, 64, 10000.0, FP16)
    H, s_len, prev = 3, 4, 7
    q, k, v = rnd((s_len, H * D), FP16, 25), rnd((s_len, H * D), FP16, 26), rnd((s_len, H * D), FP16, 27)
    oq, ok = orc.rope_layer(q, k, table, prev, H, False, FP16)
    assert np.array_equal(oq, orc.rope_single_layer(q, table, prev, H, False, FP16))
    assert np.array_equal(ok, orc.rope_single_layer(k, table, prev, H, False, FP16))
    kc = np.zeros((16, H * D), np.uint16)
    vc = np.zeros((16, H * D), np.uint16)
    orc.kv_append(kc, vc, ok, v, prev, H, D)
    assert np.array_equal(kc[prev:prev + s_len], ok) and np.array_equal(vc[prev:prev + s_len], v)
    assert not kc[:prev].any() and not kc[prev + s_len:].any()


def test_all_close_needs_both_bounds_exceeded():
    g = np.array([100.0, 1e-6], np.float32)
    assert orc.all_close(np.array([100.05, 5e-4], np.float32), g)       # rel ok / abs ok
    assert not orc.all_close(np.array([101.0, 1e-6], np.float32), g)    # both exceeded


@pytest.mark.parametrize("dt", [orc.DT_FLOAT16, orc.DT_BFLOAT16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("m,n,offset,g,kvh", [(64, 64, 0, 1, 4), (37, 300, 263, 5, 2), (1, 1000, 999, 6, 2),
                                               (200, 2200, 2000, 1, 3)])
def test_golden_mode_against_float64(dt, m, n, offset, g, kvh):
    """How exact the fp32 golden itself is: attention evaluated in float64 with numpy (softmax over the visible
    columns, no streaming, no fp32 anywhere) on seeded N(0,1) inputs of the 16-bit type.  The checker's fp32
    golden stays within 2e-6 of it, three orders of magnitude below the parity bound it is used for."""
    D = 128
    rng = np.random.default_rng(m * 7919 + n)
    H = g * kvh
    q = orc.to_bits(rng.standard_normal((m, H * D), dtype=np.float32), dt)
    k = orc.to_bits(rng.standard_normal((n, kvh * D), dtype=np.float32), dt)
    v = orc.to_bits(rng.standard_normal((n, kvh * D), dtype=np.float32), dt)
    gold = orc.attn(q, k, v, m, n, offset, g, kvh, D, dt, orc.MODE_GOLDEN, threads=4)
    q64 = orc.to_f32(q, dt).astype(np.float64).reshape(m, H, D)
    k64 = orc.to_f32(k, dt).astype(np.float64).reshape(n, kvh, D)
    v64 = orc.to_f32(v, dt).astype(np.float64).reshape(n, kvh, D)
    ref = np.empty((m, H, D))
    cols = np.arange(n)[None, :]
    visible = cols <= (np.arange(m)[:, None] + offset)
    for h in range(H):
        s = q64[:, h] @ k64[:, h // g].T / np.sqrt(D)
        s = np.where(visible, s, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        ref[:, h] = (p / p.sum(axis=1, keepdims=True)) @ v64[:, h // g]
    err = np.abs(gold.reshape(m, H, D).astype(np.float64) - ref).max()
    assert err < 2e-6, err
