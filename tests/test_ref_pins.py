"""The CPU checker pinned to REFERENCE CODE, bit for bit, wherever the reference's own
sources for the path are plain C++ that compiles here: oracle/build_ref.py builds them from
the reference tree (unmodified files with stand-in third-party headers, or code blocks
extracted at build time) into oracle/_ref/libref_pins.so.

  fp32_to_bfloat16          src/util.cpp:33-72              every 32-bit pattern
  ModelBase::InitFreqCIS    src/model_base.cpp:27-83        theta 1e4 / 1e6, fp16 / bf16, 32 896 rows
  InitFreqCIS (test twin)   tests/npu_op_test_util.cpp:109-142
  RoPE golden loop          tests/rope_single_layer_test.cpp:78-97   both pairings, both dtypes
  causal mask loop          tests/flash_attn_test.cpp:124-132
  all_close                 tests/npu_op_test_util.cpp:33-48

The two contractions of the attention golden are Eigen code and stay restated; for them torch's
CPU fp32 scaled_dot_product_attention is the independent second opinion (last tests below).
Where the reference tree is absent the live comparisons are skipped and the committed fixture
(tests/golden/ref_pins.npz, written from the same compiled reference code by
tests/golden/make_ref_pins.py) carries the pins.
"""
import ctypes
import os

import numpy as np
import pytest

from oracle import oracle as orc
from oracle import ref_pins as ref

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
live = pytest.mark.skipif(not ref.available(), reason="reference tree not present and no library built earlier")
FP16, BF16 = orc.DT_FLOAT16, orc.DT_BFLOAT16


@pytest.fixture(scope="module")
def pins():
    return np.load(os.path.join(ROOT, "tests", "golden", "ref_pins.npz"))


def round_independently(x_f32, dt):
    """fp32 -> the 16-bit type -> fp32 with a rounding that is neither the checker's nor the library's."""
    import torch
    t = torch.from_numpy(np.ascontiguousarray(x_f32, dtype=np.float32))
    return t.to(torch.float16 if dt == FP16 else torch.bfloat16).to(torch.float32).numpy()


# ---- live comparisons with the compiled reference code -------------------------------------
@live
def test_bf16_rounding_equals_the_reference_routine_on_every_pattern():
    fn = ctypes.cast(orc.lib().cpu_fp32_to_bfloat16, ctypes.c_void_p)
    assert ref.bf16_sweep(fn, 0, 1 << 32) == (0, 0)


@live
def test_tensor_rounding_equals_the_reference_routine_except_on_nan():
    """The checker rounds tensors with a plain round-to-nearest-even that keeps NaN a NaN; the
    reference's table routine agrees with it on every zero, denormal, normal and infinity."""
    fn = ctypes.cast(orc.lib().cpu_f32_bits_to_bf16, ctypes.c_void_p)
    for lo, hi in ((0, 0x7f800001), (0x80000000, 0xff800001)):
        assert ref.bf16_sweep(fn, lo, hi)[0] == 0
    n, first = ref.bf16_sweep(fn, 0x7f800001, 0x80000000)
    assert n > 0 and first == 0x7f800001          # NaN payloads: the only patterns that differ


@live
@pytest.mark.parametrize("theta", [1e4, 1e6])
@pytest.mark.parametrize("dt", [FP16, BF16])
def test_rope_table_equals_model_base_init_freq_cis(theta, dt):
    rows = 32896
    want = ref.model_init_freq_cis(128, rows, theta, dt)
    assert np.array_equal(orc.init_freq_cis(128, rows, theta, dt).view(np.uint32), want.view(np.uint32))
    from llm_simple_b200 import layer                     # the product's host builder
    assert np.array_equal(layer.init_freq_cis(128, rows, theta, dt).view(np.uint32), want.view(np.uint32))


@live
def test_rope_table_test_twin_equals_the_reference_test_utility():
    want = ref.test_init_freq_cis(128, 4100)
    assert np.array_equal(orc.init_freq_cis_test(128, 4100).view(np.uint32), want.view(np.uint32))


@live
@pytest.mark.parametrize("dt", [FP16, BF16])
@pytest.mark.parametrize("neox", [False, True])
@pytest.mark.parametrize("offset,seq,heads", [(0, 7, 3), (511, 1, 12), (32767, 2, 2), (100, 64, 8)])
def test_rope_equals_the_reference_golden_loop(dt, neox, offset, seq, heads):
    rng = np.random.default_rng(offset + seq)
    table = ref.model_init_freq_cis(128, offset + seq, 1e6 if dt == BF16 else 1e4, dt)
    x_bits = orc.to_bits(rng.standard_normal((seq, heads * 128), dtype=np.float32), dt)
    x32 = orc.to_f32(x_bits, dt)
    assert np.array_equal(x32, round_independently(x32, dt))            # widening is exact
    gold = round_independently(ref.rope_golden(x32, table, offset, heads, 128, neox), dt)
    got = orc.to_f32(orc.rope_single_layer(x_bits, table, offset, heads, neox, dt), dt)
    assert np.array_equal(got.view(np.uint32), gold.view(np.uint32))


@live
@pytest.mark.parametrize("m,n,offset", [(1, 1, 0), (7, 300, 293), (129, 257, 128), (64, 64, 0), (5, 9, 2)])
def test_mask_equals_the_reference_mask_loop(m, n, offset):
    """Zero queries make every unmasked score (0 + 0) * scale = 0 and every masked one -inf: the
    checker's scores are then the reference's mask itself."""
    q = np.zeros((m, 128), np.uint16)
    k = orc.to_bits(np.random.default_rng(0).standard_normal((n, 128), dtype=np.float32), FP16)
    s, _ = orc.scores_one_head(q, k, m, n, offset, 128, FP16, orc.MODE_GOLDEN)
    assert np.array_equal(s, ref.causal_mask(m, n, offset))


@live
def test_all_close_gives_the_reference_verdict():
    rng = np.random.default_rng(3)
    a = rng.standard_normal(4096).astype(np.float32)
    for scale in (0.0, 1e-4, 9e-4, 1.1e-3, 1e-2):
        b = a + scale * rng.standard_normal(4096).astype(np.float32)
        for tol in ((1e-3, 1e-3), (1e-2, 1e-3), (1e-4, 1e-2)):
            assert orc.all_close(b, a, *tol) == ref.all_close(b, a, *tol)
    z = np.zeros(8, np.float32)
    assert orc.all_close(z, z) and ref.all_close(z, z)


# ---- the same pins from the committed fixture (no reference tree needed) -----------------------
def test_fixture_bf16_rounding(pins):
    got = np.array([orc.lib().cpu_fp32_to_bfloat16(int(u)) for u in pins["bf16_in"]], dtype=np.uint16)
    assert np.array_equal(got, pins["bf16_out"])


@pytest.mark.parametrize("name,theta,dt", [("table_1e4_fp16", 1e4, FP16), ("table_1e6_bf16", 1e6, BF16)])
def test_fixture_rope_table_rows(pins, name, theta, dt):
    rows = pins["table_rows"]
    got = orc.init_freq_cis(128, int(rows.max()) + 1, theta, dt)[rows]
    assert np.array_equal(got.view(np.uint32), pins[name].view(np.uint32))
    from llm_simple_b200 import layer
    got = layer.init_freq_cis(128, int(rows.max()) + 1, theta, dt)[rows]
    assert np.array_equal(got.view(np.uint32), pins[name].view(np.uint32))


@pytest.mark.parametrize("dt,neox", [(FP16, False), (FP16, True), (BF16, False), (BF16, True)])
def test_fixture_rope_golden(pins, dt, neox):
    key = "rope_%s_%s" % ("fp16" if dt == FP16 else "bf16", "neox" if neox else "inter")
    offset, heads = int(pins["rope_offset"]), int(pins["rope_heads"])
    table = orc.init_freq_cis(128, offset + pins[key + "_in"].shape[0], 1e6 if dt == BF16 else 1e4, dt)
    got = orc.to_f32(orc.rope_single_layer(pins[key + "_in"], table, offset, heads, neox, dt), dt)
    assert np.array_equal(got.view(np.uint32), pins[key + "_gold"].view(np.uint32))


def test_fixture_mask(pins):
    m, n, offset = (int(x) for x in pins["mask_shape"])
    q = np.zeros((m, 128), np.uint16)
    k = np.zeros((n, 128), np.uint16)
    s, _ = orc.scores_one_head(q, k, m, n, offset, 128, FP16, orc.MODE_GOLDEN)
    assert np.array_equal(s, pins["mask"])


# ---- the contractions: torch's CPU attention as the independent second opinion ------------------
def torch_attention(q_bits, k_bits, v_bits, m, n, offset, group, kvh, dt):
    """softmax((q k^T + mask) / sqrt(D)) v in fp32 on the CPU with torch; query head h reads KV head h // group."""
    import torch
    import torch.nn.functional as F
    H = group * kvh
    q = torch.from_numpy(orc.to_f32(q_bits, dt)).reshape(m, H, 128).transpose(0, 1)           # [H][m][D]
    k = torch.from_numpy(orc.to_f32(k_bits, dt)).reshape(-1, kvh, 128)[:n].transpose(0, 1)    # [kvh][n][D]
    v = torch.from_numpy(orc.to_f32(v_bits, dt)).reshape(-1, kvh, 128)[:n].transpose(0, 1)
    k, v = k.repeat_interleave(group, 0), v.repeat_interleave(group, 0)
    visible = torch.arange(n)[None, :] <= (torch.arange(m)[:, None] + offset)
    o = F.scaled_dot_product_attention(q[None], k[None], v[None], attn_mask=visible[None, None])[0]
    return o.transpose(0, 1).reshape(m, H * 128).numpy()


@pytest.mark.parametrize("dt,m,n,offset,group,kvh", [
    (FP16, 256, 256, 0, 1, 32),          # cfg1 (Llama-2-7B shape)
    (BF16, 1, 512, 511, 6, 2),           # cfg2 decode step
    (FP16, 64, 2048, 1984, 1, 4),        # cfg3: the last rows of a 2048-token prompt, four of the 40 heads
    (BF16, 1, 3000, 2999, 5, 8),         # cfg4: one sequence
    (BF16, 48, 8192, 8144, 5, 2),        # cfg5: rows of the third 4096-token chunk, two of the eight KV heads
    (FP16, 7, 300, 293, 1, 3),
    (BF16, 129, 257, 128, 5, 1),
])
def test_attention_golden_agrees_with_torch_sdpa(dt, m, n, offset, group, kvh):
    rng = np.random.default_rng(m * 31 + n)
    H = group * kvh
    q = orc.to_bits(rng.standard_normal((m, H * 128), dtype=np.float32), dt)
    k = orc.to_bits(rng.standard_normal((n, kvh * 128), dtype=np.float32), dt)
    v = orc.to_bits(rng.standard_normal((n, kvh * 128), dtype=np.float32), dt)
    gold = orc.attn(q, k, v, m, n, offset, group, kvh, 128, dt, orc.MODE_GOLDEN, threads=8)
    want = torch_attention(q, k, v, m, n, offset, group, kvh, dt)
    # both are fp32 evaluations of the same formula; only the summation order differs
    assert np.abs(gold - want).max() <= 2e-5, np.abs(gold - want).max()
    # and the reference layer's rounding points stay within the parity bound of that
    strict = orc.to_f32(orc.attn(q, k, v, m, n, offset, group, kvh, 128, dt, orc.MODE_STRICT, threads=8), dt)
    bound = 1e-2 if dt == FP16 else 4e-2
    assert np.abs(strict - want).max() <= bound


def test_fixture_attention_agrees_with_torch_sdpa(golden):
    """The numpy-written fixtures of the attention golden against torch as well."""
    cases = sorted({k.split("/")[0] for k in golden.files if k.startswith("fa_")})
    assert cases
    for c in cases:
        dt, m, n, offset, group, kvh, _ = (int(x) for x in golden[c + "/meta"])
        want = torch_attention(golden[c + "/q"], golden[c + "/k"], golden[c + "/v"], m, n, offset, group, kvh, dt)
        assert np.abs(golden[c + "/o"] - want).max() <= 2e-5, c
