"""GPU parity of the RoPE operators and of the fused RoPE + KV-append pass,
through the C ABI, against the oracle (bit-exact: same table, same fp32
operations, one rounding).  Shapes follow tests/rope_single_layer_test.cpp and
the RopeLayer gtest (tests/npu_operator_test.cpp:930-1093)."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.gpu_util import BF16, D, FP16, dev, host, rnd_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from llm_simple_b200 import ops as o
    o.lib()
    return o


@pytest.mark.parametrize("dt", [FP16, BF16])
@pytest.mark.parametrize("neox", [False, True])
@pytest.mark.parametrize("seq_len,start,heads,theta", [(1, 0, 2, 1e4), (5, 17, 3, 1e4), (64, 511, 12, 1e6),
                                                       (33, 32767, 8, 1e6), (256, 0, 32, 1e4)])
def test_rope_single_layer_bit_exact(ops, dt, neox, seq_len, start, heads, theta):
    table = orc.init_freq_cis(D, start + seq_len, theta, dt)
    x = rnd_bits((seq_len, heads * D), dt, 100 + seq_len)
    want = orc.rope_single_layer(x, table, start, heads, neox, dt)
    tab_d = torch.from_numpy(table).cuda()
    x_d = dev(x, dt)
    y_d = torch.empty_like(x_d)
    ops.gpu_rope_single_layer(y_d, tab_d, x_d, start, seq_len, heads, heads * D, neox, dt)
    torch.cuda.synchronize()
    assert np.array_equal(host(y_d), want)


@pytest.mark.parametrize("name", ["rope_fp16_inter_s5_o0_h3", "rope_fp16_neox_s5_o17_h3",
                                  "rope_bf16_inter_s1_o63_h2", "rope_bf16_neox_s9_o40_h4"])
def test_rope_single_layer_golden_fixture(ops, golden, name):
    dt, s_len, offset, heads, neox, d = [int(v) for v in golden[name + "/meta"]]
    tab_d = torch.from_numpy(golden["rope_table_theta1e4_64"]).cuda()
    x_d = dev(golden[name + "/x"], dt)
    y_d = torch.empty_like(x_d)
    ops.gpu_rope_single_layer(y_d, tab_d, x_d, offset, s_len, heads, heads * d, neox, dt)
    torch.cuda.synchronize()
    assert np.array_equal(host(y_d), golden[name + "/y"])


@pytest.mark.parametrize("seq_len", [1, 7, 300, 2048])
def test_rope_layer_q_and_k(ops, seq_len):
    # the reference's RopeLayer gtest: fp16, interleaved, H = 40, D = 128, random start_pos
    heads, dt = 40, FP16
    start = int(np.random.default_rng(seq_len).integers(0, 2048 - seq_len + 1))
    table = orc.init_freq_cis_test(D, 2048)
    q, k = rnd_bits((seq_len, heads * D), dt, 1), rnd_bits((seq_len, heads * D), dt, 2)
    wq, wk = orc.rope_layer(q, k, table, start, heads, False, dt)
    tab_d = torch.from_numpy(table).cuda()
    q_d, k_d = dev(q, dt), dev(k, dt)
    oq, ok = torch.empty_like(q_d), torch.empty_like(k_d)
    ops.gpu_rope_layer(oq, ok, tab_d, q_d, k_d, start, seq_len, heads, heads * D, False, dt)
    torch.cuda.synchronize()
    assert np.array_equal(host(oq), wq) and np.array_equal(host(ok), wk)


@pytest.mark.parametrize("dt,neox,theta", [(FP16, False, 1e4), (BF16, True, 1e6)])
@pytest.mark.parametrize("layout", ["token", "head"])
@pytest.mark.parametrize("batch,m,H,kvH", [(1, 256, 32, 32), (3, 5, 12, 2), (8, 1, 40, 8), (5, 1001, 3, 1)])
def test_fused_rope_kv_append(ops, dt, neox, theta, layout, batch, m, H, kvH):
    max_pos = max(320, m + 64)
    rng = np.random.default_rng(batch * 1000 + m)
    starts = rng.integers(0, max_pos - m + 1, size=batch).astype(np.int32)
    table = orc.init_freq_cis(D, max_pos, theta, dt)
    q = rnd_bits((batch, m, H * D), dt, 3)
    k = rnd_bits((batch, m, kvH * D), dt, 4)
    v = rnd_bits((batch, m, kvH * D), dt, 5)
    canary = np.uint16(0x7BCD)
    desc = ops.make_desc(dt, batch, H, kvH, m, max_pos, layout=layout, is_neox=neox)
    shape = (batch, kvH, max_pos, D) if layout == "head" else (batch, max_pos, kvH, D)
    kc = np.full(shape, canary, np.uint16)
    vc = np.full(shape, canary, np.uint16)
    kc_d, vc_d = dev(kc, dt), dev(vc, dt)
    q_d, k_d, v_d = dev(q, dt), dev(k, dt), dev(v, dt)
    qo_d = torch.empty_like(q_d)
    ops.gpu_rope_kv_append_layer(desc, qo_d, kc_d, vc_d, q_d, k_d, v_d, torch.from_numpy(table).cuda(),
                                 torch.from_numpy(starts).cuda(), 0, m)
    torch.cuda.synchronize()
    got_q, got_k, got_v = host(qo_d), host(kc_d), host(vc_d)
    for b in range(batch):
        s = int(starts[b])
        wq = orc.rope_single_layer(q[b], table, s, H, neox, dt)
        wk = orc.rope_single_layer(k[b], table, s, kvH, neox, dt)
        assert np.array_equal(got_q[b], wq)
        want_k = np.full((max_pos, kvH * D), canary, np.uint16)
        want_v = np.full((max_pos, kvH * D), canary, np.uint16)
        orc.kv_append(want_k, want_v, wk, v[b], s, kvH, D)
        if layout == "head":
            want_k = want_k.reshape(max_pos, kvH, D).transpose(1, 0, 2)
            want_v = want_v.reshape(max_pos, kvH, D).transpose(1, 0, 2)
        # rows outside [s, s+m) keep the canary: the append writes nothing else
        assert np.array_equal(got_k[b].reshape(want_k.shape), want_k)
        assert np.array_equal(got_v[b].reshape(want_v.shape), want_v)


def test_rope_rejects_bad_arguments(ops):
    x = torch.zeros(4, 256, dtype=torch.float16, device="cuda")
    tab = torch.zeros(8, 64, 2, device="cuda")
    with pytest.raises(ops.GpuOpsError):
        ops.gpu_rope_single_layer(x, tab, x, 0, 4, 2, 256, False, 6)      # fp32 is not supported
    with pytest.raises(ops.GpuOpsError):
        ops.gpu_rope_single_layer(x, tab, x, 0, 4, 4, 256, False, FP16)   # head_dim 64
    with pytest.raises(ops.GpuOpsError):
        ops.gpu_rope_single_layer(x, tab, x, -1, 4, 2, 256, False, FP16)  # negative start
    assert "start_pos" in ops.last_error_string()


def test_append_beyond_the_cache_of_a_sequence_is_rejected(ops):
    """Two sequences with caches of 64 positions: rows 60..67 of a sequence would land in its neighbour's cache."""
    H, kvh, max_pos, m = 4, 2, 64, 8
    desc = ops.make_desc(FP16, 2, H, kvh, m, max_pos, layout="head")
    q = torch.zeros((2, m, H * 128), dtype=torch.float16, device="cuda")
    kv = torch.zeros((2, m, kvh * 128), dtype=torch.float16, device="cuda")
    cache = torch.zeros((2, kvh, max_pos, 128), dtype=torch.float16, device="cuda")
    tab = torch.zeros((max_pos + m, 64, 2), device="cuda")
    ops.gpu_rope_kv_append_layer(desc, q, cache, cache.clone(), q, kv, kv, tab, None, max_pos - m, m)   # fits exactly
    with pytest.raises(ops.GpuOpsError, match="do not fit the cache"):
        ops.gpu_rope_kv_append_layer(desc, q, cache, cache.clone(), q, kv, kv, tab, None, max_pos - m + 4, m)
