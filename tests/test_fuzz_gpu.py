"""Seeded random sweep of shapes through the C ABI against the oracle: the
reference-shaped GQA attention on both prefill kernels (m, n, offset, group
size, KV heads and dtype drawn at random, including values that are ragged
against every tile size of the kernels), the batched fused decode step with
ragged lengths on both cache layouts, and inputs with a wide dynamic range
(scores spread over many powers of two, which exercises the lazy rescaling of
the running maximum)."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.gpu_util import BF16, D, FP16, assert_parity, dev, host, rnd_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from llm_simple_b200 import ops as o
    o.lib()
    return o


def _attn_cases(n_cases, seed):
    rng = np.random.default_rng(seed)
    cases = []
    for i in range(n_cases):
        m = int(rng.choice([1, 2, 3, 17, 63, 64, 65, 127, 128, 129, 255, 256, 257, 300, 385]))
        offset = int(rng.choice([0, 0, 1, 63, 64, 127, 128, 200, 511]))
        g = int(rng.choice([1, 1, 2, 5, 6, 8]))
        kvh = int(rng.choice([1, 2, 3]))
        dt = int(rng.choice([FP16, BF16]))
        cases.append((i, m, offset, g, kvh, dt))
    return cases


@pytest.mark.parametrize("case", _attn_cases(24, 20250), ids=lambda c: "m%d_o%d_g%d_kv%d_dt%d" % c[1:])
@pytest.mark.parametrize("kernel", [1, 2, 3], ids=["mma", "tcgen05", "tcgen05-persistent"])
def test_random_gqa_shapes(ops, kernel, case):
    i, m, offset, g, kvh, dt = case
    n = m + offset
    H = g * kvh
    q, k, v = rnd_bits((m, H * D), dt, 100 + i), rnd_bits((n, kvh * D), dt, 200 + i), rnd_bits((n, kvh * D), dt, 300 + i)
    out = torch.empty((m, H * D), dtype=dev(q[:1], dt).dtype, device="cuda")
    ops.gpu_attn_set_prefill_kernel(kernel)
    try:
        ops.gpu_flash_attn_gqa_layer(out, dev(q, dt), dev(k, dt), dev(v, dt), m, n, offset, g, kvh, D, dt)
        torch.cuda.synchronize()
    finally:
        ops.gpu_attn_set_prefill_kernel(0)
    assert ops.gpu_ops_kernel_status() == 0
    gold = orc.attn(q, k, v, m, n, offset, g, kvh, D, dt, orc.MODE_GOLDEN, threads=8)
    assert_parity(host(out), gold, dt, "case %d" % i)


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("layout", ["token", "head"])
def test_random_ragged_decode(ops, seed, layout):
    rng = np.random.default_rng(777 + seed)
    batch = int(rng.integers(1, 9))
    kvh = int(rng.choice([1, 2, 4]))
    g = int(rng.choice([1, 4, 5, 7, 16]))
    dt = int(rng.choice([FP16, BF16]))
    neox = bool(rng.integers(0, 2))
    H = g * kvh
    max_pos = 1400
    lens = rng.integers(0, max_pos - 1, size=batch).astype(np.int32)
    lens[rng.integers(0, batch)] = int(rng.choice([0, 63, 64, 255, 256, 1023, 1024]))   # tile and split edges
    table = orc.init_freq_cis(D, max_pos, 1e6, dt)
    q, k, v = rnd_bits((batch, H * D), dt, seed), rnd_bits((batch, kvh * D), dt, 50 + seed), rnd_bits((batch, kvh * D), dt, 90 + seed)
    kc_tok = rnd_bits((batch, max_pos, kvh * D), dt, 130 + seed)      # token-major truth
    vc_tok = rnd_bits((batch, max_pos, kvh * D), dt, 170 + seed)
    if layout == "head":
        kc_dev = dev(np.ascontiguousarray(kc_tok.reshape(batch, max_pos, kvh, D).transpose(0, 2, 1, 3)), dt)
        vc_dev = dev(np.ascontiguousarray(vc_tok.reshape(batch, max_pos, kvh, D).transpose(0, 2, 1, 3)), dt)
    else:
        kc_dev, vc_dev = dev(kc_tok, dt), dev(vc_tok, dt)
    desc = ops.make_desc(dt, batch, H, kvh, 1, max_pos, layout=layout, is_neox=neox)
    mx = int(lens.max()) + 1
    ws_bytes = ops.gpu_attn_decode_workspace_bytes(desc, mx)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")
    out = torch.empty((batch, H * D), dtype=kc_dev.dtype, device="cuda")
    ops.gpu_attn_decode_layer(desc, out, None, None, dev(q, dt), dev(k, dt), dev(v, dt), kc_dev, vc_dev,
                              torch.from_numpy(table).cuda(), torch.from_numpy(lens).cuda(), None, True, mx, ws, ws_bytes)
    torch.cuda.synchronize()
    got = host(out)
    for b in range(batch):
        L = int(lens[b])
        q_r = orc.rope_single_layer(q[b:b + 1], table, L, H, neox, dt)
        k_r = orc.rope_single_layer(k[b:b + 1], table, L, kvh, neox, dt)
        kc, vc = kc_tok[b].copy(), vc_tok[b].copy()
        orc.kv_append(kc, vc, k_r, v[b:b + 1], L, kvh, D)
        gold = orc.attn(q_r, kc, vc, 1, L + 1, L, g, kvh, D, dt, orc.MODE_GOLDEN, threads=4)
        assert_parity(got[b], gold[0], dt, "seed %d seq %d len %d" % (seed, b, L))


@pytest.mark.parametrize("dt", [FP16, BF16])
@pytest.mark.parametrize("kernel", [1, 2, 3], ids=["mma", "tcgen05", "tcgen05-persistent"])
def test_wide_dynamic_range_scores(ops, kernel, dt):
    """Keys whose norm grows along the sequence: the row maximum keeps rising by large steps, so the
    accumulator is rescaled many times (and, below the threshold, not rescaled) within one row."""
    m, n, H = 256, 512, 2
    rng = np.random.default_rng(4242)
    qf = rng.standard_normal((m, H * D), dtype=np.float32)
    kf = rng.standard_normal((n, H * D), dtype=np.float32) * np.linspace(0.2, 6.0, n, dtype=np.float32)[:, None]
    vf = rng.standard_normal((n, H * D), dtype=np.float32)
    q, k, v = orc.to_bits(qf, dt), orc.to_bits(kf, dt), orc.to_bits(vf, dt)
    out = torch.empty((m, H * D), dtype=dev(q[:1], dt).dtype, device="cuda")
    ops.gpu_attn_set_prefill_kernel(kernel)
    try:
        ops.gpu_flash_attn_layer(out, dev(q, dt), dev(k, dt), dev(v, dt), m, n, n - m, H, D, dt)
        torch.cuda.synchronize()
    finally:
        ops.gpu_attn_set_prefill_kernel(0)
    assert ops.gpu_ops_kernel_status() == 0
    gold = orc.attn(q, k, v, m, n, n - m, 1, H, D, dt, orc.MODE_GOLDEN, threads=8)
    assert_parity(host(out), gold, dt, "wide range")


@pytest.mark.parametrize("budget", [1, 200 << 10, 1 << 20, 3 << 20])
def test_prefill_cta_order_does_not_change_a_bit(ops, budget):
    """The tcgen05 prefill kernel starts its CTAs in chunks of (sequence, head) pairs sized by an L2 window:
    every window (one pair per chunk, chunks that do not divide the pairs, one chunk) gives the bits of
    the default, on a batch with several row blocks per pair."""
    batch, H, kvh, m, offset, dt = 3, 10, 5, 700, 300, BF16
    n = m + offset
    q = dev(rnd_bits((batch, m, H * D), dt, 900), dt)
    kc, vc = dev(rnd_bits((batch, kvh, n, D), dt, 901), dt), dev(rnd_bits((batch, kvh, n, D), dt, 902), dt)
    desc = ops.make_desc(dt, batch, H, kvh, m, n, layout="head")
    want, got = torch.empty_like(q), torch.full_like(q, float("nan"))
    ops.gpu_attn_set_prefill_kernel(2)
    try:
        ops.gpu_attn_prefill_layer(desc, want, q, kc, vc, m, offset)
        ops.gpu_attn_set_prefill_l2_window(budget)
        ops.gpu_attn_prefill_layer(desc, got, q, kc, vc, m, offset)
        torch.cuda.synchronize()
    finally:
        ops.gpu_attn_set_prefill_l2_window(0)
        ops.gpu_attn_set_prefill_kernel(0)
    assert ops.gpu_ops_kernel_status() == 0 and ops.gpu_attn_last_prefill_kernel() == 2
    assert np.array_equal(host(got), host(want))
